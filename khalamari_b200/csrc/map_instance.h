// Table entry of one compiled map / direct kernel instance: what a launch needs to know about it.
#pragma once

#include <cuda.h>

#include "../../include/kh_gqa.h"
#include "sdpa_map.cuh"

namespace kh {

using MapKernel = void (*)(const CUtensorMap, const CUtensorMap, const MapParams);

struct MapInstance {
    MapKernel kernel;
    int threads;
    int smem_bytes;
    int stage_tokens;
    int box_rows;
    int stages;
};

// Warp-level instance for K/V pages of FP8 E4M3FN elements (sdpa_fp8.cu; compiled apart from the 16-bit instances
// so that the two translation units build side by side). `rows` = Q rows per task; `one_launch`: the instance
// must support the map + reduce in one launch form (arrival counters).
MapInstance pick_instance_fp8(kh_dtype dtype, uint32_t head_dim, uint32_t tokens_per_page, uint32_t rows,
                              bool one_launch);

}  // namespace kh
