// Map / direct kernel instances that read K/V pages of FP8 E4M3FN elements, the reference's cache format
// (components/gqa/sdpa/sliced_kv.rs:118, sliced_q.rs:202: one byte per stored element; decode on load by
// metal/gqa_fp8.metal:1-25). The kernel is sdpa_map_kernel with KVB = 1: the stream warp copies raw pages, decode
// warps expand them into the 16-bit stage ring, and the consumers are the ones of the 16-bit instances.
#include <cuda.h>
#include <cuda_runtime.h>

#include "common.h"
#include "map_instance.h"
#include "sdpa_tm.cuh"

// Consumer warps of the token-major decode instance (eight: two per scheduler).
#ifndef KH_TM_CONSUMER_WARPS
#define KH_TM_CONSUMER_WARPS 8
#endif

namespace kh {

template <typename T, int D, int P, int MT, int KVW, bool HALF, int PS = 1>
static MapInstance make_fp8_instance() {
    using G = MapGeometry<D, P, MT, KVW, PS, HALF, 1>;
    return MapInstance{sdpa_map_kernel<T, D, P, MT, KVW, PS, HALF, 1>, G::kThreads, G::kSmemBytes, G::kStageTokens,
                       G::kBoxRows, G::kRawStages};
}

// Token-major instance (sdpa_tm.cuh): the raw bytes are consumed from the copied stage, no decode warps.
template <typename T, int D, int P, int NQ, int CW, int NR>
static MapInstance make_tm_instance() {
    using G = TmGeometry<D, P, NQ, CW, 1, NR>;
    return MapInstance{sdpa_tm_kernel<T, D, P, NQ, CW, 1, NR>, G::kThreads, G::kSmemBytes, G::kStageTokens, G::kBoxRows,
                       G::kStages};
}

// Same consumer shapes by task rows as the 16-bit table; tasks of more than 64 rows stay on the warp-level
// instance (the tensor-memory kernel reads 16-bit pages only).
// Decode shapes (one row tile) at head_dim 128: two KV warp groups of two warps that split a stage's tokens,
// instead of four groups of one. The 16-bit ring (two slots per group) then takes 64 KB instead of 128 KB, and
// the raw ring, whose depth is what covers the HBM latency, twice as many stages.
template <typename T, int D, int P>
static MapInstance pick_fp8_rows(uint32_t rows, bool one_launch) {
    // Tasks of up to 32 rows (24 at head_dim 256) take the token-major kernel; the one-launch map + reduce form
    // (arrival counters) exists in the decode-warp kernel only.
    if (!one_launch) {
        if (rows <= 8) return make_tm_instance<T, D, P, 1, KH_TM_CONSUMER_WARPS, 1>();
        // wider tiles: the warps of a group take one n-tile of 8 rows each (measured against warp pairs that split
        // the head dimension on the verify workload: 0.43 ms against 0.50 ms)
        if constexpr (D == 128) {
            if (rows <= 16) return make_tm_instance<T, D, P, 2, 8, 1>();
            if (rows <= 24) return make_tm_instance<T, D, P, 3, 9, 3>();
            if (rows <= 32) return make_tm_instance<T, D, P, 4, 8, 4>();
        } else {
            if (rows <= 16) return make_tm_instance<T, D, P, 2, 8, 2>();
            if (rows <= 24) return make_tm_instance<T, D, P, 3, 9, 3>();
        }
    }
    if constexpr (D == 128) {
        if (rows <= 8) return make_fp8_instance<T, D, P, 1, 2, true, 2>();
        if (rows <= 16) return make_fp8_instance<T, D, P, 1, 2, false, 2>();
    }
    if (rows <= 8) return make_fp8_instance<T, D, P, 1, 4, true>();
    if (rows <= 16) return make_fp8_instance<T, D, P, 1, 4, false>();
    // three half tiles + decode warps are ten warps, which caps a thread at 168 registers: too few for the
    // head_dim 256 accumulators (measured 3x slower than the 16-bit twin), so those tasks take two full tiles
    if (rows <= 24 && D == 128) return make_fp8_instance<T, D, P, 3, 2, true>();
    if (rows <= 32) return make_fp8_instance<T, D, P, 2, 2, false>();
    if (rows <= 64) return make_fp8_instance<T, D, P, 4, 1, false>();
    return make_fp8_instance<T, D, P, 8, 1, false>();
}

template <typename T>
static MapInstance pick_fp8_geometry(uint32_t head_dim, uint32_t tokens_per_page, uint32_t rows, bool one_launch) {
    KH_REQUIRE(tokens_per_page == 16, "FP8 pages: this build instantiates 16-token pages (got %u)", tokens_per_page);
    if (head_dim == 128) return pick_fp8_rows<T, 128, 16>(rows, one_launch);
    KH_REQUIRE(head_dim == 256, "this build instantiates head_dim 128 and 256 only (got %u)", head_dim);
    return pick_fp8_rows<T, 256, 16>(rows, one_launch);
}

MapInstance pick_instance_fp8(kh_dtype dtype, uint32_t head_dim, uint32_t tokens_per_page, uint32_t rows,
                              bool one_launch) {
    KH_REQUIRE(rows >= 1 && rows <= 128, "a Map task holds at most 128 (Q token, Q head) rows (got %u)", rows);
    if (dtype == KH_DTYPE_BFLOAT16) return pick_fp8_geometry<__nv_bfloat16>(head_dim, tokens_per_page, rows, one_launch);
    KH_REQUIRE(dtype == KH_DTYPE_FLOAT16, "Q/output dtype must be Bfloat16 or Float16 on this backend");
    return pick_fp8_geometry<__half>(head_dim, tokens_per_page, rows, one_launch);
}

}  // namespace kh
