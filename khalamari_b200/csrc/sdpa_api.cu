// C ABI of the CUDA side of libkhcuda_gqa: device / buffer / stream objects, the request page
// table, the SlicedKv and SlicedQ compute objects (map, reduce, direct) and the LSE combine.
// Reference counterparts are cited per entry point in include/kh_gqa.h.
#include <cuda.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <mutex>
#include <vector>

#include "common.h"
#include "cuda_objects.h"
#include "host_sdpa.h"
#include "map_instance.h"
#include "sdpa_map.cuh"
#include "sdpa_tc.cuh"
#include "sdpa_tm.cuh"

namespace kh {

// ---------------------------------------------------------------------------------------------
// Reduce kernel: the partial-state merge of the reference's reducers
// (gqa_sdpa_sliced_kv_reduce.metal:9-56, gqa_sdpa_sliced_q_reduce.metal:4-62,
// docs/gqa_sdpa_selection.md:443-460). One CTA per (Q head, Q-token range); each thread owns four
// consecutive output columns.
// ---------------------------------------------------------------------------------------------
struct ReduceParams {
    const float* partial_sum;
    const float* partial_max;
    const float* partial_out;
    const uint32_t* q_ranges;  // null: range i is token i
    const uint32_t* cu;        // null: every range merges partials [0, fixed_partials)
    void* out;
    float* out_sum;            // optional merged statistics, [tokens][Hq]
    float* out_max;
    uint32_t num_q_heads;
    uint32_t head_dim;
    uint32_t max_q_tokens;
    uint32_t num_active_ranges;
    uint32_t num_active_tokens;
    uint32_t fixed_partials;
    uint64_t stat_stride;      // floats between consecutive partials of a row; 0: dense [partial][Hq][maxq]
    uint64_t out_stride;       // same for the partial outputs; 0: dense [partial][Hq][maxq][D]
    uint32_t num_partials;     // partials the buffers hold: bounds what `cu` may name
    uint32_t heads_per_block;  // > 1 (one-token ranges only): a block serves this many consecutive heads
    const uint32_t* active;    // replay: device words {tokens, Q-token tiles, templates}; the counts above bound them
    uint32_t active_range_word; // which of the words counts this launch's ranges (0: tokens, 1: Q-token tiles)
};

template <typename T>
__device__ __forceinline__ void store4(T* dst, float4 v);
template <>
__device__ __forceinline__ void store4<float>(float* dst, float4 v) {
    *reinterpret_cast<float4*>(dst) = v;
}
template <>
__device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* dst, float4 v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y);
    __nv_bfloat162 hi = __floats2bfloat162_rn(v.z, v.w);
    uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    *reinterpret_cast<uint2*>(dst) = packed;
}
template <>
__device__ __forceinline__ void store4<__half>(__half* dst, float4 v) {
    __half2 lo = __floats2half2_rn(v.x, v.y);
    __half2 hi = __floats2half2_rn(v.z, v.w);
    uint2 packed = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    *reinterpret_cast<uint2*>(dst) = packed;
}

constexpr uint32_t kReduceMaxThreads = 512;

template <typename T>
__global__ void __launch_bounds__(kReduceMaxThreads) sdpa_reduce_kernel(const ReduceParams p) {
    __shared__ float4 shared_acc[kReduceMaxThreads];
    __shared__ float2 shared_stat[kReduceMaxThreads];
    // Launched with programmatic stream serialization: the blocks may be scheduled while the kernel before (the map)
    // is still running; everything that kernel wrote is visible after this wait, nothing is read before it.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const uint32_t range = blockIdx.x;  // ranges on x: no 65,535 limit
    uint32_t num_active_ranges = p.num_active_ranges, num_active_tokens = p.num_active_tokens;
    if (p.active != nullptr) {
        num_active_ranges = min(p.active[p.active_range_word], num_active_ranges);
        num_active_tokens = min(p.active[0], num_active_tokens);
    }
    if (range >= num_active_ranges) return;
    if (p.heads_per_block > 1) {
        // decode shape: one token per range, few partials per row. A thread owns four output columns of one
        // head; no shared memory, no second wave of blocks.
        const uint32_t D = p.head_dim;
        const uint32_t slots = D / 4;
        const uint32_t head = blockIdx.y * p.heads_per_block + threadIdx.x / slots;
        const uint32_t d = (threadIdx.x % slots) * 4;
        if (head >= p.num_q_heads || threadIdx.x / slots >= p.heads_per_block) return;
        const uint32_t tok = p.q_ranges != nullptr ? p.q_ranges[range * 2] : range;
        if (tok >= num_active_tokens) return;
        // `cu` comes from the caller's device memory: a stale entry must not reach past the partial buffers
        const uint32_t last = min(p.cu != nullptr ? p.cu[range + 1] : p.fixed_partials, p.num_partials);
        const uint32_t first = min(p.cu != nullptr ? p.cu[range] : 0u, last);
        const uint64_t stride = p.stat_stride != 0 ? p.stat_stride : uint64_t(p.num_q_heads);
        const uint64_t out_stride = p.out_stride != 0 ? p.out_stride : stride * D;
        const uint64_t first_index = uint64_t(first) * p.num_q_heads + head;
        float merged_sum, merged_max;
        const float4 acc = merge_partials_vec(p.partial_sum, p.partial_max, p.partial_out, first_index, stride, out_stride,
                                              last - first, D, d, &merged_sum, &merged_max);
        const uint64_t out_row = uint64_t(tok) * p.num_q_heads + head;
        store4<T>(reinterpret_cast<T*>(p.out) + out_row * D + d, acc);
        if (p.out_sum != nullptr && d == 0) {
            p.out_sum[out_row] = merged_sum;
            p.out_max[out_row] = merged_max;
        }
        return;
    }
    const uint32_t head = blockIdx.y;
    uint32_t tok_begin = range, tok_end = range + 1;
    if (p.q_ranges != nullptr) {
        tok_begin = p.q_ranges[range * 2];
        tok_end = p.q_ranges[range * 2 + 1];
    }
    if (tok_begin >= num_active_tokens || tok_end > num_active_tokens || tok_end <= tok_begin) return;
    const uint32_t num_toks = min(tok_end - tok_begin, p.max_q_tokens);
    const uint32_t last = min(p.cu != nullptr ? p.cu[range + 1] : p.fixed_partials, p.num_partials);
    const uint32_t first = min(p.cu != nullptr ? p.cu[range] : 0u, last);
    const uint32_t D = p.head_dim;
    const uint64_t stride = p.stat_stride != 0 ? p.stat_stride : uint64_t(p.num_q_heads) * p.max_q_tokens;
    const uint64_t out_stride = p.out_stride != 0 ? p.out_stride : stride * D;
    const uint32_t slots = num_toks * D / 4;  // float4 columns of this block's rows
    // When the block has at least twice as many threads as columns, the partials of a row are divided among
    // `subsets` thread groups (contiguous shares), merged through shared memory: the loads of a long partial
    // list run side by side instead of one batch after another.
    const uint32_t subsets = slots * 2 <= blockDim.x ? blockDim.x / slots : 1;
    if (subsets == 1) {
        for (uint32_t slot = threadIdx.x; slot < slots; slot += blockDim.x) {
            const uint32_t tok = slot * 4 / D;
            const uint32_t d = slot * 4 % D;
            const uint64_t first_index = (uint64_t(first) * p.num_q_heads + head) * p.max_q_tokens + tok;
            float merged_sum, merged_max;
            const float4 acc = merge_partials_vec(p.partial_sum, p.partial_max, p.partial_out, first_index, stride,
                                                  out_stride, last - first, D, d, &merged_sum, &merged_max);
            const uint64_t out_row = uint64_t(tok_begin + tok) * p.num_q_heads + head;
            store4<T>(reinterpret_cast<T*>(p.out) + out_row * D + d, acc);
            if (p.out_sum != nullptr && d == 0) {
                p.out_sum[out_row] = merged_sum;
                p.out_max[out_row] = merged_max;
            }
        }
        return;
    }
    const uint32_t slot = threadIdx.x % slots;
    const uint32_t subset = threadIdx.x / slots;
    const uint32_t tok = slot * 4 / D;
    const uint32_t d = slot * 4 % D;
    const uint32_t count = last - first;
    const uint32_t share = (count + subsets - 1) / subsets;
    MergeState state = merge_state_empty();
    if (subset < subsets) {
        const uint32_t begin = min(subset * share, count);
        const uint32_t mine = min(share, count - begin);
        const uint64_t first_index = (uint64_t(first) * p.num_q_heads + head) * p.max_q_tokens + tok;
        merge_partials_accumulate(state, p.partial_sum + uint64_t(begin) * stride, p.partial_max + uint64_t(begin) * stride,
                                  p.partial_out + uint64_t(begin) * out_stride, first_index, stride, out_stride, mine,
                                  D, d);
    }
    shared_acc[threadIdx.x] = state.acc;
    shared_stat[threadIdx.x] = make_float2(state.sum, state.max);
    __syncthreads();
    if (subset != 0) return;
    for (uint32_t other = 1; other < subsets; ++other) {
        const uint32_t source = other * slots + slot;
        const float2 stat = shared_stat[source];
        merge_state_combine(state, MergeState{shared_acc[source], stat.x, stat.y});
    }
    float merged_sum, merged_max;
    const float4 acc = merge_state_finish(state, &merged_sum, &merged_max);
    const uint64_t out_row = uint64_t(tok_begin + tok) * p.num_q_heads + head;
    store4<T>(reinterpret_cast<T*>(p.out) + out_row * D + d, acc);
    if (p.out_sum != nullptr && d == 0) {
        p.out_sum[out_row] = merged_sum;
        p.out_max[out_row] = merged_max;
    }
}

// ---------------------------------------------------------------------------------------------
// Kernel instance table
// ---------------------------------------------------------------------------------------------
template <typename T, int D, int P, int MT, int KVW, int PS, bool HALF>
static MapInstance make_instance() {
    using G = MapGeometry<D, P, MT, KVW, PS, HALF>;
    return MapInstance{sdpa_map_kernel<T, D, P, MT, KVW, PS, HALF>, G::kThreads, G::kSmemBytes, G::kStageTokens,
                       G::kBoxRows, G::kStages};
}

// Consumer-warp shapes. `rows` = Q rows per task (max_q_tokens x max_q_heads); tasks of at most 8 rows
// (decode with a group of up to 8 heads) use the half-tile instance, which skips the softmax work of
// fragment rows 8-15 and uses them to carry the rounding remainder of the probabilities.
// head_dim 128: a stage is 32 KV tokens (two pages); 8 consumer warps = KVW stage groups x 2 warps that
// take one page each, two warps per SM sub-partition so that one warp's softmax overlaps the other's
// MMAs. head_dim 256: a stage is 16 KV tokens (one page) and a thread carries a 16 x 256 f32 accumulator
// (128 registers), so 4 consumer warps run with up to 255 registers each.
// Tasks of more than 64 rows (prefill and long verify tiles) at head_dim 128 run on tcgen05 with tensor-memory
// accumulators (a library compiled with KH_GQA_MEASURE can be told to take the warp-level instance instead).
template <typename T, int D, int P>
static MapInstance make_tc_instance() {
    using G = TcGeometry<D, P>;
    return MapInstance{sdpa_tc_kernel<T, D, P>, G::kThreads, G::kSmemBytes, G::kStageTokens, G::kBoxRows, G::kStages};
}

// Token-major instance over 16-bit pages (sdpa_tm.cuh): the KV tokens on the M side of the tiles, groups of NR
// warps that take the n-tiles of Q rows between them.
template <typename T, int D, int P, int NQ, int CW, int NR>
static MapInstance make_tm_instance() {
    using G = TmGeometry<D, P, NQ, CW, 2, NR>;
    return MapInstance{sdpa_tm_kernel<T, D, P, NQ, CW, 2, NR>, G::kThreads, G::kSmemBytes, G::kStageTokens, G::kBoxRows,
                       G::kStages};
}

template <typename T, int D, int P>
static MapInstance pick_rows(uint32_t rows, bool tensor_memory) {
    constexpr int PS = 1;
    // Verify tiles of 17-32 rows (four tokens x six or eight heads): token-major. `tensor_memory` is false for the
    // one-launch map + reduce form, which this kernel does not have.
    if constexpr (P == 16) {
        // 17-24 rows: three groups of three warps, each warp of a group taking one n-tile of 8 rows over the whole
        // head dimension (nine consumer warps at 168 registers); 25-32 rows at head_dim 128: two groups of four
        if (tensor_memory && rows > 16 && rows <= 24) return make_tm_instance<T, D, P, 3, 9, 3>();
        if constexpr (D == 128) {
            if (tensor_memory && rows > 24 && rows <= 32) return make_tm_instance<T, D, P, 4, 8, 4>();
        }
    }
    if (rows <= 8) return make_instance<T, D, P, 1, 4, PS, true>();
    if (rows <= 16) return make_instance<T, D, P, 1, 4, PS, false>();
    // 17-24 rows (verify of four tokens with a group of six heads): three half tiles; the same tensor-core work as
    // two full tiles, spread over six warps instead of four
    if (rows <= 24) return make_instance<T, D, P, 3, 2, PS, true>();
    if (rows <= 32) return make_instance<T, D, P, 2, 2, PS, false>();
    if (rows <= 64) return make_instance<T, D, P, 4, 1, PS, false>();
    if constexpr (D == 128 && P == 16) {
#ifdef KH_GQA_MEASURE
        // measurement build only: compare against the warp-level instance
        if (std::getenv("KH_GQA_NO_TCGEN05") != nullptr) tensor_memory = false;
#endif
        if (tensor_memory) return make_tc_instance<T, D, P>();
    }
    return make_instance<T, D, P, 8, 1, 1, false>();
}

template <typename T, int D>
static MapInstance pick_page(uint32_t tokens_per_page, uint32_t rows, bool tensor_memory) {
    if (tokens_per_page == 16) return pick_rows<T, D, 16>(rows, tensor_memory);
    if constexpr (D == 256) {
        // the reference's head_dim 256 profiles include 32-token pages (components/gqa/sdpa.rs:162-215)
        if (tokens_per_page == 32) return pick_rows<T, D, 32>(rows, tensor_memory);
    }
    KH_REQUIRE(tokens_per_page == 8, "this build instantiates 8- and 16-token pages, and 32-token pages at head_dim 256 (got %u)",
               tokens_per_page);
    return pick_rows<T, D, 8>(rows, tensor_memory);
}

template <typename T>
static MapInstance pick_geometry(uint32_t head_dim, uint32_t tokens_per_page, uint32_t rows, bool tensor_memory) {
    if (head_dim == 128) return pick_page<T, 128>(tokens_per_page, rows, tensor_memory);
    KH_REQUIRE(head_dim == 256, "this build instantiates head_dim 128 and 256 only (got %u)", head_dim);
    return pick_page<T, 256>(tokens_per_page, rows, tensor_memory);
}

static MapInstance pick_instance(kh_dtype dtype, uint32_t head_dim, uint32_t tokens_per_page, uint32_t rows,
                                 bool tensor_memory) {
    KH_REQUIRE(rows >= 1 && rows <= 128, "a Map task holds at most 128 (Q token, Q head) rows (got %u)", rows);
    if (dtype == KH_DTYPE_BFLOAT16) return pick_geometry<__nv_bfloat16>(head_dim, tokens_per_page, rows, tensor_memory);
    KH_REQUIRE(dtype == KH_DTYPE_FLOAT16, "Q/output dtype must be Bfloat16 or Float16 on this backend");
    return pick_geometry<__half>(head_dim, tokens_per_page, rows, tensor_memory);
}

// ---------------------------------------------------------------------------------------------
// Tensor map over the KV pool: rows = (page, plane, kv head, token in page), columns = head_dim.
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult query;
        KH_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &query));
        if (entry == nullptr || query != cudaDriverEntryPointSuccess) {
            raise(KH_UNAVAILABLE, "the CUDA driver does not export cuTensorMapEncodeTiled");
        }
        fn = reinterpret_cast<EncodeTiledFn>(entry);
    }
    return fn;
}

struct PoolMap {
    void* ptr;
    uint64_t bytes;
    CUtensorMap map;
};

struct ComputeCommon {
    kh_device* device;
    kh_dtype dtype;
    kh_dtype kv_dtype;
    uint32_t num_q_heads, num_kv_heads, head_dim, tokens_per_page, page_bytes;
    float scale;
    kh_page_table_layout layout;
    kh_execution_variant variant;
    MapInstance instance;
    MapInstance fused_instance;
    std::vector<PoolMap> pool_maps;
    std::vector<PoolMap> q_maps;

    // Encoded tensor maps are kept per (address, byte length), least recently used first: a hit moves the entry to
    // the back, a miss with the cache full drops the front. 64 entries cover a caller that rotates its Q and pool
    // buffers (one Q buffer per in-flight step and per replay bucket); beyond that a call re-encodes on the host.
    static constexpr size_t kTensorMapCacheEntries = 64;
    static const CUtensorMap* find_map(std::vector<PoolMap>& maps, kh_buffer_ref buffer) {
        for (size_t i = maps.size(); i-- > 0;) {
            if (maps[i].ptr == buffer.ptr && maps[i].bytes == buffer.bytes) {
                if (i + 1 != maps.size()) std::rotate(maps.begin() + i, maps.begin() + i + 1, maps.end());
                return &maps.back().map;
            }
        }
        return nullptr;
    }

    // Tensor map over Q [tokens * Hq rows][head_dim], one box = the Q heads of one task for one token.
    const CUtensorMap& q_map(kh_buffer_ref q) {
        if (const CUtensorMap* hit = find_map(q_maps, q)) return *hit;
        KH_REQUIRE((reinterpret_cast<uintptr_t>(q.ptr) & 127) == 0, "q must be 128-byte aligned");
        const uint64_t rows = q.bytes / (uint64_t(head_dim) * 2);
        KH_REQUIRE(rows > 0 && rows <= 0x7fffffffull, "q holds an unsupported number of rows");
        PoolMap entry{};
        entry.ptr = q.ptr;
        entry.bytes = q.bytes;
        const cuuint64_t dims[2] = {head_dim, rows};
        const cuuint64_t strides[1] = {uint64_t(head_dim) * 2};
        const cuuint32_t box[2] = {64, variant.max_q_heads};
        const cuuint32_t elem_strides[2] = {1, 1};
        const CUtensorMapDataType type =
            dtype == KH_DTYPE_BFLOAT16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        const CUresult rc = encode_tiled_fn()(&entry.map, type, 2, q.ptr, dims, strides, box, elem_strides,
                                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rc != CUDA_SUCCESS) raise(KH_INTERNAL, "cuTensorMapEncodeTiled (q) failed with code %d", int(rc));
        if (q_maps.size() >= kTensorMapCacheEntries) q_maps.erase(q_maps.begin());
        q_maps.push_back(entry);
        return q_maps.back().map;
    }

    const CUtensorMap& pool_map(kh_buffer_ref pages) {
        if (const CUtensorMap* hit = find_map(pool_maps, pages)) return *hit;
        KH_REQUIRE((reinterpret_cast<uintptr_t>(pages.ptr) & 127) == 0, "kv_pages must be 128-byte aligned");
        const uint64_t pool_pages = pages.bytes / page_bytes;
        KH_REQUIRE(pool_pages > 0, "kv_pages holds no complete page");
        const uint64_t rows = pool_pages * 2 * num_kv_heads * tokens_per_page;
        KH_REQUIRE(rows <= 0x7fffffffull, "KV pool has too many rows for one tensor map");
        PoolMap entry{};
        entry.ptr = pages.ptr;
        entry.bytes = pages.bytes;
        // Four dimensions: {64 columns, pool rows, 64-column halves of a row, K/V plane}. A copy at
        // (0, first K row of a page chunk, 0, 0) with box {64, rows, halves, 2} brings the K chunk and, one
        // plane stride (Hkv * P rows) further, the V chunk of the same (page, KV head). Rows are addressed
        // through their K-plane index only, so the row extent stops one plane short of the pool's end and a
        // page id beyond the pool falls outside it (the copy then writes zeros).
        const uint64_t plane_rows = uint64_t(num_kv_heads) * tokens_per_page;
        // FP8 pages: the same four dimensions in bytes, a 128-byte line holding 128 elements.
        const bool fp8 = kv_dtype == KH_DTYPE_FP8_E4M3FN;
        const uint32_t line = fp8 ? 128 : 64;  // elements of a 128-byte line
        const uint64_t elem = fp8 ? 1 : 2;
        const cuuint64_t dims[4] = {line, rows - plane_rows, head_dim / line, 2};
        const cuuint64_t strides[3] = {uint64_t(head_dim) * elem, 128, plane_rows * head_dim * elem};
        const cuuint32_t box[4] = {line, static_cast<cuuint32_t>(instance.box_rows), head_dim / line, 2};
        const cuuint32_t elem_strides[4] = {1, 1, 1, 1};
        const CUtensorMapDataType type = fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                             : dtype == KH_DTYPE_BFLOAT16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                                          : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
        const CUresult rc = encode_tiled_fn()(&entry.map, type, 4, pages.ptr, dims, strides, box, elem_strides,
                                              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                              CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rc != CUDA_SUCCESS) raise(KH_INTERNAL, "cuTensorMapEncodeTiled failed with code %d", int(rc));
        if (pool_maps.size() >= kTensorMapCacheEntries) pool_maps.erase(pool_maps.begin());
        pool_maps.push_back(entry);
        return pool_maps.back().map;
    }
};

static void init_common(ComputeCommon& c, kh_device* device, kh_dtype dtype, kh_dtype kv_dtype, uint32_t num_q_heads,
                        uint32_t num_kv_heads, uint32_t head_dim, float scale, uint32_t page_bytes,
                        const kh_page_table_layout& layout, const kh_execution_variant& variant) {
    use_device(device);
    const bool fp8 = kv_dtype == KH_DTYPE_FP8_E4M3FN;
    KH_REQUIRE(kv_dtype == dtype || fp8, "K/V pages hold the Q/output element type or FP8 E4M3FN");
    c.device = device;
    c.dtype = dtype;
    c.kv_dtype = kv_dtype;
    c.num_q_heads = num_q_heads;
    c.num_kv_heads = num_kv_heads;
    c.head_dim = head_dim;
    c.scale = scale;
    c.page_bytes = page_bytes;
    c.layout = layout;
    c.variant = variant;
    c.tokens_per_page = page_bytes / (2 * num_kv_heads * head_dim * dtype_size(kv_dtype));
    const uint32_t rows = variant.max_q_tokens * variant.max_q_heads;
    c.instance = fp8 ? pick_instance_fp8(dtype, head_dim, c.tokens_per_page, rows, false)
                     : pick_instance(dtype, head_dim, c.tokens_per_page, rows, true);
    // the one-launch map + reduce form counts arrivals inside the warp-level kernel
    c.fused_instance = fp8 ? pick_instance_fp8(dtype, head_dim, c.tokens_per_page, rows, true)
                           : pick_instance(dtype, head_dim, c.tokens_per_page, rows, false);
    KH_CUDA(cudaFuncSetAttribute(reinterpret_cast<const void*>(c.instance.kernel),
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, c.instance.smem_bytes));
    KH_CUDA(cudaFuncSetAttribute(reinterpret_cast<const void*>(c.fused_instance.kernel),
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, c.fused_instance.smem_bytes));
}

static void launch_map(ComputeCommon& c, kh_stream* stream, MapParams& p, kh_buffer_ref q, kh_buffer_ref kv_pages,
                       uint32_t num_templates) {
    KH_REQUIRE(stream != nullptr && stream->device == c.device, "stream does not belong to the compute's device");
    use_device(c.device);
    const CUtensorMap& map = c.pool_map(kv_pages);
    const CUtensorMap& qmap = c.q_map(q);
    p.status = c.device->status;
    p.num_templates = num_templates;
    p.active = static_cast<const uint32_t*>(stream->active_counts.ptr);
    p.num_q_heads = c.num_q_heads;
    p.num_kv_heads = c.num_kv_heads;
    p.group = c.num_q_heads / c.num_kv_heads;
    p.heads_per_task = c.variant.max_q_heads;
    p.head_ranges = div_ceil(p.group, p.heads_per_task);
    p.max_q_tokens = c.variant.max_q_tokens;
    p.num_gqa_layers = c.layout.num_gqa_layers;
    p.pages_per_request_layer = c.layout.num_blocks * c.layout.num_page_ids_per_block;
    p.pool_pages = static_cast<uint32_t>(std::min<uint64_t>(kv_pages.bytes / c.page_bytes, 0xffffffffull));
    p.scale_log2e = c.scale * 1.4426950408889634f;
    p.num_req_slots = c.layout.num_req_slots;
    p.tokens_per_page = c.tokens_per_page;
    p.wait_limit = c.device->wait_limit;
#ifdef KH_GQA_MEASURE
    // Measurement build only: KH_GQA_DEBUG=<bits> switches parts of the kernel off (see MapParams::debug) so that
    // the paged TMA gather, the tensor-core math and the hand-offs can be timed separately. Read at every launch,
    // so that one process can time several settings. The product library never reads the variable.
    {
        const char* value = std::getenv("KH_GQA_DEBUG");
        p.debug = value != nullptr ? uint32_t(std::atoi(value)) : 0u;
    }
#endif
    if (num_templates == 0) return;
    const uint64_t tasks = uint64_t(num_templates) * c.num_kv_heads * p.head_ranges;
    KH_REQUIRE(tasks <= 0xffffffffull, "GQA SDPA map task count must fit u32");
    const uint32_t grid = static_cast<uint32_t>(std::min<uint64_t>(tasks, uint64_t(c.device->sm_count)));
    const MapInstance& instance = p.cu != nullptr ? c.fused_instance : c.instance;
    instance.kernel<<<grid, instance.threads, instance.smem_bytes, stream->stream>>>(map, qmap, p);
    KH_CUDA(cudaGetLastError());
}

template <typename T>
static void launch_reduce_typed(const ReduceParams& p, uint32_t num_ranges, cudaStream_t stream) {
    ReduceParams params = p;
    dim3 grid(num_ranges, p.num_q_heads, 1);
    // a fixed, long partial list per row (the cross-slice and cross-GPU merges) gets the widest block
    uint32_t threads = (p.cu == nullptr && p.fixed_partials > 32) ? kReduceMaxThreads : 128;
    params.heads_per_block = 1;
    const uint32_t slots = p.head_dim / 4;
    if (p.max_q_tokens == 1 && threads == 128 && slots <= 64 && 128 % slots == 0) {
        params.heads_per_block = 128 / slots;
        grid.y = (p.num_q_heads + params.heads_per_block - 1) / params.heads_per_block;
    }
    // programmatic dependent launch: the launch itself overlaps the tail of the map kernel that precedes it in the
    // stream (the kernel waits for that kernel's completion before it reads anything)
    cudaLaunchConfig_t config{};
    config.gridDim = grid;
    config.blockDim = dim3(threads, 1, 1);
    config.dynamicSmemBytes = 0;
    config.stream = stream;
    cudaLaunchAttribute attribute{};
    attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
    // (not for the merges of a fixed partial list - the cross-slice and cross-GPU combines: measured slower there)
    attribute.val.programmaticStreamSerializationAllowed = p.cu != nullptr ? 1 : 0;
    config.attrs = &attribute;
    config.numAttrs = 1;
    KH_CUDA(cudaLaunchKernelEx(&config, sdpa_reduce_kernel<T>, params));
}

static void launch_reduce(kh_dtype dtype, const ReduceParams& p, uint32_t num_ranges, cudaStream_t stream) {
    KH_REQUIRE(p.head_dim % 4 == 0, "head_dim must be a multiple of 4");
    KH_REQUIRE(p.num_q_heads <= 65535, "reduce supports at most 65535 Q heads");
    if (num_ranges == 0) return;
    if (dtype == KH_DTYPE_BFLOAT16) launch_reduce_typed<__nv_bfloat16>(p, num_ranges, stream);
    else if (dtype == KH_DTYPE_FLOAT16) launch_reduce_typed<__half>(p, num_ranges, stream);
    else if (dtype == KH_DTYPE_FLOAT32) launch_reduce_typed<float>(p, num_ranges, stream);
    else raise(KH_INVALID_ARGUMENT, "unsupported output dtype");
    KH_CUDA(cudaGetLastError());
}

static void validate_layout(const kh_page_table_layout& l) {
    KH_REQUIRE(l.num_req_slots > 0 && l.num_blocks > 0 && l.num_gqa_layers > 0 && l.num_page_ids_per_block > 0,
               "GQA page-table layout dimensions must be positive");
}

static uint64_t layout_entries(const kh_page_table_layout& l) {
    return mul_u64(mul_u64(mul_u64(l.num_req_slots, l.num_gqa_layers, "GQA page-table element count"), l.num_blocks,
                           "GQA page-table element count"),
                   l.num_page_ids_per_block, "GQA page-table element count");
}

static uint32_t tokens_per_page_of(uint32_t page_bytes, uint32_t num_kv_heads, uint32_t head_dim, kh_dtype kv_dtype) {
    const uint32_t elem = dtype_size(kv_dtype);
    KH_REQUIRE(elem > 0, "unknown K/V element type");
    const uint64_t per_token = uint64_t(num_kv_heads) * head_dim * 2 * elem;
    KH_REQUIRE(per_token <= 0xffffffffull, "GQA K/V bytes per token must fit u32");
    KH_REQUIRE(page_bytes % per_token == 0, "GQA page_bytes must be divisible by the K/V bytes per token");
    const uint32_t tokens = static_cast<uint32_t>(page_bytes / per_token);
    KH_REQUIRE(tokens > 0, "GQA pages must hold at least one token");
    return tokens;
}

}  // namespace kh

using namespace kh;

struct kh_sliced_kv {
    ComputeCommon common;
    kh_sliced_kv_config config;
    kh_sliced_kv_shape shape;
    kh_sliced_kv_sizes sizes;
};

struct kh_sliced_q {
    ComputeCommon common;
    kh_sliced_q_config config;
    kh_sliced_q_shape shape;
    kh_sliced_q_sizes sizes;
    bool direct;
};

static kh_sdpa_config sdpa_config_of(const kh_sliced_kv_config& c) {
    return kh_sdpa_config{c.dtype, c.num_q_heads, c.num_kv_heads, c.head_dim,
                          tokens_per_page_of(c.page_bytes, c.num_kv_heads, c.head_dim, c.kv_dtype)};
}

static kh_sdpa_config sdpa_config_of(const kh_sliced_q_config& c) {
    return kh_sdpa_config{c.dtype, c.num_q_heads, c.num_kv_heads, c.head_dim,
                          tokens_per_page_of(c.page_bytes, c.num_kv_heads, c.head_dim, c.kv_dtype)};
}

// sliced_kv::Config::validate + Shape::validate + byte sizes (sliced_kv.rs:100-231).
static kh_sliced_kv_sizes sliced_kv_sizes(const kh_sliced_kv_config& c, const kh_sliced_kv_shape& s) {
    KH_REQUIRE(c.num_q_heads > 0 && c.num_kv_heads > 0 && c.head_dim > 0, "GQA SDPA dimensions must be positive");
    KH_REQUIRE(c.scale > 0.0f, "GQA SDPA scale must be positive");
    KH_REQUIRE(c.num_q_heads % c.num_kv_heads == 0, "GQA Q heads must be a multiple of KV heads");
    validate_layout(c.page_table_layout);
    KH_REQUIRE(c.dtype == KH_DTYPE_FLOAT32 || c.dtype == KH_DTYPE_BFLOAT16 || c.dtype == KH_DTYPE_FLOAT16,
               "GQA SDPA dtype must be Float32, Bfloat16 or Float16");
    kh_sliced_kv_sizes out{};
    out.num_tokens_per_page = tokens_per_page_of(c.page_bytes, c.num_kv_heads, c.head_dim, c.kv_dtype);
    KH_REQUIRE(s.num_total_tokens > 0, "GQA SDPA shape requires tokens");
    KH_REQUIRE(s.num_total_sdpa_map_task_templates > 0, "GQA SDPA shape requires Map task templates");
    const uint64_t values = mul_u64(mul_u64(s.num_total_tokens, c.num_q_heads, "GQA SDPA output element count"),
                                    c.head_dim, "GQA SDPA output element count");
    KH_REQUIRE(values <= 0xffffffffull, "GQA SDPA query/output exceeds the shader u32 count domain: count=%llu",
               (unsigned long long)values);
    const uint64_t stats = mul_u64(s.num_total_sdpa_map_task_templates, c.num_q_heads,
                                   "GQA SDPA partial-output statistic count");
    KH_REQUIRE(stats - 1 <= 0xffffffffull, "GQA SDPA partial-output stats exceeds the shader u32 element-index domain");
    const uint64_t partial_values = mul_u64(stats, c.head_dim, "GQA SDPA partial output element count");
    out.q_bytes = values * dtype_size(c.dtype);
    out.req_slots_bytes = uint64_t(s.num_total_tokens) * 4;
    out.page_ids_bytes = layout_entries(c.page_table_layout) * 4;
    out.sdpa_map_task_templates_bytes = uint64_t(s.num_total_sdpa_map_task_templates) * 12;
    out.cu_sdpa_partial_outputs_bytes = (uint64_t(s.num_total_tokens) + 1) * 4;
    out.partial_output_stats_bytes = stats * 4;
    out.partial_output_bytes = partial_values * 4;  // f32 partials
    return out;
}

// sliced_q::Config::validate + Shape::validate + byte sizes (sliced_q.rs:155-306).
static kh_sliced_q_sizes sliced_q_sizes(const kh_sliced_q_config& c, const kh_execution_variant& v,
                                        const kh_sliced_q_shape& s) {
    KH_REQUIRE(c.num_q_heads > 0 && c.num_kv_heads > 0, "GQA SDPA dimensions must be positive");
    KH_REQUIRE(c.num_q_heads % c.num_kv_heads == 0, "GQA Q heads must be a multiple of KV heads");
    kh_sliced_q_sizes out{};
    out.num_tokens_per_page = tokens_per_page_of(c.page_bytes, c.num_kv_heads, c.head_dim, c.kv_dtype);
    const uint32_t P = out.num_tokens_per_page;
    KH_REQUIRE((c.head_dim == 128 && (P == 8 || P == 16)) || (c.head_dim == 256 && (P == 8 || P == 16 || P == 32)),
               "GQA SplitKV SlicedQ supports only (head_dim, tokens_per_page) profiles (128, 8), (128, 16), (256, 8), "
               "(256, 16), and (256, 32), got (%u, %u)",
               c.head_dim, P);
    KH_REQUIRE(c.scale > 0.0f, "GQA SDPA scale must be positive");
    KH_REQUIRE(c.dtype == KH_DTYPE_BFLOAT16 || c.dtype == KH_DTYPE_FLOAT16,
               "GQA SplitKV SlicedQ specializes bf16 (and fp16 on this backend)");
    validate_layout(c.page_table_layout);
    KH_REQUIRE(s.num_total_tokens > 0, "GQA SDPA shape requires tokens");
    KH_REQUIRE(s.num_total_q_token_tiles > 0 && s.num_total_q_token_tiles <= s.num_total_tokens,
               "GQA SplitKV SlicedQ Q-token tiles out of range");
    KH_REQUIRE(s.num_total_sdpa_map_task_templates >= s.num_total_q_token_tiles,
               "GQA SplitKV SlicedQ needs a Map task template per Q-token tile");
    KH_REQUIRE(uint64_t(s.num_total_q_token_tiles) * 2 - 1 <= 0xffffffffull,
               "GQA SplitKV SlicedQ Q-token-range metadata exceeds the shader u32 element-index domain");
    KH_REQUIRE(uint64_t(s.num_total_tokens) * 2 - 1 <= 0xffffffffull,
               "GQA SplitKV SlicedQ visible K/V-token-range metadata exceeds the shader u32 element-index domain");
    KH_REQUIRE(uint64_t(s.num_total_sdpa_map_task_templates) * 3 - 1 <= 0xffffffffull,
               "GQA SplitKV SlicedQ map TaskTemplate metadata exceeds the shader u32 element-index domain");
    out.q_bytes = mul_u64(mul_u64(mul_u64(s.num_total_tokens, c.num_q_heads, "GQA SplitKV SlicedQ query byte length"),
                                  c.head_dim, "GQA SplitKV SlicedQ query byte length"),
                          dtype_size(c.dtype), "GQA SplitKV SlicedQ query byte length");
    const uint64_t stats = mul_u64(mul_u64(s.num_total_sdpa_map_task_templates, c.num_q_heads,
                                           "GQA SplitKV SlicedQ partial statistic byte length"),
                                   v.max_q_tokens, "GQA SplitKV SlicedQ partial statistic byte length");
    out.partial_output_stats_bytes = mul_u64(stats, 4, "GQA SplitKV SlicedQ partial statistic byte length");
    out.partial_output_bytes =
        mul_u64(mul_u64(stats, c.head_dim, "GQA SplitKV SlicedQ partial output byte length"), 4,
                "GQA SplitKV SlicedQ partial output byte length");
    return out;
}

extern "C" {

const char* kh_version(void) { return "khcuda_gqa 0.1 (sm_100a)"; }

kh_status kh_device_open(int32_t ordinal, kh_device** out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(out != nullptr, "null argument");
        int count = 0;
        cudaError_t err = cudaGetDeviceCount(&count);
        if (err != cudaSuccess || count == 0) {
            return fail(KH_UNAVAILABLE, "no CUDA device is available: %s", cudaGetErrorString(err));
        }
        KH_REQUIRE(ordinal >= 0 && ordinal < count, "device ordinal %d out of range [0, %d)", ordinal, count);
        KH_CUDA(cudaSetDevice(ordinal));
        cudaDeviceProp prop;
        KH_CUDA(cudaGetDeviceProperties(&prop, ordinal));
        if (prop.major != 10) {
            return fail(KH_UNAVAILABLE, "device %d is sm_%d%d; this library is built for sm_100a only", ordinal,
                        prop.major, prop.minor);
        }
        auto device = std::make_unique<kh_device>();
        device->ordinal = ordinal;
        device->sm_count = prop.multiProcessorCount;
        device->wait_limit = kDefaultWaitLimit;
        KH_CUDA(cudaMalloc(&device->status, sizeof(uint32_t)));
        KH_CUDA(cudaMemset(device->status, 0, sizeof(uint32_t)));
        *out = device.release();
        return KH_OK;
    });
}

kh_status kh_device_close(kh_device* device) {
    return guarded([&]() -> kh_status {
        if (device == nullptr) return KH_OK;
        cudaSetDevice(device->ordinal);
        cudaFree(device->status);
        delete device;
        return KH_OK;
    });
}

kh_status kh_device_sm_count(const kh_device* device, int32_t* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(device && out, "null argument");
        *out = device->sm_count;
        return KH_OK;
    });
}

kh_status kh_buffer_alloc(kh_device* device, uint64_t bytes, kh_buffer_ref* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(out != nullptr, "null argument");
        use_device(device);
        KH_REQUIRE(bytes > 0, "buffer must hold at least one byte");
        void* ptr = nullptr;
        KH_CUDA(cudaMalloc(&ptr, bytes));
        KH_CUDA(cudaMemset(ptr, 0, bytes));
        out->ptr = ptr;
        out->bytes = bytes;
        return KH_OK;
    });
}

kh_status kh_buffer_free(kh_device* device, kh_buffer_ref buffer) {
    return guarded([&]() -> kh_status {
        use_device(device);
        if (buffer.ptr != nullptr) KH_CUDA(cudaFree(buffer.ptr));
        return KH_OK;
    });
}

kh_status kh_buffer_write(kh_device* device, kh_buffer_ref buffer, uint64_t offset, const void* src, uint64_t bytes) {
    return guarded([&]() -> kh_status {
        use_device(device);
        KH_REQUIRE(src != nullptr || bytes == 0, "source is null");
        KH_REQUIRE(offset <= buffer.bytes && bytes <= buffer.bytes - offset, "write exceeds the buffer");
        if (bytes) KH_CUDA(cudaMemcpy(static_cast<uint8_t*>(buffer.ptr) + offset, src, bytes, cudaMemcpyHostToDevice));
        return KH_OK;
    });
}

kh_status kh_buffer_read(kh_device* device, kh_buffer_ref buffer, uint64_t offset, void* dst, uint64_t bytes) {
    return guarded([&]() -> kh_status {
        use_device(device);
        KH_REQUIRE(dst != nullptr || bytes == 0, "destination is null");
        KH_REQUIRE(offset <= buffer.bytes && bytes <= buffer.bytes - offset, "read exceeds the buffer");
        if (bytes) KH_CUDA(cudaMemcpy(dst, static_cast<const uint8_t*>(buffer.ptr) + offset, bytes, cudaMemcpyDeviceToHost));
        return KH_OK;
    });
}

kh_status kh_buffer_zero(kh_device* device, kh_buffer_ref buffer, uint64_t offset, uint64_t bytes) {
    return guarded([&]() -> kh_status {
        use_device(device);
        KH_REQUIRE(offset <= buffer.bytes && bytes <= buffer.bytes - offset, "zero range exceeds the buffer");
        if (bytes) KH_CUDA(cudaMemset(static_cast<uint8_t*>(buffer.ptr) + offset, 0, bytes));
        return KH_OK;
    });
}

kh_status kh_stream_create(kh_device* device, kh_stream** out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(out != nullptr, "null argument");
        use_device(device);
        auto stream = std::make_unique<kh_stream>();
        stream->device = device;
        stream->owned = true;
        KH_CUDA(cudaStreamCreateWithFlags(&stream->stream, cudaStreamNonBlocking));
        *out = stream.release();
        return KH_OK;
    });
}

kh_status kh_stream_wrap(kh_device* device, void* cuda_stream, kh_stream** out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(device && out, "null argument");
        auto stream = std::make_unique<kh_stream>();
        stream->device = device;
        stream->owned = false;
        stream->stream = static_cast<cudaStream_t>(cuda_stream);
        *out = stream.release();
        return KH_OK;
    });
}

kh_status kh_stream_bind_active_counts(kh_stream* stream, kh_buffer_ref active_counts) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(stream != nullptr, "null argument");
        if (active_counts.ptr != nullptr) {
            KH_REQUIRE(active_counts.bytes >= 16, "active_counts holds %llu bytes but 16 are required",
                       (unsigned long long)active_counts.bytes);
            KH_REQUIRE((reinterpret_cast<uintptr_t>(active_counts.ptr) & 3) == 0, "active_counts must be 4-byte aligned");
        }
        stream->active_counts = active_counts;
        return KH_OK;
    });
}

kh_status kh_stream_destroy(kh_stream* stream) {
    return guarded([&]() -> kh_status {
        if (stream == nullptr) return KH_OK;
        if (stream->owned) {
            cudaSetDevice(stream->device->ordinal);
            cudaStreamDestroy(stream->stream);
        }
        delete stream;
        return KH_OK;
    });
}

kh_status kh_stream_synchronize(kh_stream* stream) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(stream != nullptr, "null argument");
        use_device(stream->device);
        KH_CUDA(cudaStreamSynchronize(stream->stream));
        return KH_OK;
    });
}

kh_status kh_stream_write(kh_stream* stream, kh_buffer_ref buffer, uint64_t offset, const void* src, uint64_t bytes) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(stream != nullptr, "null argument");
        use_device(stream->device);
        KH_REQUIRE(offset <= buffer.bytes && bytes <= buffer.bytes - offset, "write exceeds the buffer");
        if (bytes) {
            KH_CUDA(cudaMemcpyAsync(static_cast<uint8_t*>(buffer.ptr) + offset, src, bytes, cudaMemcpyHostToDevice,
                                    stream->stream));
        }
        return KH_OK;
    });
}

kh_status kh_stream_read(kh_stream* stream, kh_buffer_ref buffer, uint64_t offset, void* dst, uint64_t bytes) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(stream != nullptr, "null argument");
        use_device(stream->device);
        KH_REQUIRE(offset <= buffer.bytes && bytes <= buffer.bytes - offset, "read exceeds the buffer");
        if (bytes) {
            KH_CUDA(cudaMemcpyAsync(dst, static_cast<const uint8_t*>(buffer.ptr) + offset, bytes,
                                    cudaMemcpyDeviceToHost, stream->stream));
        }
        return KH_OK;
    });
}

kh_status kh_event_create(kh_device* device, kh_event** out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(out != nullptr, "null argument");
        use_device(device);
        auto event = std::make_unique<kh_event>();
        event->device = device;
        KH_CUDA(cudaEventCreateWithFlags(&event->event, cudaEventDisableTiming));
        *out = event.release();
        return KH_OK;
    });
}

kh_status kh_event_destroy(kh_event* event) {
    return guarded([&]() -> kh_status {
        if (event == nullptr) return KH_OK;
        cudaSetDevice(event->device->ordinal);
        cudaEventDestroy(event->event);
        delete event;
        return KH_OK;
    });
}

kh_status kh_stream_record_event(kh_stream* stream, kh_event* event) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(stream && event, "null argument");
        KH_REQUIRE(stream->device == event->device, "event does not belong to the stream's device");
        use_device(stream->device);
        KH_CUDA(cudaEventRecord(event->event, stream->stream));
        return KH_OK;
    });
}

kh_status kh_stream_wait_event(kh_stream* stream, kh_event* event) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(stream && event, "null argument");
        KH_REQUIRE(stream->device == event->device, "event does not belong to the stream's device");
        use_device(stream->device);
        KH_CUDA(cudaStreamWaitEvent(stream->stream, event->event, 0));
        return KH_OK;
    });
}

kh_status kh_event_synchronize(kh_event* event) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(event != nullptr, "null argument");
        use_device(event->device);
        KH_CUDA(cudaEventSynchronize(event->event));
        return KH_OK;
    });
}

kh_status kh_device_set_wait_limit(kh_device* device, uint32_t polls) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(device != nullptr, "null argument");
        device->wait_limit = polls != 0 ? polls : kDefaultWaitLimit;
        return KH_OK;
    });
}

kh_status kh_host_alloc_pinned(uint64_t bytes, void** out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(out != nullptr && bytes > 0, "invalid pinned allocation request");
        KH_CUDA(cudaHostAlloc(out, bytes, cudaHostAllocDefault));
        return KH_OK;
    });
}

kh_status kh_host_free_pinned(void* ptr) {
    return guarded([&]() -> kh_status {
        if (ptr != nullptr) KH_CUDA(cudaFreeHost(ptr));
        return KH_OK;
    });
}

kh_status kh_device_check(kh_device* device, kh_stream* stream, uint32_t* out_status_word) {
    return guarded([&]() -> kh_status {
        use_device(device);
        if (stream != nullptr) KH_CUDA(cudaStreamSynchronize(stream->stream));
        else KH_CUDA(cudaDeviceSynchronize());
        uint32_t word = 0;
        KH_CUDA(cudaMemcpy(&word, device->status, sizeof(word), cudaMemcpyDeviceToHost));
        if (word != 0) KH_CUDA(cudaMemset(device->status, 0, sizeof(word)));
        if (out_status_word) *out_status_word = word;
        if (word != 0) {
            return fail(KH_ABORTED, "device status word 0x%x:%s%s%s", word,
                        (word & kStatusWaitExpired) ? " a bounded wait inside a kernel ran out;" : "",
                        (word & kStatusPageOutOfPool) ? " a page id addressed beyond the KV pool;" : "",
                        (word & kStatusMetadataOutOfRange)
                            ? " batch metadata named a request slot or KV range beyond the page table;" : "");
        }
        return KH_OK;
    });
}

// ---- page table -----------------------------------------------------------------------------
kh_status kh_page_table_bytes(const kh_page_table_layout* layout, uint64_t* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(layout && out, "null argument");
        validate_layout(*layout);
        *out = mul_u64(layout_entries(*layout), 4, "GQA page-table byte length");
        return KH_OK;
    });
}

static uint64_t page_table_start(const kh_page_table_layout& l, uint32_t req_slot, uint32_t layer, uint32_t block) {
    validate_layout(l);
    KH_REQUIRE(req_slot < l.num_req_slots, "GQA request page table req_slot out of range: req_slot=%u num_req_slots=%u",
               req_slot, l.num_req_slots);
    KH_REQUIRE(layer < l.num_gqa_layers, "GQA request page table layer out of range: layer_index=%u num_layers=%u",
               layer, l.num_gqa_layers);
    KH_REQUIRE(block < l.num_blocks, "GQA request page table block out of range: block_index=%u num_blocks=%u", block,
               l.num_blocks);
    return ((uint64_t(req_slot) * l.num_gqa_layers + layer) * l.num_blocks + block) * l.num_page_ids_per_block;
}

kh_status kh_page_table_index(const kh_page_table_layout* layout, uint32_t req_slot, uint32_t layer_index,
                              uint32_t block_index, uint64_t* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(layout && out, "null argument");
        *out = page_table_start(*layout, req_slot, layer_index, block_index);
        return KH_OK;
    });
}

kh_status kh_page_table_write(kh_device* device, kh_buffer_ref page_ids, const kh_page_table_layout* layout,
                              uint32_t req_slot, uint32_t layer_index, uint32_t block_index, const uint32_t* ids,
                              uint32_t count) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(layout && ids, "null argument");
        const uint64_t start = page_table_start(*layout, req_slot, layer_index, block_index);
        KH_REQUIRE(count == layout->num_page_ids_per_block,
                   "GQA page-id count must match one request/GQA-layer/block entry");
        need(page_ids, layout_entries(*layout) * 4, "page_ids");
        return kh_buffer_write(device, page_ids, start * 4, ids, uint64_t(count) * 4);
    });
}

kh_status kh_page_table_read(kh_device* device, kh_buffer_ref page_ids, const kh_page_table_layout* layout,
                             uint32_t req_slot, uint32_t layer_index, uint32_t block_index, uint32_t* ids,
                             uint32_t count) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(layout && ids, "null argument");
        const uint64_t start = page_table_start(*layout, req_slot, layer_index, block_index);
        KH_REQUIRE(count == layout->num_page_ids_per_block,
                   "GQA page-id count must match one request/GQA-layer/block entry");
        need(page_ids, layout_entries(*layout) * 4, "page_ids");
        return kh_buffer_read(device, page_ids, start * 4, ids, uint64_t(count) * 4);
    });
}

kh_status kh_page_table_reset_req_slot(kh_device* device, kh_buffer_ref page_ids, const kh_page_table_layout* layout,
                                       uint32_t req_slot) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(layout != nullptr, "null argument");
        const uint64_t start = page_table_start(*layout, req_slot, 0, 0);
        const uint64_t per_request = uint64_t(layout->num_gqa_layers) * layout->num_blocks * layout->num_page_ids_per_block;
        need(page_ids, layout_entries(*layout) * 4, "page_ids");
        return kh_buffer_zero(device, page_ids, start * 4, per_request * 4);
    });
}

// ---- SlicedKv -------------------------------------------------------------------------------
kh_status kh_sliced_kv_sizes_get(const kh_sliced_kv_config* config, const kh_sliced_kv_shape* shape,
                                 kh_sliced_kv_sizes* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(config && shape && out, "null argument");
        *out = sliced_kv_sizes(*config, *shape);
        return KH_OK;
    });
}

kh_status kh_sliced_kv_create(kh_device* device, const kh_sliced_kv_config* config,
                              const kh_execution_variant* execution, const kh_sliced_kv_shape* shape,
                              kh_sliced_kv** out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(device && config && execution && shape && out, "null argument");
        auto compute = std::make_unique<kh_sliced_kv>();
        compute->config = *config;
        compute->shape = *shape;
        compute->sizes = sliced_kv_sizes(*config, *shape);
        const kh_sdpa_config sdpa = sdpa_config_of(*config);
        KH_REQUIRE(variant_supports(*execution, sdpa), "execution variant is not supported by the SDPA config");
        KH_REQUIRE(execution->kind == KH_MAP_SLICED_KV, "SlicedKv compute requires a SlicedKv execution variant");
        const uint64_t threads = mul_u64(mul_u64(mul_u64(shape->num_total_sdpa_map_task_templates, config->num_kv_heads,
                                                         "GQA SDPA map thread count"),
                                                 div_ceil(config->num_q_heads / config->num_kv_heads, execution->max_q_heads),
                                                 "GQA SDPA map thread count"),
                                         execution->required_threads, "GQA SDPA map thread count");
        KH_REQUIRE(threads <= 0xffffffffull, "GQA SDPA map threads exceeds the shader u32 count domain");
        init_common(compute->common, device, config->dtype, config->kv_dtype, config->num_q_heads,
                    config->num_kv_heads, config->head_dim, config->scale, config->page_bytes,
                    config->page_table_layout, *execution);
        *out = compute.release();
        return KH_OK;
    });
}

kh_status kh_sliced_kv_destroy(kh_sliced_kv* compute) {
    delete compute;
    return KH_OK;
}

static void sliced_kv_launch(kh_sliced_kv* compute, kh_stream* stream, const kh_sliced_kv_map_buffers* buffers,
                             const kh_sliced_kv_reduce_buffers* fused, kh_buffer_ref arrival_counters,
                             uint32_t page_table_index, uint32_t num_active_tokens, uint32_t num_active_kv_splits) {
    KH_REQUIRE(compute && stream && buffers, "null argument");
    const kh_sliced_kv_sizes& z = compute->sizes;
    const kh_sliced_kv_shape& s = compute->shape;
    // MapInvocation::validate (sliced_kv.rs:594-612)
    KH_REQUIRE(page_table_index < compute->config.page_table_layout.num_gqa_layers, "page_table_index %u out of range",
               page_table_index);
    KH_REQUIRE(num_active_tokens >= 1 && num_active_tokens <= s.num_total_tokens,
               "num_active_tokens %u outside [1, %u]", num_active_tokens, s.num_total_tokens);
    KH_REQUIRE(num_active_kv_splits <= s.num_total_sdpa_map_task_templates, "num_active_kv_splits %u outside [0, %u]",
               num_active_kv_splits, s.num_total_sdpa_map_task_templates);
    need(buffers->q, z.q_bytes, "q");
    need(buffers->kv_pages, compute->config.page_bytes, "kv_pages");
    need(buffers->req_slots, z.req_slots_bytes, "req_slots");
    need(buffers->page_ids, z.page_ids_bytes, "page_ids");
    need(buffers->sdpa_map_task_templates, z.sdpa_map_task_templates_bytes, "sdpa_map_task_templates");
    need(buffers->partial_exp_sums, z.partial_output_stats_bytes, "partial_exp_sums");
    need(buffers->partial_max_logits, z.partial_output_stats_bytes, "partial_max_logits");
    need(buffers->partial_output, z.partial_output_bytes, "partial_output");
    MapParams p{};
    p.req_slots = static_cast<const uint32_t*>(buffers->req_slots.ptr);
    p.page_ids = static_cast<const uint32_t*>(buffers->page_ids.ptr);
    p.visible = nullptr;
    p.q_ranges = nullptr;
    p.templates = static_cast<const uint32_t*>(buffers->sdpa_map_task_templates.ptr);
    p.partial_out = static_cast<float*>(buffers->partial_output.ptr);
    p.partial_sum = static_cast<float*>(buffers->partial_exp_sums.ptr);
    p.partial_max = static_cast<float*>(buffers->partial_max_logits.ptr);
    p.out = nullptr;
    p.num_active_tokens = num_active_tokens;
    p.num_active_q_tiles = num_active_tokens;
    p.layer_index = page_table_index;
    p.direct = 0;
    if (fused != nullptr) {
        KH_REQUIRE(fused->partial_exp_sums.ptr == buffers->partial_exp_sums.ptr &&
                       fused->partial_max_logits.ptr == buffers->partial_max_logits.ptr &&
                       fused->partial_output.ptr == buffers->partial_output.ptr,
                   "the fused call needs the same partial buffers on its map and reduce sides");
        need(fused->cu_sdpa_partial_outputs, z.cu_sdpa_partial_outputs_bytes, "cu_sdpa_partial_outputs");
        need(fused->output, z.q_bytes, "output");
        const uint32_t head_ranges =
            div_ceil(compute->config.num_q_heads / compute->config.num_kv_heads, compute->common.variant.max_q_heads);
        need(arrival_counters, uint64_t(s.num_total_tokens) * compute->config.num_kv_heads * head_ranges * 4,
             "arrival_counters");
        p.cu = static_cast<const uint32_t*>(fused->cu_sdpa_partial_outputs.ptr);
        p.arrivals = static_cast<uint32_t*>(arrival_counters.ptr);
        p.out = fused->output.ptr;
    }
    launch_map(compute->common, stream, p, buffers->q, buffers->kv_pages, num_active_kv_splits);
}

kh_status kh_sliced_kv_map(kh_sliced_kv* compute, kh_stream* stream, const kh_sliced_kv_map_buffers* buffers,
                           uint32_t page_table_index, uint32_t num_active_tokens, uint32_t num_active_kv_splits) {
    return guarded([&]() -> kh_status {
        sliced_kv_launch(compute, stream, buffers, nullptr, kh_buffer_ref{}, page_table_index, num_active_tokens,
                         num_active_kv_splits);
        return KH_OK;
    });
}

kh_status kh_sliced_kv_map_reduce(kh_sliced_kv* compute, kh_stream* stream, const kh_sliced_kv_map_buffers* map_buffers,
                                  const kh_sliced_kv_reduce_buffers* reduce_buffers, kh_buffer_ref arrival_counters,
                                  uint32_t page_table_index, uint32_t num_active_tokens,
                                  uint32_t num_active_kv_splits) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(reduce_buffers != nullptr, "null argument");
        sliced_kv_launch(compute, stream, map_buffers, reduce_buffers, arrival_counters, page_table_index,
                         num_active_tokens, num_active_kv_splits);
        return KH_OK;
    });
}

kh_status kh_sliced_kv_arrival_counter_bytes(const kh_sliced_kv_config* config, const kh_execution_variant* execution,
                                             const kh_sliced_kv_shape* shape, uint64_t* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(config && execution && shape && out, "null argument");
        sliced_kv_sizes(*config, *shape);
        KH_REQUIRE(execution->max_q_heads > 0, "execution variant has no Q heads");
        const uint32_t head_ranges = div_ceil(config->num_q_heads / config->num_kv_heads, execution->max_q_heads);
        *out = uint64_t(shape->num_total_tokens) * config->num_kv_heads * head_ranges * 4;
        return KH_OK;
    });
}

kh_status kh_sliced_kv_reduce(kh_sliced_kv* compute, kh_stream* stream, const kh_sliced_kv_reduce_buffers* buffers,
                              uint32_t num_active_tokens) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(compute && stream && buffers, "null argument");
        const kh_sliced_kv_sizes& z = compute->sizes;
        const kh_sliced_kv_shape& s = compute->shape;
        KH_REQUIRE(stream->device == compute->common.device, "stream does not belong to the compute's device");
        KH_REQUIRE(num_active_tokens >= 1 && num_active_tokens <= s.num_total_tokens,
                   "num_active_tokens %u outside [1, %u]", num_active_tokens, s.num_total_tokens);
        need(buffers->partial_exp_sums, z.partial_output_stats_bytes, "partial_exp_sums");
        need(buffers->partial_max_logits, z.partial_output_stats_bytes, "partial_max_logits");
        need(buffers->partial_output, z.partial_output_bytes, "partial_output");
        need(buffers->cu_sdpa_partial_outputs, z.cu_sdpa_partial_outputs_bytes, "cu_sdpa_partial_outputs");
        need(buffers->output, z.q_bytes, "output");
        use_device(compute->common.device);
        ReduceParams p{};
        p.partial_sum = static_cast<const float*>(buffers->partial_exp_sums.ptr);
        p.partial_max = static_cast<const float*>(buffers->partial_max_logits.ptr);
        p.partial_out = static_cast<const float*>(buffers->partial_output.ptr);
        p.q_ranges = nullptr;
        p.cu = static_cast<const uint32_t*>(buffers->cu_sdpa_partial_outputs.ptr);
        p.out = buffers->output.ptr;
        p.num_q_heads = compute->config.num_q_heads;
        p.head_dim = compute->config.head_dim;
        p.max_q_tokens = 1;
        p.num_active_ranges = num_active_tokens;
        p.num_active_tokens = num_active_tokens;
        p.num_partials = s.num_total_sdpa_map_task_templates;
        p.active = static_cast<const uint32_t*>(stream->active_counts.ptr);
        p.active_range_word = 0;
        launch_reduce(compute->config.dtype, p, num_active_tokens, stream->stream);
        return KH_OK;
    });
}

// ---- SlicedQ --------------------------------------------------------------------------------
kh_status kh_sliced_q_sizes_get(const kh_sliced_q_config* config, const kh_execution_variant* execution,
                                const kh_sliced_q_shape* shape, kh_sliced_q_sizes* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(config && execution && shape && out, "null argument");
        *out = sliced_q_sizes(*config, *execution, *shape);
        return KH_OK;
    });
}

kh_status kh_sliced_q_create(kh_device* device, const kh_sliced_q_config* config,
                             const kh_execution_variant* execution, const kh_sliced_q_shape* shape,
                             int32_t direct_output, kh_sliced_q** out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(device && config && execution && shape && out, "null argument");
        auto compute = std::make_unique<kh_sliced_q>();
        compute->config = *config;
        compute->shape = *shape;
        compute->direct = direct_output != 0;
        compute->sizes = sliced_q_sizes(*config, *execution, *shape);
        const kh_sdpa_config sdpa = sdpa_config_of(*config);
        KH_REQUIRE(variant_supports(*execution, sdpa), "execution variant is not supported by the SDPA config");
        KH_REQUIRE(execution->kind != KH_MAP_SLICED_KV, "SlicedQ compute requires a sliced-Q execution variant");
        if (compute->direct) {
            KH_REQUIRE(shape->num_total_sdpa_map_task_templates == shape->num_total_q_token_tiles,
                       "direct SDPA needs exactly one Map task template per Q-token tile");
        }
        init_common(compute->common, device, config->dtype, config->kv_dtype, config->num_q_heads,
                    config->num_kv_heads, config->head_dim, config->scale, config->page_bytes,
                    config->page_table_layout, *execution);
        *out = compute.release();
        return KH_OK;
    });
}

kh_status kh_sliced_q_destroy(kh_sliced_q* compute) {
    delete compute;
    return KH_OK;
}

static void sliced_q_launch(kh_sliced_q* compute, kh_stream* stream, const kh_sliced_q_direct_buffers& in,
                            kh_buffer_ref partial_sums, kh_buffer_ref partial_max, bool direct,
                            const kh_sliced_q_reduce_buffers* fused, kh_buffer_ref arrival_counters,
                            uint32_t page_table_index, uint32_t num_active_tokens, uint32_t num_active_q_token_tiles,
                            uint32_t num_active_kv_splits) {
    const kh_sliced_q_sizes& z = compute->sizes;
    const kh_sliced_q_shape& s = compute->shape;
    KH_REQUIRE(page_table_index < compute->config.page_table_layout.num_gqa_layers, "page_table_index %u out of range",
               page_table_index);
    KH_REQUIRE(num_active_tokens >= 1 && num_active_tokens <= s.num_total_tokens,
               "num_active_tokens %u outside [1, %u]", num_active_tokens, s.num_total_tokens);
    KH_REQUIRE(num_active_q_token_tiles >= 1 && num_active_q_token_tiles <= s.num_total_q_token_tiles,
               "num_active_q_token_tiles %u outside [1, %u]", num_active_q_token_tiles, s.num_total_q_token_tiles);
    KH_REQUIRE(num_active_kv_splits >= 1 && num_active_kv_splits <= s.num_total_sdpa_map_task_templates,
               "num_active_kv_splits %u outside [1, %u]", num_active_kv_splits, s.num_total_sdpa_map_task_templates);
    // MapInvocation::validate (sliced_q.rs:521-545)
    need(in.q, z.q_bytes, "q");
    need(in.kv_pages, compute->config.page_bytes, "kv_pages");
    need(in.req_slots, uint64_t(s.num_total_tokens) * 4, "req_slots");
    need(in.page_ids, layout_entries(compute->config.page_table_layout) * 4, "page_ids");
    need(in.visible_kv_token_ranges, uint64_t(s.num_total_tokens) * 8, "visible_kv_token_ranges");
    need(in.q_token_ranges, uint64_t(s.num_total_q_token_tiles) * 8, "q_token_ranges");
    need(in.sdpa_map_task_templates, uint64_t(s.num_total_sdpa_map_task_templates) * 12, "sdpa_map_task_templates");
    if (direct) {
        need(in.output, z.q_bytes, "output");
    } else {
        need(in.output, z.partial_output_bytes, "partial_output");
        need(partial_sums, z.partial_output_stats_bytes, "partial_exp_sums");
        need(partial_max, z.partial_output_stats_bytes, "partial_max_logits");
    }
    MapParams p{};
    p.req_slots = static_cast<const uint32_t*>(in.req_slots.ptr);
    p.page_ids = static_cast<const uint32_t*>(in.page_ids.ptr);
    p.visible = static_cast<const uint32_t*>(in.visible_kv_token_ranges.ptr);
    p.q_ranges = static_cast<const uint32_t*>(in.q_token_ranges.ptr);
    p.templates = static_cast<const uint32_t*>(in.sdpa_map_task_templates.ptr);
    if (direct) {
        p.out = in.output.ptr;
    } else {
        p.partial_out = static_cast<float*>(in.output.ptr);
        p.partial_sum = static_cast<float*>(partial_sums.ptr);
        p.partial_max = static_cast<float*>(partial_max.ptr);
    }
    p.num_active_tokens = num_active_tokens;
    p.num_active_q_tiles = num_active_q_token_tiles;
    p.layer_index = page_table_index;
    p.direct = direct ? 1u : 0u;
    if (fused != nullptr) {
        KH_REQUIRE(!direct, "direct SDPA has no Reduce stage");
        KH_REQUIRE(fused->partial_exp_sums.ptr == partial_sums.ptr && fused->partial_max_logits.ptr == partial_max.ptr &&
                       fused->partial_output.ptr == in.output.ptr && fused->q_token_ranges.ptr == in.q_token_ranges.ptr,
                   "the fused call needs the same partial and range buffers on its map and reduce sides");
        need(fused->cu_sdpa_partial_outputs, (uint64_t(s.num_total_q_token_tiles) + 1) * 4, "cu_sdpa_partial_outputs");
        need(fused->output, z.q_bytes, "output");
        const uint32_t head_ranges =
            div_ceil(compute->config.num_q_heads / compute->config.num_kv_heads, compute->common.variant.max_q_heads);
        need(arrival_counters, uint64_t(s.num_total_q_token_tiles) * compute->config.num_kv_heads * head_ranges * 4,
             "arrival_counters");
        p.cu = static_cast<const uint32_t*>(fused->cu_sdpa_partial_outputs.ptr);
        p.arrivals = static_cast<uint32_t*>(arrival_counters.ptr);
        p.out = fused->output.ptr;
    }
    launch_map(compute->common, stream, p, in.q, in.kv_pages, num_active_kv_splits);
}

kh_status kh_sliced_q_map(kh_sliced_q* compute, kh_stream* stream, const kh_sliced_q_map_buffers* buffers,
                          uint32_t page_table_index, uint32_t num_active_tokens, uint32_t num_active_q_token_tiles,
                          uint32_t num_active_kv_splits) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(compute && stream && buffers, "null argument");
        KH_REQUIRE(!compute->direct, "this compute was created for direct output");
        kh_sliced_q_direct_buffers in{buffers->q,
                                      buffers->kv_pages,
                                      buffers->req_slots,
                                      buffers->page_ids,
                                      buffers->visible_kv_token_ranges,
                                      buffers->q_token_ranges,
                                      buffers->sdpa_map_task_templates,
                                      buffers->partial_output};
        sliced_q_launch(compute, stream, in, buffers->partial_exp_sums, buffers->partial_max_logits, false, nullptr,
                        kh_buffer_ref{}, page_table_index, num_active_tokens, num_active_q_token_tiles,
                        num_active_kv_splits);
        return KH_OK;
    });
}

kh_status kh_sliced_q_map_reduce(kh_sliced_q* compute, kh_stream* stream, const kh_sliced_q_map_buffers* buffers,
                                 const kh_sliced_q_reduce_buffers* reduce_buffers, kh_buffer_ref arrival_counters,
                                 uint32_t page_table_index, uint32_t num_active_tokens,
                                 uint32_t num_active_q_token_tiles, uint32_t num_active_kv_splits) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(compute && stream && buffers && reduce_buffers, "null argument");
        KH_REQUIRE(!compute->direct, "this compute was created for direct output");
        kh_sliced_q_direct_buffers in{buffers->q,
                                      buffers->kv_pages,
                                      buffers->req_slots,
                                      buffers->page_ids,
                                      buffers->visible_kv_token_ranges,
                                      buffers->q_token_ranges,
                                      buffers->sdpa_map_task_templates,
                                      buffers->partial_output};
        sliced_q_launch(compute, stream, in, buffers->partial_exp_sums, buffers->partial_max_logits, false,
                        reduce_buffers, arrival_counters, page_table_index, num_active_tokens,
                        num_active_q_token_tiles, num_active_kv_splits);
        return KH_OK;
    });
}

kh_status kh_sliced_q_arrival_counter_bytes(const kh_sliced_q_config* config, const kh_execution_variant* execution,
                                            const kh_sliced_q_shape* shape, uint64_t* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(config && execution && shape && out, "null argument");
        sliced_q_sizes(*config, *execution, *shape);
        const uint32_t head_ranges = div_ceil(config->num_q_heads / config->num_kv_heads, execution->max_q_heads);
        *out = uint64_t(shape->num_total_q_token_tiles) * config->num_kv_heads * head_ranges * 4;
        return KH_OK;
    });
}

kh_status kh_sliced_q_direct(kh_sliced_q* compute, kh_stream* stream, const kh_sliced_q_direct_buffers* buffers,
                             uint32_t page_table_index, uint32_t num_active_tokens,
                             uint32_t num_active_q_token_tiles) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(compute && stream && buffers, "null argument");
        KH_REQUIRE(compute->direct, "this compute was created for Map/Reduce output");
        sliced_q_launch(compute, stream, *buffers, kh_buffer_ref{}, kh_buffer_ref{}, true, nullptr, kh_buffer_ref{},
                        page_table_index, num_active_tokens, num_active_q_token_tiles, num_active_q_token_tiles);
        return KH_OK;
    });
}

kh_status kh_sliced_q_reduce(kh_sliced_q* compute, kh_stream* stream, const kh_sliced_q_reduce_buffers* buffers,
                             uint32_t num_active_q_token_tiles) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(compute && stream && buffers, "null argument");
        KH_REQUIRE(!compute->direct, "direct SDPA has no Reduce stage");
        const kh_sliced_q_sizes& z = compute->sizes;
        const kh_sliced_q_shape& s = compute->shape;
        KH_REQUIRE(stream->device == compute->common.device, "stream does not belong to the compute's device");
        KH_REQUIRE(num_active_q_token_tiles >= 1 && num_active_q_token_tiles <= s.num_total_q_token_tiles,
                   "num_active_q_token_tiles %u outside [1, %u]", num_active_q_token_tiles,
                   s.num_total_q_token_tiles);
        need(buffers->partial_output, z.partial_output_bytes, "partial_output");
        need(buffers->partial_exp_sums, z.partial_output_stats_bytes, "partial_exp_sums");
        need(buffers->partial_max_logits, z.partial_output_stats_bytes, "partial_max_logits");
        need(buffers->q_token_ranges, uint64_t(s.num_total_q_token_tiles) * 8, "q_token_ranges");
        need(buffers->cu_sdpa_partial_outputs, (uint64_t(s.num_total_q_token_tiles) + 1) * 4,
             "cu_sdpa_partial_outputs");
        need(buffers->output, z.q_bytes, "output");
        use_device(compute->common.device);
        ReduceParams p{};
        p.partial_sum = static_cast<const float*>(buffers->partial_exp_sums.ptr);
        p.partial_max = static_cast<const float*>(buffers->partial_max_logits.ptr);
        p.partial_out = static_cast<const float*>(buffers->partial_output.ptr);
        p.q_ranges = static_cast<const uint32_t*>(buffers->q_token_ranges.ptr);
        p.cu = static_cast<const uint32_t*>(buffers->cu_sdpa_partial_outputs.ptr);
        p.out = buffers->output.ptr;
        p.num_q_heads = compute->config.num_q_heads;
        p.head_dim = compute->config.head_dim;
        p.max_q_tokens = compute->common.variant.max_q_tokens;
        p.num_active_ranges = num_active_q_token_tiles;
        p.num_active_tokens = s.num_total_tokens;
        p.num_partials = s.num_total_sdpa_map_task_templates;
        p.active = static_cast<const uint32_t*>(stream->active_counts.ptr);
        p.active_range_word = 1;
        launch_reduce(compute->config.dtype, p, num_active_q_token_tiles, stream->stream);
        return KH_OK;
    });
}

// ---- LSE combine ----------------------------------------------------------------------------
kh_status kh_combine_partials(kh_device* device, kh_stream* stream, uint32_t num_partials, uint32_t num_rows,
                              uint32_t head_dim, kh_buffer_ref exp_sums, kh_buffer_ref max_logits,
                              kh_buffer_ref partial_output, kh_dtype out_dtype, kh_buffer_ref output,
                              kh_buffer_ref out_exp_sums, kh_buffer_ref out_max_logits) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(device && stream, "null argument");
        KH_REQUIRE(stream->device == device, "stream does not belong to the device");
        KH_REQUIRE(num_partials > 0 && num_rows > 0 && head_dim > 0, "combine needs partials, rows and a head dimension");
        KH_REQUIRE(dtype_size(out_dtype) >= 2, "unsupported output dtype");
        const uint64_t stats = uint64_t(num_partials) * num_rows;
        need(exp_sums, stats * 4, "exp_sums");
        need(max_logits, stats * 4, "max_logits");
        need(partial_output, stats * head_dim * 4, "partial_output");
        need(output, uint64_t(num_rows) * head_dim * dtype_size(out_dtype), "output");
        const bool chain = out_exp_sums.ptr != nullptr || out_max_logits.ptr != nullptr;
        if (chain) {
            need(out_exp_sums, uint64_t(num_rows) * 4, "out_exp_sums");
            need(out_max_logits, uint64_t(num_rows) * 4, "out_max_logits");
        }
        use_device(device);
        // rows ride in grid.x as "heads" of a single one-token range
        ReduceParams p{};
        p.partial_sum = static_cast<const float*>(exp_sums.ptr);
        p.partial_max = static_cast<const float*>(max_logits.ptr);
        p.partial_out = static_cast<const float*>(partial_output.ptr);
        p.q_ranges = nullptr;
        p.cu = nullptr;
        p.fixed_partials = num_partials;
        p.num_partials = num_partials;
        p.out = output.ptr;
        p.out_sum = chain ? static_cast<float*>(out_exp_sums.ptr) : nullptr;
        p.out_max = chain ? static_cast<float*>(out_max_logits.ptr) : nullptr;
        p.num_q_heads = num_rows;
        p.head_dim = head_dim;
        p.max_q_tokens = 1;
        p.num_active_ranges = 1;
        p.num_active_tokens = 1;
        launch_reduce(out_dtype, p, 1, stream->stream);
        return KH_OK;
    });
}

kh_status kh_combine_packed_partials(kh_device* device, kh_stream* stream, uint32_t num_partials, uint32_t num_rows,
                                     uint32_t head_dim, kh_buffer_ref packed, kh_dtype out_dtype,
                                     kh_buffer_ref output) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(device && stream, "null argument");
        KH_REQUIRE(stream->device == device, "stream does not belong to the device");
        KH_REQUIRE(num_partials > 0 && num_rows > 0 && head_dim > 0, "combine needs partials, rows and a head dimension");
        KH_REQUIRE(dtype_size(out_dtype) >= 2, "unsupported output dtype");
        KH_REQUIRE(num_rows % 4 == 0 && head_dim % 4 == 0,
                   "packed partials need rows and head_dim that are multiples of 4 (16-byte aligned sections)");
        KH_REQUIRE((reinterpret_cast<uintptr_t>(packed.ptr) & 15) == 0, "packed partials must be 16-byte aligned");
        const uint64_t record = uint64_t(num_rows) * (uint64_t(head_dim) + 2);
        need(packed, uint64_t(num_partials) * record * 4, "packed");
        need(output, uint64_t(num_rows) * head_dim * dtype_size(out_dtype), "output");
        use_device(device);
        const float* base = static_cast<const float*>(packed.ptr);
        ReduceParams p{};
        p.partial_sum = base;
        p.partial_max = base + num_rows;
        p.partial_out = base + 2 * uint64_t(num_rows);
        p.fixed_partials = num_partials;
        p.num_partials = num_partials;
        p.stat_stride = record;
        p.out_stride = record;
        p.out = output.ptr;
        p.num_q_heads = num_rows;
        p.head_dim = head_dim;
        p.max_q_tokens = 1;
        p.num_active_ranges = 1;
        p.num_active_tokens = 1;
        launch_reduce(out_dtype, p, 1, stream->stream);
        return KH_OK;
    });
}

}  // extern "C"

// ---- SlicedKv attention on library-held scratch ------------------------------------------------
// The partial statistics and partial outputs of one map + reduce pair live in an array of the module image:
// nothing is allocated or freed on any call. Section layout for `rows` = active templates * Q heads, each section
// starting on a 256-byte boundary: [exp sums: rows f32][max logits: rows f32][partial output: rows * D f32].
namespace kh {

constexpr uint64_t kStaticPartialFloats = KH_STATIC_PARTIALS_BYTES / 4;
static __device__ __align__(256) float g_static_partials[kStaticPartialFloats];

constexpr int kStaticMaxDevices = 64;
static float* g_static_partials_at[kStaticMaxDevices];  // address of the array on each GPU, looked up once
static std::mutex g_static_mutex;

static uint64_t static_section_floats(uint64_t rows) { return (rows + 63) / 64 * 64; }

static uint64_t static_bytes_needed(uint32_t num_q_heads, uint32_t head_dim, uint32_t num_active_kv_splits) {
    const uint64_t rows = uint64_t(num_active_kv_splits) * num_q_heads;
    return (2 * static_section_floats(rows) + static_section_floats(rows * head_dim)) * 4;
}

static float* static_partials_on(const kh_device* device) {
    KH_REQUIRE(device->ordinal >= 0 && device->ordinal < kStaticMaxDevices,
               "device ordinal %d is beyond the %d GPUs the shared partial array is tracked for", device->ordinal,
               kStaticMaxDevices);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    float*& slot = g_static_partials_at[device->ordinal];
    if (slot == nullptr) {
        use_device(device);
        float* address = nullptr;
        KH_CUDA(cudaGetSymbolAddress((void**)&address, g_static_partials));
        KH_REQUIRE(address != nullptr && (reinterpret_cast<uintptr_t>(address) & 255) == 0,
                   "the shared partial array has no 256-byte aligned device address");
        slot = address;
    }
    return slot;
}

}  // namespace kh

kh_status kh_sliced_kv_static_bytes_needed(const kh_sliced_kv_config* config, uint32_t num_active_kv_splits,
                                           uint64_t* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(config && out, "null argument");
        sliced_kv_sizes(*config, kh_sliced_kv_shape{1, 1});
        *out = static_bytes_needed(config->num_q_heads, config->head_dim, num_active_kv_splits);
        return KH_OK;
    });
}

kh_status kh_sliced_kv_attend_static(kh_sliced_kv* compute, kh_stream* stream,
                                     const kh_sliced_kv_static_buffers* buffers, uint32_t page_table_index,
                                     uint32_t num_active_tokens, uint32_t num_active_kv_splits) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(compute && stream && buffers, "null argument");
        const kh_sliced_kv_config& config = compute->config;
        const kh_sliced_kv_sizes& z = compute->sizes;
        const kh_sliced_kv_shape& s = compute->shape;
        KH_REQUIRE(stream->device == compute->common.device, "stream does not belong to the compute's device");
        KH_REQUIRE(page_table_index < config.page_table_layout.num_gqa_layers, "page_table_index %u out of range",
                   page_table_index);
        KH_REQUIRE(num_active_tokens >= 1 && num_active_tokens <= s.num_total_tokens,
                   "num_active_tokens %u outside [1, %u]", num_active_tokens, s.num_total_tokens);
        KH_REQUIRE(num_active_kv_splits <= s.num_total_sdpa_map_task_templates,
                   "num_active_kv_splits %u outside [0, %u]", num_active_kv_splits,
                   s.num_total_sdpa_map_task_templates);
        const uint64_t bytes = static_bytes_needed(config.num_q_heads, config.head_dim, num_active_kv_splits);
        if (bytes > KH_STATIC_PARTIALS_BYTES) {
            raise(KH_RESOURCE_EXHAUSTED,
                  "%u map task templates x %u Q heads x head_dim %u need %llu bytes of partial state; the shared array "
                  "holds %u: call kh_sliced_kv_map and kh_sliced_kv_reduce with your own partial buffers",
                  num_active_kv_splits, config.num_q_heads, config.head_dim, (unsigned long long)bytes,
                  unsigned(KH_STATIC_PARTIALS_BYTES));
        }
        need(buffers->q, z.q_bytes, "q");
        need(buffers->kv_pages, config.page_bytes, "kv_pages");
        need(buffers->req_slots, z.req_slots_bytes, "req_slots");
        need(buffers->page_ids, z.page_ids_bytes, "page_ids");
        need(buffers->sdpa_map_task_templates, z.sdpa_map_task_templates_bytes, "sdpa_map_task_templates");
        need(buffers->cu_sdpa_partial_outputs, z.cu_sdpa_partial_outputs_bytes, "cu_sdpa_partial_outputs");
        need(buffers->output, z.q_bytes, "output");

        float* base = static_partials_on(compute->common.device);
        const uint64_t rows = uint64_t(num_active_kv_splits) * config.num_q_heads;
        float* exp_sums = base;
        float* max_logits = exp_sums + static_section_floats(rows);
        float* partial_output = max_logits + static_section_floats(rows);

        MapParams p{};
        p.req_slots = static_cast<const uint32_t*>(buffers->req_slots.ptr);
        p.page_ids = static_cast<const uint32_t*>(buffers->page_ids.ptr);
        p.templates = static_cast<const uint32_t*>(buffers->sdpa_map_task_templates.ptr);
        p.partial_out = partial_output;
        p.partial_sum = exp_sums;
        p.partial_max = max_logits;
        p.num_active_tokens = num_active_tokens;
        p.num_active_q_tiles = num_active_tokens;
        p.layer_index = page_table_index;
        launch_map(compute->common, stream, p, buffers->q, buffers->kv_pages, num_active_kv_splits);

        ReduceParams r{};
        r.partial_sum = exp_sums;
        r.partial_max = max_logits;
        r.partial_out = partial_output;
        r.cu = static_cast<const uint32_t*>(buffers->cu_sdpa_partial_outputs.ptr);
        r.out = buffers->output.ptr;
        r.num_q_heads = config.num_q_heads;
        r.head_dim = config.head_dim;
        r.max_q_tokens = 1;
        r.num_active_ranges = num_active_tokens;
        r.num_active_tokens = num_active_tokens;
        r.num_partials = num_active_kv_splits;  // the sections of the shared array are sized for exactly these
        r.active = static_cast<const uint32_t*>(stream->active_counts.ptr);
        r.active_range_word = 0;
        launch_reduce(config.dtype, r, num_active_tokens, stream->stream);
        return KH_OK;
    });
}
