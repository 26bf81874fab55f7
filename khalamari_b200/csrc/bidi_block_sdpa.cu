// BiDi-block SDPA: dense bidirectional attention of every Q token over all tokens of its own request block, written
// as one more partial of the SplitKV partial-state layout
// (crates/inference-backend-metal/src/components/gqa/bidi_block_sdpa.rs,
//  crates/inference-backend-metal/src/components/metal/gqa_bidi_block_sdpa.metal:10-88).
// The block's K/V are contiguous rows [tokens][Hkv][D] (the proposal block is not in the paged cache yet); the block
// is a handful of tokens, so this is a latency kernel: one warp per (Q head, Q-token range, token offset) - the
// reference's grid cell - lanes across the head dimension for the scores, lanes across output columns for P V.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <memory>

#include "common.h"
#include "cuda_objects.h"

namespace kh {

struct BidiParams {
    const void* q;
    const void* local_k;
    const void* local_v;
    const uint32_t* q_token_ranges;
    const uint32_t* cu;
    float* partial_sum;
    float* partial_max;
    float* partial_out;
    const uint32_t* active;  // replay: device words {tokens, Q-token tiles, templates}; null: by-value count
    uint32_t num_active_ranges;
    uint32_t block_size;
    uint32_t max_q_tokens;
    uint32_t num_q_heads;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    uint32_t num_total_tokens;
    uint32_t num_slots;
    float scale;
};

template <typename T>
__device__ __forceinline__ float load_as_f32(const T* p);
template <>
__device__ __forceinline__ float load_as_f32<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_as_f32<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <>
__device__ __forceinline__ float load_as_f32<__half>(const __half* p) { return __half2float(*p); }

constexpr int kBidiWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kBidiWarps * 32) bidi_block_sdpa_kernel(const BidiParams p) {
    extern __shared__ float logits_all[];  // [warps][block_size]
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t head = blockIdx.x * kBidiWarps + warp;
    const uint32_t range = blockIdx.y;
    const uint32_t offset = blockIdx.z;
    uint32_t active_ranges = p.num_active_ranges;
    if (p.active != nullptr) active_ranges = min(p.active[1], active_ranges);
    if (head >= p.num_q_heads || range >= active_ranges) return;
    const uint32_t begin = p.q_token_ranges[range * 2], end = p.q_token_ranges[range * 2 + 1];
    if (end <= begin || end > p.num_total_tokens || offset >= end - begin) return;
    const uint32_t token = begin + offset;
    const uint32_t kv_head = head / (p.num_q_heads / p.num_kv_heads);
    const uint32_t block_begin = token / p.block_size * p.block_size;
    const uint32_t cu_end = p.cu[range + 1];
    if (cu_end == 0 || cu_end > p.num_slots) return;  // no slot for the block partial inside the buffers
    const uint32_t slot = cu_end - 1;
    float* logits = logits_all + warp * p.block_size;
    const T* q = static_cast<const T*>(p.q) + (uint64_t(token) * p.num_q_heads + head) * p.head_dim;
    const T* k_rows = static_cast<const T*>(p.local_k);
    const T* v_rows = static_cast<const T*>(p.local_v);
    const uint32_t D = p.head_dim;

    // scores: lanes stride the head dimension, one shuffle reduction per block token
    float block_max = -INFINITY;
    for (uint32_t j = 0; j < p.block_size; ++j) {
        const T* k = k_rows + (uint64_t(block_begin + j) * p.num_kv_heads + kv_head) * D;
        float score = 0.0f;
        for (uint32_t d = lane; d < D; d += 32) score += load_as_f32<T>(q + d) * load_as_f32<T>(k + d);
#pragma unroll
        for (int shift = 16; shift > 0; shift >>= 1) score += __shfl_xor_sync(0xffffffffu, score, shift);
        score *= p.scale;
        block_max = fmaxf(block_max, score);
        if (lane == 0) logits[j] = score;
    }
    __syncwarp();
    float exp_sum = 0.0f;
    for (uint32_t j = lane; j < p.block_size; j += 32) {
        const float weight = expf(logits[j] - block_max);
        logits[j] = weight;
        exp_sum += weight;
    }
#pragma unroll
    for (int shift = 16; shift > 0; shift >>= 1) exp_sum += __shfl_xor_sync(0xffffffffu, exp_sum, shift);
    __syncwarp();
    const uint64_t index = (uint64_t(slot) * p.num_q_heads + head) * p.max_q_tokens + offset;
    if (lane == 0) {
        p.partial_sum[index] = exp_sum;
        p.partial_max[index] = block_max;
    }
    const float inv = exp_sum > 0.0f ? 1.0f / exp_sum : 0.0f;
    for (uint32_t d = lane; d < D; d += 32) {
        float out = 0.0f;
        for (uint32_t j = 0; j < p.block_size; ++j) {
            out += logits[j] * load_as_f32<T>(v_rows + (uint64_t(block_begin + j) * p.num_kv_heads + kv_head) * D + d);
        }
        p.partial_out[index * D + d] = out * inv;
    }
}

}  // namespace kh

using namespace kh;

struct kh_bidi_block_sdpa {
    kh_device* device;
    kh_bidi_block_sdpa_config config;
};

// Config::validate (bidi_block_sdpa.rs:67-84).
static void validate_bidi_config(const kh_bidi_block_sdpa_config& c) {
    KH_REQUIRE(c.block_size > 0 && c.max_q_tokens > 0 && c.num_q_heads > 0 && c.num_kv_heads > 0 && c.head_dim > 0,
               "bidirectional block SDPA dimensions must be positive");
    KH_REQUIRE(c.num_q_heads % c.num_kv_heads == 0, "bidirectional block SDPA Q heads must be a multiple of KV heads");
    KH_REQUIRE(std::isfinite(c.scale) && c.scale > 0.0f, "bidirectional block SDPA scale must be finite and positive");
    KH_REQUIRE(c.head_dim % 32 == 0, "bidirectional block SDPA head_dim must be divisible by the SIMD width");
    KH_REQUIRE(c.dtype == KH_DTYPE_FLOAT32 || c.dtype == KH_DTYPE_BFLOAT16 || c.dtype == KH_DTYPE_FLOAT16,
               "unsupported bidirectional block SDPA dtype");
    KH_REQUIRE(uint64_t(c.block_size) * 4 * kBidiWarps <= 48 * 1024,
               "bidirectional block SDPA block_size %u needs more thread-block memory than the kernel reserves", c.block_size);
}

extern "C" {

kh_status kh_bidi_block_sdpa_create(kh_device* device, const kh_bidi_block_sdpa_config* config,
                                    kh_bidi_block_sdpa** out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(device && config && out, "null argument");
        validate_bidi_config(*config);
        auto compute = std::make_unique<kh_bidi_block_sdpa>();
        compute->device = device;
        compute->config = *config;
        *out = compute.release();
        return KH_OK;
    });
}

kh_status kh_bidi_block_sdpa_destroy(kh_bidi_block_sdpa* compute) {
    delete compute;
    return KH_OK;
}

kh_status kh_bidi_block_sdpa_invoke(kh_bidi_block_sdpa* compute, kh_stream* stream,
                                    const kh_bidi_block_sdpa_shape* shape, uint32_t num_active_q_token_ranges,
                                    const kh_bidi_block_sdpa_buffers* buffers) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(compute && stream && shape && buffers, "null argument");
        KH_REQUIRE(stream->device == compute->device, "stream does not belong to the compute's device");
        const kh_bidi_block_sdpa_config& c = compute->config;
        // Shape::validate (bidi_block_sdpa.rs:147-174)
        KH_REQUIRE(shape->num_total_tokens > 0, "bidirectional block SDPA shape requires tokens");
        KH_REQUIRE(shape->num_total_q_token_ranges > 0 && shape->num_total_q_token_ranges <= shape->num_total_tokens,
                   "bidirectional block SDPA Q-token ranges out of range");
        KH_REQUIRE(shape->num_total_partial_output_slots >= shape->num_total_q_token_ranges,
                   "bidirectional block SDPA needs a partial-output slot per Q-token range");
        KH_REQUIRE(shape->num_total_tokens % c.block_size == 0,
                   "bidirectional block SDPA tokens must contain complete request blocks");
        KH_REQUIRE(num_active_q_token_ranges >= 1 && num_active_q_token_ranges <= shape->num_total_q_token_ranges,
                   "num_active_q_token_ranges %u outside [1, %u]", num_active_q_token_ranges,
                   shape->num_total_q_token_ranges);
        const uint64_t q_elems = mul_u64(mul_u64(shape->num_total_tokens, c.num_q_heads, "bidirectional block SDPA Q element count"),
                                         c.head_dim, "bidirectional block SDPA Q element count");
        const uint64_t kv_elems = mul_u64(mul_u64(shape->num_total_tokens, c.num_kv_heads, "bidirectional block SDPA K/V element count"),
                                          c.head_dim, "bidirectional block SDPA K/V element count");
        const uint64_t stats = mul_u64(mul_u64(shape->num_total_partial_output_slots, c.num_q_heads,
                                               "bidirectional block SDPA partial-output statistic element count"),
                                       c.max_q_tokens, "bidirectional block SDPA partial-output statistic element count");
        KH_REQUIRE(q_elems <= 0xffffffffull && kv_elems <= 0xffffffffull,
                   "bidirectional block SDPA Q / K/V exceeds the shader u32 count domain");
        const uint32_t elem = dtype_size(c.dtype);
        need(buffers->q, q_elems * elem, "q");
        need(buffers->local_k, kv_elems * elem, "local_k");
        need(buffers->local_v, kv_elems * elem, "local_v");
        need(buffers->q_token_ranges, uint64_t(shape->num_total_q_token_ranges) * 8, "q_token_ranges");
        need(buffers->cu_sdpa_partial_outputs, (uint64_t(shape->num_total_q_token_ranges) + 1) * 4,
             "cu_sdpa_partial_outputs");
        need(buffers->partial_exp_sums, stats * 4, "partial_exp_sums");
        need(buffers->partial_max_logits, stats * 4, "partial_max_logits");
        need(buffers->partial_output, mul_u64(stats, c.head_dim, "bidirectional block SDPA partial output") * 4,
             "partial_output");
        KH_REQUIRE(c.max_q_tokens <= 65535 && shape->num_total_q_token_ranges <= 65535,
                   "bidirectional block SDPA grid exceeds 65535 Q-token ranges or tokens per range");
        use_device(compute->device);
        BidiParams p{};
        p.q = buffers->q.ptr;
        p.local_k = buffers->local_k.ptr;
        p.local_v = buffers->local_v.ptr;
        p.q_token_ranges = static_cast<const uint32_t*>(buffers->q_token_ranges.ptr);
        p.cu = static_cast<const uint32_t*>(buffers->cu_sdpa_partial_outputs.ptr);
        p.partial_sum = static_cast<float*>(buffers->partial_exp_sums.ptr);
        p.partial_max = static_cast<float*>(buffers->partial_max_logits.ptr);
        p.partial_out = static_cast<float*>(buffers->partial_output.ptr);
        p.active = static_cast<const uint32_t*>(stream->active_counts.ptr);
        p.num_active_ranges = num_active_q_token_ranges;
        p.block_size = c.block_size;
        p.max_q_tokens = c.max_q_tokens;
        p.num_q_heads = c.num_q_heads;
        p.num_kv_heads = c.num_kv_heads;
        p.head_dim = c.head_dim;
        p.num_total_tokens = shape->num_total_tokens;
        p.num_slots = shape->num_total_partial_output_slots;
        p.scale = c.scale;
        const dim3 grid(div_ceil(c.num_q_heads, kBidiWarps), num_active_q_token_ranges, c.max_q_tokens);
        const size_t smem = size_t(kBidiWarps) * c.block_size * 4;
        if (c.dtype == KH_DTYPE_BFLOAT16) bidi_block_sdpa_kernel<__nv_bfloat16><<<grid, kBidiWarps * 32, smem, stream->stream>>>(p);
        else if (c.dtype == KH_DTYPE_FLOAT16) bidi_block_sdpa_kernel<__half><<<grid, kBidiWarps * 32, smem, stream->stream>>>(p);
        else bidi_block_sdpa_kernel<float><<<grid, kBidiWarps * 32, smem, stream->stream>>>(p);
        KH_CUDA(cudaGetLastError());
        return KH_OK;
    });
}

}  // extern "C"
