// KV page write: scatters the new tokens' K and V rows into their pages, the step that precedes SDPA in a
// GQA layer (crates/inference-backend-metal/src/components/gqa/kv_page_write.rs:62-257,
// components/metal/gqa_kv_page_write.metal:32-80), and the FP8 E4M3FN storage codec of
// components/gqa/fp8.rs:19-58. The destination address is the one every attention kernel reads:
//   page = page_ids[((slot * L + layer) * B + t / (P * n)) * n + (t / P) % n]
//   byte = page * page_bytes + ((plane * Hkv + head) * P + t % P) * D * e + d * e,   plane 0 = K, 1 = V.
// HBM-bound copy: one thread moves 16 source bytes (8 elements) of K and of V.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cmath>
#include <cstring>
#include <memory>

#include "cuda_objects.h"

namespace kh {

// ---- FP8 E4M3FN (bias 7, no infinities, 0x7f = NaN, largest finite 448), one fixed unit scale -------------
// Round to nearest, ties to even; finite and infinite magnitudes at or above 448 saturate to 0x7e; NaN keeps
// the NaN encoding (fp8.rs:19-44). The value is exact in f32, so the rounding is done on the f32 bit pattern:
// normal results keep 3 mantissa bits, results below 2^-6 are multiples of 2^-9.
__host__ __device__ inline uint8_t fp8_e4m3_from_f32(float value) {
    uint32_t bits;
#ifdef __CUDA_ARCH__
    bits = __float_as_uint(value);
#else
    memcpy(&bits, &value, 4);
#endif
    const uint8_t sign = uint8_t((bits >> 24) & 0x80u);
    const uint32_t mag = bits & 0x7fffffffu;
    if (mag > 0x7f800000u) return sign | 0x7f;                  // NaN
    if (mag >= 0x43e00000u) return sign | 0x7e;                 // >= 448 (and infinity)
    if (mag < 0x3c800000u) {                                    // < 2^-6: multiples of 2^-9, ties to even
        float magnitude;
#ifdef __CUDA_ARCH__
        magnitude = __uint_as_float(mag);
        const uint32_t steps = uint32_t(__float2int_rn(magnitude * 512.0f));
#else
        memcpy(&magnitude, &mag, 4);
        const uint32_t steps = uint32_t(std::nearbyint(magnitude * 512.0f));
#endif
        return sign | uint8_t(steps < 8u ? steps : 8u);
    }
    // normal: keep 3 of the 23 mantissa bits, ties to even; a carry out of the mantissa raises the exponent
    const uint32_t dropped = mag & 0xfffffu;
    uint32_t kept = mag >> 20;                                  // exponent (8 bits) and 3 mantissa bits
    if (dropped > 0x80000u || (dropped == 0x80000u && (kept & 1u))) ++kept;
    const int32_t exponent = int32_t(kept >> 3) - 127 + 7;      // E4M3 biased exponent
    const uint32_t mantissa = kept & 7u;
    if (exponent > 15 || (exponent == 15 && mantissa >= 7u)) return sign | 0x7e;
    return sign | uint8_t(uint32_t(exponent) << 3) | uint8_t(mantissa);
}

// fp8.rs:46-58: exponent 0 is mantissa * 2^-9 (exact in bf16), 0x7f / 0xff are NaN.
__host__ __device__ inline uint16_t bf16_bits_from_fp8_e4m3(uint8_t bits) {
    const uint16_t sign = uint16_t(bits & 0x80u) << 8;
    const uint32_t exponent = (bits >> 3) & 0x0fu;
    const uint32_t mantissa = bits & 0x07u;
    if (exponent == 15 && mantissa == 7) return sign | 0x7fc0;
    if (exponent == 0) {
        if (mantissa == 0) return sign;
        // mantissa * 2^-9 with mantissa in 1..7: normalise by hand (leading one at bit position p)
        const uint32_t p = mantissa >= 4 ? 2 : (mantissa >= 2 ? 1 : 0);
        const uint32_t frac = (mantissa << (7 - p)) & 0x7fu;
        return sign | uint16_t((127 - 9 + p) << 7) | uint16_t(frac);
    }
    return sign | uint16_t((exponent + 120) << 7) | uint16_t(mantissa << 4);
}

__host__ __device__ inline float f32_from_bf16_bits(uint16_t bits) {
    const uint32_t wide = uint32_t(bits) << 16;
#ifdef __CUDA_ARCH__
    return __uint_as_float(wide);
#else
    float value;
    memcpy(&value, &wide, 4);
    return value;
#endif
}

struct PageWriteParams {
    uint8_t* pages;
    const uint16_t* flat_k;
    const uint16_t* flat_v;
    const uint32_t* req_slots;
    const uint32_t* flat_token_indices;
    const uint32_t* page_ids;
    uint32_t* status;
    uint32_t num_active_token_writes;
    uint32_t layer_index;
    uint32_t num_req_slots;
    uint32_t num_gqa_layers;
    uint32_t num_blocks;
    uint32_t num_page_ids_per_block;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    uint32_t tokens_per_page;
    uint32_t page_bytes;
    uint32_t pool_pages;
    uint32_t source_is_f16;
};

// KV_BYTES: bytes of a stored element (2: the source bits are copied; 1: FP8 E4M3FN).
template <int KV_BYTES>
__global__ void __launch_bounds__(256) kv_page_write_kernel(const PageWriteParams p) {
    const uint32_t vecs_per_row = p.head_dim / 8;  // 8 elements = 16 source bytes
    const uint32_t vecs_per_write = p.num_kv_heads * vecs_per_row;
    const uint64_t total = uint64_t(p.num_active_token_writes) * vecs_per_write;
    for (uint64_t gid = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; gid < total;
         gid += uint64_t(gridDim.x) * blockDim.x) {
        const uint32_t write = uint32_t(gid / vecs_per_write);
        const uint32_t rest = uint32_t(gid % vecs_per_write);
        const uint32_t head = rest / vecs_per_row;
        const uint32_t d = (rest % vecs_per_row) * 8;
        const uint32_t slot = p.req_slots[write];
        const uint32_t token = p.flat_token_indices[write];
        const uint32_t block = token / (p.tokens_per_page * p.num_page_ids_per_block);
        const uint32_t id_in_block = (token / p.tokens_per_page) % p.num_page_ids_per_block;
        if (slot >= p.num_req_slots || block >= p.num_blocks) {  // metadata that points past the page table
            atomicOr(p.status, 4u);
            continue;
        }
        const uint64_t entry =
            ((uint64_t(slot) * p.num_gqa_layers + p.layer_index) * p.num_blocks + block) * p.num_page_ids_per_block +
            id_in_block;
        const uint32_t page = p.page_ids[entry];
        if (page >= p.pool_pages) {  // never write outside the pool; report through the device status word
            atomicOr(p.status, 2u);
            continue;
        }
        const uint64_t plane_elems = uint64_t(p.num_kv_heads) * p.tokens_per_page * p.head_dim;
        const uint64_t elem = (uint64_t(head) * p.tokens_per_page + token % p.tokens_per_page) * p.head_dim + d;
        const uint64_t flat = (uint64_t(write) * p.num_kv_heads + head) * p.head_dim + d;
        const uint4 k = *reinterpret_cast<const uint4*>(p.flat_k + flat);
        const uint4 v = *reinterpret_cast<const uint4*>(p.flat_v + flat);
        uint8_t* page_base = p.pages + uint64_t(page) * p.page_bytes;
        if constexpr (KV_BYTES == 2) {
            *reinterpret_cast<uint4*>(page_base + elem * 2) = k;
            *reinterpret_cast<uint4*>(page_base + (plane_elems + elem) * 2) = v;
        } else {
            const uint32_t kw[4] = {k.x, k.y, k.z, k.w};
            const uint32_t vw[4] = {v.x, v.y, v.z, v.w};
            uint32_t ko[2] = {0, 0}, vo[2] = {0, 0};
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint16_t kb = uint16_t(kw[i / 2] >> (16 * (i & 1)));
                const uint16_t vb = uint16_t(vw[i / 2] >> (16 * (i & 1)));
                const float kf = p.source_is_f16 ? __half2float(__ushort_as_half(kb)) : f32_from_bf16_bits(kb);
                const float vf = p.source_is_f16 ? __half2float(__ushort_as_half(vb)) : f32_from_bf16_bits(vb);
                ko[i / 4] |= uint32_t(fp8_e4m3_from_f32(kf)) << (8 * (i & 3));
                vo[i / 4] |= uint32_t(fp8_e4m3_from_f32(vf)) << (8 * (i & 3));
            }
            *reinterpret_cast<uint2*>(page_base + elem) = make_uint2(ko[0], ko[1]);
            *reinterpret_cast<uint2*>(page_base + plane_elems + elem) = make_uint2(vo[0], vo[1]);
        }
    }
}

// Element-wise form for head dimensions that are not a multiple of 8 (the reference's own thread mapping,
// gqa_kv_page_write.metal:46-79: one thread per (write, KV head, element)).
template <int KV_BYTES>
__global__ void __launch_bounds__(256) kv_page_write_scalar_kernel(const PageWriteParams p) {
    const uint32_t per_write = p.num_kv_heads * p.head_dim;
    const uint64_t total = uint64_t(p.num_active_token_writes) * per_write;
    for (uint64_t gid = uint64_t(blockIdx.x) * blockDim.x + threadIdx.x; gid < total;
         gid += uint64_t(gridDim.x) * blockDim.x) {
        const uint32_t write = uint32_t(gid / per_write);
        const uint32_t rest = uint32_t(gid % per_write);
        const uint32_t head = rest / p.head_dim;
        const uint32_t d = rest % p.head_dim;
        const uint32_t slot = p.req_slots[write];
        const uint32_t token = p.flat_token_indices[write];
        const uint32_t block = token / (p.tokens_per_page * p.num_page_ids_per_block);
        const uint32_t id_in_block = (token / p.tokens_per_page) % p.num_page_ids_per_block;
        if (slot >= p.num_req_slots || block >= p.num_blocks) {  // metadata that points past the page table
            atomicOr(p.status, 4u);
            continue;
        }
        const uint64_t entry =
            ((uint64_t(slot) * p.num_gqa_layers + p.layer_index) * p.num_blocks + block) * p.num_page_ids_per_block +
            id_in_block;
        const uint32_t page = p.page_ids[entry];
        if (page >= p.pool_pages) {
            atomicOr(p.status, 2u);
            continue;
        }
        const uint64_t plane_elems = uint64_t(p.num_kv_heads) * p.tokens_per_page * p.head_dim;
        const uint64_t elem = (uint64_t(head) * p.tokens_per_page + token % p.tokens_per_page) * p.head_dim + d;
        const uint64_t flat = (uint64_t(write) * p.num_kv_heads + head) * p.head_dim + d;
        const uint16_t kb = p.flat_k[flat];
        const uint16_t vb = p.flat_v[flat];
        uint8_t* page_base = p.pages + uint64_t(page) * p.page_bytes;
        if constexpr (KV_BYTES == 2) {
            reinterpret_cast<uint16_t*>(page_base)[elem] = kb;
            reinterpret_cast<uint16_t*>(page_base)[plane_elems + elem] = vb;
        } else {
            const float kf = p.source_is_f16 ? __half2float(__ushort_as_half(kb)) : f32_from_bf16_bits(kb);
            const float vf = p.source_is_f16 ? __half2float(__ushort_as_half(vb)) : f32_from_bf16_bits(vb);
            page_base[elem] = fp8_e4m3_from_f32(kf);
            page_base[plane_elems + elem] = fp8_e4m3_from_f32(vf);
        }
    }
}

}  // namespace kh

using namespace kh;

struct kh_kv_page_write {
    kh_device* device;
    kh_kv_page_write_config config;
    uint32_t tokens_per_page;
};

// Config::validate + num_tokens_per_page (kv_page_write.rs:69-92), with the stored element size a parameter.
static uint32_t page_write_tokens_per_page(const kh_kv_page_write_config& c) {
    KH_REQUIRE(c.num_kv_heads > 0 && c.head_dim > 0, "GQA KV page write needs KV heads and a head dimension");
    KH_REQUIRE(c.dtype == KH_DTYPE_BFLOAT16 || c.dtype == KH_DTYPE_FLOAT16,
               "GQA KV page write requires BF16 (or FP16) source tensors");
    KH_REQUIRE(c.kv_dtype == KH_DTYPE_FP8_E4M3FN || c.kv_dtype == c.dtype,
               "GQA KV pages hold FP8 E4M3FN or the source element type");
    const uint64_t per_token = uint64_t(c.num_kv_heads) * c.head_dim * 2 * dtype_size(c.kv_dtype);
    KH_REQUIRE(per_token <= 0xffffffffull, "GQA K/V bytes per token must fit u32");
    KH_REQUIRE(c.page_bytes % per_token == 0, "GQA page_bytes must be divisible by the K/V bytes per token");
    KH_REQUIRE(c.page_bytes / per_token > 0, "GQA pages must hold at least one token");
    return uint32_t(c.page_bytes / per_token);
}

extern "C" {

kh_status kh_kv_page_write_create(kh_device* device, const kh_kv_page_write_config* config, kh_kv_page_write** out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(device && config && out, "null argument");
        auto compute = std::make_unique<kh_kv_page_write>();
        compute->device = device;
        compute->config = *config;
        compute->tokens_per_page = page_write_tokens_per_page(*config);
        *out = compute.release();
        return KH_OK;
    });
}

kh_status kh_kv_page_write_destroy(kh_kv_page_write* compute) {
    delete compute;
    return KH_OK;
}

kh_status kh_kv_page_write_tokens_per_page(const kh_kv_page_write_config* config, uint32_t* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(config && out, "null argument");
        *out = page_write_tokens_per_page(*config);
        return KH_OK;
    });
}

kh_status kh_kv_page_write_invoke(kh_kv_page_write* compute, kh_stream* stream, const kh_kv_page_write_shape* shape,
                                  const kh_kv_page_write_buffers* buffers, uint32_t num_active_token_writes,
                                  uint32_t page_table_index) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(compute && stream && shape && buffers, "null argument");
        KH_REQUIRE(stream->device == compute->device, "stream does not belong to the compute's device");
        const kh_kv_page_write_config& c = compute->config;
        const kh_page_table_layout& l = shape->page_table_layout;
        // Shape::validate, Invocation::validate (kv_page_write.rs:129-135, 239-256)
        KH_REQUIRE(shape->num_total_token_writes > 0, "GQA KV page write needs token writes");
        KH_REQUIRE(l.num_req_slots > 0 && l.num_blocks > 0 && l.num_gqa_layers > 0 && l.num_page_ids_per_block > 0,
                   "GQA page-table layout dimensions must be positive");
        const uint64_t values = mul_u64(mul_u64(shape->num_total_token_writes, c.num_kv_heads, "GQA KV page-write threads"),
                                        c.head_dim, "GQA KV page-write threads");
        KH_REQUIRE(values <= 0xffffffffull, "GQA KV page-write threads exceeds the shader u32 count domain: count=%llu",
                   (unsigned long long)values);
        KH_REQUIRE(num_active_token_writes >= 1 && num_active_token_writes <= shape->num_total_token_writes,
                   "num_active_token_writes %u outside [1, %u]", num_active_token_writes, shape->num_total_token_writes);
        KH_REQUIRE(page_table_index < l.num_gqa_layers, "page_table_index %u out of range", page_table_index);
        need(buffers->flat_k, values * dtype_size(c.dtype), "flat_k");
        need(buffers->flat_v, values * dtype_size(c.dtype), "flat_v");
        need(buffers->req_slots, uint64_t(shape->num_total_token_writes) * 4, "req_slots");
        need(buffers->flat_token_indices, uint64_t(shape->num_total_token_writes) * 4, "flat_token_indices");
        const uint64_t entries = mul_u64(mul_u64(mul_u64(l.num_req_slots, l.num_gqa_layers, "GQA page-table byte length"),
                                                 l.num_blocks, "GQA page-table byte length"),
                                         l.num_page_ids_per_block, "GQA page-table byte length");
        need(buffers->page_ids, entries * 4, "page_ids");
        need(buffers->pages, c.page_bytes, "pages");
        // 16 source bytes per thread when rows and bases allow it, else one element per thread
        const bool vector = c.head_dim % 8 == 0 && c.page_bytes % 16 == 0 &&
                            (reinterpret_cast<uintptr_t>(buffers->pages.ptr) & 15) == 0 &&
                            (reinterpret_cast<uintptr_t>(buffers->flat_k.ptr) & 15) == 0 &&
                            (reinterpret_cast<uintptr_t>(buffers->flat_v.ptr) & 15) == 0;
        use_device(compute->device);
        PageWriteParams p{};
        p.pages = static_cast<uint8_t*>(buffers->pages.ptr);
        p.flat_k = static_cast<const uint16_t*>(buffers->flat_k.ptr);
        p.flat_v = static_cast<const uint16_t*>(buffers->flat_v.ptr);
        p.req_slots = static_cast<const uint32_t*>(buffers->req_slots.ptr);
        p.flat_token_indices = static_cast<const uint32_t*>(buffers->flat_token_indices.ptr);
        p.page_ids = static_cast<const uint32_t*>(buffers->page_ids.ptr);
        p.status = compute->device->status;
        p.num_active_token_writes = num_active_token_writes;
        p.layer_index = page_table_index;
        p.num_req_slots = l.num_req_slots;
        p.num_gqa_layers = l.num_gqa_layers;
        p.num_blocks = l.num_blocks;
        p.num_page_ids_per_block = l.num_page_ids_per_block;
        p.num_kv_heads = c.num_kv_heads;
        p.head_dim = c.head_dim;
        p.tokens_per_page = compute->tokens_per_page;
        p.page_bytes = c.page_bytes;
        p.pool_pages = uint32_t(std::min<uint64_t>(buffers->pages.bytes / c.page_bytes, 0xffffffffull));
        p.source_is_f16 = c.dtype == KH_DTYPE_FLOAT16 ? 1u : 0u;
        const uint64_t threads =
            uint64_t(num_active_token_writes) * c.num_kv_heads * (vector ? c.head_dim / 8 : c.head_dim);
        const uint32_t blocks = uint32_t(std::min<uint64_t>((threads + 255) / 256, uint64_t(compute->device->sm_count) * 8));
        const bool fp8 = dtype_size(c.kv_dtype) == 1;
        if (vector && fp8) kv_page_write_kernel<1><<<blocks, 256, 0, stream->stream>>>(p);
        else if (vector) kv_page_write_kernel<2><<<blocks, 256, 0, stream->stream>>>(p);
        else if (fp8) kv_page_write_scalar_kernel<1><<<blocks, 256, 0, stream->stream>>>(p);
        else kv_page_write_scalar_kernel<2><<<blocks, 256, 0, stream->stream>>>(p);
        KH_CUDA(cudaGetLastError());
        return KH_OK;
    });
}

// Host-side codec (fp8.rs:19-58), for callers that prepare or inspect FP8 pages on the CPU.
uint8_t kh_fp8_e4m3_from_bf16(uint16_t bf16_bits) { return fp8_e4m3_from_f32(f32_from_bf16_bits(bf16_bits)); }
uint16_t kh_fp8_e4m3_to_bf16(uint8_t fp8_bits) { return bf16_bits_from_fp8_e4m3(fp8_bits); }

}  // extern "C"
