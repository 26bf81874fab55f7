// Cross-GPU LSE combine of one long sequence's per-GPU partial states in ONE kernel over NVLink peer memory:
// local merge of this GPU's split-KV partials, the merged (max, sum, output) row stored straight into every peer's
// inbox (plain peer stores through NVSwitch), a flag per (source rank, row), a bounded wait for the other ranks'
// flags, and the final merge from the local inbox. It replaces local merge kernel + all-gather + merge kernel
// (four dependent launches around a 16.5 KB collective) by one launch; the reference has no multi-device path, the
// merge is its reducer's (docs/gqa_sdpa_selection.md:443-460).
//
// One CTA per output row (Q head): rows are independent, so no CTA waits for another CTA of its own GPU. Every wait
// on a peer is bounded (kh_device_set_wait_limit polls); when it runs out the CTA sets the wait-expired bit of the
// device status word and returns without writing its output row. No multimem, no TMA: plain loads and stores.
//
// Inbox of a rank (device memory the peers map through CUDA IPC):
//   records  f32 [2 parities][world][rows][head_dim + 4]   (output row, then exp sum, max logit, 0, 0)
//   flags    u32 [2 parities][world][rows]                  (step number the record belongs to)
//   steps    u32 [rows]                                     (steps this rank has run; local use only)
// Step s uses parity s & 1. A peer can be at most one step ahead (its step s + 1 needs this rank's flag of step s
// ... s + 1), so two parities are enough and nothing is ever cleared.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstring>
#include <memory>

#include "common.h"
#include "cuda_objects.h"
#include "sdpa_map.cuh"

namespace kh {

constexpr int kPeerMaxWorld = 16;
constexpr uint32_t kPeerThreads = 512;

struct PeerExchangeParams {
    const float* partial_sum;   // local partials [num_partials][rows]
    const float* partial_max;
    const float* partial_out;   // [num_partials][rows][D]
    float* inbox[kPeerMaxWorld];     // records base of every rank (index = rank); own entry is local memory
    uint32_t* flags[kPeerMaxWorld];  // flags base of every rank
    uint32_t* steps;            // local [rows]
    void* out;                  // [rows][D] in the output dtype
    uint32_t* status;
    uint32_t num_partials, rows, head_dim, rank, world, wait_limit;
};

template <typename T>
__device__ __forceinline__ void store_row4(T* dst, float4 v);
template <>
__device__ __forceinline__ void store_row4<float>(float* dst, float4 v) { *reinterpret_cast<float4*>(dst) = v; }
template <>
__device__ __forceinline__ void store_row4<__nv_bfloat16>(__nv_bfloat16* dst, float4 v) { store_out4<__nv_bfloat16>(dst, v); }
template <>
__device__ __forceinline__ void store_row4<__half>(__half* dst, float4 v) { store_out4<__half>(dst, v); }

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float4 ld_volatile4(const float* p) {
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

template <typename T>
__global__ void __launch_bounds__(kPeerThreads) peer_exchange_kernel(const PeerExchangeParams p) {
    __shared__ float4 shared_acc[kPeerThreads];
    __shared__ float2 shared_stat[kPeerThreads];
    __shared__ uint32_t shared_ok;
    const uint32_t row = blockIdx.x;
    const uint32_t D = p.head_dim;
    const uint32_t slots = D / 4;                      // float4 columns of the row (<= 128)
    const uint32_t record = D + 4;                     // floats of one row record
    const uint32_t step = p.steps[row] + 1;            // every thread reads the same word; thread 0 writes it at the end
    const uint32_t parity = step & 1;
    // ---- 1. local merge of this GPU's partials for the row: the partial list is divided among thread groups
    const uint32_t subsets = kPeerThreads / slots;
    const uint32_t slot = threadIdx.x % slots, subset = threadIdx.x / slots;
    const uint32_t d = slot * 4;
    MergeState state = merge_state_empty();
    if (subset < subsets && p.num_partials > 0) {
        const uint32_t share = (p.num_partials + subsets - 1) / subsets;
        const uint32_t begin = min(subset * share, p.num_partials);
        const uint32_t mine = min(share, p.num_partials - begin);
        const uint64_t stride = p.rows;
        merge_partials_accumulate(state, p.partial_sum + uint64_t(begin) * stride, p.partial_max + uint64_t(begin) * stride,
                                  p.partial_out + uint64_t(begin) * stride * D, row, stride, stride * D, mine, D, d);
    }
    shared_acc[threadIdx.x] = state.acc;
    shared_stat[threadIdx.x] = make_float2(state.sum, state.max);
    if (threadIdx.x == 0) shared_ok = 1;
    __syncthreads();
    if (subset == 0) {
        for (uint32_t other = 1; other < subsets; ++other) {
            const uint32_t source = other * slots + slot;
            const float2 stat = shared_stat[source];
            merge_state_combine(state, MergeState{shared_acc[source], stat.x, stat.y});
        }
        float merged_sum, merged_max;
        const float4 local = merge_state_finish(state, &merged_sum, &merged_max);
        // ---- 2. the row record into every rank's inbox (own included): output columns, then the statistics
        const uint64_t at = ((uint64_t(parity) * p.world + p.rank) * p.rows + row) * record;
        for (uint32_t r = 0; r < p.world; ++r) {
            float* dst = p.inbox[r] + at;
            *reinterpret_cast<float4*>(dst + d) = local;
            if (slot == 0) *reinterpret_cast<float4*>(dst + D) = make_float4(merged_sum, merged_max, 0.0f, 0.0f);
        }
        __threadfence_system();  // the record is visible system-wide before the flag that announces it
    }
    __syncthreads();
    // ---- 3. announce: one flag per (source rank, row) in every rank's inbox
    const uint64_t flag_at = (uint64_t(parity) * p.world) * p.rows;
    if (threadIdx.x < p.world) st_release_sys(p.flags[threadIdx.x] + flag_at + uint64_t(p.rank) * p.rows + row, step);
    // ---- 4. wait (bounded) for the other ranks' records of this step
    if (threadIdx.x < p.world) {
        const uint32_t* flag = p.flags[p.rank] + flag_at + uint64_t(threadIdx.x) * p.rows + row;
        bool arrived = false;
        for (uint32_t i = 0; i < p.wait_limit; ++i) {
            if (int32_t(ld_acquire_sys(flag) - step) >= 0) {
                arrived = true;
                break;
            }
        }
        if (!arrived) {
            shared_ok = 0;
            atomicOr(p.status, kStatusWaitExpired);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) p.steps[row] = step;
    if (!shared_ok || subset != 0) return;
    // ---- 5. merge the ranks' records of the row from the local inbox
    const float* base = p.inbox[p.rank] + (uint64_t(parity) * p.world * p.rows + row) * record;
    MergeState all = merge_state_empty();
    for (uint32_t r = 0; r < p.world; ++r) {
        const float* rec = base + uint64_t(r) * p.rows * record;
        const float4 stat = ld_volatile4(rec + D);
        if (stat.x != 0.0f && isfinite(stat.y)) {
            const float4 v = ld_volatile4(rec + d);
            // a record holds a normalised output: its numerator relative to its own maximum is sum * output
            MergeState one{make_float4(v.x * stat.x, v.y * stat.x, v.z * stat.x, v.w * stat.x), stat.x, stat.y};
            merge_state_combine(all, one);
        }
    }
    const float4 result = merge_state_finish(all, nullptr, nullptr);
    store_row4<T>(reinterpret_cast<T*>(p.out) + uint64_t(row) * D + d, result);
}

}  // namespace kh

using namespace kh;

struct kh_peer_exchange {
    kh_device* device;
    uint32_t rank, world, rows, head_dim;
    float* inbox[kPeerMaxWorld];
    uint32_t* flags[kPeerMaxWorld];
    uint32_t* steps;
};

static uint64_t peer_record_floats(uint32_t world, uint32_t rows, uint32_t head_dim) {
    return 2ull * world * rows * (uint64_t(head_dim) + 4);
}

static uint64_t peer_flag_words(uint32_t world, uint32_t rows) { return 2ull * world * rows; }

extern "C" {

kh_status kh_peer_exchange_inbox_bytes(uint32_t world, uint32_t num_rows, uint32_t head_dim, uint64_t* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(out != nullptr, "null argument");
        KH_REQUIRE(world >= 1 && world <= uint32_t(kPeerMaxWorld), "peer exchange supports 1 to %d ranks", kPeerMaxWorld);
        KH_REQUIRE(num_rows > 0 && head_dim > 0 && head_dim % 4 == 0 && head_dim <= 512,
                   "peer exchange needs rows and a head_dim that is a multiple of 4, at most 512");
        *out = peer_record_floats(world, num_rows, head_dim) * 4 + (peer_flag_words(world, num_rows) + num_rows) * 4;
        return KH_OK;
    });
}

kh_status kh_ipc_export(kh_device* device, kh_buffer_ref buffer, uint8_t* handle64) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(handle64 != nullptr && buffer.ptr != nullptr, "null argument");
        use_device(device);
        static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handles are 64 bytes");
        cudaIpcMemHandle_t handle;
        KH_CUDA(cudaIpcGetMemHandle(&handle, buffer.ptr));
        memcpy(handle64, &handle, 64);
        return KH_OK;
    });
}

kh_status kh_ipc_import(kh_device* device, const uint8_t* handle64, void** out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(handle64 != nullptr && out != nullptr, "null argument");
        use_device(device);
        cudaIpcMemHandle_t handle;
        memcpy(&handle, handle64, 64);
        KH_CUDA(cudaIpcOpenMemHandle(out, handle, cudaIpcMemLazyEnablePeerAccess));
        return KH_OK;
    });
}

kh_status kh_ipc_close(kh_device* device, void* ptr) {
    return guarded([&]() -> kh_status {
        use_device(device);
        if (ptr != nullptr) KH_CUDA(cudaIpcCloseMemHandle(ptr));
        return KH_OK;
    });
}

kh_status kh_peer_exchange_create(kh_device* device, uint32_t rank, uint32_t world, uint32_t num_rows, uint32_t head_dim,
                                  void* const* inboxes, kh_peer_exchange** out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(device && inboxes && out, "null argument");
        uint64_t bytes = 0;
        const kh_status sized = kh_peer_exchange_inbox_bytes(world, num_rows, head_dim, &bytes);
        if (sized != KH_OK) return sized;
        KH_REQUIRE(rank < world, "rank %u outside a world of %u", rank, world);
        auto exchange = std::make_unique<kh_peer_exchange>();
        exchange->device = device;
        exchange->rank = rank;
        exchange->world = world;
        exchange->rows = num_rows;
        exchange->head_dim = head_dim;
        for (uint32_t r = 0; r < world; ++r) {
            KH_REQUIRE(inboxes[r] != nullptr && (reinterpret_cast<uintptr_t>(inboxes[r]) & 15) == 0,
                       "inbox of rank %u is null or not 16-byte aligned", r);
            exchange->inbox[r] = static_cast<float*>(inboxes[r]);
            exchange->flags[r] = reinterpret_cast<uint32_t*>(exchange->inbox[r] + peer_record_floats(world, num_rows, head_dim));
        }
        exchange->steps = exchange->flags[rank] + peer_flag_words(world, num_rows);
        *out = exchange.release();
        return KH_OK;
    });
}

kh_status kh_peer_exchange_destroy(kh_peer_exchange* exchange) {
    delete exchange;
    return KH_OK;
}

kh_status kh_peer_exchange_combine(kh_peer_exchange* exchange, kh_stream* stream, uint32_t num_partials,
                                   kh_buffer_ref exp_sums, kh_buffer_ref max_logits, kh_buffer_ref partial_output,
                                   kh_dtype out_dtype, kh_buffer_ref output) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(exchange && stream, "null argument");
        KH_REQUIRE(stream->device == exchange->device, "stream does not belong to the exchange's device");
        KH_REQUIRE(dtype_size(out_dtype) >= 2, "unsupported output dtype");
        const uint64_t stats = uint64_t(num_partials) * exchange->rows;
        if (num_partials > 0) {
            need(exp_sums, stats * 4, "exp_sums");
            need(max_logits, stats * 4, "max_logits");
            need(partial_output, stats * exchange->head_dim * 4, "partial_output");
        }
        need(output, uint64_t(exchange->rows) * exchange->head_dim * dtype_size(out_dtype), "output");
        use_device(exchange->device);
        PeerExchangeParams p{};
        p.partial_sum = static_cast<const float*>(exp_sums.ptr);
        p.partial_max = static_cast<const float*>(max_logits.ptr);
        p.partial_out = static_cast<const float*>(partial_output.ptr);
        for (uint32_t r = 0; r < exchange->world; ++r) {
            p.inbox[r] = exchange->inbox[r];
            p.flags[r] = exchange->flags[r];
        }
        p.steps = exchange->steps;
        p.out = output.ptr;
        p.status = exchange->device->status;
        p.num_partials = num_partials;
        p.rows = exchange->rows;
        p.head_dim = exchange->head_dim;
        p.rank = exchange->rank;
        p.world = exchange->world;
        p.wait_limit = exchange->device->wait_limit;
        const dim3 grid(exchange->rows);
        if (out_dtype == KH_DTYPE_BFLOAT16) peer_exchange_kernel<__nv_bfloat16><<<grid, kPeerThreads, 0, stream->stream>>>(p);
        else if (out_dtype == KH_DTYPE_FLOAT16) peer_exchange_kernel<__half><<<grid, kPeerThreads, 0, stream->stream>>>(p);
        else if (out_dtype == KH_DTYPE_FLOAT32) peer_exchange_kernel<float><<<grid, kPeerThreads, 0, stream->stream>>>(p);
        else raise(KH_INVALID_ARGUMENT, "unsupported output dtype");
        KH_CUDA(cudaGetLastError());
        return KH_OK;
    });
}

}  // extern "C"
