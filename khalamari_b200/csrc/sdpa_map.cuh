// Paged GQA split-KV attention "map" kernel for sm_100a.
//
// One persistent CTA per SM walks a strided list of Map tasks. A task is one map task template
// {q_token_range_index, kv_token_begin, kv_token_end} x one KV head x one Q-head range -- the
// grid cell of the reference's gqa_sdpa_sliced_kv_map / gqa_sdpa_sliced_q_map kernels
// (crates/inference-backend-metal/src/components/metal/gqa_sdpa_sliced_kv_map.metal:36,
//  crates/inference-backend-metal/src/components/metal/gqa_sdpa_sliced_q_map.metal:29).
//
// Data movement (producer warp). All global reads of the kernel are issued by one producer warp:
//  - it decodes 32 upcoming tasks at a time, one per lane (template -> Q range -> request slot is a
//    chain of dependent loads, paid once per 32 tasks),
//  - stages each task's page ids into shared memory one task ahead (cp.async),
//  - publishes the task descriptor and the task's Q rows (TMA tile copy, 128-byte swizzle) into a
//    small task ring, and
//  - streams the task's K and V page chunks from the paged pool into a ring of shared-memory stages
//    with TMA tile copies (128-byte swizzle, one mbarrier per stage, every copy private to its CTA). A page chunk
//    [tokens_per_page][head_dim] of one KV head is contiguous in the page layout [K/V][Hkv][P][D]; the
//    K chunk and the V chunk of one (page, KV head) travel in ONE four-dimensional TMA copy
//    {64 columns, page rows, column halves, K/V plane} (8 KiB at head_dim 128, 16 KiB at 256): the copy
//    engine's cost is per instruction, so few large copies are what reaches HBM bandwidth.
// Math (consumer warps). The Q rows of a task -- (Q tokens of the range) x (Q heads of the KV group)
// -- are the M dimension of warp-level tensor-core tiles, so every K/V byte is read from HBM once
// and feeds all of them. S = Q K^T and O += P V run as m16n8k16 MMAs with f32 accumulators; the
// online softmax keeps a running row maximum with quad shuffles. KV stages are dealt round robin to
// KVW "KV warps" per 16-row tile; at the end of the task every warp writes its (m, l, O) state to
// shared memory and all consumer threads merge and publish a slice each: either an f32 partial
// (max, exp-sum, normalised output) or the final output.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <type_traits>

namespace kh {

struct MapParams {
    const uint32_t* req_slots;        // [T]
    const uint32_t* page_ids;         // [slots][L][B][n]
    const uint32_t* visible;          // [T][2] request-local [begin, end) per flat Q token; null: template range
    const uint32_t* q_ranges;         // [Q][2] flat token [begin, end); null: range i is the single token i
    const uint32_t* templates;        // [Mt][3]
    float* partial_out;               // [Mt][Hq][max_q_tokens][D]
    float* partial_sum;               // [Mt][Hq][max_q_tokens]
    float* partial_max;               // [Mt][Hq][max_q_tokens]
    void* out;                        // direct output [T][Hq][D] io dtype
    uint32_t* status;                 // sticky device status word
    uint32_t num_templates;           // templates to visit (already clamped to the active count)
    uint32_t num_active_tokens;
    uint32_t num_active_q_tiles;
    uint32_t layer_index;
    uint32_t num_q_heads;
    uint32_t num_kv_heads;
    uint32_t group;                   // Hq / Hkv
    uint32_t heads_per_task;          // variant.max_q_heads
    uint32_t head_ranges;             // ceil(group / heads_per_task)
    uint32_t max_q_tokens;            // variant.max_q_tokens
    uint32_t num_gqa_layers;
    uint32_t pages_per_request_layer; // num_blocks * num_page_ids_per_block
    uint32_t pool_pages;
    float scale_log2e;                // scale * log2(e)
    uint32_t direct;                  // 1: write final output, 0: write partials
    const uint32_t* cu;               // fused reduce: [ranges + 1] first partial (= template) of every Q range; null: off
    uint32_t* arrivals;               // fused reduce: one zeroed counter per (Q range, KV head, head range)
    // Replay: when set, the active counts {tokens, Q-token tiles, map task templates} are read from this device
    // word triple when the kernel runs (a captured launch replays with new counts); num_active_tokens,
    // num_active_q_tiles and num_templates are then the recorded capacities and only bound the values read.
    const uint32_t* active;
    uint32_t num_req_slots;           // request slots of the page table (bounds the slots the metadata names)
    uint32_t tokens_per_page;
    uint32_t wait_limit;              // polls a bounded wait makes before it gives up (kDefaultWaitLimit)
    // Measurement aid. Only a library compiled with KH_GQA_MEASURE reads these bits (debug_bits() below); the
    // product build compiles every test of them away. Outputs are meaningless when set. Bits: 1 consumers release
    // every stage without computing; 2 skip the task-end merge and publish; 4 skip the Q copies; 8 issue no K/V
    // copies (consumers run on stale shared memory); 16 / 32 / 64 skip QK / softmax / PV; 128 never run the
    // in-kernel group merge; 256 do not count arrivals; 512 visit tasks template-major and never carry the running
    // state from one task to the next (outputs stay valid); 1024 tensor-memory kernel: skip the remainder MMAs;
    // 4096 FP8 pages: the decode warps hand stages on without converting them.
    uint32_t debug;
};

constexpr uint32_t kStatusWaitExpired = 1u;
constexpr uint32_t kStatusPageOutOfPool = 2u;
constexpr uint32_t kStatusMetadataOutOfRange = 4u;  // a request slot or KV range beyond the page table
constexpr uint32_t kDefaultWaitLimit = 1u << 24;

#ifdef KH_GQA_MEASURE
__device__ __forceinline__ uint32_t debug_bits(const MapParams& p) { return p.debug; }
#else
__device__ __forceinline__ constexpr uint32_t debug_bits(const MapParams&) { return 0u; }
#endif
constexpr int kMaxPidsPerSegment = 160;  // page ids staged per task segment (2048 tokens of 16 + slack)
constexpr uint32_t kBalanceMaxTemplates = 16384;  // above this, tasks are dealt round-robin (many tasks per CTA anyway)
constexpr uint32_t kTaskOverheadTokens = 48;      // fixed cost of a task, in KV tokens of streaming time
constexpr int kMaxTaskTokens = 32;       // Q tokens per task (the reference caps the tile at 32, sdpa.rs:117)

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// The barrier counts one arrival once all cp.async copies this thread issued so far have landed.
__device__ __forceinline__ void mbar_arrive_after_cp_async(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait. Once any wait of the CTA has run out, `abort_flag` (shared) is set, every later
// wait returns at once and the kernel runs to its end without touching the rings again; the host
// reads the sticky status word.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          const MapParams& p) {
    if (mbar_try_wait(bar, parity)) return true;  // common case: no shared-memory flag read on the way
    if (*abort_flag) return false;
    for (uint32_t i = 0; i < p.wait_limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    *abort_flag = 1;
    atomicOr(p.status, kStatusWaitExpired);
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int32_t x, int32_t y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// K/V pages are read once per launch and never again: the copy carries an evict-first L2 policy so that the
// stream does not push the partials, the block table and the batch metadata out of L2.
__device__ __forceinline__ uint64_t l2_evict_first_policy() {
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    return policy;
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int32_t c0, int32_t c1, int32_t c2,
                                            int32_t c3, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%2, %3, %4, %5}], [%6], %7;"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

template <typename T>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);

template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <>
__device__ __forceinline__ void mma_16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);

template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <typename T>
__device__ __forceinline__ float2 unpack2(uint32_t packed);

template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t packed) {
    return make_float2(__uint_as_float(packed << 16), __uint_as_float(packed & 0xffff0000u));
}

template <>
__device__ __forceinline__ float2 unpack2<__half>(uint32_t packed) {
    return __half22float2(*reinterpret_cast<__half2*>(&packed));
}

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int ID>
__device__ __forceinline__ void consumer_barrier(int threads) {
    asm volatile("bar.sync %0, %1;" ::"n"(ID), "r"(threads) : "memory");
}

template <typename T>
__device__ __forceinline__ void store_out4(T* dst, float4 v) {
    uint2 packed = make_uint2(pack2<T>(v.x, v.y), pack2<T>(v.z, v.w));
    *reinterpret_cast<uint2*>(dst) = packed;
}

// Partial-state merge of one output vector (four columns of one (token, head) row): the reducer's formula
// (docs/gqa_sdpa_selection.md:443-460 of the reference; gqa_sdpa_sliced_kv_reduce.metal:30-55):
// max = max_i m_i, weight_i = exp(m_i - max) * l_i (0 for an empty partial), out = sum_i weight_i o_i / sum_i weight_i.
// Partials are taken eight at a time with all their loads issued together (the merge runs while the memory system
// is saturated by K/V streaming, so dependent loads are what costs), carrying (max, sum, numerator) between groups.
// Partial j of the row sits `j * index_stride` statistics and `j * out_stride` output floats after the first.
// L2-only loads: the partials may have been written by other SMs during this launch.
struct MergeState {
    float4 acc;    // sum of weight_i * o_i, relative to `max`
    float sum;     // sum of weight_i
    float max;     // running maximum; -inf while nothing has been merged
};

__device__ __forceinline__ MergeState merge_state_empty() {
    return MergeState{make_float4(0.0f, 0.0f, 0.0f, 0.0f), 0.0f, -INFINITY};
}

// Folds `count` partials of one row into `state`.
__device__ __forceinline__ void merge_partials_accumulate(MergeState& state, const float* partial_sum,
                                                          const float* partial_max, const float* partial_out,
                                                          uint64_t first_index, uint64_t index_stride,
                                                          uint64_t out_stride, uint32_t count, uint32_t head_dim,
                                                          uint32_t d) {
    float run_max = state.max, run_sum = state.sum;
    float4 acc = state.acc;
    for (uint32_t base = 0; base < count; base += 8) {
        // statistics of eight partials first, then the output rows of those that carry weight (a task that handed
        // its running state on publishes an empty partial, so most rows of a long list are never read)
        float mx[8], sm[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const bool valid = base + j < count;
            const uint64_t index = first_index + uint64_t(base + j) * index_stride;
            mx[j] = valid ? __ldcg(partial_max + index) : -INFINITY;
            sm[j] = valid ? __ldcg(partial_sum + index) : 0.0f;
        }
        float new_max = run_max;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (sm[j] != 0.0f && isfinite(mx[j])) new_max = fmaxf(new_max, mx[j]);
        }
        float weight[8];
        float4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            weight[j] = (sm[j] != 0.0f && isfinite(mx[j])) ? expf(mx[j] - new_max) * sm[j] : 0.0f;
            const uint64_t out_index = first_index * head_dim + uint64_t(base + j) * out_stride + d;
            v[j] = weight[j] != 0.0f ? __ldcg(reinterpret_cast<const float4*>(partial_out + out_index))
                                     : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
        const float keep = run_max == -INFINITY ? 0.0f : expf(run_max - new_max);
        acc.x *= keep;
        acc.y *= keep;
        acc.z *= keep;
        acc.w *= keep;
        run_sum *= keep;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            acc.x += weight[j] * v[j].x;
            acc.y += weight[j] * v[j].y;
            acc.z += weight[j] * v[j].z;
            acc.w += weight[j] * v[j].w;
            run_sum += weight[j];
        }
        run_max = new_max;
    }
    state.acc = acc;
    state.sum = run_sum;
    state.max = run_max;
}

// Folds another state of the same row into `state` (both relative to their own maxima).
__device__ __forceinline__ void merge_state_combine(MergeState& state, const MergeState& other) {
    const float new_max = fmaxf(state.max, other.max);
    const float keep = state.max == -INFINITY ? 0.0f : expf(state.max - new_max);
    const float take = other.max == -INFINITY ? 0.0f : expf(other.max - new_max);
    state.acc.x = state.acc.x * keep + other.acc.x * take;
    state.acc.y = state.acc.y * keep + other.acc.y * take;
    state.acc.z = state.acc.z * keep + other.acc.z * take;
    state.acc.w = state.acc.w * keep + other.acc.w * take;
    state.sum = state.sum * keep + other.sum * take;
    state.max = new_max;
}

// Normalised output of a merged row; writes the merged statistics when asked.
__device__ __forceinline__ float4 merge_state_finish(const MergeState& state, float* out_sum, float* out_max) {
    const float inv = state.sum > 0.0f ? 1.0f / state.sum : 0.0f;
    if (out_sum != nullptr) {
        *out_sum = state.sum;
        *out_max = state.sum > 0.0f ? state.max : -INFINITY;
    }
    return make_float4(state.acc.x * inv, state.acc.y * inv, state.acc.z * inv, state.acc.w * inv);
}

__device__ __forceinline__ float4 merge_partials_vec(const float* partial_sum, const float* partial_max,
                                                     const float* partial_out, uint64_t first_index,
                                                     uint64_t index_stride, uint64_t out_stride, uint32_t count,
                                                     uint32_t head_dim, uint32_t d, float* out_sum, float* out_max) {
    MergeState state = merge_state_empty();
    merge_partials_accumulate(state, partial_sum, partial_max, partial_out, first_index, index_stride, out_stride,
                              count, head_dim, d);
    return merge_state_finish(state, out_sum, out_max);
}

// Merges the partials [part_begin, part_begin + part_count) of the rows (num_toks tokens x num_heads heads) of
// one task group and writes the final output. Called by every consumer thread of the CTA that completed the group.
template <typename T, int D>
__device__ __forceinline__ void reduce_group(const MapParams& p, uint32_t tok_begin, uint32_t num_toks,
                                             uint32_t head_begin, uint32_t num_heads, uint32_t part_begin,
                                             uint32_t part_count, uint32_t tid, uint32_t threads) {
    constexpr uint32_t kVecs = D / 4;
    const uint32_t rows = num_toks * num_heads;
    const uint64_t stride = uint64_t(p.num_q_heads) * p.max_q_tokens;
    for (uint32_t idx = tid; idx < rows * kVecs; idx += threads) {
        const uint32_t row = idx / kVecs;
        const uint32_t d = (idx % kVecs) * 4;
        const uint32_t tok = row / num_heads;
        const uint32_t head = head_begin + row % num_heads;
        const uint64_t first = (uint64_t(part_begin) * p.num_q_heads + head) * p.max_q_tokens + tok;
        const float4 acc = merge_partials_vec(p.partial_sum, p.partial_max, p.partial_out, first, stride, stride * D,
                                              part_count, D, d, nullptr, nullptr);
        T* dst = reinterpret_cast<T*>(p.out) + (uint64_t(tok_begin + tok) * p.num_q_heads + head) * D + d;
        store_out4<T>(dst, acc);
    }
}

// Task descriptor as the producer publishes it to the consumers (shared memory).
struct TaskSlot {
    uint32_t tmpl;
    uint32_t head_begin;   // first Q head of the task (absolute)
    uint32_t num_heads;    // active Q heads in the task
    uint32_t tok_begin;    // first flat Q token
    uint32_t num_toks;     // Q tokens in the range
    uint32_t kv_begin;
    uint32_t kv_end;
    uint32_t tile_begin;   // kv_begin rounded down to a stage boundary
    uint32_t num_tiles;
    uint32_t done;         // 1: no more tasks for this CTA
    uint32_t group;        // fused reduce: arrival counter of this task's (Q range, KV head, head range)
    uint32_t part_begin;   // fused reduce: first partial (template) of the Q range
    uint32_t part_count;   // fused reduce: partials of the Q range
    uint32_t carry;        // bit 0: continue from the previous task's running state; bit 1: hand the state on
    uint32_t kv_head;      // for the stream warp: KV head whose rows are streamed
    uint32_t req_slot;     // for the stream warp: request slot (page ids of later segments)
    uint32_t visible[2 * kMaxTaskTokens];  // per Q token [begin, end), only when MapParams::visible is set
};

// Compile-time geometry of one kernel instance.
//   D: head dimension (128 or 256). P: tokens per page. MT: 16-row tiles of Q rows per task.
//   KVW: KV warp groups per row tile (a stage goes to one group). PS: warps of a group that split one
//   stage's tokens between them. HALF: only rows 0-7 of the (single) row tile are ever valid.
//   Consumer warps = MT * KVW * PS; one extra warp produces.
// KVB: bytes of a stored K/V element. 2: the pages hold the Q/output element type and the consumers read the
// copied stages directly. 1: the pages hold FP8 E4M3FN (one unit scale); the copies land in a ring of raw
// stages and decode warps expand them into the 16-bit stage ring the consumers read.
template <int D, int P, int MT, int KVW, int PS, bool HALF, int KVB = 2>
struct MapGeometry {
    static_assert(KVB == 1 || KVB == 2, "K/V elements are stored in one or two bytes");
    // a stage holds whole pages: 32 tokens at head_dim 128, one page (16 tokens, or 32 with 32-token pages) at 256
    static constexpr int kStageTokens = (D == 128) ? 32 : (P > 16 ? P : 16);
    static constexpr int kBoxRows = (P < kStageTokens) ? P : kStageTokens;
    static constexpr int kBoxesPerPlane = kStageTokens / kBoxRows;  // token boxes per stage
    static constexpr int kColumnHalves = D / 64;                      // 128-byte column groups
    static constexpr int kBoxBytes = kBoxRows * 128;                  // one column half of one token box
    static constexpr int kPlaneBoxBytes = kColumnHalves * kBoxBytes;  // K (or V) rows of one token box
    static constexpr int kCopyBytes = 2 * kPlaneBoxBytes;             // one TMA copy: K and V of one token box
    static constexpr int kStageBytes = kBoxesPerPlane * kCopyBytes;
    static constexpr int kWarpTokens = kStageTokens / PS;            // KV tokens one warp handles per stage
    static constexpr int kMergeParts = KVW * PS;                     // (m, l, O) states merged per row tile
    static constexpr int kConsumerWarps = MT * KVW * PS;
    // FP8 pages: the decode work per stage is fixed while the tensor-core work grows with the row tiles, and
    // head_dim 256 consumers need the registers of a smaller block
    static constexpr int kDecodeWarps = (KVB == 2) ? 0 : ((MT >= 4 || D == 256) ? 2 : 4);
    static constexpr int kThreads = (kConsumerWarps + 2 + kDecodeWarps) * 32;  // + stream warp + task warp
    static constexpr int kTileRows = HALF ? 8 : 16;  // valid rows of a row tile
    static constexpr int kQRows = MT * kTileRows;  // Q rows of a task in shared memory (per 64-column half)
    static constexpr int kQBytes = kQRows * D * 2;
    static constexpr int kTaskSlots = 2;  // the producer publishes at most one task ahead of the consumers
    static constexpr int kFragRegs = HALF ? D / 4 : D / 2;        // O accumulator registers a warp parks
    static constexpr int kMergeSlotFloats = (kFragRegs + 4) * 32;  // O fragment + (m, l) x 2 rows, per lane
    static constexpr int kMergeBytes = (kMergeParts == 1) ? 0 : MT * KVW * kMergeSlotFloats * 4;  // one state: no merge
    static constexpr int kPidBytes = kTaskSlots * kMaxPidsPerSegment * 4;
    static constexpr int kTaskBytes = kTaskSlots * static_cast<int>(sizeof(TaskSlot));
    static constexpr int kFixedBytes =
        kTaskSlots * kQBytes + kMergeBytes + kPidBytes + kTaskBytes + (KVB == 1 ? 1024 : 512);
    static constexpr int kSmemLimit = 227 * 1024 - 1024 /* alignment slack */;
    static constexpr int kRawStageBytes = kStageBytes / 2;
    // FP8 pages: a short 16-bit ring (two slots per KV warp: one being read, one being decoded) and the rest
    // of shared memory for raw stages, which are what covers the HBM latency
    static constexpr bool kTwoSlotsPerWarp =
        KVW == 1 || (kSmemLimit - kFixedBytes - 2 * KVW * kStageBytes) / kRawStageBytes >= 12;
    static constexpr int kStagesFit =
        (KVB == 1) ? (kTwoSlotsPerWarp ? 2 * KVW : KVW) : (kSmemLimit - kFixedBytes) / kStageBytes;
    // A KV warp consumes the stages whose running number is congruent to its index modulo KVW. With the
    // ring depth a multiple of KVW every ring slot is always consumed by the same warp, so a warp can
    // never wait on a slot more than one phase ahead of the slot's barrier (phase parity cannot alias).
    static constexpr int kStagesCapped = kStagesFit > 24 ? 24 : kStagesFit;
    static constexpr int kStages = kStagesCapped / KVW * KVW;
    static constexpr int kRawStagesFit =
        (KVB == 1) ? (kSmemLimit - kFixedBytes - kStages * kStageBytes) / kRawStageBytes : 0;
    static constexpr int kRawStages = kRawStagesFit > 24 ? 24 : kRawStagesFit;
    static constexpr int kSmemBytes = kStages * kStageBytes + kRawStages * kRawStageBytes + kFixedBytes + 1024;
    static_assert(kStages >= 2 && kStages >= KVW, "shared memory ring too small");
    static_assert(KVB == 2 || kRawStages >= 3, "raw stage ring too small");
    // What the stream warp sees when the pages hold one-byte elements: the same token boxes at half the bytes
    // (a 128-byte line holds 128 elements, so head_dim 128 has one column group).
    struct Raw {
        static constexpr int kStageTokens = MapGeometry::kStageTokens;
        static constexpr int kBoxRows = MapGeometry::kBoxRows;
        static constexpr int kBoxesPerPlane = MapGeometry::kBoxesPerPlane;
        static constexpr int kColumnGroups = D / 128;
        static constexpr int kBoxBytes = kBoxRows * 128;
        static constexpr int kPlaneBoxBytes = kColumnGroups * kBoxBytes;
        static constexpr int kCopyBytes = 2 * kPlaneBoxBytes;
        static constexpr int kStageBytes = kBoxesPerPlane * kCopyBytes;
        static constexpr int kStages = MapGeometry::kRawStages;
        static constexpr int kTaskSlots = MapGeometry::kTaskSlots;
    };
    static_assert(Raw::kStageBytes == kRawStageBytes, "raw stage geometry");
    static_assert(D % 64 == 0 && (P == 8 || P == 16 || P == 32), "unsupported page geometry");
    static_assert((KVW & (KVW - 1)) == 0, "KV warps must be a power of two");
    static_assert((D / 8) % kMergeParts == 0, "output n-tiles must split evenly across the merging warps");
    static_assert(kWarpTokens % 16 == 0, "a warp handles whole 16-token MMA k-tiles");
    static_assert(PS == 1 || PS == 2, "a stage is split between at most two warps");
    static_assert(kStageTokens % P == 0, "a stage holds whole pages");
    static_assert(sizeof(TaskSlot) % 8 == 0, "task slots must keep the barriers 8-byte aligned");
};

// Counts a launch works with: its by-value arguments, or the device words a replayed launch reads them from.
struct ActiveCounts {
    uint32_t tokens, q_tiles, templates;
};

__device__ __forceinline__ ActiveCounts resolve_active(const MapParams& p) {
    ActiveCounts a{p.num_active_tokens, p.num_active_q_tiles, p.num_templates};
    if (p.active != nullptr) {
        a.tokens = min(p.active[0], a.tokens);
        a.q_tiles = min(p.active[1], a.q_tiles);
        a.templates = min(p.active[2], a.templates);
    }
    return a;
}

// Per-lane decoded task (producer registers).
struct TaskInfo {
    uint32_t tmpl, head_begin, num_heads, tok_begin, num_toks, kv_begin, kv_end, req_slot, kv_head, active;
    uint32_t group, part_begin, part_count;
};

// Decodes flat task index -> template, KV head, head range, and applies the reference kernels'
// early-return rules for padded and inactive templates (gqa_sdpa_sliced_kv_map.metal:56-58,
// gqa_sdpa_sliced_q_map.metal:56-67).
__device__ __forceinline__ TaskInfo decode_task(const MapParams& p, const ActiveCounts& a, uint64_t task,
                                                uint32_t total_tasks) {
    TaskInfo t;
    t.tmpl = t.head_begin = t.num_heads = t.tok_begin = t.num_toks = t.kv_begin = t.kv_end = t.req_slot = t.kv_head = 0;
    t.active = 0;
    t.group = t.part_begin = t.part_count = 0;
    if (task >= total_tasks) return t;
    const uint32_t cells = p.num_kv_heads * p.head_ranges;
    t.tmpl = uint32_t(task) / cells;
    const uint32_t cell = uint32_t(task) % cells;
    t.kv_head = cell / p.head_ranges;
    const uint32_t range = cell % p.head_ranges;
    t.head_begin = t.kv_head * p.group + range * p.heads_per_task;
    t.num_heads = min(p.heads_per_task, p.group - range * p.heads_per_task);
    const uint32_t q_range = p.templates[t.tmpl * 3];
    if (p.q_ranges == nullptr) {
        if (q_range >= a.tokens) return t;
        t.tok_begin = q_range;
        t.num_toks = 1;
    } else {
        if (q_range >= a.q_tiles) return t;
        const uint32_t begin = p.q_ranges[q_range * 2];
        const uint32_t end = p.q_ranges[q_range * 2 + 1];
        if (begin >= a.tokens || end > a.tokens || end <= begin) return t;
        t.tok_begin = begin;
        t.num_toks = min(min(end - begin, p.max_q_tokens), uint32_t(kMaxTaskTokens));
    }
    t.kv_begin = p.templates[t.tmpl * 3 + 1];
    t.kv_end = p.templates[t.tmpl * 3 + 2];
    t.req_slot = p.req_slots[t.tok_begin];
    // The slot and the KV range index the page table: metadata that points past it (a stale or padded entry) must
    // not become an address. The task is dropped and the status word says so; its partial keeps whatever it held.
    if (t.req_slot >= p.num_req_slots ||
        (t.kv_end > t.kv_begin &&
         (uint64_t(t.kv_end) + p.tokens_per_page - 1) / p.tokens_per_page > p.pages_per_request_layer)) {
        atomicOr(p.status, kStatusMetadataOutOfRange);
        return t;
    }
    if (p.cu != nullptr) {
        t.part_begin = p.cu[q_range];
        t.part_count = p.cu[q_range + 1] - t.part_begin;
        t.group = (q_range * p.num_kv_heads + t.kv_head) * p.head_ranges + range;
    }
    t.active = 1;
    return t;
}

__device__ __forceinline__ TaskInfo shfl_task(const TaskInfo& t, int lane) {
    TaskInfo r;
    r.tmpl = __shfl_sync(0xffffffffu, t.tmpl, lane);
    r.head_begin = __shfl_sync(0xffffffffu, t.head_begin, lane);
    r.num_heads = __shfl_sync(0xffffffffu, t.num_heads, lane);
    r.tok_begin = __shfl_sync(0xffffffffu, t.tok_begin, lane);
    r.num_toks = __shfl_sync(0xffffffffu, t.num_toks, lane);
    r.kv_begin = __shfl_sync(0xffffffffu, t.kv_begin, lane);
    r.kv_end = __shfl_sync(0xffffffffu, t.kv_end, lane);
    r.req_slot = __shfl_sync(0xffffffffu, t.req_slot, lane);
    r.kv_head = __shfl_sync(0xffffffffu, t.kv_head, lane);
    r.active = __shfl_sync(0xffffffffu, t.active, lane);
    r.group = __shfl_sync(0xffffffffu, t.group, lane);
    r.part_begin = __shfl_sync(0xffffffffu, t.part_begin, lane);
    r.part_count = __shfl_sync(0xffffffffu, t.part_count, lane);
    return r;
}

// Which tasks a CTA runs. Tasks are numbered template-major. With few enough templates the CTA's task warp scans
// them all (12 bytes each) and takes one CONTIGUOUS run of tasks whose cost - KV tokens plus a fixed per-task term -
// is its 1/gridDim share of the total: task k belongs to the CTA c with
// c * W / grid <= cost of tasks [0, k) < (c + 1) * W / grid. No CTA carries more than its share plus one task,
// where dealing tasks round-robin leaves the CTAs that drew the long slices several percent behind. Contiguous
// tasks are also neighbours in the page table. Above kBalanceMaxTemplates tasks are dealt round-robin.
// Called by the 32 lanes of the task warp only (a block-wide scan with two block barriers cost every launch about
// 5 us before the first copy could be issued); `scratch` is shared memory for one u32 per template that nothing
// else touches until the call returns (the K/V ring: no copy is issued before the first task is published);
// returns [begin, end) in every lane.
__device__ __forceinline__ void balanced_task_range_warp(const MapParams& p, uint32_t num_templates, int lane,
                                                         uint32_t* scratch, uint32_t& begin, uint32_t& end) {
    const uint32_t cells = p.num_kv_heads * p.head_ranges;
    const uint64_t total_tasks = uint64_t(num_templates) * cells;
    if (total_tasks <= gridDim.x) {
        // at most one task per CTA (a small batch: the launch is latency, not bandwidth): nothing to balance and no
        // reason to read the templates here
        begin = blockIdx.x;
        end = static_cast<uint32_t>(min(uint64_t(blockIdx.x) + 1, total_tasks));
        return;
    }
    // every template's cost into shared memory, read from global memory once, coalesced and with many loads in flight
    for (uint32_t t = lane; t < num_templates; t += 32) {
        const uint32_t q_range = p.templates[t * 3];
        const uint32_t kv_begin = p.templates[t * 3 + 1];
        const uint32_t kv_end = p.templates[t * 3 + 2];
        scratch[t] = (q_range == 0xffffffffu || kv_end <= kv_begin) ? 1u : kv_end - kv_begin + kTaskOverheadTokens;
    }
    __syncwarp();
    // lane l owns the contiguous chunk [first, last) of the templates
    const uint32_t chunk = (num_templates + 31) / 32;
    const uint32_t first = min(uint32_t(lane) * chunk, num_templates);
    const uint32_t last = min(first + chunk, num_templates);
    uint64_t local = 0;
    for (uint32_t t = first; t < last; ++t) local += scratch[t];
    uint64_t inclusive = local;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const uint64_t v = __shfl_up_sync(0xffffffffu, inclusive, d);
        if (lane >= d) inclusive += v;
    }
    const uint64_t total = __shfl_sync(0xffffffffu, inclusive, 31);
    const uint64_t whole = total * cells;
    const uint64_t lo = whole / gridDim.x * blockIdx.x + whole % gridDim.x * blockIdx.x / gridDim.x;
    const uint64_t hi = whole / gridDim.x * (blockIdx.x + 1) + whole % gridDim.x * (blockIdx.x + 1) / gridDim.x;
    // first task whose preceding cost reaches x: inside the template whose cost interval (S, E] holds x; one lane
    // at most finds each bound (none for a bound of 0: task 0)
    uint32_t found_begin = 0, found_end = 0;
    uint64_t start = (inclusive - local) * cells;
    for (uint32_t t = first; t < last; ++t) {
        const uint64_t c = scratch[t];
        const uint64_t stop = start + c * cells;
        if (lo > start && lo <= stop) found_begin = t * cells + uint32_t((lo - start + c - 1) / c);
        if (hi > start && hi <= stop) found_end = t * cells + uint32_t((hi - start + c - 1) / c);
        start = stop;
    }
#pragma unroll
    for (int d = 16; d >= 1; d >>= 1) {
        found_begin = max(found_begin, __shfl_xor_sync(0xffffffffu, found_begin, d));
        found_end = max(found_end, __shfl_xor_sync(0xffffffffu, found_end, d));
    }
    __syncwarp();  // the scratch is read for the last time before this
    begin = found_begin;
    end = found_end;
}

// What the producer-side warps of a kernel instance need: where the rings and barriers live, and which tasks this
// CTA runs. Built once per thread after the prologue.
struct ProducerContext {
    uint8_t* ring;             // K/V stage ring
    uint8_t* q_ring;           // Q rows of the published tasks
    uint32_t* pid_smem;        // [task slots][kMaxPidsPerSegment] page ids of a task's current segment
    TaskSlot* task_ring;
    uint32_t full_bar, empty_bar, task_full_bar, task_empty_bar, stream_full_bar;  // shared-memory addresses
    volatile uint32_t* abort_flag;
    uint32_t task_base, task_step, task_limit;
    bool balanced;             // the CTA owns one contiguous run of tasks
    bool allow_carry;          // consumers can continue a running state across tasks
    bool cell_major;           // round-robin dealing walks the tasks cell by cell (all templates of a KV head first)
    ActiveCounts active;
    int lane;
};

// ------------------------------ task warp ---------------------------------------------
// Decodes this CTA's tasks (32 at a time, one per lane) and publishes them one task ahead of the stream warp:
// descriptor, per-token visibility rows and Q rows for the consumers, the page ids of the task's first segment
// for the stream warp. Everything here has global-memory latency in it; keeping it off the stream warp is what
// lets that warp issue K/V copies without a pause at task boundaries.
template <typename G, int P>
__device__ __forceinline__ void run_task_warp(const MapParams& p, const CUtensorMap& q_map, const ProducerContext& c) {
    constexpr int ST = G::kStageTokens;
    constexpr int TQ = G::kTaskSlots;
    constexpr int NH = G::kColumnHalves;
    uint8_t* const q_ring = c.q_ring;
    uint32_t* const pid_smem = c.pid_smem;
    TaskSlot* const task_ring = c.task_ring;
    const uint32_t task_full_bar = c.task_full_bar, task_empty_bar = c.task_empty_bar, stream_full_bar = c.stream_full_bar;
    volatile uint32_t* const abort_flag = c.abort_flag;
    uint32_t task_base = c.task_base, task_limit = c.task_limit;
    const uint32_t task_step = c.task_step;
    const bool balanced = c.balanced;
    if (balanced) {
        balanced_task_range_warp(p, c.active.templates, c.lane, reinterpret_cast<uint32_t*>(c.ring), task_base, task_limit);
    }
    const int lane = c.lane;
    uint32_t pushed = 0;  // task-ring pushes so far

    // Order in which this CTA visits its contiguous run [task_base, task_limit) of template-major tasks: cell by
    // cell (cell = KV head x Q-head range), and within a cell template after template. Neighbours in this order
    // are consecutive KV slices of the same Q rows, so the consumers can carry their running state from one
    // task into the next instead of merging and publishing at every slice boundary.
    const uint32_t cells = p.num_kv_heads * p.head_ranges;
    const bool by_cell = c.allow_carry && balanced && cells <= 64 && task_limit > task_base && (debug_bits(p) & 512) == 0;
    const uint32_t run_r0 = by_cell ? task_base / cells : 0, run_c0 = by_cell ? task_base % cells : 0;
    const uint32_t run_r1 = by_cell ? (task_limit - 1) / cells : 0, run_c1 = by_cell ? (task_limit - 1) % cells + 1 : 0;
    auto visit_to_task = [&](uint64_t visit) -> uint64_t {
        if (!by_cell) {
            const uint64_t dealt = task_base + visit * task_step;
            if (!c.cell_major || dealt >= task_limit || c.active.templates == 0) return dealt;
            // the dealt index counts cell-major: the CTAs of the grid then work on the same KV head's rows at the
            // same time (task ids stay template-major)
            return (dealt % c.active.templates) * cells + dealt / c.active.templates;
        }
        if (visit >= task_limit - task_base) return task_limit;
        uint32_t before = 0;
        for (uint32_t c = 0; c < cells; ++c) {
            const uint32_t first_row = c >= run_c0 ? run_r0 : run_r0 + 1;
            const uint32_t end_row = c < run_c1 ? run_r1 + 1 : run_r1;  // one past the cell's last row
            const uint32_t count = end_row > first_row ? end_row - first_row : 0;
            if (visit < before + count) return uint64_t(first_row + (uint32_t(visit) - before)) * cells + c;
            before += count;
        }
        return task_limit;
    };
    // Lane l decodes this CTA's visit number first_index + l.
    auto decode_batch = [&](uint32_t first_index) {
        return decode_task(p, c.active, visit_to_task(uint64_t(first_index) + lane), task_limit);
    };
    uint32_t carry_in = 0;

    // Two batches of 32 decoded tasks live in registers.
    TaskInfo batch_cur = decode_batch(0);
    TaskInfo batch_next = decode_batch(32);
    TaskInfo cur = shfl_task(batch_cur, 0);
    bool aborted = false;
    for (uint32_t index = 0;; ++index) {
        if (visit_to_task(index) >= task_limit) break;
        // next task's descriptor: from the current batch, or lane 0 of the next one
        const uint32_t next_lane = (index + 1) & 31;
        const TaskInfo nxt = next_lane == 0 ? shfl_task(batch_next, 0) : shfl_task(batch_cur, next_lane);

        uint32_t tile_begin = 0, num_tiles = 0;
        if (cur.active && cur.kv_end > cur.kv_begin) {
            tile_begin = cur.kv_begin / ST * ST;
            num_tiles = (cur.kv_end - tile_begin + ST - 1) / ST;
        }
        // the next task continues this one: same Q rows, same request, its KV range starts where this one ends
        const uint32_t carry_out =
            (by_cell && p.direct == 0 && p.cu == nullptr && cur.active && nxt.active && nxt.tok_begin == cur.tok_begin &&
             nxt.num_toks == cur.num_toks && nxt.head_begin == cur.head_begin && nxt.num_heads == cur.num_heads &&
             nxt.req_slot == cur.req_slot && nxt.kv_begin == cur.kv_end && cur.kv_end > cur.kv_begin &&
             nxt.kv_end > nxt.kv_begin)
                ? 1u
                : 0u;
        if (cur.active && !aborted) {
            const uint32_t slot = pushed % TQ;
            const uint32_t phase = (pushed / TQ) & 1;
            // the slot is free once the consumers AND the stream warp are done with the task it held
            if (!mbar_wait(task_empty_bar + 8 * slot, phase ^ 1, abort_flag, p)) aborted = true;
            if (!aborted) {
                TaskSlot* ts = task_ring + slot;
                const uint32_t first_page = tile_begin / P;
                const uint32_t num_pages = num_tiles ? (cur.kv_end + P - 1) / P - first_page : 0;
                if (lane == 0) {
                    ts->tmpl = cur.tmpl;
                    ts->head_begin = cur.head_begin;
                    ts->num_heads = cur.num_heads;
                    ts->tok_begin = cur.tok_begin;
                    ts->num_toks = cur.num_toks;
                    ts->kv_begin = cur.kv_begin;
                    ts->kv_end = cur.kv_end;
                    ts->tile_begin = tile_begin;
                    ts->num_tiles = num_tiles;
                    ts->done = 0;
                    ts->group = cur.group;
                    ts->part_begin = cur.part_begin;
                    ts->part_count = cur.part_count;
                    ts->carry = carry_in | (carry_out << 1);
                    ts->kv_head = cur.kv_head;
                    ts->req_slot = cur.req_slot;
                }
                // page ids of the first segment (the stream warp stages later segments of a very long task itself)
                {
                    const uint64_t base =
                        (uint64_t(cur.req_slot) * p.num_gqa_layers + p.layer_index) * p.pages_per_request_layer;
                    const uint32_t count = min(num_pages, uint32_t(kMaxPidsPerSegment));
                    for (uint32_t i = lane; i < count; i += 32) {
                        const uint32_t dst = smem_addr(pid_smem + slot * kMaxPidsPerSegment + i);
                        const uint32_t* src = p.page_ids + base + first_page + i;
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
                    }
                    asm volatile("cp.async.commit_group;" ::: "memory");
                }
                if (p.visible != nullptr) {
                    for (uint32_t i = lane; i < 2 * cur.num_toks; i += 32) {
                        const uint32_t dst = smem_addr(&ts->visible[i]);
                        const uint32_t* src = p.visible + uint64_t(cur.tok_begin) * 2 + i;
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
                    }
                }
                if (p.visible != nullptr) mbar_arrive_after_cp_async(task_full_bar + 8 * slot);
                const uint32_t q_boxes = (debug_bits(p) & 4) ? 0u : cur.num_toks * NH;
                if (lane == 0) {
                    mbar_arrive_expect_tx(task_full_bar + 8 * slot, q_boxes * p.heads_per_task * 128);
                }
                __syncwarp();
                for (uint32_t b = lane; b < q_boxes; b += 32) {
                    const uint32_t tok = b / NH;
                    const uint32_t half = b % NH;
                    const uint32_t dst = smem_addr(q_ring + slot * G::kQBytes + half * (G::kQRows * 128) +
                                                   tok * p.heads_per_task * 128);
                    const uint32_t row = (cur.tok_begin + tok) * p.num_q_heads + cur.head_begin;
                    tma_load_2d(dst, &q_map, half * 64, static_cast<int32_t>(row), task_full_bar + 8 * slot);
                }
                // the page ids have landed: hand the task to the stream warp
                asm volatile("cp.async.wait_group 0;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(stream_full_bar + 8 * slot);
                ++pushed;
            }
        }
        // advance
        carry_in = carry_out;
        cur = nxt;
        if (next_lane == 0) {
            batch_cur = batch_next;
            batch_next = decode_batch(index + 1 + 32);
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    // ---- tell the consumers and the stream warp there is nothing more
    if (!aborted) {
        const uint32_t slot = pushed % TQ;
        const uint32_t phase = (pushed / TQ) & 1;
        if (mbar_wait(task_empty_bar + 8 * slot, phase ^ 1, abort_flag, p)) {
            if (lane == 0) {
                task_ring[slot].done = 1;
                mbar_arrive_expect_tx(task_full_bar + 8 * slot, 0);
                mbar_arrive(stream_full_bar + 8 * slot);
            }
            if (p.visible != nullptr) mbar_arrive_after_cp_async(task_full_bar + 8 * slot);
        }
    }
    // Abort path only: Q copies already issued may still be landing; wait (bounded) for them.
    if (*abort_flag) {
        for (uint32_t back = 0; back < uint32_t(TQ) && back < pushed; ++back) {
            const uint32_t c = pushed - 1 - back;
            for (uint32_t i = 0; i < p.wait_limit; ++i) {
                if (mbar_try_wait(task_full_bar + 8 * (c % TQ), (c / TQ) & 1)) break;
            }
        }
    }
}

// ------------------------------ stream warp -------------------------------------------
// Issues the K/V copies of one published task after the other into the stage ring. The per-stage loop runs in
// lane 0 alone, with running slot / phase / token counters and 32-bit row arithmetic: this loop is the one
// instruction stream that has to keep the copy engine fed, and it reads shared memory only.
// Issuing lanes of the stream warp for a ring of `stages` slots. The lanes move in lock step, so a group of L
// stages is issued when L slots are free: measured on B200, four lanes raise the decode bench (12-slot ring,
// two copies per stage) from 5.0 to 5.8 TB/s and cost the 8-slot ring of head_dim 256 12 %.
__host__ __device__ constexpr int stream_lanes(int stages) { return stages >= 12 ? 4 : 1; }

// L lanes issue: lane l takes the task's stages l, l + L, ... so that the waits, barrier arrivals and page-id loads
// of L stages (a chain of dependent shared-memory operations per stage) run side by side.
template <typename G, int P, int L = 1>
__device__ __forceinline__ void run_stream_warp(const MapParams& p, const CUtensorMap& kv_map, const ProducerContext& c) {
    static_assert(L >= 1 && L <= G::kStages && L <= 32, "issuing lanes must fit the ring");
    constexpr int ST = G::kStageTokens;
    constexpr int NS = G::kStages;
    constexpr int TQ = G::kTaskSlots;
    uint8_t* const ring = c.ring;
    uint32_t* const pid_smem = c.pid_smem;
    TaskSlot* const task_ring = c.task_ring;
    const uint32_t full_bar = c.full_bar, empty_bar = c.empty_bar, task_empty_bar = c.task_empty_bar;
    const uint32_t stream_full_bar = c.stream_full_bar;
    volatile uint32_t* const abort_flag = c.abort_flag;
    const int lane = c.lane;
    uint32_t stage_counter = 0;
    bool aborted = false;
    const uint32_t rows_per_page = 2 * p.num_kv_heads * P;
    const uint64_t kv_policy = l2_evict_first_policy();
    for (uint32_t taken = 0; !aborted; ++taken) {
        const uint32_t tslot = taken % TQ;
        if (!mbar_wait(stream_full_bar + 8 * tslot, (taken / TQ) & 1, abort_flag, p)) break;
        const TaskSlot* ts = task_ring + tslot;
        if (ts->done) break;
        const uint32_t tile_begin = ts->tile_begin, num_tiles = ts->num_tiles, kv_end = ts->kv_end;
        const uint32_t head_row = ts->kv_head * P;
        if (num_tiles > 0) {
            constexpr uint32_t kTilesPerSegment = uint32_t(kMaxPidsPerSegment) * P / ST;
            const uint32_t first_page = tile_begin / P;
            const uint32_t num_pages = (kv_end + P - 1) / P - first_page;
            const uint32_t* pids = pid_smem + tslot * kMaxPidsPerSegment;
            for (uint32_t seg_tile = 0; seg_tile < num_tiles && !aborted; seg_tile += kTilesPerSegment) {
                if (seg_tile > 0) {
                    // a task longer than one segment: restage the next run of page ids (whole warp)
                    const uint32_t seg_first = first_page + seg_tile * (ST / P);
                    const uint32_t count = min(first_page + num_pages - seg_first, uint32_t(kMaxPidsPerSegment));
                    const uint64_t base =
                        (uint64_t(ts->req_slot) * p.num_gqa_layers + p.layer_index) * p.pages_per_request_layer;
                    __syncwarp();
                    for (uint32_t i = lane; i < count; i += 32) {
                        const uint32_t dst = smem_addr(pid_smem + tslot * kMaxPidsPerSegment + i);
                        const uint32_t* src = p.page_ids + base + seg_first + i;
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
                    }
                    asm volatile("cp.async.commit_group;" ::: "memory");
                    asm volatile("cp.async.wait_group 0;" ::: "memory");
                    __syncwarp();
                }
                const uint32_t seg_tiles = min(num_tiles - seg_tile, kTilesPerSegment);
                uint32_t failed = 0;
                if (lane < L) {
                    uint32_t slot = (stage_counter + lane) % NS;
                    uint32_t parity = (((stage_counter + lane) / NS) & 1) ^ 1;
                    uint32_t tile_tok = tile_begin + (seg_tile + lane) * ST;
                    uint32_t page_in_seg = lane * (ST / P);
                    for (uint32_t tile = lane; tile < seg_tiles; tile += L) {
                        const uint32_t bar = full_bar + 8 * slot;
                        if (!mbar_wait(empty_bar + 8 * slot, parity, abort_flag, p)) {
                            failed = tile + 1;
                            break;
                        }
                        const uint32_t dst = smem_addr(ring) + slot * G::kStageBytes;
                        // measurement build only: the bytes of a task's first stage are announced and never copied
                        const bool withhold = (debug_bits(p) & 8192) != 0 && seg_tile + tile == 0;
                        if (tile_tok + ST <= kv_end && !(debug_bits(p) & 8)) {
                            mbar_arrive_expect_tx(bar, G::kStageBytes);
#pragma unroll
                            for (int b = 0; b < G::kBoxesPerPlane; ++b) {
                                const uint32_t tok_in_page = (b * G::kBoxRows) % P;
                                const uint32_t pid = pids[page_in_seg + (b * G::kBoxRows) / P];
                                if (pid >= p.pool_pages) atomicOr(p.status, kStatusPageOutOfPool);
                                if (withhold) continue;
                                tma_load_4d(dst + b * G::kCopyBytes, &kv_map, 0,
                                            static_cast<int32_t>(pid * rows_per_page + head_row + tok_in_page), 0, 0, bar, kv_policy);
                            }
                        } else {
                            // the task's last stage (or the measurement mode without copies): only boxes that hold
                            // a token below kv_end are fetched
                            uint32_t boxes_needed = 0;
#pragma unroll
                            for (int b = 0; b < G::kBoxesPerPlane; ++b) {
                                if (tile_tok + b * G::kBoxRows < kv_end) ++boxes_needed;
                            }
                            if (debug_bits(p) & 8) boxes_needed = 0;
                            mbar_arrive_expect_tx(bar, boxes_needed * G::kCopyBytes);
#pragma unroll
                            for (int b = 0; b < G::kBoxesPerPlane; ++b) {
                                if (uint32_t(b) < boxes_needed) {
                                    const uint32_t tok_in_page = (b * G::kBoxRows) % P;
                                    const uint32_t pid = pids[page_in_seg + (b * G::kBoxRows) / P];
                                    if (pid >= p.pool_pages) atomicOr(p.status, kStatusPageOutOfPool);
                                    if (withhold) continue;
                                    tma_load_4d(dst + b * G::kCopyBytes, &kv_map, 0,
                                                static_cast<int32_t>(pid * rows_per_page + head_row + tok_in_page), 0, 0,
                                                bar, kv_policy);
                                }
                            }
                        }
                        tile_tok += L * ST;
                        page_in_seg += L * (ST / P);
                        slot += L;
                        if (slot >= uint32_t(NS)) {
                            slot -= NS;
                            parity ^= 1;
                        }
                    }
                }
                if (L == 1) {
                    failed = __shfl_sync(0xffffffffu, failed, 0);
                    if (failed) {
                        aborted = true;
                        stage_counter += failed - 1;
                    } else {
                        stage_counter += seg_tiles;
                    }
                } else {
                    // which stages were issued is not a prefix then: count them all (the drain below is bounded)
                    if (__any_sync(0xffffffffu, failed != 0)) aborted = true;
                    stage_counter += seg_tiles;
                }
            }
        }
        // done with the task's descriptor and page ids
        __syncwarp();
        if (lane == 0) mbar_arrive(task_empty_bar + 8 * tslot);
    }
    // Abort path only: copies already issued may still be landing; wait (bounded) for each ring slot's
    // last issued phase before the CTA may retire.
    if (*abort_flag) {
        for (uint32_t back = 0; back < uint32_t(NS) && back < stage_counter; ++back) {
            const uint32_t c = stage_counter - 1 - back;
            for (uint32_t i = 0; i < p.wait_limit; ++i) {
                if (mbar_try_wait(full_bar + 8 * (c % NS), (c / NS) & 1)) break;
            }
        }
    }
}

// ------------------------------ decode warps (FP8 pages) ------------------------------
// Two FP8 E4M3FN bytes (bits 0-7 and 8-15 of `pair`, already moved to the high byte of each 16-bit lane) to two
// elements of T, exactly (components/gqa/fp8.rs:46-58, metal/gqa_fp8.metal:1-25): sign and the seven magnitude
// bits are placed so that the 4-bit exponent sits at the bottom of T's exponent field, then one multiplication
// by 2^(bias of T - 7) moves the exponent into place. A zero exponent field is a subnormal of T there, which the
// multiplication normalises, so the FP8 subnormals need no special case; 0x7f / 0xff (NaN) do.
template <typename T>
__device__ __forceinline__ uint32_t fp8x2_high_bytes_to_t2(uint32_t high_bytes);

template <>
__device__ __forceinline__ uint32_t fp8x2_high_bytes_to_t2<__nv_bfloat16>(uint32_t x) {
    const uint32_t placed = (x & 0x80008000u) | ((x >> 4) & 0x07f007f0u);
    uint32_t scaled;
    asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(scaled) : "r"(placed), "r"(0x7b807b80u));  // x 2^120, both lanes
    return scaled;
}

template <>
__device__ __forceinline__ uint32_t fp8x2_high_bytes_to_t2<__half>(uint32_t x) {
    const uint32_t placed = (x & 0x80008000u) | ((x >> 1) & 0x3f803f80u);
    uint32_t scaled;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(scaled) : "r"(placed), "r"(0x5c005c00u));  // x 2^8, both lanes
    return scaled;
}

// Nonzero when one of the four bytes of `word` is the NaN code (0x7f / 0xff).
__device__ __forceinline__ uint32_t fp8x4_nan_mask(uint32_t word) {
    return ((word & 0x7f7f7f7fu) + 0x01010101u) & 0x80808080u;
}

// Four FP8 bytes of `word` (element i in bits 8i..8i+7) to four elements of T in two words. PATCH: also give
// the NaN codes a NaN value (without it they decode to +-480, a value no other code has).
template <typename T, bool PATCH>
__device__ __forceinline__ void fp8x4_to_t4(uint32_t word, uint32_t& lo, uint32_t& hi) {
    lo = fp8x2_high_bytes_to_t2<T>(__byte_perm(word, 0u, 0x1404));
    hi = fp8x2_high_bytes_to_t2<T>(__byte_perm(word, 0u, 0x3424));
    if (PATCH && fp8x4_nan_mask(word)) {
        constexpr uint32_t nan_bits = 0x7fffu;  // all exponent and mantissa bits of a 16-bit element
        if ((word & 0x0000007fu) == 0x0000007fu) lo |= nan_bits;
        if ((word & 0x00007f00u) == 0x00007f00u) lo |= nan_bits << 16;
        if ((word & 0x007f0000u) == 0x007f0000u) hi |= nan_bits;
        if ((word & 0x7f000000u) == 0x7f000000u) hi |= nan_bits << 16;
    }
}

// Expands raw stages into the 16-bit stage ring: 16 raw bytes (16 elements of one K or V row) become two
// 16-byte chunks. Decode warp w takes the stages whose running number is congruent to w modulo the number of
// decode warps, so the warps work on different stages and hide one another's latencies.
// Both rings use the 128-byte swizzle of the copies (chunk c of row r at position c ^ (r & 7) of its 128-byte
// line); a raw line holds 128 elements, i.e. the 64-element lines of two column halves of the 16-bit stage.
// Lane mapping, per block of four rows: eight consecutive lanes take the lower four chunks of one row and the
// upper four of its neighbour (r ^ 1). That makes the eight 16-byte loads of a quarter warp, and each of its two
// rounds of eight 16-byte stores, cover all 32 banks.
template <typename T, typename G>
__device__ __forceinline__ void run_decode_warps(const MapParams& p, const ProducerContext& c, uint8_t* stage_ring,
                                                 uint32_t stage_full_bar, uint32_t stage_empty_bar, int decode_thread) {
    using R = typename G::Raw;
    constexpr int NS = G::kStages;
    constexpr int NR = R::kStages;
    constexpr int TQ = G::kTaskSlots;
    constexpr int DW = G::kDecodeWarps;
    constexpr int kLines = R::kBoxRows;                                   // 128-byte lines per block
    constexpr int kBlocks = R::kBoxesPerPlane * 2 * R::kColumnGroups;     // (token box, plane, column group)
    static_assert(kLines % 4 == 0, "a block is a whole number of four-row groups");
    volatile uint32_t* const abort_flag = c.abort_flag;
    const int lane = decode_thread & 31;
    const uint32_t dw = uint32_t(decode_thread) >> 5;
    // lane roles within a four-row group
    const uint32_t sub = (lane >> 2) & 1, cc = lane & 3, pair = lane >> 4, flip = (lane >> 3) & 1;
    const uint32_t row4 = 2 * pair + sub;             // row within the group
    const uint32_t upper = sub ^ flip;                // which half of the raw line: raw chunk = 4 * upper + cc
    const uint32_t raw_lane = row4 * 128 + (((4 * upper + cc) ^ row4) << 4);
    const uint32_t out_lane = upper * G::kBoxBytes + row4 * 128;
    const uint32_t even_lane = out_lane + (((2 * cc) ^ row4) << 4);
    const uint32_t odd_lane = out_lane + (((2 * cc + 1) ^ row4) << 4);
    uint32_t stage_base = 0;  // running number of the task's first stage
    for (uint32_t taken = 0;; ++taken) {
        const uint32_t tslot = taken % TQ;
        if (!mbar_wait(c.stream_full_bar + 8 * tslot, (taken / TQ) & 1, abort_flag, p)) return;
        const TaskSlot* ts = c.task_ring + tslot;
        const uint32_t done = ts->done, num_tiles = ts->num_tiles;
        __syncwarp();
        if (lane == 0) mbar_arrive(c.task_empty_bar + 8 * tslot);  // the descriptor has been read
        if (done) return;
        uint32_t stage = stage_base + (dw + DW - stage_base % DW) % DW;  // this warp's first stage of the task
        for (; stage < stage_base + num_tiles; stage += DW) {
            const uint32_t rslot = stage % NR, sslot = stage % NS;
            if (!mbar_wait(c.full_bar + 8 * rslot, (stage / NR) & 1, abort_flag, p)) return;
            if (!mbar_wait(stage_empty_bar + 8 * sslot, ((stage / NS) & 1) ^ 1, abort_flag, p)) return;
            const uint32_t raw = smem_addr(c.ring + rslot * R::kStageBytes) + raw_lane;
            const uint32_t out = smem_addr(stage_ring + sslot * G::kStageBytes);
            // The common pass has no branches (the loads, conversions and stores of the 16 units interleave
            // freely) and only notes whether a NaN code went by; a stage that held one is decoded again with
            // the patching form.
            uint32_t suspect = 0;
            auto decode_stage = [&](auto patch) {
                constexpr bool kPatch = decltype(patch)::value;
#pragma unroll
                for (int blk = 0; blk < kBlocks; ++blk) {
                    constexpr int kGroups = R::kColumnGroups;
                    const int group = blk % kGroups, plane = (blk / kGroups) & 1, box = blk / (2 * kGroups);
                    const uint32_t block_out =
                        out + box * G::kCopyBytes + plane * G::kPlaneBoxBytes + 2 * group * G::kBoxBytes;
                    // all loads of the block first: they are volatile, as are the stores, and keep their order
                    uint4 bytes[kLines / 4];
#pragma unroll
                    for (int rb = 0; rb < kLines / 4; ++rb) {
                        // rows 4-7 of an eight-row swizzle period: position bit 2 flips (64 bytes)
                        const uint32_t period = (rb & 1) * 64;
                        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(bytes[rb].x), "=r"(bytes[rb].y), "=r"(bytes[rb].z), "=r"(bytes[rb].w)
                                     : "r"((raw ^ period) + blk * kLines * 128 + rb * 512));
                    }
#pragma unroll
                    for (int rb = 0; rb < kLines / 4; ++rb) {
                        const uint32_t period = (rb & 1) * 64;
                        if (!kPatch) {
                            suspect |= fp8x4_nan_mask(bytes[rb].x) | fp8x4_nan_mask(bytes[rb].y) |
                                       fp8x4_nan_mask(bytes[rb].z) | fp8x4_nan_mask(bytes[rb].w);
                        }
                        uint4 first, second;
                        fp8x4_to_t4<T, kPatch>(bytes[rb].x, first.x, first.y);
                        fp8x4_to_t4<T, kPatch>(bytes[rb].y, first.z, first.w);
                        fp8x4_to_t4<T, kPatch>(bytes[rb].z, second.x, second.y);
                        fp8x4_to_t4<T, kPatch>(bytes[rb].w, second.z, second.w);
                        const uint32_t rows = block_out + rb * 512;
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(rows + (even_lane ^ period)),
                                     "r"(first.x), "r"(first.y), "r"(first.z), "r"(first.w) : "memory");
                        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(rows + (odd_lane ^ period)),
                                     "r"(second.x), "r"(second.y), "r"(second.z), "r"(second.w) : "memory");
                    }
                }
            };
            if (!(debug_bits(p) & 4096)) {
                decode_stage(std::false_type{});
                if (__any_sync(0xffffffffu, suspect != 0)) decode_stage(std::true_type{});
            }
            __syncwarp();
            if (lane == 0) {
                mbar_arrive(stage_full_bar + 8 * sslot);   // the 16-bit stage is written
                mbar_arrive(c.empty_bar + 8 * rslot);       // the raw stage has been read
            }
        }
        stage_base += num_tiles;
    }
}

template <typename T, int D, int P, int MT, int KVW, int PS, bool HALF, int KVB = 2>
__global__ void __launch_bounds__(MapGeometry<D, P, MT, KVW, PS, HALF, KVB>::kThreads, 1)
sdpa_map_kernel(const __grid_constant__ CUtensorMap kv_map, const __grid_constant__ CUtensorMap q_map,
                const MapParams p) {
    using G = MapGeometry<D, P, MT, KVW, PS, HALF, KVB>;
    constexpr int ST = G::kStageTokens;
    constexpr int NS = G::kStages;
    constexpr int TQ = G::kTaskSlots;
    constexpr int NCW = G::kConsumerWarps;
    constexpr int WT = G::kWarpTokens;  // KV tokens per warp per stage
    constexpr int KP = G::kMergeParts;
    constexpr int NT = WT / 8;       // S n-tiles (8 KV tokens each) per warp per stage
    constexpr int KT = WT / 16;      // PV k-tiles (16 KV tokens each) per warp per stage
    constexpr int DK = D / 16;       // QK k-steps
    constexpr int DN = D / 8;        // O n-tiles
    constexpr int NROW = HALF ? 1 : 2;  // fragment rows (g, g + 8) that can be valid

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = smem;
    uint8_t* raw_ring = ring + NS * G::kStageBytes;  // FP8 pages only (no bytes otherwise)
    uint8_t* q_ring = raw_ring + G::kRawStages * G::kRawStageBytes;
    float* merge = reinterpret_cast<float*>(q_ring + TQ * G::kQBytes);
    uint32_t* pid_smem = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(merge) + G::kMergeBytes);
    TaskSlot* task_ring = reinterpret_cast<TaskSlot*>(reinterpret_cast<uint8_t*>(pid_smem) + G::kPidBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(task_ring) + G::kTaskBytes);
    constexpr int NR = G::kRawStages;
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 2 * NS + 3 * TQ + 2 * NR);
    volatile uint32_t* last_flag = abort_flag + 1;  // fused reduce: "this CTA completed its group"

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t full_bar = smem_addr(bars);
    const uint32_t empty_bar = smem_addr(bars + NS);
    const uint32_t task_full_bar = smem_addr(bars + 2 * NS);
    const uint32_t task_empty_bar = smem_addr(bars + 2 * NS + TQ);
    const uint32_t stream_full_bar = smem_addr(bars + 2 * NS + 2 * TQ);
    const uint32_t raw_full_bar = smem_addr(bars + 2 * NS + 3 * TQ);
    const uint32_t raw_empty_bar = smem_addr(bars + 2 * NS + 3 * TQ + NR);

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            // a stage is complete when its copies have landed, or when a decode warp has written it
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, MT * PS);
        }
        for (int s = 0; s < NR; ++s) {
            mbar_init(raw_full_bar + 8 * s, 1);
            mbar_init(raw_empty_bar + 8 * s, 1);
        }
        for (int s = 0; s < TQ; ++s) {
            // the expect_tx arrival, plus (when per-token visibility rows are staged) 32 lanes' cp.async arrivals
            mbar_init(task_full_bar + 8 * s, p.visible != nullptr ? 33 : 1);
            // every consumer warp, the stream warp and the decode warps
            mbar_init(task_empty_bar + 8 * s, NCW + 1 + G::kDecodeWarps);
            mbar_init(stream_full_bar + 8 * s, 1);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    // Q rows no copy ever writes (row padding of the tile) must not hold NaN bit patterns.
    for (int i = threadIdx.x; i < TQ * G::kQBytes / 16; i += G::kThreads) {
        reinterpret_cast<uint4*>(q_ring)[i] = make_uint4(0, 0, 0, 0);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();

    // A kernel launched behind this one with programmatic stream serialization (the reducer) may be scheduled as
    // this kernel's blocks retire; it waits for this kernel's completion itself. Only where this block's shared
    // memory leaves no room for a reducer block (12 KB) beside it: reducer blocks that became resident next to a
    // still-running map block cost the one-sequence workload 8 us per step.
    if constexpr (G::kSmemBytes + 14 * 1024 > 228 * 1024) {
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    const ActiveCounts active = resolve_active(p);
    const uint32_t total_tasks = active.templates * p.num_kv_heads * p.head_ranges;

    // one contiguous, cost-balanced run of tasks per CTA (the task warp works out which), or a round-robin deal
    // (the scan keeps one word per template in the ring of K/V stages, before the first copy is issued)
    constexpr uint32_t kScanTemplates = KVB == 1 ? uint32_t(G::kRawStages) * G::kRawStageBytes / 4 : uint32_t(NS) * G::kStageBytes / 4;
    const bool balanced = active.templates <= kBalanceMaxTemplates && active.templates <= kScanTemplates;
    const uint32_t task_base = blockIdx.x;
    const uint32_t task_step = balanced ? 1u : gridDim.x;
    const uint32_t task_limit = total_tasks;

    ProducerContext producer{};
    producer.ring = ring;
    producer.q_ring = q_ring;
    producer.pid_smem = pid_smem;
    producer.task_ring = task_ring;
    producer.full_bar = full_bar;
    producer.empty_bar = empty_bar;
    producer.task_full_bar = task_full_bar;
    producer.task_empty_bar = task_empty_bar;
    producer.stream_full_bar = stream_full_bar;
    producer.abort_flag = abort_flag;
    producer.task_base = task_base;
    producer.task_step = task_step;
    producer.task_limit = task_limit;
    producer.balanced = balanced;
    producer.allow_carry = true;
    producer.active = active;
    producer.lane = lane;
    if constexpr (KVB == 1) {
        // the stream warp fills the raw ring; the decode warps sit between it and the consumers' ring
        producer.ring = raw_ring;
        producer.full_bar = raw_full_bar;
        producer.empty_bar = raw_empty_bar;
    }
    if (warp >= NCW + 2) {
        if constexpr (KVB == 1) {
            run_decode_warps<T, G>(p, producer, ring, full_bar, empty_bar, int(threadIdx.x) - (NCW + 2) * 32);
        }
    } else if (warp == NCW + 1) {
        run_task_warp<G, P>(p, q_map, producer);
    } else if (warp == NCW) {
        if constexpr (KVB == 1) {
            run_stream_warp<typename G::Raw, P, stream_lanes(G::Raw::kStages)>(p, kv_map, producer);
        } else {
            run_stream_warp<G, P, stream_lanes(G::kStages)>(p, kv_map, producer);
        }
    } else {
        // ------------------------------ consumer warps ----------------------------------------
        const int mt = warp % MT;           // row tile
        const int ps = (warp / MT) % PS;    // which part of a stage's tokens
        const int kw = warp / (MT * PS);    // KV warp group
        const int part = kw * PS + ps;      // index among the states merged for this row tile
        const int g = lane >> 2;    // fragment row group
        const int tq = lane & 3;    // thread in quad
        uint32_t stage_counter = 0;
        uint32_t my_stage = kw, my_slot = kw, my_parity = 0;
        const int lm_mat = lane >> 3;  // which of the four 8x8 matrices this lane addresses in ldmatrix
        const int lm_row = lane & 7;
        // ldmatrix lane roles. K (B operand, rows = KV tokens): matrix pair (lm_mat >> 1) picks the 8-token
        // group, (lm_mat & 1) the 16-byte chunk. V (transposed) and Q (A operand): (lm_mat & 1) picks the
        // 8-row group, (lm_mat >> 1) the chunk. Rows are taken relative to a 16-token group / 16-row tile.
        static_assert(G::kBoxRows % 8 == 0 && (16 % G::kBoxRows == 0 || G::kBoxRows % 16 == 0),
                      "token boxes must tile, or be tiled by, 16-token groups");
        const uint32_t k_row = (lm_mat >> 1) * 8 + lm_row;
        const uint32_t v_row = (lm_mat & 1) * 8 + lm_row;
        const uint32_t k_lane = (k_row / G::kBoxRows) * G::kCopyBytes + (k_row % G::kBoxRows) * 128;
        const uint32_t v_lane = (v_row / G::kBoxRows) * G::kCopyBytes + (v_row % G::kBoxRows) * 128;
        const uint32_t k_xor = (lm_mat & 1) ^ (k_row & 7);
        const uint32_t v_xor = (lm_mat >> 1) ^ (v_row & 7);

        float o[DN][4];
        float m_run[2] = {-INFINITY, -INFINITY};
        float l_run[2] = {0.0f, 0.0f};
#pragma unroll
        for (int n = 0; n < DN; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
        for (uint32_t popped = 0;; ++popped) {
            const uint32_t tslot = popped % TQ;
            if (!mbar_wait(task_full_bar + 8 * tslot, (popped / TQ) & 1, abort_flag, p)) break;
            const TaskSlot* ts = task_ring + tslot;
            if (ts->done) break;
            const uint32_t t_tmpl = ts->tmpl, t_head_begin = ts->head_begin, t_num_heads = ts->num_heads;
            const uint32_t t_tok_begin = ts->tok_begin, t_num_toks = ts->num_toks;
            const uint32_t t_kv_begin = ts->kv_begin, t_kv_end = ts->kv_end;
            const uint32_t t_tile_begin = ts->tile_begin, t_num_tiles = ts->num_tiles;
            const uint32_t t_group = ts->group, t_part_begin = ts->part_begin, t_part_count = ts->part_count;
            // fused reduce: a Q range with a single partial needs no merge, its task writes the final output
            const bool fused = p.cu != nullptr;
            const bool write_final = p.direct != 0 || (fused && t_part_count == 1);

            // ---- per-thread row bounds: rows g and g + 8 of row tile mt
            uint32_t lo[NROW], hi[NROW];
#pragma unroll
            for (int i = 0; i < NROW; ++i) {
                const uint32_t row = mt * G::kTileRows + g + 8 * i;
                const uint32_t row_tok = row / p.heads_per_task;
                const uint32_t row_head = row % p.heads_per_task;
                // rows that hold no (token, head) of this task are never published; leaving them unmasked keeps
                // the mask test below false for tiles that every real row sees completely
                lo[i] = 0;
                hi[i] = 0xffffffffu;
                if (row_tok < t_num_toks && row_head < t_num_heads) {
                    uint32_t vb = 0, ve = 0xffffffffu;
                    if (p.visible != nullptr) {
                        vb = ts->visible[row_tok * 2];
                        ve = ts->visible[row_tok * 2 + 1];
                    }
                    lo[i] = max(vb, t_kv_begin);
                    hi[i] = min(ve, t_kv_end);
                    if (hi[i] < lo[i]) hi[i] = lo[i];
                }
            }

            // A task that continues the KV range of the previous one for the same Q rows (the producer says so)
            // keeps the running (m, l, O); every other task starts from nothing.
            const uint32_t t_carry = ts->carry;
            if (!(t_carry & 1u)) {
#pragma unroll
                for (int n = 0; n < DN; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
                m_run[0] = m_run[1] = -INFINITY;
                l_run[0] = l_run[1] = 0.0f;
            }
            const uint32_t q_tile = smem_addr(q_ring + tslot * G::kQBytes) + mt * G::kTileRows * 128;
            uint32_t q_addr[4];
#pragma unroll
            for (int c4 = 0; c4 < 4; ++c4) q_addr[c4] = q_tile + v_row * 128 + (((2 * c4) ^ v_xor) << 4);
            // Half-tile tasks keep their Q fragments in registers for the whole task (rows 8-15 are zero).
            uint32_t q_regs[HALF ? DK : 1][2];
            if constexpr (HALF) {
#pragma unroll
                for (int kk = 0; kk < DK; ++kk) {
                    uint32_t a[4];
                    ldmatrix_x4(a, q_addr[kk & 3] + ((2 * kk) / 8) * (G::kQRows * 128));
                    q_regs[kk][0] = a[0];
                    q_regs[kk][1] = a[2];
                }
            }

            // This warp consumes the stages whose running number is congruent to kw modulo KVW, across tasks:
            // my_stage is the next one, my_slot / my_parity its ring slot and barrier parity.
            for (; my_stage < stage_counter + t_num_tiles; my_stage += KVW) {
                const uint32_t tile = my_stage - stage_counter;
                const uint32_t slot = my_slot;
                const uint32_t phase = my_parity;
                my_slot += KVW;
                if (my_slot >= uint32_t(NS)) {
                    my_slot -= NS;
                    my_parity ^= 1;
                }
                if (!mbar_wait(full_bar + 8 * slot, phase, abort_flag, p)) continue;
                if (debug_bits(p) & 1) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_bar + 8 * slot);
                    continue;
                }
                const uint32_t tile_tok = t_tile_begin + tile * ST + ps * WT;  // first token this warp handles
                if (PS > 1 && tile_tok >= t_kv_end) {
                    // the tokens of this warp's part of the stage are all past the end: nothing to add
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_bar + 8 * slot);
                    continue;
                }
                // stage layout: per token box [K: halves x rows x 128 B][V: halves x rows x 128 B]
                const uint32_t k_base = smem_addr(ring + slot * G::kStageBytes);
                const uint32_t v_base = k_base + G::kPlaneBoxBytes;

                // Rows of tokens at or past kv_end may never have been written (or loaded): clear them in V
                // so that a zero probability times stale bits cannot produce NaN.
                if (tile_tok + WT > t_kv_end) {
                    const uint32_t first_bad = t_kv_end - tile_tok;  // within this warp's tokens
                    for (uint32_t idx = first_bad * (D / 8) + lane; idx < uint32_t(WT) * (D / 8); idx += 32) {
                        const uint32_t r = ps * WT + idx / (D / 8);  // token row within the stage
                        const uint32_t c = idx % (D / 8);
                        const uint32_t box = r / G::kBoxRows;
                        const uint32_t addr = v_base + box * G::kCopyBytes + (c / 8) * G::kBoxBytes +
                                              (r % G::kBoxRows) * 128 + (c % 8) * 16;
                        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
                    }
                    __syncwarp();
                }

                // ---- S = Q K^T (raw dot products; the softmax scale is folded into the exponent below)
                // Swizzled ldmatrix addresses: a 16-byte chunk c of row r sits at chunk (c ^ (r & 7)) of its
                // 128-byte line. With c = 2 * step + bit, (c & 7) ^ (r & 7) = ((2 * step) & 7) ^ (bit ^ (r & 7)),
                // so four per-lane bases (one per value of (2 * step) & 7) plus compile-time offsets cover
                // every load of the tile.
                uint32_t k_addr[4], v_addr[4];
#pragma unroll
                for (int c4 = 0; c4 < 4; ++c4) {
                    k_addr[c4] = k_base + k_lane + (((2 * c4) ^ k_xor) << 4);
                    v_addr[c4] = v_base + v_lane + (((2 * c4) ^ v_xor) << 4);
                }
                float s[NT][4];
#pragma unroll
                for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
                const uint32_t knock = (debug_bits(p) >> 4) & 7;  // measurement aid
                if (!(knock & 1))
#pragma unroll
                for (int kk = 0; kk < DK; ++kk) {
                    uint32_t a[4];
                    if constexpr (HALF) {
                        a[0] = q_regs[kk][0];
                        a[1] = 0u;
                        a[2] = q_regs[kk][1];
                        a[3] = 0u;
                    } else {
                        ldmatrix_x4(a, q_addr[kk & 3] + ((2 * kk) / 8) * (G::kQRows * 128));
                    }
#pragma unroll
                    for (int jp = 0; jp < NT / 2; ++jp) {
                        uint32_t b[4];
                        ldmatrix_x4(b, k_addr[kk & 3] + ((2 * kk) / 8) * G::kBoxBytes +
                                           ((ps * WT + 16 * jp) / G::kBoxRows) * G::kCopyBytes +
                                           ((ps * WT + 16 * jp) % G::kBoxRows) * 128);
                        mma_16816<T>(s[2 * jp], a, b[0], b[1]);
                        mma_16816<T>(s[2 * jp + 1], a, b[2], b[3]);
                    }
                }

                // ---- mask (only where a row's visible range cuts the tile) and running maximum
                if (knock & 2) {
                    // skip the softmax: feed the raw scores through
#pragma unroll
                    for (int j = 0; j < NT; ++j) { s[j][0] *= 1e-9f; s[j][1] *= 1e-9f; }
                }
                bool cut = false;
#pragma unroll
                for (int i = 0; i < NROW; ++i) cut = cut || tile_tok < lo[i] || tile_tok + WT > hi[i];
                if (__any_sync(0xffffffffu, cut)) {
#pragma unroll
                    for (int j = 0; j < NT; ++j) {
#pragma unroll
                        for (int e = 0; e < 2 * NROW; ++e) {
                            const uint32_t tok = tile_tok + j * 8 + tq * 2 + (e & 1);
                            if (!(tok >= lo[e >> 1] && tok < hi[e >> 1])) s[j][e] = -INFINITY;
                        }
                    }
                }
                float tile_max[NROW];
#pragma unroll
                for (int i = 0; i < NROW; ++i) {
                    tile_max[i] = fmaxf(s[0][2 * i], s[0][2 * i + 1]);
#pragma unroll
                    for (int j = 1; j < NT; ++j) tile_max[i] = fmaxf(tile_max[i], fmaxf(s[j][2 * i], s[j][2 * i + 1]));
                }
                float alpha[NROW], shift[NROW];
                bool rescale = false;
#pragma unroll
                for (int i = 0; i < NROW; ++i) {
                    tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 1));
                    tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 2));
                    const float m_new = fmaxf(m_run[i], tile_max[i]);
                    const float base = m_new == -INFINITY ? 0.0f : m_new;
                    // nothing has been accumulated while the running maximum is -inf: no rescale needed
                    alpha[i] = m_run[i] == -INFINITY ? 1.0f : fast_exp2((m_run[i] - base) * p.scale_log2e);
                    shift[i] = -base * p.scale_log2e;
                    m_run[i] = m_new;
                    rescale = rescale || alpha[i] != 1.0f;
                }
                if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
                    for (int n = 0; n < DN; ++n) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) o[n][e] *= alpha[HALF ? 0 : (e >> 1)];
                    }
#pragma unroll
                    for (int i = 0; i < NROW; ++i) l_run[i] *= alpha[i];
                }

                // ---- P = exp2(scale * log2(e) * (S - max)) as the A operand of P V. A probability rounded to 8
                // mantissa bits would cost up to 2^-9 of |p v| per term, which short contexts turn into errors
                // of several 1e-3; P is therefore split into a rounded part and the rounding remainder, which
                // keeps 16 bits of every probability. Half-tile tasks carry the remainder in the idle fragment
                // rows 8-15 (one MMA does both); full tiles issue a second MMA per V fragment.
                uint32_t pa[KT][4], pb[KT][4];
#pragma unroll
                for (int kt = 0; kt < KT; ++kt) {
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        float pv[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                        for (int e = 0; e < 2 * NROW; ++e) {
                            pv[e] = fast_exp2(fmaf(s[2 * kt + h][e], p.scale_log2e, shift[e >> 1]));
                        }
                        l_run[0] += pv[0] + pv[1];
                        if (!HALF) l_run[1] += pv[2] + pv[3];
                        pa[kt][2 * h] = pack2<T>(pv[0], pv[1]);
                        const float2 r01 = unpack2<T>(pa[kt][2 * h]);
                        pb[kt][2 * h] = pack2<T>(pv[0] - r01.x, pv[1] - r01.y);
                        if (HALF) {
                            pa[kt][2 * h + 1] = pb[kt][2 * h];
                        } else {
                            pa[kt][2 * h + 1] = pack2<T>(pv[2], pv[3]);
                            const float2 r23 = unpack2<T>(pa[kt][2 * h + 1]);
                            pb[kt][2 * h + 1] = pack2<T>(pv[2] - r23.x, pv[3] - r23.y);
                        }
                    }
                }

                // ---- O += P V
                if (!(knock & 4))
#pragma unroll
                for (int kt = 0; kt < KT; ++kt) {
#pragma unroll
                    for (int np = 0; np < DN / 2; ++np) {
                        uint32_t b[4];
                        ldmatrix_x4_trans(b, v_addr[np & 3] + ((2 * np) / 8) * G::kBoxBytes +
                                                 ((ps * WT + 16 * kt) / G::kBoxRows) * G::kCopyBytes +
                                                 ((ps * WT + 16 * kt) % G::kBoxRows) * 128);
                        mma_16816<T>(o[2 * np], pa[kt], b[0], b[1]);
                        mma_16816<T>(o[2 * np + 1], pa[kt], b[2], b[3]);
                        if (!HALF) {
                            mma_16816<T>(o[2 * np], pb[kt], b[0], b[1]);
                            mma_16816<T>(o[2 * np + 1], pb[kt], b[2], b[3]);
                        }
                    }
                }

                // ---- release the stage
                if (tile_tok + WT > t_kv_end) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar + 8 * slot);
            }
            stage_counter += t_num_tiles;

            if (debug_bits(p) & 2) {
                __syncwarp();
                if (lane == 0) mbar_arrive(task_empty_bar + 8 * tslot);
                continue;
            }
            if (t_carry & 2u) {
                // The next task of this CTA continues these rows: nothing is merged or published now. This
                // task's template still gets a partial, an empty one (weight zero in every merge).
                if (part == 0 && tq == 0) {
#pragma unroll
                    for (int i = 0; i < NROW; ++i) {
                        const uint32_t row = mt * G::kTileRows + g + 8 * i;
                        const uint32_t row_tok = row / p.heads_per_task;
                        const uint32_t row_head = row % p.heads_per_task;
                        if (!(row_tok < t_num_toks && row_head < t_num_heads)) continue;
                        const uint64_t index =
                            (uint64_t(t_tmpl) * p.num_q_heads + t_head_begin + row_head) * p.max_q_tokens + row_tok;
                        p.partial_sum[index] = 0.0f;
                        p.partial_max[index] = -INFINITY;
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(task_empty_bar + 8 * tslot);
                continue;
            }
            if (HALF) {
#pragma unroll
                for (int n = 0; n < DN; ++n) {
                    o[n][0] += o[n][2];
                    o[n][1] += o[n][3];
                }
            }
            // ---- quad-reduce the exp-sums
#pragma unroll
            for (int i = 0; i < NROW; ++i) {
                l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
                l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
            }

            // ---- the warps park their states in shared memory (fragment order: conflict free) ...
            constexpr int FR = G::kFragRegs;
            float weight[KVW][NROW];
            float inv_l[NROW], m_all[NROW], l_all[NROW];
            if constexpr (KP > 1) {
                // one slot per (KV warp group, row tile); with two warps per group the second parks first and
                // the first folds it into its own state before parking, which halves the buffer
                float* my_slot = merge + (kw * MT + mt) * G::kMergeSlotFloats;
                auto park = [&]() {
#pragma unroll
                    for (int n = 0; n < DN; ++n) {
#pragma unroll
                        for (int e = 0; e < 2 * NROW; ++e) my_slot[(n * 2 * NROW + e) * 32 + lane] = o[n][e];
                    }
#pragma unroll
                    for (int i = 0; i < NROW; ++i) {
                        my_slot[(FR + i) * 32 + lane] = m_run[i];
                        my_slot[(FR + 2 + i) * 32 + lane] = l_run[i];
                    }
                };
                consumer_barrier<1>(NCW * 32);  // the previous task's merge reads are finished
                if (PS == 1 || ps == 1) park();
                if constexpr (PS == 2) {
                    consumer_barrier<3>(NCW * 32);
                    if (ps == 0) {
                        float fa[NROW], fb[NROW];
#pragma unroll
                        for (int i = 0; i < NROW; ++i) {
                            const float m_other = my_slot[(FR + i) * 32 + lane];
                            const float l_other = my_slot[(FR + 2 + i) * 32 + lane];
                            const float m_new = fmaxf(m_run[i], m_other);
                            const float b = m_new == -INFINITY ? 0.0f : m_new;
                            fa[i] = fast_exp2((m_run[i] - b) * p.scale_log2e);
                            fb[i] = fast_exp2((m_other - b) * p.scale_log2e);
                            l_run[i] = l_run[i] * fa[i] + l_other * fb[i];
                            m_run[i] = m_new;
                        }
#pragma unroll
                        for (int n = 0; n < DN; ++n) {
#pragma unroll
                            for (int e = 0; e < 2 * NROW; ++e) {
                                o[n][e] = o[n][e] * fa[e >> 1] + my_slot[(n * 2 * NROW + e) * 32 + lane] * fb[e >> 1];
                            }
                        }
                        park();
                    }
                }
                consumer_barrier<2>(NCW * 32);

                // ---- ... and each thread merges and publishes a slice: n-tiles [part * DN / KP, (part + 1) * DN / KP)
                // of its row tile's fragment, at its own lane position.
#pragma unroll
                for (int i = 0; i < NROW; ++i) {
                    float m_max = -INFINITY;
#pragma unroll
                    for (int k = 0; k < KVW; ++k) {
                        m_max = fmaxf(m_max, merge[(k * MT + mt) * G::kMergeSlotFloats + (FR + i) * 32 + lane]);
                    }
                    const float b = m_max == -INFINITY ? 0.0f : m_max;
                    float l_sum = 0.0f;
#pragma unroll
                    for (int k = 0; k < KVW; ++k) {
                        const float* slot_mem = merge + (k * MT + mt) * G::kMergeSlotFloats;
                        weight[k][i] = fast_exp2((slot_mem[(FR + i) * 32 + lane] - b) * p.scale_log2e);
                        l_sum += slot_mem[(FR + 2 + i) * 32 + lane] * weight[k][i];
                    }
                    m_all[i] = m_max;
                    l_all[i] = l_sum;
                    inv_l[i] = l_sum > 0.0f ? 1.0f / l_sum : 0.0f;
                }
            } else {
                // a single KV warp per row tile publishes straight from its registers
#pragma unroll
                for (int i = 0; i < NROW; ++i) {
                    weight[0][i] = 1.0f;
                    m_all[i] = m_run[i];
                    l_all[i] = l_run[i];
                    inv_l[i] = l_run[i] > 0.0f ? 1.0f / l_run[i] : 0.0f;
                }
            }
            constexpr int NTILES_PER_THREAD = DN / KP;
#pragma unroll
            for (int i = 0; i < NROW; ++i) {
                const uint32_t row = mt * G::kTileRows + g + 8 * i;
                const uint32_t row_tok = row / p.heads_per_task;
                const uint32_t row_head = row % p.heads_per_task;
                if (!(row_tok < t_num_toks && row_head < t_num_heads)) continue;
                const uint32_t head = t_head_begin + row_head;
                const uint64_t index = (uint64_t(t_tmpl) * p.num_q_heads + head) * p.max_q_tokens + row_tok;
#pragma unroll
                for (int nn = 0; nn < NTILES_PER_THREAD; ++nn) {
                    const int n = (KP == 1) ? nn : part * NTILES_PER_THREAD + nn;  // compile-time index when unsplit
                    float v0 = 0.0f, v1 = 0.0f;
                    if constexpr (KP > 1) {
#pragma unroll
                        for (int k = 0; k < KVW; ++k) {
                            const float* slot_mem = merge + (k * MT + mt) * G::kMergeSlotFloats;
                            v0 += weight[k][i] * slot_mem[(n * 2 * NROW + 2 * i) * 32 + lane];
                            v1 += weight[k][i] * slot_mem[(n * 2 * NROW + 2 * i + 1) * 32 + lane];
                        }
                    } else {
                        v0 = o[n][2 * i];
                        v1 = o[n][2 * i + 1];
                    }
                    v0 *= inv_l[i];
                    v1 *= inv_l[i];
                    if (write_final) {
                        T* dst = reinterpret_cast<T*>(p.out) +
                                 (uint64_t(t_tok_begin + row_tok) * p.num_q_heads + head) * D + n * 8 + tq * 2;
                        *reinterpret_cast<uint32_t*>(dst) = pack2<T>(v0, v1);
                    } else {
                        *reinterpret_cast<float2*>(p.partial_out + index * D + n * 8 + tq * 2) = make_float2(v0, v1);
                    }
                }
                if (!write_final && part == 0 && tq == 0) {
                    p.partial_sum[index] = l_all[i];
                    // the running maximum is a raw dot product; publish the natural-log-domain logit (dot * scale)
                    p.partial_max[index] = l_all[i] > 0.0f ? m_all[i] * (p.scale_log2e * 0.6931471805599453f) : -INFINITY;
                }
            }
            // ---- fused reduce: the CTA that publishes the last partial of a (Q range, KV head, head range)
            // group merges the group's partials (they are hot in L2) and writes the final output. Nobody waits:
            // every CTA counts its arrival and moves on; the last one does the merge and re-zeroes the counter.
            if (fused && t_part_count > 1) {
                consumer_barrier<3>(NCW * 32);     // every consumer thread has issued its partial stores
                if (threadIdx.x == 0) {
                    __threadfence();               // cumulative: orders the whole CTA's stores before the count
                    const uint32_t seen = (debug_bits(p) & 256) ? 0u : atomicAdd(p.arrivals + t_group, 1u);
                    const uint32_t last = (seen + 1 == t_part_count && !(debug_bits(p) & 128)) ? 1u : 0u;
                    if (last) p.arrivals[t_group] = 0;
                    *last_flag = last;
                }
                consumer_barrier<3>(NCW * 32);
                if (*last_flag) {
                    __threadfence();
                    reduce_group<T, D>(p, t_tok_begin, t_num_toks, t_head_begin, t_num_heads, t_part_begin, t_part_count,
                                       threadIdx.x, NCW * 32);
                }
            }
            // ---- hand the task slot (descriptor + Q rows) back to the producer
            __syncwarp();
            if (lane == 0) mbar_arrive(task_empty_bar + 8 * tslot);
        }
    }
    __syncthreads();
}

}  // namespace kh
