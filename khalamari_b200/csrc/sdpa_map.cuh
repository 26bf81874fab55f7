// Paged GQA split-KV attention "map" kernel for sm_100a.
//
// One persistent CTA per SM walks a strided list of Map tasks. A task is one map task template
// {q_token_range_index, kv_token_begin, kv_token_end} x one KV head x one Q-head range -- the
// grid cell of the reference's gqa_sdpa_sliced_kv_map / gqa_sdpa_sliced_q_map kernels
// (crates/inference-backend-metal/src/components/metal/gqa_sdpa_sliced_kv_map.metal:36,
//  crates/inference-backend-metal/src/components/metal/gqa_sdpa_sliced_q_map.metal:29).
//
// Data movement: one producer warp streams the task's K and V page chunks from the paged pool
// into a ring of shared-memory stages with TMA tile copies (128-byte swizzle, one mbarrier per
// stage, no multicast). A page chunk [tokens_per_page][head_dim] of one KV head is contiguous in
// the page layout [K/V][Hkv][P][D], so it is one TMA box per 64-element column half.
// Math: consumer warps hold all Q rows of the task -- (Q tokens of the range) x (Q heads of the KV
// group) -- as the M dimension of warp-level tensor-core tiles, so every K/V byte is read from HBM
// once and feeds all of them. S = Q K^T and O += P V run as m16n8k16 MMAs with f32 accumulators;
// the online softmax keeps a running row maximum with quad shuffles. KV stages are dealt round
// robin to KVW "KV warps" per row tile; their (m, l, O) states are merged through shared memory at
// the end of the task and either published as an f32 partial (max, exp-sum, normalised output) or
// written directly as the final output.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace kh {

struct MapParams {
    const void* q;                    // [T][Hq][D] io dtype
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
};

constexpr uint32_t kStatusWaitExpired = 1u;
constexpr uint32_t kStatusPageOutOfPool = 2u;
constexpr uint32_t kWaitLimit = 1u << 24;
constexpr int kMaxPidsPerSegment = 160;  // page ids staged per task segment (2048 tokens of 16 + slack)

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
// wait returns at once and the kernel runs to its end without touching the ring again; the host
// reads the sticky status word.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag,
                                          uint32_t* status) {
    if (*abort_flag) return false;
    for (uint32_t i = 0; i < kWaitLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    *abort_flag = 1;
    atomicOr(status, kStatusWaitExpired);
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int32_t x, int32_t y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
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

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void consumer_barrier(int threads) {
    asm volatile("bar.sync 1, %0;" ::"r"(threads) : "memory");
}

// Compile-time geometry of one kernel instance.
//   D: head dimension (128 or 256). P: tokens per page. MT: 16-row tiles of Q rows per task.
//   KVW: KV warps per row tile. Consumer warps = MT * KVW; one extra warp produces.
template <int D, int P, int MT, int KVW>
struct MapGeometry {
    static constexpr int kStageTokens = (D == 128) ? 32 : 16;
    static constexpr int kBoxRows = (P < kStageTokens) ? P : kStageTokens;
    static constexpr int kBoxesPerPlane = kStageTokens / kBoxRows;  // token boxes per stage
    static constexpr int kColumnHalves = D / 64;                      // 128-byte column groups
    static constexpr int kBoxBytes = kBoxRows * 128;
    static constexpr int kPlaneBytes = kStageTokens * D * 2;
    static constexpr int kStageBytes = 2 * kPlaneBytes;
    static constexpr int kBoxesPerStage = 2 * kBoxesPerPlane * kColumnHalves;
    static constexpr int kConsumerWarps = MT * KVW;
    static constexpr int kThreads = (kConsumerWarps + 1) * 32;
    static constexpr int kQBytes = MT * 16 * D * 2;
    static constexpr int kMergeSlotFloats = (D / 2 + 4) * 32;  // O fragment + (m, l) x 2 rows, per lane
    static constexpr int kMergeSlots = MT * (KVW / 2);
    static constexpr int kMergeBytes = kMergeSlots * kMergeSlotFloats * 4;
    static constexpr int kPidBytes = 2 * kMaxPidsPerSegment * 4;
    static constexpr int kFixedBytes = kQBytes + kMergeBytes + kPidBytes + 512 /* barriers, flags */;
    static constexpr int kSmemLimit = 227 * 1024 - 1024 /* alignment slack */;
    static constexpr int kStagesFit = (kSmemLimit - kFixedBytes) / kStageBytes;
    static constexpr int kStages = kStagesFit > 12 ? 12 : kStagesFit;
    static constexpr int kSmemBytes = kStages * kStageBytes + kFixedBytes + 1024;
    static_assert(kStages >= 3, "shared memory ring too small");
    static_assert(D % 64 == 0 && (P == 8 || P == 16 || P == 32), "unsupported page geometry");
    static_assert((KVW & (KVW - 1)) == 0, "KV warps must be a power of two");
};

struct TaskInfo {
    uint32_t tmpl;
    uint32_t kv_head;
    uint32_t head_begin;   // first Q head of the task (absolute)
    uint32_t num_heads;    // active Q heads in the task
    uint32_t tok_begin;    // first flat Q token
    uint32_t num_toks;     // Q tokens in the range
    uint32_t kv_begin;
    uint32_t kv_end;
    uint32_t req_slot;
    uint32_t tile_begin;   // kv_begin rounded down to a stage boundary
    uint32_t num_tiles;
    bool active;
};

// Decodes flat task index -> template, KV head, head range, and applies the reference kernels'
// early-return rules for padded and inactive templates (gqa_sdpa_sliced_kv_map.metal:56-58,
// gqa_sdpa_sliced_q_map.metal:56-67).
template <int STAGE_TOKENS>
__device__ __forceinline__ TaskInfo decode_task(const MapParams& p, uint32_t task) {
    TaskInfo t;
    const uint32_t cells = p.num_kv_heads * p.head_ranges;
    t.tmpl = task / cells;
    const uint32_t cell = task % cells;
    t.kv_head = cell / p.head_ranges;
    const uint32_t range = cell % p.head_ranges;
    t.head_begin = t.kv_head * p.group + range * p.heads_per_task;
    t.num_heads = min(p.heads_per_task, p.group - range * p.heads_per_task);
    t.active = false;
    t.tok_begin = t.num_toks = t.kv_begin = t.kv_end = t.req_slot = t.tile_begin = t.num_tiles = 0;
    const uint32_t q_range = p.templates[t.tmpl * 3];
    if (p.q_ranges == nullptr) {
        if (q_range >= p.num_active_tokens) return t;
        t.tok_begin = q_range;
        t.num_toks = 1;
    } else {
        if (q_range >= p.num_active_q_tiles) return t;
        const uint32_t begin = p.q_ranges[q_range * 2];
        const uint32_t end = p.q_ranges[q_range * 2 + 1];
        if (begin >= p.num_active_tokens || end > p.num_active_tokens || end <= begin) return t;
        t.tok_begin = begin;
        t.num_toks = min(end - begin, p.max_q_tokens);
    }
    t.kv_begin = p.templates[t.tmpl * 3 + 1];
    t.kv_end = p.templates[t.tmpl * 3 + 2];
    t.req_slot = p.req_slots[t.tok_begin];
    t.active = true;
    if (t.kv_end > t.kv_begin) {
        t.tile_begin = t.kv_begin / STAGE_TOKENS * STAGE_TOKENS;
        t.num_tiles = (t.kv_end - t.tile_begin + STAGE_TOKENS - 1) / STAGE_TOKENS;
    }
    return t;
}

template <typename T, int D, int P, int MT, int KVW>
__global__ void __launch_bounds__(MapGeometry<D, P, MT, KVW>::kThreads, 1)
sdpa_map_kernel(const __grid_constant__ CUtensorMap kv_map, const MapParams p) {
    using G = MapGeometry<D, P, MT, KVW>;
    constexpr int ST = G::kStageTokens;
    constexpr int NS = G::kStages;
    constexpr int NCW = G::kConsumerWarps;
    constexpr int NT = ST / 8;       // S n-tiles (8 KV tokens each) per stage
    constexpr int KT = ST / 16;      // PV k-tiles (16 KV tokens each) per stage
    constexpr int DK = D / 16;       // QK k-steps
    constexpr int DN = D / 8;        // O n-tiles

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = smem;
    uint8_t* q_smem = ring + NS * G::kStageBytes;
    float* merge = reinterpret_cast<float*>(q_smem + G::kQBytes);
    uint32_t* pid_smem = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(merge) + G::kMergeBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(pid_smem) + G::kPidBytes);
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + 2 * NS);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t full_bar = smem_addr(bars);
    const uint32_t empty_bar = smem_addr(bars + NS);

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, MT);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    const uint32_t total_tasks = p.num_templates * p.num_kv_heads * p.head_ranges;
    const uint32_t rows_per_page_plane = P;  // rows of one (page, plane, head) chunk

    if (warp == NCW) {
        // ------------------------------ producer warp -----------------------------------------
        uint32_t stage_counter = 0;
        uint32_t task = blockIdx.x;
        int buf = 0;
        TaskInfo cur = task < total_tasks ? decode_task<ST>(p, task) : TaskInfo{};
        if (task >= total_tasks) cur.active = false;

        // Stages the page ids of pages [first_page, first_page + count) of a task into pid_smem[buf].
        auto stage_pids = [&](const TaskInfo& t, uint32_t first_page, uint32_t count, int which) {
            const uint64_t base = (uint64_t(t.req_slot) * p.num_gqa_layers + p.layer_index) * p.pages_per_request_layer;
            for (uint32_t i = lane; i < count; i += 32) {
                const uint32_t dst = smem_addr(pid_smem + which * kMaxPidsPerSegment + i);
                const uint32_t* src = p.page_ids + base + first_page + i;
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        };
        auto task_pages = [&](const TaskInfo& t, uint32_t& first_page, uint32_t& num_pages) {
            first_page = t.tile_begin / P;
            num_pages = t.num_tiles == 0 ? 0 : (t.kv_end + P - 1) / P - first_page;
        };

        if (cur.active && cur.num_tiles > 0) {
            uint32_t fp, np;
            task_pages(cur, fp, np);
            stage_pids(cur, fp, min(np, uint32_t(kMaxPidsPerSegment)), buf);
        }
        while (task < total_tasks) {
            const uint32_t next_task = task + gridDim.x;
            TaskInfo nxt{};
            nxt.active = false;
            if (next_task < total_tasks) nxt = decode_task<ST>(p, next_task);
            // current task's first segment is in flight or landed; wait for it, then prefetch the next task's.
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncwarp();
            if (nxt.active && nxt.num_tiles > 0) {
                uint32_t fp, np;
                task_pages(nxt, fp, np);
                stage_pids(nxt, fp, min(np, uint32_t(kMaxPidsPerSegment)), buf ^ 1);
            }
            if (cur.active && cur.num_tiles > 0) {
                uint32_t first_page, num_pages;
                task_pages(cur, first_page, num_pages);
                uint32_t seg_first = first_page;  // first page whose id is staged in pid_smem[buf]
                uint32_t seg_count = min(num_pages, uint32_t(kMaxPidsPerSegment));
                for (uint32_t tile = 0; tile < cur.num_tiles; ++tile, ++stage_counter) {
                    const uint32_t tile_tok = cur.tile_begin + tile * ST;
                    // Page span of this stage; restage ids synchronously for very long tasks.
                    const uint32_t last_page_needed = (min(tile_tok + ST, cur.kv_end) - 1) / P;
                    if (last_page_needed >= seg_first + seg_count) {
                        // The prefetched segment of the next task shares the copy queue: drain it first.
                        asm volatile("cp.async.wait_group 0;" ::: "memory");
                        __syncwarp();
                        seg_first = tile_tok / P;
                        seg_count = min(first_page + num_pages - seg_first, uint32_t(kMaxPidsPerSegment));
                        stage_pids(cur, seg_first, seg_count, buf);
                        asm volatile("cp.async.wait_group 0;" ::: "memory");
                        __syncwarp();
                    }
                    const uint32_t slot = stage_counter % NS;
                    const uint32_t phase = (stage_counter / NS) & 1;
                    const bool ok = mbar_wait(empty_bar + 8 * slot, phase ^ 1, abort_flag, p.status);
                    if (!ok) continue;
                    // Which boxes hold at least one token below kv_end.
                    uint32_t boxes_needed = 0;
#pragma unroll
                    for (int b = 0; b < G::kBoxesPerPlane; ++b) {
                        if (tile_tok + b * G::kBoxRows < cur.kv_end) ++boxes_needed;
                    }
                    if (lane == 0) {
                        mbar_arrive_expect_tx(full_bar + 8 * slot, boxes_needed * 2 * G::kColumnHalves * G::kBoxBytes);
                    }
                    __syncwarp();
                    if (lane < G::kBoxesPerStage) {
                        // lane -> (plane, token box, column half)
                        const int half = lane % G::kColumnHalves;
                        const int box = (lane / G::kColumnHalves) % G::kBoxesPerPlane;
                        const int plane = lane / (G::kColumnHalves * G::kBoxesPerPlane);
                        const uint32_t tok = tile_tok + box * G::kBoxRows;
                        if (tok < cur.kv_end) {
                            const uint32_t page_index = tok / P;
                            const uint32_t pid = pid_smem[buf * kMaxPidsPerSegment + (page_index - seg_first)];
                            if (pid >= p.pool_pages) atomicOr(p.status, kStatusPageOutOfPool);
                            const uint64_t row = ((uint64_t(pid) * 2 + plane) * p.num_kv_heads + cur.kv_head) *
                                                     rows_per_page_plane + tok % P;
                            const uint32_t dst = smem_addr(ring + slot * G::kStageBytes + plane * G::kPlaneBytes +
                                                           (box * G::kColumnHalves + half) * G::kBoxBytes);
                            tma_load_2d(dst, &kv_map, half * 64, static_cast<int32_t>(row), full_bar + 8 * slot);
                        }
                    }
                }
            }
            cur = nxt;
            task = next_task;
            buf ^= 1;
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        // Abort path only: copies already issued may still be landing; wait (bounded) for each stage's
        // last issued phase before the CTA may retire.
        if (*abort_flag) {
            for (uint32_t back = 0; back < uint32_t(NS) && back < stage_counter; ++back) {
                const uint32_t c = stage_counter - 1 - back;
                for (uint32_t i = 0; i < kWaitLimit; ++i) {
                    if (mbar_try_wait(full_bar + 8 * (c % NS), (c / NS) & 1)) break;
                }
            }
        }
    } else {
        // ------------------------------ consumer warps ----------------------------------------
        const int mt = warp % MT;   // row tile
        const int kw = warp / MT;   // KV warp index within the row tile
        const int ctid = threadIdx.x;
        const int g = lane >> 2;    // fragment row group
        const int tq = lane & 3;    // thread in quad
        uint32_t stage_counter = 0;
        const T* q_global = reinterpret_cast<const T*>(p.q);

        for (uint32_t task = blockIdx.x; task < total_tasks; task += gridDim.x) {
            const TaskInfo t = decode_task<ST>(p, task);
            if (!t.active) continue;

            // ---- stage Q rows: row = tok_local * heads_per_task + head_local, 16-byte chunks, XOR swizzle
            for (int idx = ctid; idx < MT * 16 * (D / 8); idx += NCW * 32) {
                const int row = idx / (D / 8);
                const int chunk = idx % (D / 8);
                const uint32_t tok_local = row / p.heads_per_task;
                const uint32_t head_local = row % p.heads_per_task;
                uint4 value = make_uint4(0, 0, 0, 0);
                if (tok_local < t.num_toks && head_local < t.num_heads) {
                    const T* src = q_global +
                                   (uint64_t(t.tok_begin + tok_local) * p.num_q_heads + t.head_begin + head_local) * D +
                                   chunk * 8;
                    value = *reinterpret_cast<const uint4*>(src);
                }
                const int phys = (chunk & ~7) | ((chunk ^ row) & 7);
                *reinterpret_cast<uint4*>(q_smem + row * (D * 2) + phys * 16) = value;
            }
            consumer_barrier(NCW * 32);

            // ---- per-thread row bounds: rows g and g + 8 of row tile mt
            uint32_t lo[2], hi[2];
            bool row_valid[2];
            uint32_t row_tok[2], row_head[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const uint32_t row = mt * 16 + g + 8 * i;
                row_tok[i] = row / p.heads_per_task;
                row_head[i] = row % p.heads_per_task;
                row_valid[i] = row_tok[i] < t.num_toks && row_head[i] < t.num_heads;
                lo[i] = hi[i] = 0;
                if (row_valid[i]) {
                    uint32_t vb = 0, ve = 0xffffffffu;
                    if (p.visible != nullptr) {
                        vb = p.visible[(t.tok_begin + row_tok[i]) * 2];
                        ve = p.visible[(t.tok_begin + row_tok[i]) * 2 + 1];
                    }
                    lo[i] = max(vb, t.kv_begin);
                    hi[i] = min(ve, t.kv_end);
                    if (hi[i] < lo[i]) hi[i] = lo[i];
                }
            }

            float o[DN][4];
#pragma unroll
            for (int n = 0; n < DN; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
            float m_run[2] = {-INFINITY, -INFINITY};
            float l_run[2] = {0.0f, 0.0f};

            // ldmatrix lane roles
            const int lm_mat = lane >> 3;  // which of the four 8x8 matrices this lane addresses
            const int lm_row = lane & 7;
            const uint32_t q_tile = smem_addr(q_smem) + mt * 16 * (D * 2);

            for (uint32_t tile = kw; tile < t.num_tiles; tile += KVW) {
                const uint32_t counter = stage_counter + tile;
                const uint32_t slot = counter % NS;
                const uint32_t phase = (counter / NS) & 1;
                const bool ok = mbar_wait(full_bar + 8 * slot, phase, abort_flag, p.status);
                if (!ok) continue;
                const uint32_t tile_tok = t.tile_begin + tile * ST;
                const uint32_t k_base = smem_addr(ring + slot * G::kStageBytes);
                const uint32_t v_base = k_base + G::kPlaneBytes;

                // Rows of tokens at or past kv_end may never have been written (or loaded): clear them in V
                // so that a zero probability times stale bits cannot produce NaN.
                if (tile_tok + ST > t.kv_end) {
                    const uint32_t first_bad = t.kv_end - tile_tok;
                    for (uint32_t idx = first_bad * (D / 8) + lane; idx < uint32_t(ST) * (D / 8); idx += 32) {
                        const uint32_t r = idx / (D / 8);
                        const uint32_t c = idx % (D / 8);
                        const uint32_t box = r / G::kBoxRows;
                        const uint32_t addr = v_base + (box * G::kColumnHalves + c / 8) * G::kBoxBytes +
                                              (r % G::kBoxRows) * 128 + (c % 8) * 16;
                        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
                    }
                    __syncwarp();
                }

                // ---- S = Q K^T
                float s[NT][4];
#pragma unroll
                for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
                for (int kk = 0; kk < DK; ++kk) {
                    uint32_t a[4];
                    {
                        const int row = (lm_mat & 1) * 8 + lm_row;
                        const int chunk = 2 * kk + (lm_mat >> 1);
                        const int phys = (chunk & ~7) | ((chunk ^ row) & 7);
                        ldmatrix_x4(a, q_tile + row * (D * 2) + phys * 16);
                    }
#pragma unroll
                    for (int jp = 0; jp < NT / 2; ++jp) {
                        uint32_t b[4];
                        const int tok = (2 * jp + (lm_mat >> 1)) * 8 + lm_row;  // token within stage
                        const int chunk = 2 * kk + (lm_mat & 1);                // 16-byte chunk along D
                        const int box = tok / G::kBoxRows;
                        const int r = tok % G::kBoxRows;
                        const uint32_t addr = k_base + (box * G::kColumnHalves + chunk / 8) * G::kBoxBytes + r * 128 +
                                              (((chunk & 7) ^ (r & 7)) << 4);
                        ldmatrix_x4(b, addr);
                        mma_16816<T>(s[2 * jp], a, b[0], b[1]);
                        mma_16816<T>(s[2 * jp + 1], a, b[2], b[3]);
                    }
                }

                // ---- mask, scale, running maximum
                float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < NT; ++j) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int i = e >> 1;
                        const uint32_t tok = tile_tok + j * 8 + tq * 2 + (e & 1);
                        const bool visible = tok >= lo[i] && tok < hi[i];
                        const float value = visible ? s[j][e] * p.scale_log2e : -INFINITY;
                        s[j][e] = value;
                        tile_max[i] = fmaxf(tile_max[i], value);
                    }
                }
                float alpha[2], base[2];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 1));
                    tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 2));
                    const float m_new = fmaxf(m_run[i], tile_max[i]);
                    base[i] = m_new == -INFINITY ? 0.0f : m_new;
                    // nothing has been accumulated while the running maximum is -inf: no rescale needed
                    alpha[i] = m_run[i] == -INFINITY ? 1.0f : fast_exp2(m_run[i] - base[i]);
                    m_run[i] = m_new;
                }
                const bool rescale = (alpha[0] != 1.0f) || (alpha[1] != 1.0f);
                if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
                    for (int n = 0; n < DN; ++n) {
                        o[n][0] *= alpha[0];
                        o[n][1] *= alpha[0];
                        o[n][2] *= alpha[1];
                        o[n][3] *= alpha[1];
                    }
                    l_run[0] *= alpha[0];
                    l_run[1] *= alpha[1];
                }

                // ---- P = exp2(S - max), packed as the A operand of P V
                uint32_t pa[KT][4];
#pragma unroll
                for (int kt = 0; kt < KT; ++kt) {
                    float pv[2][4];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            pv[h][e] = fast_exp2(s[2 * kt + h][e] - base[e >> 1]);
                        }
                        l_run[0] += pv[h][0] + pv[h][1];
                        l_run[1] += pv[h][2] + pv[h][3];
                    }
                    pa[kt][0] = pack2<T>(pv[0][0], pv[0][1]);
                    pa[kt][1] = pack2<T>(pv[0][2], pv[0][3]);
                    pa[kt][2] = pack2<T>(pv[1][0], pv[1][1]);
                    pa[kt][3] = pack2<T>(pv[1][2], pv[1][3]);
                }

                // ---- O += P V
#pragma unroll
                for (int kt = 0; kt < KT; ++kt) {
#pragma unroll
                    for (int np = 0; np < DN / 2; ++np) {
                        uint32_t b[4];
                        const int tok = kt * 16 + (lm_mat & 1) * 8 + lm_row;
                        const int chunk = 2 * np + (lm_mat >> 1);
                        const int box = tok / G::kBoxRows;
                        const int r = tok % G::kBoxRows;
                        const uint32_t addr = v_base + (box * G::kColumnHalves + chunk / 8) * G::kBoxBytes + r * 128 +
                                              (((chunk & 7) ^ (r & 7)) << 4);
                        ldmatrix_x4_trans(b, addr);
                        mma_16816<T>(o[2 * np], pa[kt], b[0], b[1]);
                        mma_16816<T>(o[2 * np + 1], pa[kt], b[2], b[3]);
                    }
                }

                // ---- release the stage
                if (tile_tok + ST > t.kv_end) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar + 8 * slot);
            }
            stage_counter += t.num_tiles;

            // ---- quad-reduce the exp-sums
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
                l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
            }

            // ---- tree-merge the KV warps of this row tile through shared memory (fragment order)
#pragma unroll
            for (int step = KVW / 2; step >= 1; step /= 2) {
                float* slot_mem = merge + (mt * (KVW / 2) + (kw % step)) * G::kMergeSlotFloats;
                if (kw >= step && kw < 2 * step) {
#pragma unroll
                    for (int n = 0; n < DN; ++n) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) slot_mem[(n * 4 + e) * 32 + lane] = o[n][e];
                    }
                    slot_mem[(DN * 4 + 0) * 32 + lane] = m_run[0];
                    slot_mem[(DN * 4 + 1) * 32 + lane] = m_run[1];
                    slot_mem[(DN * 4 + 2) * 32 + lane] = l_run[0];
                    slot_mem[(DN * 4 + 3) * 32 + lane] = l_run[1];
                }
                consumer_barrier(NCW * 32);
                if (kw < step) {
                    float fa[2], fb[2];
#pragma unroll
                    for (int i = 0; i < 2; ++i) {
                        const float m_other = slot_mem[(DN * 4 + i) * 32 + lane];
                        const float l_other = slot_mem[(DN * 4 + 2 + i) * 32 + lane];
                        const float m_new = fmaxf(m_run[i], m_other);
                        const float b = m_new == -INFINITY ? 0.0f : m_new;
                        fa[i] = fast_exp2(m_run[i] - b);
                        fb[i] = fast_exp2(m_other - b);
                        l_run[i] = l_run[i] * fa[i] + l_other * fb[i];
                        m_run[i] = m_new;
                    }
#pragma unroll
                    for (int n = 0; n < DN; ++n) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            o[n][e] = o[n][e] * fa[e >> 1] + slot_mem[(n * 4 + e) * 32 + lane] * fb[e >> 1];
                        }
                    }
                }
                consumer_barrier(NCW * 32);
            }
            if (KVW == 1) consumer_barrier(NCW * 32);  // Q tile reuse fence when there is no merge

            // ---- publish
            if (kw == 0) {
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    if (!row_valid[i]) continue;
                    const float inv = l_run[i] > 0.0f ? 1.0f / l_run[i] : 0.0f;
                    const uint32_t head = t.head_begin + row_head[i];
                    if (p.direct) {
                        T* dst = reinterpret_cast<T*>(p.out) +
                                 (uint64_t(t.tok_begin + row_tok[i]) * p.num_q_heads + head) * D + tq * 2;
#pragma unroll
                        for (int n = 0; n < DN; ++n) {
                            const uint32_t packed = pack2<T>(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
                            *reinterpret_cast<uint32_t*>(dst + n * 8) = packed;
                        }
                    } else {
                        const uint64_t index = (uint64_t(t.tmpl) * p.num_q_heads + head) * p.max_q_tokens + row_tok[i];
                        float* dst = p.partial_out + index * D + tq * 2;
#pragma unroll
                        for (int n = 0; n < DN; ++n) {
                            *reinterpret_cast<float2*>(dst + n * 8) = make_float2(o[n][2 * i] * inv, o[n][2 * i + 1] * inv);
                        }
                        if (tq == 0) {
                            p.partial_sum[index] = l_run[i];
                            // the running maximum lives in the log2 domain of scale * log2(e); publish natural log
                            p.partial_max[index] = l_run[i] > 0.0f ? m_run[i] * 0.6931471805599453f : -INFINITY;
                        }
                    }
                }
            }
        }
    }
    __syncthreads();
}

}  // namespace kh
