// SlicedQ map / direct kernel for tasks of up to 128 (Q token, Q head) rows on the 5th-generation tensor
// cores: tcgen05.mma with the accumulators in tensor memory. Same task ABI, rings, task warp and stream warp as
// sdpa_map_kernel (sdpa_map.cuh); only the consumers differ.
//
//   S = Q K^T   tcgen05.mma kind::f16, M = 128 rows, N = 48 KV tokens, K = 16 head-dim elements per instruction.
//               A = the Q tile in tensor memory (copied there once per task). B = K rows in shared memory, K-major
//               with the 128-byte swizzle exactly as the TMA copies leave them; one instruction takes row group g
//               (8 token rows) of each of the stage's six pages, the only uniform stride 16-token pages offer.
//               A stage (96 tokens) is therefore worked on as two half-stages of 48 scores: row groups 0 and 1.
//               Stage size is a trade: an instruction costs about the same tensor-pipe cycles for N = 32, 48 and
//               64, so more pages per stage mean fewer cycles per token, but the ring must hold three stages for
//               the copies of a stage to start early enough, and three 8-page stages do not fit beside the Q
//               tiles. (Measured on the prefill workload: 4 pages x 4 slots 22.3 ms; 8 pages x 2 slots 22.4 ms,
//               16.9 ms without copies; boxes smaller than a whole page - 4 KB or 2 KB copies, which would allow
//               other layouts - 26 ms.)
//   P           eight softmax warps in two groups, one per half-stage (row group), one thread per row: tcgen05.ld
//               brings the thread its row's 48 scores, so the row maximum and sum need no shuffles. P goes back to
//               tensor memory as packed 16-bit pairs of the Q/output type (A and B operands of one MMA must share
//               their type); bf16 probabilities are followed by their rounding remainder, as in the warp-level kernel.
//   O += P V    A = P from tensor memory, B = the V rows in shared memory, MN-major (V is stored
//               [token][head dim], the head dim being the contiguous N dimension), N = 128, K = 16.
// The running maximum is updated lazily: O (in tensor memory) is rescaled only when a row's maximum grows by more
// than 2^8, so the common stage costs two tensor-memory loads and four stores per thread.
//
// Warps: 0-7 softmax and epilogue (two groups of four), 8 Q K^T issue (one thread), 9 stream warp (K/V copies),
// 10 task warp, 11 P V issue (one thread).
// Every wait is bounded (mbar_wait); tensor memory is allocated once and freed on every exit path.
#pragma once

#include "sdpa_map.cuh"

namespace kh {

template <int D, int P>
struct TcGeometry {
    static_assert(D == 128 && P == 16, "the tensor-memory instance is built for head_dim 128 and 16-token pages");
    static constexpr int kPagesPerStage = 6;
    static constexpr int kStageTokens = 16 * kPagesPerStage;  // Q K^T runs with N = 8 x pages (row group g of every page)
    static constexpr int kScoreTokens = 8 * kPagesPerStage;   // scores of a half-stage: one row group of all pages
    static_assert(kScoreTokens % 16 == 0 && kScoreTokens <= 64, "a half-stage is a whole number of 16-token chunks");
    static constexpr int kBoxRows = 16;
    static constexpr int kBoxesPerPlane = kStageTokens / kBoxRows;
    static constexpr int kColumnHalves = D / 64;
    static constexpr int kBoxBytes = kBoxRows * 128;
    static constexpr int kPlaneBoxBytes = kColumnHalves * kBoxBytes;
    static constexpr int kCopyBytes = 2 * kPlaneBoxBytes;
    static constexpr int kStageBytes = kBoxesPerPlane * kCopyBytes;
    static constexpr int kQRows = 128;
    static constexpr int kQBytes = kQRows * D * 2;
    static constexpr int kTaskSlots = 2;
    static constexpr int kSoftmaxWarps = 8;  // two groups of four; group w takes the stages of parity w
    static constexpr int kThreads = (kSoftmaxWarps + 4) * 32;  // + Q K^T issue, stream, task, P V issue
    static constexpr int kPidBytes = kTaskSlots * kMaxPidsPerSegment * 4;
    static constexpr int kTaskBytes = kTaskSlots * static_cast<int>(sizeof(TaskSlot));
    static constexpr int kFixedBytes = kTaskSlots * kQBytes + kPidBytes + kTaskBytes + 3072;  // barriers, row maxima and sums
    static constexpr int kSmemLimit = 227 * 1024 - 1024;
    static constexpr int kStagesFit = (kSmemLimit - kFixedBytes) / kStageBytes;
    static constexpr int kStages = kStagesFit > 12 ? 12 : kStagesFit;
    static constexpr int kSmemBytes = kStages * kStageBytes + kFixedBytes + 1024;
    static constexpr uint32_t kTmemColumns = 512;  // O 128 | S 2 x 64 | P 2 x (32 rounded + 32 remainder) | Q 2 x 64
    static_assert(kStages >= 3, "shared memory ring too small");
};

__device__ __forceinline__ uint64_t umma_smem_desc(uint32_t addr, uint32_t leading_bytes, uint32_t stride_bytes) {
    // start address, leading-dimension and stride-dimension byte offsets in 16-byte units, descriptor version 1,
    // 128-byte swizzle
    return uint64_t((addr >> 4) & 0x3fffu) | (uint64_t((leading_bytes >> 4) & 0x3fffu) << 16) |
           (uint64_t((stride_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ void umma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p; }"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

__device__ __forceinline__ void umma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{ .reg .pred p; setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p; }"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}

// Arrives on `bar` once every tcgen05 operation this thread issued before has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t (&r)[32], uint32_t taddr) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}

__device__ __forceinline__ void tmem_ld16(uint32_t (&r)[16], uint32_t taddr) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}

// Results of a tensor-memory load may be used only after this.
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
          "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
          "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
          "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <typename T>
__device__ __forceinline__ constexpr uint32_t umma_format();
template <>
__device__ __forceinline__ constexpr uint32_t umma_format<__half>() { return 0u; }
template <>
__device__ __forceinline__ constexpr uint32_t umma_format<__nv_bfloat16>() { return 1u; }

template <typename T, int D, int P>
__global__ void __launch_bounds__(TcGeometry<D, P>::kThreads, 1)
sdpa_tc_kernel(const __grid_constant__ CUtensorMap kv_map, const __grid_constant__ CUtensorMap q_map, const MapParams p) {
    using G = TcGeometry<D, P>;
    constexpr int ST = G::kStageTokens;
    constexpr int SC = G::kScoreTokens;
    constexpr int NS = G::kStages;
    constexpr int TQ = G::kTaskSlots;
    constexpr int NSW = G::kSoftmaxWarps;
    constexpr float kRescaleLog2 = 8.0f;  // O is rescaled only when a row maximum grows by more than 2^8
    // bf16 probabilities carry their rounding remainder in a second MMA; f16 probabilities (11 significant bits) do not
    constexpr bool kRemainder = std::is_same<T, __nv_bfloat16>::value;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = smem;
    uint8_t* q_ring = ring + NS * G::kStageBytes;
    uint32_t* pid_smem = reinterpret_cast<uint32_t*>(q_ring + TQ * G::kQBytes);
    TaskSlot* task_ring = reinterpret_cast<TaskSlot*>(reinterpret_cast<uint8_t*>(pid_smem) + G::kPidBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(task_ring) + G::kTaskBytes);
    constexpr int kNumBars = 2 * NS + 3 * TQ + 17;
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + kNumBars);
    uint32_t* tmem_slot = const_cast<uint32_t*>(abort_flag) + 3;
    volatile float* row_max = reinterpret_cast<volatile float*>(tmem_slot + 1);  // [128] maximum per row of the tile
    volatile float* row_sum = row_max + 128;                                     // [2][128] each group's row sum
    // [2][4] per probability buffer and softmax warp: the half-stage's rounding remainders matter (see below)
    volatile uint32_t* remainder_flag = reinterpret_cast<volatile uint32_t*>(row_sum + 256);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t full_bar = smem_addr(bars);
    const uint32_t empty_bar = smem_addr(bars + NS);
    const uint32_t task_full_bar = smem_addr(bars + 2 * NS);
    const uint32_t task_empty_bar = smem_addr(bars + 2 * NS + TQ);
    const uint32_t stream_full_bar = smem_addr(bars + 2 * NS + 2 * TQ);
    const uint32_t s_full_bar = smem_addr(bars + 2 * NS + 3 * TQ);       // [2] scores of a stage are in tensor memory
    const uint32_t s_free_bar = smem_addr(bars + 2 * NS + 3 * TQ + 2);   // [2] the softmax warps have read them
    const uint32_t p_full_bar = smem_addr(bars + 2 * NS + 3 * TQ + 4);   // [2] probabilities of a stage are stored
    const uint32_t pv_done_bar = smem_addr(bars + 2 * NS + 3 * TQ + 6);  // [2] the stage's P V products completed
    const uint32_t o_free_bar = smem_addr(bars + 2 * NS + 3 * TQ + 8);   // the epilogue has read O
    const uint32_t drain_bar = smem_addr(bars + 2 * NS + 3 * TQ + 15);   // [2] every tcgen05 operation of an issuing thread completed
    const uint32_t q_ready_bar = smem_addr(bars + 2 * NS + 3 * TQ + 9);  // [2] a task's Q tile is in tensor memory
    const uint32_t decided_bar = smem_addr(bars + 2 * NS + 3 * TQ + 11); // [2] a group fixed the row maxima of its stage
    const uint32_t epilogue_bar = smem_addr(bars + 2 * NS + 3 * TQ + 13); // [2] task-end hand-offs between the groups

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);  // one tcgen05.commit per stage
        }
        for (int s = 0; s < TQ; ++s) {
            mbar_init(task_full_bar + 8 * s, p.visible != nullptr ? 33 : 1);
            mbar_init(task_empty_bar + 8 * s, NSW + 3);  // softmax warps, the stream warp, the two issuing threads
            mbar_init(q_ready_bar + 8 * s, NSW);
            mbar_init(stream_full_bar + 8 * s, 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(s_full_bar + 8 * s, 1);
            mbar_init(s_free_bar + 8 * s, 4);   // the four warps of the group that owns the buffer
            mbar_init(p_full_bar + 8 * s, 4);
            mbar_init(pv_done_bar + 8 * s, 1);
            mbar_init(decided_bar + 8 * s, 4);
            mbar_init(epilogue_bar + 8 * s, NSW);
        }
        mbar_init(o_free_bar, NSW);
        mbar_init(drain_bar, 1);
        mbar_init(drain_bar + 8, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = threadIdx.x; i < TQ * G::kQBytes / 16; i += G::kThreads) {
        reinterpret_cast<uint4*>(q_ring)[i] = make_uint4(0, 0, 0, 0);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)),
                     "r"(G::kTmemColumns)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tmem_fence_before();
    __syncthreads();
    tmem_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_o = tmem_base;
    // A stage is worked on as two half-stages: half-stage gr holds row group gr (token rows 8 gr .. 8 gr + 7) of
    // each of the stage's pages, whose 8-row groups lie one page copy apart in shared memory (a uniform stride,
    // which is what the operand descriptor can express). Column c of half-stage gr's scores is KV token
    // tile_tok + 16 * (c / 8) + 8 * gr + c % 8. Half-stage gr uses score buffer gr, probability buffer gr and
    // softmax group gr; with G the running stage number its barrier phases have parity G & 1, and the running
    // half-stage number is 2 G + gr.
    const uint32_t tmem_s = tmem_base + 128;  // + 64 * buffer
    const uint32_t tmem_p = tmem_base + 256;  // + 64 * buffer (+ 32 for the remainder) + 8 * (16-token chunk)
    const uint32_t tmem_q = tmem_base + 384;  // + 64 * task slot: the Q tile, 16-bit pairs, 8 columns per k-step

    // A kernel launched behind this one with programmatic stream serialization (the reducer) may be scheduled as
    // this kernel's blocks retire; it waits for this kernel's completion itself. Only where this block's shared
    // memory leaves no room for a reducer block (12 KB) beside it: reducer blocks that became resident next to a
    // still-running map block cost the one-sequence workload 8 us per step.
    if constexpr (G::kSmemBytes + 14 * 1024 > 228 * 1024) {
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    }
    const ActiveCounts active = resolve_active(p);
    const uint32_t total_tasks = active.templates * p.num_kv_heads * p.head_ranges;
    // Tasks are dealt round-robin (task i to CTA i mod grid), not in contiguous runs: the CTAs then work on
    // neighbouring tasks at any moment - Q tiles of the same sequence over the same K/V rows - so the rows one CTA
    // pulls from HBM are L2 hits for the others. A chunked-prefill batch streams every sequence's K/V once per Q tile
    // (tens of GB per step through L2); contiguous runs spread the CTAs over all sequences at once and the working
    // set (hundreds of MB) no longer fits the 126 MB L2. There are tens of tasks per CTA, so the deal balances.
    // The deal walks the tasks KV head by KV head (cell-major): at any moment the grid reads one or two K/V streams.
    const bool balanced = false;

    ProducerContext producer{};
    producer.ring = ring;
    producer.cell_major = true;
    producer.q_ring = q_ring;
    producer.pid_smem = pid_smem;
    producer.task_ring = task_ring;
    producer.full_bar = full_bar;
    producer.empty_bar = empty_bar;
    producer.task_full_bar = task_full_bar;
    producer.task_empty_bar = task_empty_bar;
    producer.stream_full_bar = stream_full_bar;
    producer.abort_flag = abort_flag;
    producer.task_base = blockIdx.x;
    producer.task_step = gridDim.x;
    producer.task_limit = total_tasks;
    producer.balanced = balanced;
    producer.allow_carry = false;  // the running state lives in tensor memory and is published per task
    producer.active = active;
    producer.lane = lane;

    // Registers follow the work: the softmax warps (two warpgroups) hold a row's 64 scores and grow to 208 registers,
    // the warpgroup of the two issuing threads, the stream warp and the task warp shrinks to 80.
    if (warp >= NSW) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 80;");
    if (warp == NSW + 2) {
        run_task_warp<G, P>(p, q_map, producer);
    } else if (warp == NSW + 1) {
        run_stream_warp<G, P>(p, kv_map, producer);
    } else if (warp == NSW) {
        // ------------------------------ Q K^T issue (one thread) -------------------------------
        // tcgen05.mma is issued by single threads. Two of them share the work - this one the score products, the
        // next warp's the P V products - because one thread's issue rate (descriptor arithmetic, waits, about a
        // hundred cycles per instruction) was what bounded the kernel. Everything the two need from each other
        // goes through the softmax warps' barriers, so no ordering between the two instruction streams is assumed.
        if (lane == 0) {
            constexpr uint32_t kFormat = umma_format<T>();
            // D f32; A, B 16-bit; M = 128, N = 8 x pages, both operands K-major
            const uint32_t idesc_qk =
                (1u << 4) | (kFormat << 7) | (kFormat << 10) | ((uint32_t(SC) >> 3) << 17) | ((128u >> 4) << 24);
            // descriptor of a K operand at byte address 0 (stride between 8-row groups: one page copy); shared
            // memory addresses are below 2^18, so the 14-bit address field is a plain sum
            const uint64_t k_desc0 = umma_smem_desc(0, 16, G::kCopyBytes);
            const uint32_t ring_addr = smem_addr(ring);
            uint32_t stage_base = 0;  // stages of earlier tasks
            bool ok = true;
            for (uint32_t taken = 0; ok; ++taken) {
                const uint32_t tslot = taken % TQ;
                if (!mbar_wait(task_full_bar + 8 * tslot, (taken / TQ) & 1, abort_flag, p)) break;
                const TaskSlot* ts = task_ring + tslot;
                if (ts->done) break;
                const uint32_t num_tiles = ts->num_tiles;
                if (!mbar_wait(q_ready_bar + 8 * tslot, (taken / TQ) & 1, abort_flag, p)) break;
                const uint32_t q_tmem = tmem_q + 64 * tslot;
                for (uint32_t i = 0; i < num_tiles && ok; ++i) {
                    const uint32_t g = stage_base + i;
                    const uint32_t slot = g % NS;
                    if (!mbar_wait(full_bar + 8 * slot, (g / NS) & 1, abort_flag, p)) { ok = false; break; }
                    const uint64_t k_desc = k_desc0 + uint64_t((ring_addr + slot * G::kStageBytes) >> 4);
#pragma unroll
                    for (int gr = 0; gr < 2; ++gr) {
                        if (!mbar_wait(s_free_bar + 8 * gr, (g & 1) ^ 1, abort_flag, p)) { ok = false; break; }
                        tmem_fence_after();
#pragma unroll
                        for (int kk = 0; kk < D / 16; ++kk) {
                            // A = the Q tile in tensor memory (read once per task from shared memory, not once per
                            // instruction). B = K rows 8 * gr .. 8 * gr + 7 of the stage's pages.
                            const uint64_t k = k_desc + uint64_t(((kk / 4) * G::kBoxBytes + gr * 1024 + (kk % 4) * 32) >> 4);
                            umma_ts(tmem_s + 64 * gr, q_tmem + 8 * kk, k, idesc_qk, kk > 0 ? 1u : 0u);
                        }
                        umma_commit(s_full_bar + 8 * gr);
                    }
                }
                stage_base += num_tiles;
                if (ok) mbar_arrive(task_empty_bar + 8 * tslot);  // done with the task's descriptor
            }
            // nothing issued here may still be running when tensor memory is freed (bounded, also on the abort path)
            umma_commit(drain_bar);
            for (uint32_t i = 0; i < p.wait_limit; ++i) {
                if (mbar_try_wait(drain_bar, 0)) break;
            }
        }
    } else if (warp == NSW + 3) {
        // ------------------------------ P V issue (one thread) ---------------------------------
        if (lane == 0) {
            constexpr uint32_t kFormat = umma_format<T>();
            // D f32; A (P, tensor memory) and B 16-bit of the same type (an f16 A operand beside a bf16 B operand is
            // not a legal descriptor: it raised an illegal-instruction error); M = 128, N = D; B (V) MN-major
            const uint32_t idesc_pv =
                (1u << 4) | (kFormat << 7) | (kFormat << 10) | (1u << 16) | ((uint32_t(D) >> 3) << 17) | ((128u >> 4) << 24);
            const uint64_t v_desc0 = umma_smem_desc(0, G::kBoxBytes, G::kCopyBytes);
            const uint32_t ring_addr = smem_addr(ring);
            uint32_t stage_base = 0;
            uint32_t pv_tasks = 0;  // tasks so far that issued P V products (their epilogues release O)
            bool ok = true;
            for (uint32_t taken = 0; ok; ++taken) {
                const uint32_t tslot = taken % TQ;
                if (!mbar_wait(task_full_bar + 8 * tslot, (taken / TQ) & 1, abort_flag, p)) break;
                const TaskSlot* ts = task_ring + tslot;
                if (ts->done) break;
                const uint32_t num_tiles = ts->num_tiles;
                for (uint32_t i = 0; i < num_tiles && ok; ++i) {
                    const uint32_t g = stage_base + i;
                    const uint32_t slot = g % NS;
                    const uint64_t v_desc = v_desc0 + uint64_t((ring_addr + slot * G::kStageBytes + G::kPlaneBoxBytes) >> 4);
#pragma unroll
                    for (int gr = 0; gr < 2; ++gr) {
                        if (!mbar_wait(p_full_bar + 8 * gr, g & 1, abort_flag, p)) { ok = false; break; }
                        if (i == 0 && gr == 0 && pv_tasks > 0) {
                            // this task's first product overwrites O: the previous task's epilogue must have read it
                            if (!mbar_wait(o_free_bar, (pv_tasks - 1) & 1, abort_flag, p)) { ok = false; break; }
                        }
                        tmem_fence_after();
                        // the softmax warps say whether this half-stage's rounding remainders carry weight
                        const bool with_remainder =
                            kRemainder && !(debug_bits(p) & 1024) &&
                            (remainder_flag[4 * gr] | remainder_flag[4 * gr + 1] | remainder_flag[4 * gr + 2] |
                             remainder_flag[4 * gr + 3]) != 0u;
#pragma unroll
                        for (int j = 0; j < SC / 16; ++j) {
                            // 16-token chunk j of the half-stage's score columns: row group gr of pages 2 j and 2 j + 1
                            const uint64_t v = v_desc + uint64_t(((2 * j) * G::kCopyBytes + gr * 1024) >> 4);
                            umma_ts(tmem_o, tmem_p + 64 * gr + 8 * j, v, idesc_pv, (i == 0 && gr == 0 && j == 0) ? 0u : 1u);
                            // bf16 probabilities (8 significant bits) are followed by their rounding remainder; f16
                            // probabilities (11 bits) need none
                            if (kRemainder && with_remainder) umma_ts(tmem_o, tmem_p + 64 * gr + 32 + 8 * j, v, idesc_pv, 1u);
                        }
                        // K and V of the stage are consumed once its second half-stage's products completed (its
                        // Q K^T products completed before the probabilities could be computed)
                        if (gr == 1) umma_commit(empty_bar + 8 * slot);
                        umma_commit(pv_done_bar + 8 * gr);
                    }
                }
                if (num_tiles > 0) ++pv_tasks;
                stage_base += num_tiles;
                if (ok) mbar_arrive(task_empty_bar + 8 * tslot);  // done with the task's descriptor
            }
            umma_commit(drain_bar + 8);
            for (uint32_t i = 0; i < p.wait_limit; ++i) {
                if (mbar_try_wait(drain_bar + 8, 0)) break;
            }
        }
    }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
        // ------------------------------ softmax and epilogue warps -----------------------------
        // Two groups of four warps; both cover the tile's 128 rows (a warp reaches the tensor-memory lanes of
        // quadrant warp % 4) and take one half-stage of every stage each: group w handles row group w of the
        // stage's pages (running half-stage number 2 G + w), with score buffer w and probability buffer w. Per row, the maximum the probabilities are
        // relative to lives in shared memory; the decision about it (cheap: tile maximum, compare, the rare
        // rescale of O) is made stage after stage in order - a group waits for the other group's decision on
        // the previous stage - while the expensive part (exponentials, rounding, stores) of consecutive stages
        // overlaps. Each group keeps its own row sum, relative to the maximum it last saw.
        const uint32_t wg = uint32_t(warp) / 4;
        const uint32_t quad = uint32_t(warp) % 4;
        const uint32_t row = quad * 32 + lane;           // row of the 128-row tile this thread owns
        const uint32_t lane_base = (quad * 32) << 16;    // this warp's quarter of the tensor-memory lanes
        uint32_t stage_base = 0;
        bool remainder_zeroed = false;  // this warp's remainder columns of its probability buffer hold zeros
        for (uint32_t popped = 0;; ++popped) {
            const uint32_t tslot = popped % TQ;
            if (!mbar_wait(task_full_bar + 8 * tslot, (popped / TQ) & 1, abort_flag, p)) break;
            const TaskSlot* ts = task_ring + tslot;
            if (ts->done) break;
            const uint32_t t_tmpl = ts->tmpl, t_head_begin = ts->head_begin, t_num_heads = ts->num_heads;
            const uint32_t t_tok_begin = ts->tok_begin, t_num_toks = ts->num_toks;
            const uint32_t t_kv_begin = ts->kv_begin, t_kv_end = ts->kv_end;
            const uint32_t t_tile_begin = ts->tile_begin, t_num_tiles = ts->num_tiles;
            const uint32_t row_tok = row / p.heads_per_task;
            const uint32_t row_head = row % p.heads_per_task;
            const bool valid = row_tok < t_num_toks && row_head < t_num_heads;
            uint32_t lo = 0, hi = 0;
            if (valid) {
                uint32_t vb = 0, ve = 0xffffffffu;
                if (p.visible != nullptr) {
                    vb = ts->visible[row_tok * 2];
                    ve = ts->visible[row_tok * 2 + 1];
                }
                lo = max(vb, t_kv_begin);
                hi = min(ve, t_kv_end);
                if (hi < lo) hi = lo;
            }
            // ---- the task's Q tile goes to tensor memory once: this thread's row, un-swizzled, as 16-bit pairs;
            // each group copies one 64-column half
            {
                const uint8_t* q_row = q_ring + tslot * G::kQBytes + row * 128;
                const uint32_t h = wg;
                uint32_t q[32];
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint4 v = *reinterpret_cast<const uint4*>(q_row + h * (G::kQRows * 128) + ((c ^ (row & 7)) << 4));
                    q[4 * c] = v.x;
                    q[4 * c + 1] = v.y;
                    q[4 * c + 2] = v.z;
                    q[4 * c + 3] = v.w;
                }
                tmem_st32(tmem_q + 64 * tslot + 32 * h + lane_base, q);
                tmem_st_wait();
                tmem_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(q_ready_bar + 8 * tslot);
            }
            float m_ref = -INFINITY;  // raw dot-product domain: the maximum this group's l_run is relative to
            float l_run = 0.0f;
            bool failed = false;
            for (uint32_t i = 0; i < t_num_tiles; ++i) {
                const uint32_t g = 2 * (stage_base + i) + wg;  // running half-stage number
                const uint32_t sb = wg;
                const bool first = i == 0 && wg == 0;          // the task's first half-stage
                if (!mbar_wait(s_full_bar + 8 * sb, (g >> 1) & 1, abort_flag, p)) { failed = true; break; }
                tmem_fence_after();
                // the row's 64 scores, kept as bit patterns in one register array (register pressure decides the
                // speed of this loop: twelve warps leave 170 registers per thread)
                uint32_t sraw[SC];
#pragma unroll
                for (int c0 = 0; c0 < SC; c0 += 16) {
                    tmem_ld16(*reinterpret_cast<uint32_t(*)[16]>(&sraw[c0]), tmem_s + 64 * sb + c0 + lane_base);
                }
                tmem_ld_wait();
                tmem_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(s_free_bar + 8 * sb);
                const uint32_t tile_tok = t_tile_begin + i * ST;
                float tile_max = -INFINITY;
                // most stages of a long context lie wholly inside every row's visible range: no masking then
                const bool cut = tile_tok < lo || tile_tok + ST > hi;
                if (__any_sync(0xffffffffu, cut)) {
#pragma unroll
                    for (int j = 0; j < SC; ++j) {
                        const uint32_t tok = tile_tok + (j / 8) * 16 + wg * 8 + (j % 8);
                        if (!(tok >= lo && tok < hi)) sraw[j] = 0xff800000u;  // -inf
                        tile_max = fmaxf(tile_max, __uint_as_float(sraw[j]));
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < SC; ++j) tile_max = fmaxf(tile_max, __uint_as_float(sraw[j]));
                }
                // ---- the decision about the row maximum, in stage order
                float m_prev = -INFINITY;
                if (!first) {
                    const uint32_t gp = g - 1;  // handled by the other group
                    if (!mbar_wait(decided_bar + 8 * (wg ^ 1), (gp >> 1) & 1, abort_flag, p)) { failed = true; break; }
                    m_prev = row_max[row];
                }
                if (m_ref != m_prev) {
                    // the other group moved the maximum since this group last added to its sum
                    if (m_ref != -INFINITY) l_run *= fast_exp2((m_ref - m_prev) * p.scale_log2e);
                    m_ref = m_prev;
                }
                // lazy maximum: move it (and rescale l and O) only when the tile exceeds it by more than 2^8
                const bool grow = tile_max > -INFINITY &&
                                  (m_prev == -INFINITY || (tile_max - m_prev) * p.scale_log2e > kRescaleLog2);
                if (__any_sync(0xffffffffu, grow)) {
                    const float alpha = (grow && m_prev != -INFINITY) ? fast_exp2((m_prev - tile_max) * p.scale_log2e) : 1.0f;
                    if (grow) {
                        l_run *= alpha;
                        m_ref = tile_max;
                    }
                    if (!first) {
                        // O holds this task's earlier half-stages: wait for the previous one's products, then scale
                        const uint32_t gp = g - 1;
                        if (!mbar_wait(pv_done_bar + 8 * (gp & 1), (gp >> 1) & 1, abort_flag, p)) { failed = true; break; }
                        tmem_fence_after();
#pragma unroll
                        for (int c0 = 0; c0 < D; c0 += 32) {
                            uint32_t o[32];
                            tmem_ld32(o, tmem_o + c0 + lane_base);
                            tmem_ld_wait();
#pragma unroll
                            for (int j = 0; j < 32; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
                            tmem_st32(tmem_o + c0 + lane_base, o);
                        }
                        tmem_st_wait();
                        tmem_fence_before();
                    }
                }
                row_max[row] = m_ref;
                __syncwarp();
                if (lane == 0) mbar_arrive(decided_bar + 8 * wg);
                const float m_used = m_ref;
                const float shift = m_used == -INFINITY ? 0.0f : -m_used * p.scale_log2e;
                // the probability buffer is free once the products of this group's previous stage have completed
                if (g >= 2) {
                    const uint32_t gp = g - 2;
                    if (!mbar_wait(pv_done_bar + 8 * (gp & 1), (gp >> 1) & 1, abort_flag, p)) { failed = true; break; }
                }
                tmem_fence_after();
                // The rounding remainder of a bf16 probability is 2^-9 of it at most. Once a row's sum (so far, of
                // this group's half-stages: a lower bound of the final normaliser) is 64 times the largest
                // probability of this half-stage, what the remainders of the half-stage add to the output is below
                // 2^-9 / 8 of a V element: the second product is skipped, for all 128 rows or none (the PV
                // thread reads the four warps' flags). Rows with few or dominant tokens keep it.
                bool remainder = false;
                if constexpr (kRemainder) {
                    const float p_max = tile_max == -INFINITY ? 0.0f : fast_exp2(fmaf(tile_max, p.scale_log2e, shift));
                    remainder = __any_sync(0xffffffffu, valid && p_max * 64.0f > l_run);
                    if (lane == 0) remainder_flag[4 * sb + quad] = remainder ? 1u : 0u;
                }
#pragma unroll
                for (int chunk = 0; chunk < SC / 16; ++chunk) {
                    uint32_t packed_hi[8], packed_lo[kRemainder ? 8 : 1];  // rounded pairs and their rounding remainders
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int c = 16 * chunk + 2 * j;
                        const float p0 = fast_exp2(fmaf(__uint_as_float(sraw[c]), p.scale_log2e, shift));
                        const float p1 = fast_exp2(fmaf(__uint_as_float(sraw[c + 1]), p.scale_log2e, shift));
                        l_run += p0 + p1;
                        packed_hi[j] = pack2<T>(p0, p1);
                        if constexpr (kRemainder) {
                            if (remainder) {
                                const float2 r = unpack2<T>(packed_hi[j]);
                                packed_lo[j] = pack2<T>(p0 - r.x, p1 - r.y);
                            } else {
                                packed_lo[j] = 0u;
                            }
                        }
                    }
                    tmem_st8(tmem_p + 64 * sb + 8 * chunk + lane_base, packed_hi);
                    if constexpr (kRemainder) {
                        // another warp of the group may still ask for the second product: this warp's remainder
                        // columns then have to hold zeros, which they keep until it stores remainders again
                        if (remainder || !remainder_zeroed) tmem_st8(tmem_p + 64 * sb + 32 + 8 * chunk + lane_base, packed_lo);
                    }
                }
                if constexpr (kRemainder) remainder_zeroed = !remainder;
                tmem_st_wait();
                if (tile_tok + ST > t_kv_end) {
                    // V rows of tokens at or past kv_end may never have been loaded: clear them so that a zero
                    // probability times stale bits cannot produce NaN (generic-proxy writes, then a proxy fence
                    // before the tensor core reads them)
                    // Each group clears the rows of its own row group: the rows its half-stage's products read.
                    const uint32_t first_bad = t_kv_end > tile_tok ? t_kv_end - tile_tok : 0;
                    uint8_t* stage = ring + ((g >> 1) % NS) * G::kStageBytes;
                    for (uint32_t idx = row; idx < uint32_t(SC) * (D / 8); idx += 128) {
                        const uint32_t own = idx / (D / 8);                        // row of this half-stage
                        const uint32_t r = (own / 8) * 16 + wg * 8 + own % 8;      // token row of the stage
                        if (r < first_bad) continue;
                        const uint32_t c = idx % (D / 8);
                        uint8_t* dst = stage + (r / G::kBoxRows) * G::kCopyBytes + G::kPlaneBoxBytes + (c / 8) * G::kBoxBytes +
                                       (r % G::kBoxRows) * 128 + (c % 8) * 16;
                        *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                }
                tmem_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(p_full_bar + 8 * sb);
            }
            if (failed) break;
            stage_base += t_num_tiles;

            // ---- epilogue: both groups bring their row sums to the final maximum and add them, then each
            // publishes 64 of the row's columns
            __syncwarp();
            if (lane == 0) mbar_arrive(epilogue_bar);      // every decision of the task has been made
            if (!mbar_wait(epilogue_bar, popped & 1, abort_flag, p)) break;
            const float m_fin = t_num_tiles > 0 ? row_max[row] : -INFINITY;
            if (m_ref != m_fin && m_ref != -INFINITY) l_run *= fast_exp2((m_ref - m_fin) * p.scale_log2e);
            row_sum[wg * 128 + row] = l_run;
            __syncwarp();
            if (lane == 0) mbar_arrive(epilogue_bar + 8);  // every group's sum is written
            if (!mbar_wait(epilogue_bar + 8, popped & 1, abort_flag, p)) break;
            const float l_tot = row_sum[row] + row_sum[128 + row];
            const bool write_final = p.direct != 0;
            const float inv_l = l_tot > 0.0f ? 1.0f / l_tot : 0.0f;
            const uint32_t head = t_head_begin + row_head;
            const uint64_t index = (uint64_t(t_tmpl) * p.num_q_heads + head) * p.max_q_tokens + row_tok;
            if (t_num_tiles > 0) {
                const uint32_t gl = 2 * (stage_base - 1) + 1;  // the task's last half-stage
                if (!mbar_wait(pv_done_bar + 8 * (gl & 1), (gl >> 1) & 1, abort_flag, p)) break;
                tmem_fence_after();
#pragma unroll
                for (int c0 = 0; c0 < D / 2; c0 += 32) {
                    const int col = int(wg) * (D / 2) + c0;
                    uint32_t o[32];
                    tmem_ld32(o, tmem_o + col + lane_base);
                    tmem_ld_wait();
                    if (valid) {
                        if (write_final) {
                            T* dst = reinterpret_cast<T*>(p.out) +
                                     (uint64_t(t_tok_begin + row_tok) * p.num_q_heads + head) * D + col;
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint4 v;
                                v.x = pack2<T>(__uint_as_float(o[j]) * inv_l, __uint_as_float(o[j + 1]) * inv_l);
                                v.y = pack2<T>(__uint_as_float(o[j + 2]) * inv_l, __uint_as_float(o[j + 3]) * inv_l);
                                v.z = pack2<T>(__uint_as_float(o[j + 4]) * inv_l, __uint_as_float(o[j + 5]) * inv_l);
                                v.w = pack2<T>(__uint_as_float(o[j + 6]) * inv_l, __uint_as_float(o[j + 7]) * inv_l);
                                *reinterpret_cast<uint4*>(dst + j) = v;
                            }
                        } else {
                            float* dst = p.partial_out + index * D + col;
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                *reinterpret_cast<float4*>(dst + j) =
                                    make_float4(__uint_as_float(o[j]) * inv_l, __uint_as_float(o[j + 1]) * inv_l,
                                                __uint_as_float(o[j + 2]) * inv_l, __uint_as_float(o[j + 3]) * inv_l);
                            }
                        }
                    }
                }
                tmem_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(o_free_bar);
            } else if (valid) {
                const int col = int(wg) * (D / 2);
                if (write_final) {
                    T* dst = reinterpret_cast<T*>(p.out) + (uint64_t(t_tok_begin + row_tok) * p.num_q_heads + head) * D + col;
                    for (int j = 0; j < D / 2; j += 8) *reinterpret_cast<uint4*>(dst + j) = make_uint4(0, 0, 0, 0);
                } else {
                    float* dst = p.partial_out + index * D + col;
                    for (int j = 0; j < D / 2; j += 4) *reinterpret_cast<float4*>(dst + j) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                }
            }
            if (valid && !write_final && wg == 0) {
                p.partial_sum[index] = l_tot;
                // the maximum is a raw dot product; publish the natural-log-domain logit (dot * scale)
                p.partial_max[index] = l_tot > 0.0f ? m_fin * (p.scale_log2e * 0.6931471805599453f) : -INFINITY;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(task_empty_bar + 8 * tslot);
        }
    }
    tmem_fence_before();
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(G::kTmemColumns) : "memory");
    }
}

}  // namespace kh
