// Map / direct kernel in "token-major" form: the KV tokens of a stage are the M dimension of the warp-level
// tensor-core tiles and the task's Q rows - (Q tokens of the range) x (Q heads of the KV group), at most 32 - are
// the N dimension (8 rows per n-tile).
//
//   S^T = K Q^T     m16n8k16, A = 16 KV tokens x 16 head-dim elements, B = the Q rows.
//   O^T += V^T P^T  m16n8k16, A = 16 head-dim elements x 16 KV tokens, B = the probabilities.
//
// With the tokens on M a decode task (8 rows) costs one MMA per 16 tokens x 16 head-dim elements instead of two
// half-empty ones, every K/V fragment is loaded (and, for one-byte pages, converted) once for all Q rows of the
// task, and a thread's accumulator is D/16 x (rows/8) x 4 registers, small enough for eight consumer warps per SM.
// Tasks whose accumulator would still be too wide (17-32 rows, or head_dim 256 with more than 8 rows) share a stage
// among the NR warps of a group (row split): each warp takes NQ / NR n-tiles of Q rows over the whole head
// dimension. The warps of a group load the same K/V fragments (shared-memory bandwidth is not the limit here),
// exchange nothing, and release the stage together. Measured on the verify workload (24 rows, head_dim 256)
// against warp pairs that split the head dimension and exchange partial scores (every warp then repeats the
// softmax: 0.55 ms against 0.49 ms) and against pairs that split a 32-token stage by tokens and exchange packed
// probabilities (the same 0.49 ms, with far more machinery): the row split is what is kept.
//
// K/V pages of FP8 E4M3FN elements (KVB = 1; the reference's cache format: one byte per stored element, one unit
// scale; components/gqa/sdpa/sliced_kv.rs:113-125, decoded on load by metal/gqa_fp8.metal:1-25). At the HBM rate a
// one-byte page delivers twice the tokens per second of a 16-bit page, so everything per token has to cost half:
//  - The raw bytes are consumed straight from the copied stage, with no intermediate 16-bit copy in shared memory:
//    K through ldmatrix as if the bytes were 16-bit pairs (a thread receives four consecutive head-dim elements of
//    one token), V through the 8-bit transposing matrix load (ldmatrix .m16n16 .trans .b8: a thread receives four
//    consecutive tokens of one head-dim element). Both hand a thread *four consecutive* indices of the contraction
//    dimension where the MMA fragment wants the pairs (2t, 2t+1) and (2t+8, 2t+9): a fixed permutation of the 16
//    contraction indices. A sum is order-free, so the other operand is simply read under the same permutation: Q
//    (for K's head-dim order) by an 8-byte shared-memory load per fragment, P (for V's token order) by choosing
//    which token each row of the K tile is (ldmatrix takes a row address per lane) and transposing the packed
//    probabilities with movmatrix.
//  - Conversion is one instruction per element pair (cvt.rn.f16x2.e4m3x2, exact; the NaN codes become NaN) and the
//    MMAs run in f16 whatever the Q/output type: every E4M3 value is an f16 value, bf16 Q values convert exactly
//    inside f16's range (beyond it they saturate), and f16 probabilities carry 11 significant bits.
// K/V pages of 16-bit elements (KVB = 2): K through ldmatrix, V through ldmatrix .trans, in natural order; the MMAs
// run in the Q/output type, and bf16 probabilities carry their rounding remainder in a second MMA (a bf16
// probability alone costs up to 2^-9 of |p v| per term, which short contexts turn into errors beyond 2e-3).
//
// Task ABI, task warp, stream warp, rings and partial-state layout are those of sdpa_map_kernel (sdpa_map.cuh).
// Synchronisation between the consumer warps goes through mbarriers with bounded waits only.
#pragma once

#include "sdpa_map.cuh"

namespace kh {

// D: head dimension. P: tokens per page. NQ: n-tiles of 8 Q rows per task. CW: consumer warps. KVB: bytes of a
// stored K/V element. NR: warps that share a stage by splitting the n-tiles of Q rows between them.
template <int D, int P, int NQ, int CW, int KVB, int NR = 1>
struct TmGeometry {
    static_assert(P == 16, "the token-major kernel is built for 16-token pages (one page = one 16-token MMA tile)");
    static_assert(D == 128 || D == 256, "head_dim 128 or 256");
    static_assert(KVB == 1 || KVB == 2, "K/V elements are stored in one or two bytes");
    static_assert(NR >= 1 && NQ % NR == 0, "a row split divides the n-tiles among the warps of a group");
    static_assert(CW % NR == 0, "consumer warps come in groups of NR");
    static constexpr int kStageTokens = (D == 128) ? 32 : 16;
    static constexpr int kBoxRows = P;
    static constexpr int kBoxesPerPlane = kStageTokens / kBoxRows;   // pages per stage
    static constexpr int kLineElems = 128 / KVB;                      // stored elements of a 128-byte line
    static constexpr int kColumnGroups = D / kLineElems;              // 128-byte lines per stored row
    static constexpr int kBoxBytes = kBoxRows * 128;                  // one column group of one page
    static constexpr int kPlaneBoxBytes = kColumnGroups * kBoxBytes;  // K (or V) rows of one page
    static constexpr int kCopyBytes = 2 * kPlaneBoxBytes;             // one TMA copy: K and V of one (page, KV head)
    static constexpr int kStageBytes = kBoxesPerPlane * kCopyBytes;   // 8 KiB (one-byte pages) or 16 KiB
    static constexpr int kColumnHalves = D / 64;                      // Q tile: 64-element column halves (16-bit)
    static constexpr int kQRows = NQ * 8;
    static constexpr int kQBytes = kQRows * D * 2;
    static constexpr int kTaskSlots = 2;  // (four slots measured the same on the FP8 decode bench)
    static constexpr int kConsumerWarps = CW;
    static constexpr int kGroups = CW / NR;                           // warp groups; a stage goes to one group
    static constexpr int kThreads = (CW + 2) * 32;                    // + stream warp + task warp
    static constexpr int kRowStride = D + 4;                          // floats; makes the parking stores conflict free
    static constexpr int kParkFloats = kQRows * kRowStride + 4 * kQRows;  // O rows, then two sets of (max, sum) per row
    // Task-end merge of the groups' states through shared memory: one parking slot per group, or - where that would
    // take the stage ring's memory - half as many slots in two rounds (the second half of the groups folds its
    // state into the slots the first half parked)
    static constexpr bool kTwoRounds = kGroups >= 2 && kGroups * kParkFloats * 4 > 48 * 1024;
    static constexpr int kSlots = kTwoRounds ? (kGroups + 1) / 2 : kGroups;
    static constexpr int kMergeBytes = kSlots * kParkFloats * 4;
    static constexpr int kPidBytes = kTaskSlots * kMaxPidsPerSegment * 4;
    static constexpr int kTaskBytes = kTaskSlots * static_cast<int>(sizeof(TaskSlot));
    static constexpr int kFixedBytes = kTaskSlots * kQBytes + kMergeBytes + kPidBytes + kTaskBytes + 1024;
    static constexpr int kSmemLimit = 227 * 1024 - 1024;
    static constexpr int kStagesFit = (kSmemLimit - kFixedBytes) / kStageBytes;
    // (any depth: a ring slot may pass from group to group, see the two waits before a stage is read)
    static constexpr int kStages = kStagesFit > 24 ? 24 : kStagesFit;
    static constexpr int kSmemBytes = kStages * kStageBytes + kFixedBytes + 1024;
    // Q fragments of a task stay in registers for the whole task
    static constexpr int kQFragmentRegs = NQ / NR * (D / 16) * 2;
    static_assert(kStages >= kGroups && kStages >= 4, "shared memory ring too small");
    static_assert(kQFragmentRegs <= 64, "the task's Q fragments must fit registers");
    static_assert(NQ >= 1 && NQ <= 4, "a task holds at most 32 Q rows here");
};

__device__ __forceinline__ uint32_t cvt_e4m3x2_to_f16x2(uint16_t pair) {
    uint32_t out;
    asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(out) : "h"(pair));
    return out;
}

__device__ __forceinline__ void ldmatrix_m16n16_x2_trans_b8(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m16n16.x2.trans.shared.b8 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t v) {
    uint32_t out;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(out) : "r"(v));
    return out;
}

__device__ __forceinline__ uint32_t pack_f16x2(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Two Q elements of type T (packed) as f16x2; bf16 values beyond f16's range saturate.
template <typename T>
__device__ __forceinline__ uint32_t q_pair_to_f16x2(uint32_t packed);
template <>
__device__ __forceinline__ uint32_t q_pair_to_f16x2<__half>(uint32_t packed) { return packed; }
template <>
__device__ __forceinline__ uint32_t q_pair_to_f16x2<__nv_bfloat16>(uint32_t packed) {
    const float lo = fminf(fmaxf(__uint_as_float(packed << 16), -65504.0f), 65504.0f);
    const float hi = fminf(fmaxf(__uint_as_float(packed & 0xffff0000u), -65504.0f), 65504.0f);
    return pack_f16x2(lo, hi);
}

template <typename T, int D, int P, int NQ, int CW, int KVB, int NR = 1>
__global__ void __launch_bounds__(TmGeometry<D, P, NQ, CW, KVB, NR>::kThreads, 1)
sdpa_tm_kernel(const __grid_constant__ CUtensorMap kv_map, const __grid_constant__ CUtensorMap q_map, const MapParams p) {
    using G = TmGeometry<D, P, NQ, CW, KVB, NR>;
    constexpr int NQW = NQ / NR;      // n-tiles of Q rows a warp works on
    // the element type the MMAs run in: f16 over one-byte pages, the Q/output type over 16-bit pages
    using M = std::conditional_t<KVB == 1, __half, T>;
    constexpr bool kRemainder = KVB == 2 && std::is_same<T, __nv_bfloat16>::value;  // P V carries P's rounding remainder
    constexpr int ST = G::kStageTokens;
    constexpr int NS = G::kStages;
    constexpr int TQ = G::kTaskSlots;
    constexpr int NG = G::kGroups;
    constexpr int MTK = ST / 16;      // 16-token tiles (pages) per stage
    constexpr int DK = D / 16;        // contraction steps of K Q^T = 16-element m-tiles of O^T
    constexpr int RS = G::kRowStride;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = smem;
    uint8_t* q_ring = ring + NS * G::kStageBytes;
    float* merge = reinterpret_cast<float*>(q_ring + TQ * G::kQBytes);
    uint32_t* pid_smem = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(merge) + G::kMergeBytes);
    TaskSlot* task_ring = reinterpret_cast<TaskSlot*>(reinterpret_cast<uint8_t*>(pid_smem) + G::kPidBytes);
    uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(task_ring) + G::kTaskBytes);
    constexpr int kNumBars = 2 * NS + 3 * TQ + 3;
    volatile uint32_t* abort_flag = reinterpret_cast<volatile uint32_t*>(bars + kNumBars);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t full_bar = smem_addr(bars);
    const uint32_t empty_bar = smem_addr(bars + NS);
    const uint32_t task_full_bar = smem_addr(bars + 2 * NS);
    const uint32_t task_empty_bar = smem_addr(bars + 2 * NS + TQ);
    const uint32_t stream_full_bar = smem_addr(bars + 2 * NS + 2 * TQ);
    const uint32_t parked_bar = smem_addr(bars + 2 * NS + 3 * TQ);      // every consumer warp parked its state
    const uint32_t merged_bar = smem_addr(bars + 2 * NS + 3 * TQ + 1);  // every consumer warp read the parked states
    const uint32_t folded_bar = smem_addr(bars + 2 * NS + 3 * TQ + 2);  // second merge round: every warp folded its state

    if (threadIdx.x == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, NR);  // every warp of the group releases the stage
        }
        for (int s = 0; s < TQ; ++s) {
            mbar_init(task_full_bar + 8 * s, p.visible != nullptr ? 33 : 1);
            mbar_init(task_empty_bar + 8 * s, CW + 1);  // every consumer warp and the stream warp
            mbar_init(stream_full_bar + 8 * s, 1);
        }
        mbar_init(parked_bar, CW);
        mbar_init(merged_bar, CW);
        mbar_init(folded_bar, CW);
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
    const bool balanced = active.templates <= kBalanceMaxTemplates && active.templates <= uint32_t(NS) * G::kStageBytes / 4;

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
    producer.task_base = blockIdx.x;
    producer.task_step = balanced ? 1u : gridDim.x;
    producer.task_limit = total_tasks;
    producer.balanced = balanced;
    producer.allow_carry = true;
    producer.active = active;
    producer.lane = lane;

    if (warp == CW + 1) {
        run_task_warp<G, P>(p, q_map, producer);
    } else if (warp == CW) {
        run_stream_warp<G, P, stream_lanes(G::kStages)>(p, kv_map, producer);
    } else {
        // ------------------------------ consumer warps ----------------------------------------
        const int g = lane >> 2;   // fragment row group
        const int tq = lane & 3;   // thread in quad
        const int group = warp / NR;          // which stages this warp works on
        const int n0 = (warp % NR) * NQW;     // row split: the first n-tile of Q rows this warp works on
        // One-byte pages: row r (0-7) of a 16-token MMA tile is token 4 * (r / 2) + r % 2 of its page, row r + 8 is
        // that token + 2: a thread's accumulator pair (rows g, g + 8) then holds tokens t and t + 2, and after the
        // transposition of the packed probabilities thread (g, tq) holds tokens 4 tq .. 4 tq + 3 of Q row g - the
        // four consecutive tokens the 8-bit transposing load of V gives it. 16-bit pages: natural order.
        const uint32_t sig = KVB == 1 ? 4u * (g >> 1) + (g & 1) : uint32_t(g);
        constexpr uint32_t kUpperRow = KVB == 1 ? 2u : 8u;  // token distance between fragment rows g and g + 8
        // K: ldmatrix .x4. One-byte pages: matrix (lane >> 3) bit 0 picks the row half (tokens + 2), bit 1 the next
        // 16-byte chunk (= the next 16 head-dim elements). 16-bit pages: bit 0 picks rows 8-15, bit 1 the upper 8
        // elements of the 16-element step.
        const uint32_t k_mat = lane >> 3, k_r = lane & 7;
        const uint32_t k_tok = KVB == 1 ? 4u * (k_r >> 1) + (k_r & 1) + 2u * (k_mat & 1) : k_r + 8u * (k_mat & 1);
        const uint32_t k_lane = k_tok * 128u;
        const uint32_t k_y4 = ((k_mat >> 1) ^ (k_tok & 7)) << 4;
        // V. One-byte pages: ldmatrix .m16n16 .x2 .trans; lanes 0-15 address the 16 token rows of one 16-byte chunk,
        // lanes 16-31 those of the next chunk. 16-bit pages: ldmatrix .x4 .trans; matrix bit 0 picks the upper 8
        // elements of a 16-element m-tile, bit 1 tokens 8-15.
        const uint32_t v_tok = KVB == 1 ? uint32_t(lane & 15) : k_r + 8u * (k_mat >> 1);
        const uint32_t v_lane = v_tok * 128u;
        const uint32_t v_y4 = ((KVB == 1 ? uint32_t(lane) >> 4 : (k_mat & 1)) ^ (v_tok & 7)) << 4;

        float o[DK][NQW][4];
        float m_run[NQW][2], l_run[NQW][2];
#pragma unroll
        for (int c = 0; c < DK; ++c)
#pragma unroll
            for (int n = 0; n < NQW; ++n) o[c][n][0] = o[c][n][1] = o[c][n][2] = o[c][n][3] = 0.0f;
#pragma unroll
        for (int n = 0; n < NQW; ++n) {
            m_run[n][0] = m_run[n][1] = -INFINITY;
            l_run[n][0] = l_run[n][1] = 0.0f;
        }
        uint32_t stage_counter = 0;
        uint32_t my_stage = group, my_slot = group, my_parity = 0;
        uint32_t merges = 0;          // merges this CTA has run (phase of the two merge barriers)
        constexpr int NSLOT = G::kSlots;
        const int merge_round = G::kTwoRounds ? group / NSLOT : 0;  // which merge round this warp writes in
        float* const my_park = merge + (group % NSLOT) * G::kParkFloats;
        float* const my_stats = my_park + G::kQRows * RS + merge_round * 2 * G::kQRows;

        uint32_t qb[NQW][DK][2] = {};  // the task's Q rows as the B operand of K Q^T
        // Q rows 8 n + 2 tq + j of a task (this thread's score columns): which Q token and which head of the task
        uint32_t row_tok_of[NQW][2], row_head_of[NQW][2];
#pragma unroll
        for (int n = 0; n < NQW; ++n)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const uint32_t row = 8 * (n0 + n) + 2 * tq + j;
                row_tok_of[n][j] = row / p.heads_per_task;
                row_head_of[n][j] = row % p.heads_per_task;
            }
        for (uint32_t popped = 0;; ++popped) {
            const uint32_t tslot = popped % TQ;
            if (!mbar_wait(task_full_bar + 8 * tslot, (popped / TQ) & 1, abort_flag, p)) break;
            const TaskSlot* ts = task_ring + tslot;
            if (ts->done) break;
            const uint32_t t_tmpl = ts->tmpl, t_head_begin = ts->head_begin, t_num_heads = ts->num_heads;
            const uint32_t t_tok_begin = ts->tok_begin, t_num_toks = ts->num_toks;
            const uint32_t t_kv_begin = ts->kv_begin, t_kv_end = ts->kv_end;
            const uint32_t t_tile_begin = ts->tile_begin, t_num_tiles = ts->num_tiles;
            const uint32_t t_carry = ts->carry;
            const bool write_final = p.direct != 0;

            // ---- per-thread row bounds: Q rows 8 n + 2 tq + j of the task
            uint32_t lo[NQW][2], hi[NQW][2];
#pragma unroll
            for (int n = 0; n < NQW; ++n) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const uint32_t row_tok = row_tok_of[n][j], row_head = row_head_of[n][j];
                    lo[n][j] = 0;
                    hi[n][j] = 0xffffffffu;  // rows that hold nothing are never published: left unmasked
                    if (row_tok < t_num_toks && row_head < t_num_heads) {
                        uint32_t vb = 0, ve = 0xffffffffu;
                        if (p.visible != nullptr) {
                            vb = ts->visible[row_tok * 2];
                            ve = ts->visible[row_tok * 2 + 1];
                        }
                        lo[n][j] = max(vb, t_kv_begin);
                        hi[n][j] = min(ve, t_kv_end);
                        if (hi[n][j] < lo[n][j]) hi[n][j] = lo[n][j];
                    }
                }
            }
            if (!(t_carry & 1u)) {
#pragma unroll
                for (int c = 0; c < DK; ++c)
#pragma unroll
                    for (int n = 0; n < NQW; ++n) o[c][n][0] = o[c][n][1] = o[c][n][2] = o[c][n][3] = 0.0f;
#pragma unroll
                for (int n = 0; n < NQW; ++n) {
                    m_run[n][0] = m_run[n][1] = -INFINITY;
                    l_run[n][0] = l_run[n][1] = 0.0f;
                }
            }

            // ---- Q as the B operand of K Q^T for this warp's contraction steps. One-byte pages: under K's head-dim
            // permutation, thread (g, tq) holds elements 16 kk + 4 tq .. + 3 of Q row 8 n + g as two f16 pairs.
            // 16-bit pages: the natural fragment, elements 16 kk + 2 tq, + 1 and 16 kk + 8 + 2 tq, + 1.
            // A task that continues the previous task's running state has the same Q rows: the fragments stay.
            const uint32_t q_tile = smem_addr(q_ring + tslot * G::kQBytes);
#pragma unroll
            for (int n = 0; n < NQW; ++n) {
                if (t_carry & 1u) break;
                const uint32_t row = 8 * (n0 + n) + g;
#pragma unroll
                for (int kk = 0; kk < DK; ++kk) {
                    const uint32_t row_addr = q_tile + (kk >> 2) * (G::kQRows * 128) + row * 128;
                    if constexpr (KVB == 1) {
                        const uint32_t chunk = (2 * (kk & 3) + (tq >> 1)) ^ (row & 7);
                        uint32_t w0, w1;
                        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];"
                                     : "=r"(w0), "=r"(w1)
                                     : "r"(row_addr + (chunk << 4) + 8 * (tq & 1)));
                        qb[n][kk][0] = q_pair_to_f16x2<T>(w0);
                        qb[n][kk][1] = q_pair_to_f16x2<T>(w1);
                    } else {
                        const uint32_t c0 = (2 * (kk & 3)) ^ (row & 7), c1 = (2 * (kk & 3) + 1) ^ (row & 7);
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(qb[n][kk][0]) : "r"(row_addr + (c0 << 4) + 4 * tq));
                        asm volatile("ld.shared.u32 %0, [%1];" : "=r"(qb[n][kk][1]) : "r"(row_addr + (c1 << 4) + 4 * tq));
                    }
                }
            }
            for (; my_stage < stage_counter + t_num_tiles; my_stage += NG) {
                const uint32_t tile = my_stage - stage_counter;
                const uint32_t slot = my_slot;
                const uint32_t phase = my_parity;
                my_slot += NG;
                if (my_slot >= uint32_t(NS)) {
                    my_slot -= NS;
                    my_parity ^= 1;
                }
                // The ring depth need not be a multiple of the group count, so the slot's previous stage may have been
                // another group's. A parity wait tells "this phase" from "the phase before" only: waiting for this
                // stage's copy while the previous stage's copy is still in flight would return at once. So first
                // wait until the previous stage of the slot has been RELEASED (its phase of the empty barrier: that
                // phase cannot be followed by another one before this warp itself releases the slot), which
                // implies that its copy has landed; then wait for this stage's copy. (A ring whose depth is a multiple
                // of the group count hands a slot to the same group every time: no first wait.)
                if constexpr (NS % NG != 0) {
                    if (my_stage >= uint32_t(NS) && !mbar_wait(empty_bar + 8 * slot, phase ^ 1, abort_flag, p)) continue;
                }
                if (!mbar_wait(full_bar + 8 * slot, phase, abort_flag, p)) continue;
                if (debug_bits(p) & 1) {
                    __syncwarp();
                    if (lane == 0) mbar_arrive(empty_bar + 8 * slot);
                    continue;
                }
                const uint32_t tile_tok = t_tile_begin + tile * ST;
                const uint32_t stage_base = smem_addr(ring + slot * G::kStageBytes);

                // Rows of tokens at or past kv_end may hold anything (the tail of a page, or nothing was copied):
                // clear them in V (this warp's share of the columns) so that a zero probability times a NaN cannot
                // produce NaN.
                if (tile_tok + ST > t_kv_end) {
                    const uint32_t first_bad = t_kv_end > tile_tok ? t_kv_end - tile_tok : 0u;
                    constexpr uint32_t kChunksPerRow = D * KVB / 16;  // 16-byte chunks of a row
                    for (uint32_t idx = first_bad * kChunksPerRow + lane; idx < uint32_t(ST) * kChunksPerRow; idx += 32) {
                        const uint32_t r = idx / kChunksPerRow, c = idx % kChunksPerRow;
                        // (chunk c of row r sits at position c ^ (r & 7) of its 128-byte line)
                        const uint32_t addr = stage_base + (r / 16) * G::kCopyBytes + G::kPlaneBoxBytes +
                                              (c >> 3) * G::kBoxBytes + (r % 16) * 128 + (((c & 7) ^ (r & 7)) << 4);
                        asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
                    }
                    __syncwarp();
                }

                // ---- S^T = K Q^T (raw dot products; the softmax scale is folded into the exponent below).
                // A dependent MMA waits for the one before it, so the contraction steps go round KS accumulator
                // sets: with the tiles and n-tiles of the stage that gives at least four independent chains.
                constexpr int KS = MTK * NQW >= 4 ? 1 : MTK * NQW >= 2 ? 2 : 4;
                float s_set[KS][MTK][NQW][4];
#pragma unroll
                for (int ks = 0; ks < KS; ++ks)
#pragma unroll
                    for (int mt = 0; mt < MTK; ++mt)
#pragma unroll
                        for (int n = 0; n < NQW; ++n)
                            s_set[ks][mt][n][0] = s_set[ks][mt][n][1] = s_set[ks][mt][n][2] = s_set[ks][mt][n][3] = 0.0f;
                if (debug_bits(p) & 2) {
                    // measurement build only: no K Q^T
                } else if constexpr (KVB == 1) {
#pragma unroll
                    for (int k = 0; k < DK; k += 2) {
                        const int kk = k;  // 16-byte chunk kk of the row = elements 16 kk .. + 15
#pragma unroll
                        for (int mt = 0; mt < MTK; ++mt) {
                            const uint32_t k_base = stage_base + mt * G::kCopyBytes + k_lane;
                            uint32_t r[4];
                            ldmatrix_x4(r, k_base + (kk >> 3) * G::kBoxBytes + (k_y4 ^ ((kk & 7) << 4)));
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                uint32_t a[4];
                                a[0] = cvt_e4m3x2_to_f16x2(uint16_t(r[2 * h] & 0xffffu));
                                a[1] = cvt_e4m3x2_to_f16x2(uint16_t(r[2 * h + 1] & 0xffffu));
                                a[2] = cvt_e4m3x2_to_f16x2(uint16_t(r[2 * h] >> 16));
                                a[3] = cvt_e4m3x2_to_f16x2(uint16_t(r[2 * h + 1] >> 16));
#pragma unroll
                                for (int n = 0; n < NQW; ++n)
                                    mma_16816<M>(s_set[(k + h) % KS][mt][n], a, qb[n][k + h][0], qb[n][k + h][1]);
                            }
                        }
                    }
                } else {
#pragma unroll
                    for (int k = 0; k < DK; ++k) {
                        const int kk = k;  // elements 16 kk .. + 15 = 16-byte chunks 2 kk, 2 kk + 1
#pragma unroll
                        for (int mt = 0; mt < MTK; ++mt) {
                            const uint32_t k_base = stage_base + mt * G::kCopyBytes + k_lane;
                            uint32_t a[4];
                            ldmatrix_x4(a, k_base + ((2 * kk) >> 3) * G::kBoxBytes + (k_y4 ^ (((2 * kk) & 7) << 4)));
#pragma unroll
                            for (int n = 0; n < NQW; ++n) mma_16816<M>(s_set[k % KS][mt][n], a, qb[n][k][0], qb[n][k][1]);
                        }
                    }
                }
                float (&s)[MTK][NQW][4] = s_set[0];
#pragma unroll
                for (int ks = 1; ks < KS; ++ks)
#pragma unroll
                    for (int mt = 0; mt < MTK; ++mt)
#pragma unroll
                        for (int n = 0; n < NQW; ++n)
#pragma unroll
                            for (int e = 0; e < 4; ++e) s[mt][n][e] += s_set[ks][mt][n][e];
                // ---- mask (only where a row's visible range cuts the stage) and running maximum
                bool cut = false;
#pragma unroll
                for (int n = 0; n < NQW; ++n)
#pragma unroll
                    for (int j = 0; j < 2; ++j) cut = cut || tile_tok < lo[n][j] || tile_tok + ST > hi[n][j];
                if (__any_sync(0xffffffffu, cut)) {
#pragma unroll
                    for (int mt = 0; mt < MTK; ++mt)
#pragma unroll
                        for (int n = 0; n < NQW; ++n)
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const uint32_t tok = tile_tok + 16 * mt + sig + kUpperRow * (e >> 1);
                                if (!(tok >= lo[n][e & 1] && tok < hi[n][e & 1])) s[mt][n][e] = -INFINITY;
                            }
                }
                float alpha[NQW][2], shift[NQW][2];
                bool rescale = false;
#pragma unroll
                for (int n = 0; n < NQW; ++n) {
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        float tile_max = fmaxf(s[0][n][j], s[0][n][j + 2]);
#pragma unroll
                        for (int mt = 1; mt < MTK; ++mt) tile_max = fmaxf(tile_max, fmaxf(s[mt][n][j], s[mt][n][j + 2]));
                        // the row's tokens are spread over the eight row groups of the warp
                        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 4));
                        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 8));
                        tile_max = fmaxf(tile_max, __shfl_xor_sync(0xffffffffu, tile_max, 16));
                        const float m_new = fmaxf(m_run[n][j], tile_max);
                        const float base = m_new == -INFINITY ? 0.0f : m_new;
                        alpha[n][j] = m_run[n][j] == -INFINITY ? 1.0f : fast_exp2((m_run[n][j] - base) * p.scale_log2e);
                        shift[n][j] = -base * p.scale_log2e;
                        m_run[n][j] = m_new;
                        rescale = rescale || alpha[n][j] != 1.0f;
                    }
                }
                if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
                    for (int c = 0; c < DK; ++c)
#pragma unroll
                        for (int n = 0; n < NQW; ++n)
#pragma unroll
                            for (int e = 0; e < 4; ++e) o[c][n][e] *= alpha[n][e & 1];
#pragma unroll
                    for (int n = 0; n < NQW; ++n) {
                        l_run[n][0] *= alpha[n][0];
                        l_run[n][1] *= alpha[n][1];
                    }
                }

                // ---- P^T as the B operand of V^T P^T: exponentials, packed 16-bit pairs (rows 2 tq, 2 tq + 1 of one
                // token), transposed across the warp so that thread (g, tq) holds its four tokens of Q row g
                uint32_t pb[MTK][NQW][2], pr[kRemainder ? MTK : 1][kRemainder ? NQW : 1][2];
#pragma unroll
                for (int mt = 0; mt < MTK; ++mt) {
#pragma unroll
                    for (int n = 0; n < NQW; ++n) {
                        float pv[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) pv[e] = fast_exp2(fmaf(s[mt][n][e], p.scale_log2e, shift[n][e & 1]));
                        l_run[n][0] += pv[0] + pv[2];
                        l_run[n][1] += pv[1] + pv[3];
                        const uint32_t x0 = pack2<M>(pv[0], pv[1]), x1 = pack2<M>(pv[2], pv[3]);
                        pb[mt][n][0] = movmatrix_trans(x0);
                        pb[mt][n][1] = movmatrix_trans(x1);
                        if constexpr (kRemainder) {
                            const float2 r0 = unpack2<M>(x0), r1 = unpack2<M>(x1);
                            pr[mt][n][0] = movmatrix_trans(pack2<M>(pv[0] - r0.x, pv[1] - r0.y));
                            pr[mt][n][1] = movmatrix_trans(pack2<M>(pv[2] - r1.x, pv[3] - r1.y));
                        }
                    }
                }

                // ---- O^T += V^T P^T over this warp's output columns
#pragma unroll
                for (int mt = 0; mt < MTK; ++mt) {
                    if (debug_bits(p) & 16) break;  // measurement build only: no V^T P^T
                    const uint32_t v_base = stage_base + mt * G::kCopyBytes + G::kPlaneBoxBytes + v_lane;
                    if constexpr (KVB == 1) {
#pragma unroll
                        for (int k = 0; k < DK; k += 2) {
                            const int c = k;  // 16-byte chunk c = output columns 16 c .. + 15
                            uint32_t r[4];
                            ldmatrix_m16n16_x2_trans_b8(r, v_base + (c >> 3) * G::kBoxBytes + (v_y4 ^ ((c & 7) << 4)));
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                uint32_t a[4];
                                a[0] = cvt_e4m3x2_to_f16x2(uint16_t(r[2 * h] & 0xffffu));
                                a[1] = cvt_e4m3x2_to_f16x2(uint16_t(r[2 * h + 1] & 0xffffu));
                                a[2] = cvt_e4m3x2_to_f16x2(uint16_t(r[2 * h] >> 16));
                                a[3] = cvt_e4m3x2_to_f16x2(uint16_t(r[2 * h + 1] >> 16));
#pragma unroll
                                for (int n = 0; n < NQW; ++n) mma_16816<M>(o[k + h][n], a, pb[mt][n][0], pb[mt][n][1]);
                            }
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < DK; ++k) {
                            const int c = k;  // output columns 16 c .. + 15 = 16-byte chunks 2 c, 2 c + 1
                            uint32_t a[4];
                            ldmatrix_x4_trans(a, v_base + ((2 * c) >> 3) * G::kBoxBytes + (v_y4 ^ (((2 * c) & 7) << 4)));
#pragma unroll
                            for (int n = 0; n < NQW; ++n) mma_16816<M>(o[k][n], a, pb[mt][n][0], pb[mt][n][1]);
                        }
                        if constexpr (kRemainder) {
                            // the remainders in a pass of their own (V fragments loaded again): an MMA right
                            // behind the one that wrote its accumulator would wait for it
#pragma unroll
                            for (int k = 0; k < DK; ++k) {
                                const int c = k;
                                uint32_t a[4];
                                ldmatrix_x4_trans(a, v_base + ((2 * c) >> 3) * G::kBoxBytes + (v_y4 ^ (((2 * c) & 7) << 4)));
#pragma unroll
                                for (int n = 0; n < NQW; ++n) mma_16816<M>(o[k][n], a, pr[mt][n][0], pr[mt][n][1]);
                            }
                        }
                    }
                }


                // ---- release the stage
                if (tile_tok + ST > t_kv_end) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(empty_bar + 8 * slot);
            }
            stage_counter += t_num_tiles;

            if (t_carry & 2u) {
                // The next task of this CTA continues these rows: nothing is merged or published now. This task's
                // template still gets a partial, an empty one (weight zero in every merge).
                if (group == 0 && g == 0) {
#pragma unroll
                    for (int n = 0; n < NQW; ++n) {
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const uint32_t row_tok = row_tok_of[n][j], row_head = row_head_of[n][j];
                            if (!(row_tok < t_num_toks && row_head < t_num_heads)) continue;
                            const uint64_t index =
                                (uint64_t(t_tmpl) * p.num_q_heads + t_head_begin + row_head) * p.max_q_tokens + row_tok;
                            p.partial_sum[index] = 0.0f;
                            p.partial_max[index] = -INFINITY;
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(task_empty_bar + 8 * tslot);
                continue;
            }

            // ---- task end: every warp parks its share of (max, sum, O^T), then every thread merges and publishes a
            // slice of the rows. Row sums first: a row's tokens are spread over the row groups.
            float l_row[NQW][2];
#pragma unroll
            for (int n = 0; n < NQW; ++n) {
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    float l = l_run[n][j];
                    l += __shfl_xor_sync(0xffffffffu, l, 4);
                    l += __shfl_xor_sync(0xffffffffu, l, 8);
                    l += __shfl_xor_sync(0xffffffffu, l, 16);
                    l_row[n][j] = l;
                }
            }
            bool merge_ok = true;
            if (merges > 0) merge_ok = mbar_wait(merged_bar, (merges - 1) & 1, abort_flag, p);  // parked states are free
            auto weight_of = [&](float m, float base) {
                return m == -INFINITY ? 0.0f : fast_exp2((m - base) * p.scale_log2e);
            };
            if (merge_ok) {
                if (merge_round == 0) {
#pragma unroll
                    for (int c = 0; c < DK; ++c)
#pragma unroll
                        for (int n = 0; n < NQW; ++n)
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                my_park[(8 * (n0 + n) + 2 * tq + (e & 1)) * RS + 16 * c + g + 8 * (e >> 1)] = o[c][n][e];
                            }
                }
                if (g == 0) {
#pragma unroll
                    for (int n = 0; n < NQW; ++n)
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            my_stats[8 * (n0 + n) + 2 * tq + j] = m_run[n][j];
                            my_stats[G::kQRows + 8 * (n0 + n) + 2 * tq + j] = l_row[n][j];
                            if (G::kTwoRounds && merge_round == 0 && group + NSLOT >= NG) {
                                // no second-round group folds into this slot: its second statistics are empty
                                my_stats[2 * G::kQRows + 8 * (n0 + n) + 2 * tq + j] = -INFINITY;
                                my_stats[3 * G::kQRows + 8 * (n0 + n) + 2 * tq + j] = 0.0f;
                            }
                        }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(parked_bar);
                merge_ok = mbar_wait(parked_bar, merges & 1, abort_flag, p);
            }
            if constexpr (G::kTwoRounds) {
                if (merge_ok) {
                    if (merge_round == 1) {
                        // fold this warp's state into the slot a first-round group parked: both become relative to
                        // the larger of the two maxima (the statistics of the two rounds stay side by side)
                        const float* first = my_park + G::kQRows * RS;
                        float w_slot[NQW][2], w_mine[NQW][2];
#pragma unroll
                        for (int n = 0; n < NQW; ++n)
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                const float m_first = first[8 * (n0 + n) + 2 * tq + j];
                                const float m_new = fmaxf(m_first, m_run[n][j]);
                                const float base = m_new == -INFINITY ? 0.0f : m_new;
                                w_slot[n][j] = weight_of(m_first, base);
                                w_mine[n][j] = weight_of(m_run[n][j], base);
                            }
#pragma unroll
                        for (int c = 0; c < DK; ++c)
#pragma unroll
                            for (int n = 0; n < NQW; ++n)
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    float* at = my_park + (8 * (n0 + n) + 2 * tq + (e & 1)) * RS + 16 * c + g + 8 * (e >> 1);
                                    *at = *at * w_slot[n][e & 1] + o[c][n][e] * w_mine[n][e & 1];
                                }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(folded_bar);
                    merge_ok = mbar_wait(folded_bar, merges & 1, abort_flag, p);
                }
            }
            if (merge_ok) {
                constexpr uint32_t kVecs = D / 4;
                const uint32_t tid = warp * 32 + lane;
                for (uint32_t idx = tid; idx < uint32_t(G::kQRows) * kVecs; idx += CW * 32) {
                    const uint32_t row = idx / kVecs, d = (idx % kVecs) * 4;
                    const uint32_t row_tok = row / p.heads_per_task;
                    const uint32_t row_head = row % p.heads_per_task;
                    if (!(row_tok < t_num_toks && row_head < t_num_heads)) continue;
                    // (max, sum) of every slot: with two rounds, of the two states folded into it
                    float m_slot[NSLOT], l_slot[NSLOT];
                    float m_max = -INFINITY;
#pragma unroll
                    for (int w = 0; w < NSLOT; ++w) {
                        const float* stats = merge + w * G::kParkFloats + G::kQRows * RS;
                        m_slot[w] = stats[row];
                        l_slot[w] = stats[G::kQRows + row];
                        if constexpr (G::kTwoRounds) {
                            const float m_second = stats[2 * G::kQRows + row];
                            const float m_new = fmaxf(m_slot[w], m_second);
                            const float base = m_new == -INFINITY ? 0.0f : m_new;
                            l_slot[w] = l_slot[w] * weight_of(m_slot[w], base) +
                                        stats[3 * G::kQRows + row] * weight_of(m_second, base);
                            m_slot[w] = m_new;
                        }
                        m_max = fmaxf(m_max, m_slot[w]);
                    }
                    const float base = m_max == -INFINITY ? 0.0f : m_max;
                    float l_sum = 0.0f;
                    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                    for (int w = 0; w < NSLOT; ++w) {
                        const float weight = weight_of(m_slot[w], base);
                        l_sum += l_slot[w] * weight;
                        const float4 v = *reinterpret_cast<const float4*>(merge + w * G::kParkFloats + row * RS + d);
                        acc.x += weight * v.x;
                        acc.y += weight * v.y;
                        acc.z += weight * v.z;
                        acc.w += weight * v.w;
                    }
                    const float inv = l_sum > 0.0f ? 1.0f / l_sum : 0.0f;
                    acc.x *= inv;
                    acc.y *= inv;
                    acc.z *= inv;
                    acc.w *= inv;
                    const uint32_t head = t_head_begin + row_head;
                    if (write_final) {
                        T* dst = reinterpret_cast<T*>(p.out) + (uint64_t(t_tok_begin + row_tok) * p.num_q_heads + head) * D + d;
                        store_out4<T>(dst, acc);
                    } else {
                        const uint64_t index = (uint64_t(t_tmpl) * p.num_q_heads + head) * p.max_q_tokens + row_tok;
                        *reinterpret_cast<float4*>(p.partial_out + index * D + d) = acc;
                        if (d == 0) {
                            p.partial_sum[index] = l_sum;
                            // the running maximum is a raw dot product; publish the natural-log-domain logit
                            p.partial_max[index] = l_sum > 0.0f ? m_max * (p.scale_log2e * 0.6931471805599453f) : -INFINITY;
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(merged_bar);
                ++merges;
            }
            // ---- hand the task slot (descriptor + Q rows) back to the producer
            __syncwarp();
            if (lane == 0) mbar_arrive(task_empty_bar + 8 * tslot);
        }
    }
    __syncthreads();
}

}  // namespace kh
