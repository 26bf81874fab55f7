/*
 * CPU oracle for paged GQA split-KV scaled-dot-product attention.
 *
 * TEST INFRASTRUCTURE ONLY. This file is a plain-C restatement of the reference's CPU GQA SDPA
 * and of the index arithmetic its kernels share. It is the checker for the CUDA path and the
 * timed CPU baseline; the product library never links, loads or calls it.
 *
 * Parity pin: the restatement is checked against the reference's own known-answer tests
 * (crates/inference-executor-core/src/attn/gqa/reference.rs:84-115 and
 * crates/inference-executor-core/src/reference.rs:102-108). The reference is Rust and cannot be
 * compiled in this image, so those known answers (and the golden vectors of its host-side tests)
 * are the pin; no reference binary was run.
 *
 * Each function cites the reference file:line it follows (paths are relative to the reference
 * project root).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

#define KH_ORACLE_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------
 * softmax_reference: crates/inference-executor-core/src/reference.rs:15-31
 *   max-fold from -inf, exp(x - max), f32 sequential sum, divide.
 * Returns 0 on success, 1 when the reference would assert (empty input, or a total that is not
 * finite and positive).
 * ---------------------------------------------------------------------------------------- */
KH_ORACLE_API int kh_oracle_softmax(const float* logits, uint64_t n, float* out) {
    if (n == 0) return 1;
    float max_logit = -INFINITY;
    for (uint64_t i = 0; i < n; ++i) max_logit = fmaxf(max_logit, logits[i]);
    float total = 0.0f;
    for (uint64_t i = 0; i < n; ++i) {
        out[i] = expf(logits[i] - max_logit);
        total += out[i];
    }
    if (!(total > 0.0f) || !isfinite(total)) return 1;
    for (uint64_t i = 0; i < n; ++i) out[i] = out[i] / total;
    return 0;
}

/* One (token, q head) row of projected_gqa_reference:
 * crates/inference-executor-core/src/attn/gqa/reference.rs:44-73.
 * logits scratch must hold `visible` floats. */
static int oracle_row(const float* q_row, const float* k, const float* v, uint64_t visible, uint32_t num_kv_heads,
                      uint32_t head_dim, uint32_t kv_head, float scale, float* logits, float* out_row) {
    for (uint64_t t = 0; t < visible; ++t) {
        float dot = 0.0f;
        const float* key = k + (t * num_kv_heads + kv_head) * (uint64_t)head_dim;
        for (uint32_t d = 0; d < head_dim; ++d) dot += q_row[d] * key[d];
        logits[t] = dot * scale;
    }
    if (kh_oracle_softmax(logits, visible, logits)) return 1;
    for (uint32_t d = 0; d < head_dim; ++d) {
        float weighted = 0.0f;
        for (uint64_t t = 0; t < visible; ++t) {
            weighted += logits[t] * v[(t * num_kv_heads + kv_head) * (uint64_t)head_dim + d];
        }
        out_row[d] = weighted;
    }
    return 0;
}

/* ------------------------------------------------------------------------------------------
 * projected_gqa_reference: crates/inference-executor-core/src/attn/gqa/reference.rs:15-78
 * GQACore::validate: crates/inference-executor-core/src/attn/gqa/core.rs:33-41
 *
 *   cu_tokens[num_reqs + 1], token_indices[num_reqs] (history length of each request),
 *   q[T, Hq, D] f32, per-request contiguous K/V [ctx, Hkv, D] f32 with
 *   ctx = token_indices[r] + (cu_tokens[r+1] - cu_tokens[r]); out[T, Hq, D] f32.
 *   visible(token i of request r) = token_indices[r] + i + 1; kv_head = q_head / (Hq / Hkv).
 *
 * num_threads <= 1 runs the loops in the reference's order on one thread. num_threads > 1 runs
 * the independent (request, token, head) rows on OpenMP threads; every row's arithmetic is the
 * same sequence of operations, so no output bit changes.
 * Returns 0 on success, nonzero where the reference would assert.
 * ---------------------------------------------------------------------------------------- */
KH_ORACLE_API int kh_oracle_projected_gqa(uint32_t num_reqs, const uint32_t* cu_tokens, const uint32_t* token_indices,
                                          const float* q, const float* const* context_k_by_req,
                                          const float* const* context_v_by_req, uint32_t head_dim,
                                          uint32_t num_q_heads, uint32_t num_kv_heads, float scale, float* out,
                                          int32_t num_threads) {
    if (head_dim == 0 || num_q_heads == 0 || num_kv_heads == 0) return 2;
    if (num_q_heads % num_kv_heads != 0) return 2;
    if (!(scale > 0.0f)) return 2;
    if (cu_tokens[0] != 0) return 3;
    for (uint32_t r = 0; r < num_reqs; ++r) {
        if (cu_tokens[r] > cu_tokens[r + 1]) return 3;
    }
    const uint32_t group = num_q_heads / num_kv_heads;
    const uint64_t total_tokens = cu_tokens[num_reqs];
    uint64_t max_visible = 1;
    for (uint32_t r = 0; r < num_reqs; ++r) {
        uint64_t ctx = (uint64_t)token_indices[r] + (cu_tokens[r + 1] - cu_tokens[r]);
        if (ctx > max_visible) max_visible = ctx;
    }
    /* flat row list: row = token * Hq + head, with the owning request found by scan */
    uint32_t* req_of_token = (uint32_t*)malloc(sizeof(uint32_t) * (total_tokens ? total_tokens : 1));
    if (!req_of_token) return 4;
    for (uint32_t r = 0; r < num_reqs; ++r) {
        for (uint32_t t = cu_tokens[r]; t < cu_tokens[r + 1]; ++t) req_of_token[t] = r;
    }
    int failed = 0;
    const int64_t num_rows = (int64_t)(total_tokens * num_q_heads);
#ifdef _OPENMP
    int threads = num_threads > 1 ? num_threads : 1;
#pragma omp parallel num_threads(threads)
#endif
    {
        float* logits = (float*)malloc(sizeof(float) * max_visible);
#ifdef _OPENMP
#pragma omp for schedule(dynamic, 1)
#endif
        for (int64_t row = 0; row < num_rows; ++row) {
            const uint64_t token = (uint64_t)row / num_q_heads;
            const uint32_t head = (uint32_t)((uint64_t)row % num_q_heads);
            const uint32_t r = req_of_token[token];
            const uint64_t visible = (uint64_t)token_indices[r] + (token - cu_tokens[r]) + 1;
            if (!logits ||
                oracle_row(q + (token * num_q_heads + head) * (uint64_t)head_dim, context_k_by_req[r],
                           context_v_by_req[r], visible, num_kv_heads, head_dim, head / group, scale, logits,
                           out + (token * num_q_heads + head) * (uint64_t)head_dim)) {
#ifdef _OPENMP
#pragma omp atomic write
#endif
                failed = 1;
            }
        }
        free(logits);
    }
    (void)num_threads;
    free(req_of_token);
    return failed ? 5 : 0;
}

/* Windowed variant used by the reference's sliced-Q tests, which call the oracle on the slice
 * K[begin..end) with token_indices = end - begin - 1 (sliced_q_test.rs:186-199). One row. */
KH_ORACLE_API int kh_oracle_row(const float* q_row, const float* k, const float* v, uint64_t visible,
                                uint32_t num_kv_heads, uint32_t head_dim, uint32_t kv_head, float scale,
                                float* out_row) {
    if (visible == 0) return 1;
    float* logits = (float*)malloc(sizeof(float) * visible);
    if (!logits) return 4;
    int rc = oracle_row(q_row, k, v, visible, num_kv_heads, head_dim, kv_head, scale, logits, out_row);
    free(logits);
    return rc;
}

/* ------------------------------------------------------------------------------------------
 * Token -> page byte address, identical in every reference kernel:
 *   crates/inference-backend-metal/src/components/metal/gqa_sdpa_sliced_kv_map.metal:13-19
 *   crates/inference-backend-metal/src/components/metal/gqa_sdpa_sliced_q_map.metal:134-141,228-235
 *   crates/inference-backend-metal/src/components/metal/gqa_kv_page_write.metal:57-79
 * block = t / (P*n); i = (t / P) % n; table index = (((slot*L + layer)*B + block)*n + i);
 * byte address = page*page_bytes + ((plane*Hkv + kv_head)*P + t % P)*D*e, plane 0 = K, 1 = V.
 * Page layout [K/V][Hkv][P][D]: docs/executor_gqa.md:257-258, kv_page_write.rs:79-92.
 *
 * Gathers tokens [0, num_tokens) of one request into contiguous K and V [num_tokens, Hkv, D]
 * rows of elem_bytes-wide elements (bytes are moved, never converted). Also writes the byte
 * address of every (token, kv_head) K row and V row so index arithmetic can be compared bit
 * for bit. Returns nonzero when an index is out of range.
 * ---------------------------------------------------------------------------------------- */
KH_ORACLE_API int kh_oracle_gather_paged(const uint8_t* kv_pages, uint64_t kv_pages_bytes, const uint32_t* page_ids,
                                         uint64_t num_page_ids, uint32_t req_slot, uint32_t layer_index,
                                         uint32_t num_gqa_layers, uint32_t num_blocks,
                                         uint32_t num_page_ids_per_block, uint32_t tokens_per_page,
                                         uint32_t num_kv_heads, uint32_t head_dim, uint32_t elem_bytes,
                                         uint64_t num_tokens, uint8_t* out_k, uint8_t* out_v,
                                         uint64_t* out_k_addr, uint64_t* out_v_addr) {
    const uint64_t row_bytes = (uint64_t)head_dim * elem_bytes;
    const uint64_t page_bytes = 2ull * num_kv_heads * tokens_per_page * row_bytes;
    for (uint64_t t = 0; t < num_tokens; ++t) {
        const uint64_t block = t / ((uint64_t)tokens_per_page * num_page_ids_per_block);
        const uint64_t page_index = (t / tokens_per_page) % num_page_ids_per_block;
        if (block >= num_blocks) return 1;
        const uint64_t table_index =
            ((((uint64_t)req_slot * num_gqa_layers + layer_index) * num_blocks + block) * num_page_ids_per_block) +
            page_index;
        if (table_index >= num_page_ids) return 2;
        const uint64_t page = page_ids[table_index];
        for (uint32_t h = 0; h < num_kv_heads; ++h) {
            const uint64_t k_addr =
                page * page_bytes + (((uint64_t)0 * num_kv_heads + h) * tokens_per_page + t % tokens_per_page) * row_bytes;
            const uint64_t v_addr =
                page * page_bytes + (((uint64_t)1 * num_kv_heads + h) * tokens_per_page + t % tokens_per_page) * row_bytes;
            if (k_addr + row_bytes > kv_pages_bytes || v_addr + row_bytes > kv_pages_bytes) return 3;
            if (out_k) memcpy(out_k + (t * num_kv_heads + h) * row_bytes, kv_pages + k_addr, row_bytes);
            if (out_v) memcpy(out_v + (t * num_kv_heads + h) * row_bytes, kv_pages + v_addr, row_bytes);
            if (out_k_addr) out_k_addr[t * num_kv_heads + h] = k_addr;
            if (out_v_addr) out_v_addr[t * num_kv_heads + h] = v_addr;
        }
    }
    return 0;
}

/* Inverse of the gather: scatter contiguous K/V rows into pages (the byte layout the
 * reference's page-write kernel produces, gqa_kv_page_write.metal:57-79). Used to build test
 * pools. */
KH_ORACLE_API int kh_oracle_scatter_paged(uint8_t* kv_pages, uint64_t kv_pages_bytes, const uint32_t* page_ids,
                                          uint64_t num_page_ids, uint32_t req_slot, uint32_t layer_index,
                                          uint32_t num_gqa_layers, uint32_t num_blocks,
                                          uint32_t num_page_ids_per_block, uint32_t tokens_per_page,
                                          uint32_t num_kv_heads, uint32_t head_dim, uint32_t elem_bytes,
                                          uint64_t token_begin, uint64_t num_tokens, const uint8_t* k,
                                          const uint8_t* v) {
    const uint64_t row_bytes = (uint64_t)head_dim * elem_bytes;
    const uint64_t page_bytes = 2ull * num_kv_heads * tokens_per_page * row_bytes;
    for (uint64_t i = 0; i < num_tokens; ++i) {
        const uint64_t t = token_begin + i;
        const uint64_t block = t / ((uint64_t)tokens_per_page * num_page_ids_per_block);
        const uint64_t page_index = (t / tokens_per_page) % num_page_ids_per_block;
        if (block >= num_blocks) return 1;
        const uint64_t table_index =
            ((((uint64_t)req_slot * num_gqa_layers + layer_index) * num_blocks + block) * num_page_ids_per_block) +
            page_index;
        if (table_index >= num_page_ids) return 2;
        const uint64_t page = page_ids[table_index];
        for (uint32_t h = 0; h < num_kv_heads; ++h) {
            const uint64_t k_addr = page * page_bytes + ((uint64_t)h * tokens_per_page + t % tokens_per_page) * row_bytes;
            const uint64_t v_addr =
                page * page_bytes + (((uint64_t)num_kv_heads + h) * tokens_per_page + t % tokens_per_page) * row_bytes;
            if (k_addr + row_bytes > kv_pages_bytes || v_addr + row_bytes > kv_pages_bytes) return 3;
            memcpy(kv_pages + k_addr, k + (i * num_kv_heads + h) * row_bytes, row_bytes);
            memcpy(kv_pages + v_addr, v + (i * num_kv_heads + h) * row_bytes, row_bytes);
        }
    }
    return 0;
}

/* ------------------------------------------------------------------------------------------
 * FP8 E4M3FN storage codec of the reference's KV cache,
 *   crates/inference-backend-metal/src/components/gqa/fp8.rs:19-58
 * restated with the same arithmetic (log2 / floor / powers of two / round-ties-even in f32).
 * One fixed unit scale; finite and infinite magnitudes >= 448 saturate to 0x7e; NaN -> 0x7f.
 * ---------------------------------------------------------------------------------------- */
static float oracle_bf16_bits_to_f32(uint16_t bits) {
    const uint32_t wide = (uint32_t)bits << 16;
    float value;
    memcpy(&value, &wide, 4);
    return value;
}

KH_ORACLE_API uint8_t kh_oracle_fp8_from_bf16(uint16_t bf16_bits) {
    const float value = oracle_bf16_bits_to_f32(bf16_bits);
    const uint8_t sign = (bf16_bits & 0x8000u) ? 0x80 : 0;
    const float magnitude = fabsf(value);
    if (isnan(magnitude)) return sign | 0x7f;
    if (!isfinite(magnitude) || magnitude >= 448.0f) return sign | 0x7e;
    if (magnitude < 0.015625f) {
        const uint32_t mantissa = (uint32_t)nearbyintf(magnitude * 512.0f); /* ties to even */
        return sign | (uint8_t)(mantissa < 8u ? mantissa : 8u);
    }
    int exponent = (int)floorf(log2f(magnitude));
    uint32_t mantissa = (uint32_t)nearbyintf((magnitude * exp2f((float)-exponent) - 1.0f) * 8.0f);
    if (mantissa == 8u) {
        exponent += 1;
        mantissa = 0;
    }
    const int encoded = exponent + 7;
    if (encoded > 15 || (encoded == 15 && mantissa >= 7u)) return sign | 0x7e;
    return sign | (uint8_t)((uint32_t)encoded << 3) | (uint8_t)mantissa;
}

/* fp8.rs:46-58: returns the bf16 bits of the decoded value. */
KH_ORACLE_API uint16_t kh_oracle_fp8_to_bf16(uint8_t bits) {
    const uint32_t exponent = (bits >> 3) & 0x0fu;
    const uint32_t mantissa = bits & 0x07u;
    const uint16_t sign = (bits & 0x80u) ? 0x8000 : 0;
    if (exponent == 15 && mantissa == 7) return sign | 0x7fc0;
    const float magnitude = exponent == 0 ? (float)mantissa / 512.0f
                                          : (1.0f + (float)mantissa / 8.0f) * exp2f((float)exponent - 7.0f);
    uint32_t wide;
    memcpy(&wide, &magnitude, 4); /* exact in bf16: at most 4 significant bits */
    return sign | (uint16_t)(wide >> 16);
}

/* ------------------------------------------------------------------------------------------
 * Partial-state merge (split-KV reduce), docs/gqa_sdpa_selection.md:443-460 and
 *   crates/inference-backend-metal/src/components/metal/gqa_sdpa_sliced_kv_reduce.metal:30-55
 *   crates/inference-backend-metal/src/components/metal/gqa_sdpa_sliced_q_reduce.metal:26-62
 * max = max_i m_i; weight_i = isfinite(m_i) && l_i != 0 ? exp(m_i - max) * l_i : 0;
 * out = sum_i weight_i * o_i / sum_i weight_i (0 when the denominator is 0); natural-log domain,
 * o_i normalised. Merges num_partials partial rows of width head_dim for one (token, head).
 * Also returns the merged (max, sum) so a second merge level (across GPUs) can be chained.
 * ---------------------------------------------------------------------------------------- */
KH_ORACLE_API void kh_oracle_merge_partials(uint32_t num_partials, const float* exp_sums, const float* max_logits,
                                            const float* partial_out, uint64_t partial_stride, uint32_t head_dim,
                                            float* out, float* out_exp_sum, float* out_max_logit) {
    float global_max = -INFINITY;
    for (uint32_t i = 0; i < num_partials; ++i) global_max = fmaxf(global_max, max_logits[i]);
    float global_sum = 0.0f;
    for (uint32_t d = 0; d < head_dim; ++d) out[d] = 0.0f;
    for (uint32_t i = 0; i < num_partials; ++i) {
        const float weight =
            (isfinite(max_logits[i]) && exp_sums[i] != 0.0f) ? expf(max_logits[i] - global_max) * exp_sums[i] : 0.0f;
        global_sum += weight;
        for (uint32_t d = 0; d < head_dim; ++d) out[d] += weight * partial_out[i * partial_stride + d];
    }
    for (uint32_t d = 0; d < head_dim; ++d) out[d] = global_sum > 0.0f ? out[d] / global_sum : 0.0f;
    if (out_exp_sum) *out_exp_sum = global_sum;
    if (out_max_logit) *out_max_logit = global_sum > 0.0f ? global_max : -INFINITY;
}

/* One split-KV partial of one (token, head) row over K/V tokens [kv_begin, kv_end): the
 * natural-log-domain (max, exp_sum, normalised out) triple the map kernels publish
 * (gqa_sdpa_sliced_kv_map.metal:165-210; empty range -> exp_sum 0, max -inf, out 0). Used by the
 * CPU-rank simulation of the cross-GPU split. */
KH_ORACLE_API void kh_oracle_partial_row(const float* q_row, const float* k, const float* v, uint64_t kv_begin,
                                         uint64_t kv_end, uint32_t num_kv_heads, uint32_t head_dim, uint32_t kv_head,
                                         float scale, float* out_row, float* out_exp_sum, float* out_max_logit) {
    for (uint32_t d = 0; d < head_dim; ++d) out_row[d] = 0.0f;
    if (kv_end <= kv_begin) {
        *out_exp_sum = 0.0f;
        *out_max_logit = -INFINITY;
        return;
    }
    const uint64_t n = kv_end - kv_begin;
    float* logits = (float*)malloc(sizeof(float) * n);
    float max_logit = -INFINITY;
    for (uint64_t t = 0; t < n; ++t) {
        float dot = 0.0f;
        const float* key = k + ((kv_begin + t) * num_kv_heads + kv_head) * (uint64_t)head_dim;
        for (uint32_t d = 0; d < head_dim; ++d) dot += q_row[d] * key[d];
        logits[t] = dot * scale;
        max_logit = fmaxf(max_logit, logits[t]);
    }
    float total = 0.0f;
    for (uint64_t t = 0; t < n; ++t) {
        logits[t] = expf(logits[t] - max_logit);
        total += logits[t];
    }
    for (uint32_t d = 0; d < head_dim; ++d) {
        float weighted = 0.0f;
        for (uint64_t t = 0; t < n; ++t) {
            weighted += logits[t] * v[((kv_begin + t) * num_kv_heads + kv_head) * (uint64_t)head_dim + d];
        }
        out_row[d] = total > 0.0f ? weighted / total : 0.0f;
    }
    *out_exp_sum = total;
    *out_max_logit = total > 0.0f ? max_logit : -INFINITY;
    free(logits);
}

/* ------------------------------------------------------------------------------------------
 * bfloat16 <-> f32, round to nearest even (half 2.7.1 bf16::from_f32, pinned in the reference's
 * Cargo.lock; used only to round I/O tensors, as the reference tests do in
 * sliced_kv_test.rs:484-493). NaN stays NaN (quiet bit set).
 * ---------------------------------------------------------------------------------------- */
KH_ORACLE_API uint16_t kh_oracle_f32_to_bf16(float value) {
    uint32_t bits;
    memcpy(&bits, &value, 4);
    if ((bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((bits >> 16) | 0x0040u);
    const uint32_t round_bit = 0x00008000u;
    if ((bits & round_bit) != 0 && (bits & (3u * round_bit - 1u)) != 0) return (uint16_t)((bits >> 16) + 1u);
    return (uint16_t)(bits >> 16);
}

KH_ORACLE_API float kh_oracle_bf16_to_f32(uint16_t bits) {
    uint32_t wide = (uint32_t)bits << 16;
    float value;
    memcpy(&value, &wide, 4);
    return value;
}

KH_ORACLE_API void kh_oracle_round_bf16(const float* in, uint64_t n, uint16_t* out_bits, float* out_f32) {
    for (uint64_t i = 0; i < n; ++i) {
        uint16_t b = kh_oracle_f32_to_bf16(in[i]);
        if (out_bits) out_bits[i] = b;
        if (out_f32) out_f32[i] = kh_oracle_bf16_to_f32(b);
    }
}

/* Deterministic generators of the reference tests (formulas, not data):
 *   generated_values: sliced_kv_test.rs:501-509   value = ((state>>8)/2^24)*2 - 1
 *   generated_bf16_values: sliced_q_test.rs:611-619  value = bf16(((state>>8)/2^24) - 0.5)
 *   fixture_values: sliced_kv_test.rs:495-499
 * with state = state*1664525 + 1013904223 (wrapping u32). */
KH_ORACLE_API void kh_oracle_generated_values(uint64_t n, uint32_t seed, int32_t centered_bf16, float* out) {
    uint32_t state = seed;
    for (uint64_t i = 0; i < n; ++i) {
        state = state * 1664525u + 1013904223u;
        const float unit = (float)(state >> 8) / 16777216.0f;
        out[i] = centered_bf16 ? kh_oracle_bf16_to_f32(kh_oracle_f32_to_bf16(unit - 0.5f)) : unit * 2.0f - 1.0f;
    }
}

KH_ORACLE_API void kh_oracle_fixture_values(uint64_t n, float scale, uint64_t pattern_offset, float* out) {
    for (uint64_t i = 0; i < n; ++i) out[i] = (float)((i * 11 + pattern_offset) % 23) * scale - 11.0f * scale;
}

KH_ORACLE_API int32_t kh_oracle_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
