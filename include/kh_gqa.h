/*
 * kh_gqa.h -- C ABI of libkhcuda_gqa: paged GQA split-KV scaled-dot-product attention for
 * NVIDIA B200 (sm_100a).
 *
 * This is the boundary a Rust `inference-backend-cuda` crate (or any other host) binds. It
 * replaces, for the attention path only, what the reference reaches through its Metal backend:
 * device / buffer / stream objects, the SDPA capability registry, the SDPA selector and its
 * batch metadata, the request page table, and the SlicedKv / SlicedQ `Compute` objects with
 * their map / reduce / direct invocations. Every entry point cites the reference interface it
 * stands in for; paths are relative to the reference project root, with
 *   BM = crates/inference-backend-metal/src,  EM = crates/inference-executor-metal/src,
 *   EC = crates/inference-executor-core/src.
 *
 * Conventions
 *  - Every function returns a kh_status. On failure a thread-local message is available from
 *    kh_last_error(). Nothing unwinds across this boundary: each `assert!` of the reference's
 *    `validate()` functions is a checked KH_INVALID_ARGUMENT here.
 *  - Device buffers are passed as (pointer, byte length) pairs (kh_buffer_ref). The library
 *    never allocates inside a map / reduce / direct call and never synchronises the stream, so
 *    the calls can be captured into a CUDA graph (the analogue of the reference's recorded
 *    replay program).
 *  - Handles are not thread-safe; one owner thread per handle, as in the reference executor.
 *  - All metadata arrays are little-endian u32 and bit-identical to the reference's
 *    GQAMetadataBuffers (EM/attn/gqa/batch_metadata.rs:100-253).
 */
#ifndef KH_GQA_H_
#define KH_GQA_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(_WIN32)
#define KH_API
#else
#define KH_API __attribute__((visibility("default")))
#endif

/* ---- status codes: variant names of crates/inference-error/src/lib.rs:4-28 ---------------- */
typedef int32_t kh_status;
enum {
    KH_OK = 0,
    KH_INVALID_ARGUMENT = 1,
    KH_RESOURCE_EXHAUSTED = 2,
    KH_CANCELLED = 3,
    KH_DEADLINE_EXCEEDED = 4,
    KH_ABORTED = 5,
    KH_EVICTED = 6,
    KH_UNAVAILABLE = 7,
    KH_INTERNAL = 8
};

/* Copies the calling thread's last error message (NUL terminated) into buf; returns its length. */
KH_API size_t kh_last_error(char* buf, size_t len);
/* Library version string; also proves the library and its CUDA objects loaded. */
KH_API const char* kh_version(void);

/* ---- element types: the subset of BM/metal/dtype.rs:1-16 this path uses -------------------- */
typedef uint32_t kh_dtype;
enum {
    KH_DTYPE_FLOAT16 = 9,   /* Dtype::Float16 (ordinal in the reference enum) */
    KH_DTYPE_FLOAT32 = 10,  /* Dtype::Float32 */
    KH_DTYPE_BFLOAT16 = 12, /* Dtype::Bfloat16 */
    KH_DTYPE_FP8_E4M3FN = 100 /* KV-cache only; the reference's native cache format (BM/components/gqa/fp8.rs) */
};

/* ---- device, buffers, streams (stand in for BM/metal/{device,buffer,stream}) --------------- */
typedef struct kh_device kh_device;
typedef struct kh_stream kh_stream;

typedef struct kh_buffer_ref {
    void* ptr;      /* device pointer */
    uint64_t bytes; /* usable byte length starting at ptr */
} kh_buffer_ref;

/* Device::system_default (BM/metal/device.rs:12-15): opens CUDA device `ordinal`. */
KH_API kh_status kh_device_open(int32_t ordinal, kh_device** out);
KH_API kh_status kh_device_close(kh_device* device);
KH_API kh_status kh_device_sm_count(const kh_device* device, int32_t* out);
/* Buffer::new_zeroed (BM/metal/buffer.rs): device allocation, zero filled. */
KH_API kh_status kh_buffer_alloc(kh_device* device, uint64_t bytes, kh_buffer_ref* out);
KH_API kh_status kh_buffer_free(kh_device* device, kh_buffer_ref buffer);
/* Buffer::write_typed / read_typed / zero_bytes: synchronous host <-> device copies. */
KH_API kh_status kh_buffer_write(kh_device* device, kh_buffer_ref buffer, uint64_t offset, const void* src,
                                 uint64_t bytes);
KH_API kh_status kh_buffer_read(kh_device* device, kh_buffer_ref buffer, uint64_t offset, void* dst, uint64_t bytes);
KH_API kh_status kh_buffer_zero(kh_device* device, kh_buffer_ref buffer, uint64_t offset, uint64_t bytes);
/* Stream::new (BM/metal/stream/mod.rs); kh_stream_wrap adopts an existing cudaStream_t. */
KH_API kh_status kh_stream_create(kh_device* device, kh_stream** out);
KH_API kh_status kh_stream_wrap(kh_device* device, void* cuda_stream, kh_stream** out);
/* Replay counts, the analogue of ReplayU32::Parameter (BM/metal/stream/replay.rs; bound in
 * sliced_kv.rs:571-582, sliced_q.rs:565-582, kv-side contract in docs/executor_gqa.md:476-532). While a buffer is
 * bound to the stream, every SlicedKv / SlicedQ map, direct and reduce launch recorded on it sizes its grid from
 * the num_active_* arguments of the call - pass the recorded capacities (`num_total_*`) - and READS the counts it
 * works with from `active_counts` when the kernel runs: four u32 {num_active_tokens, num_active_q_token_tiles,
 * num_active_kv_splits, 0}, each clamped to the capacity passed at the call. A launch captured into a CUDA graph
 * can therefore be replayed for a new batch after the metadata arrays and these four words have been rewritten
 * (on the same stream, before the graph launch). Bind a null buffer to return to by-value counts. */
KH_API kh_status kh_stream_bind_active_counts(kh_stream* stream, kh_buffer_ref active_counts);
KH_API kh_status kh_stream_destroy(kh_stream* stream);
/* ReplaySubmission::wait (BM/metal/stream/submission.rs:88). */
KH_API kh_status kh_stream_synchronize(kh_stream* stream);
/* Stream-ordered host <-> device copies (pinned host memory recommended). */
KH_API kh_status kh_stream_write(kh_stream* stream, kh_buffer_ref buffer, uint64_t offset, const void* src,
                                 uint64_t bytes);
KH_API kh_status kh_stream_read(kh_stream* stream, kh_buffer_ref buffer, uint64_t offset, void* dst, uint64_t bytes);
KH_API kh_status kh_host_alloc_pinned(uint64_t bytes, void** out);
KH_API kh_status kh_host_free_pinned(void* ptr);
/* Completion of one submission, the analogue of ReplaySubmission (BM/metal/stream/submission.rs:41-101): an event
 * is recorded on a stream after the work it stands for; kh_event_synchronize blocks the host until that work is
 * done (ReplaySubmission::wait, submission.rs:88), kh_stream_wait_event orders another stream of the same device
 * after it without blocking the host (the recorded barrier of BM/metal/stream/dependency.rs:11-16 across two
 * queues). With them a caller keeps two steps in flight: the output copy of one step runs on a second stream
 * while the next step's kernels run on the first. */
typedef struct kh_event kh_event;
KH_API kh_status kh_event_create(kh_device* device, kh_event** out);
KH_API kh_status kh_event_destroy(kh_event* event);
KH_API kh_status kh_stream_record_event(kh_stream* stream, kh_event* event);
KH_API kh_status kh_stream_wait_event(kh_stream* stream, kh_event* event);
KH_API kh_status kh_event_synchronize(kh_event* event);

/* ---- SDPA capability registry: BM/components/gqa/sdpa.rs ----------------------------------- */
/* sdpa::Config (sdpa.rs:219-241). */
typedef struct kh_sdpa_config {
    kh_dtype io_dtype;
    uint32_t num_q_heads;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    uint32_t tokens_per_page;
} kh_sdpa_config;

/* MapKernelKind (sdpa.rs:22-28). */
typedef uint32_t kh_map_kernel_kind;
enum { KH_MAP_SLICED_KV = 0, KH_MAP_Q_TOKENS_PER_HEAD = 1, KH_MAP_Q_HEADS_PER_TOKEN = 2, KH_MAP_Q_TOKENS_AND_HEADS = 3 };

/* ExecutionVariant flattened (sdpa.rs:7-57): map.kind, map.thread_block.*, map.kv_cache.*, reduce.thread_block.*. */
typedef struct kh_execution_variant {
    kh_map_kernel_kind kind;
    uint32_t max_q_tokens;
    uint32_t max_q_heads;
    uint32_t kv_tokens_per_iteration;
    uint32_t required_threads;
    uint32_t tokens_per_page;
    uint32_t reduce_max_q_tokens;
    uint32_t reduce_max_q_heads;
    uint32_t reduce_required_threads;
} kh_execution_variant;

/* Config::validate (sdpa.rs:229-236). */
KH_API kh_status kh_sdpa_config_validate(const kh_sdpa_config* config);
/* ExecutionVariant::sliced_kv (sdpa.rs:60-88). */
KH_API kh_status kh_variant_sliced_kv(const kh_sdpa_config* config, uint32_t kv_tokens_per_iteration,
                                      uint32_t required_threads, uint32_t max_q_heads, kh_execution_variant* out);
/* ExecutionVariant::sliced_q / sliced_q_per_head (sdpa.rs:90-160). */
KH_API kh_status kh_variant_sliced_q(const kh_sdpa_config* config, kh_map_kernel_kind kind, uint32_t max_q_tokens,
                                     uint32_t kv_tokens_per_iteration, uint32_t max_q_heads,
                                     kh_execution_variant* out);
/* ExecutionVariant::supports (sdpa.rs:162-215): *out = 1 when the variant is legal for config. */
KH_API kh_status kh_variant_supports(const kh_execution_variant* variant, const kh_sdpa_config* config,
                                     int32_t* out);
/* Registry::new(config).variants() (sdpa.rs:255-271): writes up to `capacity` variants, sets *count. */
KH_API kh_status kh_registry_variants(const kh_sdpa_config* config, kh_execution_variant* out, uint32_t capacity,
                                      uint32_t* count);

/* ---- page table: EM/attn/gqa/request_page_table.rs, BM/components/gqa/kv_page_write.rs:33-57 */
typedef struct kh_page_table_layout {
    uint32_t num_req_slots;
    uint32_t num_gqa_layers;
    uint32_t num_blocks;
    uint32_t num_page_ids_per_block;
} kh_page_table_layout;

/* PageTableLayout::bytes (kv_page_write.rs:49-56). */
KH_API kh_status kh_page_table_bytes(const kh_page_table_layout* layout, uint64_t* out);
/* GQARequestPageTable::page_ids_start_index (request_page_table.rs:151-156): u32 element index of
 * page_ids[req_slot][layer][block][0]. */
KH_API kh_status kh_page_table_index(const kh_page_table_layout* layout, uint32_t req_slot, uint32_t layer_index,
                                     uint32_t block_index, uint64_t* out);
/* write_page_ids / read_page_ids / reset_req_slot (request_page_table.rs:86-122) on a device table. */
KH_API kh_status kh_page_table_write(kh_device* device, kh_buffer_ref page_ids, const kh_page_table_layout* layout,
                                     uint32_t req_slot, uint32_t layer_index, uint32_t block_index,
                                     const uint32_t* ids, uint32_t count);
KH_API kh_status kh_page_table_read(kh_device* device, kh_buffer_ref page_ids, const kh_page_table_layout* layout,
                                    uint32_t req_slot, uint32_t layer_index, uint32_t block_index, uint32_t* ids,
                                    uint32_t count);
KH_API kh_status kh_page_table_reset_req_slot(kh_device* device, kh_buffer_ref page_ids,
                                              const kh_page_table_layout* layout, uint32_t req_slot);

/* ---- replay buckets: EC/replay.rs:4-88, EM/attn/gqa/batch_metadata.rs:68-96 ---------------- */
/* ReplayBucketPolicy::new(max).buckets(): writes up to `capacity` buckets, sets *count to the total. */
KH_API kh_status kh_replay_buckets(uint32_t max_capacity, uint32_t* out, uint32_t capacity, uint32_t* count);
/* ReplayBucketPolicy::new(max).capacity(active). */
KH_API kh_status kh_replay_capacity(uint32_t max_capacity, uint32_t active, uint32_t* out);

/* GQAReplayShape (batch_metadata.rs:11-61). */
typedef struct kh_replay_shape {
    uint32_t num_tokens;
    uint32_t num_total_tokens;
    uint32_t num_q_token_tiles;
    uint32_t num_total_q_token_tiles;
    uint32_t num_sdpa_map_task_templates;
    uint32_t num_total_sdpa_map_task_templates;
    uint32_t reduce_sdpa_partial_outputs; /* bool */
} kh_replay_shape;

/* ---- selector: EM/attn/gqa/sdpa.rs ---------------------------------------------------------- */
/* RequestShape (sdpa.rs:15-19). */
typedef struct kh_request_shape {
    uint32_t num_history_tokens;
    uint32_t num_q_tokens;
} kh_request_shape;

/* SelectorLimits (sdpa.rs:43-48). */
typedef struct kh_selector_limits {
    uint32_t max_tokens;
    uint32_t max_map_task_templates;
    uint64_t partial_state_group_capacity;
} kh_selector_limits;

/* SelectionMetrics (sdpa.rs:64-77). */
typedef struct kh_selection_metrics {
    uint64_t num_scheduled_qk_token_pairs;
    uint64_t num_active_qk_token_pairs;
    uint64_t num_map_threadblocks_per_kv_head;
    uint64_t num_map_simdgroup_waves_per_kv_head;
    uint64_t num_active_partial_state_groups;
    uint64_t num_active_partial_states;
    uint64_t num_reserved_partial_state_groups;
    uint64_t num_replay_reserved_partial_state_groups;
    uint64_t num_logical_qk_token_pairs;
    uint32_t max_kv_iterations_per_split;
    uint32_t reserved;
} kh_selection_metrics;

/* QTokenRange (sdpa.rs:50-56). */
typedef struct kh_q_token_range {
    uint32_t request_index;
    uint32_t flat_q_token_begin;
    uint32_t flat_q_token_end;
    uint32_t num_visible_kv_tokens;
} kh_q_token_range;

/* MapTaskTemplate (sdpa.rs:58-62): the three-u32 record the kernels read. */
typedef struct kh_map_task_template {
    uint32_t q_token_range_index;
    uint32_t kv_token_begin;
    uint32_t kv_token_end;
} kh_map_task_template;

typedef struct kh_selector kh_selector;
typedef struct kh_selection kh_selection;

/* Which routing policy `kh_selector_select` applies. */
typedef uint32_t kh_selector_policy;
enum {
    KH_POLICY_REFERENCE = 0, /* the reference's rules, bit for bit (calibrated for a 40-core Apple GPU) */
    KH_POLICY_B200 = 1       /* same route table, KV slice re-derived for `sm_count` SMs */
};

/* Selector::new(Registry::from_variants(config, variants), ...) (sdpa.rs:137-165, sdpa.rs:276-285).
 * Pass num_variants = 0 to use Registry::new(config). */
KH_API kh_status kh_selector_create(const kh_sdpa_config* config, const kh_execution_variant* variants,
                                    uint32_t num_variants, uint32_t max_tokens, uint32_t max_map_task_templates,
                                    uint64_t partial_state_group_capacity, kh_selector** out);
/* Selector::for_lookup (sdpa.rs:210-276). */
KH_API kh_status kh_selector_create_for_lookup(const kh_sdpa_config* config, uint32_t max_tokens,
                                               const kh_page_table_layout* layout, kh_selector** out);
/* Selector::for_partitions (sdpa.rs:170-207); max_kv_splits[i] belongs to variants[i]. */
KH_API kh_status kh_selector_create_for_partitions(const kh_sdpa_config* config,
                                                   const kh_execution_variant* variants, uint32_t num_variants,
                                                   const uint32_t* max_kv_splits, uint32_t max_tokens,
                                                   uint32_t max_requests, kh_selector** out);
KH_API kh_status kh_selector_destroy(kh_selector* selector);
KH_API kh_status kh_selector_limits_get(const kh_selector* selector, kh_selector_limits* out);
KH_API kh_status kh_selector_variants(const kh_selector* selector, kh_execution_variant* out, uint32_t capacity,
                                      uint32_t* count);
/* Sets the routing policy and the SM count the KH_POLICY_B200 slice rule targets. */
KH_API kh_status kh_selector_set_policy(kh_selector* selector, kh_selector_policy policy, uint32_t sm_count);

/* Selector::select (sdpa.rs:278-380). The replay bucket policy is
 * GQAReplayBucketPolicy::new(policy_max_tokens, policy_max_map_task_templates). */
KH_API kh_status kh_selector_select(const kh_selector* selector, const kh_request_shape* requests,
                                    uint32_t num_requests, uint32_t policy_max_tokens,
                                    uint32_t policy_max_map_task_templates, uint32_t num_total_tokens,
                                    kh_selection** out);
/* Selector::select_partitioned (sdpa.rs:382-426). */
KH_API kh_status kh_selector_select_partitioned(const kh_selector* selector, const kh_execution_variant* variant,
                                                uint32_t kv_slice, int32_t direct_output,
                                                const kh_request_shape* requests, uint32_t num_requests,
                                                uint32_t policy_max_tokens, uint32_t policy_max_map_task_templates,
                                                uint32_t num_total_tokens, kh_selection** out);
KH_API kh_status kh_selection_destroy(kh_selection* selection);
/* Selection accessors (sdpa.rs:99-125). Array getters write up to `capacity` records and set *count. */
KH_API kh_status kh_selection_variant(const kh_selection* selection, kh_execution_variant* out);
KH_API kh_status kh_selection_direct_output(const kh_selection* selection, int32_t* out);
KH_API kh_status kh_selection_replay_shape(const kh_selection* selection, kh_replay_shape* out);
KH_API kh_status kh_selection_metrics_get(const kh_selection* selection, kh_selection_metrics* out);
KH_API kh_status kh_selection_q_token_ranges(const kh_selection* selection, kh_q_token_range* out, uint32_t capacity,
                                             uint32_t* count);
KH_API kh_status kh_selection_map_task_templates(const kh_selection* selection, kh_map_task_template* out,
                                                 uint32_t capacity, uint32_t* count);
KH_API kh_status kh_selection_cu_partial_outputs(const kh_selection* selection, uint32_t* out, uint32_t capacity,
                                                 uint32_t* count);

/* ---- batch metadata: EM/attn/gqa/batch_metadata.rs:100-253 ---------------------------------- */
/* Host images of the six device arrays GQAMetadataBuffers::update uploads. The caller owns the
 * arrays (capacities in elements); `update` fills them exactly as the reference fills its
 * buffers, including the u32::MAX padding of map templates up to the padded capacity, and does
 * not touch q_token_ranges for a SlicedKv selection. Elements past what `update` writes keep
 * their previous contents. */
typedef struct kh_metadata_arrays {
    uint32_t* req_slots;               /* [max_tokens] */
    uint32_t* flat_token_indices;      /* [max_tokens] */
    uint32_t* visible_kv_token_ranges; /* [max_tokens][2] */
    uint32_t* q_token_ranges;          /* [max_tokens][2] */
    uint32_t* sdpa_map_task_templates; /* [max_map_task_templates][3] */
    uint32_t* cu_sdpa_partial_outputs; /* [max_tokens + 1] */
    uint32_t max_tokens;
    uint32_t max_map_task_templates;
} kh_metadata_arrays;

KH_API kh_status kh_metadata_update(const kh_metadata_arrays* arrays, const uint32_t* req_slots,
                                    const uint32_t* token_indices, const uint32_t* cu_tokens, uint32_t num_requests,
                                    const kh_selection* selection, kh_replay_shape* out_shape);

/* ---- SlicedKv compute: BM/components/gqa/sdpa/sliced_kv.rs ---------------------------------- */
/* sliced_kv::Config (sliced_kv.rs:90-98) plus the KV-cache element type, which the reference
 * fixes at one byte (sliced_kv.rs:113-125) and this library makes a parameter. tokens per page =
 * page_bytes / (2 * num_kv_heads * head_dim * sizeof(kv_dtype)).
 * kv_dtype = KH_DTYPE_FP8_E4M3FN: the reference's cache format; codes are decoded on load exactly as
 * metal/gqa_fp8.metal:1-25 does (16-token pages, head_dim 128 or 256). kv_dtype = dtype: the pages hold
 * Q/output-type elements. */
typedef struct kh_sliced_kv_config {
    uint32_t num_q_heads;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    float scale;
    uint32_t page_bytes;
    kh_page_table_layout page_table_layout;
    kh_dtype dtype;    /* Q / output element type */
    kh_dtype kv_dtype; /* K/V page element type */
} kh_sliced_kv_config;

/* sliced_kv::Shape (sliced_kv.rs:215-219). */
typedef struct kh_sliced_kv_shape {
    uint32_t num_total_tokens;
    uint32_t num_total_sdpa_map_task_templates;
} kh_sliced_kv_shape;

/* sliced_kv::MapBuffers (sliced_kv.rs:236-246), binding order 0..7 of MapInvocation::record
 * (sliced_kv.rs:562-569). Partial statistics are f32 [Mt][Hq]; partial_output is f32 [Mt][Hq][D]
 * (the reference stores it in the io dtype; this library keeps it in f32). */
typedef struct kh_sliced_kv_map_buffers {
    kh_buffer_ref q;
    kh_buffer_ref kv_pages;
    kh_buffer_ref req_slots;
    kh_buffer_ref page_ids;
    kh_buffer_ref sdpa_map_task_templates;
    kh_buffer_ref partial_exp_sums;
    kh_buffer_ref partial_max_logits;
    kh_buffer_ref partial_output;
} kh_sliced_kv_map_buffers;

/* sliced_kv::ReduceBuffers (sliced_kv.rs:248-254). */
typedef struct kh_sliced_kv_reduce_buffers {
    kh_buffer_ref partial_exp_sums;
    kh_buffer_ref partial_max_logits;
    kh_buffer_ref partial_output;
    kh_buffer_ref cu_sdpa_partial_outputs;
    kh_buffer_ref output;
} kh_sliced_kv_reduce_buffers;

/* Byte sizes of Config (sliced_kv.rs:140-212). */
typedef struct kh_sliced_kv_sizes {
    uint64_t q_bytes;
    uint64_t req_slots_bytes;
    uint64_t page_ids_bytes;
    uint64_t sdpa_map_task_templates_bytes;
    uint64_t cu_sdpa_partial_outputs_bytes;
    uint64_t partial_output_stats_bytes;
    uint64_t partial_output_bytes;
    uint32_t num_tokens_per_page;
    uint32_t reserved;
} kh_sliced_kv_sizes;

typedef struct kh_sliced_kv kh_sliced_kv;

/* Config::validate + Shape::validate + byte sizes. */
KH_API kh_status kh_sliced_kv_sizes_get(const kh_sliced_kv_config* config, const kh_sliced_kv_shape* shape,
                                        kh_sliced_kv_sizes* out);
/* Compute::new(device, config, execution, shape) (sliced_kv.rs:322-355). */
KH_API kh_status kh_sliced_kv_create(kh_device* device, const kh_sliced_kv_config* config,
                                     const kh_execution_variant* execution, const kh_sliced_kv_shape* shape,
                                     kh_sliced_kv** out);
KH_API kh_status kh_sliced_kv_destroy(kh_sliced_kv* compute);
/* Compute::invoke_map(...).record (sliced_kv.rs:357-375, 558-592). */
KH_API kh_status kh_sliced_kv_map(kh_sliced_kv* compute, kh_stream* stream, const kh_sliced_kv_map_buffers* buffers,
                                  uint32_t page_table_index, uint32_t num_active_tokens,
                                  uint32_t num_active_kv_splits);
/* Compute::invoke_reduce(...).record (sliced_kv.rs:377-388, 623-638). */
KH_API kh_status kh_sliced_kv_reduce(kh_sliced_kv* compute, kh_stream* stream,
                                     const kh_sliced_kv_reduce_buffers* buffers, uint32_t num_active_tokens);

/* Map and reduce in ONE launch: what `invoke_map` followed by `invoke_reduce` computes
 * (EM/attn/gqa/backend.rs:458-482 records them back to back with a barrier between). Every map task still
 * publishes its partial through the buffers of `map_buffers`; the thread block that publishes the last partial of a
 * (token, KV head, Q-head range) group merges that group while the partials are still in L2 and writes `output`.
 * No block waits for another. A token with a single partial is written directly.
 * `arrival_counters` is scratch owned by the caller: kh_sliced_kv_arrival_counter_bytes() bytes, zero before the
 * first call; every call leaves it zero again. Calls that share it must not overlap on the GPU. Every map task
 * template of an active token must be active (as the selector's metadata guarantees). */
KH_API kh_status kh_sliced_kv_map_reduce(kh_sliced_kv* compute, kh_stream* stream,
                                         const kh_sliced_kv_map_buffers* map_buffers,
                                         const kh_sliced_kv_reduce_buffers* reduce_buffers, kh_buffer_ref arrival_counters,
                                         uint32_t page_table_index, uint32_t num_active_tokens,
                                         uint32_t num_active_kv_splits);
KH_API kh_status kh_sliced_kv_arrival_counter_bytes(const kh_sliced_kv_config* config,
                                                    const kh_execution_variant* execution,
                                                    const kh_sliced_kv_shape* shape, uint64_t* out);

/* ---- SlicedKv attention on scratch the library holds: no allocation on any call ---------------
 * No counterpart in the reference, whose layer owners allocate the partial-state scratch themselves
 * (EM/attn/gqa/scratch.rs:49-83). This entry is for a host that cannot hand the library device memory for the
 * partials and must not have it allocate either: an executor whose device arena is sized and frozen at start-up, a
 * step loop with a latency bound (a device allocation or free synchronises the whole GPU), or a caller that is
 * already inside a region where allocation is not allowed. It computes what kh_sliced_kv_map followed by
 * kh_sliced_kv_reduce compute, bit for bit, with the partial statistics and partial outputs in one array that is part
 * of the loaded library image (KH_STATIC_PARTIALS_BYTES per GPU, present from module load, never freed).
 *  - Limit: num_active_kv_splits * num_q_heads * (head_dim + 2) * 4 bytes (rounded up to 256-byte sections) must
 *    fit KH_STATIC_PARTIALS_BYTES; a larger batch is refused with KH_RESOURCE_EXHAUSTED and the message names the
 *    bytes needed - use kh_sliced_kv_map / kh_sliced_kv_reduce with buffers of your own for those.
 *  - The first call on each GPU looks up the array's address (set-up; no launch is involved), and the first call
 *    of a compute object with a new Q buffer or KV pool encodes their tensor maps on the host. Make one call per
 *    GPU and buffer pair before any stream capture or timed region; later calls only launch kernels.
 *  - All calls on one GPU share the array. Nothing in it has to be zero: the map stage writes every partial that
 *    the reduce stage of the same call reads. Two calls whose kernels can overlap on the GPU (different streams
 *    without an ordering between them) race on it; calls ordered on one stream, or by events, are safe. */
#define KH_STATIC_PARTIALS_BYTES (32u << 20)

typedef struct kh_sliced_kv_static_buffers {
    kh_buffer_ref q;
    kh_buffer_ref kv_pages;
    kh_buffer_ref req_slots;
    kh_buffer_ref page_ids;
    kh_buffer_ref sdpa_map_task_templates;
    kh_buffer_ref cu_sdpa_partial_outputs;
    kh_buffer_ref output;
} kh_sliced_kv_static_buffers;

KH_API kh_status kh_sliced_kv_attend_static(kh_sliced_kv* compute, kh_stream* stream,
                                            const kh_sliced_kv_static_buffers* buffers, uint32_t page_table_index,
                                            uint32_t num_active_tokens, uint32_t num_active_kv_splits);
/* Bytes of the shared array a call with these counts needs (the quantity checked against the limit). */
KH_API kh_status kh_sliced_kv_static_bytes_needed(const kh_sliced_kv_config* config, uint32_t num_active_kv_splits,
                                                  uint64_t* out);

/* ---- SlicedQ compute: BM/components/gqa/sdpa/sliced_q.rs ------------------------------------ */
/* sliced_q::Config (sliced_q.rs:145-153) plus kv_dtype (as in kh_sliced_kv_config; the reference fixes one
 * byte per element, sliced_q.rs:202). */
typedef struct kh_sliced_q_config {
    uint32_t num_q_heads;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    float scale;
    uint32_t page_bytes;
    kh_dtype dtype;
    kh_page_table_layout page_table_layout;
    kh_dtype kv_dtype;
} kh_sliced_q_config;

/* sliced_q::Shape (sliced_q.rs:248-253). */
typedef struct kh_sliced_q_shape {
    uint32_t num_total_tokens;
    uint32_t num_total_q_token_tiles;
    uint32_t num_total_sdpa_map_task_templates;
} kh_sliced_q_shape;

/* sliced_q::MapBuffers (sliced_q.rs:308-321). Partial ABI: statistics f32 [Mt][Hq][max_q_tokens],
 * output f32 [Mt][Hq][max_q_tokens][D] (sliced_q.rs:78-101, io dtype there, f32 here). */
typedef struct kh_sliced_q_map_buffers {
    kh_buffer_ref q;
    kh_buffer_ref kv_pages;
    kh_buffer_ref req_slots;
    kh_buffer_ref page_ids;
    kh_buffer_ref visible_kv_token_ranges;
    kh_buffer_ref q_token_ranges;
    kh_buffer_ref sdpa_map_task_templates;
    kh_buffer_ref partial_output;
    kh_buffer_ref partial_exp_sums;
    kh_buffer_ref partial_max_logits;
} kh_sliced_q_map_buffers;

/* sliced_q::DirectBuffers (sliced_q.rs:325-335). */
typedef struct kh_sliced_q_direct_buffers {
    kh_buffer_ref q;
    kh_buffer_ref kv_pages;
    kh_buffer_ref req_slots;
    kh_buffer_ref page_ids;
    kh_buffer_ref visible_kv_token_ranges;
    kh_buffer_ref q_token_ranges;
    kh_buffer_ref sdpa_map_task_templates;
    kh_buffer_ref output;
} kh_sliced_q_direct_buffers;

/* sliced_q::ReduceBuffers (sliced_q.rs:337-345). */
typedef struct kh_sliced_q_reduce_buffers {
    kh_buffer_ref partial_output;
    kh_buffer_ref partial_exp_sums;
    kh_buffer_ref partial_max_logits;
    kh_buffer_ref q_token_ranges;
    kh_buffer_ref cu_sdpa_partial_outputs;
    kh_buffer_ref output;
} kh_sliced_q_reduce_buffers;

typedef struct kh_sliced_q_sizes {
    uint64_t q_bytes;
    uint64_t partial_output_bytes;
    uint64_t partial_output_stats_bytes;
    uint32_t num_tokens_per_page;
    uint32_t reserved;
} kh_sliced_q_sizes;

typedef struct kh_sliced_q kh_sliced_q;

KH_API kh_status kh_sliced_q_sizes_get(const kh_sliced_q_config* config, const kh_execution_variant* execution,
                                       const kh_sliced_q_shape* shape, kh_sliced_q_sizes* out);
/* Compute::new / Compute::new_direct (sliced_q.rs:356-363). */
KH_API kh_status kh_sliced_q_create(kh_device* device, const kh_sliced_q_config* config,
                                    const kh_execution_variant* execution, const kh_sliced_q_shape* shape,
                                    int32_t direct_output, kh_sliced_q** out);
KH_API kh_status kh_sliced_q_destroy(kh_sliced_q* compute);
/* Compute::invoke_map(...).record (sliced_q.rs:417-454, 547-592). */
KH_API kh_status kh_sliced_q_map(kh_sliced_q* compute, kh_stream* stream, const kh_sliced_q_map_buffers* buffers,
                                 uint32_t page_table_index, uint32_t num_active_tokens,
                                 uint32_t num_active_q_token_tiles, uint32_t num_active_kv_splits);
/* Compute::invoke_direct(...).record (sliced_q.rs:456-482). */
KH_API kh_status kh_sliced_q_direct(kh_sliced_q* compute, kh_stream* stream,
                                    const kh_sliced_q_direct_buffers* buffers, uint32_t page_table_index,
                                    uint32_t num_active_tokens, uint32_t num_active_q_token_tiles);
/* Compute::invoke_reduce(...).record (sliced_q.rs:484-503, 617-642). */
KH_API kh_status kh_sliced_q_reduce(kh_sliced_q* compute, kh_stream* stream,
                                    const kh_sliced_q_reduce_buffers* buffers, uint32_t num_active_q_token_tiles);

/* Map and reduce in one launch for the sliced-Q variants (EM/attn/gqa/backend.rs:506-540); same contract as
 * kh_sliced_kv_map_reduce, with one arrival counter per (Q-token tile, KV head, Q-head range). */
KH_API kh_status kh_sliced_q_map_reduce(kh_sliced_q* compute, kh_stream* stream,
                                        const kh_sliced_q_map_buffers* map_buffers,
                                        const kh_sliced_q_reduce_buffers* reduce_buffers, kh_buffer_ref arrival_counters,
                                        uint32_t page_table_index, uint32_t num_active_tokens,
                                        uint32_t num_active_q_token_tiles, uint32_t num_active_kv_splits);
KH_API kh_status kh_sliced_q_arrival_counter_bytes(const kh_sliced_q_config* config,
                                                   const kh_execution_variant* execution,
                                                   const kh_sliced_q_shape* shape, uint64_t* out);

/* ---- KV page write: BM/components/gqa/kv_page_write.rs, gqa_kv_page_write.metal:32-80 ------- */
/* kv_page_write::Config (kv_page_write.rs:62-68) plus the stored element type. The reference stores FP8 E4M3FN
 * (`kv_dtype` = KH_DTYPE_FP8_E4M3FN, conversion of BM/components/gqa/fp8.rs:19-44: nearest-even, saturating at
 * 448, NaN kept); `kv_dtype == dtype` stores the source bits unchanged, the page format the attention kernels
 * of this library read. tokens per page = page_bytes / (2 * num_kv_heads * head_dim * sizeof(kv_dtype)). */
typedef struct kh_kv_page_write_config {
    uint32_t num_kv_heads;
    uint32_t head_dim;
    uint32_t page_bytes;
    kh_dtype dtype;    /* flat_k / flat_v element type: Bfloat16 (the reference's) or Float16 */
    kh_dtype kv_dtype;
} kh_kv_page_write_config;

/* kv_page_write::Shape (kv_page_write.rs:123-127). */
typedef struct kh_kv_page_write_shape {
    uint32_t num_total_token_writes;
    kh_page_table_layout page_table_layout;
} kh_kv_page_write_shape;

/* kv_page_write::Buffers (kv_page_write.rs:143-151), binding order 0..5 of Invocation::record (:211-216):
 * flat_k / flat_v are [writes][Hkv][D]; write i goes to request slot req_slots[i], absolute token position
 * flat_token_indices[i]. */
typedef struct kh_kv_page_write_buffers {
    kh_buffer_ref pages;
    kh_buffer_ref flat_k;
    kh_buffer_ref flat_v;
    kh_buffer_ref req_slots;
    kh_buffer_ref flat_token_indices;
    kh_buffer_ref page_ids;
} kh_kv_page_write_buffers;

typedef struct kh_kv_page_write kh_kv_page_write;

/* Compute::new (kv_page_write.rs:158-167). */
KH_API kh_status kh_kv_page_write_create(kh_device* device, const kh_kv_page_write_config* config,
                                         kh_kv_page_write** out);
KH_API kh_status kh_kv_page_write_destroy(kh_kv_page_write* compute);
/* Config::num_tokens_per_page (kv_page_write.rs:80-92). */
KH_API kh_status kh_kv_page_write_tokens_per_page(const kh_kv_page_write_config* config, uint32_t* out);
/* Compute::invoke(...).record (kv_page_write.rs:169-236): writes the first num_active_token_writes entries.
 * A page id beyond the pool is not written and sets bit 1 of the device status word. */
KH_API kh_status kh_kv_page_write_invoke(kh_kv_page_write* compute, kh_stream* stream,
                                         const kh_kv_page_write_shape* shape, const kh_kv_page_write_buffers* buffers,
                                         uint32_t num_active_token_writes, uint32_t page_table_index);
/* bf16_to_fp8_e4m3 / fp8_e4m3_to_bf16 (BM/components/gqa/fp8.rs:19-58) on bit patterns, host side. */
KH_API uint8_t kh_fp8_e4m3_from_bf16(uint16_t bf16_bits);
KH_API uint16_t kh_fp8_e4m3_to_bf16(uint8_t fp8_bits);

/* ---- BiDi-block SDPA: BM/components/gqa/bidi_block_sdpa.rs, metal/gqa_bidi_block_sdpa.metal:10-88 -------------
 * Dense bidirectional attention of every Q token over ALL tokens of its own request block (the proposal block a
 * DFlash2 drafter works on; K/V of the block are contiguous [tokens][Hkv][D] rows, not yet in the paged cache),
 * written as one more partial into the SplitKV partial-state layout: slot cu_sdpa_partial_outputs[range + 1] - 1 of
 * the token's Q-token range, index ((slot * Hq + head) * max_q_tokens + token offset) (gqa_bidi_block_sdpa.metal:36,
 * 64-66). The sliced-Q map kernel fills the range's other slots with (sliding-window) history partials and the
 * sliced-Q reducer merges them all (BM/components/gqa/bidi_block_sdpa_test.rs:174-330 records map, block, reduce).
 * Statistics as everywhere: exp sums relative to the maximum logit, maxima in the natural-log domain. Partial outputs
 * are f32 here (the reference stores the io dtype). */
/* bidi_block_sdpa::Config (bidi_block_sdpa.rs:56-64). head_dim must be a multiple of 32. */
typedef struct kh_bidi_block_sdpa_config {
    uint32_t block_size;
    uint32_t max_q_tokens;
    uint32_t num_q_heads;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    float scale;
    kh_dtype dtype; /* q / local_k / local_v element type: Bfloat16, Float16 or Float32 */
} kh_bidi_block_sdpa_config;

/* bidi_block_sdpa::Shape (bidi_block_sdpa.rs:141-145). num_total_tokens must hold complete request blocks. */
typedef struct kh_bidi_block_sdpa_shape {
    uint32_t num_total_tokens;
    uint32_t num_total_q_token_ranges;
    uint32_t num_total_partial_output_slots;
} kh_bidi_block_sdpa_shape;

/* bidi_block_sdpa::Buffers (bidi_block_sdpa.rs:177-186), binding order 0..7 of Invocation::record (:262-269). */
typedef struct kh_bidi_block_sdpa_buffers {
    kh_buffer_ref q;
    kh_buffer_ref local_k;
    kh_buffer_ref local_v;
    kh_buffer_ref q_token_ranges;
    kh_buffer_ref cu_sdpa_partial_outputs;
    kh_buffer_ref partial_exp_sums;
    kh_buffer_ref partial_max_logits;
    kh_buffer_ref partial_output;
} kh_bidi_block_sdpa_buffers;

typedef struct kh_bidi_block_sdpa kh_bidi_block_sdpa;

/* Compute::new (bidi_block_sdpa.rs:193-229). */
KH_API kh_status kh_bidi_block_sdpa_create(kh_device* device, const kh_bidi_block_sdpa_config* config,
                                           kh_bidi_block_sdpa** out);
KH_API kh_status kh_bidi_block_sdpa_destroy(kh_bidi_block_sdpa* compute);
/* Compute::invoke(shape, num_active_q_token_ranges, buffers).record (bidi_block_sdpa.rs:231-283, validation
 * :286-330). With replay counts bound to the stream the active range count is read on the device (word 1). */
KH_API kh_status kh_bidi_block_sdpa_invoke(kh_bidi_block_sdpa* compute, kh_stream* stream,
                                           const kh_bidi_block_sdpa_shape* shape, uint32_t num_active_q_token_ranges,
                                           const kh_bidi_block_sdpa_buffers* buffers);

/* build_metal_metadata of the BiDi-block GQA owner (EM/attn/bidi_block_gqa/metadata.rs:176-339): the metadata of one
 * proposal step. Tokens come in request blocks of `block_size` (request r owns flat tokens [r * block_size,
 * (r + 1) * block_size)); token t sees cached history tokens [history_begins[t], history_ends[t]) of its request (a
 * sliding window) plus its whole block. Per Q-token range (at most max_q_tokens tokens of one block): history map
 * task templates over the union of its tokens' history ranges, cut on multiples of kv_tokens_per_iteration into as
 * many splits as the template capacity allows (allocate_history_kv_splits, :341-367: longest range first, later
 * ranges win ties), then ONE padded template (u32::MAX), whose index is the block partial's slot. The template count
 * is padded to a power of two. Fills visible_kv_token_ranges, q_token_ranges, sdpa_map_task_templates,
 * cu_sdpa_partial_outputs, and - when req_slots / token_positions are given - req_slots and flat_token_indices. */
KH_API kh_status kh_bidi_block_metadata_build(const kh_metadata_arrays* arrays, const uint32_t* req_slots,
                                              const uint32_t* token_positions, const uint32_t* history_begins,
                                              const uint32_t* history_ends, uint32_t num_requests, uint32_t block_size,
                                              uint32_t max_q_tokens, uint32_t kv_tokens_per_iteration,
                                              uint32_t max_sdpa_map_task_templates, kh_replay_shape* out_shape);

/* ---- device status word: the analogue of SubmissionCheck (BM/metal/stream/check.rs:8-13) ---- */
/* Reads (after synchronising the stream) and clears the sticky status the kernels of `device`
 * write: 0 = clean; bit 0 = a bounded wait inside a kernel ran out; bit 1 = a page id addressed
 * beyond the KV pool (the copy or write was skipped); bit 2 = batch metadata named a request slot or a KV range
 * beyond the page table (the task or token write was skipped). Nonzero also returns KH_ABORTED. */
KH_API kh_status kh_device_check(kh_device* device, kh_stream* stream, uint32_t* out_status_word);
/* Every wait inside a kernel (on a copy or on another warp) polls at most `polls` times, then the kernel sets
 * bit 0 of the status word, lets its copies in flight land and returns. The default (2^24 polls, seconds) is far
 * above any healthy wait; a watchdog-style caller, or a test of the abort path, lowers it. 0 restores the default.
 * Applies to launches recorded after the call. No reference counterpart: Metal command buffers carry their own
 * GPU timeout (surfaced by SubmissionCheck, BM/metal/stream/check.rs:8-13). */
KH_API kh_status kh_device_set_wait_limit(kh_device* device, uint32_t polls);

/* ---- cross-partition / cross-GPU LSE combine ------------------------------------------------ */
/* Merges `num_partials` partial triples per (token, head) row with the partial-state merge of
 * docs/gqa_sdpa_selection.md:443-460 (the formula of gqa_sdpa_sliced_kv_reduce.metal:30-55).
 * Layout: exp_sums / max_logits f32 [num_partials][num_rows], partial_output f32
 * [num_partials][num_rows][head_dim], rows = tokens * num_q_heads. Writes `output` in `out_dtype`
 * ([num_rows][head_dim]); when out_exp_sums / out_max_logits are non-null also writes the merged
 * statistics (f32 [num_rows]) so merges can be chained (per GPU, then across GPUs after an
 * all-gather). The reference has no multi-device path; this is the merge its reducer applies,
 * exposed for partials that arrive from other GPUs. */
KH_API kh_status kh_combine_partials(kh_device* device, kh_stream* stream, uint32_t num_partials, uint32_t num_rows,
                                     uint32_t head_dim, kh_buffer_ref exp_sums, kh_buffer_ref max_logits,
                                     kh_buffer_ref partial_output, kh_dtype out_dtype, kh_buffer_ref output,
                                     kh_buffer_ref out_exp_sums, kh_buffer_ref out_max_logits);

/* The same merge over records gathered from several GPUs. Each GPU contributes one record of
 * num_rows * (head_dim + 2) f32: [exp sums: num_rows][max logits: num_rows][output: num_rows x head_dim], which
 * is what kh_combine_partials writes when its three outputs point into one buffer at those offsets; `packed`
 * holds `num_partials` such records back to back, the layout an all-gather of one record per rank leaves in
 * local memory. One collective per attention call, then this merge on local memory; no peer memory is read. */
KH_API kh_status kh_combine_packed_partials(kh_device* device, kh_stream* stream, uint32_t num_partials,
                                            uint32_t num_rows, uint32_t head_dim, kh_buffer_ref packed,
                                            kh_dtype out_dtype, kh_buffer_ref output);

/* ---- cross-GPU combine in one kernel over NVLink peer memory ---------------------------------------------------
 * No counterpart in the reference (one device). For one long sequence whose pages are split over the GPUs of a
 * node: every GPU runs its local split-KV map, then ONE launch of kh_peer_exchange_combine on every GPU merges
 * this GPU's partials, stores the merged (max, sum, output) rows straight into every peer's inbox (plain peer
 * stores through NVSwitch), flags them, waits - bounded - for the other ranks' rows and writes the final output on
 * every GPU. It stands in for kh_combine_partials + an all-gather + kh_combine_packed_partials.
 *  - Every rank allocates an inbox of kh_peer_exchange_inbox_bytes() with kh_buffer_alloc (zero filled: the step
 *    counters start at zero), exports it (kh_ipc_export, a 64-byte CUDA IPC handle to hand to the other processes
 *    by any host channel), imports the peers' (kh_ipc_import) and creates the exchange with the `world` inbox
 *    pointers in rank order, its own entry being the local buffer.
 *  - Every rank must call combine the same number of times: a call is step n on every rank. Calls of one rank are
 *    ordered on its stream. The kernels of the ranks wait for one another, so every rank needs a GPU of its own.
 *  - A peer that does not arrive within the device's wait limit (kh_device_set_wait_limit) sets bit 0 of the status
 *    word; the output row is then not written and the kernel returns.
 *  - num_partials may be 0 (a rank that holds no token of the sequence): it contributes empty rows. */
typedef struct kh_peer_exchange kh_peer_exchange;
KH_API kh_status kh_peer_exchange_inbox_bytes(uint32_t world, uint32_t num_rows, uint32_t head_dim, uint64_t* out);
KH_API kh_status kh_ipc_export(kh_device* device, kh_buffer_ref buffer, uint8_t* handle64);
KH_API kh_status kh_ipc_import(kh_device* device, const uint8_t* handle64, void** out);
KH_API kh_status kh_ipc_close(kh_device* device, void* ptr);
KH_API kh_status kh_peer_exchange_create(kh_device* device, uint32_t rank, uint32_t world, uint32_t num_rows,
                                         uint32_t head_dim, void* const* inboxes, kh_peer_exchange** out);
KH_API kh_status kh_peer_exchange_destroy(kh_peer_exchange* exchange);
/* Local partials as kh_combine_partials takes them: exp_sums / max_logits f32 [num_partials][num_rows],
 * partial_output f32 [num_partials][num_rows][head_dim]; output [num_rows][head_dim] in out_dtype. */
KH_API kh_status kh_peer_exchange_combine(kh_peer_exchange* exchange, kh_stream* stream, uint32_t num_partials,
                                          kh_buffer_ref exp_sums, kh_buffer_ref max_logits,
                                          kh_buffer_ref partial_output, kh_dtype out_dtype, kh_buffer_ref output);

#ifdef __cplusplus
}
#endif

#endif /* KH_GQA_H_ */
