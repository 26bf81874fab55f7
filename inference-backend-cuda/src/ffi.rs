//! Raw declarations of `include/kh_gqa.h`, one for one. Not compiled here; see Cargo.toml.
//!
//! Every struct is `#[repr(C)]` with the header's field order; every function returns `kh_status` (`i32`), never
//! unwinds, and leaves a thread-local message for `kh_last_error`. The reference interface each entry stands in
//! for is cited beside its declaration in the header.
#![allow(non_camel_case_types)]

pub type KhStatus = i32;
pub const KH_OK: KhStatus = 0;
pub const KH_INVALID_ARGUMENT: KhStatus = 1;
pub const KH_RESOURCE_EXHAUSTED: KhStatus = 2;
pub const KH_CANCELLED: KhStatus = 3;
pub const KH_DEADLINE_EXCEEDED: KhStatus = 4;
pub const KH_ABORTED: KhStatus = 5;
pub const KH_EVICTED: KhStatus = 6;
pub const KH_UNAVAILABLE: KhStatus = 7;
pub const KH_INTERNAL: KhStatus = 8;

pub const KH_DTYPE_FLOAT16: u32 = 9;
pub const KH_DTYPE_FLOAT32: u32 = 10;
pub const KH_DTYPE_BFLOAT16: u32 = 12;
pub const KH_DTYPE_FP8_E4M3FN: u32 = 100;

pub const KH_MAP_SLICED_KV: u32 = 0;
pub const KH_MAP_Q_TOKENS_PER_HEAD: u32 = 1;
pub const KH_MAP_Q_HEADS_PER_TOKEN: u32 = 2;
pub const KH_MAP_Q_TOKENS_AND_HEADS: u32 = 3;

pub const KH_POLICY_REFERENCE: u32 = 0;
pub const KH_POLICY_B200: u32 = 1;

/// Bytes of the partial-state array `kh_sliced_kv_attend_static` works in.
pub const KH_STATIC_PARTIALS_BYTES: u64 = 32 << 20;

/// Bits of the device status word `kh_device_check` returns.
pub const KH_STATUS_WAIT_EXPIRED: u32 = 1;
pub const KH_STATUS_PAGE_OUT_OF_POOL: u32 = 2;
pub const KH_STATUS_METADATA_OUT_OF_RANGE: u32 = 4;

/// Opaque handle (`kh_device`).
#[repr(C)]
pub struct KhDevice {
    _private: [u8; 0],
}

/// Opaque handle (`kh_stream`).
#[repr(C)]
pub struct KhStream {
    _private: [u8; 0],
}

/// Opaque handle (`kh_event`).
#[repr(C)]
pub struct KhEvent {
    _private: [u8; 0],
}

/// Opaque handle (`kh_peer_exchange`).
#[repr(C)]
pub struct KhPeerExchange {
    _private: [u8; 0],
}

/// Opaque handle (`kh_selector`).
#[repr(C)]
pub struct KhSelector {
    _private: [u8; 0],
}

/// Opaque handle (`kh_selection`).
#[repr(C)]
pub struct KhSelection {
    _private: [u8; 0],
}

/// Opaque handle (`kh_sliced_kv`).
#[repr(C)]
pub struct KhSlicedKv {
    _private: [u8; 0],
}

/// Opaque handle (`kh_sliced_q`).
#[repr(C)]
pub struct KhSlicedQ {
    _private: [u8; 0],
}

/// Opaque handle (`kh_kv_page_write`).
#[repr(C)]
pub struct KhKvPageWrite {
    _private: [u8; 0],
}

/// Opaque handle (`kh_bidi_block_sdpa`).
#[repr(C)]
pub struct KhBidiBlockSdpa {
    _private: [u8; 0],
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhBufferRef {
    pub ptr: *mut core::ffi::c_void,
    pub bytes: u64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhSdpaConfig {
    pub io_dtype: u32,
    pub num_q_heads: u32,
    pub num_kv_heads: u32,
    pub head_dim: u32,
    pub tokens_per_page: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhExecutionVariant {
    pub kind: u32,
    pub max_q_tokens: u32,
    pub max_q_heads: u32,
    pub kv_tokens_per_iteration: u32,
    pub required_threads: u32,
    pub tokens_per_page: u32,
    pub reduce_max_q_tokens: u32,
    pub reduce_max_q_heads: u32,
    pub reduce_required_threads: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhPageTableLayout {
    pub num_req_slots: u32,
    pub num_gqa_layers: u32,
    pub num_blocks: u32,
    pub num_page_ids_per_block: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhReplayShape {
    pub num_tokens: u32,
    pub num_total_tokens: u32,
    pub num_q_token_tiles: u32,
    pub num_total_q_token_tiles: u32,
    pub num_sdpa_map_task_templates: u32,
    pub num_total_sdpa_map_task_templates: u32,
    pub reduce_sdpa_partial_outputs: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhRequestShape {
    pub num_history_tokens: u32,
    pub num_q_tokens: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhSelectorLimits {
    pub max_tokens: u32,
    pub max_map_task_templates: u32,
    pub partial_state_group_capacity: u64,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhSelectionMetrics {
    pub num_scheduled_qk_token_pairs: u64,
    pub num_active_qk_token_pairs: u64,
    pub num_map_threadblocks_per_kv_head: u64,
    pub num_map_simdgroup_waves_per_kv_head: u64,
    pub num_active_partial_state_groups: u64,
    pub num_active_partial_states: u64,
    pub num_reserved_partial_state_groups: u64,
    pub num_replay_reserved_partial_state_groups: u64,
    pub num_logical_qk_token_pairs: u64,
    pub max_kv_iterations_per_split: u32,
    pub reserved: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhQTokenRange {
    pub request_index: u32,
    pub flat_q_token_begin: u32,
    pub flat_q_token_end: u32,
    pub num_visible_kv_tokens: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhMapTaskTemplate {
    pub q_token_range_index: u32,
    pub kv_token_begin: u32,
    pub kv_token_end: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhMetadataArrays {
    pub req_slots: *mut u32,
    pub flat_token_indices: *mut u32,
    pub visible_kv_token_ranges: *mut u32,
    pub q_token_ranges: *mut u32,
    pub sdpa_map_task_templates: *mut u32,
    pub cu_sdpa_partial_outputs: *mut u32,
    pub max_tokens: u32,
    pub max_map_task_templates: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhSlicedKvConfig {
    pub num_q_heads: u32,
    pub num_kv_heads: u32,
    pub head_dim: u32,
    pub scale: f32,
    pub page_bytes: u32,
    pub page_table_layout: KhPageTableLayout,
    pub dtype: u32,
    pub kv_dtype: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhSlicedKvShape {
    pub num_total_tokens: u32,
    pub num_total_sdpa_map_task_templates: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhSlicedKvMapBuffers {
    pub q: KhBufferRef,
    pub kv_pages: KhBufferRef,
    pub req_slots: KhBufferRef,
    pub page_ids: KhBufferRef,
    pub sdpa_map_task_templates: KhBufferRef,
    pub partial_exp_sums: KhBufferRef,
    pub partial_max_logits: KhBufferRef,
    pub partial_output: KhBufferRef,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhSlicedKvReduceBuffers {
    pub partial_exp_sums: KhBufferRef,
    pub partial_max_logits: KhBufferRef,
    pub partial_output: KhBufferRef,
    pub cu_sdpa_partial_outputs: KhBufferRef,
    pub output: KhBufferRef,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhSlicedKvSizes {
    pub q_bytes: u64,
    pub req_slots_bytes: u64,
    pub page_ids_bytes: u64,
    pub sdpa_map_task_templates_bytes: u64,
    pub cu_sdpa_partial_outputs_bytes: u64,
    pub partial_output_stats_bytes: u64,
    pub partial_output_bytes: u64,
    pub num_tokens_per_page: u32,
    pub reserved: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhSlicedKvStaticBuffers {
    pub q: KhBufferRef,
    pub kv_pages: KhBufferRef,
    pub req_slots: KhBufferRef,
    pub page_ids: KhBufferRef,
    pub sdpa_map_task_templates: KhBufferRef,
    pub cu_sdpa_partial_outputs: KhBufferRef,
    pub output: KhBufferRef,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhSlicedQConfig {
    pub num_q_heads: u32,
    pub num_kv_heads: u32,
    pub head_dim: u32,
    pub scale: f32,
    pub page_bytes: u32,
    pub dtype: u32,
    pub page_table_layout: KhPageTableLayout,
    pub kv_dtype: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhSlicedQShape {
    pub num_total_tokens: u32,
    pub num_total_q_token_tiles: u32,
    pub num_total_sdpa_map_task_templates: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhSlicedQMapBuffers {
    pub q: KhBufferRef,
    pub kv_pages: KhBufferRef,
    pub req_slots: KhBufferRef,
    pub page_ids: KhBufferRef,
    pub visible_kv_token_ranges: KhBufferRef,
    pub q_token_ranges: KhBufferRef,
    pub sdpa_map_task_templates: KhBufferRef,
    pub partial_output: KhBufferRef,
    pub partial_exp_sums: KhBufferRef,
    pub partial_max_logits: KhBufferRef,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhSlicedQDirectBuffers {
    pub q: KhBufferRef,
    pub kv_pages: KhBufferRef,
    pub req_slots: KhBufferRef,
    pub page_ids: KhBufferRef,
    pub visible_kv_token_ranges: KhBufferRef,
    pub q_token_ranges: KhBufferRef,
    pub sdpa_map_task_templates: KhBufferRef,
    pub output: KhBufferRef,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhSlicedQReduceBuffers {
    pub partial_output: KhBufferRef,
    pub partial_exp_sums: KhBufferRef,
    pub partial_max_logits: KhBufferRef,
    pub q_token_ranges: KhBufferRef,
    pub cu_sdpa_partial_outputs: KhBufferRef,
    pub output: KhBufferRef,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhSlicedQSizes {
    pub q_bytes: u64,
    pub partial_output_bytes: u64,
    pub partial_output_stats_bytes: u64,
    pub num_tokens_per_page: u32,
    pub reserved: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhKvPageWriteConfig {
    pub num_kv_heads: u32,
    pub head_dim: u32,
    pub page_bytes: u32,
    pub dtype: u32,
    pub kv_dtype: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhKvPageWriteShape {
    pub num_total_token_writes: u32,
    pub page_table_layout: KhPageTableLayout,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhKvPageWriteBuffers {
    pub pages: KhBufferRef,
    pub flat_k: KhBufferRef,
    pub flat_v: KhBufferRef,
    pub req_slots: KhBufferRef,
    pub flat_token_indices: KhBufferRef,
    pub page_ids: KhBufferRef,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhBidiBlockSdpaConfig {
    pub block_size: u32,
    pub max_q_tokens: u32,
    pub num_q_heads: u32,
    pub num_kv_heads: u32,
    pub head_dim: u32,
    pub scale: f32,
    pub dtype: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhBidiBlockSdpaShape {
    pub num_total_tokens: u32,
    pub num_total_q_token_ranges: u32,
    pub num_total_partial_output_slots: u32,
}

#[repr(C)]
#[derive(Clone, Copy, Debug)]
pub struct KhBidiBlockSdpaBuffers {
    pub q: KhBufferRef,
    pub local_k: KhBufferRef,
    pub local_v: KhBufferRef,
    pub q_token_ranges: KhBufferRef,
    pub cu_sdpa_partial_outputs: KhBufferRef,
    pub partial_exp_sums: KhBufferRef,
    pub partial_max_logits: KhBufferRef,
    pub partial_output: KhBufferRef,
}

#[link(name = "khcuda_gqa")]
unsafe extern "C" {
    pub fn kh_last_error(buf: *mut core::ffi::c_char, len: usize) -> usize;
    pub fn kh_version() -> *const core::ffi::c_char;
    pub fn kh_device_open(ordinal: i32, out: *mut *mut KhDevice) -> KhStatus;
    pub fn kh_device_close(device: *mut KhDevice) -> KhStatus;
    pub fn kh_device_sm_count(device: *const KhDevice, out: *mut i32) -> KhStatus;
    pub fn kh_buffer_alloc(device: *mut KhDevice, bytes: u64, out: *mut KhBufferRef) -> KhStatus;
    pub fn kh_buffer_free(device: *mut KhDevice, buffer: KhBufferRef) -> KhStatus;
    pub fn kh_buffer_write(
        device: *mut KhDevice,
        buffer: KhBufferRef,
        offset: u64,
        src: *const core::ffi::c_void,
        bytes: u64,
    ) -> KhStatus;
    pub fn kh_buffer_read(
        device: *mut KhDevice,
        buffer: KhBufferRef,
        offset: u64,
        dst: *mut core::ffi::c_void,
        bytes: u64,
    ) -> KhStatus;
    pub fn kh_buffer_zero(device: *mut KhDevice, buffer: KhBufferRef, offset: u64, bytes: u64) -> KhStatus;
    pub fn kh_stream_create(device: *mut KhDevice, out: *mut *mut KhStream) -> KhStatus;
    pub fn kh_stream_wrap(
        device: *mut KhDevice,
        cuda_stream: *mut core::ffi::c_void,
        out: *mut *mut KhStream,
    ) -> KhStatus;
    pub fn kh_stream_bind_active_counts(stream: *mut KhStream, active_counts: KhBufferRef) -> KhStatus;
    pub fn kh_stream_destroy(stream: *mut KhStream) -> KhStatus;
    pub fn kh_stream_synchronize(stream: *mut KhStream) -> KhStatus;
    pub fn kh_stream_write(
        stream: *mut KhStream,
        buffer: KhBufferRef,
        offset: u64,
        src: *const core::ffi::c_void,
        bytes: u64,
    ) -> KhStatus;
    pub fn kh_stream_read(
        stream: *mut KhStream,
        buffer: KhBufferRef,
        offset: u64,
        dst: *mut core::ffi::c_void,
        bytes: u64,
    ) -> KhStatus;
    pub fn kh_host_alloc_pinned(bytes: u64, out: *mut *mut core::ffi::c_void) -> KhStatus;
    pub fn kh_host_free_pinned(ptr: *mut core::ffi::c_void) -> KhStatus;
    pub fn kh_event_create(device: *mut KhDevice, out: *mut *mut KhEvent) -> KhStatus;
    pub fn kh_event_destroy(event: *mut KhEvent) -> KhStatus;
    pub fn kh_stream_record_event(stream: *mut KhStream, event: *mut KhEvent) -> KhStatus;
    pub fn kh_stream_wait_event(stream: *mut KhStream, event: *mut KhEvent) -> KhStatus;
    pub fn kh_event_synchronize(event: *mut KhEvent) -> KhStatus;
    pub fn kh_sdpa_config_validate(config: *const KhSdpaConfig) -> KhStatus;
    pub fn kh_variant_sliced_kv(
        config: *const KhSdpaConfig,
        kv_tokens_per_iteration: u32,
        required_threads: u32,
        max_q_heads: u32,
        out: *mut KhExecutionVariant,
    ) -> KhStatus;
    pub fn kh_variant_sliced_q(
        config: *const KhSdpaConfig,
        kind: u32,
        max_q_tokens: u32,
        kv_tokens_per_iteration: u32,
        max_q_heads: u32,
        out: *mut KhExecutionVariant,
    ) -> KhStatus;
    pub fn kh_variant_supports(
        variant: *const KhExecutionVariant,
        config: *const KhSdpaConfig,
        out: *mut i32,
    ) -> KhStatus;
    pub fn kh_registry_variants(
        config: *const KhSdpaConfig,
        out: *mut KhExecutionVariant,
        capacity: u32,
        count: *mut u32,
    ) -> KhStatus;
    pub fn kh_page_table_bytes(layout: *const KhPageTableLayout, out: *mut u64) -> KhStatus;
    pub fn kh_page_table_index(
        layout: *const KhPageTableLayout,
        req_slot: u32,
        layer_index: u32,
        block_index: u32,
        out: *mut u64,
    ) -> KhStatus;
    pub fn kh_page_table_write(
        device: *mut KhDevice,
        page_ids: KhBufferRef,
        layout: *const KhPageTableLayout,
        req_slot: u32,
        layer_index: u32,
        block_index: u32,
        ids: *const u32,
        count: u32,
    ) -> KhStatus;
    pub fn kh_page_table_read(
        device: *mut KhDevice,
        page_ids: KhBufferRef,
        layout: *const KhPageTableLayout,
        req_slot: u32,
        layer_index: u32,
        block_index: u32,
        ids: *mut u32,
        count: u32,
    ) -> KhStatus;
    pub fn kh_page_table_reset_req_slot(
        device: *mut KhDevice,
        page_ids: KhBufferRef,
        layout: *const KhPageTableLayout,
        req_slot: u32,
    ) -> KhStatus;
    pub fn kh_replay_buckets(max_capacity: u32, out: *mut u32, capacity: u32, count: *mut u32) -> KhStatus;
    pub fn kh_replay_capacity(max_capacity: u32, active: u32, out: *mut u32) -> KhStatus;
    pub fn kh_selector_create(
        config: *const KhSdpaConfig,
        variants: *const KhExecutionVariant,
        num_variants: u32,
        max_tokens: u32,
        max_map_task_templates: u32,
        partial_state_group_capacity: u64,
        out: *mut *mut KhSelector,
    ) -> KhStatus;
    pub fn kh_selector_create_for_lookup(
        config: *const KhSdpaConfig,
        max_tokens: u32,
        layout: *const KhPageTableLayout,
        out: *mut *mut KhSelector,
    ) -> KhStatus;
    pub fn kh_selector_create_for_partitions(
        config: *const KhSdpaConfig,
        variants: *const KhExecutionVariant,
        num_variants: u32,
        max_kv_splits: *const u32,
        max_tokens: u32,
        max_requests: u32,
        out: *mut *mut KhSelector,
    ) -> KhStatus;
    pub fn kh_selector_destroy(selector: *mut KhSelector) -> KhStatus;
    pub fn kh_selector_limits_get(selector: *const KhSelector, out: *mut KhSelectorLimits) -> KhStatus;
    pub fn kh_selector_variants(
        selector: *const KhSelector,
        out: *mut KhExecutionVariant,
        capacity: u32,
        count: *mut u32,
    ) -> KhStatus;
    pub fn kh_selector_set_policy(selector: *mut KhSelector, policy: u32, sm_count: u32) -> KhStatus;
    pub fn kh_selector_select(
        selector: *const KhSelector,
        requests: *const KhRequestShape,
        num_requests: u32,
        policy_max_tokens: u32,
        policy_max_map_task_templates: u32,
        num_total_tokens: u32,
        out: *mut *mut KhSelection,
    ) -> KhStatus;
    pub fn kh_selector_select_partitioned(
        selector: *const KhSelector,
        variant: *const KhExecutionVariant,
        kv_slice: u32,
        direct_output: i32,
        requests: *const KhRequestShape,
        num_requests: u32,
        policy_max_tokens: u32,
        policy_max_map_task_templates: u32,
        num_total_tokens: u32,
        out: *mut *mut KhSelection,
    ) -> KhStatus;
    pub fn kh_selection_destroy(selection: *mut KhSelection) -> KhStatus;
    pub fn kh_selection_variant(selection: *const KhSelection, out: *mut KhExecutionVariant) -> KhStatus;
    pub fn kh_selection_direct_output(selection: *const KhSelection, out: *mut i32) -> KhStatus;
    pub fn kh_selection_replay_shape(selection: *const KhSelection, out: *mut KhReplayShape) -> KhStatus;
    pub fn kh_selection_metrics_get(selection: *const KhSelection, out: *mut KhSelectionMetrics) -> KhStatus;
    pub fn kh_selection_q_token_ranges(
        selection: *const KhSelection,
        out: *mut KhQTokenRange,
        capacity: u32,
        count: *mut u32,
    ) -> KhStatus;
    pub fn kh_selection_map_task_templates(
        selection: *const KhSelection,
        out: *mut KhMapTaskTemplate,
        capacity: u32,
        count: *mut u32,
    ) -> KhStatus;
    pub fn kh_selection_cu_partial_outputs(
        selection: *const KhSelection,
        out: *mut u32,
        capacity: u32,
        count: *mut u32,
    ) -> KhStatus;
    pub fn kh_metadata_update(
        arrays: *const KhMetadataArrays,
        req_slots: *const u32,
        token_indices: *const u32,
        cu_tokens: *const u32,
        num_requests: u32,
        selection: *const KhSelection,
        out_shape: *mut KhReplayShape,
    ) -> KhStatus;
    pub fn kh_sliced_kv_sizes_get(
        config: *const KhSlicedKvConfig,
        shape: *const KhSlicedKvShape,
        out: *mut KhSlicedKvSizes,
    ) -> KhStatus;
    pub fn kh_sliced_kv_create(
        device: *mut KhDevice,
        config: *const KhSlicedKvConfig,
        execution: *const KhExecutionVariant,
        shape: *const KhSlicedKvShape,
        out: *mut *mut KhSlicedKv,
    ) -> KhStatus;
    pub fn kh_sliced_kv_destroy(compute: *mut KhSlicedKv) -> KhStatus;
    pub fn kh_sliced_kv_map(
        compute: *mut KhSlicedKv,
        stream: *mut KhStream,
        buffers: *const KhSlicedKvMapBuffers,
        page_table_index: u32,
        num_active_tokens: u32,
        num_active_kv_splits: u32,
    ) -> KhStatus;
    pub fn kh_sliced_kv_reduce(
        compute: *mut KhSlicedKv,
        stream: *mut KhStream,
        buffers: *const KhSlicedKvReduceBuffers,
        num_active_tokens: u32,
    ) -> KhStatus;
    pub fn kh_sliced_kv_map_reduce(
        compute: *mut KhSlicedKv,
        stream: *mut KhStream,
        map_buffers: *const KhSlicedKvMapBuffers,
        reduce_buffers: *const KhSlicedKvReduceBuffers,
        arrival_counters: KhBufferRef,
        page_table_index: u32,
        num_active_tokens: u32,
        num_active_kv_splits: u32,
    ) -> KhStatus;
    pub fn kh_sliced_kv_arrival_counter_bytes(
        config: *const KhSlicedKvConfig,
        execution: *const KhExecutionVariant,
        shape: *const KhSlicedKvShape,
        out: *mut u64,
    ) -> KhStatus;
    pub fn kh_sliced_kv_attend_static(
        compute: *mut KhSlicedKv,
        stream: *mut KhStream,
        buffers: *const KhSlicedKvStaticBuffers,
        page_table_index: u32,
        num_active_tokens: u32,
        num_active_kv_splits: u32,
    ) -> KhStatus;
    pub fn kh_sliced_kv_static_bytes_needed(
        config: *const KhSlicedKvConfig,
        num_active_kv_splits: u32,
        out: *mut u64,
    ) -> KhStatus;
    pub fn kh_sliced_q_sizes_get(
        config: *const KhSlicedQConfig,
        execution: *const KhExecutionVariant,
        shape: *const KhSlicedQShape,
        out: *mut KhSlicedQSizes,
    ) -> KhStatus;
    pub fn kh_sliced_q_create(
        device: *mut KhDevice,
        config: *const KhSlicedQConfig,
        execution: *const KhExecutionVariant,
        shape: *const KhSlicedQShape,
        direct_output: i32,
        out: *mut *mut KhSlicedQ,
    ) -> KhStatus;
    pub fn kh_sliced_q_destroy(compute: *mut KhSlicedQ) -> KhStatus;
    pub fn kh_sliced_q_map(
        compute: *mut KhSlicedQ,
        stream: *mut KhStream,
        buffers: *const KhSlicedQMapBuffers,
        page_table_index: u32,
        num_active_tokens: u32,
        num_active_q_token_tiles: u32,
        num_active_kv_splits: u32,
    ) -> KhStatus;
    pub fn kh_sliced_q_direct(
        compute: *mut KhSlicedQ,
        stream: *mut KhStream,
        buffers: *const KhSlicedQDirectBuffers,
        page_table_index: u32,
        num_active_tokens: u32,
        num_active_q_token_tiles: u32,
    ) -> KhStatus;
    pub fn kh_sliced_q_reduce(
        compute: *mut KhSlicedQ,
        stream: *mut KhStream,
        buffers: *const KhSlicedQReduceBuffers,
        num_active_q_token_tiles: u32,
    ) -> KhStatus;
    pub fn kh_sliced_q_map_reduce(
        compute: *mut KhSlicedQ,
        stream: *mut KhStream,
        map_buffers: *const KhSlicedQMapBuffers,
        reduce_buffers: *const KhSlicedQReduceBuffers,
        arrival_counters: KhBufferRef,
        page_table_index: u32,
        num_active_tokens: u32,
        num_active_q_token_tiles: u32,
        num_active_kv_splits: u32,
    ) -> KhStatus;
    pub fn kh_sliced_q_arrival_counter_bytes(
        config: *const KhSlicedQConfig,
        execution: *const KhExecutionVariant,
        shape: *const KhSlicedQShape,
        out: *mut u64,
    ) -> KhStatus;
    pub fn kh_kv_page_write_create(
        device: *mut KhDevice,
        config: *const KhKvPageWriteConfig,
        out: *mut *mut KhKvPageWrite,
    ) -> KhStatus;
    pub fn kh_kv_page_write_destroy(compute: *mut KhKvPageWrite) -> KhStatus;
    pub fn kh_kv_page_write_tokens_per_page(config: *const KhKvPageWriteConfig, out: *mut u32) -> KhStatus;
    pub fn kh_kv_page_write_invoke(
        compute: *mut KhKvPageWrite,
        stream: *mut KhStream,
        shape: *const KhKvPageWriteShape,
        buffers: *const KhKvPageWriteBuffers,
        num_active_token_writes: u32,
        page_table_index: u32,
    ) -> KhStatus;
    pub fn kh_fp8_e4m3_from_bf16(bf16_bits: u16) -> u8;
    pub fn kh_fp8_e4m3_to_bf16(fp8_bits: u8) -> u16;
    pub fn kh_bidi_block_sdpa_create(
        device: *mut KhDevice,
        config: *const KhBidiBlockSdpaConfig,
        out: *mut *mut KhBidiBlockSdpa,
    ) -> KhStatus;
    pub fn kh_bidi_block_sdpa_destroy(compute: *mut KhBidiBlockSdpa) -> KhStatus;
    pub fn kh_bidi_block_sdpa_invoke(
        compute: *mut KhBidiBlockSdpa,
        stream: *mut KhStream,
        shape: *const KhBidiBlockSdpaShape,
        num_active_q_token_ranges: u32,
        buffers: *const KhBidiBlockSdpaBuffers,
    ) -> KhStatus;
    pub fn kh_bidi_block_metadata_build(
        arrays: *const KhMetadataArrays,
        req_slots: *const u32,
        token_positions: *const u32,
        history_begins: *const u32,
        history_ends: *const u32,
        num_requests: u32,
        block_size: u32,
        max_q_tokens: u32,
        kv_tokens_per_iteration: u32,
        max_sdpa_map_task_templates: u32,
        out_shape: *mut KhReplayShape,
    ) -> KhStatus;
    pub fn kh_device_check(device: *mut KhDevice, stream: *mut KhStream, out_status_word: *mut u32) -> KhStatus;
    pub fn kh_device_set_wait_limit(device: *mut KhDevice, polls: u32) -> KhStatus;
    pub fn kh_combine_partials(
        device: *mut KhDevice,
        stream: *mut KhStream,
        num_partials: u32,
        num_rows: u32,
        head_dim: u32,
        exp_sums: KhBufferRef,
        max_logits: KhBufferRef,
        partial_output: KhBufferRef,
        out_dtype: u32,
        output: KhBufferRef,
        out_exp_sums: KhBufferRef,
        out_max_logits: KhBufferRef,
    ) -> KhStatus;
    pub fn kh_combine_packed_partials(
        device: *mut KhDevice,
        stream: *mut KhStream,
        num_partials: u32,
        num_rows: u32,
        head_dim: u32,
        packed: KhBufferRef,
        out_dtype: u32,
        output: KhBufferRef,
    ) -> KhStatus;
    // ---- cross-GPU combine in one kernel over NVLink peer memory (no counterpart in the reference)
    pub fn kh_peer_exchange_inbox_bytes(world: u32, num_rows: u32, head_dim: u32, out: *mut u64) -> KhStatus;
    pub fn kh_ipc_export(device: *mut KhDevice, buffer: KhBufferRef, handle64: *mut u8) -> KhStatus;
    pub fn kh_ipc_import(device: *mut KhDevice, handle64: *const u8, out: *mut *mut core::ffi::c_void) -> KhStatus;
    pub fn kh_ipc_close(device: *mut KhDevice, ptr: *mut core::ffi::c_void) -> KhStatus;
    pub fn kh_peer_exchange_create(
        device: *mut KhDevice,
        rank: u32,
        world: u32,
        num_rows: u32,
        head_dim: u32,
        inboxes: *const *mut core::ffi::c_void,
        out: *mut *mut KhPeerExchange,
    ) -> KhStatus;
    pub fn kh_peer_exchange_destroy(exchange: *mut KhPeerExchange) -> KhStatus;
    pub fn kh_peer_exchange_combine(
        exchange: *mut KhPeerExchange,
        stream: *mut KhStream,
        num_partials: u32,
        exp_sums: KhBufferRef,
        max_logits: KhBufferRef,
        partial_output: KhBufferRef,
        out_dtype: u32,
        output: KhBufferRef,
    ) -> KhStatus;
}
