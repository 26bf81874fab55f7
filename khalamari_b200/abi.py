"""ctypes view of ``include/kh_gqa.h``: struct layouts, prototypes and error mapping.

The shared library is the product. If it is missing or cannot be loaded, importing this module's
``lib()`` raises: there is no CPU fallback.
"""
from __future__ import annotations

import ctypes as C
import os
from pathlib import Path

from . import build as _build

KH_OK = 0
STATUS_NAMES = {
    0: "OK", 1: "InvalidArgument", 2: "ResourceExhausted", 3: "Cancelled", 4: "DeadlineExceeded", 5: "Aborted",
    6: "Evicted", 7: "Unavailable", 8: "Internal",
}


class KhError(RuntimeError):
    """A non-OK status from the C ABI. ``code`` names the reference's ``inference_error::Error`` variant."""

    def __init__(self, code: int, message: str):
        super().__init__(f"{STATUS_NAMES.get(code, code)}: {message}")
        self.code = code
        self.message = message


class InvalidArgument(KhError, AssertionError):
    """Raised where the reference would ``assert!``/``panic!`` on an invariant."""


class BufferRef(C.Structure):
    _fields_ = [("ptr", C.c_void_p), ("bytes", C.c_uint64)]


class SdpaConfig(C.Structure):
    _fields_ = [("io_dtype", C.c_uint32), ("num_q_heads", C.c_uint32), ("num_kv_heads", C.c_uint32),
                ("head_dim", C.c_uint32), ("tokens_per_page", C.c_uint32)]


class ExecutionVariantC(C.Structure):
    _fields_ = [("kind", C.c_uint32), ("max_q_tokens", C.c_uint32), ("max_q_heads", C.c_uint32),
                ("kv_tokens_per_iteration", C.c_uint32), ("required_threads", C.c_uint32),
                ("tokens_per_page", C.c_uint32), ("reduce_max_q_tokens", C.c_uint32),
                ("reduce_max_q_heads", C.c_uint32), ("reduce_required_threads", C.c_uint32)]


class PageTableLayoutC(C.Structure):
    _fields_ = [("num_req_slots", C.c_uint32), ("num_gqa_layers", C.c_uint32), ("num_blocks", C.c_uint32),
                ("num_page_ids_per_block", C.c_uint32)]


class ReplayShapeC(C.Structure):
    _fields_ = [("num_tokens", C.c_uint32), ("num_total_tokens", C.c_uint32), ("num_q_token_tiles", C.c_uint32),
                ("num_total_q_token_tiles", C.c_uint32), ("num_sdpa_map_task_templates", C.c_uint32),
                ("num_total_sdpa_map_task_templates", C.c_uint32), ("reduce_sdpa_partial_outputs", C.c_uint32)]


class RequestShapeC(C.Structure):
    _fields_ = [("num_history_tokens", C.c_uint32), ("num_q_tokens", C.c_uint32)]


class SelectorLimitsC(C.Structure):
    _fields_ = [("max_tokens", C.c_uint32), ("max_map_task_templates", C.c_uint32),
                ("partial_state_group_capacity", C.c_uint64)]


class SelectionMetricsC(C.Structure):
    _fields_ = [("num_scheduled_qk_token_pairs", C.c_uint64), ("num_active_qk_token_pairs", C.c_uint64),
                ("num_map_threadblocks_per_kv_head", C.c_uint64), ("num_map_simdgroup_waves_per_kv_head", C.c_uint64),
                ("num_active_partial_state_groups", C.c_uint64), ("num_active_partial_states", C.c_uint64),
                ("num_reserved_partial_state_groups", C.c_uint64),
                ("num_replay_reserved_partial_state_groups", C.c_uint64), ("num_logical_qk_token_pairs", C.c_uint64),
                ("max_kv_iterations_per_split", C.c_uint32), ("reserved", C.c_uint32)]


class QTokenRangeC(C.Structure):
    _fields_ = [("request_index", C.c_uint32), ("flat_q_token_begin", C.c_uint32), ("flat_q_token_end", C.c_uint32),
                ("num_visible_kv_tokens", C.c_uint32)]


class MapTaskTemplateC(C.Structure):
    _fields_ = [("q_token_range_index", C.c_uint32), ("kv_token_begin", C.c_uint32), ("kv_token_end", C.c_uint32)]


class MetadataArraysC(C.Structure):
    _fields_ = [("req_slots", C.POINTER(C.c_uint32)), ("flat_token_indices", C.POINTER(C.c_uint32)),
                ("visible_kv_token_ranges", C.POINTER(C.c_uint32)), ("q_token_ranges", C.POINTER(C.c_uint32)),
                ("sdpa_map_task_templates", C.POINTER(C.c_uint32)), ("cu_sdpa_partial_outputs", C.POINTER(C.c_uint32)),
                ("max_tokens", C.c_uint32), ("max_map_task_templates", C.c_uint32)]


class SlicedKvConfigC(C.Structure):
    _fields_ = [("num_q_heads", C.c_uint32), ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
                ("scale", C.c_float), ("page_bytes", C.c_uint32), ("page_table_layout", PageTableLayoutC),
                ("dtype", C.c_uint32), ("kv_dtype", C.c_uint32)]


class SlicedKvShapeC(C.Structure):
    _fields_ = [("num_total_tokens", C.c_uint32), ("num_total_sdpa_map_task_templates", C.c_uint32)]


class SlicedKvMapBuffersC(C.Structure):
    _fields_ = [(name, BufferRef) for name in (
        "q", "kv_pages", "req_slots", "page_ids", "sdpa_map_task_templates", "partial_exp_sums",
        "partial_max_logits", "partial_output")]


class SlicedKvReduceBuffersC(C.Structure):
    _fields_ = [(name, BufferRef) for name in (
        "partial_exp_sums", "partial_max_logits", "partial_output", "cu_sdpa_partial_outputs", "output")]


class KvPageWriteConfigC(C.Structure):
    _fields_ = [("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("page_bytes", C.c_uint32),
                ("dtype", C.c_uint32), ("kv_dtype", C.c_uint32)]


class KvPageWriteShapeC(C.Structure):
    _fields_ = [("num_total_token_writes", C.c_uint32), ("page_table_layout", PageTableLayoutC)]


class KvPageWriteBuffersC(C.Structure):
    _fields_ = [(name, BufferRef) for name in (
        "pages", "flat_k", "flat_v", "req_slots", "flat_token_indices", "page_ids")]


class SlicedKvStaticBuffersC(C.Structure):
    _fields_ = [(name, BufferRef) for name in (
        "q", "kv_pages", "req_slots", "page_ids", "sdpa_map_task_templates", "cu_sdpa_partial_outputs", "output")]


STATIC_PARTIALS_BYTES = 32 << 20  # KH_STATIC_PARTIALS_BYTES


class BidiBlockSdpaConfigC(C.Structure):
    _fields_ = [("block_size", C.c_uint32), ("max_q_tokens", C.c_uint32), ("num_q_heads", C.c_uint32),
                ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32), ("scale", C.c_float), ("dtype", C.c_uint32)]


class BidiBlockSdpaShapeC(C.Structure):
    _fields_ = [("num_total_tokens", C.c_uint32), ("num_total_q_token_ranges", C.c_uint32),
                ("num_total_partial_output_slots", C.c_uint32)]


class BidiBlockSdpaBuffersC(C.Structure):
    _fields_ = [(name, BufferRef) for name in ("q", "local_k", "local_v", "q_token_ranges", "cu_sdpa_partial_outputs",
                                               "partial_exp_sums", "partial_max_logits", "partial_output")]


class SlicedKvSizesC(C.Structure):
    _fields_ = [("q_bytes", C.c_uint64), ("req_slots_bytes", C.c_uint64), ("page_ids_bytes", C.c_uint64),
                ("sdpa_map_task_templates_bytes", C.c_uint64), ("cu_sdpa_partial_outputs_bytes", C.c_uint64),
                ("partial_output_stats_bytes", C.c_uint64), ("partial_output_bytes", C.c_uint64),
                ("num_tokens_per_page", C.c_uint32), ("reserved", C.c_uint32)]


class SlicedQConfigC(C.Structure):
    _fields_ = [("num_q_heads", C.c_uint32), ("num_kv_heads", C.c_uint32), ("head_dim", C.c_uint32),
                ("scale", C.c_float), ("page_bytes", C.c_uint32), ("dtype", C.c_uint32),
                ("page_table_layout", PageTableLayoutC), ("kv_dtype", C.c_uint32)]


class SlicedQShapeC(C.Structure):
    _fields_ = [("num_total_tokens", C.c_uint32), ("num_total_q_token_tiles", C.c_uint32),
                ("num_total_sdpa_map_task_templates", C.c_uint32)]


class SlicedQMapBuffersC(C.Structure):
    _fields_ = [(name, BufferRef) for name in (
        "q", "kv_pages", "req_slots", "page_ids", "visible_kv_token_ranges", "q_token_ranges",
        "sdpa_map_task_templates", "partial_output", "partial_exp_sums", "partial_max_logits")]


class SlicedQDirectBuffersC(C.Structure):
    _fields_ = [(name, BufferRef) for name in (
        "q", "kv_pages", "req_slots", "page_ids", "visible_kv_token_ranges", "q_token_ranges",
        "sdpa_map_task_templates", "output")]


class SlicedQReduceBuffersC(C.Structure):
    _fields_ = [(name, BufferRef) for name in (
        "partial_output", "partial_exp_sums", "partial_max_logits", "q_token_ranges", "cu_sdpa_partial_outputs",
        "output")]


class SlicedQSizesC(C.Structure):
    _fields_ = [("q_bytes", C.c_uint64), ("partial_output_bytes", C.c_uint64),
                ("partial_output_stats_bytes", C.c_uint64), ("num_tokens_per_page", C.c_uint32),
                ("reserved", C.c_uint32)]


P = C.POINTER
_u32 = C.c_uint32
_vp = C.c_void_p

# name -> argument types (every function returns kh_status unless listed in _SPECIAL)
PROTOTYPES = {
    "kh_device_open": [C.c_int32, P(_vp)],
    "kh_device_close": [_vp],
    "kh_device_sm_count": [_vp, P(C.c_int32)],
    "kh_buffer_alloc": [_vp, C.c_uint64, P(BufferRef)],
    "kh_buffer_free": [_vp, BufferRef],
    "kh_buffer_write": [_vp, BufferRef, C.c_uint64, _vp, C.c_uint64],
    "kh_buffer_read": [_vp, BufferRef, C.c_uint64, _vp, C.c_uint64],
    "kh_buffer_zero": [_vp, BufferRef, C.c_uint64, C.c_uint64],
    "kh_stream_create": [_vp, P(_vp)],
    "kh_stream_wrap": [_vp, _vp, P(_vp)],
    "kh_stream_bind_active_counts": [_vp, BufferRef],
    "kh_stream_destroy": [_vp],
    "kh_stream_synchronize": [_vp],
    "kh_stream_write": [_vp, BufferRef, C.c_uint64, _vp, C.c_uint64],
    "kh_stream_read": [_vp, BufferRef, C.c_uint64, _vp, C.c_uint64],
    "kh_event_create": [_vp, P(_vp)],
    "kh_event_destroy": [_vp],
    "kh_stream_record_event": [_vp, _vp],
    "kh_stream_wait_event": [_vp, _vp],
    "kh_event_synchronize": [_vp],
    "kh_device_set_wait_limit": [_vp, _u32],
    "kh_host_alloc_pinned": [C.c_uint64, P(_vp)],
    "kh_host_free_pinned": [_vp],
    "kh_sdpa_config_validate": [P(SdpaConfig)],
    "kh_variant_sliced_kv": [P(SdpaConfig), _u32, _u32, _u32, P(ExecutionVariantC)],
    "kh_variant_sliced_q": [P(SdpaConfig), _u32, _u32, _u32, _u32, P(ExecutionVariantC)],
    "kh_variant_supports": [P(ExecutionVariantC), P(SdpaConfig), P(C.c_int32)],
    "kh_registry_variants": [P(SdpaConfig), P(ExecutionVariantC), _u32, P(_u32)],
    "kh_page_table_bytes": [P(PageTableLayoutC), P(C.c_uint64)],
    "kh_page_table_index": [P(PageTableLayoutC), _u32, _u32, _u32, P(C.c_uint64)],
    "kh_page_table_write": [_vp, BufferRef, P(PageTableLayoutC), _u32, _u32, _u32, P(_u32), _u32],
    "kh_page_table_read": [_vp, BufferRef, P(PageTableLayoutC), _u32, _u32, _u32, P(_u32), _u32],
    "kh_page_table_reset_req_slot": [_vp, BufferRef, P(PageTableLayoutC), _u32],
    "kh_replay_buckets": [_u32, P(_u32), _u32, P(_u32)],
    "kh_replay_capacity": [_u32, _u32, P(_u32)],
    "kh_selector_create": [P(SdpaConfig), P(ExecutionVariantC), _u32, _u32, _u32, C.c_uint64, P(_vp)],
    "kh_selector_create_for_lookup": [P(SdpaConfig), _u32, P(PageTableLayoutC), P(_vp)],
    "kh_selector_create_for_partitions": [P(SdpaConfig), P(ExecutionVariantC), _u32, P(_u32), _u32, _u32, P(_vp)],
    "kh_selector_destroy": [_vp],
    "kh_selector_limits_get": [_vp, P(SelectorLimitsC)],
    "kh_selector_variants": [_vp, P(ExecutionVariantC), _u32, P(_u32)],
    "kh_selector_set_policy": [_vp, _u32, _u32],
    "kh_selector_select": [_vp, P(RequestShapeC), _u32, _u32, _u32, _u32, P(_vp)],
    "kh_selector_select_partitioned": [_vp, P(ExecutionVariantC), _u32, C.c_int32, P(RequestShapeC), _u32, _u32,
                                       _u32, _u32, P(_vp)],
    "kh_selection_destroy": [_vp],
    "kh_selection_variant": [_vp, P(ExecutionVariantC)],
    "kh_selection_direct_output": [_vp, P(C.c_int32)],
    "kh_selection_replay_shape": [_vp, P(ReplayShapeC)],
    "kh_selection_metrics_get": [_vp, P(SelectionMetricsC)],
    "kh_selection_q_token_ranges": [_vp, P(QTokenRangeC), _u32, P(_u32)],
    "kh_selection_map_task_templates": [_vp, P(MapTaskTemplateC), _u32, P(_u32)],
    "kh_selection_cu_partial_outputs": [_vp, P(_u32), _u32, P(_u32)],
    "kh_metadata_update": [P(MetadataArraysC), P(_u32), P(_u32), P(_u32), _u32, _vp, P(ReplayShapeC)],
    "kh_sliced_kv_sizes_get": [P(SlicedKvConfigC), P(SlicedKvShapeC), P(SlicedKvSizesC)],
    "kh_sliced_kv_create": [_vp, P(SlicedKvConfigC), P(ExecutionVariantC), P(SlicedKvShapeC), P(_vp)],
    "kh_sliced_kv_destroy": [_vp],
    "kh_sliced_kv_map": [_vp, _vp, P(SlicedKvMapBuffersC), _u32, _u32, _u32],
    "kh_sliced_kv_reduce": [_vp, _vp, P(SlicedKvReduceBuffersC), _u32],
    "kh_sliced_kv_map_reduce": [_vp, _vp, P(SlicedKvMapBuffersC), P(SlicedKvReduceBuffersC), BufferRef, _u32, _u32, _u32],
    "kh_sliced_kv_arrival_counter_bytes": [P(SlicedKvConfigC), P(ExecutionVariantC), P(SlicedKvShapeC), P(C.c_uint64)],
    "kh_sliced_kv_attend_static": [_vp, _vp, P(SlicedKvStaticBuffersC), _u32, _u32, _u32],
    "kh_sliced_kv_static_bytes_needed": [P(SlicedKvConfigC), _u32, P(C.c_uint64)],
    "kh_sliced_q_sizes_get": [P(SlicedQConfigC), P(ExecutionVariantC), P(SlicedQShapeC), P(SlicedQSizesC)],
    "kh_sliced_q_create": [_vp, P(SlicedQConfigC), P(ExecutionVariantC), P(SlicedQShapeC), C.c_int32, P(_vp)],
    "kh_sliced_q_destroy": [_vp],
    "kh_sliced_q_map": [_vp, _vp, P(SlicedQMapBuffersC), _u32, _u32, _u32, _u32],
    "kh_sliced_q_direct": [_vp, _vp, P(SlicedQDirectBuffersC), _u32, _u32, _u32],
    "kh_sliced_q_reduce": [_vp, _vp, P(SlicedQReduceBuffersC), _u32],
    "kh_sliced_q_map_reduce": [_vp, _vp, P(SlicedQMapBuffersC), P(SlicedQReduceBuffersC), BufferRef, _u32, _u32, _u32,
                               _u32],
    "kh_sliced_q_arrival_counter_bytes": [P(SlicedQConfigC), P(ExecutionVariantC), P(SlicedQShapeC), P(C.c_uint64)],
    "kh_device_check": [_vp, _vp, P(_u32)],
    "kh_combine_partials": [_vp, _vp, _u32, _u32, _u32, BufferRef, BufferRef, BufferRef, _u32, BufferRef, BufferRef,
                            BufferRef],
    "kh_kv_page_write_create": [_vp, P(KvPageWriteConfigC), P(_vp)],
    "kh_kv_page_write_destroy": [_vp],
    "kh_kv_page_write_tokens_per_page": [P(KvPageWriteConfigC), P(C.c_uint32)],
    "kh_kv_page_write_invoke": [_vp, _vp, P(KvPageWriteShapeC), P(KvPageWriteBuffersC), _u32, _u32],
    "kh_combine_packed_partials": [_vp, _vp, _u32, _u32, _u32, BufferRef, _u32, BufferRef],
    "kh_peer_exchange_inbox_bytes": [_u32, _u32, _u32, P(C.c_uint64)],
    "kh_ipc_export": [_vp, BufferRef, P(C.c_uint8)],
    "kh_ipc_import": [_vp, P(C.c_uint8), P(_vp)],
    "kh_ipc_close": [_vp, _vp],
    "kh_peer_exchange_create": [_vp, _u32, _u32, _u32, _u32, P(_vp), P(_vp)],
    "kh_peer_exchange_destroy": [_vp],
    "kh_peer_exchange_combine": [_vp, _vp, _u32, BufferRef, BufferRef, BufferRef, _u32, BufferRef],
    "kh_bidi_block_sdpa_create": [_vp, P(BidiBlockSdpaConfigC), P(_vp)],
    "kh_bidi_block_sdpa_destroy": [_vp],
    "kh_bidi_block_sdpa_invoke": [_vp, _vp, P(BidiBlockSdpaShapeC), _u32, P(BidiBlockSdpaBuffersC)],
    "kh_bidi_block_metadata_build": [P(MetadataArraysC), P(_u32), P(_u32), P(_u32), P(_u32), _u32, _u32, _u32, _u32,
                                     _u32, P(ReplayShapeC)],
}
_SPECIAL = {
    "kh_last_error": ([C.c_char_p, C.c_size_t], C.c_size_t),
    "kh_version": ([], C.c_char_p),
    "kh_fp8_e4m3_from_bf16": ([C.c_uint16], C.c_uint8),
    "kh_fp8_e4m3_to_bf16": ([C.c_uint8], C.c_uint16),
}

_lib = None


def library_path() -> Path:
    """The product library, or the measurement build (compiled with ``KH_GQA_MEASURE``: kernel parts can be
    switched off through ``KH_GQA_DEBUG`` to time the others) when ``KH_GQA_LIBRARY=measure`` asks for it. The
    product library itself reads no environment variable."""
    return _build.MEASURE_LIBRARY if os.environ.get("KH_GQA_LIBRARY") == "measure" else _build.LIBRARY


def lib() -> C.CDLL:
    """Loads ``libkhcuda_gqa.so`` (building it first when the sources are newer). Fails loudly."""
    global _lib
    if _lib is None:
        path = _build.build(measure=library_path() == _build.MEASURE_LIBRARY)
        handle = C.CDLL(str(path))
        for name, argtypes in PROTOTYPES.items():
            fn = getattr(handle, name)  # AttributeError if the header and the library drift apart
            fn.argtypes = argtypes
            fn.restype = C.c_int32
        for name, (argtypes, restype) in _SPECIAL.items():
            fn = getattr(handle, name)
            fn.argtypes = argtypes
            fn.restype = restype
        _lib = handle
    return _lib


def last_error() -> str:
    buf = C.create_string_buffer(2048)
    lib().kh_last_error(buf, len(buf))
    return buf.value.decode("utf-8", "replace")


def check(status: int) -> None:
    if status == KH_OK:
        return
    message = last_error()
    if status == 1:
        raise InvalidArgument(status, message)
    raise KhError(status, message)


def call(name: str, *args) -> None:
    check(getattr(lib(), name)(*args))
