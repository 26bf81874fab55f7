"""SDPA selector: ``RequestShape``, ``Selector``, ``Selection``
(crates/inference-executor-metal/src/attn/gqa/sdpa.rs). The planning itself runs in the C++ library;
this module mirrors the reference's names over the C ABI."""
from __future__ import annotations

import ctypes as C
import enum
from dataclasses import dataclass

from . import abi
from .replay import GQAReplayBucketPolicy, GQAReplayShape
from .request_page_table import GQAPageTableLayout
from .sdpa import Config, ExecutionVariant, MapKernelKind, Registry


class SelectorPolicy(enum.IntEnum):
    Reference = 0  # the reference's rules, bit for bit
    B200 = 1       # KV slice and Q tile re-derived for a persistent kernel on `sm_count` SMs


@dataclass(frozen=True)
class RequestShape:
    num_history_tokens: int
    num_q_tokens: int

    @staticmethod
    def from_batch(token_indices, cu_tokens) -> list["RequestShape"]:
        """``RequestShape::from_batch`` (sdpa.rs:22-41)."""
        if len(cu_tokens) != len(token_indices) + 1 or cu_tokens[0] != 0:
            raise abi.InvalidArgument(1, "GQA batch cu_tokens must start at 0 and have one entry per request plus one")
        shapes = []
        for history, begin, end in zip(token_indices, cu_tokens[:-1], cu_tokens[1:]):
            if begin > end:
                raise abi.InvalidArgument(1, "GQA batch cu_tokens must be nondecreasing")
            if end - begin == 0:
                raise abi.InvalidArgument(1, "GQA requests must contain Q tokens")
            if history + (end - begin) > 0xFFFFFFFF:
                raise abi.InvalidArgument(1, "GQA request context length must fit u32")
            shapes.append(RequestShape(int(history), int(end - begin)))
        return shapes


@dataclass(frozen=True)
class SelectorLimits:
    max_tokens: int
    max_map_task_templates: int
    partial_state_group_capacity: int


@dataclass(frozen=True)
class QTokenRange:
    request_index: int
    flat_q_token_indices: range
    num_visible_kv_tokens: int


@dataclass(frozen=True)
class MapTaskTemplate:
    q_token_range_index: int
    request_local_kv_token_indices: range


@dataclass(frozen=True)
class SelectionMetrics:
    num_scheduled_qk_token_pairs: int
    num_active_qk_token_pairs: int
    num_map_threadblocks_per_kv_head: int
    num_map_simdgroup_waves_per_kv_head: int
    num_active_partial_state_groups: int
    num_active_partial_states: int
    num_reserved_partial_state_groups: int
    num_replay_reserved_partial_state_groups: int
    max_kv_iterations_per_split: int
    num_logical_qk_token_pairs: int


class Selection:
    """``Selection`` (sdpa.rs:89-125). Owns the C handle; accessors copy out."""

    def __init__(self, handle: C.c_void_p):
        self.handle = handle

    def __del__(self):
        try:
            if self.handle:
                abi.lib().kh_selection_destroy(self.handle)
                self.handle = None
        except Exception:
            pass

    def variant(self) -> ExecutionVariant:
        out = abi.ExecutionVariantC()
        abi.call("kh_selection_variant", self.handle, C.byref(out))
        return ExecutionVariant.from_c(out)

    def direct_output(self) -> bool:
        out = C.c_int32()
        abi.call("kh_selection_direct_output", self.handle, C.byref(out))
        return bool(out.value)

    def replay_shape(self) -> GQAReplayShape:
        out = abi.ReplayShapeC()
        abi.call("kh_selection_replay_shape", self.handle, C.byref(out))
        return GQAReplayShape.from_c(out)

    def metrics(self) -> SelectionMetrics:
        m = abi.SelectionMetricsC()
        abi.call("kh_selection_metrics_get", self.handle, C.byref(m))
        return SelectionMetrics(
            m.num_scheduled_qk_token_pairs, m.num_active_qk_token_pairs, m.num_map_threadblocks_per_kv_head,
            m.num_map_simdgroup_waves_per_kv_head, m.num_active_partial_state_groups, m.num_active_partial_states,
            m.num_reserved_partial_state_groups, m.num_replay_reserved_partial_state_groups,
            m.max_kv_iterations_per_split, m.num_logical_qk_token_pairs)

    def _array(self, name, ctype):
        count = C.c_uint32()
        abi.call(name, self.handle, None, 0, C.byref(count))
        arr = (ctype * max(count.value, 1))()
        abi.call(name, self.handle, arr, count.value, C.byref(count))
        return [arr[i] for i in range(count.value)]

    def q_token_ranges(self) -> list[QTokenRange]:
        return [QTokenRange(r.request_index, range(r.flat_q_token_begin, r.flat_q_token_end), r.num_visible_kv_tokens)
                for r in self._array("kh_selection_q_token_ranges", abi.QTokenRangeC)]

    def map_task_templates(self) -> list[MapTaskTemplate]:
        return [MapTaskTemplate(t.q_token_range_index, range(t.kv_token_begin, t.kv_token_end))
                for t in self._array("kh_selection_map_task_templates", abi.MapTaskTemplateC)]

    def cu_partial_outputs_by_q_token_range(self) -> list[int]:
        return list(self._array("kh_selection_cu_partial_outputs", C.c_uint32))


def _shapes(request_shapes):
    arr = (abi.RequestShapeC * max(len(request_shapes), 1))()
    for i, shape in enumerate(request_shapes):
        arr[i] = abi.RequestShapeC(shape.num_history_tokens, shape.num_q_tokens)
    return arr


class Selector:
    """``Selector`` (sdpa.rs:129-466)."""

    def __init__(self, handle: C.c_void_p, registry_config: Config):
        self.handle = handle
        self._config = registry_config

    def __del__(self):
        try:
            if self.handle:
                abi.lib().kh_selector_destroy(self.handle)
                self.handle = None
        except Exception:
            pass

    @staticmethod
    def new(registry: Registry, max_tokens: int, max_map_task_templates: int,
            partial_state_group_capacity: int) -> "Selector":
        variants = registry.variants()
        arr = (abi.ExecutionVariantC * len(variants))(*[v.to_c() for v in variants])
        handle = C.c_void_p()
        abi.call("kh_selector_create", C.byref(registry.config().to_c()), arr, len(variants), max_tokens,
                 max_map_task_templates, partial_state_group_capacity, C.byref(handle))
        return Selector(handle, registry.config())

    @staticmethod
    def for_lookup(config: Config, max_tokens: int, layout: GQAPageTableLayout) -> "Selector":
        handle = C.c_void_p()
        abi.call("kh_selector_create_for_lookup", C.byref(config.to_c()), max_tokens, C.byref(layout.to_c()),
                 C.byref(handle))
        return Selector(handle, config)

    @staticmethod
    def for_partitions(registry: Registry, max_tokens: int, max_requests: int, max_kv_splits) -> "Selector":
        variants = registry.variants()
        arr = (abi.ExecutionVariantC * len(variants))(*[v.to_c() for v in variants])
        splits = (C.c_uint32 * len(variants))(*[int(max_kv_splits(v)) for v in variants])
        handle = C.c_void_p()
        abi.call("kh_selector_create_for_partitions", C.byref(registry.config().to_c()), arr, len(variants), splits,
                 max_tokens, max_requests, C.byref(handle))
        return Selector(handle, registry.config())

    def set_policy(self, policy: SelectorPolicy, sm_count: int = 148) -> "Selector":
        abi.call("kh_selector_set_policy", self.handle, int(policy), sm_count)
        return self

    def config(self) -> Config:
        return self._config

    def limits(self) -> SelectorLimits:
        out = abi.SelectorLimitsC()
        abi.call("kh_selector_limits_get", self.handle, C.byref(out))
        return SelectorLimits(out.max_tokens, out.max_map_task_templates, out.partial_state_group_capacity)

    def variants(self) -> list[ExecutionVariant]:
        count = C.c_uint32()
        abi.call("kh_selector_variants", self.handle, None, 0, C.byref(count))
        arr = (abi.ExecutionVariantC * count.value)()
        abi.call("kh_selector_variants", self.handle, arr, count.value, C.byref(count))
        return [ExecutionVariant.from_c(arr[i]) for i in range(count.value)]

    def select(self, request_shapes, policy: GQAReplayBucketPolicy, num_total_tokens: int) -> Selection:
        handle = C.c_void_p()
        abi.call("kh_selector_select", self.handle, _shapes(request_shapes), len(request_shapes), policy.max_tokens(),
                 policy.max_map_task_templates(), num_total_tokens, C.byref(handle))
        return Selection(handle)

    def select_partitioned(self, variant: ExecutionVariant, kv_slice: int, direct_output: bool, request_shapes,
                           policy: GQAReplayBucketPolicy, num_total_tokens: int) -> Selection:
        handle = C.c_void_p()
        abi.call("kh_selector_select_partitioned", self.handle, C.byref(variant.to_c()), kv_slice,
                 int(direct_output), _shapes(request_shapes), len(request_shapes), policy.max_tokens(),
                 policy.max_map_task_templates(), num_total_tokens, C.byref(handle))
        return Selection(handle)


__all__ = ["MapKernelKind", "MapTaskTemplate", "QTokenRange", "RequestShape", "Selection", "SelectionMetrics",
           "Selector", "SelectorLimits", "SelectorPolicy"]
