"""SlicedKv SDPA compute (single Q token per task, KV range sliced into map tasks, then reduce):
``Config``, ``Shape``, ``MapBuffers``, ``ReduceBuffers``, ``Scratch``, ``Compute``
(crates/inference-backend-metal/src/components/gqa/sdpa/sliced_kv.rs)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

from . import abi
from .device import Buffer, Device, Dtype, Stream
from .request_page_table import GQAPageTableLayout
from . import sdpa


@dataclass(frozen=True)
class Config:
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    page_bytes: int
    page_table_layout: GQAPageTableLayout
    dtype: Dtype
    kv_dtype: Dtype | None = None  # defaults to `dtype`; the reference fixes one byte per element

    def kv_element_dtype(self) -> Dtype:
        return self.dtype if self.kv_dtype is None else self.kv_dtype

    def to_c(self) -> abi.SlicedKvConfigC:
        return abi.SlicedKvConfigC(self.num_q_heads, self.num_kv_heads, self.head_dim, self.scale, self.page_bytes,
                                   self.page_table_layout.to_c(), int(self.dtype), int(self.kv_element_dtype()))

    def sizes(self, shape: "Shape") -> abi.SlicedKvSizesC:
        out = abi.SlicedKvSizesC()
        abi.call("kh_sliced_kv_sizes_get", C.byref(self.to_c()), C.byref(shape.to_c()), C.byref(out))
        return out

    def validate(self) -> None:
        self.sizes(Shape(1, 1))

    def num_tokens_per_page(self) -> int:
        return self.sizes(Shape(1, 1)).num_tokens_per_page

    def q_heads_per_kv_head(self) -> int:
        return self.num_q_heads // self.num_kv_heads

    def sdpa_config(self) -> sdpa.Config:
        return sdpa.Config(self.dtype, self.num_q_heads, self.num_kv_heads, self.head_dim, self.num_tokens_per_page())

    def num_output_values(self, shape: "Shape") -> int:
        return shape.num_total_tokens * self.num_q_heads * self.head_dim

    def q_bytes(self, shape: "Shape") -> int:
        return self.sizes(shape).q_bytes

    def partial_output_stats_bytes(self, shape: "Shape") -> int:
        return self.sizes(shape).partial_output_stats_bytes

    def partial_output_bytes(self, shape: "Shape") -> int:
        return self.sizes(shape).partial_output_bytes


@dataclass(frozen=True)
class Shape:
    num_total_tokens: int
    num_total_sdpa_map_task_templates: int

    def to_c(self) -> abi.SlicedKvShapeC:
        return abi.SlicedKvShapeC(self.num_total_tokens, self.num_total_sdpa_map_task_templates)

    def validate(self, config: Config) -> None:
        config.sizes(self)


@dataclass
class MapBuffers:
    q: Buffer
    kv_pages: Buffer
    req_slots: Buffer
    page_ids: Buffer
    sdpa_map_task_templates: Buffer
    partial_exp_sums: Buffer
    partial_max_logits: Buffer
    partial_output: Buffer

    def to_c(self) -> abi.SlicedKvMapBuffersC:
        return abi.SlicedKvMapBuffersC(*[getattr(self, name).ref for name, _ in abi.SlicedKvMapBuffersC._fields_])


@dataclass
class ReduceBuffers:
    partial_exp_sums: Buffer
    partial_max_logits: Buffer
    partial_output: Buffer
    cu_sdpa_partial_outputs: Buffer
    output: Buffer

    def to_c(self) -> abi.SlicedKvReduceBuffersC:
        return abi.SlicedKvReduceBuffersC(
            *[getattr(self, name).ref for name, _ in abi.SlicedKvReduceBuffersC._fields_])


@dataclass
class StaticBuffers:
    """Buffers of ``Compute.invoke_attend_static``: those of map and reduce without the partial state."""

    q: Buffer
    kv_pages: Buffer
    req_slots: Buffer
    page_ids: Buffer
    sdpa_map_task_templates: Buffer
    cu_sdpa_partial_outputs: Buffer
    output: Buffer

    def to_c(self) -> abi.SlicedKvStaticBuffersC:
        return abi.SlicedKvStaticBuffersC(
            *[getattr(self, name).ref for name, _ in abi.SlicedKvStaticBuffersC._fields_])


class Scratch:
    """``Scratch`` (sliced_kv.rs:256-305): partial statistics and partial output (f32 here)."""

    def __init__(self, device: Device, config: Config, shape: Shape):
        sizes = config.sizes(shape)
        self.partial_exp_sums = Buffer.new_zeroed(device, sizes.partial_output_stats_bytes)
        self.partial_max_logits = Buffer.new_zeroed(device, sizes.partial_output_stats_bytes)
        self.partial_output = Buffer.new_zeroed(device, sizes.partial_output_bytes)

    def map_buffers(self, q, kv_pages, req_slots, page_ids, sdpa_map_task_templates) -> MapBuffers:
        return MapBuffers(q, kv_pages, req_slots, page_ids, sdpa_map_task_templates, self.partial_exp_sums,
                          self.partial_max_logits, self.partial_output)

    def reduce_buffers(self, cu_sdpa_partial_outputs, output) -> ReduceBuffers:
        return ReduceBuffers(self.partial_exp_sums, self.partial_max_logits, self.partial_output,
                             cu_sdpa_partial_outputs, output)


class Compute:
    """``Compute`` (sliced_kv.rs:315-388). ``invoke_map`` / ``invoke_reduce`` enqueue on ``stream``; they are
    the ``MapInvocation::record`` / ``ReduceInvocation::record`` of the reference."""

    def __init__(self, device: Device, config: Config, execution: sdpa.ExecutionVariant, shape: Shape):
        handle = C.c_void_p()
        abi.call("kh_sliced_kv_create", device.handle, C.byref(config.to_c()), C.byref(execution.to_c()),
                 C.byref(shape.to_c()), C.byref(handle))
        self.handle = handle
        self.config = config
        self.shape = shape
        self.execution = execution

    @staticmethod
    def new(device, config, execution, shape) -> "Compute":
        return Compute(device, config, execution, shape)

    def invoke_map(self, stream: Stream, buffers: MapBuffers, page_table_index: int, num_active_tokens: int,
                   num_active_kv_splits: int) -> None:
        abi.call("kh_sliced_kv_map", self.handle, stream.handle, C.byref(buffers.to_c()), page_table_index,
                 num_active_tokens, num_active_kv_splits)

    def invoke_reduce(self, stream: Stream, buffers: ReduceBuffers, num_active_tokens: int) -> None:
        abi.call("kh_sliced_kv_reduce", self.handle, stream.handle, C.byref(buffers.to_c()), num_active_tokens)

    def arrival_counter_bytes(self) -> int:
        out = C.c_uint64()
        abi.call("kh_sliced_kv_arrival_counter_bytes", C.byref(self.config.to_c()), C.byref(self.execution.to_c()),
                 C.byref(self.shape.to_c()), C.byref(out))
        return out.value

    def invoke_map_reduce(self, stream: Stream, map_buffers: MapBuffers, reduce_buffers: ReduceBuffers,
                          arrival_counters: Buffer, page_table_index: int, num_active_tokens: int,
                          num_active_kv_splits: int) -> None:
        """``invoke_map`` + ``invoke_reduce`` in one launch (the last block of every group merges it)."""
        abi.call("kh_sliced_kv_map_reduce", self.handle, stream.handle, C.byref(map_buffers.to_c()),
                 C.byref(reduce_buffers.to_c()), arrival_counters.ref, page_table_index, num_active_tokens,
                 num_active_kv_splits)

    def static_bytes_needed(self, num_active_kv_splits: int) -> int:
        out = C.c_uint64()
        abi.call("kh_sliced_kv_static_bytes_needed", C.byref(self.config.to_c()), num_active_kv_splits, C.byref(out))
        return out.value

    def invoke_attend_static(self, stream: Stream, buffers: StaticBuffers, page_table_index: int,
                             num_active_tokens: int, num_active_kv_splits: int) -> None:
        """``invoke_map`` + ``invoke_reduce`` with the partial state in the array the library holds
        (``abi.STATIC_PARTIALS_BYTES`` per GPU): no allocation on any call, one call in flight per GPU."""
        abi.call("kh_sliced_kv_attend_static", self.handle, stream.handle, C.byref(buffers.to_c()), page_table_index,
                 num_active_tokens, num_active_kv_splits)

    def __del__(self):
        try:
            if self.handle:
                abi.lib().kh_sliced_kv_destroy(self.handle)
                self.handle = None
        except Exception:
            pass
