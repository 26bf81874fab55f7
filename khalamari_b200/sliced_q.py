"""SlicedQ SDPA compute (a tile of Q tokens x Q heads per task: verify, append, prefill), with split
map + reduce or direct output: ``Config``, ``Shape``, ``MapBuffers``, ``DirectBuffers``, ``ReduceBuffers``,
``Compute`` (crates/inference-backend-metal/src/components/gqa/sdpa/sliced_q.rs)."""
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
    dtype: Dtype
    page_table_layout: GQAPageTableLayout
    kv_dtype: Dtype | None = None

    def kv_element_dtype(self) -> Dtype:
        return self.dtype if self.kv_dtype is None else self.kv_dtype

    def to_c(self) -> abi.SlicedQConfigC:
        return abi.SlicedQConfigC(self.num_q_heads, self.num_kv_heads, self.head_dim, self.scale, self.page_bytes,
                                  int(self.dtype), self.page_table_layout.to_c(), int(self.kv_element_dtype()))

    def sizes(self, execution: sdpa.ExecutionVariant, shape: "Shape") -> abi.SlicedQSizesC:
        out = abi.SlicedQSizesC()
        abi.call("kh_sliced_q_sizes_get", C.byref(self.to_c()), C.byref(execution.to_c()), C.byref(shape.to_c()),
                 C.byref(out))
        return out

    def num_tokens_per_page(self) -> int:
        return self.page_bytes // (2 * self.num_kv_heads * self.head_dim * self.kv_element_dtype().item_size())

    def q_heads_per_kv_head(self) -> int:
        return self.num_q_heads // self.num_kv_heads

    def sdpa_config(self) -> sdpa.Config:
        return sdpa.Config(self.dtype, self.num_q_heads, self.num_kv_heads, self.head_dim, self.num_tokens_per_page())

    def q_bytes(self, shape: "Shape") -> int:
        return shape.num_total_tokens * self.num_q_heads * self.head_dim * self.dtype.item_size()

    def partial_output_bytes(self, execution, shape) -> int:
        return self.sizes(execution, shape).partial_output_bytes

    def partial_output_stats_bytes(self, execution, shape) -> int:
        return self.sizes(execution, shape).partial_output_stats_bytes


@dataclass(frozen=True)
class Shape:
    num_total_tokens: int
    num_total_q_token_tiles: int
    num_total_sdpa_map_task_templates: int

    def to_c(self) -> abi.SlicedQShapeC:
        return abi.SlicedQShapeC(self.num_total_tokens, self.num_total_q_token_tiles,
                                 self.num_total_sdpa_map_task_templates)


@dataclass
class MapBuffers:
    q: Buffer
    kv_pages: Buffer
    req_slots: Buffer
    page_ids: Buffer
    visible_kv_token_ranges: Buffer
    q_token_ranges: Buffer
    sdpa_map_task_templates: Buffer
    partial_output: Buffer
    partial_exp_sums: Buffer
    partial_max_logits: Buffer

    def to_c(self) -> abi.SlicedQMapBuffersC:
        return abi.SlicedQMapBuffersC(*[getattr(self, name).ref for name, _ in abi.SlicedQMapBuffersC._fields_])


@dataclass
class DirectBuffers:
    q: Buffer
    kv_pages: Buffer
    req_slots: Buffer
    page_ids: Buffer
    visible_kv_token_ranges: Buffer
    q_token_ranges: Buffer
    sdpa_map_task_templates: Buffer
    output: Buffer

    def to_c(self) -> abi.SlicedQDirectBuffersC:
        return abi.SlicedQDirectBuffersC(
            *[getattr(self, name).ref for name, _ in abi.SlicedQDirectBuffersC._fields_])


@dataclass
class ReduceBuffers:
    partial_output: Buffer
    partial_exp_sums: Buffer
    partial_max_logits: Buffer
    q_token_ranges: Buffer
    cu_sdpa_partial_outputs: Buffer
    output: Buffer

    def to_c(self) -> abi.SlicedQReduceBuffersC:
        return abi.SlicedQReduceBuffersC(
            *[getattr(self, name).ref for name, _ in abi.SlicedQReduceBuffersC._fields_])


class Compute:
    """``Compute`` (sliced_q.rs:347-503)."""

    def __init__(self, device: Device, config: Config, execution: sdpa.ExecutionVariant, shape: Shape,
                 direct_output: bool = False):
        handle = C.c_void_p()
        abi.call("kh_sliced_q_create", device.handle, C.byref(config.to_c()), C.byref(execution.to_c()),
                 C.byref(shape.to_c()), int(direct_output), C.byref(handle))
        self.handle = handle
        self.config = config
        self.shape = shape
        self.execution = execution
        self.direct_output = direct_output

    @staticmethod
    def new(device, config, execution, shape) -> "Compute":
        return Compute(device, config, execution, shape, False)

    @staticmethod
    def new_direct(device, config, execution, shape) -> "Compute":
        return Compute(device, config, execution, shape, True)

    def invoke_map(self, stream: Stream, buffers: MapBuffers, page_table_index: int, num_active_tokens: int,
                   num_active_q_token_tiles: int, num_active_kv_splits: int) -> None:
        abi.call("kh_sliced_q_map", self.handle, stream.handle, C.byref(buffers.to_c()), page_table_index,
                 num_active_tokens, num_active_q_token_tiles, num_active_kv_splits)

    def invoke_direct(self, stream: Stream, buffers: DirectBuffers, page_table_index: int, num_active_tokens: int,
                      num_active_q_token_tiles: int) -> None:
        abi.call("kh_sliced_q_direct", self.handle, stream.handle, C.byref(buffers.to_c()), page_table_index,
                 num_active_tokens, num_active_q_token_tiles)

    def invoke_reduce(self, stream: Stream, buffers: ReduceBuffers, num_active_q_token_tiles: int) -> None:
        abi.call("kh_sliced_q_reduce", self.handle, stream.handle, C.byref(buffers.to_c()),
                 num_active_q_token_tiles)

    def arrival_counter_bytes(self) -> int:
        out = C.c_uint64()
        abi.call("kh_sliced_q_arrival_counter_bytes", C.byref(self.config.to_c()), C.byref(self.execution.to_c()),
                 C.byref(self.shape.to_c()), C.byref(out))
        return out.value

    def invoke_map_reduce(self, stream: Stream, map_buffers: MapBuffers, reduce_buffers: ReduceBuffers,
                          arrival_counters: Buffer, page_table_index: int, num_active_tokens: int,
                          num_active_q_token_tiles: int, num_active_kv_splits: int) -> None:
        """``invoke_map`` + ``invoke_reduce`` in one launch (the last block of every group merges it)."""
        abi.call("kh_sliced_q_map_reduce", self.handle, stream.handle, C.byref(map_buffers.to_c()),
                 C.byref(reduce_buffers.to_c()), arrival_counters.ref, page_table_index, num_active_tokens,
                 num_active_q_token_tiles, num_active_kv_splits)

    def __del__(self):
        try:
            if self.handle:
                abi.lib().kh_sliced_q_destroy(self.handle)
                self.handle = None
        except Exception:
            pass
