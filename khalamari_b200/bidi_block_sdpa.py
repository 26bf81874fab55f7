"""BiDi-block SDPA: ``Config``, ``Shape``, ``Buffers``, ``Compute``
(crates/inference-backend-metal/src/components/gqa/bidi_block_sdpa.rs) and the metadata of one proposal step
(``build_metal_metadata``, crates/inference-executor-metal/src/attn/bidi_block_gqa/metadata.rs:176-339).

Dense bidirectional attention of every Q token over all tokens of its own request block, written as one more
partial (slot ``cu_sdpa_partial_outputs[range + 1] - 1``) of the SplitKV partial-state layout; the sliced-Q map
kernel supplies the history partials of the same ranges and the sliced-Q reducer merges them."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import abi
from .device import Buffer, Device, Dtype, Stream
from .replay import GQAReplayShape


@dataclass(frozen=True)
class Config:
    block_size: int
    max_q_tokens: int
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    scale: float
    dtype: Dtype

    def to_c(self) -> abi.BidiBlockSdpaConfigC:
        return abi.BidiBlockSdpaConfigC(self.block_size, self.max_q_tokens, self.num_q_heads, self.num_kv_heads,
                                        self.head_dim, self.scale, int(self.dtype))

    def q_elements(self, shape: "Shape") -> int:
        return shape.num_total_tokens * self.num_q_heads * self.head_dim

    def kv_elements(self, shape: "Shape") -> int:
        return shape.num_total_tokens * self.num_kv_heads * self.head_dim

    def partial_output_stat_elements(self, shape: "Shape") -> int:
        return shape.num_total_partial_output_slots * self.num_q_heads * self.max_q_tokens

    def partial_output_values(self, shape: "Shape") -> int:
        return self.partial_output_stat_elements(shape) * self.head_dim


@dataclass(frozen=True)
class Shape:
    num_total_tokens: int
    num_total_q_token_ranges: int
    num_total_partial_output_slots: int

    def to_c(self) -> abi.BidiBlockSdpaShapeC:
        return abi.BidiBlockSdpaShapeC(self.num_total_tokens, self.num_total_q_token_ranges,
                                       self.num_total_partial_output_slots)


@dataclass
class Buffers:
    q: Buffer
    local_k: Buffer
    local_v: Buffer
    q_token_ranges: Buffer
    cu_sdpa_partial_outputs: Buffer
    partial_exp_sums: Buffer
    partial_max_logits: Buffer
    partial_output: Buffer

    def to_c(self) -> abi.BidiBlockSdpaBuffersC:
        return abi.BidiBlockSdpaBuffersC(*[getattr(self, name).ref for name, _ in abi.BidiBlockSdpaBuffersC._fields_])


class Compute:
    """``Compute`` (bidi_block_sdpa.rs:188-244); ``invoke`` enqueues on ``stream`` (``Invocation::record``)."""

    def __init__(self, device: Device, config: Config):
        handle = C.c_void_p()
        abi.call("kh_bidi_block_sdpa_create", device.handle, C.byref(config.to_c()), C.byref(handle))
        self.handle = handle
        self.config = config

    @staticmethod
    def new(device: Device, config: Config) -> "Compute":
        return Compute(device, config)

    def invoke(self, stream: Stream, shape: Shape, num_active_q_token_ranges: int, buffers: Buffers) -> None:
        abi.call("kh_bidi_block_sdpa_invoke", self.handle, stream.handle, C.byref(shape.to_c()),
                 num_active_q_token_ranges, C.byref(buffers.to_c()))

    def __del__(self):
        try:
            if self.handle:
                abi.lib().kh_bidi_block_sdpa_destroy(self.handle)
                self.handle = None
        except Exception:
            pass


@dataclass
class BlockMetadata:
    """Host images of the metadata of one proposal step (``BiDiBlockGQAMetadataUpload``, metadata.rs:20-28)."""

    req_slots: np.ndarray
    flat_token_indices: np.ndarray
    visible_kv_token_ranges: np.ndarray
    q_token_ranges: np.ndarray
    sdpa_map_task_templates: np.ndarray
    cu_sdpa_partial_outputs: np.ndarray
    replay_shape: GQAReplayShape


def build_metadata(req_slots, token_positions, history_begins, history_ends, block_size: int, max_q_tokens: int,
                   kv_tokens_per_iteration: int, max_sdpa_map_task_templates: int) -> BlockMetadata:
    """``build_metal_metadata`` (metadata.rs:176-339) through ``kh_bidi_block_metadata_build``. ``req_slots`` has one
    entry per request, the other arrays one per token (``num_requests * block_size`` tokens)."""
    slots = np.ascontiguousarray(req_slots, dtype=np.uint32)
    positions = np.ascontiguousarray(token_positions, dtype=np.uint32)
    begins = np.ascontiguousarray(history_begins, dtype=np.uint32)
    ends = np.ascontiguousarray(history_ends, dtype=np.uint32)
    tokens = slots.size * block_size
    if not (positions.size == begins.size == ends.size == tokens):
        raise abi.InvalidArgument(1, "BiDiBlockGQA metadata needs one position and history range per token")
    images = {
        "req_slots": np.zeros(tokens, np.uint32), "flat_token_indices": np.zeros(tokens, np.uint32),
        "visible_kv_token_ranges": np.zeros(tokens * 2, np.uint32), "q_token_ranges": np.zeros(tokens * 2, np.uint32),
        "sdpa_map_task_templates": np.full(max_sdpa_map_task_templates * 3, 0xFFFFFFFF, np.uint32),
        "cu_sdpa_partial_outputs": np.zeros(tokens + 1, np.uint32),
    }
    u32p = C.POINTER(C.c_uint32)
    arrays = abi.MetadataArraysC(*[images[name].ctypes.data_as(u32p) for name, _ in abi.MetadataArraysC._fields_[:6]],
                                 tokens, max_sdpa_map_task_templates)
    shape_c = abi.ReplayShapeC()
    abi.call("kh_bidi_block_metadata_build", C.byref(arrays), slots.ctypes.data_as(u32p), positions.ctypes.data_as(u32p),
             begins.ctypes.data_as(u32p), ends.ctypes.data_as(u32p), slots.size, block_size, max_q_tokens,
             kv_tokens_per_iteration, max_sdpa_map_task_templates, C.byref(shape_c))
    shape = GQAReplayShape.from_c(shape_c)
    ranges = shape.num_q_token_tiles
    return BlockMetadata(images["req_slots"], images["flat_token_indices"], images["visible_kv_token_ranges"],
                         images["q_token_ranges"][:ranges * 2],
                         images["sdpa_map_task_templates"][:shape.num_total_sdpa_map_task_templates * 3],
                         images["cu_sdpa_partial_outputs"][:ranges + 1], shape)
