"""Batch metadata ABI: ``GQAMetadataBuffers``
(crates/inference-executor-metal/src/attn/gqa/batch_metadata.rs:100-320). Six capacity-sized u32 device
arrays refreshed from one complete selection. Host images live in page-locked memory so that ``update``
is a fill plus stream-ordered copies."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import abi
from .device import Buffer, Device, PinnedArray, Stream
from .replay import GQAReplayShape
from .sdpa import ExecutionVariant, MapKernelKind
from .selector import Selection

_FIELDS = (("req_slots", 1), ("flat_token_indices", 1), ("visible_kv_token_ranges", 2), ("q_token_ranges", 2),
           ("sdpa_map_task_templates", 3), ("cu_sdpa_partial_outputs", 1))


class GQAMetadataBuffers:
    def __init__(self, device: Device, max_tokens: int, max_map_task_templates: int):
        if max_tokens <= 0:
            raise abi.InvalidArgument(1, "GQA batch metadata requires tokens")
        if max_map_task_templates <= 0:
            raise abi.InvalidArgument(1, "GQA batch metadata requires Map task templates")
        self._device = device
        self._max_tokens = max_tokens
        self._max_maps = max_map_task_templates
        counts = {
            "req_slots": max_tokens, "flat_token_indices": max_tokens, "visible_kv_token_ranges": max_tokens * 2,
            "q_token_ranges": max_tokens * 2, "sdpa_map_task_templates": max_map_task_templates * 3,
            "cu_sdpa_partial_outputs": max_tokens + 1,
        }
        # One page-locked host block and one device block hold all arrays (each on a 256-byte boundary) and the four
        # replay-count words, so that ``update`` is one fill and ONE stream-ordered copy; the arrays handed to the
        # kernels are views into the device block.
        self._offsets = {}
        cursor = 256  # the first 256 bytes hold the replay-count words
        self._counts_offset = 0
        # the template array (the only large one) goes last, so that the copy can stop after the templates in use
        order = [name for name in counts if name != "sdpa_map_task_templates"] + ["sdpa_map_task_templates"]
        for name in order:
            count = counts[name]
            self._offsets[name] = (cursor, count)
            cursor += -(-count * 4 // 256) * 256
        self._block_bytes = cursor
        self._host_block = PinnedArray(cursor // 4, np.uint32)
        self._host_block.array[:] = 0
        self._dev_block = Buffer.new_zeroed(device, cursor)
        self._host = {name: self._host_block.array[off // 4: off // 4 + count] for name, (off, count) in self._offsets.items()}
        self._host_ptr = {name: self._host_block.ptr + off for name, (off, _) in self._offsets.items()}
        self._dev = {name: Buffer.wrap(device, self._dev_block.ref.ptr + off, count * 4)
                     for name, (off, count) in self._offsets.items()}
        # replay counts {num_active_tokens, num_active_q_token_tiles, num_active_kv_splits, 0}: the device words a
        # recorded (graph-captured) launch reads its active counts from (Stream.bind_active_counts)
        self._host_counts = self._host_block.array[self._counts_offset // 4: self._counts_offset // 4 + 4]
        self._active_counts = Buffer.wrap(device, self._dev_block.ref.ptr + self._counts_offset, 16)
        self._uploaded_bytes = 0
        self._replay_shape = None
        self._variant = None

    def max_tokens(self) -> int:
        return self._max_tokens

    def max_map_task_templates(self) -> int:
        return self._max_maps

    def update(self, req_slots, token_indices, cu_tokens, selection: Selection,
               stream: Stream | None = None) -> GQAReplayShape:
        """``GQAMetadataBuffers::update`` (batch_metadata.rs:171-253): fills the host images through the C
        ABI and uploads the written prefixes (on ``stream`` when given, else synchronously)."""
        rs = np.ascontiguousarray(req_slots, dtype=np.uint32)
        ti = np.ascontiguousarray(token_indices, dtype=np.uint32)
        cu = np.ascontiguousarray(cu_tokens, dtype=np.uint32)
        if rs.size != ti.size or cu.size != rs.size + 1:
            raise abi.InvalidArgument(1, "GQA metadata update needs one slot and index per request and n+1 offsets")
        u32p = C.POINTER(C.c_uint32)
        arrays = abi.MetadataArraysC(
            *[C.cast(self._host_ptr[name], u32p) for name, _ in _FIELDS], self._max_tokens, self._max_maps)
        shape_c = abi.ReplayShapeC()
        abi.call("kh_metadata_update", C.byref(arrays), rs.ctypes.data_as(u32p), ti.ctypes.data_as(u32p),
                 cu.ctypes.data_as(u32p), rs.size, selection.handle, C.byref(shape_c))
        shape = GQAReplayShape.from_c(shape_c)
        variant = selection.variant()
        self._host_counts[:] = (shape.num_tokens, shape.num_q_token_tiles, shape.num_sdpa_map_task_templates, 0)
        used = self._offsets["sdpa_map_task_templates"][0] + shape.num_total_sdpa_map_task_templates * 12
        self._uploaded_bytes = used
        if stream is None:
            self._dev_block.write(0, self._host_block.array[:used // 4])
        else:
            stream.write(self._dev_block, 0, self._host_block.ptr, used)
        self._replay_shape = shape
        self._variant = variant
        return shape

    def upload_bytes(self) -> int:
        """Bytes the last ``update`` copied to the device (the block up to the last template in use)."""
        return self._uploaded_bytes

    def req_slots(self) -> Buffer:
        return self._dev["req_slots"]

    def flat_token_indices(self) -> Buffer:
        return self._dev["flat_token_indices"]

    def visible_kv_token_ranges(self) -> Buffer:
        return self._dev["visible_kv_token_ranges"]

    def q_token_ranges(self) -> Buffer:
        return self._dev["q_token_ranges"]

    def sdpa_map_task_templates(self) -> Buffer:
        return self._dev["sdpa_map_task_templates"]

    def cu_sdpa_partial_outputs(self) -> Buffer:
        return self._dev["cu_sdpa_partial_outputs"]

    def active_counts(self) -> Buffer:
        return self._active_counts

    def host_image(self, name: str) -> np.ndarray:
        return self._host[name]

    def replay_shape(self) -> GQAReplayShape:
        if self._replay_shape is None:
            raise abi.InvalidArgument(1, "GQA batch metadata must be updated before recording")
        return self._replay_shape

    def variant(self) -> ExecutionVariant:
        if self._variant is None:
            raise abi.InvalidArgument(1, "GQA batch metadata must be updated before recording")
        return self._variant

    def direct_output(self) -> bool:
        return self.variant().kind != MapKernelKind.SlicedKv and not self.replay_shape().reduce_sdpa_partial_outputs
