"""Request page table: ``GQAPageTableLayout`` / ``GQARequestPageTable``
(crates/inference-executor-metal/src/attn/gqa/request_page_table.rs:7-161). The table is a device u32
tensor ``[num_req_slots, num_gqa_layers, num_blocks, num_page_ids_per_block]``; one physical page holds
``[K/V, kv_head, page_token_index, head_dim]``."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

import numpy as np

from . import abi
from .device import Buffer, Device


@dataclass(frozen=True)
class GQAPageTableLayout:
    num_req_slots: int
    num_gqa_layers: int
    num_blocks: int
    num_page_ids_per_block: int

    def to_c(self) -> abi.PageTableLayoutC:
        return abi.PageTableLayoutC(self.num_req_slots, self.num_gqa_layers, self.num_blocks,
                                    self.num_page_ids_per_block)

    def validate(self) -> None:
        self.bytes()

    def bytes(self) -> int:
        out = C.c_uint64()
        abi.call("kh_page_table_bytes", C.byref(self.to_c()), C.byref(out))
        return out.value

    def num_page_ids(self) -> int:
        return self.bytes() // 4

    def num_physical_pages_per_request(self) -> int:
        return self.num_blocks * self.num_page_ids_per_block

    def start_index(self, req_slot: int, layer_index: int, block_index: int) -> int:
        out = C.c_uint64()
        abi.call("kh_page_table_index", C.byref(self.to_c()), req_slot, layer_index, block_index, C.byref(out))
        return out.value


PageTableLayout = GQAPageTableLayout  # the backend twin (components/gqa/kv_page_write.rs:33-57)


class GQARequestPageTable:
    def __init__(self, device: Device, layout: GQAPageTableLayout):
        layout.validate()
        self._layout = layout
        self._device = device
        self._page_ids = Buffer.new_zeroed(device, layout.bytes())

    def layout(self) -> GQAPageTableLayout:
        return self._layout

    def num_req_slots(self) -> int:
        return self._layout.num_req_slots

    def num_layers(self) -> int:
        return self._layout.num_gqa_layers

    def num_blocks(self) -> int:
        return self._layout.num_blocks

    def num_page_ids_per_block(self) -> int:
        return self._layout.num_page_ids_per_block

    def page_ids_buffer(self) -> Buffer:
        return self._page_ids

    def write_page_ids(self, req_slot: int, layer_index: int, block_index: int, page_ids) -> None:
        ids = np.ascontiguousarray(page_ids, dtype=np.uint32)
        abi.call("kh_page_table_write", self._device.handle, self._page_ids.ref, C.byref(self._layout.to_c()),
                 req_slot, layer_index, block_index, ids.ctypes.data_as(C.POINTER(C.c_uint32)), ids.size)

    def read_page_ids(self, req_slot: int, layer_index: int, block_index: int) -> list[int]:
        ids = np.zeros(self._layout.num_page_ids_per_block, dtype=np.uint32)
        abi.call("kh_page_table_read", self._device.handle, self._page_ids.ref, C.byref(self._layout.to_c()),
                 req_slot, layer_index, block_index, ids.ctypes.data_as(C.POINTER(C.c_uint32)), ids.size)
        return ids.tolist()

    def reset_req_slot(self, req_slot: int) -> None:
        abi.call("kh_page_table_reset_req_slot", self._device.handle, self._page_ids.ref,
                 C.byref(self._layout.to_c()), req_slot)

    def reset_req_slots(self, req_slots) -> None:
        for slot in req_slots:
            self.reset_req_slot(slot)
