"""KV page write: ``Config``, ``Shape``, ``Buffers``, ``Compute``
(crates/inference-backend-metal/src/components/gqa/kv_page_write.rs) and the FP8 E4M3FN storage codec of
crates/inference-backend-metal/src/components/gqa/fp8.rs."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

from . import abi
from .device import Buffer, Device, Dtype, Stream
from .request_page_table import GQAPageTableLayout

MAX_FINITE = 448.0


def bf16_to_fp8_e4m3(bf16_bits: int) -> int:
    """``bf16_to_fp8_e4m3`` (fp8.rs:19-44) on bit patterns."""
    return int(abi.lib().kh_fp8_e4m3_from_bf16(int(bf16_bits) & 0xFFFF))


def fp8_e4m3_to_bf16(fp8_bits: int) -> int:
    """``fp8_e4m3_to_bf16`` (fp8.rs:46-58) on bit patterns."""
    return int(abi.lib().kh_fp8_e4m3_to_bf16(int(fp8_bits) & 0xFF))


@dataclass(frozen=True)
class Config:
    num_kv_heads: int
    head_dim: int
    page_bytes: int
    dtype: Dtype = Dtype.Bfloat16
    kv_dtype: Dtype = Dtype.Fp8E4M3FN  # the reference's cache format; ``dtype`` stores the source bits unchanged

    def to_c(self) -> abi.KvPageWriteConfigC:
        return abi.KvPageWriteConfigC(self.num_kv_heads, self.head_dim, self.page_bytes, int(self.dtype),
                                      int(self.kv_dtype))

    def num_tokens_per_page(self) -> int:
        out = C.c_uint32()
        abi.call("kh_kv_page_write_tokens_per_page", C.byref(self.to_c()), C.byref(out))
        return out.value

    def validate(self) -> None:
        self.num_tokens_per_page()

    def num_total_threads(self, shape: "Shape") -> int:
        return shape.num_total_token_writes * self.num_kv_heads * self.head_dim

    def flat_kv_bytes(self, shape: "Shape") -> int:
        return self.num_total_threads(shape) * self.dtype.item_size()

    def index_bytes(self, shape: "Shape") -> int:
        return shape.num_total_token_writes * 4


@dataclass(frozen=True)
class Shape:
    num_total_token_writes: int
    page_table_layout: GQAPageTableLayout

    def to_c(self) -> abi.KvPageWriteShapeC:
        return abi.KvPageWriteShapeC(self.num_total_token_writes, self.page_table_layout.to_c())

    def page_ids_bytes(self) -> int:
        return self.page_table_layout.num_page_ids() * 4


@dataclass
class Buffers:
    pages: Buffer
    flat_k: Buffer
    flat_v: Buffer
    req_slots: Buffer
    flat_token_indices: Buffer
    page_ids: Buffer

    def to_c(self) -> abi.KvPageWriteBuffersC:
        return abi.KvPageWriteBuffersC(*[getattr(self, name).ref for name, _ in abi.KvPageWriteBuffersC._fields_])


class Compute:
    """``Compute`` (kv_page_write.rs:153-193); ``invoke`` enqueues on ``stream`` (``Invocation::record``)."""

    def __init__(self, device: Device, config: Config):
        handle = C.c_void_p()
        abi.call("kh_kv_page_write_create", device.handle, C.byref(config.to_c()), C.byref(handle))
        self.handle = handle
        self.config = config

    @staticmethod
    def new(device: Device, config: Config) -> "Compute":
        return Compute(device, config)

    def invoke(self, stream: Stream, shape: Shape, buffers: Buffers, num_active_token_writes: int,
               page_table_index: int = 0) -> None:
        abi.call("kh_kv_page_write_invoke", self.handle, stream.handle, C.byref(shape.to_c()),
                 C.byref(buffers.to_c()), num_active_token_writes, page_table_index)

    def __del__(self):
        try:
            if self.handle:
                abi.lib().kh_kv_page_write_destroy(self.handle)
                self.handle = None
        except Exception:
            pass
