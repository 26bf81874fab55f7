"""Device, Buffer and Stream: the CUDA stand-ins for the reference's Metal runtime objects
(crates/inference-backend-metal/src/metal/{device,buffer,stream}). Thin wrappers over the C ABI."""
from __future__ import annotations

import ctypes as C
import enum

import numpy as np

from . import abi


class Dtype(enum.IntEnum):
    """Element types; values are the ordinals of the reference's ``Dtype`` enum (metal/dtype.rs:1-16)."""

    Uint32 = 3
    Float16 = 9
    Float32 = 10
    Bfloat16 = 12
    Fp8E4M3FN = 100

    def item_size(self) -> int:
        return {Dtype.Uint32: 4, Dtype.Float16: 2, Dtype.Float32: 4, Dtype.Bfloat16: 2, Dtype.Fp8E4M3FN: 1}[self]


class Device:
    """``Device::system_default`` (metal/device.rs:12-15) for CUDA device ``ordinal``."""

    def __init__(self, ordinal: int = 0):
        handle = C.c_void_p()
        abi.call("kh_device_open", ordinal, C.byref(handle))
        self.handle = handle
        self.ordinal = ordinal

    @staticmethod
    def system_default() -> "Device":
        return Device(0)

    def sm_count(self) -> int:
        out = C.c_int32()
        abi.call("kh_device_sm_count", self.handle, C.byref(out))
        return out.value

    def check(self, stream: "Stream | None" = None) -> int:
        """Reads and clears the sticky device status word; raises ``KhError`` (Aborted) when nonzero."""
        word = C.c_uint32()
        abi.call("kh_device_check", self.handle, stream.handle if stream else None, C.byref(word))
        return word.value

    def set_wait_limit(self, polls: int) -> None:
        """Polls a wait inside a kernel makes before it gives up and the kernel returns with bit 0 of the status
        word set (``kh_device_set_wait_limit``); 0 restores the default."""
        abi.call("kh_device_set_wait_limit", self.handle, int(polls))

    def close(self) -> None:
        if self.handle:
            abi.call("kh_device_close", self.handle)
            self.handle = None


class Buffer:
    """Device buffer: ``Buffer::new_zeroed`` / ``from_slice`` / ``write_typed`` / ``read_typed``."""

    def __init__(self, device: Device, ref: abi.BufferRef, owned: bool):
        self.device = device
        self.ref = ref
        self.owned = owned

    @staticmethod
    def new_zeroed(device: Device, num_bytes: int) -> "Buffer":
        ref = abi.BufferRef()
        abi.call("kh_buffer_alloc", device.handle, int(num_bytes), C.byref(ref))
        return Buffer(device, ref, True)

    @staticmethod
    def new_zeroed_elements(device: Device, count: int, dtype: Dtype) -> "Buffer":
        return Buffer.new_zeroed(device, count * Dtype(dtype).item_size())

    @staticmethod
    def from_slice(device: Device, values: np.ndarray) -> "Buffer":
        values = np.ascontiguousarray(values)
        buf = Buffer.new_zeroed(device, max(values.nbytes, 1))
        buf.write(0, values)
        return buf

    @staticmethod
    def wrap(device: Device, ptr: int, num_bytes: int) -> "Buffer":
        """Adopts device memory owned by someone else (for example a torch tensor's ``data_ptr()``)."""
        return Buffer(device, abi.BufferRef(ptr, num_bytes), False)

    def len_bytes(self) -> int:
        return int(self.ref.bytes)

    def write(self, byte_offset: int, values: np.ndarray) -> None:
        values = np.ascontiguousarray(values)
        abi.call("kh_buffer_write", self.device.handle, self.ref, int(byte_offset), values.ctypes.data, values.nbytes)

    def write_typed(self, element_offset: int, values) -> None:
        values = np.ascontiguousarray(values)
        self.write(element_offset * values.itemsize, values)

    def read(self, byte_offset: int, count: int, dtype) -> np.ndarray:
        out = np.empty(count, dtype=dtype)
        abi.call("kh_buffer_read", self.device.handle, self.ref, int(byte_offset), out.ctypes.data, out.nbytes)
        return out

    def read_typed(self, element_offset: int, count: int, dtype=np.uint32) -> np.ndarray:
        return self.read(element_offset * np.dtype(dtype).itemsize, count, dtype)

    def zero_bytes(self, byte_offset: int, num_bytes: int) -> None:
        abi.call("kh_buffer_zero", self.device.handle, self.ref, int(byte_offset), int(num_bytes))

    def free(self) -> None:
        if self.owned and self.ref.ptr:
            abi.call("kh_buffer_free", self.device.handle, self.ref)
            self.ref = abi.BufferRef()

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class Stream:
    """``Stream::new`` (metal/stream/mod.rs); ``wrap`` adopts an existing ``cudaStream_t``."""

    def __init__(self, device: Device, cuda_stream: int | None = None):
        handle = C.c_void_p()
        if cuda_stream is None:
            abi.call("kh_stream_create", device.handle, C.byref(handle))
        else:
            abi.call("kh_stream_wrap", device.handle, C.c_void_p(cuda_stream), C.byref(handle))
        self.handle = handle
        self.device = device

    def synchronize(self) -> None:
        abi.call("kh_stream_synchronize", self.handle)

    def write(self, buffer: Buffer, byte_offset: int, host_ptr: int, num_bytes: int) -> None:
        abi.call("kh_stream_write", self.handle, buffer.ref, int(byte_offset), C.c_void_p(host_ptr), int(num_bytes))

    def read(self, buffer: Buffer, byte_offset: int, host_ptr: int, num_bytes: int) -> None:
        abi.call("kh_stream_read", self.handle, buffer.ref, int(byte_offset), C.c_void_p(host_ptr), int(num_bytes))

    def bind_active_counts(self, counts: "Buffer | None") -> None:
        """While bound, SDPA launches recorded on this stream read their active counts from ``counts`` when they
        run (four u32: tokens, Q-token tiles, map task templates, 0); ``None`` returns to by-value counts."""
        abi.call("kh_stream_bind_active_counts", self.handle, counts.ref if counts is not None else abi.BufferRef())

    def record_event(self, event: "Event") -> None:
        abi.call("kh_stream_record_event", self.handle, event.handle)

    def wait_event(self, event: "Event") -> None:
        """Orders the work recorded on this stream from now on after ``event``; the host does not block."""
        abi.call("kh_stream_wait_event", self.handle, event.handle)

    def destroy(self) -> None:
        if self.handle:
            abi.call("kh_stream_destroy", self.handle)
            self.handle = None


class Event:
    """Completion of the work recorded on a stream so far: the analogue of ``ReplaySubmission``
    (metal/stream/submission.rs:41-101); ``synchronize`` is its ``wait``."""

    def __init__(self, device: Device):
        handle = C.c_void_p()
        abi.call("kh_event_create", device.handle, C.byref(handle))
        self.handle = handle
        self.device = device

    def synchronize(self) -> None:
        abi.call("kh_event_synchronize", self.handle)

    def destroy(self) -> None:
        if self.handle:
            abi.call("kh_event_destroy", self.handle)
            self.handle = None


class PinnedArray:
    """A numpy view over page-locked host memory (``cudaHostAlloc``), for stream-ordered copies."""

    def __init__(self, shape, dtype):
        self.dtype = np.dtype(dtype)
        self.shape = tuple(np.atleast_1d(shape).tolist())
        self.nbytes = int(np.prod(self.shape)) * self.dtype.itemsize
        ptr = C.c_void_p()
        abi.call("kh_host_alloc_pinned", max(self.nbytes, 1), C.byref(ptr))
        self.ptr = ptr.value
        raw = (C.c_uint8 * max(self.nbytes, 1)).from_address(self.ptr)
        self.array = np.frombuffer(raw, dtype=self.dtype, count=int(np.prod(self.shape))).reshape(self.shape)

    def free(self) -> None:
        if self.ptr:
            self.array = None
            abi.call("kh_host_free_pinned", C.c_void_p(self.ptr))
            self.ptr = None
