//! Device, buffer, stream and recorder objects with the names the Metal backend gives them
//! (`inference-backend-metal/src/metal/{device,buffer,dtype}.rs`, `metal/stream/{mod,operation,submission,
//! check}.rs`), over CUDA. Not compiled here; see Cargo.toml.
//!
//! The module keeps the name `metal` on purpose: `use inference_backend_cuda::metal::{Buffer, Device}` is then the
//! only line a call site of the attention path changes.
use std::cell::Cell;
use std::ptr;

use crate::error::{check, expect_ok};
use crate::ffi;

/// Element types; discriminants are the ordinals the library reads (`metal/dtype.rs:1-16`).
#[derive(Clone, Copy, Debug, Eq, Hash, PartialEq)]
#[repr(u32)]
pub enum Dtype {
    Float16 = ffi::KH_DTYPE_FLOAT16,
    Float32 = ffi::KH_DTYPE_FLOAT32,
    Bfloat16 = ffi::KH_DTYPE_BFLOAT16,
    /// KV-cache pages only: the reference's one-byte cache format (`components/gqa/fp8.rs`).
    Fp8E4M3FN = ffi::KH_DTYPE_FP8_E4M3FN,
}

impl Dtype {
    pub fn item_size(self) -> usize {
        match self {
            Dtype::Float16 | Dtype::Bfloat16 => 2,
            Dtype::Float32 => 4,
            Dtype::Fp8E4M3FN => 1,
        }
    }
}

/// `Device::system_default` (`metal/device.rs:12-15`) for one CUDA device. One owner thread per device.
#[derive(Debug)]
pub struct Device {
    raw: *mut ffi::KhDevice,
}

impl Device {
    pub fn open(ordinal: i32) -> inference_error::Result<Self> {
        let mut raw = ptr::null_mut();
        check(unsafe { ffi::kh_device_open(ordinal, &mut raw) })?;
        Ok(Self { raw })
    }

    pub fn system_default() -> inference_error::Result<Self> {
        Self::open(0)
    }

    pub fn raw(&self) -> *mut ffi::KhDevice {
        self.raw
    }

    pub fn sm_count(&self) -> u32 {
        let mut out = 0i32;
        expect_ok(unsafe { ffi::kh_device_sm_count(self.raw, &mut out) }, "kh_device_sm_count");
        out as u32
    }

    /// `SubmissionCheck` (`metal/stream/check.rs:8-13`): waits for `stream`, then reads and clears the sticky
    /// status word the kernels write. `Err(Aborted)` names the bits: a bounded wait ran out, a page id beyond the
    /// pool, metadata beyond the page table.
    pub fn check(&self, stream: Option<&Stream>) -> inference_error::Result<()> {
        let mut word = 0u32;
        check(unsafe { ffi::kh_device_check(self.raw, stream.map_or(ptr::null_mut(), Stream::raw), &mut word) })
    }

    /// Polls a wait inside a kernel makes before the kernel gives up (0: the default).
    pub fn set_wait_limit(&self, polls: u32) {
        expect_ok(unsafe { ffi::kh_device_set_wait_limit(self.raw, polls) }, "kh_device_set_wait_limit");
    }
}

impl Drop for Device {
    fn drop(&mut self) {
        unsafe { ffi::kh_device_close(self.raw) };
    }
}

/// Device memory (`metal/buffer.rs`): owned (`new_zeroed`, `from_slice`) or a view of memory someone else owns.
#[derive(Debug)]
pub struct Buffer {
    device: *mut ffi::KhDevice,
    raw: ffi::KhBufferRef,
    owned: bool,
}

impl Buffer {
    pub fn new_zeroed(device: &Device, num_bytes: usize) -> inference_error::Result<Self> {
        let mut raw = ffi::KhBufferRef { ptr: ptr::null_mut(), bytes: 0 };
        check(unsafe { ffi::kh_buffer_alloc(device.raw(), num_bytes as u64, &mut raw) })?;
        Ok(Self { device: device.raw(), raw, owned: true })
    }

    pub fn from_slice<T: Copy>(device: &Device, values: &[T]) -> inference_error::Result<Self> {
        let buffer = Self::new_zeroed(device, std::mem::size_of_val(values).max(1))?;
        buffer.write_typed(0, values);
        Ok(buffer)
    }

    /// Adopts device memory owned elsewhere (a CUDA allocation of the executor's arena).
    ///
    /// # Safety
    /// `ptr .. ptr + num_bytes` must stay valid device memory of `device` for the life of the view.
    pub unsafe fn wrap(device: &Device, ptr: *mut core::ffi::c_void, num_bytes: usize) -> Self {
        Self { device: device.raw(), raw: ffi::KhBufferRef { ptr, bytes: num_bytes as u64 }, owned: false }
    }

    pub fn len_bytes(&self) -> usize {
        self.raw.bytes as usize
    }

    pub fn raw(&self) -> ffi::KhBufferRef {
        self.raw
    }

    pub fn write_typed<T: Copy>(&self, element_offset: usize, values: &[T]) {
        let bytes = std::mem::size_of_val(values) as u64;
        let offset = (element_offset * std::mem::size_of::<T>()) as u64;
        expect_ok(unsafe { ffi::kh_buffer_write(self.device, self.raw, offset, values.as_ptr().cast(), bytes) },
                  "Buffer::write_typed");
    }

    pub fn read_typed<T: Copy + Default>(&self, element_offset: usize, count: usize) -> Vec<T> {
        let mut out = vec![T::default(); count];
        let offset = (element_offset * std::mem::size_of::<T>()) as u64;
        expect_ok(unsafe { ffi::kh_buffer_read(self.device, self.raw, offset, out.as_mut_ptr().cast(),
                                               (count * std::mem::size_of::<T>()) as u64) },
                  "Buffer::read_typed");
        out
    }

    pub fn zero_bytes(&self, byte_offset: usize, num_bytes: usize) {
        expect_ok(unsafe { ffi::kh_buffer_zero(self.device, self.raw, byte_offset as u64, num_bytes as u64) },
                  "Buffer::zero_bytes");
    }
}

impl Drop for Buffer {
    fn drop(&mut self) {
        if self.owned {
            unsafe { ffi::kh_buffer_free(self.device, self.raw) };
        }
    }
}

/// One in-order queue (`metal/stream/mod.rs`): a CUDA stream, created here or adopted from the executor.
#[derive(Debug)]
pub struct Stream {
    raw: *mut ffi::KhStream,
}

impl Stream {
    pub fn new(device: &Device) -> inference_error::Result<Self> {
        let mut raw = ptr::null_mut();
        check(unsafe { ffi::kh_stream_create(device.raw(), &mut raw) })?;
        Ok(Self { raw })
    }

    /// # Safety
    /// `cuda_stream` must be a live `cudaStream_t` of `device`.
    pub unsafe fn wrap(device: &Device, cuda_stream: *mut core::ffi::c_void) -> inference_error::Result<Self> {
        let mut raw = ptr::null_mut();
        check(unsafe { ffi::kh_stream_wrap(device.raw(), cuda_stream, &mut raw) })?;
        Ok(Self { raw })
    }

    pub fn raw(&self) -> *mut ffi::KhStream {
        self.raw
    }

    /// Records operators; the analogue of building a replay program's command list. Launches go to the stream at
    /// once (CUDA has no separate encode step); capture the stream into a CUDA graph to get a replayable program.
    pub fn recorder(&self) -> CommandRecorder<'_> {
        CommandRecorder { stream: self, parameters: Cell::new(None) }
    }

    /// Marks the work recorded so far; `Submission::wait` is `ReplaySubmission::wait`
    /// (`metal/stream/submission.rs:88`).
    pub fn submit(&self, device: &Device) -> inference_error::Result<Submission> {
        let mut raw = ptr::null_mut();
        check(unsafe { ffi::kh_event_create(device.raw(), &mut raw) })?;
        let submission = Submission { raw };
        check(unsafe { ffi::kh_stream_record_event(self.raw, raw) })?;
        Ok(submission)
    }

    /// Orders what is recorded on this stream from now on after `submission` (recorded on another stream of the
    /// same device); the host does not block.
    pub fn wait_for(&self, submission: &Submission) {
        expect_ok(unsafe { ffi::kh_stream_wait_event(self.raw, submission.raw) }, "Stream::wait_for");
    }

    pub fn synchronize(&self) {
        expect_ok(unsafe { ffi::kh_stream_synchronize(self.raw) }, "Stream::synchronize");
    }
}

impl Drop for Stream {
    fn drop(&mut self) {
        unsafe { ffi::kh_stream_destroy(self.raw) };
    }
}

/// Completion handle of the work a stream held when `Stream::submit` was called.
#[derive(Debug)]
pub struct Submission {
    raw: *mut ffi::KhEvent,
}

impl Submission {
    pub fn wait(&self) {
        expect_ok(unsafe { ffi::kh_event_synchronize(self.raw) }, "Submission::wait");
    }
}

impl Drop for Submission {
    fn drop(&mut self) {
        unsafe { ffi::kh_event_destroy(self.raw) };
    }
}

/// A count an invocation takes (`metal/stream/replay.rs`): a value fixed at record time, or a parameter the
/// launch reads on the device when it runs, so that one recorded (graph-captured) program serves every batch of
/// a replay bucket. The library knows one parameter block per stream: four `u32`
/// `{num_active_tokens, num_active_q_token_tiles, num_active_kv_splits, 0}`; `Parameter { capacity }` names the
/// recorded capacity the device value is clamped to.
#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub enum ReplayU32 {
    Value(u32),
    Parameter { capacity: u32 },
}

impl ReplayU32 {
    /// What the library is given as the by-value count: the value, or the capacity that bounds the device word.
    pub fn bound(self) -> u32 {
        match self {
            ReplayU32::Value(value) => value,
            ReplayU32::Parameter { capacity } => capacity,
        }
    }

    pub fn is_parameter(self) -> bool {
        matches!(self, ReplayU32::Parameter { .. })
    }
}

/// Recordable backend execution unit (`metal/stream/operation.rs:17-24`).
pub trait Operator {
    fn record(self, recorder: &CommandRecorder<'_>);
}

/// Where operators record: the stream, plus the device words replay parameters are read from.
pub struct CommandRecorder<'a> {
    stream: &'a Stream,
    parameters: Cell<Option<ffi::KhBufferRef>>,
}

impl<'a> CommandRecorder<'a> {
    pub fn stream(&self) -> &'a Stream {
        self.stream
    }

    /// Binds the four replay-count words (16 bytes of device memory the metadata owner rewrites per batch). While
    /// bound, every attention launch recorded here reads its active counts from them.
    pub fn bind_replay_counts(&self, counts: Option<&Buffer>) {
        let raw = counts.map_or(ffi::KhBufferRef { ptr: ptr::null_mut(), bytes: 0 }, Buffer::raw);
        expect_ok(unsafe { ffi::kh_stream_bind_active_counts(self.stream.raw(), raw) }, "bind_replay_counts");
        self.parameters.set(counts.map(Buffer::raw));
    }

    /// An invocation recorded with `ReplayU32::Parameter` counts needs the words bound.
    pub fn require_replay_counts(&self, any_parameter: bool) {
        assert!(!any_parameter || self.parameters.get().is_some(),
                "an invocation with ReplayU32::Parameter counts was recorded without bind_replay_counts");
    }

    /// `record_with_barrier_before` of the reference orders an operator after the previous one; a CUDA stream is
    /// in order already, so this only records.
    pub fn record_with_barrier_before<O: Operator>(&self, operator: O) {
        operator.record(self);
    }

    pub fn record<O: Operator>(&self, operator: O) {
        operator.record(self);
    }
}
