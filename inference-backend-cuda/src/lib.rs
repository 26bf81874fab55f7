//! `inference-backend-cuda`: the B200 (sm_100a) backend of khalamari's paged GQA split-KV attention.
//!
//! **Not compiled in this repository's build image** (it has no Rust toolchain). This crate is the source a
//! maintainer adds beside `inference-backend-metal`; it exposes, for the attention path only, the type names,
//! fields and method signatures of `inference-backend-metal/src/components/gqa/{sdpa.rs, sdpa/sliced_kv.rs,
//! sdpa/sliced_q.rs, kv_page_write.rs}` over the C ABI of `libkhcuda_gqa` (`include/kh_gqa.h`), so that
//! `GQA::record_sdpa` (`inference-executor-metal/src/attn/gqa/backend.rs:438-542`) reads the same against it.
//!
//! What differs from the Metal backend, by design:
//! * partial outputs are `f32` (`[Mt][Hq][max_q_tokens][D]`): size scratch from `Config::sizes`;
//! * `Config` carries `kv_dtype`: `Dtype::Fp8E4M3FN` is the reference's one-byte cache format,
//!   `kv_dtype == dtype` (bf16 / fp16 pages) the faster one;
//! * a `CommandRecorder` is a CUDA stream; `Operator::record` enqueues on it and never blocks;
//! * invalid invocations panic, as the reference's `validate()` asserts do: the library returns
//!   `KH_INVALID_ARGUMENT` with the failed condition in its message and the wrapper panics with that message;
//!   fallible set-up (`Device::open`, allocation) returns `inference_error::Result`.

pub mod components;
pub mod error;
pub mod ffi;
pub mod metal;
pub mod selector;

pub use metal::{Buffer, CommandRecorder, Device, Dtype, Operator, ReplayU32, Stream, Submission};
