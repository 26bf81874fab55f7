//! `kh_status` -> `inference_error::Error` (the status codes are named after its variants,
//! `crates/inference-error/src/lib.rs:4-28`). Not compiled here; see Cargo.toml.
use inference_error::Error;

use crate::ffi;

/// The calling thread's last library message.
pub fn last_error() -> String {
    let mut buffer = vec![0u8; 2048];
    let length = unsafe { ffi::kh_last_error(buffer.as_mut_ptr().cast(), buffer.len()) };
    buffer.truncate(length.min(buffer.len().saturating_sub(1)));
    String::from_utf8_lossy(&buffer).into_owned()
}

pub fn check(status: ffi::KhStatus) -> inference_error::Result<()> {
    let message = || last_error();
    match status {
        ffi::KH_OK => Ok(()),
        ffi::KH_INVALID_ARGUMENT => Err(Error::InvalidArgument(message())),
        ffi::KH_RESOURCE_EXHAUSTED => Err(Error::ResourceExhausted(message())),
        ffi::KH_CANCELLED => Err(Error::Cancelled(message())),
        ffi::KH_DEADLINE_EXCEEDED => Err(Error::DeadlineExceeded(message())),
        ffi::KH_ABORTED => Err(Error::Aborted(message())),
        ffi::KH_EVICTED => Err(Error::Evicted(message())),
        ffi::KH_UNAVAILABLE => Err(Error::Unavailable(message())),
        _ => Err(Error::Internal(message())),
    }
}

/// For the call sites where the reference panics (`validate()` asserts, `Operator::record`).
pub fn expect_ok(status: ffi::KhStatus, what: &str) {
    if status != ffi::KH_OK {
        panic!("{what}: {}", last_error());
    }
}
