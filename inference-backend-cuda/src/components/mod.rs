//! Components follow the reference's convention `Config / Shape / Buffers / Compute / Invocation: Operator`
//! (`inference-backend-metal/src/components/mod.rs:8-14`). Not compiled here; see Cargo.toml.
pub mod gqa;
