//! GQA attention components of the CUDA backend. Not compiled here; see Cargo.toml.
pub mod bidi_block_sdpa;
pub mod kv_page_write;
pub mod sdpa;

pub use kv_page_write::PageTableLayout;
