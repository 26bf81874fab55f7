//! KV page write and the page-table layout (`inference-backend-metal/src/components/gqa/kv_page_write.rs:33-257`),
//! plus the FP8 E4M3FN storage codec on bit patterns (`components/gqa/fp8.rs:19-58`). Not compiled here; see
//! Cargo.toml.
use crate::error::expect_ok;
use crate::ffi;
use crate::metal::{Buffer, CommandRecorder, Device, Dtype, Operator, ReplayU32};

/// `page_ids[num_req_slots][num_gqa_layers][num_blocks][num_page_ids_per_block]` (`kv_page_write.rs:33-57`).
#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub struct PageTableLayout {
    pub num_req_slots: u32,
    pub num_gqa_layers: u32,
    pub num_blocks: u32,
    pub num_page_ids_per_block: u32,
}

impl PageTableLayout {
    pub fn bytes(self) -> usize {
        let mut out = 0u64;
        expect_ok(unsafe { ffi::kh_page_table_bytes(&self.to_ffi(), &mut out) }, "PageTableLayout::bytes");
        out as usize
    }

    pub fn to_ffi(self) -> ffi::KhPageTableLayout {
        ffi::KhPageTableLayout {
            num_req_slots: self.num_req_slots,
            num_gqa_layers: self.num_gqa_layers,
            num_blocks: self.num_blocks,
            num_page_ids_per_block: self.num_page_ids_per_block,
        }
    }
}

/// `kv_page_write::Config` (`kv_page_write.rs:62-68`) plus the stored element type: `Dtype::Fp8E4M3FN` is the
/// reference's store; `kv_dtype == dtype` keeps the source bits (the page format the 16-bit kernels read).
#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub struct Config {
    pub num_kv_heads: u32,
    pub head_dim: u32,
    pub page_bytes: u32,
    pub dtype: Dtype,
    pub kv_dtype: Dtype,
}

impl Config {
    pub fn num_tokens_per_page(self) -> u32 {
        let mut out = 0u32;
        expect_ok(unsafe { ffi::kh_kv_page_write_tokens_per_page(&self.to_ffi(), &mut out) },
                  "kv_page_write::Config::validate");
        out
    }

    pub fn to_ffi(self) -> ffi::KhKvPageWriteConfig {
        ffi::KhKvPageWriteConfig {
            num_kv_heads: self.num_kv_heads,
            head_dim: self.head_dim,
            page_bytes: self.page_bytes,
            dtype: self.dtype as u32,
            kv_dtype: self.kv_dtype as u32,
        }
    }
}

#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub struct Shape {
    pub num_total_token_writes: u32,
    pub page_table_layout: PageTableLayout,
}

#[derive(Clone, Copy)]
pub struct Buffers<'a> {
    pub pages: &'a Buffer,
    pub flat_k: &'a Buffer,
    pub flat_v: &'a Buffer,
    pub req_slots: &'a Buffer,
    pub flat_token_indices: &'a Buffer,
    pub page_ids: &'a Buffer,
}

pub struct Compute {
    raw: *mut ffi::KhKvPageWrite,
}

impl Compute {
    pub fn new(device: &Device, config: Config) -> Self {
        let mut raw = std::ptr::null_mut();
        expect_ok(unsafe { ffi::kh_kv_page_write_create(device.raw(), &config.to_ffi(), &mut raw) },
                  "kv_page_write::Compute::new");
        Self { raw }
    }

    pub fn invoke<'a>(&'a self, shape: Shape, buffers: Buffers<'a>, num_active_token_writes: ReplayU32,
                      page_table_index: ReplayU32) -> Invocation<'a> {
        Invocation { compute: self, shape, buffers, num_active_token_writes, page_table_index }
    }
}

impl Drop for Compute {
    fn drop(&mut self) {
        unsafe { ffi::kh_kv_page_write_destroy(self.raw) };
    }
}

pub struct Invocation<'a> {
    compute: &'a Compute,
    shape: Shape,
    buffers: Buffers<'a>,
    num_active_token_writes: ReplayU32,
    page_table_index: ReplayU32,
}

impl Operator for Invocation<'_> {
    fn record(self, recorder: &CommandRecorder<'_>) {
        let (ReplayU32::Value(writes), ReplayU32::Value(layer)) = (self.num_active_token_writes, self.page_table_index)
        else {
            panic!("kv page write takes its counts by value on the CUDA backend");
        };
        let shape = ffi::KhKvPageWriteShape {
            num_total_token_writes: self.shape.num_total_token_writes,
            page_table_layout: self.shape.page_table_layout.to_ffi(),
        };
        let buffers = ffi::KhKvPageWriteBuffers {
            pages: self.buffers.pages.raw(),
            flat_k: self.buffers.flat_k.raw(),
            flat_v: self.buffers.flat_v.raw(),
            req_slots: self.buffers.req_slots.raw(),
            flat_token_indices: self.buffers.flat_token_indices.raw(),
            page_ids: self.buffers.page_ids.raw(),
        };
        expect_ok(unsafe { ffi::kh_kv_page_write_invoke(self.compute.raw, recorder.stream().raw(), &shape, &buffers,
                                                        writes, layer) },
                  "kv page write");
    }
}

/// `bf16_to_fp8_e4m3` (`fp8.rs:19-44`) on bit patterns.
pub fn bf16_to_fp8_e4m3(bf16_bits: u16) -> u8 {
    unsafe { ffi::kh_fp8_e4m3_from_bf16(bf16_bits) }
}

/// `fp8_e4m3_to_bf16` (`fp8.rs:46-58`) on bit patterns.
pub fn fp8_e4m3_to_bf16(fp8_bits: u8) -> u16 {
    unsafe { ffi::kh_fp8_e4m3_to_bf16(fp8_bits) }
}
