//! BiDi-block SDPA: dense bidirectional attention inside one request block, written into the block's slot of the
//! SplitKV partial-state layout (`inference-backend-metal/src/components/gqa/bidi_block_sdpa.rs`). Not compiled
//! here; see Cargo.toml.
use crate::error::expect_ok;
use crate::ffi;
use crate::metal::{Buffer, CommandRecorder, Device, Dtype, Operator, ReplayU32};

#[derive(Clone, Copy, Debug, PartialEq)]
pub struct Config {
    pub block_size: u32,
    pub max_q_tokens: u32,
    pub num_q_heads: u32,
    pub num_kv_heads: u32,
    pub head_dim: u32,
    pub scale: f32,
    pub dtype: Dtype,
}

impl Config {
    pub fn to_ffi(self) -> ffi::KhBidiBlockSdpaConfig {
        ffi::KhBidiBlockSdpaConfig {
            block_size: self.block_size,
            max_q_tokens: self.max_q_tokens,
            num_q_heads: self.num_q_heads,
            num_kv_heads: self.num_kv_heads,
            head_dim: self.head_dim,
            scale: self.scale,
            dtype: self.dtype as u32,
        }
    }
}

#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub struct Shape {
    pub num_total_tokens: u32,
    pub num_total_q_token_ranges: u32,
    pub num_total_partial_output_slots: u32,
}

#[derive(Clone, Copy)]
pub struct Buffers<'a> {
    pub q: &'a Buffer,
    pub local_k: &'a Buffer,
    pub local_v: &'a Buffer,
    pub q_token_ranges: &'a Buffer,
    pub cu_sdpa_partial_outputs: &'a Buffer,
    pub partial_exp_sums: &'a Buffer,
    pub partial_max_logits: &'a Buffer,
    /// f32 on this backend (the Metal backend stores the io dtype).
    pub partial_output: &'a Buffer,
}

pub struct Compute {
    raw: *mut ffi::KhBidiBlockSdpa,
}

impl Compute {
    pub fn new(device: &Device, config: Config) -> Self {
        let mut raw = std::ptr::null_mut();
        expect_ok(unsafe { ffi::kh_bidi_block_sdpa_create(device.raw(), &config.to_ffi(), &mut raw) },
                  "bidi_block_sdpa::Compute::new");
        Self { raw }
    }

    pub fn invoke<'a>(&'a self, shape: Shape, num_active_q_token_ranges: ReplayU32, buffers: Buffers<'a>) -> Invocation<'a> {
        Invocation { compute: self, shape, num_active_q_token_ranges, buffers }
    }
}

impl Drop for Compute {
    fn drop(&mut self) {
        unsafe { ffi::kh_bidi_block_sdpa_destroy(self.raw) };
    }
}

pub struct Invocation<'a> {
    compute: &'a Compute,
    shape: Shape,
    num_active_q_token_ranges: ReplayU32,
    buffers: Buffers<'a>,
}

impl Operator for Invocation<'_> {
    fn record(self, recorder: &CommandRecorder<'_>) {
        recorder.require_replay_counts(self.num_active_q_token_ranges.is_parameter());
        let shape = ffi::KhBidiBlockSdpaShape {
            num_total_tokens: self.shape.num_total_tokens,
            num_total_q_token_ranges: self.shape.num_total_q_token_ranges,
            num_total_partial_output_slots: self.shape.num_total_partial_output_slots,
        };
        let buffers = ffi::KhBidiBlockSdpaBuffers {
            q: self.buffers.q.raw(),
            local_k: self.buffers.local_k.raw(),
            local_v: self.buffers.local_v.raw(),
            q_token_ranges: self.buffers.q_token_ranges.raw(),
            cu_sdpa_partial_outputs: self.buffers.cu_sdpa_partial_outputs.raw(),
            partial_exp_sums: self.buffers.partial_exp_sums.raw(),
            partial_max_logits: self.buffers.partial_max_logits.raw(),
            partial_output: self.buffers.partial_output.raw(),
        };
        expect_ok(unsafe { ffi::kh_bidi_block_sdpa_invoke(self.compute.raw, recorder.stream().raw(), &shape,
                                                          self.num_active_q_token_ranges.bound(), &buffers) },
                  "bidi block sdpa");
    }
}
