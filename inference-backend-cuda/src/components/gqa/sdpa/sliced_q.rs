//! SplitKV SlicedQ SDPA: verify, append and chunked prefill; Map + Reduce, or direct output
//! (`inference-backend-metal/src/components/gqa/sdpa/sliced_q.rs:145-643`). Not compiled here; see Cargo.toml.
//!
//! Tasks of up to 64 (Q token, Q head) rows run on warp-level tensor-core tiles; 65-128 rows at head_dim 128 and
//! 16-token pages run on tcgen05 with tensor-memory accumulators. The choice is made from the variant's
//! `max_q_tokens * max_q_heads` when the compute object is created.
use crate::components::gqa::kv_page_write::PageTableLayout;
use crate::components::gqa::sdpa;
use crate::error::expect_ok;
use crate::ffi;
use crate::metal::{Buffer, CommandRecorder, Device, Dtype, Operator, ReplayU32};

/// `sliced_q::Config` (`sliced_q.rs:145-153`) plus the K/V page element type (`sliced_q.rs:202` fixes one byte).
#[derive(Clone, Copy, Debug, PartialEq)]
pub struct Config {
    pub num_q_heads: u32,
    pub num_kv_heads: u32,
    pub head_dim: u32,
    pub scale: f32,
    pub page_bytes: u32,
    pub dtype: Dtype,
    pub page_table_layout: PageTableLayout,
    pub kv_dtype: Dtype,
}

impl Config {
    pub fn sizes(self, execution: sdpa::ExecutionVariant, shape: Shape) -> ffi::KhSlicedQSizes {
        let mut out = unsafe { std::mem::zeroed::<ffi::KhSlicedQSizes>() };
        expect_ok(unsafe { ffi::kh_sliced_q_sizes_get(&self.to_ffi(), &execution.to_ffi(), &shape.to_ffi(), &mut out) },
                  "sliced_q::Config::validate");
        out
    }

    pub fn to_ffi(self) -> ffi::KhSlicedQConfig {
        ffi::KhSlicedQConfig {
            num_q_heads: self.num_q_heads,
            num_kv_heads: self.num_kv_heads,
            head_dim: self.head_dim,
            scale: self.scale,
            page_bytes: self.page_bytes,
            dtype: self.dtype as u32,
            page_table_layout: self.page_table_layout.to_ffi(),
            kv_dtype: self.kv_dtype as u32,
        }
    }
}

#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub struct Shape {
    pub num_total_tokens: u32,
    pub num_total_q_token_tiles: u32,
    pub num_total_sdpa_map_task_templates: u32,
}

impl Shape {
    pub fn to_ffi(self) -> ffi::KhSlicedQShape {
        ffi::KhSlicedQShape {
            num_total_tokens: self.num_total_tokens,
            num_total_q_token_tiles: self.num_total_q_token_tiles,
            num_total_sdpa_map_task_templates: self.num_total_sdpa_map_task_templates,
        }
    }
}

#[derive(Clone, Copy)]
pub struct MapBuffers<'a> {
    pub q: &'a Buffer,
    pub kv_pages: &'a Buffer,
    pub req_slots: &'a Buffer,
    pub page_ids: &'a Buffer,
    /// Per-flat-Q-token half-open request-local visible K/V ranges.
    pub visible_kv_token_ranges: &'a Buffer,
    pub q_token_ranges: &'a Buffer,
    pub sdpa_map_task_templates: &'a Buffer,
    pub partial_output: &'a Buffer,
    pub partial_exp_sums: &'a Buffer,
    pub partial_max_logits: &'a Buffer,
}

/// Unsplit SDPA inputs and final output: exactly one Map template per Q range.
#[derive(Clone, Copy)]
pub struct DirectBuffers<'a> {
    pub q: &'a Buffer,
    pub kv_pages: &'a Buffer,
    pub req_slots: &'a Buffer,
    pub page_ids: &'a Buffer,
    pub visible_kv_token_ranges: &'a Buffer,
    pub q_token_ranges: &'a Buffer,
    pub sdpa_map_task_templates: &'a Buffer,
    pub output: &'a Buffer,
}

#[derive(Clone, Copy)]
pub struct ReduceBuffers<'a> {
    pub partial_output: &'a Buffer,
    pub partial_exp_sums: &'a Buffer,
    pub partial_max_logits: &'a Buffer,
    pub q_token_ranges: &'a Buffer,
    pub cu_sdpa_partial_outputs: &'a Buffer,
    pub output: &'a Buffer,
}

pub struct Compute {
    raw: *mut ffi::KhSlicedQ,
    shape: Shape,
    direct_output: bool,
}

impl Compute {
    pub fn new(device: &Device, config: Config, execution: sdpa::ExecutionVariant, shape: Shape) -> Self {
        Self::create(device, config, execution, shape, false)
    }

    pub fn new_direct(device: &Device, config: Config, execution: sdpa::ExecutionVariant, shape: Shape) -> Self {
        assert_eq!(shape.num_total_sdpa_map_task_templates, shape.num_total_q_token_tiles);
        Self::create(device, config, execution, shape, true)
    }

    fn create(device: &Device, config: Config, execution: sdpa::ExecutionVariant, shape: Shape, direct: bool) -> Self {
        let mut raw = std::ptr::null_mut();
        expect_ok(unsafe { ffi::kh_sliced_q_create(device.raw(), &config.to_ffi(), &execution.to_ffi(), &shape.to_ffi(),
                                                   direct as i32, &mut raw) },
                  "sliced_q::Compute::new");
        Self { raw, shape, direct_output: direct }
    }

    pub fn shape(&self) -> Shape {
        self.shape
    }

    pub fn invoke_map<'a>(&'a self, buffers: MapBuffers<'a>, page_table_index: ReplayU32,
                          num_active_tokens: ReplayU32, num_active_q_token_tiles: ReplayU32,
                          num_active_kv_splits: ReplayU32) -> MapInvocation<'a> {
        assert!(!self.direct_output);
        MapInvocation {
            compute: self,
            buffers: MapOrDirect::Map(buffers),
            page_table_index,
            num_active_tokens,
            num_active_q_token_tiles,
            num_active_kv_splits,
        }
    }

    pub fn invoke_direct<'a>(&'a self, buffers: DirectBuffers<'a>, page_table_index: ReplayU32,
                             num_active_tokens: ReplayU32, num_active_q_token_tiles: ReplayU32) -> MapInvocation<'a> {
        assert!(self.direct_output);
        MapInvocation {
            compute: self,
            buffers: MapOrDirect::Direct(buffers),
            page_table_index,
            num_active_tokens,
            num_active_q_token_tiles,
            num_active_kv_splits: num_active_q_token_tiles,
        }
    }

    pub fn invoke_reduce<'a>(&'a self, buffers: ReduceBuffers<'a>, num_active_q_token_tiles: ReplayU32)
        -> ReduceInvocation<'a> {
        assert!(!self.direct_output);
        ReduceInvocation { compute: self, buffers, num_active_q_token_tiles }
    }
}

impl Drop for Compute {
    fn drop(&mut self) {
        unsafe { ffi::kh_sliced_q_destroy(self.raw) };
    }
}

enum MapOrDirect<'a> {
    Map(MapBuffers<'a>),
    Direct(DirectBuffers<'a>),
}

pub struct MapInvocation<'a> {
    compute: &'a Compute,
    buffers: MapOrDirect<'a>,
    page_table_index: ReplayU32,
    num_active_tokens: ReplayU32,
    num_active_q_token_tiles: ReplayU32,
    num_active_kv_splits: ReplayU32,
}

impl Operator for MapInvocation<'_> {
    fn record(self, recorder: &CommandRecorder<'_>) {
        let ReplayU32::Value(page_table_index) = self.page_table_index else {
            panic!("sliced_q map: page_table_index must be a value on the CUDA backend");
        };
        recorder.require_replay_counts(self.num_active_tokens.is_parameter()
            || self.num_active_q_token_tiles.is_parameter() || self.num_active_kv_splits.is_parameter());
        let stream = recorder.stream().raw();
        match self.buffers {
            MapOrDirect::Map(b) => {
                let buffers = ffi::KhSlicedQMapBuffers {
                    q: b.q.raw(),
                    kv_pages: b.kv_pages.raw(),
                    req_slots: b.req_slots.raw(),
                    page_ids: b.page_ids.raw(),
                    visible_kv_token_ranges: b.visible_kv_token_ranges.raw(),
                    q_token_ranges: b.q_token_ranges.raw(),
                    sdpa_map_task_templates: b.sdpa_map_task_templates.raw(),
                    partial_output: b.partial_output.raw(),
                    partial_exp_sums: b.partial_exp_sums.raw(),
                    partial_max_logits: b.partial_max_logits.raw(),
                };
                expect_ok(unsafe { ffi::kh_sliced_q_map(self.compute.raw, stream, &buffers, page_table_index,
                                                        self.num_active_tokens.bound(),
                                                        self.num_active_q_token_tiles.bound(),
                                                        self.num_active_kv_splits.bound()) },
                          "sliced_q map");
            }
            MapOrDirect::Direct(b) => {
                let buffers = ffi::KhSlicedQDirectBuffers {
                    q: b.q.raw(),
                    kv_pages: b.kv_pages.raw(),
                    req_slots: b.req_slots.raw(),
                    page_ids: b.page_ids.raw(),
                    visible_kv_token_ranges: b.visible_kv_token_ranges.raw(),
                    q_token_ranges: b.q_token_ranges.raw(),
                    sdpa_map_task_templates: b.sdpa_map_task_templates.raw(),
                    output: b.output.raw(),
                };
                expect_ok(unsafe { ffi::kh_sliced_q_direct(self.compute.raw, stream, &buffers, page_table_index,
                                                           self.num_active_tokens.bound(),
                                                           self.num_active_q_token_tiles.bound()) },
                          "sliced_q direct");
            }
        }
    }
}

pub struct ReduceInvocation<'a> {
    compute: &'a Compute,
    buffers: ReduceBuffers<'a>,
    num_active_q_token_tiles: ReplayU32,
}

impl Operator for ReduceInvocation<'_> {
    fn record(self, recorder: &CommandRecorder<'_>) {
        recorder.require_replay_counts(self.num_active_q_token_tiles.is_parameter());
        let buffers = ffi::KhSlicedQReduceBuffers {
            partial_output: self.buffers.partial_output.raw(),
            partial_exp_sums: self.buffers.partial_exp_sums.raw(),
            partial_max_logits: self.buffers.partial_max_logits.raw(),
            q_token_ranges: self.buffers.q_token_ranges.raw(),
            cu_sdpa_partial_outputs: self.buffers.cu_sdpa_partial_outputs.raw(),
            output: self.buffers.output.raw(),
        };
        expect_ok(unsafe { ffi::kh_sliced_q_reduce(self.compute.raw, recorder.stream().raw(), &buffers,
                                                   self.num_active_q_token_tiles.bound()) },
                  "sliced_q reduce");
    }
}
