//! SplitKV SlicedKv SDPA: one Q token per Map task, the KV range cut into slices, then Reduce
//! (`inference-backend-metal/src/components/gqa/sdpa/sliced_kv.rs:90-663`). Not compiled here; see Cargo.toml.
use crate::components::gqa::kv_page_write::PageTableLayout;
use crate::components::gqa::sdpa;
use crate::error::{check, expect_ok};
use crate::ffi;
use crate::metal::{Buffer, CommandRecorder, Device, Dtype, Operator, ReplayU32};

/// `sliced_kv::Config` (`sliced_kv.rs:90-98`) plus the element type of the K/V pages, which the reference fixes
/// at one byte (`sliced_kv.rs:113-125`).
#[derive(Clone, Copy, Debug, PartialEq)]
pub struct Config {
    pub num_q_heads: u32,
    pub num_kv_heads: u32,
    pub head_dim: u32,
    pub scale: f32,
    pub page_bytes: u32,
    pub page_table_layout: PageTableLayout,
    pub dtype: Dtype,
    pub kv_dtype: Dtype,
}

impl Config {
    pub fn validate(self) {
        self.sizes(Shape { num_total_tokens: 1, num_total_sdpa_map_task_templates: 1 });
    }

    /// Byte sizes of every buffer an invocation binds; also runs `Config::validate` and `Shape::validate`.
    /// Partial outputs are f32 on this backend: size `GQAScratch` from here.
    pub fn sizes(self, shape: Shape) -> ffi::KhSlicedKvSizes {
        let mut out = unsafe { std::mem::zeroed::<ffi::KhSlicedKvSizes>() };
        expect_ok(unsafe { ffi::kh_sliced_kv_sizes_get(&self.to_ffi(), &shape.to_ffi(), &mut out) },
                  "sliced_kv::Config::validate");
        out
    }

    pub fn num_tokens_per_page(self) -> u32 {
        self.sizes(Shape { num_total_tokens: 1, num_total_sdpa_map_task_templates: 1 }).num_tokens_per_page
    }

    pub fn q_heads_per_kv_head(self) -> u32 {
        self.num_q_heads / self.num_kv_heads
    }

    pub fn q_bytes(self, shape: Shape) -> usize {
        self.sizes(shape).q_bytes as usize
    }

    pub fn partial_output_stats_bytes(self, shape: Shape) -> usize {
        self.sizes(shape).partial_output_stats_bytes as usize
    }

    pub fn partial_output_bytes(self, shape: Shape) -> usize {
        self.sizes(shape).partial_output_bytes as usize
    }

    pub fn to_ffi(self) -> ffi::KhSlicedKvConfig {
        ffi::KhSlicedKvConfig {
            num_q_heads: self.num_q_heads,
            num_kv_heads: self.num_kv_heads,
            head_dim: self.head_dim,
            scale: self.scale,
            page_bytes: self.page_bytes,
            page_table_layout: self.page_table_layout.to_ffi(),
            dtype: self.dtype as u32,
            kv_dtype: self.kv_dtype as u32,
        }
    }
}

#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub struct Shape {
    pub num_total_tokens: u32,
    pub num_total_sdpa_map_task_templates: u32,
}

impl Shape {
    pub fn validate(self, config: Config) {
        config.sizes(self);
    }

    pub fn to_ffi(self) -> ffi::KhSlicedKvShape {
        ffi::KhSlicedKvShape {
            num_total_tokens: self.num_total_tokens,
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
    pub sdpa_map_task_templates: &'a Buffer,
    pub partial_exp_sums: &'a Buffer,
    pub partial_max_logits: &'a Buffer,
    pub partial_output: &'a Buffer,
}

#[derive(Clone, Copy)]
pub struct ReduceBuffers<'a> {
    pub partial_exp_sums: &'a Buffer,
    pub partial_max_logits: &'a Buffer,
    pub partial_output: &'a Buffer,
    pub cu_sdpa_partial_outputs: &'a Buffer,
    pub output: &'a Buffer,
}

/// Partial statistics and partial outputs (`Scratch`, `sliced_kv.rs:256-305`), f32 here.
pub struct Scratch {
    pub partial_exp_sums: Buffer,
    pub partial_max_logits: Buffer,
    pub partial_output: Buffer,
}

impl Scratch {
    pub fn new(device: &Device, config: Config, shape: Shape) -> inference_error::Result<Self> {
        let sizes = config.sizes(shape);
        Ok(Self {
            partial_exp_sums: Buffer::new_zeroed(device, sizes.partial_output_stats_bytes as usize)?,
            partial_max_logits: Buffer::new_zeroed(device, sizes.partial_output_stats_bytes as usize)?,
            partial_output: Buffer::new_zeroed(device, sizes.partial_output_bytes as usize)?,
        })
    }
}

pub struct Compute {
    raw: *mut ffi::KhSlicedKv,
    shape: Shape,
}

impl Compute {
    /// `Compute::new(device, config, execution, shape)` (`sliced_kv.rs:322-355`). Panics where the reference's
    /// asserts would (an unsupported variant, a shape outside the u32 domains).
    pub fn new(device: &Device, config: Config, execution: sdpa::ExecutionVariant, shape: Shape) -> Self {
        let mut raw = std::ptr::null_mut();
        expect_ok(unsafe { ffi::kh_sliced_kv_create(device.raw(), &config.to_ffi(), &execution.to_ffi(),
                                                    &shape.to_ffi(), &mut raw) },
                  "sliced_kv::Compute::new");
        Self { raw, shape }
    }

    pub fn try_new(device: &Device, config: Config, execution: sdpa::ExecutionVariant, shape: Shape)
        -> inference_error::Result<Self> {
        let mut raw = std::ptr::null_mut();
        check(unsafe { ffi::kh_sliced_kv_create(device.raw(), &config.to_ffi(), &execution.to_ffi(),
                                                &shape.to_ffi(), &mut raw) })?;
        Ok(Self { raw, shape })
    }

    pub fn shape(&self) -> Shape {
        self.shape
    }

    pub fn invoke_map<'a>(&'a self, buffers: MapBuffers<'a>, page_table_index: ReplayU32,
                          num_active_tokens: ReplayU32, num_active_kv_splits: ReplayU32) -> MapInvocation<'a> {
        MapInvocation { compute: self, buffers, page_table_index, num_active_tokens, num_active_kv_splits }
    }

    pub fn invoke_reduce<'a>(&'a self, buffers: ReduceBuffers<'a>, num_active_tokens: ReplayU32)
        -> ReduceInvocation<'a> {
        ReduceInvocation { compute: self, buffers, num_active_tokens }
    }
}

impl Drop for Compute {
    fn drop(&mut self) {
        unsafe { ffi::kh_sliced_kv_destroy(self.raw) };
    }
}

pub struct MapInvocation<'a> {
    compute: &'a Compute,
    buffers: MapBuffers<'a>,
    page_table_index: ReplayU32,
    num_active_tokens: ReplayU32,
    num_active_kv_splits: ReplayU32,
}

impl Operator for MapInvocation<'_> {
    fn record(self, recorder: &CommandRecorder<'_>) {
        // the page-table (layer) index is fixed per recorded layer on this backend
        let ReplayU32::Value(page_table_index) = self.page_table_index else {
            panic!("sliced_kv map: page_table_index must be a value on the CUDA backend");
        };
        recorder.require_replay_counts(self.num_active_tokens.is_parameter() || self.num_active_kv_splits.is_parameter());
        let buffers = ffi::KhSlicedKvMapBuffers {
            q: self.buffers.q.raw(),
            kv_pages: self.buffers.kv_pages.raw(),
            req_slots: self.buffers.req_slots.raw(),
            page_ids: self.buffers.page_ids.raw(),
            sdpa_map_task_templates: self.buffers.sdpa_map_task_templates.raw(),
            partial_exp_sums: self.buffers.partial_exp_sums.raw(),
            partial_max_logits: self.buffers.partial_max_logits.raw(),
            partial_output: self.buffers.partial_output.raw(),
        };
        // MapInvocation::validate (sliced_kv.rs:594-612) runs inside the library; a violation panics here
        expect_ok(unsafe { ffi::kh_sliced_kv_map(self.compute.raw, recorder.stream().raw(), &buffers, page_table_index,
                                                 self.num_active_tokens.bound(), self.num_active_kv_splits.bound()) },
                  "sliced_kv map");
    }
}

pub struct ReduceInvocation<'a> {
    compute: &'a Compute,
    buffers: ReduceBuffers<'a>,
    num_active_tokens: ReplayU32,
}

impl Operator for ReduceInvocation<'_> {
    fn record(self, recorder: &CommandRecorder<'_>) {
        recorder.require_replay_counts(self.num_active_tokens.is_parameter());
        let buffers = ffi::KhSlicedKvReduceBuffers {
            partial_exp_sums: self.buffers.partial_exp_sums.raw(),
            partial_max_logits: self.buffers.partial_max_logits.raw(),
            partial_output: self.buffers.partial_output.raw(),
            cu_sdpa_partial_outputs: self.buffers.cu_sdpa_partial_outputs.raw(),
            output: self.buffers.output.raw(),
        };
        expect_ok(unsafe { ffi::kh_sliced_kv_reduce(self.compute.raw, recorder.stream().raw(), &buffers,
                                                    self.num_active_tokens.bound()) },
                  "sliced_kv reduce");
    }
}
