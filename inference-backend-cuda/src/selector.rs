//! The SDPA selector and batch metadata as the library's host code computes them: `Selector`, `Selection`,
//! `RequestShape`, `GQAReplayShape` and the metadata fill
//! (`inference-executor-metal/src/attn/gqa/sdpa.rs:15-466`, `batch_metadata.rs:11-253`). Not compiled here; see
//! Cargo.toml.
//!
//! The executor may keep its own Rust selector: the kernels read the arrays `GQAMetadataBuffers::update` writes,
//! bit for bit. What this module adds is the route table re-derived for the SM count of the GPU
//! (`SelectorPolicy::B200`); `SelectorPolicy::Reference` reproduces the reference's routes exactly.
use crate::components::gqa::kv_page_write::PageTableLayout;
use crate::components::gqa::sdpa::{Config, ExecutionVariant};
use crate::error::expect_ok;
use crate::ffi;

#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub struct RequestShape {
    pub num_history_tokens: u32,
    pub num_q_tokens: u32,
}

impl RequestShape {
    /// `RequestShape::from_batch` (`sdpa.rs:22-41`): history lengths and cumulative new-token offsets of a batch.
    pub fn from_batch(token_indices: &[u32], cu_tokens: &[u32]) -> Vec<Self> {
        assert_eq!(cu_tokens.len(), token_indices.len() + 1);
        token_indices
            .iter()
            .zip(cu_tokens.windows(2))
            .map(|(&history, pair)| Self { num_history_tokens: history, num_q_tokens: pair[1] - pair[0] })
            .collect()
    }
}

#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub enum SelectorPolicy {
    Reference,
    B200,
}

pub type GQAReplayShape = ffi::KhReplayShape;
pub type SelectorLimits = ffi::KhSelectorLimits;
pub type MapTaskTemplate = ffi::KhMapTaskTemplate;
pub type QTokenRange = ffi::KhQTokenRange;

pub struct Selector {
    raw: *mut ffi::KhSelector,
}

impl Selector {
    /// `Selector::for_lookup` (`sdpa.rs:210-276`).
    pub fn for_lookup(config: Config, max_tokens: u32, layout: PageTableLayout) -> Self {
        let mut raw = std::ptr::null_mut();
        expect_ok(unsafe { ffi::kh_selector_create_for_lookup(&config.to_ffi(), max_tokens, &layout.to_ffi(), &mut raw) },
                  "Selector::for_lookup");
        Self { raw }
    }

    pub fn set_policy(&mut self, policy: SelectorPolicy, sm_count: u32) {
        let policy = match policy {
            SelectorPolicy::Reference => ffi::KH_POLICY_REFERENCE,
            SelectorPolicy::B200 => ffi::KH_POLICY_B200,
        };
        expect_ok(unsafe { ffi::kh_selector_set_policy(self.raw, policy, sm_count) }, "Selector::set_policy");
    }

    pub fn limits(&self) -> SelectorLimits {
        let mut out = unsafe { std::mem::zeroed::<SelectorLimits>() };
        expect_ok(unsafe { ffi::kh_selector_limits_get(self.raw, &mut out) }, "Selector::limits");
        out
    }

    /// `Selector::select` (`sdpa.rs:278-380`); the replay buckets are those of
    /// `GQAReplayBucketPolicy::new(limits.max_tokens, limits.max_map_task_templates)`.
    pub fn select(&self, requests: &[RequestShape], num_total_tokens: u32) -> Selection {
        let limits = self.limits();
        let raw_requests: Vec<ffi::KhRequestShape> = requests
            .iter()
            .map(|r| ffi::KhRequestShape { num_history_tokens: r.num_history_tokens, num_q_tokens: r.num_q_tokens })
            .collect();
        let mut raw = std::ptr::null_mut();
        expect_ok(unsafe { ffi::kh_selector_select(self.raw, raw_requests.as_ptr(), raw_requests.len() as u32,
                                                   limits.max_tokens, limits.max_map_task_templates, num_total_tokens,
                                                   &mut raw) },
                  "Selector::select");
        Selection { raw }
    }

    /// `Selector::select_partitioned` (`sdpa.rs:382-426`): a forced variant and KV slice.
    pub fn select_partitioned(&self, variant: ExecutionVariant, kv_slice: u32, direct_output: bool,
                              requests: &[RequestShape], num_total_tokens: u32) -> Selection {
        let limits = self.limits();
        let raw_requests: Vec<ffi::KhRequestShape> = requests
            .iter()
            .map(|r| ffi::KhRequestShape { num_history_tokens: r.num_history_tokens, num_q_tokens: r.num_q_tokens })
            .collect();
        let mut raw = std::ptr::null_mut();
        expect_ok(unsafe { ffi::kh_selector_select_partitioned(self.raw, &variant.to_ffi(), kv_slice, direct_output as i32,
                                                               raw_requests.as_ptr(), raw_requests.len() as u32,
                                                               limits.max_tokens, limits.max_map_task_templates,
                                                               num_total_tokens, &mut raw) },
                  "Selector::select_partitioned");
        Selection { raw }
    }
}

impl Drop for Selector {
    fn drop(&mut self) {
        unsafe { ffi::kh_selector_destroy(self.raw) };
    }
}

/// `Selection` (`sdpa.rs:89-125`).
pub struct Selection {
    raw: *mut ffi::KhSelection,
}

impl Selection {
    pub fn variant(&self) -> ExecutionVariant {
        let mut out = unsafe { std::mem::zeroed::<ffi::KhExecutionVariant>() };
        expect_ok(unsafe { ffi::kh_selection_variant(self.raw, &mut out) }, "Selection::variant");
        ExecutionVariant::from_ffi(out)
    }

    pub fn direct_output(&self) -> bool {
        let mut out = 0i32;
        expect_ok(unsafe { ffi::kh_selection_direct_output(self.raw, &mut out) }, "Selection::direct_output");
        out != 0
    }

    pub fn replay_shape(&self) -> GQAReplayShape {
        let mut out = unsafe { std::mem::zeroed::<GQAReplayShape>() };
        expect_ok(unsafe { ffi::kh_selection_replay_shape(self.raw, &mut out) }, "Selection::replay_shape");
        out
    }

    pub fn map_task_templates(&self) -> Vec<MapTaskTemplate> {
        let mut count = 0u32;
        expect_ok(unsafe { ffi::kh_selection_map_task_templates(self.raw, std::ptr::null_mut(), 0, &mut count) },
                  "Selection::map_task_templates");
        let mut out = vec![MapTaskTemplate { q_token_range_index: 0, kv_token_begin: 0, kv_token_end: 0 }; count as usize];
        expect_ok(unsafe { ffi::kh_selection_map_task_templates(self.raw, out.as_mut_ptr(), count, &mut count) },
                  "Selection::map_task_templates");
        out
    }

    /// `GQAMetadataBuffers::update` (`batch_metadata.rs:171-253`) into host images the caller owns (page-locked
    /// memory it then copies to the device arrays with one stream-ordered copy). Returns the replay shape.
    pub fn fill_metadata(&self, arrays: &ffi::KhMetadataArrays, req_slots: &[u32], token_indices: &[u32],
                         cu_tokens: &[u32]) -> GQAReplayShape {
        assert_eq!(req_slots.len(), token_indices.len());
        assert_eq!(cu_tokens.len(), req_slots.len() + 1);
        let mut shape = unsafe { std::mem::zeroed::<GQAReplayShape>() };
        expect_ok(unsafe { ffi::kh_metadata_update(arrays, req_slots.as_ptr(), token_indices.as_ptr(), cu_tokens.as_ptr(),
                                                   req_slots.len() as u32, self.raw, &mut shape) },
                  "GQAMetadataBuffers::update");
        shape
    }
}

impl Drop for Selection {
    fn drop(&mut self) {
        unsafe { ffi::kh_selection_destroy(self.raw) };
    }
}
