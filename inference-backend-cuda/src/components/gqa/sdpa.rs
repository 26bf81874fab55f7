//! SDPA capability registry: `Config`, `MapKernelKind`, `ExecutionVariant`, `Registry`
//! (`inference-backend-metal/src/components/gqa/sdpa.rs:7-302`), answered by the library's host code so that
//! the variant tables of the two backends cannot drift. Not compiled here; see Cargo.toml.
use crate::error::expect_ok;
use crate::ffi;
use crate::metal::Dtype;

pub mod sliced_kv;
pub mod sliced_q;

#[derive(Clone, Copy, Debug, Eq, Hash, PartialEq)]
pub struct MapThreadBlockConstants {
    pub max_q_tokens: u32,
    pub max_q_heads: u32,
    pub kv_tokens_per_iteration: u32,
    pub required_threads: u32,
}

#[derive(Clone, Copy, Debug, Eq, Hash, PartialEq)]
pub struct KVCacheConstants {
    pub tokens_per_page: u32,
}

#[derive(Clone, Copy, Debug, Eq, Hash, PartialEq)]
pub enum MapKernelKind {
    SlicedKv,
    QTokensPerHead,
    QHeadsPerToken,
    QTokensAndHeads,
}

impl MapKernelKind {
    fn to_ffi(self) -> u32 {
        match self {
            MapKernelKind::SlicedKv => ffi::KH_MAP_SLICED_KV,
            MapKernelKind::QTokensPerHead => ffi::KH_MAP_Q_TOKENS_PER_HEAD,
            MapKernelKind::QHeadsPerToken => ffi::KH_MAP_Q_HEADS_PER_TOKEN,
            MapKernelKind::QTokensAndHeads => ffi::KH_MAP_Q_TOKENS_AND_HEADS,
        }
    }

    fn from_ffi(kind: u32) -> Self {
        match kind {
            ffi::KH_MAP_SLICED_KV => MapKernelKind::SlicedKv,
            ffi::KH_MAP_Q_TOKENS_PER_HEAD => MapKernelKind::QTokensPerHead,
            ffi::KH_MAP_Q_HEADS_PER_TOKEN => MapKernelKind::QHeadsPerToken,
            ffi::KH_MAP_Q_TOKENS_AND_HEADS => MapKernelKind::QTokensAndHeads,
            other => panic!("unknown map kernel kind {other}"),
        }
    }
}

#[derive(Clone, Copy, Debug, Eq, Hash, PartialEq)]
pub struct MapKernelConstants {
    pub kind: MapKernelKind,
    pub thread_block: MapThreadBlockConstants,
    pub kv_cache: KVCacheConstants,
}

#[derive(Clone, Copy, Debug, Eq, Hash, PartialEq)]
pub struct ReduceThreadBlockConstants {
    pub max_q_tokens: u32,
    pub max_q_heads: u32,
    pub required_threads: u32,
}

#[derive(Clone, Copy, Debug, Eq, Hash, PartialEq)]
pub struct ReduceKernelConstants {
    pub thread_block: ReduceThreadBlockConstants,
}

/// One legal pairing of a Map and a Reduce kernel shape. On this backend `required_threads` and
/// `kv_tokens_per_iteration` keep their meaning for the selector and the partial ABI; the CUDA kernels choose
/// their own block shapes from `max_q_tokens * max_q_heads` (rows per task).
#[derive(Clone, Copy, Debug, Eq, Hash, PartialEq)]
pub struct ExecutionVariant {
    pub map: MapKernelConstants,
    pub reduce: ReduceKernelConstants,
}

impl ExecutionVariant {
    pub fn sliced_kv(config: Config, kv_tokens_per_iteration: u32, required_threads: u32, max_q_heads: u32) -> Self {
        let mut out = empty_variant();
        expect_ok(unsafe { ffi::kh_variant_sliced_kv(&config.to_ffi(), kv_tokens_per_iteration, required_threads,
                                                     max_q_heads, &mut out) },
                  "ExecutionVariant::sliced_kv");
        Self::from_ffi(out)
    }

    pub fn sliced_q(config: Config, kind: MapKernelKind, max_q_tokens: u32, kv_tokens_per_iteration: u32,
                    max_q_heads: u32) -> Self {
        let mut out = empty_variant();
        expect_ok(unsafe { ffi::kh_variant_sliced_q(&config.to_ffi(), kind.to_ffi(), max_q_tokens,
                                                    kv_tokens_per_iteration, max_q_heads, &mut out) },
                  "ExecutionVariant::sliced_q");
        Self::from_ffi(out)
    }

    pub fn supports(self, config: Config) -> bool {
        let mut out = 0i32;
        expect_ok(unsafe { ffi::kh_variant_supports(&self.to_ffi(), &config.to_ffi(), &mut out) },
                  "ExecutionVariant::supports");
        out != 0
    }

    pub fn to_ffi(self) -> ffi::KhExecutionVariant {
        ffi::KhExecutionVariant {
            kind: self.map.kind.to_ffi(),
            max_q_tokens: self.map.thread_block.max_q_tokens,
            max_q_heads: self.map.thread_block.max_q_heads,
            kv_tokens_per_iteration: self.map.thread_block.kv_tokens_per_iteration,
            required_threads: self.map.thread_block.required_threads,
            tokens_per_page: self.map.kv_cache.tokens_per_page,
            reduce_max_q_tokens: self.reduce.thread_block.max_q_tokens,
            reduce_max_q_heads: self.reduce.thread_block.max_q_heads,
            reduce_required_threads: self.reduce.thread_block.required_threads,
        }
    }

    pub fn from_ffi(raw: ffi::KhExecutionVariant) -> Self {
        Self {
            map: MapKernelConstants {
                kind: MapKernelKind::from_ffi(raw.kind),
                thread_block: MapThreadBlockConstants {
                    max_q_tokens: raw.max_q_tokens,
                    max_q_heads: raw.max_q_heads,
                    kv_tokens_per_iteration: raw.kv_tokens_per_iteration,
                    required_threads: raw.required_threads,
                },
                kv_cache: KVCacheConstants { tokens_per_page: raw.tokens_per_page },
            },
            reduce: ReduceKernelConstants {
                thread_block: ReduceThreadBlockConstants {
                    max_q_tokens: raw.reduce_max_q_tokens,
                    max_q_heads: raw.reduce_max_q_heads,
                    required_threads: raw.reduce_required_threads,
                },
            },
        }
    }
}

fn empty_variant() -> ffi::KhExecutionVariant {
    ffi::KhExecutionVariant {
        kind: 0, max_q_tokens: 0, max_q_heads: 0, kv_tokens_per_iteration: 0, required_threads: 0,
        tokens_per_page: 0, reduce_max_q_tokens: 0, reduce_max_q_heads: 0, reduce_required_threads: 0,
    }
}

/// Static GQA SDPA workload facts used for capability filtering (`sdpa.rs:219-241`). `io_dtype` may also be
/// `Dtype::Float16` here.
#[derive(Clone, Copy, Debug, Eq, PartialEq)]
pub struct Config {
    pub io_dtype: Dtype,
    pub num_q_heads: u32,
    pub num_kv_heads: u32,
    pub head_dim: u32,
    pub tokens_per_page: u32,
}

impl Config {
    pub fn validate(self) {
        expect_ok(unsafe { ffi::kh_sdpa_config_validate(&self.to_ffi()) }, "sdpa::Config::validate");
    }

    pub fn q_heads_per_kv_head(self) -> u32 {
        self.num_q_heads / self.num_kv_heads
    }

    pub fn to_ffi(self) -> ffi::KhSdpaConfig {
        ffi::KhSdpaConfig {
            io_dtype: self.io_dtype as u32,
            num_q_heads: self.num_q_heads,
            num_kv_heads: self.num_kv_heads,
            head_dim: self.head_dim,
            tokens_per_page: self.tokens_per_page,
        }
    }
}

/// Backend-owned registry of legal execution variants (`sdpa.rs:248-302`): static capability filtering only.
#[derive(Clone, Debug, Eq, PartialEq)]
pub struct Registry {
    config: Config,
    variants: Vec<ExecutionVariant>,
}

impl Registry {
    pub fn new(config: Config) -> Self {
        config.validate();
        let mut count = 0u32;
        expect_ok(unsafe { ffi::kh_registry_variants(&config.to_ffi(), std::ptr::null_mut(), 0, &mut count) },
                  "Registry::new");
        let mut raw = vec![empty_variant(); count as usize];
        expect_ok(unsafe { ffi::kh_registry_variants(&config.to_ffi(), raw.as_mut_ptr(), count, &mut count) },
                  "Registry::new");
        Self { config, variants: raw.into_iter().map(ExecutionVariant::from_ffi).collect() }
    }

    pub fn from_variants(config: Config, variants: Vec<ExecutionVariant>) -> Self {
        config.validate();
        for variant in &variants {
            assert!(variant.supports(config), "execution variant is not supported by the SDPA config");
        }
        Self { config, variants }
    }

    pub fn config(&self) -> Config {
        self.config
    }

    pub fn variants(&self) -> &[ExecutionVariant] {
        &self.variants
    }
}
