// Host-side SDPA planning: capability registry, replay buckets, selector, batch metadata.
// Mirrors the behaviour of the reference's
//   crates/inference-backend-metal/src/components/gqa/sdpa.rs        (Config, ExecutionVariant, Registry)
//   crates/inference-executor-core/src/replay.rs                     (ReplayBucketPolicy)
//   crates/inference-executor-metal/src/attn/gqa/sdpa.rs             (Selector, Selection)
//   crates/inference-executor-metal/src/attn/gqa/batch_metadata.rs   (GQAReplayShape, metadata arrays)
#pragma once

#include <cstdint>
#include <vector>

#include "common.h"

namespace kh {

void validate_config(const kh_sdpa_config& c);
inline uint32_t group_size(const kh_sdpa_config& c) { return c.num_q_heads / c.num_kv_heads; }

kh_execution_variant make_sliced_kv(const kh_sdpa_config& c, uint32_t kv_tokens_per_iteration,
                                    uint32_t required_threads, uint32_t max_q_heads);
kh_execution_variant make_sliced_q(const kh_sdpa_config& c, kh_map_kernel_kind kind, uint32_t max_q_tokens,
                                   uint32_t kv_tokens_per_iteration, uint32_t max_q_heads);
bool variant_supports(const kh_execution_variant& v, const kh_sdpa_config& c);
bool variant_equal(const kh_execution_variant& a, const kh_execution_variant& b);
std::vector<kh_execution_variant> registry_variants(const kh_sdpa_config& c);

// ReplayBucketPolicy (replay.rs:4-88) without topology boundaries.
class BucketPolicy {
public:
    explicit BucketPolicy(uint32_t max_capacity);
    uint32_t max_capacity() const { return max_; }
    const std::vector<uint32_t>& buckets() const { return buckets_; }
    uint32_t capacity(uint32_t active) const;

private:
    uint32_t max_;
    std::vector<uint32_t> buckets_;
};

kh_replay_shape make_replay_shape(uint32_t num_tokens, uint32_t num_total_tokens, uint32_t num_q_token_tiles,
                                  uint32_t num_total_q_token_tiles, uint32_t num_maps, uint32_t num_total_maps,
                                  bool reduce);

}  // namespace kh

// Opaque C handles.
struct kh_selection {
    kh_execution_variant variant;
    std::vector<kh_q_token_range> q_token_ranges;
    std::vector<kh_map_task_template> map_task_templates;
    std::vector<uint32_t> cu_partial_outputs;
    kh_replay_shape replay_shape;
    kh_selection_metrics metrics;
    bool direct_output() const { return variant.kind != KH_MAP_SLICED_KV && !replay_shape.reduce_sdpa_partial_outputs; }
};

struct kh_selector {
    kh_sdpa_config config;
    std::vector<kh_execution_variant> variants;
    kh_selector_limits limits;
    bool lookup = false;
    kh_selector_policy policy = KH_POLICY_REFERENCE;
    uint32_t sm_count = 148;
};
