// Host-side SDPA planning. See host_sdpa.h for the reference files each part mirrors.
#include "host_sdpa.h"

#include <algorithm>
#include <cstring>
#include <memory>
#include <cstdlib>
#include <queue>
#include <tuple>

namespace kh {

namespace {
thread_local std::string g_last_error;
}

kh_status fail(kh_status code, const char* format, ...) {
    char buffer[1024];
    va_list args;
    va_start(args, format);
    vsnprintf(buffer, sizeof(buffer), format, args);
    va_end(args);
    g_last_error = buffer;
    return code;
}

void clear_error() { g_last_error.clear(); }

void raise(kh_status code, const char* format, ...) {
    char buffer[1024];
    va_list args;
    va_start(args, format);
    vsnprintf(buffer, sizeof(buffer), format, args);
    va_end(args);
    throw Failure{code, buffer};
}

const std::string& last_error() { return g_last_error; }

// ---------------------------------------------------------------------------------------------
// sdpa::Config::validate (sdpa.rs:229-236). Float16 is accepted in addition to the reference's
// Float32 | Bfloat16 because this library adds an fp16 I/O path.
// ---------------------------------------------------------------------------------------------
void validate_config(const kh_sdpa_config& c) {
    KH_REQUIRE(c.io_dtype == KH_DTYPE_FLOAT32 || c.io_dtype == KH_DTYPE_BFLOAT16 || c.io_dtype == KH_DTYPE_FLOAT16,
               "GQA SDPA io dtype must be Float32, Bfloat16 or Float16");
    KH_REQUIRE(c.num_q_heads > 0, "GQA SDPA requires Q heads");
    KH_REQUIRE(c.num_kv_heads > 0, "GQA SDPA requires KV heads");
    KH_REQUIRE(c.num_q_heads % c.num_kv_heads == 0, "GQA Q heads must be a multiple of KV heads");
    KH_REQUIRE(c.head_dim > 0, "GQA SDPA requires a head dimension");
    KH_REQUIRE(c.tokens_per_page > 0, "GQA SDPA requires tokens per page");
}

bool variant_equal(const kh_execution_variant& a, const kh_execution_variant& b) {
    return std::memcmp(&a, &b, sizeof(a)) == 0;
}

static bool sliced_q_profile(uint32_t head_dim, uint32_t tokens_per_page) {
    return (head_dim == 128 && (tokens_per_page == 8 || tokens_per_page == 16)) ||
           (head_dim == 256 && (tokens_per_page == 8 || tokens_per_page == 16 || tokens_per_page == 32));
}

static bool is_pow2(uint32_t v) { return v != 0 && (v & (v - 1)) == 0; }

static bool sliced_q_groups(kh_map_kernel_kind kind, uint32_t max_q_tokens, uint32_t max_q_heads, uint64_t* groups) {
    uint64_t g = 0;
    switch (kind) {
        case KH_MAP_Q_TOKENS_PER_HEAD:
            g = uint64_t(div_ceil(max_q_tokens, 8)) * max_q_heads;
            break;
        case KH_MAP_Q_HEADS_PER_TOKEN:
            g = uint64_t(div_ceil(max_q_heads, 8)) * max_q_tokens;
            break;
        case KH_MAP_Q_TOKENS_AND_HEADS:
            g = div_ceil64(uint64_t(max_q_tokens) * max_q_heads, 8);
            break;
        default:
            return false;
    }
    if (g * 32 > 0xffffffffull) return false;
    *groups = g;
    return true;
}

// ExecutionVariant::supports (sdpa.rs:162-215).
bool variant_supports(const kh_execution_variant& v, const kh_sdpa_config& c) {
    if (v.tokens_per_page != c.tokens_per_page || v.max_q_tokens == 0 || v.max_q_heads == 0 ||
        v.max_q_heads > group_size(c) || v.kv_tokens_per_iteration == 0 || v.required_threads == 0 ||
        v.reduce_max_q_tokens == 0 || v.reduce_max_q_heads == 0 || v.reduce_required_threads == 0) {
        return false;
    }
    if (v.kind == KH_MAP_SLICED_KV) {
        const uint32_t coords = 256 / std::min<uint32_t>(c.head_dim, 256);
        const uint32_t want_heads = std::max<uint32_t>(std::min(c.num_q_heads, coords), 1);
        const uint32_t want_tokens = std::max<uint32_t>(coords / want_heads, 1);
        return v.max_q_tokens == 1 && v.max_q_heads <= 8 && v.kv_tokens_per_iteration <= 1024 &&
               is_pow2(v.required_threads) && v.required_threads >= 32 && v.required_threads <= 256 &&
               v.reduce_max_q_tokens == want_tokens && v.reduce_max_q_heads == want_heads &&
               v.reduce_required_threads == 256;
    }
    uint64_t groups = 0;
    if (!sliced_q_groups(v.kind, v.max_q_tokens, v.max_q_heads, &groups)) return false;
    const uint64_t threads = groups * 32;
    const uint32_t t = v.max_q_tokens;
    const uint32_t s = v.kv_tokens_per_iteration;
    // The reference accepts only Bfloat16 here; Float16 shares every kernel of this library.
    const bool io_ok = c.io_dtype == KH_DTYPE_BFLOAT16 || c.io_dtype == KH_DTYPE_FLOAT16;
    return io_ok && sliced_q_profile(c.head_dim, c.tokens_per_page) &&
           (t == 1 || t == 2 || t == 4 || t == 8 || t == 16 || t == 32) &&
           (s == 8 || s == 16 || s == 32 || s == 64 || s == 128) && v.required_threads == threads &&
           v.required_threads <= 1024 && v.reduce_max_q_tokens == v.max_q_tokens && v.reduce_max_q_heads == 1 &&
           v.reduce_required_threads == v.required_threads;
}

// ExecutionVariant::sliced_kv (sdpa.rs:60-88).
kh_execution_variant make_sliced_kv(const kh_sdpa_config& c, uint32_t kv_tokens_per_iteration,
                                    uint32_t required_threads, uint32_t max_q_heads) {
    validate_config(c);
    const uint32_t coords = 256 / std::min<uint32_t>(c.head_dim, 256);
    const uint32_t reduce_heads = std::max<uint32_t>(std::min(c.num_q_heads, coords), 1);
    const uint32_t reduce_tokens = std::max<uint32_t>(coords / reduce_heads, 1);
    kh_execution_variant v{};
    v.kind = KH_MAP_SLICED_KV;
    v.max_q_tokens = 1;
    v.max_q_heads = max_q_heads;
    v.kv_tokens_per_iteration = kv_tokens_per_iteration;
    v.required_threads = required_threads;
    v.tokens_per_page = c.tokens_per_page;
    v.reduce_max_q_tokens = reduce_tokens;
    v.reduce_max_q_heads = reduce_heads;
    v.reduce_required_threads = 256;
    KH_REQUIRE(variant_supports(v, c), "GQA SlicedKv execution variant is not supported by its config");
    return v;
}

// ExecutionVariant::sliced_q (sdpa.rs:105-160).
kh_execution_variant make_sliced_q(const kh_sdpa_config& c, kh_map_kernel_kind kind, uint32_t max_q_tokens,
                                   uint32_t kv_tokens_per_iteration, uint32_t max_q_heads) {
    validate_config(c);
    KH_REQUIRE(max_q_tokens == 1 || max_q_tokens == 2 || max_q_tokens == 4 || max_q_tokens == 8 ||
                   max_q_tokens == 16 || max_q_tokens == 32,
               "GQA sliced-Q tile must hold 1, 2, 4, 8, 16 or 32 Q tokens");
    KH_REQUIRE(max_q_heads > 0 && max_q_heads <= group_size(c), "GQA sliced-Q head tile must fit one KV group");
    KH_REQUIRE(kind != KH_MAP_SLICED_KV, "SlicedKv uses its own constructor");
    uint64_t groups = 0;
    KH_REQUIRE(sliced_q_groups(kind, max_q_tokens, max_q_heads, &groups), "GQA tile geometry must fit u32");
    kh_execution_variant v{};
    v.kind = kind;
    v.max_q_tokens = max_q_tokens;
    v.max_q_heads = max_q_heads;
    v.kv_tokens_per_iteration = kv_tokens_per_iteration;
    v.required_threads = static_cast<uint32_t>(groups * 32);
    v.tokens_per_page = c.tokens_per_page;
    v.reduce_max_q_tokens = max_q_tokens;
    v.reduce_max_q_heads = 1;
    v.reduce_required_threads = v.required_threads;
    KH_REQUIRE(variant_supports(v, c), "GQA sliced-Q execution variant is not supported by its config");
    return v;
}

// Registry::new (sdpa.rs:255-271) with its helper constructors (sdpa.rs:304-330).
std::vector<kh_execution_variant> registry_variants(const kh_sdpa_config& c) {
    validate_config(c);
    const uint32_t ratio = group_size(c);
    std::vector<kh_execution_variant> out;
    {
        uint32_t kv_tokens = next_pow2(std::min<uint32_t>(std::max<uint32_t>(c.head_dim, 32), 256));
        out.push_back(make_sliced_kv(c, kv_tokens, std::min<uint32_t>(kv_tokens, 128), std::min<uint32_t>(ratio, 8)));
    }
    const bool sliced_q_ok = c.io_dtype == KH_DTYPE_BFLOAT16 && sliced_q_profile(c.head_dim, c.tokens_per_page) && ratio <= 8;
    if (sliced_q_ok) {
        const uint32_t max_heads = 256 / (8 / 8 * 32);  // eight-token tile: one SIMD group per head
        const uint32_t full = std::min(ratio, max_heads);
        const bool d128 = c.head_dim == 128 && (c.tokens_per_page == 8 || c.tokens_per_page == 16);
        if (!d128) {
            const uint32_t half = std::min(div_ceil(ratio, 2), max_heads);
            if (half != full) out.push_back(make_sliced_q(c, KH_MAP_Q_TOKENS_PER_HEAD, 8, 16, half));
        }
        out.push_back(make_sliced_q(c, KH_MAP_Q_TOKENS_PER_HEAD, 8, 16, full));
        if (c.head_dim == 256) out.push_back(make_sliced_q(c, KH_MAP_Q_TOKENS_PER_HEAD, 8, 32, full));
    }
    return out;
}

// ---------------------------------------------------------------------------------------------
// ReplayBucketPolicy (replay.rs:1-88): 1,2,4,6,8,12,16,20,24,32,40,48,56,64, then four equal steps
// per doubling, and the terminal capacity itself.
// ---------------------------------------------------------------------------------------------
BucketPolicy::BucketPolicy(uint32_t max_capacity) : max_(max_capacity) {
    KH_REQUIRE(max_capacity > 0, "replay bucket capacity must be positive");
    static const uint32_t base[] = {1, 2, 4, 6, 8, 12, 16, 20, 24, 32, 40, 48, 56, 64};
    for (uint32_t b : base) {
        if (b > max_capacity) break;
        buckets_.push_back(b);
    }
    uint64_t lower = 64;
    bool done = false;
    while (!done && lower < max_capacity) {
        const uint64_t step = lower / 4;
        for (uint64_t part = 1; part <= 4; ++part) {
            const uint64_t candidate = std::min<uint64_t>(lower + step * part, 0xffffffffull);
            if (candidate >= max_capacity) {
                done = true;
                break;
            }
            buckets_.push_back(static_cast<uint32_t>(candidate));
        }
        lower = std::min<uint64_t>(lower * 2, 0xffffffffull);
    }
    buckets_.push_back(max_capacity);
    std::sort(buckets_.begin(), buckets_.end());
    buckets_.erase(std::unique(buckets_.begin(), buckets_.end()), buckets_.end());
}

uint32_t BucketPolicy::capacity(uint32_t active) const {
    KH_REQUIRE(active > 0, "replay bucket requires active work");
    KH_REQUIRE(active <= max_, "replay active work exceeds capacity");
    return *std::lower_bound(buckets_.begin(), buckets_.end(), active);
}

// GQAReplayShape::new + validate (batch_metadata.rs:29-61).
kh_replay_shape make_replay_shape(uint32_t num_tokens, uint32_t num_total_tokens, uint32_t num_q_token_tiles,
                                  uint32_t num_total_q_token_tiles, uint32_t num_maps, uint32_t num_total_maps,
                                  bool reduce) {
    KH_REQUIRE(num_tokens > 0, "GQA replay shape requires tokens");
    KH_REQUIRE(num_tokens <= num_total_tokens, "GQA replay shape tokens exceed their capacity");
    KH_REQUIRE(num_q_token_tiles > 0 && num_q_token_tiles <= num_tokens, "GQA replay shape Q tiles out of range");
    KH_REQUIRE(num_q_token_tiles <= num_total_q_token_tiles, "GQA replay shape Q tiles exceed their capacity");
    KH_REQUIRE(num_maps >= num_q_token_tiles, "GQA replay shape needs a Map per Q tile");
    KH_REQUIRE(num_maps <= num_total_maps, "GQA replay shape Maps exceed their capacity");
    kh_replay_shape s{};
    s.num_tokens = num_tokens;
    s.num_total_tokens = num_total_tokens;
    s.num_q_token_tiles = num_q_token_tiles;
    s.num_total_q_token_tiles = num_total_q_token_tiles;
    s.num_sdpa_map_task_templates = num_maps;
    s.num_total_sdpa_map_task_templates = num_total_maps;
    s.reduce_sdpa_partial_outputs = reduce ? 1u : 0u;
    return s;
}

// ---------------------------------------------------------------------------------------------
// Selector (EM/attn/gqa/sdpa.rs)
// ---------------------------------------------------------------------------------------------
namespace {

struct RangeWork {
    kh_q_token_range range;
    uint32_t num_kv_iterations;
    uint32_t num_kv_splits;
};

// build_q_token_ranges (sdpa.rs:780-819).
std::vector<RangeWork> build_ranges(const kh_request_shape* requests, uint32_t num_requests, uint32_t max_q_tokens,
                                    uint32_t kv_tokens_per_iteration) {
    std::vector<RangeWork> ranges;
    uint32_t request_begin = 0;
    for (uint32_t r = 0; r < num_requests; ++r) {
        const uint32_t request_end = to_u32(uint64_t(request_begin) + requests[r].num_q_tokens, "GQA flat Q-token end");
        uint32_t begin = request_begin;
        while (begin < request_end) {
            const uint32_t end = static_cast<uint32_t>(std::min<uint64_t>(uint64_t(begin) + max_q_tokens, request_end));
            const uint32_t visible =
                to_u32(uint64_t(requests[r].num_history_tokens) + (end - request_begin), "GQA visible KV-token count");
            const uint32_t iterations = div_ceil(visible, kv_tokens_per_iteration);
            KH_REQUIRE(iterations <= 0xffffffffu / kv_tokens_per_iteration, "GQA padded KV-token range must fit u32");
            ranges.push_back(RangeWork{{r, begin, end, visible}, iterations, 1});
            begin = end;
        }
        request_begin = request_end;
    }
    KH_REQUIRE(!ranges.empty(), "GQA SDPA selector requires Q-token ranges");
    return ranges;
}

// allocate_kv_splits (sdpa.rs:821-850): hand one more split at a time to the range whose splits
// carry the most KV iterations; earlier ranges win ties.
void allocate_splits(std::vector<RangeWork>& ranges, uint32_t max_maps) {
    const size_t count = ranges.size();
    if (count == max_maps) return;
    if (count == 1) {
        ranges[0].num_kv_splits = std::min(ranges[0].num_kv_iterations, max_maps);
        return;
    }
    // (per-split work, -index): std::priority_queue is a max-heap, so the smaller index wins ties.
    using Entry = std::pair<uint32_t, int64_t>;
    std::priority_queue<Entry> heap;
    for (size_t i = 0; i < count; ++i) {
        if (ranges[i].num_kv_splits < ranges[i].num_kv_iterations) {
            heap.push({div_ceil(ranges[i].num_kv_iterations, ranges[i].num_kv_splits), -int64_t(i)});
        }
    }
    for (size_t used = count; used < max_maps; ++used) {
        if (heap.empty()) break;
        const size_t index = size_t(-heap.top().second);
        heap.pop();
        RangeWork& range = ranges[index];
        range.num_kv_splits += 1;
        if (range.num_kv_splits < range.num_kv_iterations) {
            heap.push({div_ceil(range.num_kv_iterations, range.num_kv_splits), -int64_t(index)});
        }
    }
}

// Route table of the default lookup (sdpa.rs:667-675).
// Rows: D128/G<=8, D128/G>8, D256/G<=8, D256/G>8. Columns: query capacity 1,2,4,8,16,32.
// 0: D128 short query; 1: shared Q tokens/heads; 2: Q tokens per head; 3: single query.
const uint8_t kLookupStrategies[4][6] = {
    {3, 0, 1, 1, 1, 1},
    {3, 1, 1, 1, 1, 1},
    {3, 1, 1, 2, 2, 2},
    {3, 1, 1, 1, 1, 1},
};

uint8_t lookup_strategy(const kh_sdpa_config& c, uint32_t queries) {
    const uint32_t ratio = group_size(c);
    return kLookupStrategies[(c.head_dim == 256 ? 2 : 0) + (ratio > 8 ? 1 : 0)][ilog2(queries)];
}

// lookup_variant (sdpa.rs:677-713).
kh_execution_variant lookup_variant(const kh_sdpa_config& c, uint32_t queries, uint32_t end, bool enough_decode_grid) {
    const uint32_t ratio = group_size(c);
    const uint8_t strategy = lookup_strategy(c, queries);
    kh_map_kernel_kind kind;
    uint32_t tile, stage;
    if (end <= 32 || (queries > 1 && end <= 512)) {
        kind = KH_MAP_Q_TOKENS_AND_HEADS;
        tile = std::min<uint32_t>(queries, 1u << ilog2(32 / ratio));
        stage = 16;
    } else if (strategy == 0 && end <= 4096) {
        kind = KH_MAP_Q_HEADS_PER_TOKEN;
        tile = queries;
        stage = 16;
    } else if (strategy == 1) {
        stage = c.head_dim == 128 ? 64 : 16;
        tile = std::min<uint32_t>(queries, 1u << ilog2(16384 / c.head_dim / ratio));
        const uint32_t joint = div_ceil(tile * ratio, 8);
        const uint32_t head = tile * div_ceil(ratio, 8);
        kind = (head > joint && div_ceil(stage, joint) > 16) ? KH_MAP_Q_HEADS_PER_TOKEN : KH_MAP_Q_TOKENS_AND_HEADS;
    } else if (strategy == 2) {
        kind = KH_MAP_Q_TOKENS_PER_HEAD;
        tile = 8;
        stage = 16;
    } else if (strategy == 3 && c.head_dim == 256 && ratio > 8 && enough_decode_grid) {
        kind = KH_MAP_Q_TOKENS_AND_HEADS;
        tile = 1;
        stage = 16;
    } else {
        return make_sliced_kv(c, c.head_dim, 128, std::min<uint32_t>(ratio, 8));
    }
    return make_sliced_q(c, kind, tile, stage, ratio);
}

// lookup_decode_slice (sdpa.rs:715-718); `target` is 1280 SIMD groups in the reference.
uint32_t decode_slice(uint32_t end, unsigned __int128 work, uint32_t min_slice, uint32_t max_slice,
                      unsigned __int128 target) {
    unsigned __int128 quotient = work / target;
    if (quotient < 1) quotient = 1;
    uint32_t log = 0;
    while ((quotient >> (log + 1)) != 0) ++log;
    unsigned __int128 slice = (unsigned __int128)1 << log;
    if (slice < min_slice) slice = min_slice;
    if (slice > max_slice) slice = max_slice;
    if (slice > end) slice = end;
    return static_cast<uint32_t>(slice);
}

struct Route {
    kh_execution_variant variant;
    uint32_t slice;
    bool direct;
};

// lookup_route (sdpa.rs:720-778).
Route lookup_route_reference(const kh_sdpa_config& c, const kh_request_shape* requests, uint32_t num_requests) {
    uint32_t max_q = 0, end = 0;
    unsigned __int128 visible = 0;
    for (uint32_t r = 0; r < num_requests; ++r) {
        max_q = std::max(max_q, requests[r].num_q_tokens);
        const uint32_t ctx = requests[r].num_history_tokens + requests[r].num_q_tokens;
        end = std::max(end, ctx);
        visible += ctx;
    }
    const uint32_t queries = next_pow2(std::min<uint32_t>(max_q, 32));
    const uint32_t ratio = group_size(c);
    const uint32_t head_groups = c.num_kv_heads * div_ceil(ratio, 8);
    const uint32_t matrix_slice = decode_slice(end, visible * head_groups, 256, 512, 1280);
    unsigned __int128 matrix_grid = 0;
    for (uint32_t r = 0; r < num_requests; ++r) {
        matrix_grid += div_ceil(requests[r].num_history_tokens + requests[r].num_q_tokens, matrix_slice);
    }
    matrix_grid *= head_groups;
    const kh_execution_variant variant = lookup_variant(c, queries, end, matrix_grid >= 160);
    const uint8_t strategy = lookup_strategy(c, queries);
    const uint32_t groups = variant.required_threads / 32;
    uint32_t slice;
    if (end <= 32 || (queries > 1 && end <= 512)) {
        slice = end;
    } else if (strategy == 3) {
        const uint32_t max_slice = variant.kind == KH_MAP_SLICED_KV ? 1024 : 512;
        slice = decode_slice(end, visible * c.num_kv_heads * div_ceil(ratio, variant.max_q_heads) * groups, 256,
                             max_slice, 1280);
    } else {
        const unsigned __int128 feature =
            (unsigned __int128)end * end * num_requests * (unsigned __int128)groups * groups;
        if (feature <= ((unsigned __int128)1 << 26)) slice = 64;
        else if (feature <= ((unsigned __int128)1 << 30)) slice = 128;
        else if (feature <= ((unsigned __int128)1 << 34)) slice = 256;
        else slice = 512;
        slice = std::min(slice, end);
    }
    const bool direct = variant.kind != KH_MAP_SLICED_KV && slice == end;
    return Route{variant, slice, direct};
}

// The same routing question answered for a B200: one persistent CTA per SM pulls Map tasks
// (one task = one template x one KV head x one Q-head range), each CTA streams its tasks' pages
// through a deep shared-memory ring, and all Q heads of a KV group (and all Q tokens of a verify
// tile) ride in the rows of one tensor-core tile so that a K/V byte is read once. The only free
// choices are therefore the Q tile and the KV slice:
//  - Q tile: as many of the request's Q tokens as fit 128 rows together with the whole group.
//  - KV slice: a power of two such that every SM sees about `kTasksPerSm` tasks (balance across
//    148 SMs with static task striding), never below 256 tokens (sixteen 16-token pages keep the
//    ring busy; 64 for batches too small to give every SM a task) and never above 2048 (bounds the per-task
//    tail).
Route lookup_route_b200(const kh_sdpa_config& c, const kh_request_shape* requests, uint32_t num_requests,
                        uint32_t sm_count) {
    // measured: decode (one Q token per task) runs best with about 4 tasks per SM (2,048-token slices on the decode
    // bench and on 1M tokens); Q-tile tasks, fewer and costlier, balance better with about 8
    constexpr uint32_t kTasksPerSm = 8;
    uint32_t kDecodeTasksPerSm = 4;
    uint32_t min_slice = 256;
#ifdef KH_GQA_MEASURE
    // measurement build only: try other decode slice policies without rebuilding
    if (const char* v = std::getenv("KH_GQA_DECODE_TASKS_PER_SM")) kDecodeTasksPerSm = uint32_t(std::atoi(v));
    if (const char* v = std::getenv("KH_GQA_MIN_SLICE")) min_slice = uint32_t(std::atoi(v));
#endif
    uint32_t max_q = 0, end = 0;
    unsigned __int128 visible = 0;
    for (uint32_t r = 0; r < num_requests; ++r) {
        max_q = std::max(max_q, requests[r].num_q_tokens);
        const uint32_t ctx = requests[r].num_history_tokens + requests[r].num_q_tokens;
        end = std::max(end, ctx);
        visible += ctx;
    }
    const uint32_t queries = next_pow2(std::min<uint32_t>(max_q, 32));
    const uint32_t ratio = group_size(c);
    const bool tensor_profile = sliced_q_profile(c.head_dim, c.tokens_per_page) &&
                                (c.io_dtype == KH_DTYPE_BFLOAT16 || c.io_dtype == KH_DTYPE_FLOAT16) && ratio <= 32;
    kh_execution_variant variant;
    if (queries == 1 && (ratio <= 8 || !tensor_profile)) {
        variant = make_sliced_kv(c, c.head_dim, 128, std::min<uint32_t>(ratio, 8));
    } else {
        const uint32_t heads = ratio;
        uint32_t tile = std::min<uint32_t>(queries, 1u << ilog2(std::max<uint32_t>(128 / heads, 1)));
        variant = make_sliced_q(c, KH_MAP_Q_TOKENS_AND_HEADS, tile, 16, heads);
    }
    uint32_t slice;
    const bool sliced_q = variant.kind != KH_MAP_SLICED_KV;
    if (sliced_q && (end <= 32 || (queries > 1 && end <= 512))) {
        slice = end;
    } else {
        const uint32_t head_groups = c.num_kv_heads * div_ceil(ratio, variant.max_q_heads);
        unsigned __int128 work = 0;
        uint64_t tiles_total = 0;
        for (uint32_t r = 0; r < num_requests; ++r) {
            const uint32_t tiles = div_ceil(requests[r].num_q_tokens, variant.max_q_tokens);
            tiles_total += tiles;
            work += (unsigned __int128)tiles * (requests[r].num_history_tokens + requests[r].num_q_tokens);
        }
        if (sliced_q && tiles_total * head_groups >= uint64_t(sm_count) * kTasksPerSm) {
            // enough (Q tile, head group) tasks to fill every SM several times over without cutting the KV range:
            // one task per tile writes the output directly, no partials and no reduce (chunked prefill)
            slice = end;
        } else {
            slice = decode_slice(end, work * head_groups, min_slice, 2048,
                                 (unsigned __int128)sm_count * (sliced_q ? kTasksPerSm : kDecodeTasksPerSm));
            // A small batch cut at 256 tokens leaves most SMs without a task (four short decode requests with two
            // KV heads: 32 tasks on 148 SMs, and the batch sits in L2, so the step is pure latency). When the tasks
            // at this slice do not reach the SM count, aim at one task per SM and allow slices down to 64 tokens.
            uint64_t tasks = 0;
            for (uint32_t r = 0; r < num_requests; ++r) {
                const uint32_t ctx = requests[r].num_history_tokens + requests[r].num_q_tokens;
                tasks += uint64_t(div_ceil(requests[r].num_q_tokens, variant.max_q_tokens)) * div_ceil(ctx, slice);
            }
            if (tasks * head_groups < sm_count) {
                slice = decode_slice(end, work * head_groups, 64, 2048, (unsigned __int128)sm_count);
            }
        }
    }
    const bool direct = sliced_q && slice == end;
    return Route{variant, slice, direct};
}

void validate_policy(const kh_selector& s, uint32_t policy_max_tokens, uint32_t policy_max_maps) {
    KH_REQUIRE(policy_max_tokens == s.limits.max_tokens,
               "GQA replay bucket policy must match the SDPA token capacity");
    KH_REQUIRE(policy_max_maps == s.limits.max_map_task_templates,
               "GQA replay bucket policy must match the SDPA Map task-template capacity");
}

uint32_t validate_requests(const kh_selector& s, const kh_request_shape* requests, uint32_t num_requests,
                           uint32_t policy_max_tokens, uint32_t policy_max_maps, uint32_t num_total_tokens) {
    validate_policy(s, policy_max_tokens, policy_max_maps);
    KH_REQUIRE(num_requests > 0 && requests != nullptr, "GQA SDPA selector requires requests");
    uint64_t tokens = 0;
    for (uint32_t r = 0; r < num_requests; ++r) {
        KH_REQUIRE(requests[r].num_q_tokens > 0, "GQA requests must contain Q tokens");
        KH_REQUIRE(uint64_t(requests[r].num_history_tokens) + requests[r].num_q_tokens <= 0xffffffffull,
                   "GQA request context length must fit u32");
        tokens += requests[r].num_q_tokens;
    }
    KH_REQUIRE(tokens <= 0xffffffffull, "GQA SDPA token count must fit u32");
    KH_REQUIRE(tokens <= s.limits.max_tokens, "GQA SDPA token count exceeds the selector capacity");
    KH_REQUIRE(tokens <= num_total_tokens, "GQA active token count must not exceed the total token count");
    KH_REQUIRE(num_total_tokens <= policy_max_tokens, "GQA total token count must not exceed the metadata capacity");
    return static_cast<uint32_t>(tokens);
}

bool contains_variant(const kh_selector& s, const kh_execution_variant& v) {
    for (const auto& candidate : s.variants) {
        if (variant_equal(candidate, v)) return true;
    }
    return false;
}

// materialize_candidate (sdpa.rs:476-664).
kh_selection* materialize(const kh_selector& s, const kh_execution_variant& variant, const kh_request_shape* requests,
                          uint32_t num_requests, uint32_t policy_max_tokens, uint32_t policy_max_maps,
                          uint32_t num_total_tokens, bool has_slice, uint32_t kv_slice, bool direct_output) {
    const kh_selector_limits& limits = s.limits;
    std::vector<RangeWork> ranges =
        build_ranges(requests, num_requests, variant.max_q_tokens, variant.kv_tokens_per_iteration);
    if (has_slice) {
        uint64_t maps = 0;
        for (auto& range : ranges) {
            range.num_kv_splits = div_ceil(range.range.num_visible_kv_tokens, kv_slice);
            maps += range.num_kv_splits;
        }
        KH_REQUIRE(maps <= limits.max_map_task_templates, "GQA fixed slices exceed the Map task-template capacity");
    } else {
        uint32_t budget = limits.max_map_task_templates;
        if (variant.kind != KH_MAP_SLICED_KV && variant.kv_tokens_per_iteration == 32) {
            budget = static_cast<uint32_t>(std::min<uint64_t>(uint64_t(ranges.size()) * 2, limits.max_map_task_templates));
        }
        KH_REQUIRE(ranges.size() <= budget, "GQA Q-token ranges exceed the Map task-template capacity");
        allocate_splits(ranges, budget);
    }

    auto selection = std::make_unique<kh_selection>();
    selection->variant = variant;
    selection->cu_partial_outputs.push_back(0);
    uint32_t max_iterations_per_split = 0;
    for (size_t index = 0; index < ranges.size(); ++index) {
        const RangeWork& range = ranges[index];
        selection->q_token_ranges.push_back(range.range);
        for (uint32_t split = 0; split < range.num_kv_splits; ++split) {
            uint32_t begin, end;
            if (has_slice) {
                const uint64_t b = uint64_t(split) * kv_slice;
                begin = static_cast<uint32_t>(b);
                end = static_cast<uint32_t>(std::min<uint64_t>(b + kv_slice, range.range.num_visible_kv_tokens));
            } else {
                const uint64_t it_begin = uint64_t(range.num_kv_iterations) * split / range.num_kv_splits;
                const uint64_t it_end = uint64_t(range.num_kv_iterations) * (split + 1) / range.num_kv_splits;
                begin = static_cast<uint32_t>(it_begin) * variant.kv_tokens_per_iteration;
                end = std::min(range.range.num_visible_kv_tokens,
                               static_cast<uint32_t>(it_end) * variant.kv_tokens_per_iteration);
            }
            max_iterations_per_split =
                std::max(max_iterations_per_split, div_ceil(end - begin, variant.kv_tokens_per_iteration));
            selection->map_task_templates.push_back({to_u32(index, "GQA SDPA Q-token-range index"), begin, end});
        }
        selection->cu_partial_outputs.push_back(
            to_u32(selection->map_task_templates.size(), "GQA SDPA partial-output count"));
    }

    const uint32_t num_ranges = to_u32(selection->q_token_ranges.size(), "GQA SDPA Q-token-range count");
    const uint32_t num_maps = to_u32(selection->map_task_templates.size(), "GQA SDPA Map task-template count");
    KH_REQUIRE(num_maps <= limits.max_map_task_templates, "GQA Map task templates exceed their capacity");
    uint32_t num_tokens = 0;
    for (uint32_t r = 0; r < num_requests; ++r) num_tokens += requests[r].num_q_tokens;
    const BucketPolicy range_buckets(policy_max_tokens);
    const BucketPolicy map_buckets(policy_max_maps);
    const uint32_t total_ranges = range_buckets.capacity(num_ranges);
    uint32_t total_maps = map_buckets.capacity(num_maps);
    if (direct_output) {
        // One direct Map owns each Q range; both padded domains share one extent.
        total_maps = total_ranges;
        KH_REQUIRE(total_maps <= limits.max_map_task_templates, "GQA direct Maps exceed their capacity");
    }
    selection->replay_shape = make_replay_shape(
        num_tokens, num_total_tokens, num_ranges, total_ranges, num_maps, total_maps,
        !direct_output && (variant.kind != KH_MAP_SLICED_KV || num_maps > num_tokens));

    kh_selection_metrics m{};
    if (!direct_output) {
        for (const auto& range : ranges) {
            m.num_active_partial_state_groups +=
                uint64_t(range.range.flat_q_token_end - range.range.flat_q_token_begin) * range.num_kv_splits;
        }
        m.num_reserved_partial_state_groups = uint64_t(num_maps) * variant.max_q_tokens;
        m.num_replay_reserved_partial_state_groups = uint64_t(total_maps) * variant.max_q_tokens;
    }
    KH_REQUIRE(m.num_replay_reserved_partial_state_groups <= limits.partial_state_group_capacity,
               "GQA SDPA replay exceeds its partial-state-group capacity");
    for (const auto& t : selection->map_task_templates) {
        const kh_q_token_range& range = selection->q_token_ranges[t.q_token_range_index];
        const uint64_t staged =
            uint64_t(div_ceil(t.kv_token_end - t.kv_token_begin, variant.kv_tokens_per_iteration)) *
            variant.kv_tokens_per_iteration;
        m.num_scheduled_qk_token_pairs += staged * variant.max_q_tokens;
        m.num_active_qk_token_pairs += staged * (range.flat_q_token_end - range.flat_q_token_begin);
    }
    const uint32_t head_ranges = div_ceil(group_size(s.config), variant.max_q_heads);
    m.num_map_threadblocks_per_kv_head = uint64_t(num_maps) * head_ranges;
    m.num_map_simdgroup_waves_per_kv_head = m.num_map_threadblocks_per_kv_head * (variant.required_threads / 32);
    for (uint32_t r = 0; r < num_requests; ++r) {
        const uint64_t q = requests[r].num_q_tokens;
        m.num_logical_qk_token_pairs += q * (uint64_t(requests[r].num_history_tokens) + 1) + q * (q - 1) / 2;
    }
    m.num_active_partial_states = mul_u64(m.num_active_partial_state_groups, s.config.num_q_heads,
                                          "GQA active partial-state count");
    m.max_kv_iterations_per_split = max_iterations_per_split;
    selection->metrics = m;
    return selection.release();
}

uint64_t overhead_score(const kh_selection_metrics& m) {
    return m.num_map_threadblocks_per_kv_head + m.num_map_simdgroup_waves_per_kv_head +
           m.num_active_partial_state_groups + m.num_replay_reserved_partial_state_groups;
}

// prefer_d256_page16_sliced_q (sdpa.rs:852-869), D256_PAGE16_MIN_SELECTION_SCORE = 2048.
bool prefer_sliced_q_d256_p16(const kh_selection& sliced_kv, const kh_selection& sliced_q) {
    const uint64_t score = sliced_kv.metrics.num_logical_qk_token_pairs +
                           std::min(overhead_score(sliced_kv.metrics), overhead_score(sliced_q.metrics));
    const bool utilised =
        sliced_q.metrics.num_active_qk_token_pairs * 2 >= sliced_q.metrics.num_scheduled_qk_token_pairs;
    return utilised && score >= 2048;
}

kh_selector* new_selector(const kh_sdpa_config& config, std::vector<kh_execution_variant> variants,
                          uint64_t max_tokens, uint64_t max_maps, uint64_t partial_capacity) {
    KH_REQUIRE(max_tokens > 0, "GQA SDPA selector requires tokens");
    KH_REQUIRE(max_maps > 0, "GQA SDPA selector requires Map task templates");
    KH_REQUIRE(partial_capacity > 0, "GQA SDPA selector requires partial-state groups");
    KH_REQUIRE(!variants.empty(), "GQA SDPA registry requires an execution variant");
    for (const auto& v : variants) {
        KH_REQUIRE(variant_supports(v, config), "GQA SDPA registry contains an unsupported execution variant");
    }
    auto s = std::make_unique<kh_selector>();
    s->config = config;
    s->variants = std::move(variants);
    s->limits.max_tokens = to_u32(max_tokens, "GQA SDPA token capacity");
    s->limits.max_map_task_templates = to_u32(max_maps, "GQA SDPA Map task-template capacity");
    s->limits.partial_state_group_capacity = partial_capacity;
    return s.release();
}

uint32_t registry_max_q_tokens(const std::vector<kh_execution_variant>& variants) {
    uint32_t best = 0;
    for (const auto& v : variants) best = std::max(best, v.max_q_tokens);
    return best;
}

}  // namespace

}  // namespace kh

using namespace kh;

template <typename T>
static kh_status copy_out(const std::vector<T>& values, T* out, uint32_t capacity, uint32_t* count) {
    KH_REQUIRE(count != nullptr, "null argument");
    *count = static_cast<uint32_t>(values.size());
    for (uint32_t i = 0; out != nullptr && i < capacity && i < values.size(); ++i) out[i] = values[i];
    return KH_OK;
}

extern "C" {

size_t kh_last_error(char* buf, size_t len) {
    const std::string& message = kh::last_error();
    if (buf != nullptr && len > 0) {
        const size_t n = std::min(len - 1, message.size());
        std::memcpy(buf, message.data(), n);
        buf[n] = '\0';
    }
    return message.size();
}

kh_status kh_sdpa_config_validate(const kh_sdpa_config* config) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(config != nullptr, "config is null");
        validate_config(*config);
        return KH_OK;
    });
}

kh_status kh_variant_sliced_kv(const kh_sdpa_config* config, uint32_t kv_tokens_per_iteration,
                               uint32_t required_threads, uint32_t max_q_heads, kh_execution_variant* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(config && out, "null argument");
        *out = make_sliced_kv(*config, kv_tokens_per_iteration, required_threads, max_q_heads);
        return KH_OK;
    });
}

kh_status kh_variant_sliced_q(const kh_sdpa_config* config, kh_map_kernel_kind kind, uint32_t max_q_tokens,
                              uint32_t kv_tokens_per_iteration, uint32_t max_q_heads, kh_execution_variant* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(config && out, "null argument");
        *out = make_sliced_q(*config, kind, max_q_tokens, kv_tokens_per_iteration, max_q_heads);
        return KH_OK;
    });
}

kh_status kh_variant_supports(const kh_execution_variant* variant, const kh_sdpa_config* config, int32_t* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(variant && config && out, "null argument");
        *out = variant_supports(*variant, *config) ? 1 : 0;
        return KH_OK;
    });
}

kh_status kh_registry_variants(const kh_sdpa_config* config, kh_execution_variant* out, uint32_t capacity,
                               uint32_t* count) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(config && count, "null argument");
        const auto variants = registry_variants(*config);
        *count = static_cast<uint32_t>(variants.size());
        for (uint32_t i = 0; out != nullptr && i < capacity && i < variants.size(); ++i) out[i] = variants[i];
        return KH_OK;
    });
}

kh_status kh_replay_buckets(uint32_t max_capacity, uint32_t* out, uint32_t capacity, uint32_t* count) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(count != nullptr, "null argument");
        const BucketPolicy policy(max_capacity);
        *count = static_cast<uint32_t>(policy.buckets().size());
        for (uint32_t i = 0; out != nullptr && i < capacity && i < policy.buckets().size(); ++i) {
            out[i] = policy.buckets()[i];
        }
        return KH_OK;
    });
}

kh_status kh_replay_capacity(uint32_t max_capacity, uint32_t active, uint32_t* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(out != nullptr, "null argument");
        *out = BucketPolicy(max_capacity).capacity(active);
        return KH_OK;
    });
}

kh_status kh_selector_create(const kh_sdpa_config* config, const kh_execution_variant* variants,
                             uint32_t num_variants, uint32_t max_tokens, uint32_t max_map_task_templates,
                             uint64_t partial_state_group_capacity, kh_selector** out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(config && out, "null argument");
        validate_config(*config);
        std::vector<kh_execution_variant> list;
        if (num_variants == 0) {
            list = registry_variants(*config);
        } else {
            KH_REQUIRE(variants != nullptr, "variants is null");
            list.assign(variants, variants + num_variants);
        }
        *out = new_selector(*config, std::move(list), max_tokens, max_map_task_templates,
                            partial_state_group_capacity);
        return KH_OK;
    });
}

// Selector::for_lookup (sdpa.rs:210-276).
kh_status kh_selector_create_for_lookup(const kh_sdpa_config* config, uint32_t max_tokens,
                                        const kh_page_table_layout* layout, kh_selector** out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(config && layout && out, "null argument");
        const kh_sdpa_config& c = *config;
        validate_config(c);
        KH_REQUIRE(layout->num_req_slots > 0 && layout->num_blocks > 0 && layout->num_gqa_layers > 0 &&
                       layout->num_page_ids_per_block > 0,
                   "GQA page-table layout dimensions must be positive");
        KH_REQUIRE(max_tokens > 0, "GQA lookup requires tokens");
        // The reference's route table is written for BF16 (its only tensor-tile type); FP16 Q / output, which
        // this backend also takes, follows the same routes.
        const bool tile_type = c.io_dtype == KH_DTYPE_BFLOAT16 || c.io_dtype == KH_DTYPE_FLOAT16;
        if (!tile_type || !sliced_q_profile(c.head_dim, c.tokens_per_page) || group_size(c) > 32) {
            auto variants = registry_variants(c);
            const uint64_t partials = mul_u64(max_tokens, registry_max_q_tokens(variants),
                                              "GQA partial-state-group capacity");
            *out = new_selector(c, std::move(variants), max_tokens, max_tokens, partials);
            return KH_OK;
        }
        const uint32_t max_visible = mul_u32(mul_u32(layout->num_blocks, layout->num_page_ids_per_block,
                                                     "GQA page-table token capacity"),
                                             c.tokens_per_page, "GQA page-table token capacity");
        std::vector<kh_execution_variant> variants;
        const uint32_t query_limit = next_pow2(std::min<uint32_t>(max_tokens, 32));
        for (uint32_t queries : {1u, 2u, 4u, 8u, 16u, 32u}) {
            if (queries > query_limit) break;
            for (uint32_t end : {32u, 512u, 4096u, 8192u}) {
                for (bool enough : {false, true}) {
                    const kh_execution_variant v = lookup_variant(c, queries, end, enough);
                    bool seen = false;
                    for (const auto& have : variants) seen = seen || variant_equal(have, v);
                    if (!seen) variants.push_back(v);
                }
            }
        }
        uint32_t max_splits = 0;
        for (const auto& v : variants) {
            max_splits = std::max(max_splits, std::max(div_ceil(max_visible, 256), div_ceil(512, v.required_threads / 32)));
        }
        const uint32_t max_maps =
            std::max(max_tokens, mul_u32(layout->num_req_slots, max_splits, "GQA Map task-template capacity"));
        const uint64_t max_partials =
            mul_u64(max_maps, registry_max_q_tokens(variants), "GQA partial-state-group capacity");
        kh_selector* s = new_selector(c, std::move(variants), max_tokens, max_maps, max_partials);
        s->lookup = true;
        *out = s;
        return KH_OK;
    });
}

// Selector::for_partitions (sdpa.rs:170-207).
kh_status kh_selector_create_for_partitions(const kh_sdpa_config* config, const kh_execution_variant* variants,
                                            uint32_t num_variants, const uint32_t* max_kv_splits,
                                            uint32_t max_tokens, uint32_t max_requests, kh_selector** out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(config && variants && max_kv_splits && out && num_variants > 0, "null argument");
        KH_REQUIRE(max_tokens > 0, "GQA partition envelope requires tokens");
        KH_REQUIRE(max_requests > 0, "GQA partition envelope requires requests");
        const uint32_t requests = std::min(max_requests, max_tokens);
        std::vector<uint32_t> bounds(num_variants);
        uint32_t max_maps = 0;
        for (uint32_t i = 0; i < num_variants; ++i) {
            const uint32_t ranges = requests + (max_tokens - requests) / variants[i].max_q_tokens;
            KH_REQUIRE(max_kv_splits[i] > 0, "GQA partition envelope requires KV splits");
            bounds[i] = mul_u32(ranges, max_kv_splits[i], "GQA partition Map task-template count");
            max_maps = std::max(max_maps, bounds[i]);
        }
        const BucketPolicy buckets(max_maps);
        uint64_t capacity = 0;
        for (uint32_t i = 0; i < num_variants; ++i) {
            capacity = std::max(capacity, mul_u64(buckets.capacity(bounds[i]), variants[i].max_q_tokens,
                                                  "GQA partition partial-state-group capacity"));
        }
        validate_config(*config);
        *out = new_selector(*config, std::vector<kh_execution_variant>(variants, variants + num_variants), max_tokens,
                            max_maps, capacity);
        return KH_OK;
    });
}

kh_status kh_selector_destroy(kh_selector* selector) {
    delete selector;
    return KH_OK;
}

kh_status kh_selector_limits_get(const kh_selector* selector, kh_selector_limits* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(selector && out, "null argument");
        *out = selector->limits;
        return KH_OK;
    });
}

kh_status kh_selector_variants(const kh_selector* selector, kh_execution_variant* out, uint32_t capacity,
                               uint32_t* count) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(selector && count, "null argument");
        *count = static_cast<uint32_t>(selector->variants.size());
        for (uint32_t i = 0; out != nullptr && i < capacity && i < selector->variants.size(); ++i) {
            out[i] = selector->variants[i];
        }
        return KH_OK;
    });
}

kh_status kh_selector_set_policy(kh_selector* selector, kh_selector_policy policy, uint32_t sm_count) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(selector != nullptr, "null argument");
        KH_REQUIRE(policy == KH_POLICY_REFERENCE || policy == KH_POLICY_B200, "unknown selector policy");
        KH_REQUIRE(sm_count > 0, "selector policy requires an SM count");
        selector->policy = policy;
        selector->sm_count = sm_count;
        if (policy == KH_POLICY_B200 && selector->lookup) {
            // Make every variant the B200 route can return a member of the registry, so that
            // Selection::variant() always belongs to the selector that produced it.
            const kh_sdpa_config& c = selector->config;
            const uint32_t limit = next_pow2(std::min<uint32_t>(selector->limits.max_tokens, 32));
            uint32_t max_tile = registry_max_q_tokens(selector->variants);
            for (uint32_t queries = 1; queries <= limit; queries *= 2) {
                for (uint32_t end : {32u, 8192u}) {
                    kh_request_shape probe{end - std::min(end, queries), queries};
                    const Route route = lookup_route_b200(c, &probe, 1, sm_count);
                    if (!contains_variant(*selector, route.variant)) selector->variants.push_back(route.variant);
                    max_tile = std::max(max_tile, route.variant.max_q_tokens);
                }
            }
            selector->limits.partial_state_group_capacity =
                std::max(selector->limits.partial_state_group_capacity,
                         mul_u64(selector->limits.max_map_task_templates, max_tile,
                                 "GQA partial-state-group capacity"));
        }
        return KH_OK;
    });
}

// Selector::select (sdpa.rs:278-380).
kh_status kh_selector_select(const kh_selector* selector, const kh_request_shape* requests, uint32_t num_requests,
                             uint32_t policy_max_tokens, uint32_t policy_max_map_task_templates,
                             uint32_t num_total_tokens, kh_selection** out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(selector && out, "null argument");
        const kh_selector& s = *selector;
        const uint32_t num_tokens = validate_requests(s, requests, num_requests, policy_max_tokens,
                                                      policy_max_map_task_templates, num_total_tokens);
        const kh_sdpa_config& c = s.config;
        auto run = [&](const kh_execution_variant& v, bool has_slice, uint32_t slice, bool direct) {
            return materialize(s, v, requests, num_requests, policy_max_tokens, policy_max_map_task_templates,
                               num_total_tokens, has_slice, slice, direct);
        };
        if (s.lookup) {
            Route route = s.policy == KH_POLICY_B200 ? lookup_route_b200(c, requests, num_requests, s.sm_count)
                                                     : lookup_route_reference(c, requests, num_requests);
            if (!route.direct) {
                // sum ceil(visible / slice) <= ceil(sum_visible / slice) + ranges - 1: coarsen the
                // slice until the templates fit the initialised capacity (sdpa.rs:290-307).
                const uint64_t tile = route.variant.max_q_tokens;
                uint64_t num_ranges = 0, visible = 0;
                for (uint32_t r = 0; r < num_requests; ++r) {
                    const uint64_t queries = requests[r].num_q_tokens;
                    const uint64_t ranges = div_ceil64(queries, tile);
                    visible += ranges * requests[r].num_history_tokens + tile * ranges * (ranges - 1) / 2 + queries;
                    num_ranges += ranges;
                }
                KH_REQUIRE(num_ranges <= s.limits.max_map_task_templates,
                           "GQA Q-token ranges exceed the Map task-template capacity");
                const uint64_t budget = uint64_t(s.limits.max_map_task_templates) - num_ranges + 1;
                const uint64_t required = div_ceil64(visible, budget);
                route.slice = to_u32(std::max<uint64_t>(route.slice, required), "GQA KV slice");
            }
            *out = run(route.variant, true, route.slice, route.direct);
            return KH_OK;
        }
        const kh_execution_variant* sliced_kv = nullptr;
        const kh_execution_variant* first_sliced_q = nullptr;
        for (const auto& v : s.variants) {
            if (v.kind == KH_MAP_SLICED_KV && !sliced_kv) sliced_kv = &v;
            if (v.kind != KH_MAP_SLICED_KV && !first_sliced_q) first_sliced_q = &v;
        }
        if (!first_sliced_q) {
            *out = run(*sliced_kv, false, 0, false);
            return KH_OK;
        }
        if (!sliced_kv) {
            *out = run(*first_sliced_q, false, 0, false);
            return KH_OK;
        }
        // Q-range density rejects variants before KV split allocation (sdpa.rs:327-338).
        uint64_t num_ranges = 0;
        for (uint32_t r = 0; r < num_requests; ++r) {
            num_ranges += div_ceil(requests[r].num_q_tokens, first_sliced_q->max_q_tokens);
        }
        if (uint64_t(num_tokens) < 2 * num_ranges) {
            *out = run(*sliced_kv, false, 0, false);
            return KH_OK;
        }
        uint32_t full_heads = 0;
        for (const auto& v : s.variants) {
            if (v.kind != KH_MAP_SLICED_KV) full_heads = std::max(full_heads, v.max_q_heads);
        }
        const bool d128 = c.head_dim == 128 && (c.tokens_per_page == 8 || c.tokens_per_page == 16);
        const uint32_t desired_heads = (!d128 && uint64_t(num_tokens) < 4 * num_ranges)
                                           ? std::min(div_ceil(group_size(c), 2), full_heads)
                                           : full_heads;
        const uint32_t desired_kv =
            (c.head_dim == 256 && num_tokens >= 1024 && uint64_t(num_tokens) >= 4 * num_ranges) ? 32 : 16;
        // max_by_key over (kv_tokens_per_iteration == desired): the last maximal element wins.
        const kh_execution_variant* chosen = nullptr;
        bool chosen_key = false;
        for (const auto& v : s.variants) {
            if (v.kind == KH_MAP_SLICED_KV || v.max_q_heads != desired_heads) continue;
            const bool key = v.kv_tokens_per_iteration == desired_kv;
            if (!chosen || key >= chosen_key) {
                chosen = &v;
                chosen_key = key;
            }
        }
        if (!chosen) chosen = first_sliced_q;
        std::unique_ptr<kh_selection> q_selection(run(*chosen, false, 0, false));
        if (c.head_dim == 256 && c.tokens_per_page == 16) {
            std::unique_ptr<kh_selection> kv_selection(run(*sliced_kv, false, 0, false));
            if (!prefer_sliced_q_d256_p16(*kv_selection, *q_selection)) {
                *out = kv_selection.release();
                return KH_OK;
            }
        }
        *out = q_selection.release();
        return KH_OK;
    });
}

// Selector::select_partitioned (sdpa.rs:382-426).
kh_status kh_selector_select_partitioned(const kh_selector* selector, const kh_execution_variant* variant,
                                         uint32_t kv_slice, int32_t direct_output, const kh_request_shape* requests,
                                         uint32_t num_requests, uint32_t policy_max_tokens,
                                         uint32_t policy_max_map_task_templates, uint32_t num_total_tokens,
                                         kh_selection** out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(selector && variant && out, "null argument");
        validate_requests(*selector, requests, num_requests, policy_max_tokens, policy_max_map_task_templates,
                          num_total_tokens);
        KH_REQUIRE(contains_variant(*selector, *variant), "GQA route must belong to its initialized registry");
        KH_REQUIRE(kv_slice > 0, "GQA KV slice must contain tokens");
        uint32_t max_visible = 0;
        for (uint32_t r = 0; r < num_requests; ++r) {
            max_visible = std::max(max_visible, requests[r].num_history_tokens + requests[r].num_q_tokens);
        }
        if (direct_output) {
            KH_REQUIRE(variant->kind != KH_MAP_SLICED_KV, "GQA SlicedKv requires Map/Reduce output");
            KH_REQUIRE(kv_slice >= max_visible, "GQA direct output requires an unsplit KV range");
        }
        *out = materialize(*selector, *variant, requests, num_requests, policy_max_tokens,
                           policy_max_map_task_templates, num_total_tokens, true, kv_slice, direct_output != 0);
        return KH_OK;
    });
}

kh_status kh_selection_destroy(kh_selection* selection) {
    delete selection;
    return KH_OK;
}

kh_status kh_selection_variant(const kh_selection* selection, kh_execution_variant* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(selection && out, "null argument");
        *out = selection->variant;
        return KH_OK;
    });
}

kh_status kh_selection_direct_output(const kh_selection* selection, int32_t* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(selection && out, "null argument");
        *out = selection->direct_output() ? 1 : 0;
        return KH_OK;
    });
}

kh_status kh_selection_replay_shape(const kh_selection* selection, kh_replay_shape* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(selection && out, "null argument");
        *out = selection->replay_shape;
        return KH_OK;
    });
}

kh_status kh_selection_metrics_get(const kh_selection* selection, kh_selection_metrics* out) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(selection && out, "null argument");
        *out = selection->metrics;
        return KH_OK;
    });
}

kh_status kh_selection_q_token_ranges(const kh_selection* selection, kh_q_token_range* out, uint32_t capacity,
                                      uint32_t* count) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(selection != nullptr, "null argument");
        return copy_out(selection->q_token_ranges, out, capacity, count);
    });
}

kh_status kh_selection_map_task_templates(const kh_selection* selection, kh_map_task_template* out,
                                          uint32_t capacity, uint32_t* count) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(selection != nullptr, "null argument");
        return copy_out(selection->map_task_templates, out, capacity, count);
    });
}

kh_status kh_selection_cu_partial_outputs(const kh_selection* selection, uint32_t* out, uint32_t capacity,
                                          uint32_t* count) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(selection != nullptr, "null argument");
        return copy_out(selection->cu_partial_outputs, out, capacity, count);
    });
}

// GQAMetadataBuffers::update (batch_metadata.rs:171-253).
kh_status kh_metadata_update(const kh_metadata_arrays* arrays, const uint32_t* req_slots,
                             const uint32_t* token_indices, const uint32_t* cu_tokens, uint32_t num_requests,
                             const kh_selection* selection, kh_replay_shape* out_shape) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(arrays && req_slots && token_indices && cu_tokens && selection, "null argument");
        KH_REQUIRE(arrays->req_slots && arrays->flat_token_indices && arrays->visible_kv_token_ranges &&
                       arrays->q_token_ranges && arrays->sdpa_map_task_templates && arrays->cu_sdpa_partial_outputs,
                   "metadata array is null");
        KH_REQUIRE(cu_tokens[0] == 0, "GQA batch cu_tokens must start at zero");
        const kh_replay_shape& shape = selection->replay_shape;
        KH_REQUIRE(cu_tokens[num_requests] == shape.num_tokens, "GQA batch token count must match its selection");
        KH_REQUIRE(shape.num_total_tokens <= arrays->max_tokens, "GQA total tokens exceed the metadata capacity");
        KH_REQUIRE(shape.num_total_q_token_tiles <= arrays->max_tokens,
                   "GQA total Q tiles exceed the metadata capacity");
        KH_REQUIRE(shape.num_total_sdpa_map_task_templates <= arrays->max_map_task_templates,
                   "GQA total Map task templates exceed the metadata capacity");
        uint32_t flat = 0;
        for (uint32_t r = 0; r < num_requests; ++r) {
            KH_REQUIRE(cu_tokens[r] <= cu_tokens[r + 1], "GQA batch cu_tokens must be nondecreasing");
            const uint32_t count = cu_tokens[r + 1] - cu_tokens[r];
            KH_REQUIRE(uint64_t(token_indices[r]) + count <= 0xffffffffull, "GQA request context length must fit u32");
            for (uint32_t i = 0; i < count; ++i, ++flat) {
                const uint32_t position = token_indices[r] + i;
                arrays->req_slots[flat] = req_slots[r];
                arrays->flat_token_indices[flat] = position;
                arrays->visible_kv_token_ranges[2 * flat] = 0;
                arrays->visible_kv_token_ranges[2 * flat + 1] = position + 1;
            }
        }
        KH_REQUIRE(flat == shape.num_tokens, "GQA batch token count must match its selection");
        KH_REQUIRE(selection->q_token_ranges.size() == shape.num_q_token_tiles, "GQA selection Q tiles mismatch");
        if (selection->variant.kind != KH_MAP_SLICED_KV) {
            for (size_t i = 0; i < selection->q_token_ranges.size(); ++i) {
                arrays->q_token_ranges[2 * i] = selection->q_token_ranges[i].flat_q_token_begin;
                arrays->q_token_ranges[2 * i + 1] = selection->q_token_ranges[i].flat_q_token_end;
            }
        }
        KH_REQUIRE(selection->map_task_templates.size() == shape.num_sdpa_map_task_templates,
                   "GQA selection Map templates mismatch");
        for (size_t i = 0; i < selection->map_task_templates.size(); ++i) {
            arrays->sdpa_map_task_templates[3 * i] = selection->map_task_templates[i].q_token_range_index;
            arrays->sdpa_map_task_templates[3 * i + 1] = selection->map_task_templates[i].kv_token_begin;
            arrays->sdpa_map_task_templates[3 * i + 2] = selection->map_task_templates[i].kv_token_end;
        }
        for (size_t i = selection->map_task_templates.size() * 3;
             i < size_t(shape.num_total_sdpa_map_task_templates) * 3; ++i) {
            arrays->sdpa_map_task_templates[i] = 0xffffffffu;
        }
        KH_REQUIRE(selection->cu_partial_outputs.size() == size_t(shape.num_q_token_tiles) + 1,
                   "GQA selection cumulative partial-output count mismatch");
        for (size_t i = 0; i < selection->cu_partial_outputs.size(); ++i) {
            arrays->cu_sdpa_partial_outputs[i] = selection->cu_partial_outputs[i];
        }
        if (out_shape) *out_shape = shape;
        return KH_OK;
    });
}

// build_metal_metadata + allocate_history_kv_splits of the BiDi-block GQA owner
// (crates/inference-executor-metal/src/attn/bidi_block_gqa/metadata.rs:176-367).
kh_status kh_bidi_block_metadata_build(const kh_metadata_arrays* arrays, const uint32_t* req_slots,
                                       const uint32_t* token_positions, const uint32_t* history_begins,
                                       const uint32_t* history_ends, uint32_t num_requests, uint32_t block_size,
                                       uint32_t max_q_tokens, uint32_t kv_tokens_per_iteration,
                                       uint32_t max_sdpa_map_task_templates, kh_replay_shape* out_shape) {
    return guarded([&]() -> kh_status {
        KH_REQUIRE(arrays && history_begins && history_ends, "null argument");
        KH_REQUIRE(arrays->visible_kv_token_ranges && arrays->q_token_ranges && arrays->sdpa_map_task_templates &&
                       arrays->cu_sdpa_partial_outputs,
                   "metadata array is null");
        KH_REQUIRE(num_requests > 0 && block_size > 0, "BiDiBlockGQA needs requests and a block size");
        KH_REQUIRE(kv_tokens_per_iteration > 0, "BiDiBlockGQA KV-token iteration size must be positive");
        KH_REQUIRE(max_q_tokens > 0, "BiDiBlockGQA Q-token range must contain tokens");
        const uint64_t num_tokens64 = uint64_t(num_requests) * block_size;
        KH_REQUIRE(num_tokens64 <= arrays->max_tokens, "BiDiBlockGQA tokens exceed the metadata capacity");
        const uint32_t num_tokens = uint32_t(num_tokens64);
        KH_REQUIRE(max_sdpa_map_task_templates <= arrays->max_map_task_templates,
                   "BiDiBlockGQA TaskTemplate capacity exceeds the metadata capacity");
        KH_REQUIRE((max_sdpa_map_task_templates & (max_sdpa_map_task_templates - 1)) == 0 &&
                       max_sdpa_map_task_templates > 0,
                   "BiDiBlockGQA TaskTemplate capacity must be a power of two");
        for (uint32_t t = 0; t < num_tokens; ++t) {
            arrays->visible_kv_token_ranges[2 * t] = history_begins[t];
            arrays->visible_kv_token_ranges[2 * t + 1] = history_ends[t];
            if (req_slots != nullptr && arrays->req_slots != nullptr) arrays->req_slots[t] = req_slots[t / block_size];
            if (token_positions != nullptr && arrays->flat_token_indices != nullptr) {
                arrays->flat_token_indices[t] = token_positions[t];
            }
        }
        // Q-token ranges: runs of at most max_q_tokens tokens inside one request block
        std::vector<std::pair<uint32_t, uint32_t>> ranges;
        for (uint32_t r = 0; r < num_requests; ++r) {
            const uint32_t request_end = (r + 1) * block_size;
            for (uint32_t begin = r * block_size; begin < request_end;) {
                const uint32_t end = std::min(begin + max_q_tokens, request_end);
                ranges.emplace_back(begin, end);
                begin = end;
            }
        }
        KH_REQUIRE(uint64_t(max_sdpa_map_task_templates) >= uint64_t(ranges.size()) * 2,
                   "BiDiBlockGQA needs at least two TaskTemplates per Q-token range");
        // union of the history ranges of a Q-token range, and its KV iterations
        std::vector<std::pair<uint32_t, uint32_t>> history(ranges.size());
        std::vector<uint64_t> iterations(ranges.size());
        for (size_t i = 0; i < ranges.size(); ++i) {
            uint32_t begin = 0xffffffffu, end = 0;
            for (uint32_t t = ranges[i].first; t < ranges[i].second; ++t) {
                begin = std::min(begin, history_begins[t]);
                end = std::max(end, history_ends[t]);
            }
            KH_REQUIRE(begin < end, "BiDiBlockGQA history range must not be empty");
            history[i] = {begin, end};
            iterations[i] = div_ceil64(end - begin, kv_tokens_per_iteration);
            KH_REQUIRE(iterations[i] <= (0xffffffffull - begin) / kv_tokens_per_iteration,
                       "BiDiBlockGQA padded history-token range must fit u32");
        }
        // allocate_history_kv_splits: one split each, then the remaining templates go, one at a time, to the range
        // with the most iterations per split (later ranges win ties)
        const uint64_t budget = max_sdpa_map_task_templates - ranges.size();
        std::vector<uint64_t> splits(ranges.size(), 1);
        if (ranges.size() == 1) {
            splits[0] = std::min<uint64_t>(iterations[0], budget);
        } else if (ranges.size() < budget) {
            std::priority_queue<std::pair<uint64_t, size_t>> candidates;
            for (size_t i = 0; i < ranges.size(); ++i) {
                if (iterations[i] > 1) candidates.emplace(iterations[i], i);
            }
            for (uint64_t used = ranges.size(); used < budget && !candidates.empty(); ++used) {
                const size_t index = candidates.top().second;
                candidates.pop();
                splits[index] += 1;
                if (splits[index] < iterations[index]) {
                    candidates.emplace(div_ceil64(iterations[index], splits[index]), index);
                }
            }
        }
        uint32_t templates = 0;
        arrays->cu_sdpa_partial_outputs[0] = 0;
        for (size_t i = 0; i < ranges.size(); ++i) {
            arrays->q_token_ranges[2 * i] = ranges[i].first;
            arrays->q_token_ranges[2 * i + 1] = ranges[i].second;
            for (uint64_t k = 0; k < splits[i]; ++k) {
                const uint64_t first = iterations[i] * k / splits[i], last = iterations[i] * (k + 1) / splits[i];
                const uint32_t kv_begin = history[i].first + uint32_t(first) * kv_tokens_per_iteration;
                const uint32_t kv_end =
                    std::min<uint64_t>(history[i].second, uint64_t(history[i].first) + last * kv_tokens_per_iteration);
                KH_REQUIRE(templates < max_sdpa_map_task_templates, "BiDiBlockGQA replay TaskTemplate count exceeds capacity");
                arrays->sdpa_map_task_templates[3 * templates] = uint32_t(i);
                arrays->sdpa_map_task_templates[3 * templates + 1] = kv_begin;
                arrays->sdpa_map_task_templates[3 * templates + 2] = kv_end;
                ++templates;
            }
            // the padded template whose index is the block partial's slot
            KH_REQUIRE(templates < max_sdpa_map_task_templates, "BiDiBlockGQA replay TaskTemplate count exceeds capacity");
            for (int f = 0; f < 3; ++f) arrays->sdpa_map_task_templates[3 * templates + f] = 0xffffffffu;
            ++templates;
            arrays->cu_sdpa_partial_outputs[i + 1] = templates;
        }
        const uint32_t total = next_pow2(templates);
        KH_REQUIRE(total <= max_sdpa_map_task_templates, "BiDiBlockGQA replay TaskTemplate count exceeds capacity");
        for (uint32_t i = templates * 3; i < total * 3; ++i) arrays->sdpa_map_task_templates[i] = 0xffffffffu;
        if (out_shape != nullptr) {
            *out_shape = make_replay_shape(num_tokens, num_tokens, uint32_t(ranges.size()), uint32_t(ranges.size()),
                                           templates, total, true);
        }
        return KH_OK;
    });
}

}  // extern "C"
