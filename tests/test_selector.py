"""Host planning logic against the golden vectors of the reference's own tests
(crates/inference-executor-metal/src/attn/gqa/sdpa_test.rs, batch_metadata.rs:328-466,
crates/inference-backend-metal/src/components/gqa/sdpa.rs:346-376,
crates/inference-executor-core/src/replay.rs:92-171). No GPU needed."""
import itertools

import numpy as np
import pytest

from khalamari_b200 import abi
from khalamari_b200.device import Dtype
from khalamari_b200.replay import GQAReplayBucketPolicy, GQAReplayShape, ReplayBucketPolicy
from khalamari_b200.request_page_table import GQAPageTableLayout
from khalamari_b200.sdpa import Config, ExecutionVariant, MapKernelKind, Registry
from khalamari_b200.selector import RequestShape, Selector, SelectorPolicy

U32_MAX = 0xFFFFFFFF


def cfg(head_dim=256, hq=24, hkv=4, page=16, dtype=Dtype.Bfloat16):
    return Config(dtype, hq, hkv, head_dim, page)


def selector_for(config):
    registry = Registry(config)
    return Selector.new(registry, 128, 128, 128 * registry.max_q_tokens_per_map_task())


def selection(token_indices, request_tokens, config=None):
    cu = [0] + list(itertools.accumulate(request_tokens))
    shapes = RequestShape.from_batch(token_indices, cu)
    return selector_for(config or cfg()).select(shapes, GQAReplayBucketPolicy(128, 128), cu[-1])


def is_sliced_kv(sel):
    return sel.variant().kind == MapKernelKind.SlicedKv


# ---- replay.rs ------------------------------------------------------------------------------
def test_default_buckets():
    assert ReplayBucketPolicy(128).buckets() == [1, 2, 4, 6, 8, 12, 16, 20, 24, 32, 40, 48, 56, 64, 80, 96, 112, 128]
    assert ReplayBucketPolicy(70).buckets()[-1] == 70
    assert ReplayBucketPolicy(6).buckets() == [1, 2, 4, 6]
    for cap in [65, 79, 80, 81, 127, 128, 129, U32_MAX]:
        policy = ReplayBucketPolicy(cap)
        assert policy.buckets()[-1] == cap and policy.capacity(cap) == cap
        assert all(a < b for a, b in zip(policy.buckets(), policy.buckets()[1:]))
    policy = ReplayBucketPolicy(64)
    assert [policy.capacity(n) for n in (1, 3, 5, 9, 25, 64)] == [1, 4, 6, 12, 32, 64]
    assert policy.capacity_allow_zero(0) == 0
    with pytest.raises(AssertionError):
        policy.capacity(0)
    with pytest.raises(AssertionError):
        policy.capacity(65)


# ---- sdpa.rs registry -----------------------------------------------------------------------
def test_registry_filters_static_execution_capabilities():
    counts = []
    for head_dim, ratio, page in [(256, 6, 32), (256, 6, 16), (256, 6, 8), (128, 8, 16), (128, 8, 8), (256, 8, 4)]:
        config = Config(Dtype.Bfloat16, 2 * ratio, 2, head_dim, page)
        registry = Registry(config)
        counts.append(len(registry.variants()))
        assert all(v.supports(config) for v in registry.variants())
    assert counts == [4, 4, 4, 2, 2, 1]


def test_variant_constructors():
    c = cfg()
    v = ExecutionVariant.sliced_kv(c, 256, 128, 6)
    assert (v.kind, v.thread_block.max_q_tokens, v.reduce.required_threads) == (MapKernelKind.SlicedKv, 1, 256)
    assert (v.reduce.max_q_heads, v.reduce.max_q_tokens) == (1, 1)
    q = ExecutionVariant.sliced_q(c, MapKernelKind.QTokensAndHeads, 4, 16, 6)
    assert q.thread_block.required_threads == 96 and q.reduce.max_q_tokens == 4 and q.reduce.required_threads == 96
    assert ExecutionVariant.sliced_q_per_head(c, 8, 16, 6).thread_block.required_threads == 192
    assert ExecutionVariant.sliced_q(c, MapKernelKind.QHeadsPerToken, 2, 16, 6).thread_block.required_threads == 64
    with pytest.raises(AssertionError):
        ExecutionVariant.sliced_q(c, MapKernelKind.QTokensPerHead, 3, 16, 6)   # tile must be a power of two <= 32
    with pytest.raises(AssertionError):
        ExecutionVariant.sliced_q(c, MapKernelKind.QTokensPerHead, 8, 16, 7)   # more heads than the group
    with pytest.raises(AssertionError):
        ExecutionVariant.sliced_kv(c, 256, 96, 6)                              # threads must be a power of two
    with pytest.raises(AssertionError):
        Config(Dtype.Bfloat16, 10, 4, 128, 16).validate()


# ---- sdpa_test.rs ---------------------------------------------------------------------------
def test_lookup_preserves_f32_execution_capability():
    for head_dim in (128, 256):
        config = cfg(head_dim, dtype=Dtype.Float32)
        sel = Selector.for_lookup(config, 128, GQAPageTableLayout(4, 1, 1024, 1))
        policy = GQAReplayBucketPolicy(128, sel.limits().max_map_task_templates)
        for history in (0, 4096):
            for q in (1, 8):
                result = sel.select([RequestShape(history, q)], policy, q)
                assert is_sliced_kv(result) and result.variant().supports(config)


def test_lookup_preserves_single_query_kv_parallelism_across_short_context_boundary():
    for hq, hkv, head_dim in [(24, 4, 256), (16, 2, 256), (40, 8, 128)]:
        sel = Selector.for_lookup(cfg(head_dim, hq, hkv), 128, GQAPageTableLayout(8, 1, 128, 1))
        policy = GQAReplayBucketPolicy(128, sel.limits().max_map_task_templates)
        for history in (0, 31, 32, 128, 384, 511, 512, 1024):
            for requests in (1, 4, 8):
                result = sel.select([RequestShape(history, 1)] * requests, policy, requests)
                if history < 32:
                    assert result.direct_output()
                else:
                    assert is_sliced_kv(result) and not result.direct_output()
                    assert result.variant().thread_block.required_threads == 128


@pytest.mark.parametrize("dim,ratio", [(128, 1), (128, 6), (128, 8), (128, 12), (256, 6), (256, 8), (256, 12),
                                       (256, 32)])
def test_lookup_covers_ragged_queries_and_continuous_context_within_replay_capacity(dim, ratio):
    config = Config(Dtype.Bfloat16, 4 * ratio, 4, dim, 16)
    sel = Selector.for_lookup(config, 2048, GQAPageTableLayout(8, 1, 16400, 1))
    limits = sel.limits()
    policy = GQAReplayBucketPolicy(2048, limits.max_map_task_templates)
    for history in (0, 63, 64, 255, 256, 511, 512, 513, 1023, 2048, 4095, 4096, 4097, 8191, 16383, 32768, 65535,
                    98317, 131073, 262144):
        for queries in (1, 2, 3, 4, 5, 7, 8, 12, 16, 32, 64, 256):
            for requests in (1, 2, 8):
                shapes = [RequestShape(history - min(history, i), queries - min(i, queries - 1))
                          for i in range(requests)]
                result = sel.select(shapes, policy, 2048)
                assert result.replay_shape().num_total_sdpa_map_task_templates <= limits.max_map_task_templates
                assert (result.metrics().num_replay_reserved_partial_state_groups
                        <= limits.partial_state_group_capacity)
                ends = [0] * len(result.q_token_ranges())
                for m in result.map_task_templates():
                    assert m.request_local_kv_token_indices.start == ends[m.q_token_range_index]
                    ends[m.q_token_range_index] = m.request_local_kv_token_indices.stop
                assert ends == [r.num_visible_kv_tokens for r in result.q_token_ranges()]


def test_partition_envelope_keeps_variant_maps_and_token_tiles_coupled():
    config = cfg()
    single = ExecutionVariant.sliced_kv(config, 256, 128, 6)
    sliced_q = ExecutionVariant.sliced_q_per_head(config, 8, 16, 6)
    registry = Registry.from_variants(config, [single, sliced_q])
    sel = Selector.for_partitions(registry, 128, 8, lambda _: -(-32768 // 512))
    assert sel.limits().max_map_task_templates == 8192
    assert sel.limits().partial_state_group_capacity == 12288
    sel = Selector.for_partitions(registry, 128, 8, lambda v: 64 if v.kind == MapKernelKind.SlicedKv else 8)
    assert sel.limits().max_map_task_templates == 8192
    assert sel.limits().partial_state_group_capacity == 8192


def test_partition_envelope_rejects_map_count_overflow_before_allocation():
    config = Config(Dtype.Bfloat16, 1, 1, 128, 16)
    variant = ExecutionVariant.sliced_kv(config, 128, 128, 1)
    with pytest.raises(AssertionError, match="GQA partition Map task-template count must fit u32"):
        Selector.for_partitions(Registry.from_variants(config, [variant]), U32_MAX, 1, lambda _: 2)


def test_fixed_slices_cover_ragged_causal_ranges():
    config = Config(Dtype.Bfloat16, 12, 2, 128, 16)
    variant = ExecutionVariant.sliced_q(config, MapKernelKind.QTokensAndHeads, 4, 16, 6)
    sel = Selector.new(Registry.from_variants(config, [variant]), 16, 64, 256)
    requests = RequestShape.from_batch([120, 2], [0, 5, 8])
    policy = GQAReplayBucketPolicy(16, 64)
    result = sel.select_partitioned(variant, 64, False, requests, policy, 8)
    ranges = [(r.request_index, r.flat_q_token_indices, r.num_visible_kv_tokens) for r in result.q_token_ranges()]
    assert ranges == [(0, range(0, 4), 124), (0, range(4, 5), 125), (1, range(5, 8), 5)]
    maps = [(m.q_token_range_index, m.request_local_kv_token_indices) for m in result.map_task_templates()]
    assert maps == [(0, range(0, 64)), (0, range(64, 124)), (1, range(0, 64)), (1, range(64, 125)), (2, range(0, 5))]
    assert result.cu_partial_outputs_by_q_token_range() == [0, 2, 4, 5]
    assert result.metrics().max_kv_iterations_per_split == 4
    assert not result.direct_output()
    result = sel.select_partitioned(variant, 65, False, requests, policy, 8)
    maps = [(m.q_token_range_index, m.request_local_kv_token_indices) for m in result.map_task_templates()]
    assert maps == [(0, range(0, 65)), (0, range(65, 124)), (1, range(0, 65)), (1, range(65, 125)), (2, range(0, 5))]
    assert result.cu_partial_outputs_by_q_token_range() == [0, 2, 4, 5]
    assert result.metrics().max_kv_iterations_per_split == 5
    assert result.metrics().num_scheduled_qk_token_pairs == 1216
    assert result.metrics().num_active_qk_token_pairs == 768


def test_direct_output_preserves_padded_range_identity_without_partials():
    config = Config(Dtype.Bfloat16, 1, 1, 128, 16)
    variant = ExecutionVariant.sliced_q_per_head(config, 1, 16, 1)
    sel = Selector.new(Registry.from_variants(config, [variant]), 9, 64, 1)
    requests = RequestShape.from_batch([64, 2], [0, 7, 9])
    result = sel.select_partitioned(variant, 71, True, requests, GQAReplayBucketPolicy(9, 64), 9)
    shape = result.replay_shape()
    assert result.direct_output()
    assert shape.num_q_token_tiles == 9 and shape.num_sdpa_map_task_templates == 9
    assert shape.num_total_q_token_tiles == shape.num_total_sdpa_map_task_templates
    assert result.metrics().num_active_partial_state_groups == 0
    assert result.metrics().num_replay_reserved_partial_state_groups == 0
    for r, m in zip(result.q_token_ranges(), result.map_task_templates()):
        assert m.request_local_kv_token_indices == range(0, r.num_visible_kv_tokens)


def test_selector_preserves_measured_d256_page16_crossovers():
    for tokens, context in [(1, 65536), (2, 65536), (4, 128), (8, 128), (25, 32)]:
        assert is_sliced_kv(selection([context], [tokens]))
    for tokens, context in [(4, 512), (8, 512), (16, 128), (25, 128), (64, 0)]:
        assert not is_sliced_kv(selection([context], [tokens]))


def test_selector_preserves_other_profile_selection():
    shapes = RequestShape.from_batch([0] * 4, [0, 2, 4, 6, 8])
    policy = GQAReplayBucketPolicy(128, 128)
    v = selector_for(cfg(256, 24, 4, 32)).select(shapes, policy, 8).variant()
    assert (v.thread_block.max_q_tokens, v.thread_block.max_q_heads) == (8, 3)
    v = selector_for(cfg(128, 32, 4, 16)).select(shapes, policy, 8).variant()
    assert (v.thread_block.max_q_tokens, v.thread_block.max_q_heads) == (8, 8)
    v = selector_for(cfg(256, 32, 4, 4)).select(shapes, policy, 8).variant()
    assert v.thread_block.max_q_tokens == 1


def test_selector_prices_request_local_tail_ranges():
    assert is_sliced_kv(selection([65536] * 8, [1] * 8))
    assert is_sliced_kv(selection([1024, 65536], [64, 1]))
    assert is_sliced_kv(selection([65536, 1024], [1, 8]))
    assert not is_sliced_kv(selection([65536, 65536], [8, 1]))


def test_selection_materializes_current_sliced_q_capacity_and_metrics():
    assert is_sliced_kv(selection([1024, 65536], [64, 1]))
    mixed = selection([8192, 65536], [64, 64])
    cu = mixed.cu_partial_outputs_by_q_token_range()
    assert [b - a for a, b in zip(cu, cu[1:])] == [2] * 8 + [14] * 8
    sel = selection([65536], [25])
    assert not is_sliced_kv(sel)
    assert len(sel.q_token_ranges()) == 4 and len(sel.map_task_templates()) == 128
    assert sel.replay_shape().num_total_sdpa_map_task_templates == 128
    m = sel.metrics()
    assert m.num_active_partial_state_groups == 800 and m.num_active_partial_states == 800 * 24
    assert m.num_reserved_partial_state_groups == 1024 and m.num_replay_reserved_partial_state_groups == 1024


def test_selection_map_tasks_cover_each_visible_kv_range_once():
    for history, q in [([1024], [25]), ([8192, 65536], [64, 64]), ([0], [1]), ([0], [128]),
                       ([65536] * 128, [1] * 128)]:
        sel = selection(history, q)
        cu = sel.cu_partial_outputs_by_q_token_range()
        stage = sel.variant().thread_block.kv_tokens_per_iteration
        iterations = sum(-(-r.num_visible_kv_tokens // stage) for r in sel.q_token_ranges())
        templates = sel.map_task_templates()
        assert len(templates) == min(iterations, 128)
        for i, r in enumerate(sel.q_token_ranges()):
            mine = templates[cu[i]:cu[i + 1]]
            assert mine[0].request_local_kv_token_indices.start == 0
            assert mine[-1].request_local_kv_token_indices.stop == r.num_visible_kv_tokens
            for a, b in zip(mine, mine[1:]):
                assert a.request_local_kv_token_indices.stop == b.request_local_kv_token_indices.start


def test_dense_prefill_kv32_preserves_request_ranges_and_replay_capacity():
    registry = Registry(cfg())
    sel = Selector.new(registry, 2048, 2048, 2048 * registry.max_q_tokens_per_map_task())
    policy = GQAReplayBucketPolicy(2048, 2048)
    for histories, cu in [([0], [0, 1024]), ([4096], [0, 1024]), ([0, 16384], [0, 512, 1024])]:
        result = sel.select(RequestShape.from_batch(histories, cu), policy, 2048)
        assert result.variant().thread_block.kv_tokens_per_iteration == 32
        assert result.replay_shape().num_tokens == 1024 and result.replay_shape().num_total_tokens == 2048
        assert len(result.map_task_templates()) == 256
    short = sel.select(RequestShape.from_batch([4096], [0, 256]), policy, 2048)
    assert short.variant().thread_block.kv_tokens_per_iteration == 16
    decode = sel.select(RequestShape.from_batch([4096] * 1024, list(range(1025))), policy, 2048)
    assert decode.variant().thread_block.max_q_tokens == 1


def test_map_capacity_preserves_token_domain_and_replay_padding():
    config = Config(Dtype.Bfloat16, 1, 1, 128, 8)
    variant = ExecutionVariant.sliced_kv(config, 64, 128, 1)
    sel = Selector.new(Registry.from_variants(config, [variant]), 4, 32, 32)
    policy = GQAReplayBucketPolicy(4, 32)
    result = sel.select(RequestShape.from_batch([1088], [0, 1]), policy, 2)
    shape = result.replay_shape()
    assert sel.limits().max_tokens == 4
    assert (shape.num_tokens, shape.num_total_tokens) == (1, 2)
    assert (shape.num_sdpa_map_task_templates, shape.num_total_sdpa_map_task_templates) == (18, 20)
    assert result.metrics().num_replay_reserved_partial_state_groups == 20
    assert result.map_task_templates()[-1].request_local_kv_token_indices == range(1088, 1089)
    with pytest.raises(AssertionError):
        sel.select(RequestShape.from_batch([0], [0, 5]), policy, 4)


def test_capacity_and_token_count_rejections():
    config = Config(Dtype.Bfloat16, 1, 1, 128, 8)
    variant = ExecutionVariant.sliced_kv(config, 64, 128, 1)
    sel = Selector.new(Registry.from_variants(config, [variant]), 4, 32, 18)
    with pytest.raises(AssertionError, match="GQA SDPA replay exceeds its partial-state-group capacity"):
        sel.select(RequestShape.from_batch([1088], [0, 1]), GQAReplayBucketPolicy(4, 32), 2)
    shapes = RequestShape.from_batch([0], [0, 5])
    with pytest.raises(AssertionError, match="GQA active token count must not exceed the total token count"):
        selector_for(cfg()).select(shapes, GQAReplayBucketPolicy(128, 128), 4)
    with pytest.raises(AssertionError, match="GQA total token count must not exceed the metadata capacity"):
        selector_for(cfg()).select(shapes, GQAReplayBucketPolicy(128, 128), 129)
    with pytest.raises(AssertionError, match="GQA replay bucket policy must match"):
        selector_for(cfg()).select(shapes, GQAReplayBucketPolicy(64, 128), 5)


# ---- batch_metadata.rs golden arrays (host images; the device upload is checked on the GPU) -----
def _metadata_arrays(max_tokens, max_maps, fill=0):
    import ctypes as C
    names = ["req_slots", "flat_token_indices", "visible_kv_token_ranges", "q_token_ranges",
             "sdpa_map_task_templates", "cu_sdpa_partial_outputs"]
    sizes = [max_tokens, max_tokens, 2 * max_tokens, 2 * max_tokens, 3 * max_maps, max_tokens + 1]
    host = {n: np.full(s, fill, dtype=np.uint32) for n, s in zip(names, sizes)}
    u32p = C.POINTER(C.c_uint32)
    arrays = abi.MetadataArraysC(*[host[n].ctypes.data_as(u32p) for n in names], max_tokens, max_maps)
    return host, arrays


def _update(host_arrays, req_slots, token_indices, cu_tokens, selection):
    import ctypes as C
    u32p = C.POINTER(C.c_uint32)
    host, arrays = host_arrays
    a = [np.ascontiguousarray(x, dtype=np.uint32) for x in (req_slots, token_indices, cu_tokens)]
    shape = abi.ReplayShapeC()
    abi.call("kh_metadata_update", C.byref(arrays), a[0].ctypes.data_as(u32p), a[1].ctypes.data_as(u32p),
             a[2].ctypes.data_as(u32p), len(req_slots), selection.handle, C.byref(shape))
    return GQAReplayShape.from_c(shape)


def small_config():
    return Config(Dtype.Bfloat16, 2, 2, 128, 8)


def small_selector(max_tokens, variant):
    return Selector.new(Registry.from_variants(small_config(), [variant]), max_tokens, max_tokens,
                        max_tokens * variant.thread_block.max_q_tokens)


def test_map_metadata_capacity_is_independent_of_token_capacity():
    meta = _metadata_arrays(4, 32)
    variant = ExecutionVariant.sliced_kv(small_config(), 64, 128, 1)
    sel = Selector.new(Registry.from_variants(small_config(), [variant]), 4, 32, 32)
    result = sel.select(RequestShape.from_batch([1088], [0, 1]), GQAReplayBucketPolicy(4, 32), 2)
    shape = _update(meta, [1], [1088], [0, 1], result)
    host = meta[0]
    assert (shape.num_tokens, shape.num_total_tokens) == (1, 2)
    assert (shape.num_sdpa_map_task_templates, shape.num_total_sdpa_map_task_templates) == (18, 20)
    assert host["flat_token_indices"][0] == 1088
    assert host["visible_kv_token_ranges"][:2].tolist() == [0, 1089]
    assert host["sdpa_map_task_templates"][18 * 3:20 * 3].tolist() == [U32_MAX] * 6
    assert host["cu_sdpa_partial_outputs"][:2].tolist() == [0, 18]


def test_metadata_upload_preserves_current_abi_for_complete_selections():
    meta = _metadata_arrays(8, 8)
    host = meta[0]
    shapes = RequestShape.from_batch([7, 20], [0, 2, 5])
    policy = GQAReplayBucketPolicy(8, 8)
    single = ExecutionVariant.sliced_kv(small_config(), 8, 32, 1)
    shape = _update(meta, [2, 5], [7, 20], [0, 2, 5], small_selector(8, single).select(shapes, policy, 5))
    assert host["req_slots"][:5].tolist() == [2, 2, 5, 5, 5]
    assert host["flat_token_indices"][:5].tolist() == [7, 8, 20, 21, 22]
    assert host["visible_kv_token_ranges"][:10].tolist() == [0, 8, 0, 9, 0, 21, 0, 22, 0, 23]
    assert host["sdpa_map_task_templates"][:24].tolist() == [
        0, 0, 8, 1, 0, 9, 2, 0, 8, 2, 8, 21, 3, 0, 8, 3, 8, 22, 4, 0, 8, 4, 8, 23]
    assert host["cu_sdpa_partial_outputs"][:6].tolist() == [0, 1, 2, 4, 6, 8]
    assert shape == GQAReplayShape.new(5, 5, 5, 6, 8, 8, True)

    sliced_q = ExecutionVariant.sliced_q_per_head(small_config(), 8, 8, 1)
    shape = _update(meta, [2, 5], [7, 20], [0, 2, 5], small_selector(8, sliced_q).select(shapes, policy, 5))
    assert host["q_token_ranges"][:4].tolist() == [0, 2, 2, 5]
    assert host["sdpa_map_task_templates"][:18].tolist() == [
        0, 0, 8, 0, 8, 9, 1, 0, 8, 1, 8, 16, 1, 16, 23, U32_MAX, U32_MAX, U32_MAX]
    assert host["cu_sdpa_partial_outputs"][:3].tolist() == [0, 2, 5]
    assert shape == GQAReplayShape.new(5, 5, 2, 2, 5, 6, True)


def test_selection_preserves_non_kv_metadata_tail():
    meta = _metadata_arrays(12, 12)
    host = meta[0]
    host["visible_kv_token_ranges"][:] = 0x94949494
    host["q_token_ranges"][:] = 0xA5A5A5A5
    host["sdpa_map_task_templates"][:] = 0xB6B6B6B6
    host["cu_sdpa_partial_outputs"][:] = 0xC7C7C7C7
    variant = ExecutionVariant.sliced_q_per_head(small_config(), 8, 8, 1)
    result = small_selector(12, variant).select(RequestShape.from_batch([0, 0, 0], [0, 4, 8, 9]),
                                                GQAReplayBucketPolicy(12, 12), 12)
    shape = _update(meta, [2, 5, 7], [0, 0, 0], [0, 4, 8, 9], result)
    assert shape == GQAReplayShape.new(9, 12, 3, 4, 3, 4, True)
    assert host["visible_kv_token_ranges"][18:20].tolist() == [0x94949494] * 2
    assert host["q_token_ranges"][6:8].tolist() == [0xA5A5A5A5] * 2
    assert host["sdpa_map_task_templates"][9:12].tolist() == [U32_MAX] * 3
    assert host["cu_sdpa_partial_outputs"][4] == 0xC7C7C7C7


# ---- B200 policy ----------------------------------------------------------------------------
def test_b200_policy_produces_legal_contiguous_plans():
    for hq, hkv, d in [(64, 8, 128), (24, 4, 256), (16, 2, 256), (32, 2, 128)]:
        config = Config(Dtype.Bfloat16, hq, hkv, d, 16)
        sel = Selector.for_lookup(config, 1024, GQAPageTableLayout(64, 1, 4096, 1)).set_policy(SelectorPolicy.B200, 148)
        limits = sel.limits()
        policy = GQAReplayBucketPolicy(1024, limits.max_map_task_templates)
        rng = np.random.default_rng(hq)
        for q in (1, 2, 4, 16):
            shapes = [RequestShape(int(rng.integers(0, 60000)), q) for _ in range(int(rng.integers(1, 60)))]
            result = sel.select(shapes, policy, 1024)
            variant = result.variant()
            assert variant.supports(config) and variant in sel.variants()
            assert variant.thread_block.max_q_tokens * variant.thread_block.max_q_heads <= 128
            if q == 1 and hq // hkv <= 8:
                assert is_sliced_kv(result)
            ends = [0] * len(result.q_token_ranges())
            for m in result.map_task_templates():
                assert m.request_local_kv_token_indices.start == ends[m.q_token_range_index]
                ends[m.q_token_range_index] = m.request_local_kv_token_indices.stop
            assert ends == [r.num_visible_kv_tokens for r in result.q_token_ranges()]
            assert result.metrics().num_replay_reserved_partial_state_groups <= limits.partial_state_group_capacity


def test_b200_policy_sizes_slices_for_148_sms():
    config = Config(Dtype.Bfloat16, 64, 8, 128, 16)
    sel = Selector.for_lookup(config, 64, GQAPageTableLayout(64, 1, 512, 1)).set_policy(SelectorPolicy.B200, 148)
    policy = GQAReplayBucketPolicy(64, sel.limits().max_map_task_templates)
    # 64 x 4608 tokens x 8 KV heads over 148 SMs x 4 tasks -> 2048-token slices (the upper clamp)
    result = sel.select([RequestShape(4607, 1)] * 64, policy, 64)
    sizes = {len(m.request_local_kv_token_indices) for m in result.map_task_templates()}
    assert max(sizes) == 2048
    # four short requests give every SM a task at the floor of 256 tokens (4 x 8 slices x 8 KV heads = 256 tasks)
    result = sel.select([RequestShape(2047, 1)] * 4, policy, 64)
    assert {len(m.request_local_kv_token_indices) for m in result.map_task_templates()} == {256}
    # a single short request does not (64 tasks on 148 SMs): the slice drops towards one task per SM, not below 64
    result = sel.select([RequestShape(2047, 1)], policy, 64)
    assert {len(m.request_local_kv_token_indices) for m in result.map_task_templates()} == {64}
    result = sel.select([RequestShape(255, 1)], policy, 64)
    assert {len(m.request_local_kv_token_indices) for m in result.map_task_templates()} == {64}
