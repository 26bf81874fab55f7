"""Parity of the CUDA path against the CPU oracle, through the C ABI (``-m gpu``).

Scenarios follow the reference's own kernel tests
(crates/inference-backend-metal/src/components/gqa/sdpa/sliced_kv_test.rs, sliced_q_test.rs and
crates/inference-executor-metal/tests/gqa_sdpa_sliced_q.rs), restated for bf16 / fp16 KV pages and the
head dimensions this backend instantiates, plus the build's own configurations.
Tolerance (stated by the build contract): per element |a - b| <= 2e-3 or |a - b| <= 1e-2 |b|."""
import numpy as np
import pytest

import oracle
from helpers import DeviceCase, assert_within_contract, bits_to_f32, make_case, round_to

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    from khalamari_b200.device import Device
    dev = Device(0)
    yield dev


def _variant_kv(attention, slice_threads=128):
    from khalamari_b200.sdpa import ExecutionVariant
    cfg = attention.sdpa_config
    return ExecutionVariant.sliced_kv(cfg, cfg.head_dim, slice_threads, min(cfg.q_heads_per_kv_head(), 8))


def _forced_selector(case, dtype, variants, max_tokens, max_maps):
    from khalamari_b200.sdpa import Config, Registry
    from khalamari_b200.selector import Selector
    cfg = Config(dtype, case.num_q_heads, case.num_kv_heads, case.head_dim, case.tokens_per_page)
    tile = max(v.thread_block.max_q_tokens for v in variants)
    return Selector.new(Registry.from_variants(cfg, variants), max_tokens, max_maps, max_maps * tile)


# ---------------------------------------------------------------------------------------------------
# Build configuration 1: batch 4, contexts {128, 517, 1024, 2048}, q_len 1, Hq16/Hkv2, D256, fp16, seed 0
# ---------------------------------------------------------------------------------------------------
def test_config1_fp16_decode(device):
    contexts = [128, 517, 1024, 2048]
    case = make_case(0, "f16", 16, 2, 256, [c - 1 for c in contexts], [1] * 4, scale=1.0 / 16.0)
    run = DeviceCase(device, case)
    out = run.run()
    assert out.shape == (4, 16, 256)
    assert_within_contract(out, case.oracle_output(), "config 1")


@pytest.mark.parametrize("dtype_name,hq,hkv,d", [("bf16", 64, 8, 128), ("bf16", 16, 2, 256), ("f16", 64, 8, 128),
                                                 ("bf16", 24, 4, 256), ("bf16", 4, 4, 128), ("bf16", 32, 2, 128)])
def test_decode_matches_oracle_on_ragged_batches(device, dtype_name, hq, hkv, d):
    rng = np.random.default_rng(hq * 7 + d)
    contexts = [1, 15, 16, 17, 31, 32, 33, 500, 512, 513, 1024, int(rng.integers(1025, 3000)), 2049]
    case = make_case(1, dtype_name, hq, hkv, d, [c - 1 for c in contexts], [1] * len(contexts))
    out = DeviceCase(device, case).run()
    assert_within_contract(out, case.oracle_output(), f"decode {dtype_name} Hq{hq}/Hkv{hkv}/D{d}")


@pytest.mark.parametrize("kv_slice", [16, 65, 256, 512, 4096])
def test_decode_fixed_slices_including_unaligned(device, kv_slice):
    """Forced split-KV slices (Selector::select_partitioned); 65 puts slice boundaries inside pages."""
    from khalamari_b200.device import Dtype
    contexts = [700, 33, 1500, 64]
    case = make_case(2, "bf16", 64, 8, 128, [c - 1 for c in contexts], [1] * 4)
    probe = DeviceCase(device, case)
    variant = _variant_kv(probe.attention)
    selector = _forced_selector(case, Dtype.Bfloat16, [variant], 8, 512)
    run = DeviceCase(device, case, max_tokens=8, selector=selector)
    selection = run.attention.select_partitioned(variant, kv_slice, False, case.token_indices, case.cu_tokens)
    expected_maps = sum(-(-c // kv_slice) for c in contexts)
    assert len(selection.map_task_templates()) == expected_maps
    out = run.run(selection)
    assert_within_contract(out, case.oracle_output(), f"slice {kv_slice}")


def test_page_indexing_is_bit_exact(device):
    """A query that matches exactly one cached token makes softmax a one-hot, so the output row must equal
    that token's V row bit for bit. Walking the target over pages, page offsets, KV heads, layers and
    page-ids-per-block checks the block-table gather and the page address arithmetic end to end."""
    hq, hkv, d, page = 8, 2, 128, 16
    ctx = 16 * 9 + 5
    case = make_case(3, "bf16", hq, hkv, d, [ctx - 1], [1], num_gqa_layers=3, layer_index=2,
                     num_page_ids_per_block=2, extra_slots=2, scale=1.0)
    rng = np.random.default_rng(17)
    targets = [0, 1, 15, 16, 17, 31, 100, ctx - 6, ctx - 1] + rng.integers(0, ctx, size=6).tolist()
    k = case.k_f32[0].copy()
    v = case.v_f32[0]
    # K rows are +-1 patterns unique per token: q = 64 * k[target] gives logit 64 * D for the target and
    # far less for every other token, so every other probability underflows to exactly zero.
    signs = rng.integers(0, 2, size=(ctx, hkv, d)).astype(np.float32) * 2 - 1
    k[:] = signs
    k_bits, _ = round_to("bf16", k)
    v_bits, _ = round_to("bf16", v)
    oracle.scatter_paged(case.pool, case.page_ids, case.layout, case.req_slots[0], case.layer_index, page, hkv, d, 2,
                         0, k_bits, v_bits)
    case.k_f32[0] = k
    run = DeviceCase(device, case)
    for target in targets:
        q = np.zeros((1, hq, d), dtype=np.float32)
        for h in range(hq):
            q[0, h] = 64.0 * k[target, h // (hq // hkv)]
        q_bits, q_round = round_to("bf16", q)
        run.q.write(0, q_bits)
        case.q_f32 = q_round
        out_bits = None
        run.run()
        out_bits = run.output.read(0, hq * d, np.uint16).reshape(hq, d)
        for h in range(hq):
            assert np.array_equal(out_bits[h], v_bits[target, h // (hq // hkv)]), (target, h)


def test_replay_matches_reference_across_active_counts(device):
    """sliced_kv_test.rs:118-187: one recorded shape, active token counts 1,8,3,7,2,6,4,5; token i sees i+1 KV
    tokens of one shared request; rows at or past the active count stay untouched."""
    from khalamari_b200 import sliced_kv
    from khalamari_b200.device import Buffer, Dtype, Stream
    from khalamari_b200.request_page_table import GQAPageTableLayout
    from khalamari_b200.sdpa import ExecutionVariant
    hq, hkv, d, page = 16, 2, 128, 16
    q = oracle.generated_values(8 * hq * d, 0x8B1D5A73)
    k = oracle.generated_values(8 * hkv * d, 0x8B1D5A74).reshape(8, hkv, d)
    v = oracle.generated_values(8 * hkv * d, 0x8B1D5A75).reshape(8, hkv, d)
    q_bits, q_round = round_to("bf16", q)
    k_bits, k_round = round_to("bf16", k)
    v_bits, v_round = round_to("bf16", v)
    layout = GQAPageTableLayout(1, 1, 1, 1)
    config = sliced_kv.Config(hq, hkv, d, 0.5, 2 * hkv * page * d * 2, layout, Dtype.Bfloat16)
    shape = sliced_kv.Shape(8, 8)
    pool = np.zeros(config.page_bytes, dtype=np.uint8)
    table = np.zeros(1, dtype=np.uint32)
    oracle.scatter_paged(pool, table, oracle.PageTableLayout(1, 1, 1, 1), 0, 0, page, hkv, d, 2, 0, k_bits, v_bits)
    execution = ExecutionVariant.sliced_kv(config.sdpa_config(), 128, 128, 8)
    compute = sliced_kv.Compute(device, config, execution, shape)
    stream = Stream(device)
    scratch = sliced_kv.Scratch(device, config, shape)
    templates = np.array([[i, 0, i + 1] for i in range(8)], dtype=np.uint32)
    bufs = dict(
        q=Buffer.from_slice(device, q_bits), kv=Buffer.from_slice(device, pool),
        slots=Buffer.from_slice(device, np.zeros(8, np.uint32)), ids=Buffer.from_slice(device, table),
        templates=Buffer.from_slice(device, templates), cu=Buffer.from_slice(device, np.arange(9, dtype=np.uint32)))
    row = hq * d
    for active in [1, 8, 3, 7, 2, 6, 4, 5]:
        output = Buffer.from_slice(device, np.full(8 * row, 0x4228, dtype=np.uint16))
        compute.invoke_map(stream, scratch.map_buffers(bufs["q"], bufs["kv"], bufs["slots"], bufs["ids"],
                                                       bufs["templates"]), 0, active, active)
        compute.invoke_reduce(stream, scratch.reduce_buffers(bufs["cu"], output), active)
        stream.synchronize()
        assert device.check(stream) == 0
        bits = output.read(0, 8 * row, np.uint16)
        assert np.all(bits[active * row:] == 0x4228)
        expected = oracle.projected_gqa([0, active], [0], q_round[:active * row], [k_round[:active]],
                                        [v_round[:active]], d, hq, hkv, 0.5)
        assert_within_contract(bits_to_f32("bf16", bits[:active * row]).reshape(active, hq, d), expected,
                               f"active {active}")


def test_ragged_requests_and_multiple_page_ids_per_block(device):
    """sliced_kv_test.rs:190-281: two requests sharing one batch with slots [0, 1, 1]; two page ids per
    block; a nonzero layer slot."""
    case = make_case(5, "bf16", 16, 2, 256, [1, 0], [1, 2], num_gqa_layers=2, layer_index=1,
                     num_page_ids_per_block=2)
    out = DeviceCase(device, case).run()
    assert_within_contract(out, case.oracle_output(), "ragged")
    case = make_case(6, "bf16", 16, 2, 128, [63], [1], num_page_ids_per_block=2)
    out = DeviceCase(device, case).run()
    assert_within_contract(out, case.oracle_output(), "two page ids per block")


# ---------------------------------------------------------------------------------------------------
# Verify (MTP / DFlash): q_len 2 and 4, causal among the new tokens (build configuration 3 geometry)
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("hq,hkv,d", [(24, 4, 256), (64, 8, 128)])
def test_verify_q2_q4_causal(device, hq, hkv, d):
    histories = [0, 5, 14, 15, 16, 300, 511, 512, 1000, 2000]
    q_lens = [2, 4, 2, 4, 4, 2, 4, 4, 2, 4]
    case = make_case(7, "bf16", hq, hkv, d, histories, q_lens)
    out = DeviceCase(device, case, max_tokens=64).run()
    assert_within_contract(out, case.oracle_output(), f"verify Hq{hq}/Hkv{hkv}/D{d}")


def test_prefill_chunks_and_mixed_batch(device):
    """gqa_sdpa_sliced_q.rs:26-48: tokens per request [16]x8, ragged [1,2,4,6,8,11,16,16], [32,8], [1,4,8,13]."""
    for hq, hkv, d, q_lens, start in [(8, 1, 256, [16] * 4, 0), (6, 1, 256, [16] * 2, 40),
                                      (16, 2, 128, [1, 2, 4, 6, 8, 11, 16, 16], 100), (16, 2, 128, [32, 8], 7),
                                      (5, 1, 128, [1, 4, 8, 13], 0)]:
        case = make_case(8 + hq, "bf16", hq, hkv, d, [start + 3 * i for i in range(len(q_lens))], q_lens)
        out = DeviceCase(device, case, max_tokens=128).run()
        assert_within_contract(out, case.oracle_output(), f"prefill {q_lens}")


@pytest.mark.parametrize("kind_name,ratio,tile,heads,stage,head_dim", [
    ("QHeadsPerToken", 6, 4, 6, 8, 128), ("QTokensAndHeads", 6, 4, 6, 16, 128), ("QTokensAndHeads", 6, 4, 3, 32, 256),
    ("QHeadsPerToken", 8, 2, 4, 64, 256), ("QTokensAndHeads", 12, 4, 12, 128, 256),
    ("QTokensPerHead", 12, 1, 6, 64, 128), ("QTokensPerHead", 6, 8, 6, 16, 256), ("QTokensPerHead", 8, 16, 8, 16, 128),
])
@pytest.mark.parametrize("direct", [False, True])
def test_q_token_head_assignments_and_direct_output(device, kind_name, ratio, tile, heads, stage, head_dim, direct):
    """sliced_q_test.rs:221-401: every Q token/head assignment, split map + reduce and direct output."""
    from khalamari_b200.device import Dtype
    from khalamari_b200.sdpa import Config, ExecutionVariant, MapKernelKind
    hkv = 2
    hq = hkv * ratio
    histories, q_lens = [40, 3], [tile + 1 if tile > 1 else 3, 1]
    case = make_case(31, "bf16", hq, hkv, head_dim, histories, q_lens)
    cfg = Config(Dtype.Bfloat16, hq, hkv, head_dim, 16)
    variant = ExecutionVariant.sliced_q(cfg, MapKernelKind[kind_name], tile, stage, heads)
    selector = _forced_selector(case, Dtype.Bfloat16, [variant], 32, 64)
    run = DeviceCase(device, case, max_tokens=32, selector=selector)
    kv_slice = 4096 if direct else 16
    selection = run.attention.select_partitioned(variant, kv_slice, direct, case.token_indices, case.cu_tokens)
    assert selection.direct_output() == direct
    out = run.run(selection)
    assert_within_contract(out, case.oracle_output(), f"{kind_name} direct={direct}")


def test_windowed_and_empty_visibility_with_descending_pages(device):
    """sliced_q_test.rs:53-218: two GQA layers (layer 1 used), three blocks of two page ids, physical pages
    handed out in descending order, per-token visibility windows (sliding and empty), and output rows of
    inactive tokens left untouched."""
    from khalamari_b200 import sliced_q
    from khalamari_b200.device import Buffer, Dtype, Stream
    from khalamari_b200.request_page_table import GQAPageTableLayout
    from khalamari_b200.sdpa import ExecutionVariant
    for head_dim in (128, 256):
        hq, hkv, page = 6, 2, 16
        layout = GQAPageTableLayout(2, 2, 3, 2)
        config = sliced_q.Config(hq, hkv, head_dim, head_dim ** -0.5, 4 * page * head_dim * 2, Dtype.Bfloat16, layout)
        shape = sliced_q.Shape(20, 4, 8)
        execution = ExecutionVariant.sliced_q_per_head(config.sdpa_config(), 16, 16, 2)
        compute = sliced_q.Compute(device, config, execution, shape)
        q_vals = oracle.generated_values(20 * hq * head_dim, 17, centered_bf16=True)
        kv_width = hkv * head_dim
        lens = [36, 7]
        keys = [oracle.generated_values(n * kv_width, 31, True).reshape(n, hkv, head_dim) for n in lens]
        values = [oracle.generated_values(n * kv_width, 47, True).reshape(n, hkv, head_dim) for n in lens]
        table = np.full(24, 0xFFFFFFFF, dtype=np.uint32)
        pool = np.zeros(12 * config.page_bytes, dtype=np.uint8)
        next_page = 11
        olayout = oracle.PageTableLayout(2, 2, 3, 2)
        for req, slot in enumerate([1, 0]):
            pages = -(-lens[req] // page)
            for i in range(pages):
                table[slot * 12 + 6 + i] = next_page
                next_page -= 1
            oracle.scatter_paged(pool, table, olayout, slot, 1, page, hkv, head_dim, 2, 0,
                                 round_to("bf16", keys[req])[0], round_to("bf16", values[req])[0])
        slots = np.ones(20, dtype=np.uint32)
        slots[17] = 0
        ranges = np.array([0, 16, 16, 17, 17, 18, 0xFFFFFFFF, 0xFFFFFFFF], dtype=np.uint32)
        templates = np.array([0, 0, 16, 0, 16, 35, 1, 0, 16, 1, 16, 36, 2, 0, 7, 2, 7, 7] + [0xFFFFFFFF] * 6,
                             dtype=np.uint32)
        cu = np.array([0, 2, 4, 6, 0xFFFFFFFF], dtype=np.uint32)
        sizes = config.sizes(execution, shape)
        stream = Stream(device)
        d_q = Buffer.from_slice(device, round_to("bf16", q_vals)[0])
        d_pool, d_table = Buffer.from_slice(device, pool), Buffer.from_slice(device, table)
        d_slots, d_ranges = Buffer.from_slice(device, slots), Buffer.from_slice(device, ranges)
        d_templates, d_cu = Buffer.from_slice(device, templates), Buffer.from_slice(device, cu)
        d_visible = Buffer.new_zeroed(device, 40 * 4)
        d_po = Buffer.new_zeroed(device, sizes.partial_output_bytes)
        d_ps = Buffer.new_zeroed(device, sizes.partial_output_stats_bytes)
        d_pm = Buffer.new_zeroed(device, sizes.partial_output_stats_bytes)
        q_width = hq * head_dim
        for windowed in (False, True):
            d_out = Buffer.from_slice(device, np.full(20 * q_width, 0x4228, dtype=np.uint16))
            visibility, expected = [], []
            for token in range(18):
                req = int(token == 17)
                end = 20 + token if req == 0 else 7
                begin = (end - 3 if req == 0 else end) if windowed else 0
                visibility += [begin, end]
                if begin == end:
                    expected.append(np.zeros((hq, head_dim), np.float32))
                else:
                    expected.append(oracle.projected_gqa(
                        [0, 1], [end - begin - 1], q_vals[token * q_width:(token + 1) * q_width],
                        [keys[req][begin:end]], [values[req][begin:end]], head_dim, hq, hkv, config.scale)[0])
            d_visible.write(0, np.array(visibility + [0] * 4, dtype=np.uint32))
            compute.invoke_map(stream, sliced_q.MapBuffers(d_q, d_pool, d_slots, d_table, d_visible, d_ranges,
                                                           d_templates, d_po, d_ps, d_pm), 1, 18, 3, 6)
            compute.invoke_reduce(stream, sliced_q.ReduceBuffers(d_po, d_ps, d_pm, d_ranges, d_cu, d_out), 3)
            stream.synchronize()
            assert device.check(stream) == 0
            bits = d_out.read(0, 20 * q_width, np.uint16)
            assert np.all(bits[18 * q_width:] == 0x4228)
            assert_within_contract(bits_to_f32("bf16", bits[:18 * q_width]).reshape(18, hq, head_dim),
                                   np.stack(expected), f"windowed={windowed} D{head_dim}")


def test_empty_first_partial_is_ignored_by_reduce(device):
    """sliced_q_test.rs:440-540: the first of two map tasks has an empty KV range; map publishes the
    canonical empty partial and reduce keeps the second task's result, for active token counts 1,4,3,2."""
    from khalamari_b200 import sliced_q
    from khalamari_b200.device import Buffer, Dtype, Stream
    from khalamari_b200.request_page_table import GQAPageTableLayout
    from khalamari_b200.sdpa import ExecutionVariant
    hq, hkv, d, page = 5, 1, 128, 16
    layout = GQAPageTableLayout(1, 1, 1, 1)
    config = sliced_q.Config(hq, hkv, d, d ** -0.5, 2 * page * d * 2, Dtype.Bfloat16, layout)
    shape = sliced_q.Shape(4, 1, 2)
    execution = ExecutionVariant.sliced_q_per_head(config.sdpa_config(), 8, 16, 5)
    compute = sliced_q.Compute(device, config, execution, shape)
    q_vals = oracle.generated_values(4 * hq * d, 0x47514154, True)
    k = oracle.generated_values(page * d, 0x47514155, True).reshape(page, 1, d)
    v = oracle.generated_values(page * d, 0x47514156, True).reshape(page, 1, d)
    pool = np.zeros(config.page_bytes, dtype=np.uint8)
    oracle.scatter_paged(pool, np.zeros(1, np.uint32), oracle.PageTableLayout(1, 1, 1, 1), 0, 0, page, 1, d, 2, 0,
                         round_to("bf16", k)[0], round_to("bf16", v)[0])
    sizes = config.sizes(execution, shape)
    stream = Stream(device)
    d_q = Buffer.from_slice(device, round_to("bf16", q_vals)[0])
    d_pool, d_table = Buffer.from_slice(device, pool), Buffer.from_slice(device, np.zeros(1, np.uint32))
    d_slots = Buffer.new_zeroed(device, 16)
    d_visible = Buffer.from_slice(device, np.array([[0, i + 1] for i in range(4)], dtype=np.uint32))
    d_ranges, d_templates = Buffer.new_zeroed(device, 8), Buffer.new_zeroed(device, 24)
    d_cu = Buffer.from_slice(device, np.array([0, 2], dtype=np.uint32))
    d_po = Buffer.new_zeroed(device, sizes.partial_output_bytes)
    d_ps = Buffer.from_slice(device, np.full(sizes.partial_output_stats_bytes // 4, 7.0, np.float32))
    d_pm = Buffer.from_slice(device, np.full(sizes.partial_output_stats_bytes // 4, 7.0, np.float32))
    d_out = Buffer.new_zeroed(device, sizes.q_bytes)
    for active in [1, 4, 3, 2]:
        d_ranges.write(0, np.array([0, active], dtype=np.uint32))
        d_templates.write(0, np.array([0, 0, 0, 0, 0, active], dtype=np.uint32))
        compute.invoke_map(stream, sliced_q.MapBuffers(d_q, d_pool, d_slots, d_table, d_visible, d_ranges,
                                                       d_templates, d_po, d_ps, d_pm), 0, active, 1, 2)
        compute.invoke_reduce(stream, sliced_q.ReduceBuffers(d_po, d_ps, d_pm, d_ranges, d_cu, d_out), 1)
        stream.synchronize()
        assert device.check(stream) == 0
        sums = d_ps.read(0, hq * 8, np.float32).reshape(hq, 8)
        maxs = d_pm.read(0, hq * 8, np.float32).reshape(hq, 8)
        assert np.all(sums[:, :active] == 0.0) and np.all(np.isneginf(maxs[:, :active]))
        expected = oracle.projected_gqa([0, active], [0], q_vals[:active * hq * d], [k[:active]], [v[:active]], d, hq,
                                        hkv, config.scale)
        bits = d_out.read(0, active * hq * d, np.uint16)
        assert_within_contract(bits_to_f32("bf16", bits).reshape(active, hq, d), expected, f"active {active}")


def test_poisoned_tail_pages_do_not_leak(device):
    """The unwritten rest of a last page (and whole unallocated pages) hold NaN bit patterns; outputs must
    stay finite and correct for contexts ending at every offset inside a page."""
    contexts = list(range(33, 49))
    case = make_case(11, "bf16", 16, 2, 128, [c - 1 for c in contexts], [1] * len(contexts), poison=True)
    out = DeviceCase(device, case).run()
    assert_within_contract(out, case.oracle_output(), "poisoned tails")


def test_cross_rank_combine_matches_unsplit_attention(device):
    """Split one long sequence into N contiguous page ranges (the cross-GPU split of the long-context
    configuration), run each range as its own attention call producing an (max, exp-sum, output) triple per
    (token, head), and merge the triples with kh_combine_partials: the result equals the unsplit call."""
    from khalamari_b200 import sliced_kv
    from khalamari_b200.device import Buffer, Dtype, Stream
    from khalamari_b200.gqa import combine_partials
    hq, hkv, d, ctx = 16, 2, 256, 6000
    case = make_case(12, "bf16", hq, hkv, d, [ctx - 1], [1], scale=1.0 / 16.0)
    full = DeviceCase(device, case).run()
    expected = case.oracle_output()
    assert_within_contract(full, expected, "unsplit")
    for ranks in (2, 4, 8):
        run = DeviceCase(device, case)
        att = run.attention
        variant = _variant_kv(att)
        stream = run.stream
        rows = hq
        all_sum = Buffer.new_zeroed(device, ranks * rows * 4)
        all_max = Buffer.new_zeroed(device, ranks * rows * 4)
        all_out = Buffer.new_zeroed(device, ranks * rows * d * 4)
        pages = -(-ctx // 16)
        for r in range(ranks):
            begin = (pages * r // ranks) * 16
            end = min((pages * (r + 1) // ranks) * 16, ctx)
            # rank r sees only tokens [begin, end): templates of 512 tokens inside that range
            templates = [[0, b, min(b + 512, end)] for b in range(begin, end, 512)]
            n = len(templates)
            shape = sliced_kv.Shape(1, n)
            config = sliced_kv.Config(hq, hkv, d, case.scale, case.page_bytes, run.layout, Dtype.Bfloat16)
            compute = sliced_kv.Compute(device, config, variant, shape)
            scratch = sliced_kv.Scratch(device, config, shape)
            d_templates = Buffer.from_slice(device, np.array(templates, dtype=np.uint32))
            d_slots = Buffer.from_slice(device, np.array(case.req_slots, dtype=np.uint32))
            compute.invoke_map(stream, scratch.map_buffers(run.q, run.kv_pages, d_slots, run.page_ids, d_templates), 0,
                               1, n)
            rank_out = Buffer.wrap(device, all_out.ref.ptr + r * rows * d * 4, rows * d * 4)
            rank_sum = Buffer.wrap(device, all_sum.ref.ptr + r * rows * 4, rows * 4)
            rank_max = Buffer.wrap(device, all_max.ref.ptr + r * rows * 4, rows * 4)
            combine_partials(device, stream, n, rows, d, scratch.partial_exp_sums, scratch.partial_max_logits,
                             scratch.partial_output, Dtype.Float32, rank_out, rank_sum, rank_max)
            stream.synchronize()
        final = Buffer.new_zeroed(device, rows * d * 2)
        combine_partials(device, stream, ranks, rows, d, all_sum, all_max, all_out, Dtype.Bfloat16, final)
        stream.synchronize()
        assert device.check(stream) == 0
        got = bits_to_f32("bf16", final.read(0, rows * d, np.uint16)).reshape(1, hq, d)
        assert_within_contract(got, expected, f"{ranks} ranks")


def test_invalid_arguments_are_reported_not_launched(device):
    from khalamari_b200 import abi, sliced_kv
    from khalamari_b200.device import Buffer, Dtype, Stream
    from khalamari_b200.request_page_table import GQAPageTableLayout
    from khalamari_b200.sdpa import ExecutionVariant
    layout = GQAPageTableLayout(1, 1, 4, 1)
    config = sliced_kv.Config(16, 2, 128, 0.5, 2 * 2 * 16 * 128 * 2, layout, Dtype.Bfloat16)
    shape = sliced_kv.Shape(2, 4)
    execution = ExecutionVariant.sliced_kv(config.sdpa_config(), 128, 128, 8)
    compute = sliced_kv.Compute(device, config, execution, shape)
    scratch = sliced_kv.Scratch(device, config, shape)
    stream = Stream(device)
    small = Buffer.new_zeroed(device, 16)
    good = dict(q=Buffer.new_zeroed(device, config.q_bytes(shape)), kv=Buffer.new_zeroed(device, config.page_bytes * 4),
                slots=Buffer.new_zeroed(device, 8), ids=Buffer.new_zeroed(device, 16),
                templates=Buffer.new_zeroed(device, 48))
    with pytest.raises(abi.InvalidArgument, match="q buffer"):
        compute.invoke_map(stream, scratch.map_buffers(small, good["kv"], good["slots"], good["ids"],
                                                       good["templates"]), 0, 1, 1)
    with pytest.raises(abi.InvalidArgument, match="num_active_tokens"):
        compute.invoke_map(stream, scratch.map_buffers(good["q"], good["kv"], good["slots"], good["ids"],
                                                       good["templates"]), 0, 3, 1)
    with pytest.raises(abi.InvalidArgument, match="page_table_index"):
        compute.invoke_map(stream, scratch.map_buffers(good["q"], good["kv"], good["slots"], good["ids"],
                                                       good["templates"]), 1, 1, 1)
    with pytest.raises(abi.InvalidArgument):
        sliced_kv.Compute(device, sliced_kv.Config(16, 2, 64, 0.5, 2 * 2 * 16 * 64 * 2, layout, Dtype.Bfloat16),
                          ExecutionVariant.sliced_kv(config.sdpa_config(), 128, 128, 8), shape)
    with pytest.raises(abi.InvalidArgument, match="shader u32 count domain"):
        sliced_kv.Config(2, 1, 2, 1.0, 8, GQAPageTableLayout(1, 1, 1, 1), Dtype.Bfloat16,
                         ).sizes(sliced_kv.Shape(1 << 30, 1))
    assert device.check(stream) == 0


def test_page_id_beyond_pool_sets_status_word(device):
    """A block-table entry that points past the KV pool reads zeros (the tensor map bounds the copy) and
    raises the sticky status word, the analogue of the reference's SubmissionCheck."""
    from khalamari_b200 import abi
    case = make_case(13, "bf16", 16, 2, 128, [99], [1])
    run = DeviceCase(device, case)
    base = case.req_slots[0] * case.layout.num_blocks
    bad = case.page_ids.copy()
    bad[base + 2] = 1 << 20
    run.page_ids.write(0, bad)
    run.attention.prepare(case.req_slots, case.token_indices, case.cu_tokens)
    run.attention.record_sdpa(run.stream, run.q, run.kv_pages, run.page_ids, run.output)
    with pytest.raises(abi.KhError) as info:
        device.check(run.stream)
    assert info.value.code == 5 and "beyond the KV pool" in str(info.value)
    assert device.check(run.stream) == 0  # the word is cleared by the read


def test_metadata_upload_matches_host_images(device):
    """GQAMetadataBuffers::update uploads exactly the host images (batch_metadata.rs:366-394)."""
    from khalamari_b200.batch_metadata import GQAMetadataBuffers
    from khalamari_b200.device import Dtype
    from khalamari_b200.replay import GQAReplayBucketPolicy, GQAReplayShape
    from khalamari_b200.sdpa import Config, ExecutionVariant, Registry
    from khalamari_b200.selector import RequestShape, Selector
    cfg = Config(Dtype.Bfloat16, 2, 2, 128, 8)
    variant = ExecutionVariant.sliced_kv(cfg, 8, 32, 1)
    selector = Selector.new(Registry.from_variants(cfg, [variant]), 8, 8, 8)
    meta = GQAMetadataBuffers(device, 8, 8)
    selection = selector.select(RequestShape.from_batch([7, 20], [0, 2, 5]), GQAReplayBucketPolicy(8, 8), 5)
    shape = meta.update([2, 5], [7, 20], [0, 2, 5], selection)
    assert shape == GQAReplayShape.new(5, 5, 5, 6, 8, 8, True)
    assert meta.req_slots().read_typed(0, 5).tolist() == [2, 2, 5, 5, 5]
    assert meta.flat_token_indices().read_typed(0, 5).tolist() == [7, 8, 20, 21, 22]
    assert meta.visible_kv_token_ranges().read_typed(0, 10).tolist() == [0, 8, 0, 9, 0, 21, 0, 22, 0, 23]
    assert meta.sdpa_map_task_templates().read_typed(0, 24).tolist() == [
        0, 0, 8, 1, 0, 9, 2, 0, 8, 2, 8, 21, 3, 0, 8, 3, 8, 22, 4, 0, 8, 4, 8, 23]
    assert meta.cu_sdpa_partial_outputs().read_typed(0, 6).tolist() == [0, 1, 2, 4, 6, 8]


def test_page_table_lifecycle(device):
    """request_page_table.rs:179-213."""
    from khalamari_b200 import abi
    from khalamari_b200.request_page_table import GQAPageTableLayout, GQARequestPageTable
    table = GQARequestPageTable(device, GQAPageTableLayout(4, 3, 6, 2))
    table.write_page_ids(1, 0, 0, [10, 11])
    table.write_page_ids(1, 0, 1, [12, 13])
    table.write_page_ids(1, 2, 0, [20, 21])
    table.write_page_ids(2, 1, 0, [30, 31])
    table.write_page_ids(3, 0, 0, [40, 41])
    assert table.read_page_ids(1, 0, 0) == [10, 11] and table.read_page_ids(1, 0, 1) == [12, 13]
    assert table.read_page_ids(1, 2, 0) == [20, 21]
    table.reset_req_slot(1)
    assert table.read_page_ids(1, 0, 0) == [0, 0] and table.read_page_ids(1, 2, 0) == [0, 0]
    assert table.read_page_ids(2, 1, 0) == [30, 31] and table.read_page_ids(3, 0, 0) == [40, 41]
    with pytest.raises(abi.InvalidArgument, match="req_slot out of range"):
        table.write_page_ids(4, 0, 0, [1, 2])
    with pytest.raises(abi.InvalidArgument, match="page-id count"):
        table.write_page_ids(0, 0, 0, [1])
