"""Pins the CPU oracle to the reference's own known-answer tests and checks the paged gather."""
import math

import numpy as np
import pytest

import oracle


def test_causal_attention_known_answer():
    # crates/inference-executor-core/src/attn/gqa/reference.rs:84-115
    out = oracle.projected_gqa([0, 2], [0], [1.0, 0.0, 1.0, 0.0, 0.0, 2.0, 0.0, 2.0], [[1.0, 0.0, 0.0, 1.0]],
                               [[10.0, 0.0, 0.0, 20.0]], head_dim=2, num_q_heads=2, num_kv_heads=1, scale=1.0)
    f = np.float32
    first = f(np.exp(f(-2.0)))  # the reference computes its expectation in f32
    total = f(first + f(1.0))
    w1, w2 = f(first / total), f(f(1.0) / total)
    expected = [f(10.0), f(0.0), f(10.0), f(0.0), f(f(10.0) * w1), f(f(20.0) * w2), f(f(10.0) * w1), f(f(20.0) * w2)]
    assert np.all(np.abs(out.reshape(-1) - np.array(expected, dtype=np.float32)) < 1.0e-6)


def test_softmax_known_answer():
    # crates/inference-executor-core/src/reference.rs:102-108
    out = oracle.softmax(np.array([0.0, math.log(3.0)], dtype=np.float32))
    assert abs(out[0] - 0.25) < 1.0e-6 and abs(out[1] - 0.75) < 1.0e-6


def test_softmax_rejects_empty_and_non_finite():
    with pytest.raises(AssertionError):
        oracle.softmax(np.zeros(0, dtype=np.float32))
    with pytest.raises(AssertionError):
        oracle.softmax(np.array([np.inf], dtype=np.float32))


def test_validation_matches_core_validate():
    # GQACore::validate (core.rs:33-41): Hq % Hkv == 0, scale > 0
    with pytest.raises(AssertionError):
        oracle.projected_gqa([0, 1], [0], np.zeros(6), [np.zeros(4)], [np.zeros(4)], 2, 3, 2, 1.0)
    with pytest.raises(AssertionError):
        oracle.projected_gqa([0, 1], [0], np.zeros(4), [np.zeros(2)], [np.zeros(2)], 2, 2, 1, 0.0)


def test_threads_do_not_change_a_bit():
    rng = np.random.default_rng(3)
    hq, hkv, d = 8, 2, 32
    ctx = [37, 5]
    q = rng.standard_normal((3, hq, d)).astype(np.float32)
    ks = [rng.standard_normal((c, hkv, d)).astype(np.float32) for c in ctx]
    vs = [rng.standard_normal((c, hkv, d)).astype(np.float32) for c in ctx]
    a = oracle.projected_gqa([0, 2, 3], [35, 4], q, ks, vs, d, hq, hkv, 0.17, num_threads=1)
    b = oracle.projected_gqa([0, 2, 3], [35, 4], q, ks, vs, d, hq, hkv, 0.17, num_threads=4)
    assert np.array_equal(a.view(np.uint32), b.view(np.uint32))


def test_oracle_matches_float64_attention():
    rng = np.random.default_rng(11)
    hq, hkv, d, ctx = 4, 2, 16, 50
    q = rng.standard_normal((1, hq, d)).astype(np.float32)
    k = rng.standard_normal((ctx, hkv, d)).astype(np.float32)
    v = rng.standard_normal((ctx, hkv, d)).astype(np.float32)
    out = oracle.projected_gqa([0, 1], [ctx - 1], q, [k], [v], d, hq, hkv, 0.25)
    for h in range(hq):
        logits = (k[:, h // 2, :].astype(np.float64) @ q[0, h].astype(np.float64)) * 0.25
        p = np.exp(logits - logits.max())
        p /= p.sum()
        assert np.allclose(out[0, h], p @ v[:, h // 2, :].astype(np.float64), atol=1e-5)


def test_bf16_rounding_is_nearest_even():
    values = np.array([1.0, 1.00390625, 1.01171875, -2.5, 3.0e38, 0.0, 1.0000001], dtype=np.float32)
    bits, back = oracle.round_bf16(values)
    # 1.00390625 = 1 + 2^-8 is a tie between 0x3f80 and 0x3f81: even wins; 1.01171875 = 1 + 3*2^-8 ties up to 0x3f82
    assert bits.tolist()[:3] == [0x3F80, 0x3F80, 0x3F82]
    assert back[3] == -2.5 and back[5] == 0.0
    import torch
    t = torch.from_numpy(values).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(bits, t)


def test_generators_match_their_formulas():
    # sliced_kv_test.rs:501-509
    state = 0x8B1D5A73
    expect = []
    for _ in range(5):
        state = (state * 1664525 + 1013904223) & 0xFFFFFFFF
        expect.append(np.float32(np.float32(state >> 8) / np.float32(16777216.0)) * np.float32(2.0) - np.float32(1.0))
    assert np.array_equal(oracle.generated_values(5, 0x8B1D5A73), np.array(expect, dtype=np.float32))
    # sliced_kv_test.rs:495-499
    fix = oracle.fixture_values(6, 0.125, 3)
    assert np.array_equal(fix, np.array([((i * 11 + 3) % 23) * 0.125 - 11 * 0.125 for i in range(6)], np.float32))


def _build_pool(rng, layout, tokens_per_page, hkv, d, elem_bytes, num_pool_pages):
    return rng.integers(0, 256, size=num_pool_pages * 2 * hkv * tokens_per_page * d * elem_bytes, dtype=np.uint8)


def test_paged_gather_follows_the_page_formulas():
    # block = t/(P*n); i = (t/P)%n; idx = (((slot*L+layer)*B+block)*n+i);
    # addr = page*page_bytes + ((plane*Hkv+h)*P + t%P)*D*e   (gqa_sdpa_sliced_kv_map.metal:13-19)
    rng = np.random.default_rng(5)
    layout = oracle.PageTableLayout(num_req_slots=3, num_gqa_layers=2, num_blocks=4, num_page_ids_per_block=2)
    P, hkv, d, e = 4, 2, 8, 2
    pool_pages = 40
    pool = _build_pool(rng, layout, P, hkv, d, e, pool_pages)
    table = rng.permutation(pool_pages).astype(np.uint32)
    table = np.resize(table, layout.num_page_ids())
    n_tokens = 29
    k, v, ka, va = oracle.gather_paged(pool, table, layout, req_slot=2, layer_index=1, tokens_per_page=P,
                                       num_kv_heads=hkv, head_dim=d, elem_bytes=e, num_tokens=n_tokens,
                                       want_addresses=True)
    page_bytes = 2 * hkv * P * d * e
    for t in range(n_tokens):
        block, i = t // (P * 2), (t // P) % 2
        idx = (((2 * 2 + 1) * 4 + block) * 2) + i
        page = int(table[idx])
        for h in range(hkv):
            ak = page * page_bytes + ((0 * hkv + h) * P + t % P) * d * e
            av = page * page_bytes + ((1 * hkv + h) * P + t % P) * d * e
            assert ka[t, h] == ak and va[t, h] == av
            assert np.array_equal(k[t, h], pool[ak:ak + d * e])
            assert np.array_equal(v[t, h], pool[av:av + d * e])


def test_scatter_then_gather_round_trips_bytes():
    rng = np.random.default_rng(9)
    layout = oracle.PageTableLayout(2, 1, 5, 1)
    P, hkv, d, e = 16, 2, 32, 2
    pool = np.zeros(12 * 2 * hkv * P * d * e, dtype=np.uint8)
    table = np.zeros(layout.num_page_ids(), dtype=np.uint32)
    table[5:10] = [7, 3, 11, 0, 5]
    n = 70
    k = rng.integers(0, 65536, size=(n, hkv, d), dtype=np.uint16)
    v = rng.integers(0, 65536, size=(n, hkv, d), dtype=np.uint16)
    oracle.scatter_paged(pool, table, layout, 1, 0, P, hkv, d, e, 0, k, v)
    gk, gv = oracle.gather_paged(pool, table, layout, 1, 0, P, hkv, d, e, n)
    assert np.array_equal(gk.view(np.uint16).reshape(n, hkv, d), k)
    assert np.array_equal(gv.view(np.uint16).reshape(n, hkv, d), v)
    with pytest.raises(IndexError):
        oracle.gather_paged(pool, table, layout, 1, 0, P, hkv, d, e, 81)  # sixth block does not exist


def test_split_partials_merge_to_the_unsplit_oracle():
    # CPU-rank simulation of split-KV: N slices, one (max, sum, out) triple each, merged with the
    # reducer's formula (docs/gqa_sdpa_selection.md:443-460), equal the unsplit oracle.
    rng = np.random.default_rng(21)
    hkv, d, ctx = 2, 64, 1000
    q = rng.standard_normal(d).astype(np.float32)
    k = rng.standard_normal((ctx, hkv, d)).astype(np.float32)
    v = rng.standard_normal((ctx, hkv, d)).astype(np.float32)
    full = oracle.oracle_row(q, k, v, ctx, hkv, d, 1, 0.125)
    for ranks in (1, 2, 4, 8):
        bounds = [ctx * r // ranks for r in range(ranks + 1)]
        triples = [oracle.partial_row(q, k, v, bounds[r], bounds[r + 1], hkv, d, 1, 0.125) for r in range(ranks)]
        triples.append(oracle.partial_row(q, k, v, ctx, ctx, hkv, d, 1, 0.125))  # an empty slice is ignored
        out, s, m = oracle.merge_partials([t[1] for t in triples], [t[2] for t in triples],
                                          np.stack([t[0] for t in triples]))
        assert np.max(np.abs(out - full)) < 2e-6
        assert s > 0 and math.isfinite(m)
    out, s, m = oracle.merge_partials([0.0], [-np.inf], np.zeros((1, d), np.float32))
    assert s == 0.0 and m == -np.inf and not out.any()
