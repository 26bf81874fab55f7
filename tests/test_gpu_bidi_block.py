"""BiDi-block SDPA (``-m gpu``): the block kernel alone and the composite with sliding-window history partials
through the sliced-Q map kernel and the shared reducer. Scenarios of
crates/inference-backend-metal/src/components/gqa/bidi_block_sdpa_test.rs:41-330, checked against the CPU oracle:
the block partial against ``partial_row`` (one split-KV partial over the block's rows), the composite against
``projected_gqa`` over each token's visible history rows followed by its block's rows."""
import numpy as np
import pytest

import oracle
from helpers import assert_within_contract, bits_to_f32, round_to

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    from khalamari_b200.device import Device
    return Device(0)


def _store(device, values, dtype_name):
    from khalamari_b200.device import Buffer
    if dtype_name == "f32":
        return Buffer.from_slice(device, np.ascontiguousarray(values, np.float32)), np.asarray(values, np.float32)
    bits, rounded = round_to(dtype_name, np.asarray(values, np.float32))
    return Buffer.from_slice(device, bits), rounded


def _dtype(dtype_name):
    from khalamari_b200.device import Dtype
    return {"f32": Dtype.Float32, "bf16": Dtype.Bfloat16, "f16": Dtype.Float16}[dtype_name]


@pytest.mark.parametrize("dtype_name", ["f32", "bf16", "f16"])
def test_block_kernel_matches_the_oracle_partial(device, dtype_name):
    """bidi_block_sdpa_test.rs:41-49, 331-420: block size 3, two ranges of one block each, 5 Q heads on 1 KV head,
    head_dim 32; the block partial of range r lands in slot cu[r + 1] - 1."""
    from khalamari_b200 import bidi_block_sdpa as bidi
    from khalamari_b200.device import Buffer, Stream
    config = bidi.Config(3, 8, 5, 1, 32, 32.0 ** -0.5, _dtype(dtype_name))
    shape = bidi.Shape(6, 2, 8)
    q_buf, q = _store(device, np.arange(config.q_elements(shape)) * 0.03125 - 0.4, dtype_name)
    k_buf, k = _store(device, np.arange(config.kv_elements(shape)) * -0.025 + 0.3, dtype_name)
    v_buf, v = _store(device, np.arange(config.kv_elements(shape)) * 0.05 - 0.2, dtype_name)
    stats = config.partial_output_stat_elements(shape)
    sums = Buffer.from_slice(device, np.full(stats, -7.0, np.float32))
    maxes = Buffer.from_slice(device, np.full(stats, -7.0, np.float32))
    outs = Buffer.from_slice(device, np.full(stats * 32, -7.0, np.float32))
    stream = Stream(device)
    bidi.Compute(device, config).invoke(stream, shape, 2, bidi.Buffers(
        q_buf, k_buf, v_buf, Buffer.from_slice(device, np.array([0, 3, 3, 6], np.uint32)),
        Buffer.from_slice(device, np.array([0, 1, 2], np.uint32)), sums, maxes, outs))
    stream.synchronize()
    assert device.check(stream) == 0
    got_sum = sums.read(0, stats, np.float32).reshape(8, 5, 8)
    got_max = maxes.read(0, stats, np.float32).reshape(8, 5, 8)
    got_out = outs.read(0, stats * 32, np.float32).reshape(8, 5, 8, 32)
    q, k, v = q.reshape(6, 5, 32), k.reshape(6, 1, 32), v.reshape(6, 1, 32)
    for token in range(6):
        slot, offset, block = token // 3, token % 3, token // 3 * 3
        for head in range(5):
            out, exp_sum, max_logit = oracle.partial_row(q[token, head], k, v, block, block + 3, 1, 32, 0, config.scale)
            assert abs(got_max[slot, head, offset] - max_logit) < 1e-4
            assert abs(got_sum[slot, head, offset] - exp_sum) < 1e-4 * max(1.0, exp_sum)
            assert np.max(np.abs(got_out[slot, head, offset] - out)) < 1e-4
    # nothing outside the two block slots was written
    assert np.all(got_sum[2:] == -7.0) and np.all(got_sum[:2, :, 3:] == -7.0)


def test_replayed_active_range_counts(device):
    """bidi_block_sdpa_test.rs:51-157: one recorded launch, the active Q-token-range count read on the device."""
    from khalamari_b200 import bidi_block_sdpa as bidi
    from khalamari_b200.device import Buffer, Dtype, Stream
    n, d = 8, 32
    config = bidi.Config(n, 1, 1, 1, d, d ** -0.5, Dtype.Float32)
    shape = bidi.Shape(n, n, n)
    q = (np.arange(n * d) * 0.003 - 0.4).astype(np.float32)
    k = (np.arange(n * d) * -0.002 + 0.3).astype(np.float32)
    v = (np.arange(n * d) * 0.004 - 0.2).astype(np.float32)
    ranges = np.array([[i, i + 1] for i in range(n)], np.uint32).reshape(-1)
    stream = Stream(device)
    counts = Buffer.new_zeroed(device, 16)
    compute = bidi.Compute(device, config)
    sums, maxes = Buffer.new_zeroed(device, n * 4), Buffer.new_zeroed(device, n * 4)
    outs = Buffer.new_zeroed(device, n * d * 4)
    buffers = bidi.Buffers(Buffer.from_slice(device, q), Buffer.from_slice(device, k), Buffer.from_slice(device, v),
                           Buffer.from_slice(device, ranges), Buffer.from_slice(device, np.arange(n + 1, dtype=np.uint32)),
                           sums, maxes, outs)
    for active in [1, 8, 3, 7, 2, 6, 4, 5]:
        outs.zero_bytes(0, n * d * 4)
        counts.write(0, np.array([n, active, 0, 0], np.uint32))
        stream.bind_active_counts(counts)
        compute.invoke(stream, shape, n, buffers)  # recorded with the capacity; the device word decides
        stream.bind_active_counts(None)
        stream.synchronize()
        got = outs.read(0, n * d, np.float32).reshape(n, d)
        for token in range(n):
            if token < active:
                out, _, _ = oracle.partial_row(q[token * d:(token + 1) * d], k, v, 0, n, 1, d, 0, config.scale)
                assert np.max(np.abs(got[token] - out)) < 1e-4
            else:
                assert not got[token].any(), "an inactive range was written"


@pytest.mark.parametrize("windows", [[0] * 7, [4, 5, 6, 7, 8, 9, 10, 11]])
@pytest.mark.parametrize("page,kv_fp8", [(8, False), (16, False), (16, True)])
def test_history_and_block_composite(device, windows, page, kv_fp8):
    """bidi_block_sdpa_test.rs:159-330: history partials from the sliced-Q map kernel (per-token sliding windows
    [begin, 12) over 16 cached tokens, two history tasks), the block partial in the range's last slot, one reduce.
    History and block maxima are close but distinct, which makes the result sensitive to the log base of the shared
    statistics."""
    from khalamari_b200 import bidi_block_sdpa as bidi, sliced_q
    from khalamari_b200.device import Buffer, Dtype, Stream
    from khalamari_b200.request_page_table import GQAPageTableLayout
    from khalamari_b200.sdpa import ExecutionVariant
    from helpers import fp8_codes
    tokens, history, hq, hkv, d = len(windows), 16, 5, 1, 128
    scale = d ** -0.5
    kv_dtype = Dtype.Fp8E4M3FN if kv_fp8 else Dtype.Bfloat16
    elem = 1 if kv_fp8 else 2
    layout = GQAPageTableLayout(1, 1, 2, 1)
    config = sliced_q.Config(hq, hkv, d, scale, 2 * hkv * page * d * elem, Dtype.Bfloat16, layout, kv_dtype)
    execution = ExecutionVariant.sliced_q_per_head(config.sdpa_config(), 8, 16, 5)
    q_shape = sliced_q.Shape(tokens, 1, 4)
    rng = np.random.default_rng(91)
    # the reference's constants, plus a little noise so that every token and column differs
    q_vals = 1.0 + 0.05 * rng.standard_normal((tokens, hq, d)).astype(np.float32)
    hist_k = 0.17677669 + 0.02 * rng.standard_normal((history, hkv, d)).astype(np.float32)
    hist_v = 1.0 + 0.1 * rng.standard_normal((history, hkv, d)).astype(np.float32)
    local_k = 0.22097087 + 0.02 * rng.standard_normal((tokens, hkv, d)).astype(np.float32)
    local_v = -1.0 + 0.1 * rng.standard_normal((tokens, hkv, d)).astype(np.float32)
    q_buf, q_r = _store(device, q_vals, "bf16")
    lk_buf, lk_r = _store(device, local_k, "bf16")
    lv_buf, lv_r = _store(device, local_v, "bf16")
    # FP8 pages: the reference's cache format; the oracle sees the decoded codes (sliced_kv_test.rs:171-182)
    hk_bits, hk_r = fp8_codes(hist_k) if kv_fp8 else round_to("bf16", hist_k)
    hv_bits, hv_r = fp8_codes(hist_v) if kv_fp8 else round_to("bf16", hist_v)
    pool = np.zeros(2 * config.page_bytes, np.uint8)
    table = np.array([1, 0], np.uint32)  # descending physical pages
    oracle.scatter_paged(pool, table, oracle.PageTableLayout(1, 1, 2, 1), 0, 0, page, hkv, d, elem, 0, hk_bits, hv_bits)
    visible = np.array([[w, 12] for w in windows], np.uint32).reshape(-1)
    stream = Stream(device)
    sizes = config.sizes(execution, q_shape)
    d_po = Buffer.new_zeroed(device, sizes.partial_output_bytes)
    d_ps = Buffer.new_zeroed(device, sizes.partial_output_stats_bytes)
    d_pm = Buffer.new_zeroed(device, sizes.partial_output_stats_bytes)
    d_ranges = Buffer.from_slice(device, np.array([0, tokens], np.uint32))
    d_cu = Buffer.from_slice(device, np.array([0, 3], np.uint32))
    d_out = Buffer.new_zeroed(device, tokens * hq * d * 2)
    templates = np.array([0, 0, 4, 0, 4, 12] + [0xFFFFFFFF] * 6, np.uint32)
    history_map = sliced_q.Compute(device, config, execution, q_shape)
    history_map.invoke_map(stream, sliced_q.MapBuffers(
        q_buf, Buffer.from_slice(device, pool), Buffer.from_slice(device, np.zeros(tokens, np.uint32)),
        Buffer.from_slice(device, table), Buffer.from_slice(device, visible), d_ranges,
        Buffer.from_slice(device, templates), d_po, d_ps, d_pm), 0, tokens, 1, 3)
    block_config = bidi.Config(tokens, 8, hq, hkv, d, scale, Dtype.Bfloat16)
    bidi.Compute(device, block_config).invoke(stream, bidi.Shape(tokens, 1, 4), 1, bidi.Buffers(
        q_buf, lk_buf, lv_buf, d_ranges, d_cu, d_ps, d_pm, d_po))
    history_map.invoke_reduce(stream, sliced_q.ReduceBuffers(d_po, d_ps, d_pm, d_ranges, d_cu, d_out), 1)
    stream.synchronize()
    assert device.check(stream) == 0
    actual = bits_to_f32("bf16", d_out.read(0, tokens * hq * d, np.uint16)).reshape(tokens, hq, d)
    # oracle: every token is a request of its own whose context is its visible history rows, then its block's rows
    ks = [np.concatenate([hk_r[w:12], lk_r]) for w in windows]
    vs = [np.concatenate([hv_r[w:12], lv_r]) for w in windows]
    expected = oracle.projected_gqa(list(range(tokens + 1)), [len(k) - 1 for k in ks], q_r, ks, vs, d, hq, hkv, scale)
    assert_within_contract(actual, expected, f"history + block composite, windows {windows}")
