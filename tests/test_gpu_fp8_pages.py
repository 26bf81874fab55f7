"""Attention over K/V pages of FP8 E4M3FN codes, the reference's cache format (one byte per stored element,
components/gqa/sdpa/sliced_kv.rs:118; decoded on load by metal/gqa_fp8.metal:1-25).

The pool holds the codes the reference's page write produces (bf16 rounding, then components/gqa/fp8.rs:19-44);
the oracle computes on their decoded values, as sliced_kv_test.rs:171-182 and sliced_q_test.rs do. Decoding is
exact, so the bound is the contract's: per element 2e-3 absolute or 1e-2 relative."""
import numpy as np
import pytest

from helpers import DeviceCase, assert_within_contract, make_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    from khalamari_b200.device import Device
    return Device(0)


def _check(device, case, what, fused=False):
    run = DeviceCase(device, case)
    actual = run.run(fused=fused)
    return assert_within_contract(actual, case.oracle_output(), what)


@pytest.mark.parametrize("dtype_name", ["bf16", "f16"])
@pytest.mark.parametrize("heads", [(64, 8, 128), (16, 2, 256), (32, 8, 128)])
def test_decode_over_fp8_pages(device, dtype_name, heads):
    hq, hkv, d = heads
    contexts = [3000, 17, 1024, 1, 2500, 640, 16, 33]
    case = make_case(501, dtype_name, hq, hkv, d, [c - 1 for c in contexts], [1] * len(contexts), kv_fp8=True)
    _check(device, case, f"fp8 decode {dtype_name} {heads}")


@pytest.mark.parametrize("dtype_name", ["bf16", "f16"])
def test_subnormal_and_saturated_codes(device, dtype_name):
    """Values around 2^-6 (the smallest normal) land on FP8 subnormals, values beyond 448 saturate to 0x7e; Q is
    small so that the logits stay in range."""
    small = make_case(502, dtype_name, 16, 2, 128, [700, 95], [1, 1], kv_fp8=True, kv_std=0.01)
    codes = small.pool[small.pool != 0x7F]
    assert np.count_nonzero((codes & 0x78) == 0) > codes.size // 4, "the fixture must exercise subnormal codes"
    _check(device, small, f"fp8 subnormal codes {dtype_name}")
    large = make_case(503, dtype_name, 16, 2, 128, [300, 40], [1, 1], kv_fp8=True, kv_std=200.0, q_std=0.002)
    assert np.count_nonzero((large.pool & 0x7F) == 0x7E) > 0, "the fixture must exercise the saturated code"
    run = DeviceCase(device, large)
    actual = run.run(fused=False)
    expected = large.oracle_output()
    # outputs are sums of values up to 448: the relative bound is the one that applies
    assert_within_contract(actual / 448.0, expected / 448.0, f"fp8 saturated codes {dtype_name}")


@pytest.mark.parametrize("q_len,heads", [(4, (48, 8, 128)), (4, (64, 8, 128)), (8, (64, 8, 128)), (4, (16, 2, 256)),
                                         (2, (64, 8, 128))])
def test_verify_tiles_over_fp8_pages(device, q_len, heads):
    """Speculative-verify batches: several new tokens per request, causal within the new tokens (row tiles of 12 to
    64 rows: every warp-level consumer shape)."""
    hq, hkv, d = heads
    histories = [2000, 0, 513, 77, 1290]
    case = make_case(504, "bf16", hq, hkv, d, histories, [q_len] * len(histories), kv_fp8=True)
    _check(device, case, f"fp8 verify q{q_len} {heads}")


def test_chunked_prefill_over_fp8_pages(device):
    """Prefill chunks of 64 and 200 new tokens over a cached prefix: 128-row tiles (eight row tiles per task)."""
    case = make_case(505, "bf16", 16, 2, 128, [1000, 0], [64, 200], kv_fp8=True)
    _check(device, case, "fp8 chunked prefill")


def test_one_launch_form_over_fp8_pages(device):
    case = make_case(506, "bf16", 64, 8, 128, [c - 1 for c in [4000, 900, 60]], [1, 1, 1], kv_fp8=True)
    run = DeviceCase(device, case)
    actual = run.run(fused=None)  # both forms, compared with each other inside
    assert_within_contract(actual, case.oracle_output(), "fp8 one-launch form")


def test_page_write_then_attention(device):
    """The library's own FP8 page write feeds the attention: K/V rows (bf16) are written token by token into an
    empty pool through kh_kv_page_write_invoke, then the decode runs over those pages; the oracle sees the values
    the codec gives for the same rows."""
    from khalamari_b200 import kv_page_write
    from khalamari_b200.device import Buffer
    from helpers import fp8_codes, round_to

    contexts = [300, 45, 1000]
    case = make_case(507, "bf16", 32, 8, 128, [c - 1 for c in contexts], [1] * 3, kv_fp8=True)
    run = DeviceCase(device, case)
    # an empty pool (all NaN codes), then every token of every request written by the kernel
    pool_bytes = case.pool.size
    run.kv_pages = Buffer.from_slice(device, np.full(pool_bytes, 0x7F, dtype=np.uint8))
    rng = np.random.default_rng(99)
    config = kv_page_write.Config(case.num_kv_heads, case.head_dim, case.page_bytes)  # bf16 rows, FP8 pages
    total = sum(contexts)
    k = rng.standard_normal((total, case.num_kv_heads, case.head_dim), dtype=np.float32)
    v = rng.standard_normal((total, case.num_kv_heads, case.head_dim), dtype=np.float32)
    k_bits, _ = round_to("bf16", k)
    v_bits, _ = round_to("bf16", v)
    slots, tokens = [], []
    for r, ctx in enumerate(contexts):
        slots += [case.req_slots[r]] * ctx
        tokens += list(range(ctx))
    kv_page_write.Compute(device, config).invoke(
        run.stream, kv_page_write.Shape(total, run.layout),
        kv_page_write.Buffers(run.kv_pages, Buffer.from_slice(device, k_bits.reshape(-1)),
                              Buffer.from_slice(device, v_bits.reshape(-1)),
                              Buffer.from_slice(device, np.asarray(slots, dtype=np.uint32)),
                              Buffer.from_slice(device, np.asarray(tokens, dtype=np.uint32)), run.page_ids),
        total, case.layer_index)
    run.stream.synchronize()
    assert device.check(run.stream) == 0
    begin = 0
    case.k_f32, case.v_f32 = [], []
    for ctx in contexts:
        case.k_f32.append(fp8_codes(k[begin:begin + ctx])[1])
        case.v_f32.append(fp8_codes(v[begin:begin + ctx])[1])
        begin += ctx
    actual = run.run(fused=False)
    assert_within_contract(actual, case.oracle_output(), "fp8 page write then attention")
