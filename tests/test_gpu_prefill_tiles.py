"""Large Q tiles (more than 64 (token, head) rows per task at head_dim 128): the instance that runs Q K^T and
P V on tcgen05 with tensor-memory accumulators (``-m gpu``). Causal chunked prefill against the CPU oracle with
split and direct output, ragged chunks, KV ranges that end inside a page, fp16, and a short-context case where
every probability is large."""
import numpy as np
import pytest

from helpers import DeviceCase, assert_within_contract, make_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    from khalamari_b200.device import Device
    return Device(0)


def _forced(case, dtype, variant, max_tokens, max_maps):
    from khalamari_b200.sdpa import Config, Registry
    from khalamari_b200.selector import Selector
    cfg = Config(dtype, case.num_q_heads, case.num_kv_heads, case.head_dim, case.tokens_per_page)
    return Selector.new(Registry.from_variants(cfg, [variant]), max_tokens, max_maps,
                        max_maps * variant.thread_block.max_q_tokens)


@pytest.mark.parametrize("dtype_name", ["bf16", "f16"])
def test_policy_routes_prefill_chunks_to_128_row_tiles(device, dtype_name):
    """Hq64/Hkv8: the B200 policy picks 16 tokens x 8 heads = 128 rows per task."""
    histories, q_lens = [0, 100, 517, 33], [64, 33, 16, 1]
    case = make_case(51, dtype_name, 64, 8, 128, histories, q_lens)
    run = DeviceCase(device, case, max_tokens=128)
    out = run.run(fused=False)
    variant = run.attention.metadata.variant()
    assert variant.thread_block.max_q_tokens * variant.thread_block.max_q_heads == 128
    assert_within_contract(out, case.oracle_output(), f"prefill tiles {dtype_name}")


@pytest.mark.parametrize("kv_slice,direct", [(16, False), (48, False), (512, False), (4096, True)])
@pytest.mark.parametrize("ratio,tile", [(8, 16), (4, 32), (6, 16)])
def test_forced_tiles_split_and_direct(device, kv_slice, direct, ratio, tile):
    """Slices of one page, of three pages (boundaries inside a stage), long slices, and direct output; a group of
    six heads leaves rows 96-127 of the tile without a (token, head)."""
    from khalamari_b200.device import Dtype
    from khalamari_b200.sdpa import Config, ExecutionVariant, MapKernelKind
    hkv = 2
    hq = hkv * ratio
    histories, q_lens = [70, 5, 0], [tile + 3, 2 * tile, 7]
    case = make_case(52, "bf16", hq, hkv, 128, histories, q_lens)
    cfg = Config(Dtype.Bfloat16, hq, hkv, 128, 16)
    variant = ExecutionVariant.sliced_q(cfg, MapKernelKind.QTokensAndHeads, tile, 16, ratio)
    selector = _forced(case, Dtype.Bfloat16, variant, 128, 256)
    run = DeviceCase(device, case, max_tokens=128, selector=selector)
    selection = run.attention.select_partitioned(variant, kv_slice, direct, case.token_indices, case.cu_tokens)
    out = run.run(selection)
    assert_within_contract(out, case.oracle_output(), f"tile {tile}x{ratio} slice {kv_slice} direct {direct}")


def test_long_prefix_and_growing_maxima(device):
    """A 3,000-token prefix with keys scaled so that row maxima keep growing along the context: exercises the
    lazy rescale of the accumulator in tensor memory."""
    histories, q_lens = [3000], [48]
    case = make_case(53, "bf16", 64, 8, 128, histories, q_lens, scale=0.35, q_std=1.5)
    out = DeviceCase(device, case, max_tokens=64).run(fused=False)
    assert_within_contract(out, case.oracle_output(), "growing maxima")


def test_matches_the_warp_level_instance(device):
    """The one-launch form runs the warp-level instance on the same batch; both must agree (DeviceCase.run)."""
    histories, q_lens = [257, 31], [40, 24]
    case = make_case(54, "bf16", 64, 8, 128, histories, q_lens)
    out = DeviceCase(device, case, max_tokens=64).run()
    assert_within_contract(out, case.oracle_output(), "tensor-memory vs warp-level")
