"""8-token pages (``-m gpu``): the other page size of the reference's tile profiles (128 x {8, 16},
256 x {8, 16, 32}; crates/inference-backend-metal/src/components/gqa/sdpa.rs:105-160). Same parity bar as the
16-token cases: decode with slices that end inside pages, verify, prefill tiles, two page ids per block."""
import pytest

from helpers import DeviceCase, assert_within_contract, make_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    from khalamari_b200.device import Device
    return Device(0)


@pytest.mark.parametrize("dtype_name,hq,hkv,d", [("bf16", 64, 8, 128), ("bf16", 16, 2, 256), ("f16", 24, 4, 256)])
def test_decode_on_8_token_pages(device, dtype_name, hq, hkv, d):
    contexts = [1, 7, 8, 9, 63, 64, 65, 500, 1029, 2500]
    case = make_case(71, dtype_name, hq, hkv, d, [c - 1 for c in contexts], [1] * len(contexts), tokens_per_page=8,
                     num_page_ids_per_block=2)
    out = DeviceCase(device, case).run()
    assert_within_contract(out, case.oracle_output(), f"decode P8 {dtype_name} D{d}")


@pytest.mark.parametrize("kv_slice", [8, 20, 256])
def test_forced_slices_on_8_token_pages(device, kv_slice):
    from khalamari_b200.device import Dtype
    from khalamari_b200.sdpa import Config, ExecutionVariant, Registry
    from khalamari_b200.selector import Selector
    contexts = [300, 33, 700]
    case = make_case(72, "bf16", 64, 8, 128, [c - 1 for c in contexts], [1] * 3, tokens_per_page=8)
    cfg = Config(Dtype.Bfloat16, 64, 8, 128, 8)
    variant = ExecutionVariant.sliced_kv(cfg, 128, 128, 8)
    selector = Selector.new(Registry.from_variants(cfg, [variant]), 8, 256, 256)
    run = DeviceCase(device, case, max_tokens=8, selector=selector)
    selection = run.attention.select_partitioned(variant, kv_slice, False, case.token_indices, case.cu_tokens)
    assert_within_contract(run.run(selection), case.oracle_output(), f"P8 slice {kv_slice}")


@pytest.mark.parametrize("hq,hkv,d,q_lens", [(24, 4, 256, [4, 4, 2]), (64, 8, 128, [40, 17, 1])])
def test_verify_and_prefill_on_8_token_pages(device, hq, hkv, d, q_lens):
    histories = [130, 7, 900]
    case = make_case(73, "bf16", hq, hkv, d, histories, q_lens, tokens_per_page=8)
    out = DeviceCase(device, case, max_tokens=64).run()
    assert_within_contract(out, case.oracle_output(), f"P8 q_lens {q_lens}")
