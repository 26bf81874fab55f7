"""32-token pages at head_dim 256 (``-m gpu``): the fifth (head_dim, tokens_per_page) profile of the reference's
sliced-Q kernels (128 x {8, 16}, 256 x {8, 16, 32}; crates/inference-backend-metal/src/components/gqa/sdpa.rs:162-215,
exercised for all five by sliced_q_test.rs:53-218). Same parity bar as the 16-token cases: decode with slices that
end inside pages, verify, prefill tiles, two page ids per block and a second GQA layer, the registry's own
variants, and the page write that fills such pages."""
import numpy as np
import pytest

from helpers import DeviceCase, assert_within_contract, make_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    from khalamari_b200.device import Device
    return Device(0)


@pytest.mark.parametrize("dtype_name,hq,hkv", [("bf16", 16, 2), ("f16", 24, 4), ("bf16", 8, 8)])
def test_decode_on_32_token_pages(device, dtype_name, hq, hkv):
    contexts = [1, 31, 32, 33, 63, 64, 65, 500, 1029, 2500]
    case = make_case(81, dtype_name, hq, hkv, 256, [c - 1 for c in contexts], [1] * len(contexts), tokens_per_page=32,
                     num_page_ids_per_block=2, num_gqa_layers=2, layer_index=1)
    out = DeviceCase(device, case).run()
    assert_within_contract(out, case.oracle_output(), f"decode P32 {dtype_name} Hq{hq}/Hkv{hkv}")


@pytest.mark.parametrize("kv_slice", [32, 50, 256])
def test_forced_slices_on_32_token_pages(device, kv_slice):
    from khalamari_b200.device import Dtype
    from khalamari_b200.sdpa import Config, ExecutionVariant, Registry
    from khalamari_b200.selector import Selector
    contexts = [300, 33, 700]
    case = make_case(82, "bf16", 16, 2, 256, [c - 1 for c in contexts], [1] * 3, tokens_per_page=32)
    cfg = Config(Dtype.Bfloat16, 16, 2, 256, 32)
    variant = ExecutionVariant.sliced_kv(cfg, 256, 128, 8)
    selector = Selector.new(Registry.from_variants(cfg, [variant]), 8, 256, 256)
    run = DeviceCase(device, case, max_tokens=8, selector=selector)
    selection = run.attention.select_partitioned(variant, kv_slice, False, case.token_indices, case.cu_tokens)
    assert_within_contract(run.run(selection), case.oracle_output(), f"P32 slice {kv_slice}")


@pytest.mark.parametrize("hq,hkv,q_lens", [(24, 4, [4, 4, 2]), (16, 2, [40, 17, 1]), (8, 2, [33, 2, 16])])
def test_verify_and_prefill_on_32_token_pages(device, hq, hkv, q_lens):
    histories = [130, 7, 900]
    case = make_case(83, "bf16", hq, hkv, 256, histories, q_lens, tokens_per_page=32)
    out = DeviceCase(device, case, max_tokens=64).run()
    assert_within_contract(out, case.oracle_output(), f"P32 q_lens {q_lens}")


def test_every_registry_variant_of_the_profile_runs(device):
    """Registry::new for (head_dim 256, 32-token pages) lists its legal variants (sdpa.rs:255-271); each of them,
    forced, must reproduce the oracle, split and (for the sliced-Q kinds) direct."""
    from khalamari_b200.device import Dtype
    from khalamari_b200.sdpa import Config, MapKernelKind, Registry
    from khalamari_b200.selector import Selector
    hq, hkv = 12, 2
    cfg = Config(Dtype.Bfloat16, hq, hkv, 256, 32)
    variants = Registry(cfg).variants()
    assert len(variants) >= 2
    for variant in variants:
        tile = variant.thread_block.max_q_tokens
        q_lens = [1, 1] if variant.kind == MapKernelKind.SlicedKv else [tile + 1 if tile > 1 else 3, 1]
        case = make_case(84, "bf16", hq, hkv, 256, [70, 3], q_lens, tokens_per_page=32)
        selector = Selector.new(Registry.from_variants(cfg, [variant]), 64, 128, 128 * max(tile, 1))
        for direct in ([False] if variant.kind == MapKernelKind.SlicedKv else [False, True]):
            run = DeviceCase(device, case, max_tokens=64, selector=selector)
            selection = run.attention.select_partitioned(variant, 4096 if direct else 32, direct, case.token_indices,
                                                         case.cu_tokens)
            out = run.run(selection)
            assert_within_contract(out, case.oracle_output(), f"P32 variant {variant} direct={direct}")


def test_page_write_then_attention_on_32_token_pages(device):
    """kv_page_write (kv_page_write.rs:169-236) into 32-token pages, then decode over what it wrote."""
    from khalamari_b200 import kv_page_write
    from khalamari_b200.device import Buffer, Dtype

    case = make_case(85, "bf16", 16, 2, 256, [99, 40], [1, 1], tokens_per_page=32, poison=False)
    run = DeviceCase(device, case)
    # rewrite the last 5 tokens of request 0 through the page-write kernel with new values, and tell the oracle
    rng = np.random.default_rng(850)
    import oracle
    new_k = rng.standard_normal((5, 2, 256), dtype=np.float32)
    new_v = rng.standard_normal((5, 2, 256), dtype=np.float32)
    k_bits, k_round = oracle.round_bf16(new_k)
    v_bits, v_round = oracle.round_bf16(new_v)
    compute = kv_page_write.Compute(device, kv_page_write.Config(2, 256, case.page_bytes, Dtype.Bfloat16, Dtype.Bfloat16))
    positions = np.arange(95, 100, dtype=np.uint32)
    buffers = kv_page_write.Buffers(run.kv_pages, Buffer.from_slice(device, k_bits), Buffer.from_slice(device, v_bits),
                                    Buffer.from_slice(device, np.full(5, case.req_slots[0], np.uint32)),
                                    Buffer.from_slice(device, positions), run.page_ids)
    compute.invoke(run.stream, kv_page_write.Shape(5, run.layout), buffers, 5, case.layer_index)
    case.k_f32[0][95:100] = k_round
    case.v_f32[0][95:100] = v_round
    out = run.run(fused=False)
    assert_within_contract(out, case.oracle_output(), "P32 page write then decode")
