"""``kh_sliced_kv_attend_static``: SlicedKv map + reduce with the partial state in the array the library holds.

Collected last (file name) so that it runs after every other GPU test has used the device, and it also passes
when run alone. The entry point is called through the C ABI and compared, bit for bit, with
``kh_sliced_kv_map`` + ``kh_sliced_kv_reduce`` on caller-owned partial buffers, on two different batches in a
row (the second call finds the first call's partials in the shared array)."""
import numpy as np
import pytest

from helpers import DeviceCase, assert_within_contract, make_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    from khalamari_b200.device import Device
    return Device(0)


def _run_both(device, case):
    """Returns (output through caller-owned partial buffers, output through the shared array)."""
    from khalamari_b200 import sdpa, sliced_kv

    run = DeviceCase(device, case)
    attention = run.attention
    attention.prepare(case.req_slots, case.token_indices, case.cu_tokens)
    meta = attention.metadata
    assert meta.variant().kind == sdpa.MapKernelKind.SlicedKv
    expected = run.run(fused=False)

    shape = meta.replay_shape()
    compute = attention._sliced_kv(shape, meta.variant())
    needed = compute.static_bytes_needed(shape.num_sdpa_map_task_templates)
    from khalamari_b200 import abi
    assert 0 < needed <= abi.STATIC_PARTIALS_BYTES
    run.output.write(0, np.full(run.out_rows * case.num_q_heads * case.head_dim, run.canary, dtype=np.uint16))
    compute.invoke_attend_static(
        run.stream,
        sliced_kv.StaticBuffers(run.q, run.kv_pages, meta.req_slots(), run.page_ids, meta.sdpa_map_task_templates(),
                                meta.cu_sdpa_partial_outputs(), run.output),
        case.layer_index, shape.num_tokens, shape.num_sdpa_map_task_templates)
    run.stream.synchronize()
    assert device.check(run.stream) == 0
    return expected, run.read_output()


def test_two_calls_in_a_row_match_the_caller_buffer_path(device):
    first = make_case(41, "bf16", 64, 8, 128, [c - 1 for c in [3000, 17, 1024, 2500, 640]], [1] * 5)
    second = make_case(42, "f16", 16, 2, 256, [c - 1 for c in [900, 4100, 33]], [1] * 3)
    for case in (first, second):
        expected, actual = _run_both(device, case)
        assert np.array_equal(expected, actual), "shared-array result differs from the caller-buffer result"
        assert_within_contract(actual, case.oracle_output(), "shared-array attention")


def test_a_batch_beyond_the_shared_array_is_refused(device):
    """50 requests x 64 slices x 64 heads x (128 + 2) floats = 106 MB of partial state: more than the array holds."""
    from khalamari_b200 import abi, sliced_kv

    from khalamari_b200.device import Dtype
    from khalamari_b200.sdpa import Config, ExecutionVariant, Registry
    from khalamari_b200.selector import Selector

    contexts = [1024] * 50
    case = make_case(43, "bf16", 64, 8, 128, [c - 1 for c in contexts], [1] * 50, keep_f32=False)
    cfg = Config(Dtype.Bfloat16, case.num_q_heads, case.num_kv_heads, case.head_dim, case.tokens_per_page)
    variant = ExecutionVariant.sliced_kv(cfg, cfg.head_dim, 128, 8)
    selector = Selector.new(Registry.from_variants(cfg, [variant]), 64, 4096, 4096)
    run = DeviceCase(device, case, max_tokens=64, selector=selector)
    attention = run.attention
    selection = attention.select_partitioned(variant, 16, False, case.token_indices, case.cu_tokens)
    attention.prepare(case.req_slots, case.token_indices, case.cu_tokens, selection=selection)
    meta = attention.metadata
    shape = meta.replay_shape()
    compute = attention._sliced_kv(shape, meta.variant())
    assert compute.static_bytes_needed(shape.num_sdpa_map_task_templates) > abi.STATIC_PARTIALS_BYTES
    with pytest.raises(abi.KhError, match="shared array holds"):
        compute.invoke_attend_static(
            run.stream,
            sliced_kv.StaticBuffers(run.q, run.kv_pages, meta.req_slots(), run.page_ids,
                                    meta.sdpa_map_task_templates(), meta.cu_sdpa_partial_outputs(), run.output),
            case.layer_index, shape.num_tokens, shape.num_sdpa_map_task_templates)
    run.stream.synchronize()
    assert device.check(run.stream) == 0
