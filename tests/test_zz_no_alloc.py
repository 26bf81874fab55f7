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


def _setup(device, case):
    """Prepares ``case`` and returns (run, compute, buffers, shape, output through caller-owned partial buffers)."""
    from khalamari_b200 import abi, sdpa, sliced_kv

    run = DeviceCase(device, case)
    attention = run.attention
    attention.prepare(case.req_slots, case.token_indices, case.cu_tokens)
    meta = attention.metadata
    assert meta.variant().kind == sdpa.MapKernelKind.SlicedKv
    expected = run.run(fused=False)

    shape = meta.replay_shape()
    compute = attention._sliced_kv(shape, meta.variant())
    needed = compute.static_bytes_needed(shape.num_sdpa_map_task_templates)
    assert 0 < needed <= abi.STATIC_PARTIALS_BYTES
    buffers = sliced_kv.StaticBuffers(run.q, run.kv_pages, meta.req_slots(), run.page_ids,
                                      meta.sdpa_map_task_templates(), meta.cu_sdpa_partial_outputs(), run.output)
    return run, compute, buffers, shape, expected


def _fill_output_with_canary(run, case):
    run.output.write(0, np.full(run.out_rows * case.num_q_heads * case.head_dim, run.canary, dtype=np.uint16))


def _run_both(device, case):
    """Returns (output through caller-owned partial buffers, output through the shared array)."""
    run, compute, buffers, shape, expected = _setup(device, case)
    _fill_output_with_canary(run, case)
    compute.invoke_attend_static(run.stream, buffers, case.layer_index, shape.num_tokens,
                                 shape.num_sdpa_map_task_templates)
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


def test_later_calls_leave_the_free_device_memory_unchanged(device):
    """The claim of the entry point: no call allocates or frees device memory. After one warm call (kernel images
    and tensor maps in place) the free memory the driver reports stays the same over further calls."""
    import torch

    case = make_case(44, "bf16", 16, 2, 128, [c - 1 for c in [700, 90, 1500]], [1] * 3)
    run, compute, buffers, shape, expected = _setup(device, case)
    args = (run.stream, buffers, case.layer_index, shape.num_tokens, shape.num_sdpa_map_task_templates)
    compute.invoke_attend_static(*args)
    run.stream.synchronize()
    torch.cuda.mem_get_info(0)  # the first query may itself set up state
    free_before = torch.cuda.mem_get_info(0)[0]
    for _ in range(8):
        compute.invoke_attend_static(*args)
    run.stream.synchronize()
    free_after = torch.cuda.mem_get_info(0)[0]
    assert free_after == free_before, f"free device memory changed by {free_before - free_after} bytes over 8 calls"
    assert device.check(run.stream) == 0
    assert np.array_equal(expected, run.read_output())


def test_capacity_call_reads_the_active_counts_bound_to_the_stream(device):
    """Replay form: the host arguments carry the recorded capacities, the stream's bound count words carry what is
    active this submission (tokens, -, map task templates). Rows beyond the active tokens keep their bytes."""
    from khalamari_b200.device import Buffer

    case = make_case(45, "bf16", 16, 2, 128, [c - 1 for c in [1200, 300, 2000, 64]], [1] * 4)
    run, compute, buffers, shape, expected = _setup(device, case)
    _fill_output_with_canary(run, case)
    counts = Buffer.from_slice(device, np.array([shape.num_tokens, shape.num_tokens, shape.num_sdpa_map_task_templates, 0],
                                                dtype=np.uint32))
    run.stream.bind_active_counts(counts)
    try:
        compute.invoke_attend_static(run.stream, buffers, case.layer_index, shape.num_total_tokens,
                                     shape.num_total_sdpa_map_task_templates)
        run.stream.synchronize()
        assert device.check(run.stream) == 0
        assert np.array_equal(expected, run.read_output())

        # fewer active tokens than recorded: the last request's row must stay untouched
        _fill_output_with_canary(run, case)
        counts.write(0, np.array([shape.num_tokens - 1], dtype=np.uint32))
        compute.invoke_attend_static(run.stream, buffers, case.layer_index, shape.num_total_tokens,
                                     shape.num_total_sdpa_map_task_templates)
        run.stream.synchronize()
        assert device.check(run.stream) == 0
    finally:
        run.stream.bind_active_counts(None)
    out = run.read_output()
    assert np.array_equal(out[:shape.num_tokens - 1], expected[:shape.num_tokens - 1])
    raw = run.output.read(0, run.out_rows * case.num_q_heads * case.head_dim, np.uint16)
    row = case.num_q_heads * case.head_dim
    assert np.all(raw[(shape.num_tokens - 1) * row:shape.num_tokens * row] == run.canary)


def test_zero_active_splits_writes_zero_rows_and_reads_nothing_stale(device):
    """``num_active_kv_splits == 0``: no map task runs, every range merges zero partials and writes a zero row
    (the reducer's empty-list rule), whatever ``cu_sdpa_partial_outputs`` still holds from the batch before."""
    case = make_case(46, "bf16", 16, 2, 128, [c - 1 for c in [900, 40]], [1] * 2)
    run, compute, buffers, shape, _ = _setup(device, case)
    _fill_output_with_canary(run, case)
    compute.invoke_attend_static(run.stream, buffers, case.layer_index, shape.num_tokens, 0)
    run.stream.synchronize()
    assert device.check(run.stream) == 0
    out = run.read_output()
    assert np.all(out[:shape.num_tokens] == 0)
