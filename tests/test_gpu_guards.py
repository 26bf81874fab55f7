"""Guards of the CUDA path (``-m gpu``): metadata that points past the page table, a partial-offset array that
names more partials than the buffers hold, the abort path of a bounded wait, and two host steps in flight.

Nothing here faults or hangs a GPU: every bad index is checked on the device before it becomes an address, and
the wait that runs out is a bounded one (the kernel returns and reports through the status word, the analogue
of the reference's SubmissionCheck, crates/inference-backend-metal/src/metal/stream/check.rs:8-13)."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from helpers import DeviceCase, assert_within_contract, bits_to_f32, make_case

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


@pytest.fixture(scope="module")
def device():
    from khalamari_b200.device import Device
    return Device(0)


def _prepared(device, case):
    run = DeviceCase(device, case)
    run.attention.prepare(case.req_slots, case.token_indices, case.cu_tokens)
    return run


def _expect_status(device, run, fragment):
    from khalamari_b200 import abi
    with pytest.raises(abi.KhError) as info:
        device.check(run.stream)
    assert info.value.code == 5 and fragment in str(info.value)
    assert device.check(run.stream) == 0  # the word is cleared by the read


def test_stale_request_slot_is_dropped_and_reported(device):
    """A req_slots entry beyond the page table (a padded or stale row) must not index the block table."""
    case = make_case(61, "bf16", 16, 2, 128, [700, 99], [1, 1])
    run = _prepared(device, case)
    run.attention.metadata.req_slots().write_typed(1, np.array([case.layout.num_req_slots + 1000], np.uint32))
    run.attention.record_sdpa(run.stream, run.q, run.kv_pages, run.page_ids, run.output)
    _expect_status(device, run, "beyond the page table")
    # the host-side plan refuses the same slot before anything is launched
    from khalamari_b200 import abi
    with pytest.raises(abi.InvalidArgument, match="slot"):
        run.attention.prepare([case.req_slots[0], case.layout.num_req_slots], case.token_indices, case.cu_tokens)
    # and the next clean call on the same device is right
    out = run.run(fused=False)
    assert_within_contract(out, case.oracle_output(), "call after a dropped task")


def test_kv_range_beyond_the_block_table_is_dropped_and_reported(device):
    case = make_case(62, "bf16", 16, 2, 256, [333], [1])
    run = _prepared(device, case)
    templates = run.attention.metadata.sdpa_map_task_templates()
    first = templates.read_typed(0, 3)
    capacity = case.layout.num_blocks * case.layout.num_page_ids_per_block * case.tokens_per_page
    templates.write_typed(0, np.array([first[0], first[1], capacity + 4096], np.uint32))
    run.attention.record_sdpa(run.stream, run.q, run.kv_pages, run.page_ids, run.output)
    _expect_status(device, run, "beyond the page table")
    from khalamari_b200 import abi
    with pytest.raises(abi.InvalidArgument, match="exceeds the page table"):
        run.attention.prepare(case.req_slots, [capacity + 5], case.cu_tokens)


def test_page_write_with_slot_or_token_beyond_the_table_writes_nothing(device):
    from khalamari_b200 import abi, kv_page_write
    from khalamari_b200.device import Buffer, Dtype, Stream
    from khalamari_b200.request_page_table import GQAPageTableLayout

    hkv, d, page = 2, 128, 16
    layout = GQAPageTableLayout(2, 1, 3, 1)
    page_bytes = 2 * hkv * page * d * 2
    pool = Buffer.from_slice(device, np.full(8 * page_bytes // 2, 0x1234, dtype=np.uint16))
    table = Buffer.from_slice(device, np.arange(6, dtype=np.uint32))
    compute = kv_page_write.Compute(device, kv_page_write.Config(hkv, d, page_bytes, Dtype.Bfloat16, Dtype.Bfloat16))
    rows = np.full((2, hkv, d), 0x3F80, dtype=np.uint16)
    stream = Stream(device)
    # write 0: slot 7 of a 2-slot table; write 1: token 48 = block 3 of a 3-block table
    buffers = kv_page_write.Buffers(pool, Buffer.from_slice(device, rows), Buffer.from_slice(device, rows),
                                    Buffer.from_slice(device, np.array([7, 1], np.uint32)),
                                    Buffer.from_slice(device, np.array([0, 48], np.uint32)), table)
    compute.invoke(stream, kv_page_write.Shape(2, layout), buffers, 2, 0)
    stream.synchronize()
    with pytest.raises(abi.KhError) as info:
        device.check(stream)
    assert info.value.code == 5 and "beyond the page table" in str(info.value)
    assert np.all(pool.read(0, 8 * page_bytes // 2, np.uint16) == 0x1234), "a guarded write reached the pool"


def test_reduce_never_reads_partials_beyond_its_buffers(device):
    """``cu_sdpa_partial_outputs`` comes from the caller's device memory. An entry larger than the partials the
    buffers hold (a stale array from a larger batch) is clamped: the partial buffers here are views into larger
    allocations whose tails hold poison partials of enormous weight, which an unclamped merge would pick up."""
    from khalamari_b200 import sliced_kv
    from khalamari_b200.device import Buffer

    case = make_case(63, "bf16", 64, 8, 128, [2100, 900], [1, 1])
    run = DeviceCase(device, case)
    expected = run.run(fused=False)
    attention = run.attention
    meta = attention.metadata
    shape = meta.replay_shape()
    compute = attention._sliced_kv(shape, meta.variant())
    sizes = compute.config.sizes(compute.shape)
    stats, outs = sizes.partial_output_stats_bytes // 4, sizes.partial_output_bytes // 4
    extra = 64 * case.num_q_heads  # poison partial rows behind the real ones

    def with_tail(count, fill, tail_count, poison):
        return Buffer.from_slice(device, np.concatenate([np.full(count, fill, np.float32),
                                                         np.full(tail_count, poison, np.float32)]))

    big_sum = with_tail(stats, 0.0, extra, 1.0e30)
    big_max = with_tail(stats, -np.inf, extra, 80.0)
    big_out = with_tail(outs, 0.0, extra * case.head_dim, 7.0e4)
    view = lambda big, count: Buffer.wrap(device, big.ref.ptr, count * 4)
    sums, maxes, partial = view(big_sum, stats), view(big_max, stats), view(big_out, outs)
    compute.invoke_map(run.stream, sliced_kv.MapBuffers(run.q, run.kv_pages, meta.req_slots(), run.page_ids,
                                                       meta.sdpa_map_task_templates(), sums, maxes, partial),
                       case.layer_index, shape.num_tokens, shape.num_sdpa_map_task_templates)
    stale = meta.cu_sdpa_partial_outputs().read_typed(0, shape.num_tokens + 1).copy()
    stale[-1] = shape.num_total_sdpa_map_task_templates + 40  # names partials that do not exist
    capacity = attention.policy.q_token_ranges.capacity(case.num_tokens)
    cu_dev = Buffer.from_slice(device, np.concatenate([stale, np.zeros(capacity, np.uint32)]))
    run.output.write(0, np.full(run.out_rows * case.num_q_heads * case.head_dim, run.canary, dtype=np.uint16))
    compute.invoke_reduce(run.stream, sliced_kv.ReduceBuffers(sums, maxes, partial, cu_dev, run.output),
                          shape.num_tokens)
    run.stream.synchronize()
    assert device.check(run.stream) == 0
    # templates between the active count and the recorded capacity hold empty partials (weight zero), so the clamped
    # merge of the last token equals the ordinary one; the poison rows behind the buffers would swamp it
    assert_within_contract(run.read_output(), expected, "reduce with a stale partial-offset array")


def test_two_host_steps_in_flight_match_the_synchronous_path(device):
    """HostPipeline: Q from page-locked memory, plan, map + reduce, output back, with a step's output copy running
    beside the next step's kernels. Alternating batches must come back exactly as the one-at-a-time path gives
    them."""
    from khalamari_b200.device import PinnedArray
    from khalamari_b200.gqa import HostPipeline

    case = make_case(64, "bf16", 64, 8, 128, [1500, 700, 33, 2047], [1, 1, 1, 1])
    run = DeviceCase(device, case, max_tokens=8)
    expected = run.run(fused=False)
    elems = case.num_tokens * case.num_q_heads * case.head_dim
    q_hosts = [PinnedArray(elems, np.uint16) for _ in range(2)]
    out_hosts = [PinnedArray(elems, np.uint16) for _ in range(3)]
    q_hosts[0].array[:] = case.q_bits.reshape(-1)
    q_hosts[1].array[:] = case.q_bits.reshape(-1)[::-1].copy()  # a second, different batch of Q rows
    pipeline = HostPipeline(run.attention, run.stream)
    tickets = []
    for i in range(6):
        out_hosts[i % 3].array[:] = 0
        ticket, launches, h2d, d2h = pipeline.submit(
            q_hosts[i % 2], out_hosts[i % 3], run.kv_pages, run.page_ids, case.req_slots, case.token_indices,
            case.cu_tokens, case.layer_index, 512 if i % 2 else None)
        assert launches == 2 and d2h == elems * 2 and h2d > elems * 2
        tickets.append(ticket)
        if i >= 1:
            pipeline.wait(tickets[i - 1])
            got = bits_to_f32("bf16", out_hosts[(i - 1) % 3].array.copy()).reshape(expected.shape)
            if (i - 1) % 2 == 0:
                assert_within_contract(got, expected, f"pipelined step {i - 1}")
    pipeline.drain()
    assert device.check(run.stream) == 0
    got = bits_to_f32("bf16", out_hosts[4 % 3].array.copy()).reshape(expected.shape)
    assert_within_contract(got, case.oracle_output(), "pipelined step 4 against the oracle")


@pytest.mark.parametrize("tile", ["decode", "prefill"])
def test_a_wait_that_runs_out_aborts_the_kernel_and_the_device_stays_usable(tile):
    """Runs in a child process on the measurement build of the library (the product build has no switch that
    withholds a copy): the stream warp announces the bytes of each task's first stage and never copies them, the
    wait limit is lowered to a few thousand polls, the consumers' wait runs out, every warp leaves through the
    abort path (tensor memory freed on the tcgen05 instance), ``kh_device_check`` reports bit 0, and the next,
    clean call on the same device matches the oracle."""
    env = dict(os.environ, KH_GQA_LIBRARY="measure")
    env.pop("KH_GQA_DEBUG", None)
    done = subprocess.run([sys.executable, str(ROOT / "tests" / "wait_expiry_worker.py"), tile], env=env,
                          capture_output=True, text=True, timeout=900)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-2000:]
    report = json.loads(done.stdout.strip().splitlines()[-1])
    assert report["aborted_code"] == 5 and report["status_word"] & 1, report
    assert "bounded wait" in report["message"]
    assert report["clean_word_after"] == 0 and report["next_call_within_contract"], report
