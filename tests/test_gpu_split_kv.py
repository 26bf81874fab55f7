"""One long sequence split in token order over W ranks (``-m gpu``), emulated on one GPU: the ranks run one
after another on the same device, each over a pool that holds only its own pages; their records are
concatenated the way an all-gather leaves them and merged by ``kh_combine_packed_partials``. The NCCL exchange
itself is covered on CPU ranks over gloo (test_split_kv_ranks.py)."""
import numpy as np
import pytest

import oracle
from helpers import DeviceCase, PagedCase, assert_within_contract, bits_to_f32, make_case, round_to

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    from khalamari_b200.device import Device
    return Device(0)


def _local_case(full: PagedCase, begin: int, end: int, seed: int) -> PagedCase:
    """The pages of tokens [begin, end) as a rank holds them: own pool, own block table, local token order."""
    local_len = end - begin
    page = full.tokens_per_page
    pages = max(-(-local_len // page), 1)
    layout = oracle.PageTableLayout(1, 1, pages, 1)
    pool16 = np.full((pages + 2) * full.page_bytes // 2, 0x7FC0, dtype=np.uint16)
    pool = pool16.view(np.uint8)
    table = np.zeros(layout.num_page_ids(), dtype=np.uint32)
    table[:pages] = np.random.default_rng(seed).permutation(pages + 2)[:pages]
    k = full.k_f32[0][begin:end]
    v = full.v_f32[0][begin:end]
    if local_len:
        k_bits, _ = round_to(full.dtype_name, k)
        v_bits, _ = round_to(full.dtype_name, v)
        oracle.scatter_paged(pool, table, layout, 0, 0, page, full.num_kv_heads, full.head_dim, 2, 0, k_bits, v_bits)
    return PagedCase(full.dtype_name, full.num_q_heads, full.num_kv_heads, full.head_dim, page, full.scale, layout,
                     0, [0], [max(local_len - 1, 0)], [1], [0, 1], full.q_bits, full.q_f32, pool, table, [k], [v])


@pytest.mark.parametrize("context_len,world,partition", [(20000, 2, 1024), (20000, 4, 512), (4099, 8, 256),
                                                        (40, 4, 256)])
def test_ranks_merge_to_the_unsplit_oracle(device, context_len, world, partition):
    import torch

    from khalamari_b200 import abi, split_kv
    from khalamari_b200.device import Buffer, Dtype

    full = make_case(7, "bf16", 16, 2, 256, [context_len - 1], [1], scale=1.0 / 16.0)
    expected = full.oracle_output()
    ranges = split_kv.split_context(context_len, world, full.tokens_per_page)
    records, keep = [], []
    for rank, (begin, end) in enumerate(ranges):
        run = DeviceCase(device, _local_case(full, begin, end, 100 + rank))
        decode = split_kv.SplitKvDecode(device, run.attention, 1)
        decode.prepare(0, end - begin, partition)
        decode.record_local(run.stream, run.q, run.kv_pages, run.page_ids)
        run.stream.synchronize()
        torch.cuda.synchronize()
        assert device.check(run.stream) == 0
        records.append(decode.local_record.clone())
        keep.append((run, decode))
    gathered = torch.cat(records)
    run = keep[0][0]
    out = Buffer.new_zeroed(device, 16 * 256 * 2)
    abi.call("kh_combine_packed_partials", device.handle, run.stream.handle, world, 16, 256,
             Buffer.wrap(device, gathered.data_ptr(), gathered.numel() * 4).ref, int(Dtype.Bfloat16), out.ref)
    run.stream.synchronize()
    actual = bits_to_f32("bf16", out.read(0, 16 * 256, np.uint16)).reshape(1, 16, 256)
    assert_within_contract(actual, expected, f"split over {world} ranks")
    # the rank-local records themselves: merging them on the host with the reducer's formula gives the same rows
    sums, maxes, outs = split_kv.unpack_records(gathered.cpu().numpy(), world, 16, 256)
    host = np.stack([oracle.merge_partials(sums[:, h], maxes[:, h], outs[:, h])[0] for h in range(16)])
    assert np.max(np.abs(host[None] - expected)) < 2e-3


def test_single_rank_step_matches_the_two_launch_path(device):
    """world 1: record_step (map, local merge, record copy, packed merge) equals map + reduce."""
    import torch

    from khalamari_b200 import split_kv

    full = make_case(8, "bf16", 16, 2, 256, [5000 - 1], [1], scale=1.0 / 16.0)
    run = DeviceCase(device, full)
    torch_stream = torch.cuda.current_stream()
    from khalamari_b200.device import Stream
    stream = Stream(device, torch_stream.cuda_stream)
    decode = split_kv.SplitKvDecode(device, run.attention, 1)
    decode.prepare(full.req_slots[0], 5000, 512)
    launches = decode.record_step(stream, run.q, run.kv_pages, run.page_ids, run.output)
    torch.cuda.synchronize()
    assert launches == 3 and device.check(stream) == 0
    assert_within_contract(run.read_output(), full.oracle_output(), "single-rank split-KV step")


def _inbox_image(world, rows, head_dim, step, records):
    """Host image of an inbox in which the ranks of ``records`` ({rank: (sums, maxes, outputs)}) have already
    delivered their rows of step ``step`` (parity step & 1)."""
    record = head_dim + 4
    floats = np.zeros(2 * world * rows * record, np.float32)
    flags = np.zeros(2 * world * rows + rows, np.uint32)
    parity = step & 1
    for rank, (sums, maxes, outs) in records.items():
        for row in range(rows):
            at = ((parity * world + rank) * rows + row) * record
            floats[at:at + head_dim] = outs[row]
            floats[at + head_dim] = sums[row]
            floats[at + head_dim + 1] = maxes[row]
            flags[(parity * world + rank) * rows + row] = step
    return np.concatenate([floats.view(np.uint32), flags])


@pytest.mark.parametrize("world,my_rank", [(1, 0), (4, 2), (8, 7)])
def test_peer_exchange_kernel_merges_delivered_rows(device, world, my_rank):
    """The one-kernel exchange (kh_peer_exchange_combine) on ONE GPU: the other ranks' rows of the step are put
    into this rank's inbox by the host beforehand (kernels that wait for one another must not share a GPU), and the
    "peer" inboxes this rank writes into are scratch buffers on the same device. Checks the local merge, the rows
    this rank delivers to every inbox, and the final merge against the unsplit oracle."""
    from khalamari_b200 import split_kv
    from khalamari_b200.device import Buffer, Dtype, Stream

    context_len, rows, d = 6000, 16, 256
    full = make_case(9, "bf16", rows, 2, d, [context_len - 1], [1], scale=1.0 / 16.0)
    expected = full.oracle_output()[0]
    ranges = split_kv.split_context(context_len, world, full.tokens_per_page)
    q = full.q_f32[0]
    # what the other ranks deliver: their slice's partial per row, straight from the oracle
    delivered = {}
    for rank, (begin, end) in enumerate(ranges):
        if rank == my_rank:
            continue
        parts = [oracle.partial_row(q[h], full.k_f32[0], full.v_f32[0], begin, end, 2, d, h // 8, full.scale)
                 if end > begin else (np.zeros(d, np.float32), 0.0, -np.inf) for h in range(rows)]
        delivered[rank] = ([p[1] for p in parts], [p[2] for p in parts], [p[0] for p in parts])
    exchange = split_kv.PeerExchange(device, my_rank, world, rows, d)
    step = 1
    exchange.inbox.write(0, _inbox_image(world, rows, d, step, delivered))
    scratch = [Buffer.new_zeroed(device, exchange.inbox.len_bytes()) for _ in range(world)]
    exchange.attach([exchange.inbox.ref.ptr if r == my_rank else scratch[r].ref.ptr for r in range(world)])
    # this rank's own slice through the real local map
    begin, end = ranges[my_rank]
    run = DeviceCase(device, _local_case(full, begin, end, 300))
    decode = split_kv.SplitKvDecode(device, run.attention, world, peer_exchange=exchange)
    decode.prepare(0, end - begin, 256)
    out = Buffer.new_zeroed(device, rows * d * 2)
    launches = decode.record_step(run.stream, run.q, run.kv_pages, run.page_ids, out)
    run.stream.synchronize()
    assert device.check(run.stream) == 0 and launches == 2
    actual = bits_to_f32("bf16", out.read(0, rows * d, np.uint16)).reshape(rows, d)
    assert_within_contract(actual, expected, f"peer exchange, rank {my_rank} of {world}")
    # the rows this rank delivered to a peer's inbox are its own slice's partial
    if world > 1:
        peer = (my_rank + 1) % world
        image = scratch[peer].read(0, 2 * world * rows * (d + 4), np.float32).reshape(2, world, rows, d + 4)
        mine = image[step & 1, my_rank]
        for h in (0, rows - 1):
            part = oracle.partial_row(q[h], full.k_f32[0], full.v_f32[0], begin, end, 2, d, h // 8, full.scale)
            assert np.max(np.abs(mine[h, :d] - part[0])) < 2e-3 and abs(mine[h, d + 1] - part[2]) < 1e-3
        flags = scratch[peer].read(2 * world * rows * (d + 4) * 4, 2 * world * rows, np.uint32).reshape(2, world, rows)
        assert np.all(flags[step & 1, my_rank] == step)
    exchange.close()


def test_peer_exchange_wait_runs_out_without_hanging(device):
    """A rank whose peers never deliver: the bounded wait expires, the status word says so, no output row is
    written, and the device stays usable."""
    from khalamari_b200 import abi, split_kv
    from khalamari_b200.device import Buffer, Dtype, Stream

    rows, d, world = 16, 256, 2
    exchange = split_kv.PeerExchange(device, 0, world, rows, d)
    scratch = Buffer.new_zeroed(device, exchange.inbox.len_bytes())
    exchange.attach([exchange.inbox.ref.ptr, scratch.ref.ptr])
    stream = Stream(device)
    partial_stats = Buffer.from_slice(device, np.ones(rows, np.float32))
    partial_max = Buffer.from_slice(device, np.zeros(rows, np.float32))
    partial_out = Buffer.from_slice(device, np.ones(rows * d, np.float32))
    out = Buffer.from_slice(device, np.full(rows * d, 0x4228, np.uint16))
    device.set_wait_limit(2000)
    try:
        exchange.combine(stream, 1, partial_stats, partial_max, partial_out, Dtype.Bfloat16, out)
        with pytest.raises(abi.KhError) as info:
            device.check(stream)
        assert info.value.code == 5 and "bounded wait" in str(info.value)
    finally:
        device.set_wait_limit(0)
    assert np.all(out.read(0, rows * d, np.uint16) == 0x4228)
    assert device.check(stream) == 0
    exchange.close()
