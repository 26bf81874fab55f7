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
