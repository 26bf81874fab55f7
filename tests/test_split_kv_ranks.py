"""Host logic of the multi-GPU shardings, on CPU: rank arithmetic, and world_size-2 ``gloo`` runs of the record
exchange and merge (the CUDA kernels are replaced by the CPU oracle; the collective and the record layout are the
product's)."""
import multiprocessing as mp
import socket

import numpy as np
import pytest

import oracle
import rank_worker
from khalamari_b200 import abi, split_kv


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run_ranks(target, world, *args):
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=target, args=(rank, world, port, *args)) for rank in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    for p in procs:
        if p.is_alive():
            p.kill()
            pytest.fail("a rank did not finish")
        assert p.exitcode == 0


def test_split_context_is_contiguous_page_aligned_and_balanced():
    for context_len, world, page in [(1048576, 8, 16), (131072, 4, 16), (517, 2, 16), (5, 4, 16), (0, 2, 16),
                                     (1000, 3, 16), (16, 2, 16), (33, 8, 16)]:
        ranges = split_kv.split_context(context_len, world, page)
        assert len(ranges) == world
        assert ranges[0][0] == 0 and ranges[-1][1] == context_len
        for (b0, e0), (b1, e1) in zip(ranges, ranges[1:]):
            assert e0 == b1 and b0 <= e0
        for begin, end in ranges[:-1]:
            assert begin % page == 0 and end % page == 0
        pages = [-(-(e - b) // page) for b, e in ranges]
        assert max(pages) - min(pages) <= 1
    with pytest.raises(abi.InvalidArgument):
        split_kv.split_context(10, 0, 16)


def test_assign_requests_covers_every_request_once_and_balances():
    rng = np.random.default_rng(1)
    contexts = rng.integers(1024, 8193, size=64).tolist()
    for world in (1, 2, 4, 8):
        bins = split_kv.assign_requests(contexts, world)
        flat = sorted(i for b in bins for i in b)
        assert flat == list(range(64))
        loads = [sum(contexts[i] for i in b) for b in bins]
        assert max(loads) - min(loads) <= max(contexts)        # greedy bound
        assert max(loads) <= 1.02 * sum(contexts) / world      # and in practice within 2 % of the mean
    assert split_kv.assign_requests([], 2) == [[], []]
    assert split_kv.assign_requests([5, 5, 5], 2) == [[0, 2], [1]]


def test_record_layout_round_trips():
    rng = np.random.default_rng(0)
    rows, d, n = 16, 256, 3
    assert split_kv.record_floats(rows, d) * 4 == 16512          # one rank's record at Hq16 / D256
    records = []
    for _ in range(n):
        records.append(split_kv.pack_record(rng.random(rows), rng.random(rows), rng.random((rows, d))))
    sums, maxes, outs = split_kv.unpack_records(np.concatenate(records), n, rows, d)
    assert sums.shape == (n, rows) and maxes.shape == (n, rows) and outs.shape == (n, rows, d)
    assert np.array_equal(outs[2].reshape(-1), records[2][2 * rows:])
    empty = split_kv.empty_record(rows, d)
    assert np.all(empty[:rows] == 0) and np.all(np.isneginf(empty[rows:2 * rows]))


@pytest.mark.parametrize("context_len", [1000, 17])
def test_two_ranks_merge_to_the_unsplit_oracle(tmp_path, context_len):
    """world_size 2 over gloo; 17 tokens with 16-token pages leaves rank 0 with one page and rank 1 with one token."""
    world, seed, page = 2, 5, 16
    _run_ranks(rank_worker.split_kv_rank, world, seed, context_len, page, str(tmp_path))
    hq, hkv, d = 8, 2, 64
    q, k, v = rank_worker.make_sequence(seed, context_len, hq, hkv, d)
    expected = np.stack([oracle.oracle_row(q[h], k, v, context_len, hkv, d, h // (hq // hkv), 0.125)
                         for h in range(hq)])
    for rank in range(world):
        merged = np.load(tmp_path / f"merged_{rank}.npy")
        assert np.max(np.abs(merged - expected)) < 2e-6
    ranges = [np.load(tmp_path / f"range_{r}.npy").tolist() for r in range(world)]
    assert ranges == [list(r) for r in split_kv.split_context(context_len, world, page)]


def test_an_empty_rank_has_zero_weight(tmp_path):
    """5 tokens over 2 ranks: all pages land on rank 1 and rank 0 contributes the empty record."""
    world, seed, page, context_len = 2, 6, 16, 5
    _run_ranks(rank_worker.split_kv_rank, world, seed, context_len, page, str(tmp_path))
    hq, hkv, d = 8, 2, 64
    q, k, v = rank_worker.make_sequence(seed, context_len, hq, hkv, d)
    expected = np.stack([oracle.oracle_row(q[h], k, v, context_len, hkv, d, h // (hq // hkv), 0.125)
                         for h in range(hq)])
    assert np.load(tmp_path / "range_0.npy").tolist() == [0, 0]
    assert np.max(np.abs(np.load(tmp_path / "merged_0.npy") - expected)) < 2e-6


def test_two_ranks_own_the_whole_batch(tmp_path):
    contexts = np.random.default_rng(1).integers(1024, 8193, size=64).tolist()
    _run_ranks(rank_worker.request_bins_rank, 2, contexts, str(tmp_path))
    r0, r1 = np.load(tmp_path / "bins_0.npy"), np.load(tmp_path / "bins_1.npy")
    assert r0[2] == r1[2] == float(sum(contexts)) and r0[3] == r1[3] == 64.0
    assert r0[0] + r1[0] == float(sum(contexts))
    assert r0[4] == max(r0[0], r1[0])
