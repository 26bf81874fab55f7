"""Rank body of the world_size-2 ``gloo`` tests (CPU): imported by the spawned processes."""
import os

import numpy as np


def make_sequence(seed, context_len, num_q_heads, num_kv_heads, head_dim):
    rng = np.random.default_rng(seed)
    q = rng.standard_normal((num_q_heads, head_dim), dtype=np.float32)
    k = rng.standard_normal((context_len, num_kv_heads, head_dim), dtype=np.float32)
    v = rng.standard_normal((context_len, num_kv_heads, head_dim), dtype=np.float32)
    return q, k, v


def split_kv_rank(rank, world, port, seed, context_len, tokens_per_page, result_dir):
    """Every rank computes the partial state of its token range with the CPU oracle (standing in for the CUDA
    map, which cannot run here), exchanges records over gloo with the product's ``gather_records`` and merges
    them with the reducer's formula; rank r stores what it got for the parent to compare."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch
    import torch.distributed as dist

    import oracle
    from khalamari_b200 import split_kv

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        hq, hkv, d = 8, 2, 64
        scale = 0.125
        q, k, v = make_sequence(seed, context_len, hq, hkv, d)
        begin, end = split_kv.split_context(context_len, world, tokens_per_page)[rank]
        if end > begin:
            sums, maxes, outs = np.zeros(hq, np.float32), np.zeros(hq, np.float32), np.zeros((hq, d), np.float32)
            for head in range(hq):
                outs[head], sums[head], maxes[head] = oracle.partial_row(q[head], k, v, begin, end, hkv, d,
                                                                         head // (hq // hkv), scale)
            record = split_kv.pack_record(sums, maxes, outs)
        else:
            record = split_kv.empty_record(hq, d)
        gathered = split_kv.gather_records(torch.from_numpy(record)).numpy()
        all_sums, all_maxes, all_outs = split_kv.unpack_records(gathered, world, hq, d)
        merged = np.stack([oracle.merge_partials(all_sums[:, head], all_maxes[:, head], all_outs[:, head])[0]
                           for head in range(hq)])
        np.save(os.path.join(result_dir, f"merged_{rank}.npy"), merged)
        np.save(os.path.join(result_dir, f"range_{rank}.npy"), np.array([begin, end]))
    finally:
        dist.destroy_process_group()


def request_bins_rank(rank, world, port, contexts, result_dir):
    """Data-parallel decode: every rank derives the same request assignment, takes its own bin and reports the
    context tokens it owns; the sum over ranks (all-reduce) must be the whole batch."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    import torch
    import torch.distributed as dist

    from khalamari_b200 import split_kv

    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        bins = split_kv.assign_requests(contexts, world)
        mine = torch.tensor([float(sum(contexts[i] for i in bins[rank])), float(len(bins[rank]))], dtype=torch.float64)
        total = mine.clone()
        dist.all_reduce(total)
        peak = mine.clone()
        dist.all_reduce(peak, op=dist.ReduceOp.MAX)
        np.save(os.path.join(result_dir, f"bins_{rank}.npy"), np.array([*mine.tolist(), *total.tolist(), *peak.tolist()]))
    finally:
        dist.destroy_process_group()
