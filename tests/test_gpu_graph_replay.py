"""Replay (``-m gpu``): one recorded attention program serves many batches. The launches are captured once into a
CUDA graph with grids sized by the recorded capacities; every later batch only rewrites the metadata arrays, the
four replay-count words and Q, then launches the graph (the reference's active / total replay contract,
docs/executor_gqa.md:476-532, with a CUDA graph in the place of the indirect command buffer)."""
import numpy as np
import pytest

import oracle
from helpers import DeviceCase, assert_within_contract, bits_to_f32, make_case

pytestmark = pytest.mark.gpu


def _expected(case, subset):
    cu = list(range(len(subset) + 1))
    histories = [case.token_indices[i] for i in subset]
    q = case.q_f32[subset]
    return oracle.projected_gqa(cu, histories, q, [case.k_f32[i] for i in subset], [case.v_f32[i] for i in subset],
                                case.head_dim, case.num_q_heads, case.num_kv_heads, case.scale, oracle.max_threads())


@pytest.mark.parametrize("hq,hkv,d", [(64, 8, 128), (16, 2, 256)])
def test_one_captured_program_serves_batches_of_different_sizes(hq, hkv, d):
    import torch

    from khalamari_b200.device import Device, Dtype, Stream
    from khalamari_b200.sdpa import Config, ExecutionVariant, Registry
    from khalamari_b200.selector import Selector

    device = Device(0)
    contexts = [300, 700, 520, 260, 900, 515, 1000]
    case = make_case(61, "bf16", hq, hkv, d, [c - 1 for c in contexts], [1] * len(contexts))
    cfg = Config(Dtype.Bfloat16, hq, hkv, d, 16)
    variant = ExecutionVariant.sliced_kv(cfg, d, 128, min(hq // hkv, 8))
    selector = Selector.new(Registry.from_variants(cfg, [variant]), 8, 64, 64)
    run = DeviceCase(device, case, max_tokens=8, selector=selector)
    attention = run.attention
    torch_stream = torch.cuda.Stream()
    stream = Stream(device, torch_stream.cuda_stream)
    row = hq * d

    def prepare(subset):
        slots = [case.req_slots[i] for i in subset]
        histories = [case.token_indices[i] for i in subset]
        cu = list(range(len(subset) + 1))
        # the recorded capacity: every batch of three or four tokens is planned into the four-token bucket
        selection = attention.select_partitioned(variant, 256, False, histories, cu, num_total_tokens=4)
        attention.prepare(slots, histories, cu, num_total_tokens=4, selection=selection, stream=stream)
        q_rows = np.full((8, row), 0x7FC0, dtype=np.uint16)  # unused capacity rows hold NaN bits
        q_rows[:len(subset)] = case.q_bits[subset].reshape(len(subset), row)
        stream.synchronize()
        run.q_capacity.write(0, q_rows.reshape(-1))
        return attention.metadata.replay_shape()

    from khalamari_b200.device import Buffer
    run.q_capacity = Buffer.new_zeroed(device, 8 * row * 2)
    out = Buffer.from_slice(device, np.full(8 * row, run.canary, dtype=np.uint16))

    batches = [[0, 1, 2, 3], [4, 1, 5], [3, 0, 2, 1], [6, 3, 0, 5], [4, 6, 1]]
    first = prepare(batches[0])
    totals = (first.num_total_tokens, first.num_total_q_token_tiles, first.num_total_sdpa_map_task_templates)
    # once outside capture: tensor maps for these buffers are encoded here, not while capturing
    attention.record_replay(stream, run.q_capacity, run.kv_pages, run.page_ids, out, case.layer_index)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=torch_stream):
        launches = attention.record_replay(stream, run.q_capacity, run.kv_pages, run.page_ids, out, case.layer_index)
    assert launches == 2
    for subset in batches:
        shape = prepare(subset)
        assert (shape.num_total_tokens, shape.num_total_q_token_tiles, shape.num_total_sdpa_map_task_templates) == totals, \
            "the batch left the recorded replay bucket"
        out.write(0, np.full(8 * row, run.canary, dtype=np.uint16))
        with torch.cuda.stream(torch_stream):
            graph.replay()
        torch_stream.synchronize()
        assert device.check(stream) == 0
        bits = out.read(0, 8 * row, np.uint16)
        n = len(subset)
        assert np.all(bits[n * row:] == run.canary), "rows past the active tokens were written"
        actual = bits_to_f32("bf16", bits[:n * row]).reshape(n, hq, d)
        assert_within_contract(actual, _expected(case, np.array(subset)), f"replayed batch {subset}")
