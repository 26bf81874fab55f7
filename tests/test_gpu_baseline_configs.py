"""Parity against the CPU oracle at the sizes the build's configurations state (``-m gpu``), through the C ABI.

The other GPU tests stay small so that the oracle answers in milliseconds; these run the configurations at their
full shapes, where 32-bit row arithmetic over a 40,000-page pool, page-id segments of long tasks, 65,536-entry
block tables and merges of a thousand partials are exercised:

* configuration 2 exactly as ``bench.py`` runs it (batch 64, contexts U[1024, 8192] seed 1, 40,000-page pool,
  512-token partitions) and with the selector's own slice;
* configuration 3 in full (batch 32, q_len 4 and 2, prefixes U[4096, 32768] seed 2);
* configuration 4 on one GPU at 131,072 / 524,288 / 1,048,576 tokens, all 16 heads;
* configuration 5 (8 prefill chunks of 2,048 tokens + 56 decode rows in one call), oracle-checked the way the
  reference's benchmark gate samples it (crates/inference-backend-metal/benches/gqa/matrix.rs:116-151): every
  decode row plus the first, middle and last query token of each prefill sequence, all heads; and a full check of
  the same mix with 256-token chunks on prefixes a tenth as long.

Oracle inputs are the rounded storage values (sliced_kv_test.rs:171-182). Tolerance: per element
|a - b| <= 2e-3 or |a - b| <= 1e-2 |b| (helpers.assert_within_contract)."""
import dataclasses
import os

import numpy as np
import pytest

import oracle
from helpers import DeviceCase, assert_within_contract, make_case

import bench

pytestmark = pytest.mark.gpu
WORKERS = max(2, min(16, os.cpu_count() or 2))  # threads that draw and page the synthetic K/V


@pytest.fixture(scope="module")
def device():
    from khalamari_b200.device import Device
    return Device(0)


def _decode_variant(attention):
    return next(v for v in attention.selector.variants() if v.kind == 0 and v.thread_block.max_q_tokens == 1)


# ---------------------------------------------------------------------------------------------------
# configuration 2
# ---------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def config2_case():
    spec = bench.WORKLOADS["c2"]
    contexts = bench.contexts_for(spec, 0)
    assert len(contexts) == 64 and min(contexts) >= 1024 and max(contexts) <= 8192
    return make_case(spec["seed"], "bf16", spec["hq"], spec["hkv"], spec["d"], [c - 1 for c in contexts],
                     [1] * len(contexts), pool_pages=spec["pool_pages"], poison=False, workers=WORKERS)


@pytest.mark.parametrize("partition", [512, 0])
def test_config2_batched_decode_as_benched(device, config2_case, partition):
    case = config2_case
    run = DeviceCase(device, case)
    selection = None
    if partition:
        selection = run.attention.select_partitioned(_decode_variant(run.attention), partition, False,
                                                     case.token_indices, case.cu_tokens)
        assert len(selection.map_task_templates()) == sum(-(-c // partition) for c in case.contexts())
    out = run.run(selection, fused=False)
    assert out.shape == (64, 64, 128)
    assert_within_contract(out, case.oracle_output(), f"config 2, partition {partition or 'selector'}")


# ---------------------------------------------------------------------------------------------------
# configuration 3
# ---------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def config3_case():
    spec = bench.WORKLOADS["c3"]
    contexts = bench.contexts_for(spec, 0)
    assert len(contexts) == 32 and min(contexts) >= 4096 and max(contexts) <= 32768
    return make_case(spec["seed"], "bf16", spec["hq"], spec["hkv"], spec["d"], [c - 4 for c in contexts],
                     [4] * len(contexts), scale=1.0 / 16.0, poison=False, workers=WORKERS)


def _shorter_verify(case, q_len):
    """The same requests verifying ``q_len`` of their (four) new tokens: same pool and block tables; the cached
    rows of the dropped tokens stay in the pages past every visible range."""
    full = case.q_lens[0]
    rows = np.concatenate([np.arange(r * full, r * full + q_len) for r in range(len(case.q_lens))])
    contexts = [h + q_len for h in case.token_indices]
    return dataclasses.replace(
        case, q_lens=[q_len] * len(case.q_lens), cu_tokens=[r * q_len for r in range(len(case.q_lens) + 1)],
        q_bits=np.ascontiguousarray(case.q_bits[rows]), q_f32=np.ascontiguousarray(case.q_f32[rows]),
        k_f32=[k[:c] for k, c in zip(case.k_f32, contexts)], v_f32=[v[:c] for v, c in zip(case.v_f32, contexts)])


@pytest.mark.parametrize("q_len", [4, 2])
def test_config3_speculative_verify(device, config3_case, q_len):
    case = config3_case if q_len == 4 else _shorter_verify(config3_case, q_len)
    out = DeviceCase(device, case).run(fused=False)
    assert out.shape == (32 * q_len, 24, 256)
    assert_within_contract(out, case.oracle_output(), f"config 3, q_len {q_len}")


# ---------------------------------------------------------------------------------------------------
# configuration 4 on one GPU
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("context_len", [131072, 524288, 1048576])
def test_config4_long_sequence_on_one_gpu(device, context_len):
    case = make_case(3, "bf16", 16, 2, 256, [context_len - 1], [1], scale=1.0 / 16.0, poison=False, workers=WORKERS)
    assert case.layout.num_blocks == context_len // 16
    run = DeviceCase(device, case)
    out = run.run(fused=False)
    templates = run.attention.metadata.replay_shape().num_sdpa_map_task_templates
    assert templates >= context_len // 2048, "a long sequence must be cut into KV slices"
    assert_within_contract(out, case.oracle_output(), f"config 4, {context_len} tokens, {templates} slices")


# ---------------------------------------------------------------------------------------------------
# configuration 5
# ---------------------------------------------------------------------------------------------------
def _mixed_case(chunk, prefix_hi, seed=4):
    rng = np.random.default_rng(seed)
    prefixes = rng.integers(0, prefix_hi + 1, size=8).tolist()
    decode_contexts = rng.integers(1024, 8192 + 1, size=56).tolist()
    histories = prefixes + [c - 1 for c in decode_contexts]
    q_lens = [chunk] * 8 + [1] * 56
    return make_case(seed, "bf16", 64, 8, 128, histories, q_lens, poison=False, workers=WORKERS)


def _sampled_oracle(case, rows_by_request):
    """The oracle's rows for the sampled (request, token in request) pairs: each sampled token becomes a request of
    its own with one new token, whose context is the cached rows it may see."""
    q_rows, ks, vs, histories = [], [], [], []
    for request, tokens in rows_by_request:
        for t in tokens:
            visible = case.token_indices[request] + t + 1
            q_rows.append(case.q_f32[case.cu_tokens[request] + t])
            ks.append(case.k_f32[request][:visible])
            vs.append(case.v_f32[request][:visible])
            histories.append(visible - 1)
    cu = list(range(len(q_rows) + 1))
    return oracle.projected_gqa(cu, histories, np.stack(q_rows), ks, vs, case.head_dim, case.num_q_heads,
                                case.num_kv_heads, case.scale, oracle.max_threads())


def test_config5_prefill_and_decode_in_one_call_sampled(device):
    case = _mixed_case(2048, 30720)
    out = DeviceCase(device, case).run(fused=False)
    assert out.shape == (8 * 2048 + 56, 64, 128)
    samples = [(r, [0, 1023, 2047]) for r in range(8)] + [(r, [0]) for r in range(8, 64)]
    expected = _sampled_oracle(case, samples)
    flat = [case.cu_tokens[r] + t for r, tokens in samples for t in tokens]
    assert len(flat) == 80
    assert_within_contract(out[flat], expected, "config 5, sampled rows")


def test_config5_mix_with_short_chunks_in_full(device):
    case = _mixed_case(256, 3072)
    out = DeviceCase(device, case).run(fused=False)
    assert_within_contract(out, case.oracle_output(), "config 5 mix, 256-token chunks, every row")


def _run_mixed(device, case):
    """The batch through MixedBatchAttention (decode run and prefill run as two selections, back to back), on the
    buffers a DeviceCase uploaded."""
    from khalamari_b200.gqa import GQACore, MixedBatchAttention
    run = DeviceCase(device, case)
    mixed = MixedBatchAttention(device, GQACore(case.head_dim, case.num_q_heads, case.num_kv_heads, case.scale),
                                run.dtype, case.page_bytes, run.layout, case.num_tokens, max_decode_tokens=64)
    mixed.prepare(case.req_slots, case.token_indices, case.cu_tokens)
    assert len(mixed.plan) == 2, "eight prefill requests then 56 decode requests split into two selections"
    launches = mixed.record_sdpa(run.stream, run.q, run.kv_pages, run.page_ids, run.output, case.layer_index)
    run.stream.synchronize()
    assert device.check(run.stream) == 0
    return run.read_output(), launches


def test_config5_as_two_selections_in_one_call_sampled(device):
    case = _mixed_case(2048, 30720)
    out, launches = _run_mixed(device, case)
    assert 2 <= launches <= 4
    samples = [(r, [0, 1023, 2047]) for r in range(8)] + [(r, [0]) for r in range(8, 64)]
    flat = [case.cu_tokens[r] + t for r, tokens in samples for t in tokens]
    assert_within_contract(out[flat], _sampled_oracle(case, samples), "config 5 as two selections, sampled rows")


def test_config5_as_two_selections_short_chunks_in_full(device):
    case = _mixed_case(256, 3072)
    out, _ = _run_mixed(device, case)
    assert_within_contract(out, case.oracle_output(), "config 5 mix as two selections, every row")


def test_mixed_batch_in_any_other_order_falls_back_to_one_selection(device):
    from khalamari_b200.gqa import GQACore, MixedBatchAttention
    case = make_case(5, "bf16", 64, 8, 128, [300, 40, 900, 77], [1, 24, 1, 19])
    run = DeviceCase(device, case, max_tokens=64)
    mixed = MixedBatchAttention(device, GQACore(128, 64, 8, case.scale), run.dtype, case.page_bytes, run.layout, 64)
    mixed.prepare(case.req_slots, case.token_indices, case.cu_tokens)
    assert len(mixed.plan) == 1
    mixed.record_sdpa(run.stream, run.q, run.kv_pages, run.page_ids, run.output, case.layer_index)
    run.stream.synchronize()
    assert device.check(run.stream) == 0
    assert_within_contract(run.read_output(), case.oracle_output(), "interleaved mix through one selection")
