"""Seeded random batches (``-m gpu``): head layouts, head dimensions, page sizes, query lengths, histories and KV
slices drawn at random, every case checked against the CPU oracle. The seeds are fixed, so a failure names a
reproducible case."""
import os

import numpy as np
import pytest

from helpers import DeviceCase, assert_within_contract, make_case

pytestmark = pytest.mark.gpu

HEADS = [(64, 8), (16, 2), (24, 4), (32, 8), (8, 8), (32, 2), (12, 2)]


@pytest.fixture(scope="module")
def device():
    from khalamari_b200.device import Device
    return Device(0)


# KH_FUZZ_SEEDS widens the sweep for an occasional longer run
@pytest.mark.parametrize("seed", range(int(os.environ.get("KH_FUZZ_SEEDS", "24"))))
def test_random_batches_match_the_oracle(device, seed):
    rng = np.random.default_rng(1000 + seed)
    hq, hkv = HEADS[int(rng.integers(len(HEADS)))]
    d = int(rng.choice([128, 256]))
    page = int(rng.choice([8, 16]))
    dtype_name = "bf16" if rng.random() < 0.8 else "f16"
    num_reqs = int(rng.integers(1, 7))
    mode = rng.random()
    if mode < 0.4:        # decode
        q_lens = [1] * num_reqs
    elif mode < 0.7:      # verify
        q_lens = [int(rng.choice([2, 4, 8]))] * num_reqs
    else:                 # mixed prefill chunks and decode tokens
        q_lens = [int(rng.integers(1, 48)) for _ in range(num_reqs)]
    longest = 2200 if seed < 24 else int(rng.choice([300, 2200, 9000]))
    histories = [int(rng.integers(0, longest)) if rng.random() < 0.8 else 0 for _ in range(num_reqs)]
    case = make_case(2000 + seed, dtype_name, hq, hkv, d, histories, q_lens, tokens_per_page=page,
                     num_gqa_layers=int(rng.integers(1, 3)), layer_index=0,
                     num_page_ids_per_block=int(rng.choice([1, 2, 4])))
    run = DeviceCase(device, case, max_tokens=max(64, case.num_tokens))
    out = run.run()
    assert_within_contract(out, case.oracle_output(),
                           f"seed {seed}: Hq{hq}/Hkv{hkv}/D{d}/P{page} {dtype_name} q{q_lens} h{histories}")
