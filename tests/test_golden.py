"""Committed golden vectors (tests/golden/attention_cases.npz, written by tests/golden/make_golden.py).
CPU: the oracle still reproduces them bit for bit. GPU: the CUDA path matches them within the contract."""
import sys
from pathlib import Path

import numpy as np
import pytest

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"
sys.path.insert(0, str(GOLDEN_DIR))

import make_golden  # noqa: E402
from helpers import DeviceCase, assert_within_contract  # noqa: E402


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN_DIR / "attention_cases.npz")


@pytest.mark.parametrize("name", sorted(make_golden.CASES))
def test_oracle_reproduces_the_committed_vectors(golden, name):
    expected = golden[name]
    actual = make_golden.build(name).oracle_output()
    assert actual.shape == expected.shape
    assert np.array_equal(actual.view(np.uint32), expected.view(np.uint32))


@pytest.mark.gpu
@pytest.mark.parametrize("name", sorted(make_golden.CASES))
def test_cuda_path_matches_the_committed_vectors(golden, name):
    from khalamari_b200.device import Device
    case = make_golden.build(name)
    out = DeviceCase(Device(0), case, max_tokens=max(case.num_tokens, 64)).run()
    assert_within_contract(out, golden[name], name)
