"""Writes ``tests/golden/attention_cases.npz``: outputs of the CPU oracle (pinned to the reference's known-answer
tests by tests/test_oracle.py) on a few seeded paged batches. The reference itself is Rust and cannot run in the
build image, so these vectors come from its C restatement; they freeze today's oracle so that a later change to
either the oracle or the CUDA path shows up as a difference against a committed file.

Run from the repository root:  python tests/golden/make_golden.py
"""
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from helpers import make_case  # noqa: E402

# name: (seed, dtype, Hq, Hkv, D, histories, q_lens)
CASES = {
    "decode_fp16_config1": (0, "f16", 16, 2, 256, [127, 516, 1023, 2047], [1, 1, 1, 1]),
    "decode_bf16_ragged": (3, "bf16", 64, 8, 128, [0, 15, 16, 530, 1999], [1, 1, 1, 1, 1]),
    "verify_bf16_q4": (5, "bf16", 24, 4, 256, [300, 17], [4, 4]),
    "prefill_bf16_tiles": (7, "bf16", 16, 2, 128, [90, 0], [24, 19]),
}


def build(name):
    seed, dtype_name, hq, hkv, d, histories, q_lens = CASES[name]
    scale = 1.0 / 16.0 if d == 256 else None
    return make_case(seed, dtype_name, hq, hkv, d, histories, q_lens, scale=scale)


def main():
    arrays = {}
    for name in CASES:
        arrays[name] = build(name).oracle_output().astype(np.float32)
    out = Path(__file__).with_name("attention_cases.npz")
    np.savez_compressed(out, **arrays)
    print(out, {k: v.shape for k, v in arrays.items()}, out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
