"""CPU oracle for the paged GQA split-KV SDPA path (test infrastructure, not product code).

``gqa_oracle.c`` restates the reference's CPU GQA SDPA
(crates/inference-executor-core/src/attn/gqa/reference.rs:15-78) and the page index arithmetic
its kernels share. This module compiles it with gcc and exposes it through ctypes. Only the test
suite, the smoke check and the CPU-baseline leg of the benchmark may import it.

Parity pin: checked against the reference's own known-answer tests (reference.rs:84-115,
crates/inference-executor-core/src/reference.rs:102-108). The reference itself is Rust and was
not run: no Rust toolchain exists in this image.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SRC = _HERE / "gqa_oracle.c"
_SO = _HERE / "libkh_oracle.so"

_u32p = np.ctypeslib.ndpointer(dtype=np.uint32, flags="C_CONTIGUOUS")
_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")


def build(force: bool = False) -> Path:
    """Compile the C restatement into ``oracle/libkh_oracle.so`` (gcc, OpenMP, no FP contraction)."""
    if not force and _SO.exists() and _SO.stat().st_mtime >= _SRC.stat().st_mtime:
        return _SO
    tmp = _SO.with_suffix(f".so.tmp{os.getpid()}")
    cmd = [
        "gcc", "-O2", "-std=c11", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
        "-fvisibility=hidden", "-o", str(tmp), str(_SRC), "-lm",
    ]
    subprocess.run(cmd, check=True)
    os.replace(tmp, _SO)
    return _SO


_lib = None


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = build()
        handle = ctypes.CDLL(str(path))
        handle.kh_oracle_softmax.argtypes = [_f32p, ctypes.c_uint64, _f32p]
        handle.kh_oracle_softmax.restype = ctypes.c_int
        handle.kh_oracle_projected_gqa.argtypes = [
            ctypes.c_uint32, _u32p, _u32p, _f32p, ctypes.POINTER(ctypes.c_void_p), ctypes.POINTER(ctypes.c_void_p),
            ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_float, _f32p, ctypes.c_int32,
        ]
        handle.kh_oracle_projected_gqa.restype = ctypes.c_int
        handle.kh_oracle_row.argtypes = [
            _f32p, _f32p, _f32p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_float,
            _f32p,
        ]
        handle.kh_oracle_row.restype = ctypes.c_int
        handle.kh_oracle_gather_paged.argtypes = [
            ctypes.c_void_p, ctypes.c_uint64, _u32p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_uint32,
            ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32,
            ctypes.c_uint32, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
        ]
        handle.kh_oracle_gather_paged.restype = ctypes.c_int
        handle.kh_oracle_scatter_paged.argtypes = [
            ctypes.c_void_p, ctypes.c_uint64, _u32p, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_uint32,
            ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32,
            ctypes.c_uint32, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p,
        ]
        handle.kh_oracle_scatter_paged.restype = ctypes.c_int
        handle.kh_oracle_merge_partials.argtypes = [
            ctypes.c_uint32, _f32p, _f32p, _f32p, ctypes.c_uint64, ctypes.c_uint32, _f32p,
            ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_float),
        ]
        handle.kh_oracle_merge_partials.restype = None
        handle.kh_oracle_partial_row.argtypes = [
            _f32p, _f32p, _f32p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_uint32, ctypes.c_uint32,
            ctypes.c_float, _f32p, ctypes.POINTER(ctypes.c_float), ctypes.POINTER(ctypes.c_float),
        ]
        handle.kh_oracle_partial_row.restype = None
        handle.kh_oracle_fp8_from_bf16.argtypes = [ctypes.c_uint16]
        handle.kh_oracle_fp8_from_bf16.restype = ctypes.c_uint8
        handle.kh_oracle_fp8_to_bf16.argtypes = [ctypes.c_uint8]
        handle.kh_oracle_fp8_to_bf16.restype = ctypes.c_uint16
        handle.kh_oracle_round_bf16.argtypes = [_f32p, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_void_p]
        handle.kh_oracle_round_bf16.restype = None
        handle.kh_oracle_generated_values.argtypes = [ctypes.c_uint64, ctypes.c_uint32, ctypes.c_int32, _f32p]
        handle.kh_oracle_generated_values.restype = None
        handle.kh_oracle_fixture_values.argtypes = [ctypes.c_uint64, ctypes.c_float, ctypes.c_uint64, _f32p]
        handle.kh_oracle_fixture_values.restype = None
        handle.kh_oracle_max_threads.argtypes = []
        handle.kh_oracle_max_threads.restype = ctypes.c_int32
        _lib = handle
    return _lib


class PageTableLayout:
    """Block-table shape ``[num_req_slots, num_gqa_layers, num_blocks, num_page_ids_per_block]``
    (crates/inference-executor-metal/src/attn/gqa/request_page_table.rs:7-20)."""

    def __init__(self, num_req_slots: int, num_gqa_layers: int, num_blocks: int, num_page_ids_per_block: int):
        self.num_req_slots = num_req_slots
        self.num_gqa_layers = num_gqa_layers
        self.num_blocks = num_blocks
        self.num_page_ids_per_block = num_page_ids_per_block

    def num_page_ids(self) -> int:
        return self.num_req_slots * self.num_gqa_layers * self.num_blocks * self.num_page_ids_per_block


def softmax(logits: np.ndarray) -> np.ndarray:
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    out = np.empty_like(logits)
    rc = lib().kh_oracle_softmax(logits, logits.size, out)
    if rc:
        raise AssertionError("softmax reference requires finite positive total")
    return out


def projected_gqa(cu_tokens, token_indices, q, context_k_by_req, context_v_by_req, head_dim, num_q_heads,
                  num_kv_heads, scale, num_threads: int = 1) -> np.ndarray:
    """``projected_gqa_reference`` (reference.rs:15-78). q: f32 ``[T*Hq*D]``; per-request K/V f32
    ``[ctx*Hkv*D]``. Returns f32 ``[T, Hq, D]``."""
    cu = np.ascontiguousarray(cu_tokens, dtype=np.uint32)
    ti = np.ascontiguousarray(token_indices, dtype=np.uint32)
    num_reqs = ti.size
    assert cu.size == num_reqs + 1
    qf = np.ascontiguousarray(q, dtype=np.float32).reshape(-1)
    total = int(cu[-1])
    assert qf.size == total * num_q_heads * head_dim
    ks = [np.ascontiguousarray(k, dtype=np.float32).reshape(-1) for k in context_k_by_req]
    vs = [np.ascontiguousarray(v, dtype=np.float32).reshape(-1) for v in context_v_by_req]
    assert len(ks) == num_reqs and len(vs) == num_reqs
    for r in range(num_reqs):
        ctx = int(ti[r]) + int(cu[r + 1] - cu[r])
        assert ks[r].size == ctx * num_kv_heads * head_dim, (r, ks[r].size, ctx)
        assert vs[r].size == ctx * num_kv_heads * head_dim
    kp = (ctypes.c_void_p * max(num_reqs, 1))(*[k.ctypes.data for k in ks])
    vp = (ctypes.c_void_p * max(num_reqs, 1))(*[v.ctypes.data for v in vs])
    out = np.zeros(total * num_q_heads * head_dim, dtype=np.float32)
    rc = lib().kh_oracle_projected_gqa(num_reqs, cu, ti, qf, kp, vp, head_dim, num_q_heads, num_kv_heads,
                                       float(scale), out, int(num_threads))
    if rc:
        raise AssertionError(f"projected_gqa_reference rejected its input (code {rc})")
    return out.reshape(total, num_q_heads, head_dim)


def oracle_row(q_row, k, v, visible, num_kv_heads, head_dim, kv_head, scale) -> np.ndarray:
    q_row = np.ascontiguousarray(q_row, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float32).reshape(-1)
    v = np.ascontiguousarray(v, dtype=np.float32).reshape(-1)
    out = np.zeros(head_dim, dtype=np.float32)
    rc = lib().kh_oracle_row(q_row, k, v, visible, num_kv_heads, head_dim, kv_head, float(scale), out)
    if rc:
        raise AssertionError("oracle row rejected its input")
    return out


def gather_paged(kv_pages: np.ndarray, page_ids: np.ndarray, layout: PageTableLayout, req_slot: int,
                 layer_index: int, tokens_per_page: int, num_kv_heads: int, head_dim: int, elem_bytes: int,
                 num_tokens: int, want_addresses: bool = False):
    """Gather tokens ``[0, num_tokens)`` of one request from the paged pool (byte moves only).
    Returns (K, V) as uint8 ``[num_tokens, Hkv, D*elem_bytes]`` and, optionally, the byte address of
    every K and V row."""
    pages = np.ascontiguousarray(kv_pages).view(np.uint8).reshape(-1)
    ids = np.ascontiguousarray(page_ids, dtype=np.uint32).reshape(-1)
    shape = (num_tokens, num_kv_heads, head_dim * elem_bytes)
    out_k = np.zeros(shape, dtype=np.uint8)
    out_v = np.zeros(shape, dtype=np.uint8)
    ka = np.zeros((num_tokens, num_kv_heads), dtype=np.uint64) if want_addresses else None
    va = np.zeros((num_tokens, num_kv_heads), dtype=np.uint64) if want_addresses else None
    rc = lib().kh_oracle_gather_paged(
        pages.ctypes.data, pages.size, ids, ids.size, req_slot, layer_index, layout.num_gqa_layers,
        layout.num_blocks, layout.num_page_ids_per_block, tokens_per_page, num_kv_heads, head_dim, elem_bytes,
        num_tokens, out_k.ctypes.data, out_v.ctypes.data,
        ka.ctypes.data if want_addresses else None, va.ctypes.data if want_addresses else None)
    if rc:
        raise IndexError(f"paged gather index out of range (code {rc})")
    if want_addresses:
        return out_k, out_v, ka, va
    return out_k, out_v


def scatter_paged(kv_pages: np.ndarray, page_ids: np.ndarray, layout: PageTableLayout, req_slot: int,
                  layer_index: int, tokens_per_page: int, num_kv_heads: int, head_dim: int, elem_bytes: int,
                  token_begin: int, k: np.ndarray, v: np.ndarray) -> None:
    """Write contiguous K/V rows ``[n, Hkv, D]`` of a request into its pages (in place)."""
    assert kv_pages.flags["C_CONTIGUOUS"] and kv_pages.dtype == np.uint8
    ids = np.ascontiguousarray(page_ids, dtype=np.uint32).reshape(-1)
    kb = np.ascontiguousarray(k).view(np.uint8).reshape(-1)
    vb = np.ascontiguousarray(v).view(np.uint8).reshape(-1)
    row = num_kv_heads * head_dim * elem_bytes
    assert kb.size == vb.size and kb.size % row == 0
    rc = lib().kh_oracle_scatter_paged(
        kv_pages.ctypes.data, kv_pages.size, ids, ids.size, req_slot, layer_index, layout.num_gqa_layers,
        layout.num_blocks, layout.num_page_ids_per_block, tokens_per_page, num_kv_heads, head_dim, elem_bytes,
        token_begin, kb.size // row, kb.ctypes.data, vb.ctypes.data)
    if rc:
        raise IndexError(f"paged scatter index out of range (code {rc})")


def merge_partials(exp_sums, max_logits, partial_out):
    """LSE merge of ``n`` partial rows ``[n, D]``. Returns (out[D], exp_sum, max_logit)."""
    exp_sums = np.ascontiguousarray(exp_sums, dtype=np.float32)
    max_logits = np.ascontiguousarray(max_logits, dtype=np.float32)
    partial_out = np.ascontiguousarray(partial_out, dtype=np.float32)
    n, d = partial_out.shape
    out = np.zeros(d, dtype=np.float32)
    s = ctypes.c_float()
    m = ctypes.c_float()
    lib().kh_oracle_merge_partials(n, exp_sums, max_logits, partial_out.reshape(-1), d, d, out, ctypes.byref(s),
                                   ctypes.byref(m))
    return out, s.value, m.value


def partial_row(q_row, k, v, kv_begin, kv_end, num_kv_heads, head_dim, kv_head, scale):
    """One split-KV partial (out[D], exp_sum, max_logit) over tokens ``[kv_begin, kv_end)``."""
    q_row = np.ascontiguousarray(q_row, dtype=np.float32)
    k = np.ascontiguousarray(k, dtype=np.float32).reshape(-1)
    v = np.ascontiguousarray(v, dtype=np.float32).reshape(-1)
    out = np.zeros(head_dim, dtype=np.float32)
    s = ctypes.c_float()
    m = ctypes.c_float()
    lib().kh_oracle_partial_row(q_row, k, v, kv_begin, kv_end, num_kv_heads, head_dim, kv_head, float(scale), out,
                                ctypes.byref(s), ctypes.byref(m))
    return out, s.value, m.value


def round_bf16(values: np.ndarray):
    """Round f32 to bfloat16 (nearest even). Returns (uint16 bits, f32 round-trip)."""
    flat = np.ascontiguousarray(values, dtype=np.float32).reshape(-1)
    bits = np.empty(flat.size, dtype=np.uint16)
    back = np.empty(flat.size, dtype=np.float32)
    lib().kh_oracle_round_bf16(flat, flat.size, bits.ctypes.data, back.ctypes.data)
    return bits.reshape(values.shape), back.reshape(values.shape)


def bf16_bits_to_f32(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def round_f16(values: np.ndarray):
    """Round f32 to IEEE half (nearest even). Returns (uint16 bits, f32 round-trip)."""
    half = np.asarray(values, dtype=np.float32).astype(np.float16)
    return half.view(np.uint16), half.astype(np.float32)


def generated_values(count: int, seed: int, centered_bf16: bool = False) -> np.ndarray:
    """LCG generators of the reference tests (sliced_kv_test.rs:501-509, sliced_q_test.rs:611-619)."""
    out = np.empty(count, dtype=np.float32)
    lib().kh_oracle_generated_values(count, seed & 0xFFFFFFFF, int(centered_bf16), out)
    return out


def fixture_values(count: int, scale: float, pattern_offset: int) -> np.ndarray:
    """``fixture_values`` of sliced_kv_test.rs:495-499."""
    out = np.empty(count, dtype=np.float32)
    lib().kh_oracle_fixture_values(count, float(scale), pattern_offset, out)
    return out


def fp8_from_bf16_bits(bits) -> np.ndarray:
    """FP8 E4M3FN encoding of bf16 bit patterns (fp8.rs:19-44), element by element."""
    flat = np.ascontiguousarray(bits, dtype=np.uint16).reshape(-1)
    fn = lib().kh_oracle_fp8_from_bf16
    return np.array([fn(int(b)) for b in flat], dtype=np.uint8).reshape(np.shape(bits))


def fp8_to_bf16_bits(bits) -> np.ndarray:
    """bf16 bit patterns of FP8 E4M3FN codes (fp8.rs:46-58)."""
    flat = np.ascontiguousarray(bits, dtype=np.uint8).reshape(-1)
    fn = lib().kh_oracle_fp8_to_bf16
    return np.array([fn(int(b)) for b in flat], dtype=np.uint16).reshape(np.shape(bits))


def max_threads() -> int:
    return int(lib().kh_oracle_max_threads())
