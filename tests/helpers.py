"""Shared builders for the parity tests: seeded paged KV pools, block tables and the oracle's answer.

RNG: ``numpy.random.default_rng(seed)`` (PCG64) standard normals, rounded to the storage dtype and upcast
to f32 for the oracle, as the reference's tests do (sliced_kv_test.rs:171-182)."""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

import oracle

ABS_TOL = 2.0e-3   # max-abs bound of the build contract
REL_TOL = 1.0e-2   # max-rel bound of the build contract


def round_to(dtype_name: str, values: np.ndarray):
    """Returns (uint16 storage bits, f32 value of those bits)."""
    if dtype_name == "bf16":
        return oracle.round_bf16(values)
    if dtype_name == "f16":
        return oracle.round_f16(values)
    raise ValueError(dtype_name)


def bits_to_f32(dtype_name: str, bits: np.ndarray) -> np.ndarray:
    if dtype_name == "bf16":
        return oracle.bf16_bits_to_f32(bits)
    return np.ascontiguousarray(bits, dtype=np.uint16).view(np.float16).astype(np.float32)


def nan_bits(dtype_name: str) -> int:
    return 0x7FC0 if dtype_name == "bf16" else 0x7E00


def assert_within_contract(actual: np.ndarray, expected: np.ndarray, what: str = "") -> tuple[float, float]:
    """Pass rule, per element: |a - b| <= 2e-3 OR |a - b| <= 1e-2 * |b|. Returns (max abs, max rel)."""
    actual = np.asarray(actual, dtype=np.float32)
    expected = np.asarray(expected, dtype=np.float32)
    assert actual.shape == expected.shape, (actual.shape, expected.shape)
    assert np.all(np.isfinite(actual)), f"{what}: non-finite output"
    err = np.abs(actual - expected)
    ok = (err <= ABS_TOL) | (err <= REL_TOL * np.abs(expected))
    max_abs = float(err.max()) if err.size else 0.0
    rel = err / np.maximum(np.abs(expected), 1e-30)
    max_rel = float(rel[err > ABS_TOL].max()) if np.any(err > ABS_TOL) else 0.0
    assert np.all(ok), (f"{what}: {np.count_nonzero(~ok)} of {ok.size} elements outside tolerance; "
                        f"max abs {max_abs:.3e}, max rel beyond abs bound {max_rel:.3e}")
    return max_abs, max_rel


@dataclass
class PagedCase:
    dtype_name: str
    num_q_heads: int
    num_kv_heads: int
    head_dim: int
    tokens_per_page: int
    scale: float
    layout: oracle.PageTableLayout
    layer_index: int
    req_slots: list
    token_indices: list          # history length per request
    q_lens: list
    cu_tokens: list
    q_bits: np.ndarray           # [T, Hq, D] uint16
    q_f32: np.ndarray            # rounded values
    pool: np.ndarray             # uint8 bytes of the page pool
    page_ids: np.ndarray         # uint32 flat table
    k_f32: list = field(default_factory=list)   # per request [ctx, Hkv, D]
    v_f32: list = field(default_factory=list)
    kv_elem_bytes: int = 2       # 1: the pages hold FP8 E4M3FN codes (the reference's cache format)

    @property
    def page_bytes(self) -> int:
        return 2 * self.num_kv_heads * self.tokens_per_page * self.head_dim * self.kv_elem_bytes

    @property
    def num_tokens(self) -> int:
        return int(self.cu_tokens[-1])

    def contexts(self) -> list:
        return [h + q for h, q in zip(self.token_indices, self.q_lens)]

    def kv_bytes(self) -> int:
        """Algorithmic KV bytes: every (request, kv head, visible token) K and V row counted once."""
        return sum(self.contexts()) * 2 * self.num_kv_heads * self.head_dim * self.kv_elem_bytes

    def oracle_output(self, num_threads: int = 0) -> np.ndarray:
        threads = num_threads or oracle.max_threads()
        return oracle.projected_gqa(self.cu_tokens, self.token_indices, self.q_f32, self.k_f32, self.v_f32,
                                    self.head_dim, self.num_q_heads, self.num_kv_heads, self.scale, threads)


def make_case(seed: int, dtype_name: str, num_q_heads: int, num_kv_heads: int, head_dim: int, histories, q_lens,
              tokens_per_page: int = 16, num_gqa_layers: int = 1, layer_index: int = 0, num_page_ids_per_block: int = 1,
              pool_pages: int | None = None, extra_slots: int = 0, poison: bool = True, scale: float | None = None,
              keep_f32: bool = True, q_std: float = 1.0, kv_fp8: bool = False, kv_std: float = 1.0,
              workers: int = 1) -> PagedCase:
    """Builds requests with ``histories[r]`` cached tokens and ``q_lens[r]`` new tokens (already in the cache,
    as after the page-write step), a shared pool whose pages are handed out by a seeded permutation, and an
    unwritten pool filled with NaN bit patterns when ``poison`` (the tail of a last page must not leak).
    ``kv_fp8``: K and V go through the reference's page-write conversion (rounded to bf16, then to FP8 E4M3FN,
    components/gqa/fp8.rs:19-44); the pool holds the codes and the oracle sees their decoded values, as in
    sliced_kv_test.rs:171-182.
    ``workers`` > 1 (the full-size configurations): K and V are drawn in chunks of 16,384 tokens, each from a
    generator of its own seeded ``[seed, request, first token]``, on a pool of threads; chunk boundaries fall on page
    boundaries, so the chunks fill disjoint pages side by side."""
    rng = np.random.default_rng(seed)
    num_reqs = len(histories)
    contexts = [int(h) + int(q) for h, q in zip(histories, q_lens)]
    pages_needed = [-(-c // tokens_per_page) for c in contexts]
    max_pages = max(pages_needed)
    num_blocks = -(-max_pages // num_page_ids_per_block)
    num_slots = num_reqs + extra_slots
    layout = oracle.PageTableLayout(num_slots, num_gqa_layers, num_blocks, num_page_ids_per_block)
    total_pages = sum(pages_needed)
    if pool_pages is None:
        pool_pages = total_pages + 3
    assert pool_pages >= total_pages
    kv_elem = 1 if kv_fp8 else 2
    page_bytes = 2 * num_kv_heads * tokens_per_page * head_dim * kv_elem
    if kv_fp8:
        pool = np.full(pool_pages * page_bytes, 0x7F if poison else 0, dtype=np.uint8)  # 0x7f: the NaN code
    else:
        if poison:
            pool = np.full(pool_pages * page_bytes // 2, nan_bits(dtype_name), dtype=np.uint16).view(np.uint8)
        else:
            pool = np.zeros(pool_pages * page_bytes, dtype=np.uint8)
    table = np.zeros(layout.num_page_ids(), dtype=np.uint32)
    # request r lives in slot order shuffled so that slot != request index
    slots = rng.permutation(num_slots)[:num_reqs].astype(np.uint32)
    free_pages = rng.permutation(pool_pages).astype(np.uint32)
    first_page = np.concatenate([[0], np.cumsum(pages_needed)]).astype(np.int64)
    for r in range(num_reqs):
        ids = free_pages[first_page[r]:first_page[r + 1]]
        base = ((int(slots[r]) * num_gqa_layers + layer_index) * num_blocks) * num_page_ids_per_block
        table[base:base + ids.size] = ids

    def fill(r, generator):
        k = generator.standard_normal((contexts[r], num_kv_heads, head_dim), dtype=np.float32) * np.float32(kv_std)
        v = generator.standard_normal((contexts[r], num_kv_heads, head_dim), dtype=np.float32) * np.float32(kv_std)
        if kv_fp8:
            k_bits, k_round = fp8_codes(k)
            v_bits, v_round = fp8_codes(v)
        else:
            k_bits, k_round = round_to(dtype_name, k)
            v_bits, v_round = round_to(dtype_name, v)
        oracle.scatter_paged(pool, table, layout, int(slots[r]), layer_index, tokens_per_page, num_kv_heads,
                             head_dim, kv_elem, 0, k_bits, v_bits)
        return (k_round, v_round) if keep_f32 else None

    if workers > 1:
        from concurrent.futures import ThreadPoolExecutor
        chunk_tokens = 16384
        whole = [(np.empty((c, num_kv_heads, head_dim), np.float32), np.empty((c, num_kv_heads, head_dim), np.float32))
                 if keep_f32 else None for c in contexts]

        def fill_chunk(unit):
            r, begin = unit
            end = min(begin + chunk_tokens, contexts[r])
            generator = np.random.default_rng([seed, r, begin])
            shape = (end - begin, num_kv_heads, head_dim)
            k = generator.standard_normal(shape, dtype=np.float32) * np.float32(kv_std)
            v = generator.standard_normal(shape, dtype=np.float32) * np.float32(kv_std)
            k_bits, k_round = fp8_codes(k) if kv_fp8 else round_to(dtype_name, k)
            v_bits, v_round = fp8_codes(v) if kv_fp8 else round_to(dtype_name, v)
            oracle.scatter_paged(pool, table, layout, int(slots[r]), layer_index, tokens_per_page, num_kv_heads,
                                 head_dim, kv_elem, begin, k_bits, v_bits)
            if keep_f32:
                whole[r][0][begin:end] = k_round
                whole[r][1][begin:end] = v_round

        units = [(r, begin) for r in range(num_reqs) for begin in range(0, contexts[r], chunk_tokens)]
        with ThreadPoolExecutor(workers) as pool_of_threads:
            list(pool_of_threads.map(fill_chunk, units))
        filled = whole
    else:
        filled = [fill(r, rng) for r in range(num_reqs)]
    case_k = [f[0] for f in filled] if keep_f32 else []
    case_v = [f[1] for f in filled] if keep_f32 else []
    cu = [0]
    for q in q_lens:
        cu.append(cu[-1] + int(q))
    q = rng.standard_normal((cu[-1], num_q_heads, head_dim), dtype=np.float32) * np.float32(q_std)
    q_bits, q_round = round_to(dtype_name, q)
    if scale is None:
        scale = 1.0 / float(np.sqrt(head_dim))
    return PagedCase(dtype_name, num_q_heads, num_kv_heads, head_dim, tokens_per_page, scale, layout, layer_index,
                     slots.tolist(), [int(h) for h in histories], [int(x) for x in q_lens], cu, q_bits, q_round, pool,
                     table, case_k, case_v, kv_elem)


def fp8_codes(values: np.ndarray):
    """Returns (uint8 FP8 E4M3FN codes of the bf16-rounded values, f32 value of those codes)."""
    bf16_bits, _ = oracle.round_bf16(values)
    codes = oracle.fp8_from_bf16_bits(bf16_bits.reshape(-1)).reshape(values.shape)
    decoded = oracle.bf16_bits_to_f32(oracle.fp8_to_bf16_bits(codes.reshape(-1))).reshape(values.shape)
    return codes, decoded


class DeviceCase:
    """Uploads a ``PagedCase`` and runs it through ``GQAAttention`` (the component seam)."""

    def __init__(self, device, case: PagedCase, max_tokens: int | None = None, policy=None, selector=None):
        from khalamari_b200.device import Buffer, Dtype, Stream
        from khalamari_b200.gqa import GQAAttention, GQACore
        from khalamari_b200.request_page_table import GQAPageTableLayout
        from khalamari_b200.selector import SelectorPolicy

        self.case = case
        self.device = device
        self.dtype = Dtype.Bfloat16 if case.dtype_name == "bf16" else Dtype.Float16
        self.layout = GQAPageTableLayout(case.layout.num_req_slots, case.layout.num_gqa_layers,
                                         case.layout.num_blocks, case.layout.num_page_ids_per_block)
        self.stream = Stream(device)
        self.kv_pages = Buffer.from_slice(device, case.pool)
        self.page_ids = Buffer.from_slice(device, case.page_ids)
        row = case.num_q_heads * case.head_dim
        self.canary = 0x4228 if case.dtype_name == "bf16" else 0x5140  # 42.0
        self.attention = GQAAttention(
            device, GQACore(case.head_dim, case.num_q_heads, case.num_kv_heads, case.scale), self.dtype,
            case.page_bytes, self.layout, max_tokens or max(case.num_tokens, 1),
            policy if policy is not None else SelectorPolicy.B200, selector,
            kv_dtype=Dtype.Fp8E4M3FN if case.kv_elem_bytes == 1 else None)
        # Q and output are sized for the recorded token capacity (the replay bucket of the batch), as the executor
        # sizes them; rows past the active tokens hold NaN bits (Q) and a canary (output)
        capacity = self.attention.policy.q_token_ranges.capacity(max(case.num_tokens, 1))
        q_rows = np.full(capacity * row, nan_bits(case.dtype_name), dtype=np.uint16)
        q_rows[:case.num_tokens * row] = np.ascontiguousarray(case.q_bits).reshape(-1)
        self.q = Buffer.from_slice(device, q_rows)
        self.out_rows = capacity + 2
        self.output = Buffer.from_slice(device, np.full(self.out_rows * row, self.canary, dtype=np.uint16))

    def run(self, selection=None, fused: bool | None = None) -> np.ndarray:
        """Runs the batch through map + reduce in one launch and, unless ``fused`` pins one form, also through the
        reference's two-launch form (invoke_map, invoke_reduce); both must produce the same bits."""
        case = self.case
        self.attention.prepare(case.req_slots, case.token_indices, case.cu_tokens, selection=selection)
        outputs = []
        for mode in ([True, False] if fused is None else [fused]):
            self.attention.fused = mode
            self.output.write(0, np.full(self.out_rows * case.num_q_heads * case.head_dim, self.canary, dtype=np.uint16))
            self.attention.record_sdpa(self.stream, self.q, self.kv_pages, self.page_ids, self.output,
                                       case.layer_index)
            self.stream.synchronize()
            assert self.device.check(self.stream) == 0
            outputs.append(self.read_output())
            counters = self.attention.arrival_counters.read(0, self.attention.arrival_counters.len_bytes() // 4,
                                                            np.uint32)
            assert not counters.any(), "arrival counters must be left zero"
        self.attention.fused = False
        if len(outputs) == 2:
            # Same inputs, two kernels (the one-launch form always runs the warp-level instance; a one-partial
            # range is written straight from registers there): they agree to the rounding of the output type,
            # checked with the contract's bound
            assert_within_contract(outputs[0], outputs[1], "one-launch against two-launch")
        return outputs[0]

    def read_output(self) -> np.ndarray:
        case = self.case
        row = case.num_q_heads * case.head_dim
        bits = self.output.read(0, self.out_rows * row, np.uint16)
        tail = bits[case.num_tokens * row:]
        assert np.all(tail == self.canary), "rows past the active tokens were written"
        return bits_to_f32(case.dtype_name, bits[:case.num_tokens * row]).reshape(case.num_tokens, case.num_q_heads,
                                                                                 case.head_dim)
