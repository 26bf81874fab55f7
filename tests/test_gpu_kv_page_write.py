"""KV page write through the C ABI (``-m gpu``): the reference's kernel tests
(crates/inference-backend-metal/src/components/gqa/kv_page_write.rs:262-451) byte for byte, then the build's page
geometry, where the written pages are also read back by the attention kernels."""
import numpy as np
import pytest

import oracle
from helpers import DeviceCase, assert_within_contract, make_case, round_to

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    from khalamari_b200.device import Device
    return Device(0)


def _bf16_bits(values):
    bits, _ = oracle.round_bf16(np.asarray(values, dtype=np.float32))
    return bits


def test_replay_matches_page_reference_across_active_counts(device):
    """kv_page_write.rs:284-365: 8 writes over 2 request slots, FP8 pages of 16 bytes, one launch per active count."""
    from khalamari_b200 import kv_page_write as kvw
    from khalamari_b200.device import Buffer, Stream
    from khalamari_b200.request_page_table import GQAPageTableLayout

    stream = Stream(device)
    page_values, num_pages, initial = 16, 4, 0x55
    flat_k_values = [1.0 + i * 0.125 for i in range(16)]
    flat_v_values = [-1.0 - i * 0.125 for i in range(16)]
    req_slot_values = [0, 1, 0, 1, 0, 1, 0, 1]
    token_index_values = [0, 0, 1, 1, 2, 2, 3, 3]
    page_id_values = [0, 1, 2, 3]
    pages = Buffer.from_slice(device, np.full(num_pages * page_values, initial, dtype=np.uint8))
    flat_k = Buffer.from_slice(device, _bf16_bits(flat_k_values))
    flat_v = Buffer.from_slice(device, _bf16_bits(flat_v_values))
    req_slots = Buffer.from_slice(device, np.array(req_slot_values, dtype=np.uint32))
    token_indices = Buffer.from_slice(device, np.array(token_index_values, dtype=np.uint32))
    page_ids = Buffer.from_slice(device, np.array(page_id_values, dtype=np.uint32))
    config = kvw.Config(1, 2, page_values)
    shape = kvw.Shape(8, GQAPageTableLayout(2, 1, 2, 1))
    kernel = kvw.Compute(device, config)
    tokens_per_page = config.num_tokens_per_page()
    assert tokens_per_page == 4
    plane = config.num_kv_heads * tokens_per_page * config.head_dim
    k_bits, v_bits = _bf16_bits(flat_k_values), _bf16_bits(flat_v_values)
    for active in [1, 8, 3, 7, 2, 6, 4, 5]:
        pages.write(0, np.full(num_pages * page_values, initial, dtype=np.uint8))
        kernel.invoke(stream, shape, kvw.Buffers(pages, flat_k, flat_v, req_slots, token_indices, page_ids), active, 0)
        stream.synchronize()
        expected = np.full(num_pages * page_values, initial, dtype=np.uint8)
        for write in range(active):
            slot, token = req_slot_values[write], token_index_values[write]
            page = page_id_values[slot * 2 + token // tokens_per_page]
            for dim in range(config.head_dim):
                offset = (token % tokens_per_page) * config.head_dim + dim
                flat = write * config.head_dim + dim
                expected[page * page_values + offset] = oracle.fp8_from_bf16_bits(k_bits[flat])
                expected[page * page_values + plane + offset] = oracle.fp8_from_bf16_bits(v_bits[flat])
        assert np.array_equal(pages.read(0, expected.size, np.uint8), expected), active
    assert device.check(stream) == 0


def test_fp8_replay_matches_page_reference(device):
    """kv_page_write.rs:367-390: signed zero, subnormals, ties, saturation and infinity, head_dim 9."""
    from khalamari_b200 import kv_page_write as kvw
    from khalamari_b200.device import Buffer, Stream
    from khalamari_b200.request_page_table import GQAPageTableLayout

    stream = Stream(device)
    k_values = [-0.0, 2.0 ** -10, 2.0 ** -9, 1.0625, 1.1875, 400.0, 448.0, 449.0, np.inf]
    v_values = [-x for x in k_values]
    n = len(k_values)
    expected = np.zeros(4 * n, dtype=np.uint8)
    expected[n:2 * n] = oracle.fp8_from_bf16_bits(_bf16_bits(k_values))
    expected[3 * n:4 * n] = oracle.fp8_from_bf16_bits(_bf16_bits(v_values))
    pages = Buffer.new_zeroed(device, expected.size)
    config = kvw.Config(1, n, expected.size)
    shape = kvw.Shape(1, GQAPageTableLayout(1, 1, 1, 1))
    kvw.Compute(device, config).invoke(
        stream, shape,
        kvw.Buffers(pages, Buffer.from_slice(device, _bf16_bits(k_values)), Buffer.from_slice(device, _bf16_bits(v_values)),
                    Buffer.from_slice(device, np.array([0], dtype=np.uint32)),
                    Buffer.from_slice(device, np.array([1], dtype=np.uint32)),
                    Buffer.from_slice(device, np.array([0], dtype=np.uint32))), 1, 0)
    stream.synchronize()
    assert np.array_equal(pages.read(0, expected.size, np.uint8), expected)


def test_shape_rejects_shader_count_overflow(device):
    """kv_page_write.rs:262-282."""
    from khalamari_b200 import abi, kv_page_write as kvw
    from khalamari_b200.device import Buffer, Stream
    from khalamari_b200.request_page_table import GQAPageTableLayout

    stream = Stream(device)
    tiny = Buffer.new_zeroed(device, 64)
    kernel = kvw.Compute(device, kvw.Config(2, 2, 16))
    with pytest.raises(abi.KhError, match="GQA KV page-write threads exceeds the shader u32 count domain"):
        kernel.invoke(stream, kvw.Shape(1 << 30, GQAPageTableLayout(1, 1, 1, 1)),
                      kvw.Buffers(tiny, tiny, tiny, tiny, tiny, tiny), 1, 0)
    with pytest.raises(abi.KhError, match="divisible"):
        kvw.Compute(device, kvw.Config(2, 2, 15))


@pytest.mark.parametrize("kv_fp8", [False, True])
def test_new_tokens_land_where_attention_reads_them(device, kv_fp8):
    """Build geometry (Hkv8, D128, P16, two layers, two page ids per block): the new tokens of a ragged batch
    are written by the kernel into a pool that already holds the history; bytes must equal the oracle's scatter,
    untouched bytes must stay, and (bf16 pages) attention over the written pool must match the oracle."""
    from khalamari_b200 import kv_page_write as kvw
    from khalamari_b200.device import Buffer, Dtype, Stream
    from khalamari_b200.request_page_table import GQAPageTableLayout

    histories, q_lens = [37, 0, 500, 16, 255], [4, 3, 1, 16, 2]
    case = make_case(11, "bf16", 64, 8, 128, histories, q_lens, num_gqa_layers=2, layer_index=1,
                     num_page_ids_per_block=2)
    elem = 1 if kv_fp8 else 2
    page_bytes = case.page_bytes // 2 * elem
    layout = case.layout
    # pool with the history only; the expectation adds the new tokens through the oracle's scatter
    pool_pages = case.pool.size // case.page_bytes
    start = np.full(pool_pages * page_bytes, 0xA5, dtype=np.uint8)
    flat_k, flat_v, slots, positions = [], [], [], []
    for r, (h, q) in enumerate(zip(histories, q_lens)):
        k_bits, _ = round_to("bf16", case.k_f32[r])
        v_bits, _ = round_to("bf16", case.v_f32[r])
        stored_k = oracle.fp8_from_bf16_bits(k_bits) if kv_fp8 else k_bits
        stored_v = oracle.fp8_from_bf16_bits(v_bits) if kv_fp8 else v_bits
        if h:
            oracle.scatter_paged(start, case.page_ids, layout, case.req_slots[r], 1, 16, 8, 128, elem, 0,
                                 stored_k[:h], stored_v[:h])
        flat_k.append(k_bits[h:h + q])
        flat_v.append(v_bits[h:h + q])
        slots += [case.req_slots[r]] * q
        positions += list(range(h, h + q))
    expected = start.copy()
    for r, (h, q) in enumerate(zip(histories, q_lens)):
        k_bits, _ = round_to("bf16", case.k_f32[r])
        v_bits, _ = round_to("bf16", case.v_f32[r])
        stored_k = oracle.fp8_from_bf16_bits(k_bits[h:h + q]) if kv_fp8 else k_bits[h:h + q]
        stored_v = oracle.fp8_from_bf16_bits(v_bits[h:h + q]) if kv_fp8 else v_bits[h:h + q]
        oracle.scatter_paged(expected, case.page_ids, layout, case.req_slots[r], 1, 16, 8, 128, elem, h,
                             stored_k, stored_v)
    writes = len(slots)
    capacity = writes + 3  # recorded capacity above the active count: the padding rows must not be written
    pad_rows = np.full((3, 8, 128), 0x7FC0, dtype=np.uint16)
    stream = Stream(device)
    pages = Buffer.from_slice(device, start)
    buffers = kvw.Buffers(pages, Buffer.from_slice(device, np.concatenate(flat_k + [pad_rows])),
                          Buffer.from_slice(device, np.concatenate(flat_v + [pad_rows])),
                          Buffer.from_slice(device, np.array(slots + [0] * 3, dtype=np.uint32)),
                          Buffer.from_slice(device, np.array(positions + [0] * 3, dtype=np.uint32)),
                          Buffer.from_slice(device, case.page_ids))
    config = kvw.Config(8, 128, page_bytes, Dtype.Bfloat16, Dtype.Fp8E4M3FN if kv_fp8 else Dtype.Bfloat16)
    shape = kvw.Shape(capacity, GQAPageTableLayout(layout.num_req_slots, 2, layout.num_blocks, 2))
    assert config.num_tokens_per_page() == 16
    kvw.Compute(device, config).invoke(stream, shape, buffers, writes, 1)
    stream.synchronize()
    assert device.check(stream) == 0
    assert np.array_equal(pages.read(0, expected.size, np.uint8), expected)
    if not kv_fp8:
        run = DeviceCase(device, case)
        run.kv_pages = pages
        assert_within_contract(run.run(), case.oracle_output(), "attention over pages the write kernel filled")
