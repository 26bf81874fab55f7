"""FP8 E4M3FN storage codec: the reference's own tests
(crates/inference-backend-metal/src/components/gqa/fp8.rs:64-139) run against the oracle's restatement and
against the library's host-side codec (bit arithmetic, the same function the page-write kernel uses)."""
import math

import numpy as np
import pytest

import oracle
from khalamari_b200 import kv_page_write


def _bf16(value: float) -> int:
    bits, _ = oracle.round_bf16(np.array([value], dtype=np.float32))
    return int(bits[0])


def _f32(bf16_bits: int) -> float:
    return float(oracle.bf16_bits_to_f32(np.array([bf16_bits], dtype=np.uint16))[0])


def _oracle_encode(bits: int) -> int:
    return int(oracle.lib().kh_oracle_fp8_from_bf16(bits))


def _oracle_decode(bits: int) -> int:
    return int(oracle.lib().kh_oracle_fp8_to_bf16(bits))


CODECS = [pytest.param((_oracle_encode, _oracle_decode), id="oracle"),
          pytest.param((kv_page_write.bf16_to_fp8_e4m3, kv_page_write.fp8_e4m3_to_bf16), id="library")]


@pytest.mark.parametrize("codec", CODECS)
def test_e4m3fn_fixed_encodings_and_saturation(codec):
    encode, _ = codec
    cases = [(0.0, 0x00), (-0.0, 0x80), (2.0 ** -9, 0x01), (2.0 ** -6, 0x08), (1.0, 0x38), (1.5, 0x3C),
             (448.0, 0x7E), (-448.0, 0xFE), (449.0, 0x7E), (-449.0, 0xFE), (math.inf, 0x7E), (-math.inf, 0xFE)]
    for value, expected in cases:
        assert encode(_bf16(value)) == expected, value
    assert encode(0x7FC0) & 0x7F == 0x7F  # NaN stays NaN


@pytest.mark.parametrize("codec", CODECS)
def test_e4m3fn_rounds_ties_to_even(codec):
    encode, _ = codec
    assert encode(_bf16(1.0625)) == encode(_bf16(1.0))
    assert encode(_bf16(1.1875)) == encode(_bf16(1.25))


@pytest.mark.parametrize("codec", CODECS)
def test_e4m3fn_exhaustive_finite_round_trip(codec):
    encode, decode = codec
    for bits in range(256):
        if bits & 0x7F == 0x7F:
            continue
        assert encode(decode(bits)) == bits


@pytest.mark.parametrize("codec", CODECS)
def test_e4m3fn_quantization_error_bounds(codec):
    encode, decode = codec
    min_normal = 2.0 ** -6
    for sample in range(0, 4097, 7):
        source = _bf16(min_normal * sample / 4096.0)
        error = abs(_f32(decode(encode(source))) - _f32(source))
        assert error <= 2.0 ** -10
    for sample in range(0, 458737, 911):
        value = min_normal + sample / 1024.0
        if value > kv_page_write.MAX_FINITE:
            break
        source = _bf16(value)
        relative = abs(_f32(decode(encode(source))) - _f32(source)) / _f32(source)
        assert relative <= 0.0625


def test_library_codec_equals_the_oracle_on_every_bf16_value():
    encode = kv_page_write.bf16_to_fp8_e4m3
    for bits in range(0, 65536):
        ours, theirs = encode(bits), _oracle_encode(bits)
        assert ours == theirs or (ours & 0x7F == 0x7F and theirs & 0x7F == 0x7F), hex(bits)
    for bits in range(256):
        assert kv_page_write.fp8_e4m3_to_bf16(bits) == _oracle_decode(bits)


def test_fp8_page_pool_fixture_round_trips_through_the_paged_gather():
    """The FP8 attention fixture (helpers.make_case with kv_fp8): the codes gathered back from the pool decode to
    the values the oracle is given, and the quality bound of sliced_kv_test.rs:69-114 holds between attention on
    the decoded values and on the bf16 values they came from (mean abs error <= 0.025 of the output scale)."""
    from helpers import make_case

    fp8_case = make_case(77, "bf16", 8, 2, 128, [40, 130], [1, 1], kv_fp8=True)
    for r, slot in enumerate(fp8_case.req_slots):
        ctx = fp8_case.contexts()[r]
        k_codes, v_codes = oracle.gather_paged(fp8_case.pool, fp8_case.page_ids, fp8_case.layout, slot, 0,
                                               fp8_case.tokens_per_page, 2, 128, 1, ctx)
        k = oracle.bf16_bits_to_f32(oracle.fp8_to_bf16_bits(k_codes.reshape(-1))).reshape(ctx, 2, 128)
        v = oracle.bf16_bits_to_f32(oracle.fp8_to_bf16_bits(v_codes.reshape(-1))).reshape(ctx, 2, 128)
        assert np.array_equal(k, fp8_case.k_f32[r]) and np.array_equal(v, fp8_case.v_f32[r])
    wide_case = make_case(77, "bf16", 8, 2, 128, [40, 130], [1, 1])  # same seed: the same values before rounding
    fp8_out, wide_out = fp8_case.oracle_output(), wide_case.oracle_output()
    assert np.mean(np.abs(fp8_out - wide_out)) <= 0.025
