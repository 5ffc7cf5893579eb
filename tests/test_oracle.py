"""The CPU oracle against the golden vectors the reference produced (CPU only).

Pins every oracle function -- C, numpy and torch restatements -- to outputs of
the reference's own quantiser, dequantize and REFERENCE kernels
(tests/golden/make_golden.py).
"""
import numpy as np
import pytest

from conftest import CASES


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_unpack_int4(case, oracle):
    if case.bits != 4:
        pytest.skip("int8 is not packed")
    assert np.array_equal(oracle.c_unpack_int4(case.qweight), case.unpacked)
    assert np.array_equal(oracle.np_unpack_int4(case.qweight), case.unpacked)
    # split-half: low nibbles are rows 0..K/2-1, high nibbles rows K/2..K-1
    half = case.k // 2
    assert np.array_equal(case.unpacked[:half], case.qweight & 0x0F)
    assert np.array_equal(case.unpacked[half:], case.qweight >> 4)


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_dequantize_bit_exact(case, oracle):
    got_c = oracle.c_dequantize(case.qweight, case.scales, case.zeros, case.group, case.bits)
    got_np = oracle.np_dequantize(case.qweight, case.scales, case.zeros, case.group, case.bits)
    assert np.array_equal(got_c, case.dense)
    assert np.array_equal(got_np, case.dense)


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_torch_restatement_bit_exact(case, oracle):
    import torch

    def t16(a):
        return None if a is None else torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)

    dense = oracle.torch_dequantize(torch.from_numpy(case.qweight.copy()), t16(case.scales),
                                    t16(case.zeros), case.group, case.bits)
    assert np.array_equal(dense.view(torch.int16).numpy().view(np.uint16), case.dense)
    y = oracle.torch_wq_gemm(t16(case.x), torch.from_numpy(case.qweight.copy()), t16(case.scales),
                             t16(case.zeros), t16(case.bias), case.group, case.bits)
    # same library, same op sequence as the reference: identical bits
    assert np.array_equal(y.view(torch.int16).numpy().view(np.uint16), case.y)


@pytest.mark.parametrize("case", CASES, ids=lambda c: c.name)
def test_gemm_matches_reference(case, oracle):
    got = oracle.c_wq_gemm(case.x, case.qweight, case.scales, case.zeros, case.bias, case.group,
                           case.bits)
    want = oracle.bf16_bits_to_f32(case.y)
    err = oracle.max_normalised_error(oracle.bf16_bits_to_f32(got), want)
    # fp32 accumulation in a different order than torch's CPU bf16 matmul: the
    # north-star tolerance is 1e-2 (max-normalised); the C oracle sits far inside it.
    assert err < 1e-2, err
    assert err < 4e-3, f"oracle drifted from the reference more than bf16 rounding explains: {err}"


@pytest.mark.parametrize("case", [c for c in CASES if c.w is not None], ids=lambda c: c.name)
def test_numpy_quantiser_bit_exact(case, oracle):
    q, s, z = oracle.np_quantize(case.w, case.bits, case.group, case.symmetric)
    assert np.array_equal(q, case.qweight)
    assert np.array_equal(s, case.scales)
    assert (z is None) == (case.zeros is None)
    if z is not None:
        assert np.array_equal(z, case.zeros)


def test_bf16_rounding_helpers(oracle):
    vals = np.array([0.0, 1.0, -1.0, 1.00390625, 1.01171875, 3.0e-39, 65504.0, 1e38], dtype=np.float32)
    import torch

    want = torch.from_numpy(vals).to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(oracle.f32_to_bf16_bits(vals), want)
    assert np.array_equal(oracle.bf16_bits_to_f32(want),
                          torch.from_numpy(vals).to(torch.bfloat16).float().numpy())


def test_dequantize_rejects_bad_shapes(oracle):
    q = np.zeros((4, 8), dtype=np.uint8)
    s = np.zeros((1, 8), dtype=np.uint16)
    with pytest.raises(ValueError):
        oracle.c_dequantize(q, s, None, 3, 4)  # K=8 not a multiple of the group
    with pytest.raises(ValueError):
        oracle.c_dequantize(q, s, None, 4, 5)  # bits must be 4 or 8
