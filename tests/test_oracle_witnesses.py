"""Independent witnesses for the parts of the oracle the reference does not pin (it types BlockScaled tensors but never quantizes one).

``ml_dtypes`` (numpy extension types float4_e2m1fn, float8_e4m3fn, float8_e8m0fnu; not used anywhere in the package or in the oracle)
gives the element casts and the scale decoding; a few lines of numpy give the block rules. The oracle's torch code must produce the same
bytes. Where the two differ by design it is said here: ml_dtypes turns an e4m3 overflow into NaN, the oracle (like the reference's cast,
python/src/tilefish/_reference.py:121-141, and the hardware's cvt.rn.satfinite) saturates at 448; NaN inputs are left out.
"""

import numpy as np
import pytest
import torch

from oracle import blockscaled as O

ml_dtypes = pytest.importorskip("ml_dtypes")


def _adversarial(n, seed):
    """randn * 2**randint(-24, 25), the sampler pattern of the reference's fusion verifier (python/src/tilefish/_fusion.py:2100-2137), finite values only."""
    rng = np.random.default_rng(seed)
    return (rng.standard_normal(n) * np.exp2(rng.integers(-24, 25, n))).astype(np.float32)


def test_e2m1_cast_matches_ml_dtypes():
    grid = np.array([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=np.float32)
    mids = (grid[:-1] + grid[1:]) / 2
    pts = np.concatenate([grid, mids, np.nextafter(mids, np.float32(0)), np.nextafter(mids, np.float32(9)), [6.5, 7.0, 1e30, np.inf, 2.0**-140, 0.24999999]]).astype(np.float32)
    x = np.concatenate([pts, -pts, _adversarial(20000, 1), np.linspace(-7, 7, 28001, dtype=np.float32)])
    want = x.astype(ml_dtypes.float4_e2m1fn).astype(np.float32)
    got = O.e2m1_to_f32(O.cast_e2m1(torch.from_numpy(x))).numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))  # bit patterns: -0 stays -0


def test_e4m3_cast_matches_ml_dtypes_inside_the_finite_range():
    codes = np.arange(256, dtype=np.uint8)
    vals = codes.view(ml_dtypes.float8_e4m3fn).astype(np.float32)
    vals = np.unique(vals[np.isfinite(vals)])
    mids = (vals[:-1] + vals[1:]) / 2
    x = np.concatenate([vals, mids, np.nextafter(mids, np.float32(-1e9)), np.nextafter(mids, np.float32(1e9)), np.clip(_adversarial(50000, 2), -448, 448)]).astype(np.float32)
    want = x.astype(ml_dtypes.float8_e4m3fn).view(np.uint8)
    got = O.cast_e4m3(torch.from_numpy(x)).numpy()
    assert np.array_equal(got, want)
    # outside the range the oracle saturates where ml_dtypes gives NaN
    big = torch.tensor([449.0, 464.0, 480.0, 1e9, float("inf"), -1e9])
    assert O.cast_e4m3(big).tolist() == [0x7E, 0x7E, 0x7E, 0x7E, 0x7E, 0xFE]


def test_ue8m0_scale_decoding_matches_ml_dtypes():
    b = np.arange(0, 255, dtype=np.uint8)
    want = b.view(ml_dtypes.float8_e8m0fnu).astype(np.float32)
    codes = torch.zeros((255, 32), dtype=torch.uint8) + 0x38  # e4m3 1.0 in every element
    got = O.dequantize(codes, torch.from_numpy(b.copy()).view(255, 1), "mxfp8")[:, 0].numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def _np_quantize_mx(x_bf16: torch.Tensor, elem):
    """The MX rule in numpy + ml_dtypes: scale = 2**(floor(log2 amax) - emax), codes = cast(x / scale), saturating."""
    x = x_bf16.float().numpy()
    m, k = x.shape
    xb = x.reshape(m, k // 32, 32)
    amax = np.abs(xb).max(-1)
    emax, top, dt = (8, 448.0, ml_dtypes.float8_e4m3fn) if elem == "e4m3" else (2, 6.0, ml_dtypes.float4_e2m1fn)
    with np.errstate(divide="ignore"):
        e = np.floor(np.log2(amax.astype(np.float64))).astype(np.int64)
    biased = np.where(amax == 0, 127, np.clip(e + 127 - emax, 0, 254))
    biased = np.where((amax != 0) & (e + 127 <= 0), np.clip(0 - emax, 0, 254), biased)  # a subnormal amax has exponent field 0
    scale = np.exp2((biased - 127).astype(np.float64))
    q = (xb.astype(np.float64) / scale[..., None]).astype(np.float32)  # a power-of-two quotient: exact
    q = np.clip(q, -top, top)
    return q.astype(dt), biased.astype(np.uint8)


@pytest.mark.parametrize("fmt,elem", [("mxfp8", "e4m3"), ("mxfp4", "e2m1")])
def test_mx_quantizer_matches_an_independent_numpy_statement(fmt, elem):
    for seed, x in enumerate([O.outlier_input(64, 256, seed=3), torch.from_numpy(_adversarial(64 * 256, 9)).view(64, 256).to(torch.bfloat16)]):
        codes, scales, _ = O.quantize(x, fmt)
        q, biased = _np_quantize_mx(x, elem)
        assert np.array_equal(scales.numpy(), biased), (fmt, seed)
        want = q.reshape(64, 256).astype(np.float32)
        got = (O.e4m3_to_f32(codes) if elem == "e4m3" else O.e2m1_to_f32(O.unpack_e2m1(codes))).numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (fmt, seed)


def test_nvfp4_quantizer_matches_an_independent_numpy_statement():
    x = O.outlier_input(48, 512, seed=5)
    codes, s8, gs = O.quantize(x, "nvfp4")
    xf = x.float().numpy().reshape(48, 32, 16)
    f32 = np.float32
    amax_t = f32(np.abs(xf).max())
    g = f32(amax_t / f32(2688.0))
    assert f32(gs.item()) == g
    inv_t = f32(f32(1.0) / f32(f32(6.0) * g))
    amax_b = np.abs(xf).max(-1).astype(np.float32)
    s = (amax_b * inv_t).astype(np.float32)
    s_codes = np.clip(s, -448, 448).astype(ml_dtypes.float8_e4m3fn)
    assert np.array_equal(s8.numpy(), s_codes.view(np.uint8))
    d = (s_codes.astype(np.float32) * g).astype(np.float32)
    with np.errstate(divide="ignore"):
        inv = np.where(d == 0, f32(0), (f32(1.0) / d).astype(np.float32)).astype(np.float32)
    q = (xf * inv[..., None]).astype(np.float32)
    want = np.clip(q, -6, 6).astype(ml_dtypes.float4_e2m1fn).astype(np.float32).reshape(48, 512)
    got = O.e2m1_to_f32(O.unpack_e2m1(codes)).numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
