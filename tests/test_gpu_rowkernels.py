"""GPU parity of the row kernels (quantize, swizzle, residual_add_rmsnorm, SiLU gate) against the CPU oracle.

Quantized codes, scale bytes and the global scale are compared bit for bit. The rmsnorm residual is bit-exact; its bf16
output and the SiLU gate use the tolerances the reference asserts for its own binaries
(python/tests/test_gpu_reference.py:198-210, :226-230): max|d| <= 2**-7 * max|ref| and at most 0.01 % / 0.02 % of the
elements different.
"""

import pytest
import torch

from oracle import blockscaled as O

pytestmark = pytest.mark.gpu

FMTS = ["mxfp8", "mxfp4", "nvfp4"]


@pytest.fixture(scope="module")
def K():
    from tilefish_b200 import kernels

    kernels.require_cuda()
    return kernels


def adversarial(m, k, seed):
    """randn * 2**randint(-24, 25) with special values first (no NaN): the sampler pattern of the reference's fusion verifier
    (python/src/tilefish/_fusion.py:2100-2137)."""
    g = torch.Generator().manual_seed(seed)
    x = torch.randn((m, k), generator=g) * torch.exp2(torch.randint(-24, 25, (m, k), generator=g).float())
    flat = x.view(-1)
    special = torch.tensor([0.0, -0.0, 1.0, -1.0, 448.0, -448.0, 6.0, 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 2.0**-133, -(2.0**-130),
                            3.0e38, -3.0e38, float("inf"), -float("inf")])
    n = min(flat.numel(), special.numel())
    flat[:n] = special[:n]
    return x.to(torch.bfloat16)


def check_quant(K, x, fmt, layout):
    q = K.quantize(x.cuda(), fmt, layout=layout)
    torch.cuda.synchronize()
    codes, scales, gs = O.quantize(x, fmt)
    m, k = x.shape
    cols = k // O.FORMATS[fmt][2]
    if gs is not None:
        assert q.global_scale.cpu().view(torch.int32).item() == gs.view(torch.int32).item()
    assert torch.equal(q.plain_scales().cpu(), scales), f"{fmt} scales differ"
    if layout == "swizzled":
        assert torch.equal(q.scales.cpu(), O.swizzle_scales(scales)), f"{fmt} swizzled bytes (padding included) differ"
    assert torch.equal(q.codes.cpu(), codes), f"{fmt} codes differ"


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("m", [1, 2, 31, 32, 33, 127, 128, 129, 300])
@pytest.mark.parametrize("k", [32, 64, 288, 4096])
def test_quantize_is_bit_exact(K, fmt, m, k):
    x = O.outlier_input(m, k, seed=m * 7 + k)
    check_quant(K, x, fmt, "swizzled")
    check_quant(K, x, fmt, "plain")


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("m,k", [(300, 2048), (160, 2560), (100, 4128), (24, 28672), (297, 8192)])
def test_quantize_long_rows_streaming_form_is_bit_exact(K, fmt, m, k):
    """Long rows: the mxfp8 quantizer and the nvfp4 amax pass stage rows of at least 2048 elements through a shared-memory ring
    (bulk copies of 4 KB row chunks) once there are enough chunks to fill the GPU; the e2m1 quantizers keep the register form.
    Full chunks, a ragged last chunk per row, many chunks per row, and a strided input."""
    x = O.outlier_input(m, k, seed=m + k)
    check_quant(K, x, fmt, "swizzled")
    wide = torch.zeros((m, k + 64), dtype=torch.bfloat16)
    wide[:, :k] = x
    q = K.quantize(wide.cuda()[:, :k], fmt, layout="plain")
    codes, scales, _ = O.quantize(x, fmt)
    assert torch.equal(q.codes.cpu(), codes) and torch.equal(q.plain_scales().cpu(), scales)


@pytest.mark.parametrize("fmt", FMTS)
def test_quantize_sweep_point_8192_is_bit_exact(K, fmt):
    """M = 8192, K = 4096 with 1 % outliers x100 (a point of the quantize sweep), every byte compared with the oracle."""
    x = O.outlier_input(8192, 4096, seed=0)
    check_quant(K, x, fmt, "swizzled")


@pytest.mark.parametrize("fmt", FMTS)
def test_quantize_adversarial_values(K, fmt):
    x = adversarial(64, 512, seed=11)
    if fmt == "nvfp4":
        x = torch.where(torch.isinf(x), torch.full_like(x, 3.0e38), x)  # inf / inf is NaN in the nvfp4 scale: finite inputs only
    check_quant(K, x, fmt, "swizzled")


@pytest.mark.parametrize("fmt", FMTS)
def test_quantize_zeros_and_strided_input(K, fmt):
    check_quant(K, torch.zeros((5, 64), dtype=torch.bfloat16), fmt, "swizzled")
    x = O.outlier_input(40, 256, seed=5)
    wide = torch.zeros((40, 512), dtype=torch.bfloat16)
    wide[:, :256] = x
    q = K.quantize(wide.cuda()[:, :256], fmt, layout="plain")
    codes, scales, _ = O.quantize(x, fmt)
    assert torch.equal(q.codes.cpu(), codes) and torch.equal(q.plain_scales().cpu(), scales)


def test_quantize_empty_and_refusals(K):
    from tilefish_b200 import TilefishPreconditionError

    q = K.quantize(torch.empty((0, 64), dtype=torch.bfloat16, device="cuda"), "mxfp8")
    assert q.codes.numel() == 0
    with pytest.raises(TilefishPreconditionError) as e:
        K.quantize(torch.zeros((4, 48), dtype=torch.bfloat16, device="cuda"), "mxfp8")
    assert e.value.kind == "divisible"
    with pytest.raises(TilefishPreconditionError) as e:
        K.quantize(torch.zeros((4, 64), dtype=torch.float16, device="cuda"), "mxfp8")
    assert e.value.kind == "dtype"
    with pytest.raises(TilefishPreconditionError) as e:
        K.quantize(torch.zeros((4, 64), dtype=torch.bfloat16), "mxfp8")
    assert e.value.kind == "device"


@pytest.mark.parametrize("rows,cols", [(1, 1), (127, 3), (128, 4), (129, 5), (300, 128)])
def test_swizzle_kernels(K, rows, cols):
    g = torch.Generator().manual_seed(rows + cols)
    s = torch.randint(1, 256, (rows, cols), generator=g, dtype=torch.uint8)
    sw = K.swizzle_scales(s.cuda())
    assert torch.equal(sw.cpu(), O.swizzle_scales(s))
    assert torch.equal(K.unswizzle_scales(sw, rows, cols).cpu(), s)


@pytest.mark.parametrize("fmt", FMTS)
def test_quantize_full_size_properties(K, fmt):
    """M = 65536, K = 4096 (the largest sweep point): sampled rows bit-exact, every block's dequantization error bounded."""
    m, k = 65536, 4096
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((m, k), generator=g, device="cuda", dtype=torch.float32)
    mask = torch.rand((m, k), generator=g, device="cuda") < 0.01
    x = torch.where(mask, x * 100, x).to(torch.bfloat16)
    del mask
    q = K.quantize(x, fmt)
    rows = torch.randint(0, m, (192,), generator=torch.Generator().manual_seed(1))
    rows[:4] = torch.tensor([0, 127, 128, m - 1])
    xs = x[rows.cuda()].cpu()
    gs = None
    if fmt == "nvfp4":
        amax = x.abs().amax().float().cpu()
        gs = amax / torch.tensor(2688.0)
        assert q.global_scale.cpu().view(torch.int32).item() == gs.view(torch.int32).item()
    codes, scales, _ = O.quantize(xs, fmt, gs)
    assert torch.equal(q.codes[rows.cuda()].cpu(), codes)
    assert torch.equal(q.plain_scales()[rows.cuda()].cpu(), scales)
    # checksum of checksums: the swizzled buffer holds exactly the plain scale bytes (a permutation, no padding here)
    assert int(q.scales.to(torch.int64).sum()) == int(q.plain_scales().to(torch.int64).sum())


# ---- residual_add_rmsnorm ------------------------------------------------------------------------------------------------
def rms_inputs(m, d, seed, xs=1.0, rmean=0.0):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn((m, d), generator=g) * xs).to(torch.bfloat16)
    res = torch.randn((m, d), generator=g) + rmean
    w = (1 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16)
    return x, res, w


def assert_close_bf16(got, ref, max_frac, what):
    g, r = got.float(), ref.float()
    bound = 2.0**-7 * float(r.abs().max())
    assert float((g - r).abs().max()) <= bound, what
    frac = float((got.view(torch.int16) != ref.view(torch.int16)).float().mean())
    assert frac <= max_frac, f"{what}: {frac:.6f} of the elements differ"


@pytest.mark.parametrize("m,d", [(256, 2560), (1, 2560), (32, 2560), (257, 2560), (64, 8192), (7, 64), (5, 4104), (3, 32768)])
@pytest.mark.parametrize("xs,rmean", [(1.0, 0.0), (0.01, 0.0), (30.0, 100.0)])
def test_residual_add_rmsnorm(K, m, d, xs, rmean):
    x, res, w = rms_inputs(m, d, seed=0, xs=xs, rmean=rmean)
    r_ref, out_ref = O.residual_add_rmsnorm(x, res, w)
    res_gpu = res.cuda()
    out = K.residual_add_rmsnorm(x.cuda(), res_gpu, w.cuda())
    assert torch.equal(res_gpu.cpu(), r_ref), "the residual must be byte-identical"
    assert_close_bf16(out.cpu(), out_ref, 1e-4 if m * d >= 100000 else 2e-3, "rmsnorm out")


def test_residual_add_rmsnorm_golden_vectors(K, golden):
    x = torch.from_numpy(golden["rms_x"].copy()).view(torch.bfloat16)
    res = torch.from_numpy(golden["rms_res_in"].copy()).cuda()
    w = torch.from_numpy(golden["rms_w"].copy()).view(torch.bfloat16)
    out = K.residual_add_rmsnorm(x.cuda(), res, w.cuda())
    assert torch.equal(res.cpu(), torch.from_numpy(golden["rms_res_out"].copy()))
    assert_close_bf16(out.cpu(), torch.from_numpy(golden["rms_out"].copy()).view(torch.bfloat16), 1e-3, "rmsnorm vs reference vectors")


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("m,d", [(256, 2560), (33, 8192), (1, 64)])
def test_rmsnorm_fused_quantize_equals_quantize_of_its_own_output(K, fmt, m, d):
    x, res, w = rms_inputs(m, d, seed=2)
    gs = torch.tensor([0.002], dtype=torch.float32) if fmt == "nvfp4" else None
    res_gpu = res.cuda()
    out, q = K.residual_add_rmsnorm(x.cuda(), res_gpu, w.cuda(), quantize_to=fmt, q_global_scale=gs.cuda() if gs is not None else None)
    codes, scales, _ = O.quantize(out.cpu(), fmt, gs)
    assert torch.equal(q.codes.cpu(), codes)
    assert torch.equal(q.scales.cpu(), O.swizzle_scales(scales))
    # quantized output alone (no bf16 copy) gives the same bytes
    res2 = res.cuda()
    none, q2 = K.residual_add_rmsnorm(x.cuda(), res2, w.cuda(), quantize_to=fmt, want_bf16=False, q_global_scale=gs.cuda() if gs is not None else None)
    assert none is None and torch.equal(q2.codes, q.codes) and torch.equal(q2.scales, q.scales)
    assert torch.equal(res2, res_gpu)


def test_first_benchmark_configuration(K):
    """residual_add_rmsnorm then MXFP8 quantize, 256 x 2560, seed 0: residual, bf16 output, e4m3 codes and ue8m0 scales."""
    x, res, w = rms_inputs(256, 2560, seed=0)
    r_ref, out_ref = O.residual_add_rmsnorm(x, res, w)
    res_gpu = res.cuda()
    out, q = K.residual_add_rmsnorm(x.cuda(), res_gpu, w.cuda(), quantize_to="mxfp8")
    assert torch.equal(res_gpu.cpu(), r_ref)
    assert_close_bf16(out.cpu(), out_ref, 1e-4, "out")
    codes, scales, _ = O.quantize(out.cpu(), "mxfp8")  # bit-exact given the same bf16 input
    assert torch.equal(q.codes.cpu(), codes) and torch.equal(q.plain_scales().cpu(), scales)
    codes_e2e, scales_e2e, _ = O.quantize(out_ref, "mxfp8")  # end to end: inherits the rare 1-ulp bf16 differences
    assert float((q.codes.cpu() != codes_e2e).float().mean()) <= 1e-3
    assert float((q.plain_scales().cpu() != scales_e2e).float().mean()) <= 1e-3


# ---- SiLU gate -----------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("m,f", [(1, 3072), (32, 3072), (257, 384), (512, 3072)])
def test_silu_gate(K, m, f):
    t = (O.randn((m, 2 * f), 3) * 3).to(torch.bfloat16)
    ref = O.silu_gate(t[:, :f], t[:, f:])
    out = K.silu_gate(t.cuda())
    assert_close_bf16(out.cpu(), ref, 2e-4 if m * f > 100000 else 2e-3, "silu gate")


def test_silu_gate_golden_vectors(K, golden):
    t = torch.from_numpy(golden["silu_t"].copy()).view(torch.bfloat16)
    out = K.silu_gate(t.cuda())
    assert_close_bf16(out.cpu(), torch.from_numpy(golden["silu_out"].copy()).view(torch.bfloat16), 2e-3, "silu gate vs reference vectors")
