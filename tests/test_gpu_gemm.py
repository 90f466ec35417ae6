"""GPU parity of the block-scaled GEMM (tcgen05) and its fused epilogues against the CPU oracle.

Oracle O1: bf16( f32 matmul of the DEQUANTIZED operands ), the same codes and scale bytes the kernel consumed (they are
bit-exact with the oracle's, which test_gpu_rowkernels.py proves). Bound: max|d| <= 2**-8 * max|ref| * 1.01, the bound the
reference asserts for its own GEMM (python/tests/test_gpu_gemm.py:103-114). A GEMM with a wrong scale layout, nibble order
or K order fails this by orders of magnitude, so this test is also what proves the swizzled scale layout.
"""

import pytest
import torch

from oracle import blockscaled as O

pytestmark = pytest.mark.gpu

FMTS = ["mxfp8", "mxfp4", "nvfp4"]
TOL = 2.0**-8 * 1.01


@pytest.fixture(scope="module")
def K():
    from tilefish_b200 import kernels

    kernels.require_cuda()
    return kernels


def operands(m, n_rows, k, seed):
    """bf16 a ~ N(0,1), w ~ N(0, 1/K), each 32-block rescaled by a random power of two so the scale bytes vary."""
    g = torch.Generator().manual_seed(seed)
    a = torch.randn((m, k), generator=g)
    w = torch.randn((n_rows, k), generator=g) * k**-0.5
    a = a * torch.exp2(torch.randint(-2, 3, (m, k // 32), generator=g).float()).repeat_interleave(32, dim=1)
    w = w * torch.exp2(torch.randint(-3, 4, (n_rows, k // 32), generator=g).float()).repeat_interleave(32, dim=1)
    return a.to(torch.bfloat16), w.to(torch.bfloat16)


def oracle_acc(a, w, fmt):
    qa, qb = O.quantize(a, fmt), O.quantize(w, fmt)
    return O.dequantize(qa[0], qa[1], fmt, qa[2]) @ O.dequantize(qb[0], qb[1], fmt, qb[2]).t()


def assert_gemm_close(got, ref, what):
    g, r = got.float(), ref.float()
    bound = TOL * float(r.abs().max())
    err = float((g - r).abs().max())
    assert err <= bound, f"{what}: max|d| = {err} > {bound}"


def no_device_timeout():
    from tilefish_b200 import _native

    assert _native.device_status() == (0, 0)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("m,n,k", [(128, 256, 256), (128, 128, 128 + 128), (1, 256, 256), (16, 512, 2560), (130, 264, 288), (257, 136, 32 * 5),
                                   (128, 6144, 2560), (384, 2560, 3072)])
def test_gemm_matches_dequantized_oracle(K, fmt, m, n, k):
    a, w = operands(m, n, k, seed=m + n + k)
    out = K.gemm_blockscaled(K.quantize(a.cuda(), fmt), K.quantize(w.cuda(), fmt))
    assert out.shape == (m, n) and out.dtype == torch.bfloat16
    assert_gemm_close(out.cpu(), O.f32_to_bf16(oracle_acc(a, w, fmt)), f"{fmt} {m}x{n}x{k}")
    no_device_timeout()


@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
def test_gemm_bf16_a_is_quantized_on_the_fly(K, fmt):
    a, w = operands(64, 256, 512, seed=3)
    qb = K.quantize(w.cuda(), fmt)
    out = K.gemm(a.cuda(), qb)
    ref = O.gemm_bf16_a(a, O.quantize(w, fmt), fmt)
    assert_gemm_close(out.cpu(), ref, fmt)
    # informational second oracle: the bf16 activation against the dequantized weight (activation quantization error)
    ob = O.quantize(w, fmt)
    semantic = O.reference_gemm(a, O.dequantize(ob[0], ob[1], fmt, ob[2]))
    rel = float((out.cpu().float() - semantic.float()).norm() / semantic.float().norm())
    assert rel < {"mxfp8": 0.05, "nvfp4": 0.15}[fmt]


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("m,f,k", [(128, 128, 256), (200, 384, 512), (32, 3072, 2560)])
def test_gemm_silu_gate_epilogue(K, fmt, m, f, k):
    a, w = operands(m, 2 * f, k, seed=f + k)
    out = K.gemm_blockscaled(K.quantize(a.cuda(), fmt), K.quantize(w.cuda(), fmt), epilogue="silu_gate")
    assert out.shape == (m, f)
    t = O.f32_to_bf16(oracle_acc(a, w, fmt))
    ref = O.silu_gate(t[:, :f], t[:, f:])
    # a 1-ulp difference of the bf16 GEMM result moves through silu(g)*u: bound by the GEMM tolerance times the gate's gain
    g, r = out.cpu().float(), ref.float()
    gain = float(t.float().abs().max()) + 1.0
    assert float((g - r).abs().max()) <= TOL * float(t.float().abs().max()) * gain
    frac = float(((g - r).abs() > 2.0**-7 * r.abs().max()).float().mean())
    assert frac == 0.0
    # and it equals the unfused pair of kernels on the same GEMM result up to that result's own rounding
    unfused = K.silu_gate(K.gemm_blockscaled(K.quantize(a.cuda(), fmt), K.quantize(w.cuda(), fmt)))
    if K.gemm_workspace_bytes(m, f, k, fmt, "silu_gate") == 0 and K.gemm_workspace_bytes(m, 2 * f, k, fmt) == 0:
        assert torch.equal(unfused, out), "fused epilogue must reproduce gemm -> bf16 -> silu_gate bit for bit"
    else:
        # small M: either call may cut K into ranges (its own choice per epilogue), which changes the order of the f32 sums
        d = (unfused.float() - out.float()).abs()
        assert float(d.max()) <= TOL * float(t.float().abs().max()) * gain
        assert float((d > 0).float().mean()) < 0.02
    no_device_timeout()


@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
def test_gemm_residual_epilogue(K, fmt):
    m, n, k = 130, 264, 288
    a, w = operands(m, n, k, seed=9)
    res0 = O.randn((m, n), 4)
    res = res0.cuda()
    out = K.gemm_blockscaled(K.quantize(a.cuda(), fmt), K.quantize(w.cuda(), fmt), epilogue="residual", residual=res)
    plain = K.gemm_blockscaled(K.quantize(a.cuda(), fmt), K.quantize(w.cuda(), fmt))
    assert torch.equal(out, plain)
    assert torch.equal(res.cpu(), res0 + plain.cpu().float()), "residual += f32(bf16 result): one exact f32 add"


@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
def test_gemm_full_size_sampled_rows(K, fmt):
    """M = 4096, N = 6144, K = 2560 (the GEMM benchmark shape): 48 sampled rows against the oracle, plus linearity in A's rows."""
    m, n, k = 4096, 6144, 2560
    g = torch.Generator().manual_seed(0)
    a = torch.randn((m, k), generator=g).to(torch.bfloat16)
    w = (torch.randn((n, k), generator=g) * k**-0.5).to(torch.bfloat16)
    gs = None
    if fmt == "nvfp4":
        gs = torch.tensor([float(a.float().abs().max()) / 2688.0], dtype=torch.float32)
    qa = K.quantize(a.cuda(), fmt, global_scale=gs.cuda() if gs is not None else None)
    qb = K.quantize(w.cuda(), fmt)
    out = K.gemm_blockscaled(qa, qb)
    rows = torch.randint(0, m, (48,), generator=g)
    rows[:3] = torch.tensor([0, 127, m - 1])
    oa = O.quantize(a[rows], fmt, gs.reshape(()) if gs is not None else None)
    ob = O.quantize(w, fmt)
    ref = O.f32_to_bf16(O.dequantize(oa[0], oa[1], fmt, oa[2]) @ O.dequantize(ob[0], ob[1], fmt, ob[2]).t())
    assert_gemm_close(out[rows.cuda()].cpu(), ref, f"{fmt} sampled rows")
    # rows are independent: the same rows computed as their own small GEMM (which takes the split-K path, another summation
    # order) agree to the GEMM tolerance
    sub = K.gemm_blockscaled(K.quantize(a[rows].cuda(), fmt, global_scale=gs.cuda() if gs is not None else None), qb)
    assert_gemm_close(sub.cpu(), out[rows.cuda()].cpu(), f"{fmt} sub-problem")
    no_device_timeout()


def test_gemm_refusals(K):
    from tilefish_b200 import TilefishPreconditionError

    a, w = operands(16, 128, 64, seed=1)
    qa, qb = K.quantize(a.cuda(), "mxfp8"), K.quantize(w.cuda(), "mxfp4")
    with pytest.raises(TilefishPreconditionError) as e:
        K.gemm_blockscaled(qa, qb)
    assert e.value.kind == "dtype"
    qb8 = K.quantize(operands(16, 128, 96, seed=1)[1].cuda(), "mxfp8")
    with pytest.raises(TilefishPreconditionError) as e:
        K.gemm_blockscaled(qa, qb8)
    assert e.value.kind == "shape"
    plain = K.quantize(w.cuda(), "mxfp8", layout="plain")
    with pytest.raises(TilefishPreconditionError):
        K.gemm_blockscaled(qa, plain)
    empty = K.gemm_blockscaled(K.quantize(torch.empty((0, 64), dtype=torch.bfloat16, device="cuda"), "mxfp8"), K.quantize(w.cuda(), "mxfp8"))
    assert empty.shape == (0, 128)


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("m,n,k,epi", [(1, 2560, 8192, "none"), (16, 6144, 8192, "none"), (64, 1024, 8192, "none"), (32, 1536, 2560, "silu_gate"),
                                       (40, 512, 4096, "residual"), (130, 1024, 4096, "residual"), (200, 512, 8192, "silu_gate")])
def test_gemm_small_m_takes_the_split_k_path(K, fmt, m, n, k, epi):
    """Few output tiles and a long K: the problem is cut along K into an f32 workspace and reduced by a second kernel. Same
    oracle, same bound; the partial sums are added in split order, so two runs give identical bytes."""
    assert K.gemm_workspace_bytes(m, n, k, fmt, epi) > 0, "this shape is meant to exercise split-K"
    rows_b = 2 * n if epi == "silu_gate" else n
    a, w = operands(m, rows_b, k, seed=m + n)
    qa, qb = K.quantize(a.cuda(), fmt), K.quantize(w.cuda(), fmt)
    res0 = O.randn((m, n), 8)
    res = res0.cuda() if epi == "residual" else None
    amax = torch.zeros(1, device="cuda")
    out = K.gemm_blockscaled(qa, qb, epilogue=epi, residual=res, amax_out=amax)
    acc = O.f32_to_bf16(oracle_acc(a, w, fmt))
    if epi == "silu_gate":
        ref = O.silu_gate(acc[:, :n], acc[:, n:])
        g, r = out.cpu().float(), ref.float()
        assert float(((g - r).abs() > 2.0**-7 * r.abs().max()).float().mean()) == 0.0
        assert float((g - r).abs().max()) <= TOL * float(acc.float().abs().max()) * (float(acc.float().abs().max()) + 1.0)
    else:
        assert_gemm_close(out.cpu(), acc, f"{fmt} split-K {m}x{n}x{k}")
    assert float(amax.item()) == float(out.float().abs().max().item())
    if epi == "residual":
        assert torch.equal(res.cpu(), res0 + out.cpu().float())
    again = K.gemm_blockscaled(qa, qb, epilogue=epi, residual=res0.cuda() if epi == "residual" else None)
    assert torch.equal(again, out), "split-K must be deterministic"
    from tilefish_b200 import TilefishPreconditionError

    with pytest.raises(TilefishPreconditionError) as e:
        K.gemm_blockscaled(qa, qb, epilogue=epi, residual=res0.cuda() if epi == "residual" else None,
                           workspace=torch.empty(256, dtype=torch.uint8, device="cuda"))
    assert e.value.kind == "workspace"
    no_device_timeout()


def test_two_cta_kernel_variant_matches_the_default_kernel():
    """TF_GEMM_TWO_CTA=1 selects the cta_group::2 kernel (a CTA pair per 256 x 256 tile). It is read once per process, so the
    variant runs in a child process and ships its result back as bytes; both kernels must satisfy the oracle bound, and they
    agree with each other to that bound (the accumulation order inside the tensor core may differ)."""
    import os
    import subprocess
    import sys
    import tempfile

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = """
import sys, torch
sys.path.insert(0, %r)
from tilefish_b200 import kernels as K, _native
from oracle import blockscaled as O
outs = {}
for fmt in ("mxfp8", "nvfp4"):
    a = O.randn((384, 2560), 1, torch.bfloat16); w = O.randn((1536, 2560), 2, torch.bfloat16, scale=2560 ** -0.5)
    qa, qb = K.quantize(a.cuda(), fmt), K.quantize(w.cuda(), fmt)
    outs[fmt] = K.gemm_blockscaled(qa, qb).cpu()
    outs[fmt + "_silu"] = K.gemm_blockscaled(qa, qb, epilogue="silu_gate").cpu()
assert _native.device_status() == (0, 0)
torch.save(outs, sys.argv[1])
""" % root
    results = {}
    with tempfile.TemporaryDirectory() as d:
        for flag in ("0", "1"):
            path = os.path.join(d, f"out{flag}.pt")
            env = dict(os.environ, TF_GEMM_TWO_CTA=flag)
            r = subprocess.run([sys.executable, "-c", script, path], env=env, capture_output=True, text=True, timeout=300)
            assert r.returncode == 0, r.stderr[-2000:]
            results[flag] = torch.load(path)
    for key, one in results["0"].items():
        two = results["1"][key]
        bound = TOL * float(one.float().abs().max()) * (4.0 if key.endswith("_silu") else 1.0)
        assert float((one.float() - two.float()).abs().max()) <= bound, key
    a = O.randn((384, 2560), 1, torch.bfloat16)
    w = O.randn((1536, 2560), 2, torch.bfloat16, scale=2560**-0.5)
    for fmt in ("mxfp8", "nvfp4"):
        assert_gemm_close(results["1"][fmt], O.f32_to_bf16(oracle_acc(a, w, fmt)), f"two-CTA {fmt}")


def test_a_wait_that_runs_out_is_reported_and_the_context_survives(K):
    """Failure detection without a fault: a kernel waits (with a 20 ms limit) on a barrier nothing signals. It must return by
    itself, leave TF_ERR_DEVICE_TIMEOUT in the device status word, and the next GEMM on the same context must be correct."""
    import time

    from tilefish_b200 import _native as N

    assert N.device_status() == (0, 0)
    t0 = time.perf_counter()
    N.check(N.load().tf_selftest_bounded_wait(20, torch.cuda.current_stream().cuda_stream), "tf_selftest_bounded_wait")
    status, detail = N.device_status()  # synchronizes
    assert time.perf_counter() - t0 < 1.0
    assert status == N.TF_ERR_DEVICE_TIMEOUT and detail >> 16 == 9
    assert N.device_status() == (0, 0), "reading the status clears it"
    a, w = operands(64, 256, 256, seed=2)
    out = K.gemm_blockscaled(K.quantize(a.cuda(), "mxfp8"), K.quantize(w.cuda(), "mxfp8"))
    assert_gemm_close(out.cpu(), O.f32_to_bf16(oracle_acc(a, w, "mxfp8")), "after a timeout")


@pytest.mark.parametrize("fmt", ["mxfp8", "mxfp4"])
@pytest.mark.parametrize("m,n,k,epi", [(256, 512, 512, "none"), (300, 384, 2560, "silu_gate"), (130, 288, 288, "none"), (32, 1536, 2560, "silu_gate"),
                                       (16, 1024, 4096, "none")])
def test_gemm_quantized_output_equals_quantize_of_the_bf16_output(K, fmt, m, n, k, epi):
    """The epilogue's own MX quantization (one 32-element block per thread) against the quantizer kernel on the same bf16
    result: codes and swizzled scale bytes (padding included) identical, with and without the bf16 copy, one-pass and split-K."""
    rows_b = 2 * n if epi == "silu_gate" else n
    a, w = operands(m, rows_b, k, seed=m * 3 + n)
    qa, qb = K.quantize(a.cuda(), fmt), K.quantize(w.cuda(), fmt)
    out, q = K.gemm_blockscaled(qa, qb, epilogue=epi, quantize_out=True)
    plain = K.gemm_blockscaled(qa, qb, epilogue=epi)
    assert torch.equal(out, plain)
    ref = K.quantize(plain, fmt)
    assert torch.equal(q.codes, ref.codes) and torch.equal(q.scales, ref.scales)
    none, q2 = K.gemm_blockscaled(qa, qb, epilogue=epi, quantize_out=True, want_bf16=False)
    assert none is None and torch.equal(q2.codes, ref.codes) and torch.equal(q2.scales, ref.scales)
    codes, scales, _ = O.quantize(plain.cpu(), fmt)
    assert torch.equal(q.codes.cpu(), codes) and torch.equal(q.scales.cpu(), O.swizzle_scales(scales))
    no_device_timeout()


@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
@pytest.mark.parametrize("m,n,k", [(256, 256, 512), (384, 640, 1024)])
def test_vendor_blockscaled_gemm_reads_the_same_swizzled_operands(fmt, m, n, k):
    """An independent witness for the scale layout, the nibble order and the quantizer's bytes: cuBLASLt's block-scaled GEMM (through
    torch._scaled_mm) is handed THIS package's codes and swizzled scale bytes, reinterpreted, and must meet the same bound against the
    dequantized-operand oracle as this package's GEMM (2**-8 max|ref| x 1.01). A wrong layout or nibble order misses by orders of
    magnitude. Rows get very different magnitudes so that every scale byte matters. The vendor GEMM is a checker here, never a product path."""
    from tilefish_b200 import kernels as K

    g = torch.Generator().manual_seed(m + n + k)
    a = (torch.randn((m, k), generator=g) * torch.exp2(torch.randint(-6, 7, (m, 1), generator=g).float())).to(torch.bfloat16)
    b = (torch.randn((n, k), generator=g) * k**-0.5 * torch.exp2(torch.randint(-4, 5, (n, 1), generator=g).float())).to(torch.bfloat16)
    # magnitudes also vary along K, block by block
    a = (a.float() * torch.exp2(torch.randint(-3, 4, (1, k // 32), generator=g).float()).repeat_interleave(32, dim=1)).to(torch.bfloat16)
    qa, qb = K.quantize(a.cuda(), fmt), K.quantize(b.cuda(), fmt)
    if fmt == "mxfp8":
        ops = (qa.codes.view(torch.float8_e4m3fn), qb.codes.view(torch.float8_e4m3fn), qa.scales.view(torch.float8_e8m0fnu), qb.scales.view(torch.float8_e8m0fnu))
    else:
        ops = (qa.codes.view(torch.float4_e2m1fn_x2), qb.codes.view(torch.float4_e2m1fn_x2), qa.scales.view(torch.float8_e4m3fn), qb.scales.view(torch.float8_e4m3fn))
    try:
        theirs = torch._scaled_mm(ops[0], ops[1].t(), ops[2], ops[3], out_dtype=torch.float32)
    except Exception as e:  # noqa: BLE001
        pytest.skip(f"this torch build has no block-scaled library GEMM for {fmt}: {type(e).__name__}")
    if fmt == "nvfp4":
        theirs = theirs * (qa.global_scale * qb.global_scale)
    mine = K.gemm_blockscaled(qa, qb)
    ref = O.gemm_blockscaled(O.quantize(a, fmt), O.quantize(b, fmt), fmt).float()
    bound = 2.0**-8 * float(ref.abs().max()) * 1.01
    assert float((mine.cpu().float() - ref).abs().max()) <= bound
    assert float((theirs.cpu() - ref).abs().max()) <= bound


@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
@pytest.mark.parametrize("owners,rows_per_owner,n,k", [(2, 128, 512, 512), (4, 256, 1024, 1024), (8, 128, 256, 2048)])
def test_scattered_output_holds_the_rows_of_the_plain_gemm(K, fmt, owners, rows_per_owner, n, k):
    """tf_gemm_blockscaled_scatter writes row block i to its own destination (here: separate local buffers with a padded row
    stride): every destination must hold exactly the bytes of those rows of the ordinary GEMM, and nothing beside them."""
    m = owners * rows_per_owner
    a, w = operands(m, n, k, seed=owners + n)
    qa, qb = K.quantize(a.cuda(), fmt), K.quantize(w.cuda(), fmt)
    plain = K.gemm_blockscaled(qa, qb)
    ldo = n + 64
    dests = [torch.full((rows_per_owner, ldo), -7.0, dtype=torch.bfloat16, device="cuda") for _ in range(owners)]
    K.gemm_blockscaled_scatter(qa, qb, [d.data_ptr() for d in dests], rows_per_owner, ldo)
    torch.cuda.synchronize()
    for i, d in enumerate(dests):
        assert torch.equal(d[:, :n], plain[i * rows_per_owner:(i + 1) * rows_per_owner]), f"row block {i}"
        assert bool((d[:, n:] == -7.0).all()), f"row block {i}: bytes beyond n were written"


def test_scattered_output_refuses_what_it_cannot_do(K):
    from tilefish_b200.errors import TilefishPreconditionError

    a, w = operands(128, 256, 8192, seed=1)
    qa, qb = K.quantize(a.cuda(), "mxfp8"), K.quantize(w.cuda(), "mxfp8")
    d = torch.empty((128, 256), dtype=torch.bfloat16, device="cuda")
    if K.gemm_workspace_bytes(128, 256, 8192, "mxfp8") > 0:  # split along K: no scattered output
        with pytest.raises(TilefishPreconditionError):
            K.gemm_blockscaled_scatter(qa, qb, [d.data_ptr()], 128, 256)
    with pytest.raises(TilefishPreconditionError):
        K.gemm_blockscaled_scatter(qa, qb, [d.data_ptr(), d.data_ptr()], 128, 256)  # m is not owners x rows_per_owner
    with pytest.raises(TilefishPreconditionError):
        K.gemm_blockscaled_scatter(qa, qb, [d.data_ptr() + 2], 128, 256)  # unaligned destination
