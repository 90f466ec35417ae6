"""tilefish.run / runtime.export / replay / capture of the typed decoder-block graph on a GPU, against the CPU oracle.

The graph is the README's (python/tests/test_graphs.py:27-49 of the reference) with BlockScaled weights, preceded by
residual_add_rmsnorm: what the fourth benchmark configuration runs (H = 2560, F = 3072, MXFP8).
"""

import pytest
import torch

import tilefish_b200 as tilefish
from oracle import blockscaled as O
from tilefish_b200 import Dim, InOut, Tensor, bf16, const, f32, mxfp8, nvfp4

pytestmark = pytest.mark.gpu

M = Dim("M", buckets=[1, 32, 512])
H = Dim("H", 2560)
F = Dim("F", 3072)


def declare(fmt):
    @tilefish.kernel
    def residual_add_rmsnorm(x: Tensor[M, H, bf16], residual: InOut[Tensor[M, H, f32]], w: Tensor[H, bf16], *, eps: const[f32] = 1e-6) -> Tensor[M, H, bf16]:
        r = residual + x.to(f32)
        residual[...] = r
        rstd = tilefish.rsqrt(tilefish.mean(r * r, axis=-1, keepdims=True) + eps)
        return (r * rstd * w.to(f32)).to(bf16)

    @tilefish.library("gemm_gu", acc=f32)
    def gemm_gu(a: Tensor[M, H, bf16], b: Tensor[2 * F, H, fmt]) -> Tensor[M, 2 * F, bf16]: ...

    @tilefish.library("gemm_d", acc=f32)
    def gemm_d(a: Tensor[M, F, bf16], b: Tensor[H, F, fmt]) -> Tensor[M, H, bf16]: ...

    @tilefish.graph(inputs=("x",), weights=("w_n", "w_gu", "w_d"))
    def block(x: Tensor[M, H, bf16], residual: InOut[Tensor[M, H, f32]], w_n: Tensor[H, bf16], w_gu: Tensor[2 * F, H, fmt], w_d: Tensor[H, F, fmt]):
        h = residual_add_rmsnorm(x, residual, w_n)
        g, u = gemm_gu(h, w_gu).split(F, axis=-1)
        return gemm_d((tilefish.silu(g.to(f32)) * u.to(f32)).to(bf16), w_d)

    return residual_add_rmsnorm, gemm_gu, block


def inputs(m, seed=0):
    x = O.randn((m, 2560), seed, torch.bfloat16)
    res = O.randn((m, 2560), seed + 1)
    w_n = (1 + 0.1 * O.randn((2560,), seed + 2)).to(torch.bfloat16)
    w_gu = O.randn((6144, 2560), seed + 3, torch.bfloat16, scale=2560**-0.5)
    w_d = O.randn((2560, 3072), seed + 4, torch.bfloat16, scale=3072**-0.5)
    return x, res, w_n, w_gu, w_d


def check_block(y, res_gpu, x, res, w_n, w_gu, w_d, fmt_name):
    r_ref, y_ref = O.decoder_block(x, res.clone(), w_n, O.quantize(w_gu, fmt_name), O.quantize(w_d, fmt_name), fmt_name)
    assert torch.equal(res_gpu.cpu(), r_ref)
    g, r = y.cpu().float(), y_ref.float()
    assert float((g - r).abs().max()) <= 2.0**-6 * float(r.abs().max())
    assert float((g - r).norm() / r.norm()) <= 1e-2


@pytest.mark.parametrize("fmt", [mxfp8, nvfp4], ids=["mxfp8", "nvfp4"])
@pytest.mark.parametrize("m", [1, 32, 512])
def test_run_graph_jit(fmt, m):
    _, _, block = declare(fmt)
    x, res, w_n, w_gu, w_d = inputs(m)
    name = fmt.format_name
    q_gu, q_d = tilefish.quantize(w_gu.cuda(), name), tilefish.quantize(w_d.cuda(), name)
    res_gpu = res.cuda()
    y = tilefish.run(block, x.cuda(), res_gpu, w_n.cuda(), q_gu, q_d)
    assert y.shape == (m, 2560) and y.dtype == torch.bfloat16
    check_block(y, res_gpu, x, res, w_n, w_gu, w_d, name)


def test_run_single_operators():
    rms, gemm_gu, _ = declare(mxfp8)
    x, res, w_n, w_gu, _ = inputs(32)
    res_gpu = res.cuda()
    h = rms(x.cuda(), res_gpu, w_n.cuda())  # calling a declaration with tensors runs it
    r_ref, h_ref = O.residual_add_rmsnorm(x, res, w_n)
    assert torch.equal(res_gpu.cpu(), r_ref)
    assert float((h.cpu().float() - h_ref.float()).abs().max()) <= 2.0**-7 * float(h_ref.float().abs().max())
    t = tilefish.run(gemm_gu, h, tilefish.quantize(w_gu.cuda(), "mxfp8"))
    ref = O.gemm_bf16_a(h.cpu(), O.quantize(w_gu, "mxfp8"), "mxfp8")
    assert float((t.cpu().float() - ref.float()).abs().max()) <= 2.0**-8 * 1.01 * float(ref.float().abs().max())


def test_preconditions_are_checked_before_any_launch():
    from tilefish_b200 import TilefishPreconditionError

    _, _, block = declare(mxfp8)
    x, res, w_n, w_gu, w_d = inputs(32)
    q_gu, q_d = tilefish.quantize(w_gu.cuda(), "mxfp8"), tilefish.quantize(w_d.cuda(), "mxfp8")
    res_gpu = res.cuda()
    before = res_gpu.clone()
    cases = [
        ((x.cuda().float(), res_gpu, w_n.cuda(), q_gu, q_d), "dtype"),
        ((x.cuda()[:, :2048].contiguous(), res_gpu, w_n.cuda(), q_gu, q_d), "static_size"),
        ((x.cuda(), res_gpu[:16], w_n.cuda(), q_gu, q_d), "shape"),
        ((x.cuda(), res_gpu, w_n.cuda(), tilefish.quantize(w_gu.cuda(), "mxfp4"), q_d), "dtype"),
        ((x.cuda(), res_gpu, w_n.cuda(), w_gu.cuda(), q_d), "dtype"),
        ((x, res_gpu, w_n.cuda(), q_gu, q_d), "device"),
    ]
    for args, kind in cases:
        with pytest.raises(TilefishPreconditionError) as e:
            tilefish.run(block, *args)
        assert e.value.kind == kind, (kind, str(e.value))
    assert torch.equal(res_gpu, before), "a refused call must not have launched anything"


def test_export_replay_and_capture(tmp_path):
    from tilefish_b200 import TilefishManifestError, TilefishPreconditionError, runtime

    _, _, block = declare(mxfp8)
    exp = runtime.export(block, str(tmp_path / "mlp"))
    assert len(exp.digest) == 64 and (tmp_path / "mlp" / "plan.json").exists() and (tmp_path / "mlp" / "manifest.json").exists()
    x, res, w_n, w_gu, w_d = inputs(32, seed=7)
    q_gu, q_d = tilefish.quantize(w_gu.cuda(), "mxfp8"), tilefish.quantize(w_d.cuda(), "mxfp8")
    res_a, res_b = res.cuda(), res.cuda()
    y_jit = tilefish.run(block, x.cuda(), res_a, w_n.cuda(), q_gu, q_d)
    y_rep = tilefish.run(block, x.cuda(), res_b, w_n.cuda(), q_gu, q_d, mode="replay", plan=exp.directory, pin=exp.digest)
    assert torch.equal(y_jit, y_rep) and torch.equal(res_a, res_b), "replay and jit run the same kernels: identical bytes"
    check_block(y_rep, res_b, x, res, w_n, w_gu, w_d, "mxfp8")
    with pytest.raises(TilefishManifestError):
        tilefish.run(block, x.cuda(), res_b, w_n.cuda(), q_gu, q_d, mode="replay", plan=exp.directory, pin="0" * 64)
    x7 = O.randn((7, 2560), 1, torch.bfloat16).cuda()
    with pytest.raises(TilefishPreconditionError) as e:
        tilefish.run(block, x7, torch.zeros((7, 2560), device="cuda"), w_n.cuda(), q_gu, q_d, mode="replay", plan=exp.directory, pin=exp.digest)
    assert e.value.kind == "bucket"

    # capture: one CUDA graph launch per step; new inputs are written into the captured tensors
    xg, rg = x.cuda(), res.cuda()
    cap = tilefish.capture(block, xg, rg, w_n.cuda(), q_gu, q_d, plan=exp.directory, pin=exp.digest)
    x2, res2 = O.randn((32, 2560), 11, torch.bfloat16), O.randn((32, 2560), 12)
    xg.copy_(x2.cuda())
    rg.copy_(res2.cuda())
    y = cap.replay()
    torch.cuda.synchronize()
    check_block(y, rg, x2, res2, w_n, w_gu, w_d, "mxfp8")


def test_replay_trust_anchor_outputs_taps_bound_weights_and_single_steps(tmp_path):
    """The rest of the reference's run-time API for a graph (python/src/tilefish/runtime.py:1275-1406): a replay needs a trust anchor,
    ``outputs=`` receives the result, ``taps=`` copies a plan buffer out after a step, ``bind_weights`` binds the weights once,
    ``prepare`` does the allocations ahead of a capture, ``run_step`` launches one step of the verified plan."""
    from tilefish_b200 import TilefishManifestError, TilefishRuntimeError, runtime

    _, _, block = declare(nvfp4)
    exp = runtime.export(block, str(tmp_path / "mlp4"))
    x, res, w_n, w_gu, w_d = inputs(32, seed=3)
    q_gu, q_d = tilefish.quantize(w_gu.cuda(), "nvfp4"), tilefish.quantize(w_d.cuda(), "nvfp4")
    args = lambda r: (x.cuda(), r, w_n.cuda(), q_gu, q_d)  # noqa: E731
    with pytest.raises(TilefishManifestError, match="trust anchor"):
        tilefish.run(block, *args(res.cuda()), mode="replay", plan=exp.directory)
    with pytest.raises(TilefishManifestError, match="not both"):
        tilefish.run(block, *args(res.cuda()), mode="replay", plan=exp.directory, pin=exp.digest, trust_directory=True)
    with pytest.raises(TilefishRuntimeError, match="for mode='replay'"):
        tilefish.run(block, *args(res.cuda()), pin=exp.digest)
    res_a = res.cuda()
    y_ref = tilefish.run(block, *args(res_a), mode="replay", plan=exp.directory, pin=exp.digest)
    check_block(y_ref, res_a, x, res, w_n, w_gu, w_d, "nvfp4")

    # outputs= and taps=: the result lands in the caller's tensor; the bf16 activation of the first GEMM is copied out after its step
    doc = exp.plan.doc
    steps = next(b for b in doc["buckets"] if b["values"] == {"M": 32})["steps"]
    gemm1 = next(i for i, s in enumerate(steps) if s.get("entry", "").startswith("gemm_gu"))
    a_name = next(a["binding"] for a in steps[gemm1]["args"] if a["name"] == "out")
    out = torch.empty((32, 2560), dtype=torch.bfloat16, device="cuda")
    tap = torch.zeros((32, 3072), dtype=torch.bfloat16, device="cuda")
    res_b = res.cuda()
    y = tilefish.run(block, *args(res_b), mode="replay", plan=exp.directory, trust_directory=True, outputs=[out], taps={a_name: tap})
    assert y is out and torch.equal(out, y_ref) and torch.equal(res_b, res_a)
    assert float(tap.float().abs().max()) > 0  # silu(g) * u of the block, as the plan computed it
    r_ref, h_ref = O.residual_add_rmsnorm(x, res.clone(), w_n)
    t_ref = O.gemm_bf16_a(h_ref, O.quantize(w_gu, "nvfp4"), "nvfp4")
    a_ref = O.silu_gate(t_ref[:, :3072], t_ref[:, 3072:])
    assert float((tap.cpu().float() - a_ref.float()).norm() / a_ref.float().norm()) <= 1e-2

    # weights bound once; prepare() before a capture
    runtime.prepare(block, mode="replay", plan=exp.directory, pin=exp.digest)
    w = tilefish.bind_weights(block, {"w_n": w_n.cuda(), "w_gu": q_gu, "w_d": q_d}, mode="replay", plan=exp.directory, pin=exp.digest)
    res_c = res.cuda()
    assert torch.equal(w.run(x.cuda(), res_c), y_ref) and torch.equal(res_c, res_a)
    xg, rg = x.cuda(), res.cuda()
    cap = w.capture(xg, rg)
    rg.copy_(res.cuda())
    assert torch.equal(cap.replay(), y_ref)
    torch.cuda.synchronize()
    with pytest.raises(TilefishRuntimeError, match="not a weight"):
        tilefish.bind_weights(block, {"x": x.cuda()})

    # one step of the plan on the caller's tensors: the last GEMM, fed the quantized activation the tap of its input gives
    last = len(steps) - 1
    binds = {a["name"]: a["binding"] for a in steps[last]["args"]}
    aq = tilefish.quantize(tap, "nvfp4")
    out2 = torch.empty((32, 2560), dtype=torch.bfloat16, device="cuda")
    tilefish.run_step(block, last, {binds["a"]: aq, "w_d": q_d, "out0": out2}, mode="replay", plan=exp.directory, pin=exp.digest, bucket={"M": 32})
    torch.cuda.synchronize()
    assert float((out2.float() - y_ref.float()).norm() / y_ref.float().norm()) <= 2e-2  # the plan derived a's global scale from the producer's amax: same value


def test_config4_block_at_8192_rows_matches_the_oracle_on_sampled_rows():
    """The fourth benchmark configuration's largest bucket (M = 8192, H = 2560, F = 3072, MXFP8), through the typed API: rows are independent
    for the MX formats, so 96 sampled rows are compared with the oracle run on those rows alone."""
    Mbig = Dim("M", buckets=[8192])

    @tilefish.kernel
    def residual_add_rmsnorm(x: Tensor[Mbig, H, bf16], residual: InOut[Tensor[Mbig, H, f32]], w: Tensor[H, bf16], *, eps: const[f32] = 1e-6) -> Tensor[Mbig, H, bf16]:
        r = residual + x.to(f32)
        residual[...] = r
        rstd = tilefish.rsqrt(tilefish.mean(r * r, axis=-1, keepdims=True) + eps)
        return (r * rstd * w.to(f32)).to(bf16)

    @tilefish.library("gemm_gu", acc=f32)
    def gemm_gu(a: Tensor[Mbig, H, bf16], b: Tensor[2 * F, H, mxfp8]) -> Tensor[Mbig, 2 * F, bf16]: ...

    @tilefish.library("gemm_d", acc=f32)
    def gemm_d(a: Tensor[Mbig, F, bf16], b: Tensor[H, F, mxfp8]) -> Tensor[Mbig, H, bf16]: ...

    @tilefish.graph(inputs=("x",), weights=("w_n", "w_gu", "w_d"))
    def block(x: Tensor[Mbig, H, bf16], residual: InOut[Tensor[Mbig, H, f32]], w_n: Tensor[H, bf16], w_gu: Tensor[2 * F, H, mxfp8], w_d: Tensor[H, F, mxfp8]):
        h = residual_add_rmsnorm(x, residual, w_n)
        g, u = gemm_gu(h, w_gu).split(F, axis=-1)
        return gemm_d((tilefish.silu(g.to(f32)) * u.to(f32)).to(bf16), w_d)

    x, res, w_n, w_gu, w_d = inputs(8192, seed=21)
    q_gu, q_d = tilefish.quantize(w_gu.cuda(), "mxfp8"), tilefish.quantize(w_d.cuda(), "mxfp8")
    res_gpu = res.cuda()
    y = tilefish.run(block, x.cuda(), res_gpu, w_n.cuda(), q_gu, q_d)
    rows = torch.randint(0, 8192, (96,), generator=torch.Generator().manual_seed(2))
    rows[:3] = torch.tensor([0, 127, 8191])
    r_ref, y_ref = O.decoder_block(x[rows], res[rows].clone(), w_n, O.quantize(w_gu, "mxfp8"), O.quantize(w_d, "mxfp8"), "mxfp8")
    assert torch.equal(res_gpu[rows.cuda()].cpu(), r_ref)
    g, r = y[rows.cuda()].cpu().float(), y_ref.float()
    assert float((g - r).abs().max()) <= 2.0**-6 * float(r.abs().max())
    assert float((g - r).norm() / r.norm()) <= 1e-2


@pytest.mark.parametrize("fmt", [mxfp8, nvfp4], ids=["mxfp8", "nvfp4"])
def test_native_replay_loop_gives_the_python_runner_s_bytes(fmt, tmp_path):
    """The C++ replay loop (tf_plan_*, csrc/plan_replay.cu) over the exported directory: launched step by step and replayed from the
    CUDA graph it captures, it must produce the bytes the Python runner produces (they call the same entry points with the same
    arguments), for every bucket; a missing binding is refused before anything is launched."""
    from tilefish_b200 import TilefishPreconditionError, runtime
    from tilefish_b200.native_plan import NativePlan

    _, _, block = declare(fmt)
    name = fmt.format_name
    exp = runtime.export(block, str(tmp_path / "native"))
    plan = NativePlan(exp.directory, pin=exp.digest)
    assert plan.digest == exp.digest
    for m in (1, 32, 512):
        x, res, w_n, w_gu, w_d = inputs(m, seed=m)
        q_gu, q_d = tilefish.quantize(w_gu.cuda(), name), tilefish.quantize(w_d.cuda(), name)
        res_py = res.cuda()
        y_py = tilefish.run(block, x.cuda(), res_py, w_n.cuda(), q_gu, q_d, mode="replay", plan=exp.directory, pin=exp.digest)
        xg, res_n, wn = x.cuda(), res.cuda(), w_n.cuda()
        out = torch.empty((m, 2560), dtype=torch.bfloat16, device="cuda")
        bucket = plan.find_bucket(M=m)
        if m == 1:
            plan.bind(x=xg, residual=res_n, w_n=wn, w_gu=q_gu, w_d=q_d)
            before = res_n.clone()
            with pytest.raises(TilefishPreconditionError, match="no tensor is bound to buffer 'out0'"):
                plan.launch(bucket)
            torch.cuda.synchronize()
            assert torch.equal(res_n, before), "a refused launch must not have run a step"
        plan.bind(x=xg, residual=res_n, w_n=wn, w_gu=q_gu, w_d=q_d, out0=out)
        plan.launch(bucket)
        torch.cuda.synchronize()
        assert torch.equal(out, y_py) and torch.equal(res_n, res_py)
        g = plan.capture(bucket)
        res_n.copy_(res.cuda())
        out.zero_()
        plan.replay(g)
        torch.cuda.synchronize()
        assert torch.equal(out, y_py) and torch.equal(res_n, res_py)
    plan.close()
