"""The typed front end (Dim / Tensor / BlockScaled, @kernel / @library / @graph) and the plan machinery, without a GPU.

What is asserted is the public behaviour the reference's own CPU tests pin for this subset (python/tests/test_types.py:78-112,
python/tests/test_graphs.py:51-119, python/tests/test_calls.py:216-228): spellings, equality, the node list and text form of the
README kernel and graph, rounding points, and the refusals of the call checker.
"""

import json

import pytest

import tilefish_b200 as tilefish
from tilefish_b200 import BlockScaled, Dim, InOut, Tensor, bf16, const, e2m1, e4m3, f32, ue8m0
from tilefish_b200 import TilefishDeclarationError, TilefishLoweringError, TilefishManifestError, TilefishPlanError, TilefishTypeError

M = Dim("M", buckets=[1, 32])
D = Dim("D", 2560)
H = Dim("H", 1024)
F = Dim("F", 3072)
K = Dim("K", divisible_by=32)
N = Dim("N", divisible_by=128)
mxfp8 = BlockScaled(elem=e4m3, scale=ue8m0, block=32, axis=-1)
nvfp4 = BlockScaled(elem=e2m1, scale=e4m3, block=16, global_scale=f32)


@tilefish.library("gemm", acc=f32)
def gemm(a: Tensor[M, K, bf16], b: Tensor[N, K, mxfp8]) -> Tensor[M, N, bf16]: ...


@tilefish.graph
def mlp(x: Tensor[M, H, bf16], w_gu: Tensor[2 * F, H, mxfp8], w_d: Tensor[H, F, mxfp8]):
    g, u = gemm(x, w_gu).split(F, axis=-1)
    a = (tilefish.silu(g.to(f32)) * u.to(f32)).to(bf16)
    return gemm(a, w_d)


@tilefish.kernel
def residual_add_rmsnorm(x: Tensor[M, D, bf16], residual: InOut[Tensor[M, D, f32]], w: Tensor[D, bf16], *, eps: const[f32] = 1e-6) -> Tensor[M, D, bf16]:
    r = residual + x.to(f32)
    residual[...] = r
    rstd = tilefish.rsqrt(tilefish.mean(r * r, axis=-1, keepdims=True) + eps)
    return (r * rstd * w.to(f32)).to(bf16)


def test_dims():
    assert repr(Dim("M")) == "Dim('M')" and repr(D) == "Dim('D', 2560)" and repr(K) == "Dim('K', divisible_by=32)"
    assert repr(M) == "Dim('M', buckets=[1, 32])" and str(M) == "M"
    assert D == 2560 and 2 * F == 6144 and 2 * F == F + F and repr(2 * F) == "DimExpr(6144)"
    assert repr(2 * Dim("T")) == "DimExpr(2*T)" and repr(Dim("T") + 1) == "DimExpr(T + 1)"
    assert Dim("K", divisible_by=32) == K and Dim("K") != K
    assert tilefish.cdiv(K, 32) != tilefish.cdiv(K, 16)
    with pytest.raises(TilefishDeclarationError):
        Dim("X", 4, buckets=[1])
    with pytest.raises(TilefishDeclarationError):
        Dim("X", buckets=[2, 1])


def test_blockscaled_types():
    assert repr(mxfp8) == "BlockScaled(elem=e4m3, scale=ue8m0, block=32, axis=-1)" and str(mxfp8) == "blockscaled(e4m3, ue8m0, 32)"
    assert str(nvfp4) == "blockscaled(e2m1, e4m3, 16, global_scale=f32)"
    t = Tensor[M, K, mxfp8]
    assert repr(t) == "Tensor[M, K, blockscaled(e4m3, ue8m0, 32)]" and t.rank == 2 and t.contiguous
    assert repr(t.scale_type) == "Tensor[M, cdiv(K, 32), ue8m0]"
    assert Tensor[M, 4096, nvfp4].scale_shape == (M, 256)
    assert Tensor[M, K, BlockScaled(e4m3, ue8m0, 32, axis=1)] == t  # axis -1 and its normalised spelling are one type
    assert e2m1.elems_per_byte == 2 and not e4m3.computable
    assert mxfp8.format_name == "mxfp8" and nvfp4.format_name == "nvfp4" and BlockScaled(e4m3, ue8m0, 64).format_name is None
    with pytest.raises(TilefishTypeError):
        Tensor[M, Dim("Q"), mxfp8]  # the blocked axis is not provably a multiple of 32
    with pytest.raises(TilefishDeclarationError):
        BlockScaled(e2m1, ue8m0, 3)
    assert repr(Tensor[M, F, bf16].as_view()) == "View[M, F, bf16]" and Tensor[M, F, bf16].as_view() != Tensor[M, F, bf16]
    assert repr(InOut[Tensor[M, D, f32]]) == "InOut[Tensor[M, D, f32]]" and repr(const[f32]) == "const[f32]"


def test_mlp_traces_to_the_readme_node_list():
    g = mlp.graph
    assert isinstance(mlp, tilefish.GraphOp) and isinstance(gemm, tilefish.LibraryOp) and gemm.acc is f32
    assert g.kind == "graph" and g.name == "mlp"
    assert g.ops() == ["gemm", "split", "cast", "silu", "cast", "mul", "cast", "gemm"]
    gemm_up, split, cast_g, silu, cast_u, mul, cast_a, gemm_down = g.nodes
    assert gemm_up.output_types == (Tensor[M, 6144, bf16],) and gemm_up.attrs["acc"] is f32
    assert split.attrs == {"axis": 1, "sizes": (F, F)}
    assert split.output_types == (Tensor[M, F, bf16].as_view(),) * 2
    assert cast_a.attrs == {"to": bf16, "rounding": True} and not cast_g.is_rounding_point
    assert gemm_down.output_types == (Tensor[M, H, bf16],) and g.outputs == gemm_down.outputs
    assert g.symbols == (M,)
    text = str(g)
    assert text.startswith("graph mlp(%x: Tensor[M, H, bf16], %w_gu: Tensor[6144, H, blockscaled(e4m3, ue8m0, 32)]")
    assert "%1: View[M, F, bf16], %2: View[M, F, bf16] = split(%0) {axis=1, sizes=(F, F)}" in text
    assert "%7: Tensor[M, F, bf16] = cast(%6) {to=bf16, rounding=true}  # rounding point" in text
    assert text.endswith("return %8")
    assert mlp.signature.returns == (Tensor[M, H, bf16],)


def test_rmsnorm_kernel_trace():
    g = residual_add_rmsnorm.graph
    assert isinstance(residual_add_rmsnorm, tilefish.KernelOp) and g.kind == "kernel"
    assert g.ops() == ["cast", "add", "store", "mul", "mean", "add", "rsqrt", "mul", "cast", "mul", "cast"]
    assert len(g.rounding_points()) == 1 and g.rounding_points()[0].outputs == g.outputs
    assert g.nodes[2].attrs == {"target": "residual"} and g.nodes[4].attrs == {"axes": (1,), "keepdims": True}
    assert g.nodes[4].output_types == (Tensor[M, 1, f32],)
    assert g.nodes[5].inputs[1].name == "eps" and g.nodes[5].inputs[1].dtype is f32
    assert "eps: const[f32] = 1e-06" in str(g) and str(g).endswith("final residual = %2")


def test_call_checker_refusals():
    mxfp4 = BlockScaled(elem=e2m1, scale=ue8m0, block=32)
    with pytest.raises(TilefishTypeError, match="expected blockscaled"):
        @tilefish.graph
        def bad(x: Tensor[M, H, bf16], w: Tensor[2 * F, H, mxfp4]):
            return gemm(x, w)
    with pytest.raises(TilefishTypeError, match="strided view"):
        @tilefish.graph
        def bad2(x: Tensor[M, H, bf16], w: Tensor[2 * F, H, mxfp8], w2: Tensor[H, F, mxfp8]):
            g, u = gemm(x, w).split(F, axis=-1)
            return gemm(g, w2)
    with pytest.raises(TilefishTypeError, match="no implicit promotion"):
        @tilefish.kernel
        def bad3(x: Tensor[M, D, bf16], y: Tensor[M, D, f32]) -> Tensor[M, D, f32]:
            return x + y
    with pytest.raises(TilefishTypeError, match="storage only"):
        @tilefish.kernel
        def bad4(x: Tensor[M, D, e4m3]) -> Tensor[M, D, e4m3]:
            return x + x
    with pytest.raises(TilefishDeclarationError, match="never written"):
        @tilefish.kernel
        def bad5(x: Tensor[M, D, bf16], r: InOut[Tensor[M, D, f32]]) -> Tensor[M, D, f32]:
            return x.to(f32)


def test_quantize_is_a_traced_cast():
    @tilefish.graph
    def q(x: Tensor[M, H, bf16], w: Tensor[N, H, mxfp8]):
        return gemm(x.to(mxfp8), w) if False else gemm(x, w)

    @tilefish.library("gemm_q", acc=f32)
    def gemm_q(a: Tensor[M, K, mxfp8], b: Tensor[N, K, mxfp8]) -> Tensor[M, N, bf16]: ...

    @tilefish.graph
    def q2(x: Tensor[M, H, bf16], w: Tensor[256, H, mxfp8]):
        return gemm_q(x.to(mxfp8), w)

    assert q2.graph.ops() == ["quantize", "gemm_q"]
    assert q2.graph.nodes[0].output_types == (Tensor[M, H, mxfp8],)


def block_graph(fmt):
    Mb, Hb, Fb = Dim("M", buckets=[1, 32, 512]), Dim("H", 2560), Dim("F", 3072)

    @tilefish.kernel
    def rms(x: Tensor[Mb, Hb, bf16], residual: InOut[Tensor[Mb, Hb, f32]], w: Tensor[Hb, bf16], *, eps: const[f32] = 1e-6) -> Tensor[Mb, Hb, bf16]:
        r = residual + x.to(f32)
        residual[...] = r
        rstd = tilefish.rsqrt(tilefish.mean(r * r, axis=-1, keepdims=True) + eps)
        return (r * rstd * w.to(f32)).to(bf16)

    @tilefish.library("gemm_gu", acc=f32)
    def gemm_gu(a: Tensor[Mb, Hb, bf16], b: Tensor[2 * Fb, Hb, fmt]) -> Tensor[Mb, 2 * Fb, bf16]: ...

    @tilefish.library("gemm_d", acc=f32)
    def gemm_d(a: Tensor[Mb, Fb, bf16], b: Tensor[Hb, Fb, fmt]) -> Tensor[Mb, Hb, bf16]: ...

    @tilefish.graph(inputs=("x",), weights=("w_n", "w_gu", "w_d"))
    def block(x: Tensor[Mb, Hb, bf16], residual: InOut[Tensor[Mb, Hb, f32]], w_n: Tensor[Hb, bf16], w_gu: Tensor[2 * Fb, Hb, fmt], w_d: Tensor[Hb, Fb, fmt]):
        h = rms(x, residual, w_n)
        g, u = gemm_gu(h, w_gu).split(Fb, axis=-1)
        return gemm_d((tilefish.silu(g.to(f32)) * u.to(f32)).to(bf16), w_d)

    return block


def test_plan_of_the_decoder_block():
    from tilefish_b200 import _plan

    block = block_graph(mxfp8)
    p = tilefish.plan(block)
    doc = p.doc
    assert doc["schema"] == "tilefish.plan.v1" and doc["arena_alignment"] == 256 and sorted(doc["buckets"]) == ["M=1", "M=32", "M=512"]
    # three launches: both activation quantizations are done by the kernels that produce the activations
    assert [s["entry"] for s in doc["steps"]] == ["rms", "gemm_gu", "gemm_d"]
    assert [s["kind"] for s in doc["steps"]] == ["kernel", "library", "library"]
    assert doc["steps"][1]["attrs"] == {"format": "mxfp8", "epilogue": "silu_gate", "impl": "sm100.gemm_blockscaled", "q_format": "mxfp8"}
    assert doc["steps"][0]["attrs"]["q_format"] == "mxfp8" and "out" not in doc["steps"][0]["args"]  # rmsnorm emits the quantized copy only
    assert "out" not in doc["steps"][1]["args"] and doc["steps"][2]["args"]["a"] == doc["steps"][1]["args"]["q"]  # `a` never exists in bf16
    roles = {b["name"]: b["role"] for b in doc["buffers"]}
    assert roles["x"] == "input" and roles["residual"] == "inout" and roles["w_gu"] == "weight" and roles["out0"] == "output"
    b32 = doc["buckets"]["M=32"]
    for name, entry in b32["buffers"].items():
        for off in entry.get("offset", {}).values():
            assert off % 256 == 0
    act = next(n for n, r in roles.items() if r == "intermediate" and b32["buffers"][n]["bytes"].get("codes") == 32 * 2560)
    assert b32["buffers"][act]["bytes"]["scales"] == 512 * 20  # one row tile x 20 column tiles of swizzled ue8m0 bytes
    assert p.digest == tilefish.plan(block).digest and len(p.digest) == 64
    assert p.digest == _plan.digest("tilefish.plan-digest.v1", {k: v for k, v in doc.items() if k != "plan_digest"})
    # nvfp4: amax is reduced by the producers and consumed by the quantizers; an aux buffer carries it
    steps = tilefish.plan(block_graph(nvfp4)).doc["steps"]
    assert [s["entry"] for s in steps] == ["rms", "quantize.nvfp4", "gemm_gu", "quantize.nvfp4", "gemm_d"]
    assert steps[0]["args"]["amax"] == steps[1]["args"]["amax"] == "aux[0]" and steps[2]["args"]["amax"] == steps[3]["args"]["amax"] == "aux[1]"


def test_plan_refusals_and_unfused_form():
    from tilefish_b200 import _plan, backend

    bufs, steps = backend.compile_graph(block_graph(mxfp8), fuse=False)
    assert [s.impl for s in steps] == ["tf_residual_add_rmsnorm", "tf_quantize_mxfp8", "tf_gemm_blockscaled", "tf_silu_gate", "tf_quantize_mxfp8",
                                       "tf_gemm_blockscaled"]
    assert steps[3].args["gate"].endswith("[:, 0]") and steps[3].args["up"].endswith("[:, 1]")

    with pytest.raises(TilefishPlanError, match="no buckets"):
        tilefish.plan(mlp.__class__(mlp.fn, "m2", mlp.signature, _free_graph().graph, {}))
    with pytest.raises(TilefishLoweringError) as e:
        @tilefish.kernel
        def other(x: Tensor[M, D, bf16]) -> Tensor[M, D, bf16]:
            return (x.to(f32) * 2.0).to(bf16)
        backend.match_kernel(other)
    assert e.value.rule == "no-template"

    @tilefish.library("gemm_bf16", acc=f32)
    def gemm_bf16(a: Tensor[M, K, bf16], b: Tensor[N, K, bf16]) -> Tensor[M, N, bf16]: ...

    @tilefish.graph
    def g_bf16(x: Tensor[M, H, bf16], w: Tensor[256, H, bf16]):
        return gemm_bf16(x, w)

    with pytest.raises(TilefishPlanError, match="BlockScaled weights only"):
        tilefish.plan(g_bf16)


def _free_graph():
    T = Dim("T")

    @tilefish.graph
    def free(x: Tensor[T, H, bf16], w: Tensor[256, H, mxfp8]):
        return gemm(x, w)

    return free


def test_export_files_round_trip_and_tamper_detection(tmp_path):
    from tilefish_b200 import _plan

    block = block_graph(mxfp8)
    p, manifest = _plan.make_plan(block, library={"file": "libtilefish_b200.so", "sha256": "0" * 64, "version": "test"})
    d = str(tmp_path / "export")
    _plan.write_export(d, p, manifest)
    doc, man = _plan.load_export(d, pin=p.digest)
    assert doc == p.doc and man == manifest
    with pytest.raises(TilefishManifestError, match="pins"):
        _plan.load_export(d, pin="f" * 64)
    with pytest.raises(TilefishManifestError, match="already holds"):
        _plan.write_export(d, p, manifest)
    path = tmp_path / "export" / "plan.json"
    tampered = json.loads(path.read_text())
    tampered["steps"][1]["attrs"]["epilogue"] = "none"
    path.write_text(json.dumps(tampered))
    with pytest.raises(TilefishManifestError, match="does not match its own digest"):
        _plan.load_export(d)
    path.write_text("{not json")
    with pytest.raises(TilefishManifestError, match="not valid JSON"):
        _plan.load_export(d)


def test_runner_checks_everything_before_the_first_launch():
    """A recording backend in place of the CUDA one: nothing is launched when a precondition fails (the pattern of the
    reference's FakeBackend, python/tests/test_planrun.py:49)."""
    from tilefish_b200 import runtime
    from tilefish_b200.errors import TilefishPreconditionError

    class Recording(runtime.Backend):
        def __init__(self):
            self.calls = []

        def alloc_arena(self, nbytes, device):
            raise AssertionError("nothing may be allocated for a refused call")

        def launch(self, step, tensors):
            self.calls.append(step["entry"])

        def gemm(self, step, tensors):
            self.calls.append(step["entry"])

    rec = Recording()
    runner = runtime.PlanRunner(tilefish.plan(block_graph(mxfp8)).doc, backend=rec)
    with pytest.raises(TilefishPreconditionError) as e:
        runner.run("M=7", {}, device=None)
    assert e.value.kind == "bucket" and rec.calls == []
    with pytest.raises(tilefish.TilefishRuntimeError, match="not part of this backend"):
        runtime.run(block_graph(mxfp8), mode="reference")
