"""The typed front end (Dim / Tensor / BlockScaled, @kernel / @library / @graph) and the plan machinery, without a GPU.

What is asserted is the public behaviour the reference's own CPU tests pin for this subset (python/tests/test_types.py:78-112,
python/tests/test_graphs.py:51-119, python/tests/test_calls.py:216-228): spellings, equality, the node list and text form of the
README kernel and graph, rounding points, and the refusals of the call checker.
"""

import json
import os

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
    assert Dim("X", buckets=[2, 1]).buckets == (1, 2)  # kept sorted, as the reference does
    with pytest.raises(TilefishDeclarationError):
        Dim("X", buckets=[2, 2])


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
    with pytest.raises(TilefishTypeError, match="expected dtype blockscaled"):
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
    with pytest.raises(TilefishTypeError, match="storage dtype"):
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


def _steps(doc, m):
    return next(b for b in doc["buckets"] if b["values"] == {"M": m})["steps"]


def _args(step):
    return {a["name"]: a["binding"] for a in step["args"]}


def test_plan_of_the_decoder_block():
    from tilefish_b200 import _plan

    block = block_graph(mxfp8)
    p = tilefish.plan(block)
    doc = p.doc
    # the reference's plan schema 1: exactly these top-level keys (docs/en/plan-schema-1.md, section 2)
    assert set(doc) == set(_plan.TOP_KEYS) | {"roles"} and doc["roles"] == "declared"
    assert doc["schema"] == "tilefish.plan.v1" and doc["arena_alignment"] == 256 and doc["dims"] == {"M": [1, 32, 512]} and doc["outputs"] == ["out0"]
    assert doc["arch"] is None and doc["manifest_digest"] is None  # a plan that was only made; an exported one names sm_100 and its manifest
    assert [b["values"] for b in doc["buckets"]] == [{"M": 1}, {"M": 32}, {"M": 512}]
    # three launches: both activation quantizations are done by the kernels that produce the activations
    steps = _steps(doc, 32)
    assert [s["entry"] for s in steps] == ["rms_qmxfp8", "gemm_gu_silu_gate_qmxfp8.M32", "gemm_d.M32"]
    assert [s["kind"] for s in steps] == ["kernel", "library", "library"]
    assert set(steps[0]) == {"entry", "kind", "args"} and set(steps[1]) == {"entry", "kind", "args", "workspace"}
    lib = p.manifest["library"]["gemm_gu_silu_gate_qmxfp8.M32"]
    assert lib["attrs"] == {"format": "mxfp8", "epilogue": "silu_gate", "q_format": "mxfp8"} and lib["impl"] == "sm100.gemm_blockscaled"
    assert lib["symbol"] == "tf_gemm_blockscaled" and (lib["m"], lib["n"], lib["k"]) == (32, 3072, 2560)
    a0, a1, a2 = _args(steps[0]), _args(steps[1]), _args(steps[2])
    assert "out" not in a0 and "out" not in a1  # rmsnorm and the first gemm emit the quantized copies only: `a` never exists in bf16
    assert a1["a"] == a0["q"] and a1["a_scales"] == a0["q_scales"] and a2["a"] == a1["q"] and a2["a_scales"] == a1["q_scales"]
    # a BlockScaled tensor is separate bindings: codes, swizzled scale bytes (and the global scale for nvfp4)
    assert a1["b"] == "w_gu" and a1["b_scales"] == "w_gu__scales" and [a["name"] for a in steps[1]["args"]] == lib["params"]
    bufs = {b["name"]: b for b in doc["buffers"]}
    assert [b["name"] for b in doc["buffers"]][:7] == ["x", "residual", "w_n", "w_gu", "w_gu__scales", "w_d", "w_d__scales"]
    assert bufs["x"]["role"] == "input" and bufs["residual"]["role"] == "inout" and bufs["w_gu"]["role"] == "weight" and bufs["out0"]["role"] == "output"
    assert bufs["w_gu"]["dtype"] == "e4m3" and bufs["w_gu"]["shape"] == [6144, 2560] and bufs["x"]["shape"] == ["M", 2560]
    for b in doc["buffers"]:
        assert set(b) == {"name", "role", "dtype", "shape", "offset", "bytes"}
        assert (b["offset"] is None) == (b["role"] not in ("intermediate", "workspace"))
        assert b["offset"] is None or (b["offset"] % 256 == 0 and b["offset"] + b["bytes"] <= doc["arena_bytes"])
    act = bufs[a0["q"]]
    assert act["role"] == "intermediate" and act["dtype"] == "e4m3" and act["bytes"] == 512 * 2560
    assert bufs[a0["q_scales"]]["bytes"] == 4 * 20 * 512  # four row tiles x 20 column tiles of swizzled ue8m0 bytes at the largest bucket
    assert bufs["workspace"]["role"] == "workspace" and bufs["workspace"]["bytes"] >= max(e["workspace_bytes"] for e in p.manifest["library"].values())
    assert p.digest == tilefish.plan(block).digest and len(p.digest) == 64
    assert p.digest == _plan.digest("tilefish.plan-digest.v1", {k: v for k, v in doc.items() if k not in ("plan_digest", "tilefish")})
    # nvfp4: amax is reduced by the producers and consumed by the quantizers; an aux buffer carries it and a memset step zeroes it
    doc4 = tilefish.plan(block_graph(nvfp4)).doc
    steps = _steps(doc4, 32)
    assert [s.get("entry", s["kind"]) for s in steps] == ["memset", "rms_amax", "quantize_nvfp4_amax", "gemm_gu_silu_gate_amax.M32", "quantize_nvfp4_amax", "gemm_d.M32"]
    assert steps[0] == {"kind": "memset", "args": [{"name": "dst", "binding": "aux"}]}
    amax = [next(a for a in s["args"] if a["name"] == "amax") for s in steps[1:5]]
    assert [a["view"]["offset"] for a in amax] == [0, 0, 1, 1] and all(a["binding"] == "aux" and a["view"]["shape"] == [1] for a in amax)
    assert {"name": "b_global", "binding": "w_gu__global"} in steps[3]["args"]


def test_reference_validator_accepts_the_plan_and_the_ir_text_is_the_references():
    """With the reference checked out next to this repository: its own ``validate_doc`` reads the documents this package writes, its
    digest function agrees, and the graph prints byte for byte as the reference prints it. Skipped elsewhere."""
    import sys

    src = "/root/reference/python/src"
    if not os.path.isdir(src):
        pytest.skip("the reference checkout is not on this machine")
    from tilefish_b200 import _plan

    sys.path.insert(0, src)
    try:
        import tilefish as ref
        import tilefish._plan as ref_plan
    finally:
        sys.path.remove(src)
    for fmt in (mxfp8, tilefish.mxfp4, nvfp4):
        for fuse in (True, False):
            p = _plan.make_plan(block_graph(fmt), library={"file": "libtilefish_b200.so", "sha256": "0" * 64, "version": "test"}, fuse=fuse)
            ref_plan.validate_doc(p.doc)
            assert ref_plan.plan_digest(p.doc) == p.digest
    ref_plan.validate_doc(tilefish.plan(block_graph(mxfp8)).doc, made=True)

    def declare(t, fmt):
        Mb, Hb, Fb = t.Dim("M", buckets=[1, 32, 512]), t.Dim("H", 2560), t.Dim("F", 3072)

        @t.kernel
        def residual_add_rmsnorm(x: t.Tensor[Mb, Hb, t.bf16], residual: t.InOut[t.Tensor[Mb, Hb, t.f32]], w: t.Tensor[Hb, t.bf16], *, eps: t.const[t.f32] = 1e-6) -> t.Tensor[Mb, Hb, t.bf16]:
            r = residual + x.to(t.f32)
            residual[...] = r
            rstd = t.rsqrt(t.mean(r * r, axis=-1, keepdims=True) + eps)
            return (r * rstd * w.to(t.f32)).to(t.bf16)

        @t.library("gemm_gu", acc=t.f32)
        def gemm_gu(a: t.Tensor[Mb, Hb, t.bf16], b: t.Tensor[2 * Fb, Hb, fmt]) -> t.Tensor[Mb, 2 * Fb, t.bf16]: ...

        @t.library("gemm_d", acc=t.f32)
        def gemm_d(a: t.Tensor[Mb, Fb, t.bf16], b: t.Tensor[Hb, Fb, fmt]) -> t.Tensor[Mb, Hb, t.bf16]: ...

        @t.graph(inputs=("x",), weights=("w_n", "w_gu", "w_d"))
        def block(x: t.Tensor[Mb, Hb, t.bf16], residual: t.InOut[t.Tensor[Mb, Hb, t.f32]], w_n: t.Tensor[Hb, t.bf16], w_gu: t.Tensor[2 * Fb, Hb, fmt],
                  w_d: t.Tensor[Hb, Fb, fmt]):
            h = residual_add_rmsnorm(x, residual, w_n)
            g, u = gemm_gu(h, w_gu).split(Fb, axis=-1)
            return gemm_d((t.silu(g.to(t.f32)) * u.to(t.f32)).to(t.bf16), w_d)

        return str(residual_add_rmsnorm.graph), str(block.graph)

    theirs = declare(ref, ref.BlockScaled(ref.e4m3, ref.ue8m0, 32))
    ours = declare(tilefish, tilefish.BlockScaled(tilefish.e4m3, tilefish.ue8m0, 32))
    assert ours == theirs
    assert "{kind=kernel, consts={eps: 1e-06}, inout=(residual,)}" in ours[1] and ours[1].endswith("final residual = %1")


def test_plan_refusals_and_unfused_form():
    from tilefish_b200 import _plan, backend

    bufs, steps = backend.compile_graph(block_graph(mxfp8), fuse=False)
    assert [s.impl for s in steps] == ["tf_residual_add_rmsnorm", "tf_quantize_mxfp8", "tf_gemm_blockscaled", "tf_silu_gate", "tf_quantize_mxfp8",
                                       "tf_gemm_blockscaled"]
    assert steps[3].args["gate"].endswith("[:, 0]") and steps[3].args["up"].endswith("[:, 1]")
    # in the document the column halves are views of one buffer (docs/en/plan-schema-1.md, section 7.1)
    doc = _plan.make_plan(block_graph(mxfp8), fuse=False).doc
    silu = _steps(doc, 32)[3]
    assert silu["entry"] == "silu_gate" and silu["args"][0]["view"] == {"shape": [32, 3072], "strides": [6144, 1], "offset": 0}
    assert silu["args"][1]["view"] == {"shape": [32, 3072], "strides": [6144, 1], "offset": 3072} and silu["args"][0]["binding"] == silu["args"][1]["binding"]

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


def test_planner_split_rule_matches_the_kernel_library():
    """The planner sizes the workspace from its own restatement of the library's split-K rule for 148 SMs; where the library is built
    (its host-side query needs no GPU and assumes 148 SMs without one) the two must agree."""
    from tilefish_b200 import _native, _plan

    if not os.path.exists(_native.LIB_PATH):
        pytest.skip("library not built here")
    lib = _native.load()
    for fmt, fid in (("mxfp8", 0), ("mxfp4", 1), ("nvfp4", 2)):
        for epi, eid in (("none", 0), ("silu_gate", 1), ("residual", 2)):
            for (m, n, k) in [(1, 6144, 2560), (16, 3072, 2560), (32, 2560, 3072), (64, 28672, 8192), (128, 8192, 28672), (200, 512, 768), (256, 128, 4096),
                              (257, 6144, 2560), (4096, 6144, 2560)]:
                assert _plan.gemm_workspace_bytes(m, n, k, fmt, epi) == lib.tf_gemm_workspace_bytes(m, n, k, fid, eid), (fmt, epi, m, n, k)


def test_export_files_round_trip_and_tamper_detection(tmp_path):
    from tilefish_b200 import _plan

    block = block_graph(mxfp8)
    p = _plan.make_plan(block, library={"file": "libtilefish_b200.so", "sha256": "0" * 64, "version": "test"})
    assert p.doc["arch"] == "sm_100" and p.doc["manifest_digest"] == p.manifest["manifest_digest"]
    d = str(tmp_path / "export")
    _plan.write_export(d, p)
    doc, man = _plan.load_export(d, pin=p.digest)
    assert doc == p.doc and man == p.manifest
    with pytest.raises(TilefishManifestError, match="but the pin is"):
        _plan.load_export(d, pin="f" * 64)
    with pytest.raises(TilefishManifestError, match="already holds"):
        _plan.write_export(d, p)
    with pytest.raises(TilefishManifestError, match="trust anchor"):
        _plan.check_anchor(None, False)
    with pytest.raises(TilefishManifestError, match="not both"):
        _plan.check_anchor(p.digest, True)
    path = tmp_path / "export" / "plan.json"
    good = path.read_text()
    tampered = json.loads(good)
    tampered["buckets"][1]["steps"][1]["entry"] = "gemm_d.M32"
    path.write_text(json.dumps(tampered))
    with pytest.raises(TilefishManifestError, match="was edited"):
        _plan.load_export(d, trust_directory=True)
    # an edit that also rewrites the digest is caught by the pin, and by the manifest's entries when only the directory is trusted
    tampered["plan_digest"] = _plan.plan_digest(tampered)
    path.write_text(json.dumps(tampered))
    with pytest.raises(TilefishManifestError, match="but the pin is"):
        _plan.load_export(d, pin=p.digest)
    with pytest.raises(TilefishManifestError, match="the entry takes"):
        _plan.load_export(d, trust_directory=True)
    path.write_text("{not json")
    with pytest.raises(TilefishManifestError, match="not valid JSON"):
        _plan.load_export(d, trust_directory=True)
    path.write_text(good.replace('"arena_alignment": 256', '"arena_alignment": 256, "arena_alignment": 256'))
    with pytest.raises(TilefishManifestError, match="duplicate key"):
        _plan.load_export(d, trust_directory=True)


class _FakeTensor:
    """What the runner needs of a tensor: an address."""

    def __init__(self, address):
        self.address = address

    def data_ptr(self):
        return self.address


def test_runner_drives_the_backend_through_the_reference_signatures():
    """A recording backend in place of the CUDA one (the pattern of the reference's FakeBackend, python/tests/test_planrun.py:49): the
    order of the launches, the raw addresses (arena + offset, + view.offset * itemsize) and the derived scalars, without a GPU; and
    nothing is allocated or launched when a precondition fails."""
    from tilefish_b200 import _plan, runtime
    from tilefish_b200.errors import TilefishPreconditionError
    from tilefish_b200.kernels import BlockScaledTensor

    class Recording(runtime.Backend):
        ARENA = 0x7F00_0000_0000

        def __init__(self):
            self.calls = []
            self.arenas = 0

        def device_index(self, device):
            return 0

        def current_device(self):
            return 0

        def capturing(self, index):
            return False

        def stream(self, index):
            return 77

        def alloc_arena(self, nbytes, index):
            self.arenas += 1
            return object(), self.ARENA

        def empty(self, shape, dtype, index):
            return _FakeTensor(0x5000_0000)

        def load(self, built, index):
            return built

        def launch(self, loaded, grid, args, stream, scratch=None):
            self.calls.append(("launch", loaded.symbol, tuple(grid), list(args), stream))

        def memset(self, dst, nbytes, stream):
            self.calls.append(("memset", dst, nbytes, stream))

        def gemm(self, spec, algo, a, b, bias, out, workspace, stream, index, c=None, *, scaled=None):
            self.calls.append(("gemm", spec, a, b, bias, out, workspace, stream, index, c, scaled))

    def bs(fmt, shape, base):
        t = BlockScaledTensor(fmt, shape, _FakeTensor(base), _FakeTensor(base + 0x100_0000), _FakeTensor(base + 0x200_0000) if fmt == "nvfp4" else None)
        return t

    for fmt, name in ((mxfp8, "mxfp8"), (nvfp4, "nvfp4")):
        p = _plan.make_plan(block_graph(fmt), exported=False)
        rec = Recording()
        runner = runtime.PlanRunner(p.doc, p.manifest, backend=rec)
        with pytest.raises(TilefishPreconditionError) as e:
            runner.run({"M": 7}, {}, device=None)
        assert e.value.kind == "bucket" and rec.calls == [] and rec.arenas == 0
        tensors = {"x": _FakeTensor(0x1000_0000), "residual": _FakeTensor(0x2000_0000), "w_n": _FakeTensor(0x3000_0000),
                   "w_gu": bs(name, (6144, 2560), 0x4000_0000), "w_d": bs(name, (2560, 3072), 0x4800_0000)}
        # a misaligned pointer is a refusal before anything is enqueued
        bad = dict(tensors, x=_FakeTensor(0x1000_0004))
        with pytest.raises(TilefishPreconditionError) as e:
            runner.run({"M": 32}, bad, device=None)
        assert e.value.kind == "pointer_alignment" and rec.calls == []
        out = runner.run({"M": 32}, tensors, device=None)
        assert out.data_ptr() == 0x5000_0000 and rec.arenas == 1
        bufs = {b["name"]: b for b in p.doc["buffers"]}
        kinds = [c[0] if c[0] != "launch" else c[1] for c in rec.calls]
        if name == "mxfp8":
            assert kinds == ["tf_residual_add_rmsnorm", "gemm", "gemm"]
            rms = rec.calls[0]
            q, qs = (bufs[n]["offset"] + Recording.ARENA for n in ("t0", "t0__scales"))
            assert rms[2] == () and rms[4] == 77
            assert rms[3] == [("ptr", 0x1000_0000), ("ptr", 0x2000_0000), ("ptr", 0x3000_0000), ("ptr", None), ("i64", 32), ("i64", 2560), ("f32", _plan.f32_from_bits(0x358637BD)), ("i32", 0),
                              ("ptr", q), ("ptr", qs), ("i32", 1), ("ptr", None), ("ptr", None)]
            g1 = rec.calls[1]
            spec = g1[1]
            assert (spec.m, spec.n, spec.k, spec.format, spec.epilogue) == (32, 3072, 2560, "mxfp8", "silu_gate") and spec.workspace_bytes == bufs["workspace"]["bytes"]
            assert g1[2] == q and g1[3] == 0x4000_0000 and g1[4] is None and g1[5] is None and g1[6] == Recording.ARENA + bufs["workspace"]["offset"] and g1[7] == 77
            assert g1[10].a_scales == qs and g1[10].b_scales == 0x4100_0000 and g1[10].q_codes == Recording.ARENA + bufs["t1"]["offset"]
            g2 = rec.calls[2]
            assert g2[2] == g1[10].q_codes and g2[5] == 0x5000_0000 and g2[1].ldo == 2560
        else:
            assert kinds == ["memset", "tf_residual_add_rmsnorm", "tf_quantize_nvfp4_from_amax", "gemm", "tf_quantize_nvfp4_from_amax", "gemm"]
            aux = Recording.ARENA + bufs["aux"]["offset"]
            assert rec.calls[0] == ("memset", aux, 32, 77)
            assert rec.calls[1][3][-1] == ("ptr", aux) and rec.calls[2][3][-2] == ("ptr", aux)          # amax slot 0: produced, then consumed
            assert rec.calls[3][10].amax == aux + 4 and rec.calls[4][3][-2] == ("ptr", aux + 4)         # slot 1: view offset 1 x 4 bytes
            assert rec.calls[3][10].b_global == 0x4200_0000 and rec.calls[3][10].a_global == rec.calls[2][3][-1][1]
    with pytest.raises(tilefish.TilefishRuntimeError, match="not part of this backend"):
        runtime.run(block_graph(mxfp8), mode="reference")


def test_native_replay_loop_reads_and_verifies_an_export(tmp_path):
    """tf_plan_load (csrc/plan_replay.cu) on a directory runtime.export wrote: its own JSON reader, canonical writer and SHA-256 give the
    digest Python gave; a pin that differs, an edited file and a plan whose manifest was swapped are refused. Needs no GPU."""
    from tilefish_b200 import _native, _plan

    if not os.path.exists(_native.LIB_PATH):
        pytest.skip("library not built here")
    from tilefish_b200.errors import TilefishPreconditionError
    from tilefish_b200.native_plan import NativePlan

    for fmt in (mxfp8, nvfp4):
        p = _plan.make_plan(block_graph(fmt), library={"file": "libtilefish_b200.so", "sha256": "0" * 64, "version": "test"})
        d = str(tmp_path / ("export_" + str(fmt.format_name)))
        _plan.write_export(d, p)
        n = NativePlan(d, pin=p.digest)
        assert n.digest == p.digest and n.arena_bytes == p.doc["arena_bytes"]
        assert n.find_bucket(M=32) == 1 and n.step_count(1) == len(p.doc["buckets"][1]["steps"])
        with pytest.raises(TilefishPreconditionError) as e:
            n.find_bucket(M=7)
        assert e.value.kind == "bucket"
        n.close()
        with pytest.raises(TilefishPreconditionError, match="but the pin is"):
            NativePlan(d, pin="f" * 64)
        NativePlan(d, trust_directory=True).close()
        with pytest.raises(TilefishManifestError, match="trust anchor"):
            NativePlan(d)
    path = tmp_path / "export_mxfp8" / "plan.json"
    good = path.read_text()
    path.write_text(good.replace('"arena_bytes": ', '"arena_bytes": 1'))
    with pytest.raises(TilefishPreconditionError, match="was edited"):
        NativePlan(str(tmp_path / "export_mxfp8"), trust_directory=True)
    path.write_text(good.replace('"reuse": false', '"reuse": false, "reuse": false'))
    with pytest.raises(TilefishPreconditionError, match="duplicate key"):
        NativePlan(str(tmp_path / "export_mxfp8"), trust_directory=True)
    path.write_text(good)
    mpath = tmp_path / "export_mxfp8" / "manifest.json"
    mpath.write_text(mpath.read_text().replace("tf_residual_add_rmsnorm", "tf_silu_gate"))
    with pytest.raises(TilefishPreconditionError, match="manifest.json does not match its own digest"):
        NativePlan(str(tmp_path / "export_mxfp8"), trust_directory=True)


def test_symbolic_divisibility_becomes_a_requirement_on_the_graph():
    """A callee's divisible_by on a dimension the caller has not constrained is recorded on the traced graph (and printed), once per
    size, instead of being refused; a static violation stays an error (reference: python/tests/test_calls.py:163-207)."""
    from tilefish_b200 import Requirement

    Kd = Dim("Kd", divisible_by=32)
    Nn = Dim("Nn")

    @tilefish.library("gemm_plain", acc=f32)
    def gemm_plain(a: Tensor[M, Kd, bf16], b: Tensor[Nn, Kd, bf16]) -> Tensor[M, Nn, bf16]: ...

    Kg = Dim("Kg")

    @tilefish.graph
    def g(x: Tensor[M, Kg, bf16], w: Tensor[256, Kg, bf16], v: Tensor[256, Kg, bf16]):
        return gemm_plain(x, w), gemm_plain(x, v)

    assert g.graph.requirements == (Requirement(Kg, 32, "gemm_plain: argument 'a'"),)
    assert "requires Kg % 32 == 0  (required by gemm_plain: argument 'a')" in str(g.graph)
    with pytest.raises(TilefishTypeError, match=r"Kd requires divisible_by=32 but dimension 1 is 100"):
        @tilefish.graph
        def bad(x: Tensor[M, 100, bf16], w: Tensor[256, 100, bf16]):
            return gemm_plain(x, w)


def test_tracer_rules_of_the_elementwise_language():
    """The rules the reference's tracer tests pin (python/tests/test_trace.py), on values made by hand in a fresh trace."""
    from tilefish_b200 import Out, i32
    from tilefish_b200.ir import Scalar
    from tilefish_b200.trace import Const, TraceContext

    ctx = TraceContext("test", "graph")
    n = [0]

    def val(t, name=None, access="in"):
        n[0] += 1
        return ctx.new_value(t, name=name or f"p{n[0]}", access=access, is_param=True)

    m = Dim("m")
    x = val(Tensor[m, D, bf16])
    r = 2 * x + 0.5  # python numbers adopt the tensor's dtype; the operand order of a reflected operator is kept
    assert r.type == Tensor[m, D, bf16] and ctx.nodes[0].inputs == (Scalar(2.0, bf16), x) and ctx.nodes[1].inputs[1] == Scalar(0.5, bf16)
    assert tilefish.silu(x).type == x.type and x.to(bf16) is x  # math functions take any float dtype; a cast to the same dtype is no node
    before = len(ctx.nodes)
    with pytest.raises(TilefishTypeError, match=r"add \(\+\): no implicit promotion"):
        x + val(Tensor[m, D, f32])
    with pytest.raises(TilefishTypeError, match=r"cannot broadcast .* dimension D vs m at axis -1"):
        x * val(Tensor[m, bf16])
    with pytest.raises(TilefishTypeError, match="is a float scalar"):
        val(Tensor[m, i32]) + 0.5
    with pytest.raises(TilefishTypeError, match=r"const 'eps' is const\[f32\] but the other operand has dtype bf16"):
        x + Const("eps", 1e-6, f32)
    with pytest.raises(TilefishTypeError, match="python number or a const parameter"):
        x + True
    for use in (lambda v: v ** 2, lambda v: abs(v), lambda v: v @ v, lambda v: len(v)):
        with pytest.raises(TilefishTypeError, match="not supported in M1"):
            use(x)
    with pytest.raises(TilefishTypeError, match="truth value"):
        bool(x)
    assert len(ctx.nodes) == before  # a refused operation leaves nothing behind
    # reductions follow numpy; no axis means all of them
    y = val(Tensor[m, D, f32])
    assert tilefish.sum(y).type == Tensor[f32] and y.mean(axis=1).type == Tensor[m, f32]
    assert tilefish.max(y, axis=(0, 1), keepdims=True).type == Tensor[1, 1, f32]
    with pytest.raises(TilefishTypeError, match="duplicate axes"):
        tilefish.sum(y, axis=(0, -2))
    # stores: an InOut parameter is read at its stored copy afterwards, an Out parameter is write-only and has no version
    res = val(Tensor[m, D, f32], "res", "inout")
    res[...] = res + 1
    version = res.live
    assert version is not res and ctx.nodes[-1].op == "store" and ctx.nodes[-1].outputs == (version,)
    res * 2
    assert ctx.nodes[-1].inputs[0] is version
    out = val(Tensor[m, D, f32], "y", "out")
    out[...] = y
    assert ctx.nodes[-1].outputs == ()
    with pytest.raises(TilefishTypeError, match="Out parameter 'y', which is write-only"):
        out + 1
    with pytest.raises(TilefishTypeError, match=r"store into 'res': expected Tensor\[m, D, f32\], got Tensor\[m, D, bf16\]"):
        res[...] = x
    with pytest.raises(TilefishTypeError, match="read-only"):
        y[...] = y
    # split: equal chunks or explicit sizes; an axis is always given
    q, k = val(Tensor[m, 100, f32]).split([60, 40], axis=1)
    assert q.type == Tensor[m, 60, f32].as_view() and k.shape[1] == 40
    with pytest.raises(TilefishTypeError, match="add up to 90 but axis 1"):
        val(Tensor[m, 100, f32]).split([60, 30], axis=1)
    with pytest.raises(TilefishTypeError, match="needs a size and an axis"):
        y.split(2)
    with pytest.raises(TilefishTypeError, match="chunk type is invalid.*not divisible by block=32"):
        val(Tensor[m, 128, mxfp8]).split(16, axis=1)
    assert Out is not None


def test_a_call_may_give_a_const_another_value_and_pass_its_own_const_on():
    from tilefish_b200 import i32

    @tilefish.library("scale_by")
    def scale_by(x: Tensor[M, bf16], *, factor: const[f32] = 1.0, steps: const[i32] = 1) -> Tensor[M, bf16]: ...

    @tilefish.graph
    def g(x: Tensor[M, bf16], *, f: const[f32] = 3.0):
        return scale_by(x, factor=2), scale_by(x), scale_by(x, factor=f)

    assert [n.attrs["consts"] for n in g.graph.nodes] == [{"factor": 2.0, "steps": 1}, {"factor": 1.0, "steps": 1}, {"factor": 3.0, "steps": 1}]
    assert isinstance(g.graph.nodes[0].attrs["consts"]["factor"], float)
    with pytest.raises(TilefishTypeError, match="argument 'steps' is const.*needs an int"):

        @tilefish.graph
        def bad(x: Tensor[M, bf16]):
            return scale_by(x, steps=1.5)


def test_an_extern_kernel_is_declared_and_traced_but_not_lowered():
    from tilefish_b200 import Out, Requirement

    n = Dim("n", divisible_by=16)

    @tilefish.extern(triton="my_kernels:gelu", grid=lambda n: (tilefish.cdiv(n, 1024),))
    def gelu(x: Tensor[n, bf16], y: Out[Tensor[n, bf16]], n_elem: n, BLOCK: const = 1024): ...

    @tilefish.graph
    def g(x: Tensor[4096, bf16]):
        return gelu(x)

    (node,) = g.graph.nodes
    assert node.attrs == {"kind": "extern", "triton": "my_kernels:gelu", "consts": {"BLOCK": 1024}}
    assert node.inputs == (g.graph.inputs[0],) and g.graph.outputs[0].type == Tensor[4096, bf16]  # y is a result, n_elem is derived

    s = Dim("s")

    @tilefish.graph
    def sym(x: Tensor[s, bf16]):
        return gelu(x)

    assert sym.graph.requirements == (Requirement(s, 16, "gelu: argument 'x'"),)
    with pytest.raises(TilefishTypeError, match="constexpr 'BLOCK' is fixed to 1024 by the extern declaration"):

        @tilefish.graph
        def changed(x: Tensor[4096, bf16]):
            return gelu(x, BLOCK=512)

    with pytest.raises(TilefishDeclarationError, match="module:function"):
        tilefish.extern(triton="no_colon")
    with pytest.raises(TilefishDeclarationError, match="grid parameter 'q' is not a dimension"):

        @tilefish.extern(triton="m:f", grid=lambda q: (q,))
        def e3(x: Tensor[n, bf16]): ...

    with pytest.raises(TilefishLoweringError, match="extern kernel"):
        tilefish.plan(g)
