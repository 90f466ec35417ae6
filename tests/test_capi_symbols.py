"""The C-ABI library loads and exports every symbol include/tilefish_b200.h declares (no compute calls: runs without a GPU)."""

import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "tilefish_b200.h")).read()
    return sorted(set(re.findall(r"TF_API[^;(]*?\b(tf_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_expected_entry_points():
    names = declared_symbols()
    for must in ("tf_quantize_mxfp8", "tf_quantize_mxfp4", "tf_quantize_nvfp4", "tf_residual_add_rmsnorm", "tf_silu_gate",
                 "tf_gemm_blockscaled", "tf_swizzle_scales", "tf_last_error"):
        assert must in names


def test_library_exports_every_declared_symbol():
    from tilefish_b200 import _native

    if not os.path.exists(_native.LIB_PATH):
        pytest.skip("library not built here (python tilefish_b200/csrc/build.py)")
    lib = _native.load()
    for name in declared_symbols():
        assert hasattr(lib, name), name
        assert name in _native.SIGNATURES, f"{name} has no ctypes signature"
    assert set(_native.SIGNATURES) == set(declared_symbols())
    assert _native.version().startswith("tilefish_b200")


def header_prototypes():
    """{name: (return class, [argument classes])} of every TF_API declaration; classes: "ptr", "i32", "i64", "u64", "f32", "str"."""
    text = open(os.path.join(ROOT, "include", "tilefish_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", " ", text, flags=re.S)

    def cls(ctype: str) -> str:
        t = " ".join(ctype.replace("const", " ").split())
        if t == "void":
            return "void"
        if "*" in t:
            return "str" if t.replace(" ", "") == "char*" else "ptr"
        base = t.split()[0] if t else "void"
        return {"int32_t": "i32", "tf_status": "i32", "int64_t": "i64", "uint64_t": "u64", "float": "f32"}[base]

    out = {}
    for m in re.finditer(r"TF_API\s+([^;(]*?)\b(tf_[a-z0-9_]+)\s*\(([^)]*)\)\s*;", text, flags=re.S):
        ret, name, params = m.group(1).strip(), m.group(2), m.group(3).strip()
        args = []
        if params and params != "void":
            for prm in params.split(","):
                prm = prm.strip()
                ctype = prm.rsplit(None, 1)[0] if "*" not in prm else prm[: prm.rindex("*") + 1]
                args.append(cls(ctype))
        out[name] = (cls(ret), args)
    return out


def _ctypes_class(t) -> str:
    import ctypes

    if t is None:
        return "void"
    if t is ctypes.c_char_p:
        return "str"
    if t is ctypes.c_void_p or (isinstance(t, type) and issubclass(t, ctypes._Pointer)):
        return "ptr"
    return {ctypes.c_int32: "i32", ctypes.c_int64: "i64", ctypes.c_uint64: "u64", ctypes.c_float: "f32"}[t]


def test_ctypes_signatures_match_the_header_prototypes():
    """Arity and C type of every argument of every entry point: include/tilefish_b200.h against tilefish_b200/_native.py."""
    from tilefish_b200 import _native

    protos = header_prototypes()
    assert set(protos) == set(_native.SIGNATURES)
    for name, (ret, args) in protos.items():
        res, argtypes = _native.SIGNATURES[name]
        assert _ctypes_class(res) == ret, name
        assert [_ctypes_class(a) for a in argtypes] == args, (name, args)
    assert len(protos["tf_gemm_blockscaled"][1]) == 21 and len(protos["tf_gemm_blockscaled_static"][1]) == 16


def test_integration_snippet_matches_the_header_prototypes():
    """The ctypes binding INTEGRATION.md shows a maintainer: every ``_lib.tf_*.argtypes`` line has the header's arity and types,
    and every call of an entry point in the snippet passes that many arguments."""
    protos = header_prototypes()
    text = open(os.path.join(ROOT, "INTEGRATION.md")).read()
    code = text[text.index("```python") + 9:text.index("```", text.index("```python") + 9)]
    alias = {"P": "ptr", "I64": "i64", "I32": "i32", "F32": "f32", "U64": "u64"}
    seen = 0
    for m in re.finditer(r"_lib\.(tf_[a-z0-9_]+)\.argtypes = \[([^\]]*)\]", code):
        name, items = m.group(1), [x.strip() for x in m.group(2).split(",") if x.strip()]
        assert [alias[x] for x in items] == protos[name][1], name
        seen += 1
    assert seen >= 5
    for m in re.finditer(r"_lib\.(tf_[a-z0-9_]+)\(", code):
        name = m.group(1)
        depth, i, commas = 1, m.end(), 0
        while depth:
            ch = code[i]
            depth += ch in "(["
            depth -= ch in ")]"
            commas += ch == "," and depth == 1
            i += 1
        passed = 0 if not code[m.end():i - 1].strip() else commas + 1
        assert passed == len(protos[name][1]), f"{name}: the snippet passes {passed} arguments, the header declares {len(protos[name][1])}"


def test_host_only_queries():
    from tilefish_b200 import _native

    if not os.path.exists(_native.LIB_PATH):
        pytest.skip("library not built here")
    assert _native.scale_bytes(_native.FMT_MXFP8, 256, 4096, _native.SCALES_PLAIN) == 256 * 128
    assert _native.scale_bytes(_native.FMT_NVFP4, 1, 64, _native.SCALES_SWIZZLED) == 512
    assert _native.scale_bytes(_native.FMT_MXFP4, 129, 160, _native.SCALES_SWIZZLED) == 2 * 2 * 512
    from tilefish_b200 import TilefishPreconditionError

    with pytest.raises(TilefishPreconditionError):
        _native.scale_bytes(7, 1, 32, 0)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from tilefish_b200 import TilefishRuntimeError, _native

    monkeypatch.setattr(_native, "_lib", None)
    monkeypatch.setattr(_native, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(TilefishRuntimeError, match="no CPU or Triton fallback"):
        _native.load()


def test_allreduce_refuses_bad_arguments_before_any_launch():
    """tf_allreduce_bf16 decides its argument errors on the host: this runs without a GPU."""
    import ctypes

    from tilefish_b200 import _native

    if not os.path.exists(_native.LIB_PATH):
        pytest.skip("library not built here (python tilefish_b200/csrc/build.py)")
    lib = _native.load()
    ptrs = (ctypes.c_uint64 * 2)(0x1000, 0x2000)
    call = lambda *a: lib.tf_allreduce_bf16(*a)  # noqa: E731
    assert call(None, ptrs, 0, 0, 0, 2, 0, 16, 8, None) != 0                 # no buffer table
    assert call(ptrs, ptrs, 0, 0, 0, 1, 0, 16, 8, None) != 0                 # a single rank has nothing to exchange
    assert call(ptrs, ptrs, 0, 0, 2, 2, 0, 16, 8, None) != 0                 # rank outside the group
    assert call(ptrs, ptrs, 0, 0, 0, 2, 0, 24, 8, None) != 0                 # count not a multiple of 8 x world
    assert call(ptrs, ptrs, 0, 0, 0, 2, 8, 16, 8, None) != 0                 # offset not a multiple of 16
    assert call(ptrs, ptrs, 0, 0, 0, 2, 0, 16, 0, None) != 0                 # no CTAs
    assert b"num_ctas" in lib.tf_last_error()
    bad = (ctypes.c_uint64 * 2)(0x1000, 0x2004)
    assert call(bad, ptrs, 0, 0, 0, 2, 0, 16, 8, None) != 0                  # unaligned peer pointer


def test_norm_exchange_refuses_bad_arguments_before_any_launch():
    """tf_tp_norm_exchange decides its argument errors on the host: this runs without a GPU."""
    import ctypes

    from tilefish_b200 import _native

    if not os.path.exists(_native.LIB_PATH):
        pytest.skip("library not built here (python tilefish_b200/csrc/build.py)")
    lib = _native.load()
    ptrs = (ctypes.c_uint64 * 2)(0x1000, 0x2000)
    buf = ctypes.c_void_p(0x4000)

    def call(world=2, rank=0, rows=256, d=1024, fmt=2, ctas=8, part=0, amax=buf, res=buf):
        return lib.tf_tp_norm_exchange(ptrs, ptrs, 0, 0, rank, world, part, 4096, 8192, 12288, rows, d, 1, res, buf, buf, amax, 1e-6, fmt, ctas, None)

    assert call(world=9) != 0                 # more ranks than the kernel's tables hold
    assert call(rank=2) != 0                  # rank outside the group
    assert call(rows=128) != 0                # rows not a multiple of 128 x world
    assert b"128 x world" in lib.tf_last_error()
    assert call(d=1000) != 0                  # row length not a multiple of 128
    assert call(fmt=7) != 0                   # unknown format
    assert call(amax=None) != 0               # nvfp4 needs the amax word
    assert call(ctas=0) != 0                  # no CTAs
    assert call(part=8) != 0                  # offset not a multiple of 16
    assert call(res=None) != 0                # no residual rows
