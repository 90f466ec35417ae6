"""Generates tests/golden/reference_vectors.npz by running the UNMODIFIED reference package on the CPU.

Run once in a container that has the reference checkout (its Python package is pure Python over torch):

    python tests/golden/make_golden.py /path/to/reference

Nothing here is needed at test time: the tests read the .npz only. The vectors pin the parts of the path that the
reference implements (its ``reference`` mode): the e4m3 satfinite cast, ``residual_add_rmsnorm``, the SiLU gate and
the f32-accumulate GEMM. The block-scaled quantizers have no counterpart in the reference, so nothing pins them here.
"""

import hashlib
import os
import sys

import numpy as np
import torch


def sha(t: torch.Tensor) -> str:
    return hashlib.sha256(t.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def bits16(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().copy()


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "python", "src"))
    import tilefish as ref
    from tilefish import Dim, InOut, Tensor, bf16, const, e4m3, f32
    from tilefish._library import reference_gemm

    out = {}

    # ---- e4m3 cast: the reference's own known-answer inputs plus an adversarial sweep --------------------------
    n = Dim("n")

    @ref.kernel
    def to_e4m3(x: Tensor[n, f32]) -> Tensor[n, e4m3]:
        return x.to(e4m3)

    inf, nan = float("inf"), float("nan")
    kat = [447.0, 448.0, 449.0, 465.0, 1000.0, 1e5, -448.0, -500.0, inf, -inf, nan, 1.0, 0.001, 1e-5]
    g = torch.Generator().manual_seed(7)
    sweep = torch.randn(4096, generator=g) * torch.exp2(torch.randint(-12, 11, (4096,), generator=g).float())
    # every midpoint between adjacent positive e4m3 values, and one f32 ulp either side
    codes = torch.arange(0, 0x7F, dtype=torch.uint8).view(torch.float8_e4m3fn).float()
    mids = (codes[:-1] + codes[1:]) / 2
    mids = torch.cat([mids, torch.nextafter(mids, torch.tensor(inf)), torch.nextafter(mids, torch.tensor(-inf))])
    x = torch.cat([torch.tensor(kat), sweep, mids, -mids])
    y = ref.run(to_e4m3, x, mode="reference")
    out["e4m3_in_bits"] = x.view(torch.int32).numpy().copy()
    out["e4m3_out"] = y.view(torch.uint8).numpy().copy()

    # ---- residual_add_rmsnorm (the README kernel), D = 2560 ------------------------------------------------------
    M = Dim("M")
    D = Dim("D", 2560)

    @ref.kernel
    def residual_add_rmsnorm(x: Tensor[M, D, bf16], residual: InOut[Tensor[M, D, f32]], w: Tensor[D, bf16], *,
                             eps: const[f32] = 1e-6) -> Tensor[M, D, bf16]:
        r = residual + x.to(f32)
        residual[...] = r
        rstd = ref.rsqrt(ref.mean(r * r, axis=-1, keepdims=True) + eps)
        return (r * rstd * w.to(f32)).to(bf16)

    def rms_inputs(m: int, seed: int):
        g = torch.Generator().manual_seed(seed)
        x = torch.randn((m, 2560), generator=g).to(torch.bfloat16)
        res = torch.randn((m, 2560), generator=g)
        w = (1 + 0.1 * torch.randn(2560, generator=g)).to(torch.bfloat16)
        return x, res, w

    x, res, w = rms_inputs(16, 0)
    res_in = res.clone()
    y = ref.run(residual_add_rmsnorm, x, res, w, mode="reference")
    out["rms_x"] = bits16(x)
    out["rms_res_in"] = res_in.numpy().copy()
    out["rms_w"] = bits16(w)
    out["rms_res_out"] = res.numpy().copy()
    out["rms_out"] = bits16(y)

    # the full first benchmark configuration (256 x 2560, seed 0): digests only
    x, res, w = rms_inputs(256, 0)
    digest_in = sha(x) + sha(res) + sha(w)
    y = ref.run(residual_add_rmsnorm, x, res, w, mode="reference")
    out["rms256_digests"] = np.array([digest_in, sha(res), sha(y)])

    # ---- SiLU gate over the column halves of a [M, 2F] tensor ---------------------------------------------------
    F = Dim("F", 384)

    @ref.kernel
    def silu_gate(g: Tensor[M, F, bf16], u: Tensor[M, F, bf16]) -> Tensor[M, F, bf16]:
        return (ref.silu(g.to(f32)) * u.to(f32)).to(bf16)

    g2 = torch.Generator().manual_seed(3)
    t = (torch.randn((8, 768), generator=g2) * 3).to(torch.bfloat16)
    a = ref.run(silu_gate, t[:, :384].contiguous(), t[:, 384:].contiguous(), mode="reference")
    out["silu_t"] = bits16(t)
    out["silu_out"] = bits16(a)

    # ---- f32-accumulate GEMM, one rounding ----------------------------------------------------------------------
    g3 = torch.Generator().manual_seed(5)
    ga = torch.randn((24, 256), generator=g3).to(torch.bfloat16)
    gb = (torch.randn((40, 256), generator=g3) / 16).to(torch.bfloat16)
    gy = reference_gemm({"a": ga, "b": gb}, "TN", "bf16")
    out["gemm_a"] = bits16(ga)
    out["gemm_b"] = bits16(gb)
    out["gemm_out"] = bits16(gy)

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference")
    main(sys.argv[1])
