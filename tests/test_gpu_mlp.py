"""The decoder block (residual_add_rmsnorm -> gemm + SiLU gate -> gemm) on one GPU against the CPU oracle.

The oracle quantizes the activations at the same two points with the same rules and multiplies in f32. Bound:
max|d| <= 2**-6 * max|ref| and a relative Frobenius error <= 1e-2 (re-quantizing ``a`` can flip a code where the two
bf16 GEMM results differ by one ulp, so this is looser than a single GEMM; the reference asserts 4 * 2**-8 * max|ref| for
a whole bf16 transformer block, python/tests/test_gpu_plan.py:333-348).
"""

import pytest
import torch

from oracle import blockscaled as O

pytestmark = pytest.mark.gpu


def make(m, h, f, seed=0):
    x = O.randn((m, h), seed, torch.bfloat16)
    res = O.randn((m, h), seed + 1)
    w_n = (1 + 0.1 * O.randn((h,), seed + 2)).to(torch.bfloat16)
    w_gu = O.randn((2 * f, h), seed + 3, torch.bfloat16, scale=h**-0.5)
    w_d = O.randn((h, f), seed + 4, torch.bfloat16, scale=f**-0.5)
    return x, res, w_n, w_gu, w_d


@pytest.mark.parametrize("fmt", ["mxfp8", "mxfp4", "nvfp4"])
@pytest.mark.parametrize("m,h,f", [(1, 256, 384), (32, 2560, 3072), (200, 512, 768)])
def test_decoder_block_matches_oracle(fmt, m, h, f):
    from tilefish_b200 import _native
    from tilefish_b200 import mlp as MLP

    x, res, w_n, w_gu, w_d = make(m, h, f)
    w = MLP.quantize_weights(w_n.cuda(), w_gu.cuda(), w_d.cuda(), fmt)
    res_gpu = res.cuda()
    y = MLP.decoder_block(x.cuda(), res_gpu, w)
    r_ref, y_ref = O.decoder_block(x, res.clone(), w_n, O.quantize(w_gu, fmt), O.quantize(w_d, fmt), fmt)
    assert torch.equal(res_gpu.cpu(), r_ref)
    g, r = y.cpu().float(), y_ref.float()
    assert float((g - r).abs().max()) <= 2.0**-6 * float(r.abs().max())
    assert float((g - r).norm() / r.norm()) <= 1e-2
    assert _native.device_status() == (0, 0)


def test_stack_carries_the_residual_stream():
    from tilefish_b200 import mlp as MLP

    m, h, f = 64, 256, 384
    layers = []
    ref_w = []
    for i in range(3):
        _, _, w_n, w_gu, w_d = make(m, h, f, seed=10 * i)
        layers.append(MLP.quantize_weights(w_n.cuda(), w_gu.cuda(), w_d.cuda(), "mxfp8"))
        ref_w.append((w_n, O.quantize(w_gu, "mxfp8"), O.quantize(w_d, "mxfp8")))
    x = O.randn((m, h), 99, torch.bfloat16)
    res = torch.zeros((m, h))
    res_gpu = res.cuda()
    y = MLP.MlpStack(layers)(x.cuda(), res_gpu)
    xr, rr = x, res.clone()
    for w_n, qgu, qd in ref_w:
        rr, xr = O.decoder_block(xr, rr, w_n, qgu, qd, "mxfp8")
    g, r = y.cpu().float(), xr.float()
    assert float((g - r).norm() / r.norm()) <= 2e-2
    assert float((res_gpu.cpu() - rr).norm() / rr.norm()) <= 1e-2


def test_sharded_weights_hold_the_bytes_of_the_full_weights():
    """Tensor-parallel shards are cut from the quantized full weights: the sum of the shards' partial products equals the
    single-GPU product up to the bf16 rounding of each partial (n * 2**-8 * max|ref|)."""
    from tilefish_b200 import kernels as K
    from tilefish_b200 import mlp as MLP

    m, h, f, world = 48, 256, 512, 2
    x, res, w_n, w_gu, w_d = make(m, h, f, seed=5)
    for fmt in ("mxfp8", "nvfp4"):
        full = MLP.quantize_weights(w_n.cuda(), w_gu.cuda(), w_d.cuda(), fmt)
        y_full = MLP.decoder_block(x.cuda(), res.cuda(), full)
        parts = []
        for rank in range(world):
            sh = MLP.quantize_weights(w_n.cuda(), w_gu.cuda(), w_d.cuda(), fmt, rank=rank, world=world)
            assert sh.w_gu.shape == (2 * f // world, h) and sh.w_d.shape == (h, f // world)
            fl = f // world
            full_codes = full.w_gu.codes
            assert torch.equal(sh.w_gu.codes[:fl], full_codes[rank * fl:(rank + 1) * fl])
            assert torch.equal(sh.w_gu.codes[fl:], full_codes[f + rank * fl:f + (rank + 1) * fl])
            parts.append(MLP.decoder_block(x.cuda(), res.cuda(), sh).float())
        y_tp = sum(parts)
        # mxfp8: the shards' activations quantize to the same codes (32-blocks never straddle a shard), so only the bf16
        # rounding of each partial product differs. nvfp4: each shard derives the global scale of its slice of ``a`` from
        # its own amax, so block scales and codes differ: the two results are two quantizations of the same product and
        # agree to quantization noise, not to rounding.
        err = float((y_tp - y_full.float()).abs().max())
        top = float(y_full.float().abs().max())
        if fmt == "mxfp8":
            assert err <= world * 2.0**-8 * top * 1.01, (fmt, err)
        else:
            rel = float((y_tp - y_full.float()).norm() / y_full.float().norm())
            assert rel <= 0.08, (fmt, rel)


def test_row_chunks_and_graph_capture_reproduce_the_plain_stack(tmp_path):
    """The multi-GPU machinery on one rank (an NCCL group of size 1): two row chunks on two streams with the all-reduce in
    between, and the same step captured into a CUDA graph. MXFP8 quantization is per 32-element block of a row, so cutting the
    rows into chunks must not change a single byte."""
    import torch.distributed as dist

    from tilefish_b200 import mlp as MLP

    if not dist.is_initialized():
        dist.init_process_group("nccl", init_method=f"file://{tmp_path}/pg", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    try:
        m, h, f = 512, 256, 384
        layers = []
        for i in range(3):
            _, _, w_n, w_gu, w_d = make(m, h, f, seed=20 * i)
            layers.append(MLP.quantize_weights(w_n.cuda(), w_gu.cuda(), w_d.cuda(), "mxfp8"))
        x = O.randn((m, h), 5, torch.bfloat16).cuda()
        res0 = O.randn((m, h), 6).cuda()
        r_plain = res0.clone()
        y_plain = MLP.MlpStack(layers)(x, r_plain)
        stack = MLP.MlpStack(layers, group=dist.group.WORLD, chunks=2)
        r_chunk = res0.clone()
        y_chunk = stack(x, r_chunk)
        torch.cuda.synchronize()
        assert torch.equal(y_chunk, y_plain) and torch.equal(r_chunk, r_plain)
        for chunks in (1, 2):  # the row-sharded exchange (reduce-scatter + all-gather of the quantized rows), full and rank-local I/O
            sg = MLP.MlpStack(layers, group=dist.group.WORLD, chunks=chunks, comm="scatter_gather")
            r_sg = res0.clone()
            y_sg = sg(x, r_sg)
            torch.cuda.synchronize()
            assert torch.equal(y_sg, y_plain) and torch.equal(r_sg, r_plain), chunks
            r_loc = res0.clone()
            y_loc = sg(x, r_loc, rows_local=True)
            torch.cuda.synchronize()
            assert torch.equal(y_loc, y_plain) and torch.equal(r_loc, r_plain), chunks
        xg, rg = x.clone(), res0.clone()
        cap = stack.capture(xg, rg)
        rg.copy_(res0)
        y_graph = cap.replay()
        torch.cuda.synchronize()
        assert torch.equal(y_graph, y_plain) and torch.equal(rg, r_plain)
    finally:
        pass  # the process group is left to the interpreter: destroying it after a graph captured its collectives blocks


@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
@pytest.mark.parametrize("m", [16, 512])
def test_programmatic_launch_gives_the_same_bytes(fmt, m):
    """With programmatic dependent launch every kernel may start while its predecessor drains and waits for it before touching
    memory: the stack's output and residual stream must not change by a bit, eagerly and from a replayed CUDA graph."""
    from tilefish_b200 import _native
    from tilefish_b200 import kernels as K
    from tilefish_b200 import mlp as MLP

    h, f = 1024, 1536
    layers = []
    for i in range(3):
        _, _, w_n, w_gu, w_d = make(m, h, f, seed=7 * i)
        layers.append(MLP.quantize_weights(w_n.cuda(), w_gu.cuda(), w_d.cuda(), fmt))
    x = O.randn((m, h), 3, torch.bfloat16).cuda()
    stack = MLP.MlpStack(layers)
    res0 = torch.zeros((m, h), device="cuda")
    y0 = stack(x, res0).clone()
    K.set_programmatic_launch(True)
    try:
        for _ in range(3):  # repeated: an ordering bug would show as run-to-run differences
            res1 = torch.zeros((m, h), device="cuda")
            y1 = stack(x, res1)
            assert torch.equal(y1, y0) and torch.equal(res1, res0)
        res2 = torch.zeros((m, h), device="cuda")
        cap = stack.capture(x, res2)
        for _ in range(2):
            res2.zero_()
            y2 = cap.replay()
            torch.cuda.synchronize()
            assert torch.equal(y2, y0) and torch.equal(res2, res0)
    finally:
        K.set_programmatic_launch(False)
    assert _native.device_status() == (0, 0)


@pytest.mark.parametrize("fmt", ["mxfp8", "mxfp4", "nvfp4"])
@pytest.mark.parametrize("chunks", [1, 2])
def test_fused_exchange_kernel_reproduces_the_unfused_kernels(fmt, chunks):
    """comm="fused_exchange" replaces all-reduce + residual_add_rmsnorm + quantize by one kernel (tf_tp_norm_exchange). On a
    single-rank group there is nothing to sum, so it must give the bytes of the stack built from the separate kernels with the
    same row chunks (same normalisation arithmetic, same quantizer, per-row-block nvfp4 global scales in the GEMM)."""
    import os

    import torch.distributed as dist

    from tilefish_b200 import mlp as MLP

    if not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29517")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=torch.device("cuda", 0))
    m, h, f = 512, 1024, 1536
    layers = []
    for i in range(3):
        _, _, w_n, w_gu, w_d = make(m, h, f, seed=11 * i)
        layers.append(MLP.quantize_weights(w_n.cuda(), w_gu.cuda(), w_d.cuda(), fmt))
    x = O.randn((m, h), 5, torch.bfloat16).cuda()
    res0 = O.randn((m, h), 6).cuda()
    ref_res = res0.clone()
    ref = MLP.MlpStack(layers, group=dist.group.WORLD, chunks=chunks, comm="all_reduce")(x, ref_res)
    stack = MLP.MlpStack(layers, group=dist.group.WORLD, chunks=chunks, comm="fused_exchange", sm_margin=24)
    for _ in range(2):  # twice: the kernel's call counter and barriers carry over
        res = res0.clone()
        y = stack(x, res)
        torch.cuda.synchronize()
        assert torch.equal(res, ref_res)
        assert torch.equal(y, ref)
    res = res0.clone()
    cap = stack.capture(x, res)
    res.copy_(res0)
    y = cap.replay()
    torch.cuda.synchronize()
    assert torch.equal(y, ref) and torch.equal(res, ref_res)
    assert stack._peer.status() == 0
