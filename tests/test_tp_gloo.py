"""The tensor-parallel split of the MLP, on CPU ranks (gloo, world size 2): the host-side partitioning and the all-reduce.

Each rank cuts its shard from the quantized full weights (gate rows + matching up rows of w_gu, a K-slice of w_d), runs the
block's arithmetic with the CPU oracle, and the ranks all-reduce their bf16 partial results. The sum must equal the
single-rank result up to the rounding of the partials: n * 2**-8 * max|ref| (mxfp8, where a shard's activation blocks are
the full tensor's blocks).
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import blockscaled as O


def shard_rows(f, rank, world):
    fl = f // world
    return torch.cat([torch.arange(rank * fl, (rank + 1) * fl), torch.arange(f + rank * fl, f + (rank + 1) * fl)])


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, h, f, fmt = 16, 128, 256, "mxfp8"
        x = O.randn((m, h), 0, torch.bfloat16)
        res = O.randn((m, h), 1)
        w_n = torch.ones(h, dtype=torch.bfloat16)
        w_gu = O.randn((2 * f, h), 3, torch.bfloat16, scale=h**-0.5)
        w_d = O.randn((h, f), 4, torch.bfloat16, scale=f**-0.5)
        q_gu, q_d = O.quantize(w_gu, fmt), O.quantize(w_d, fmt)
        rows = shard_rows(f, rank, world)
        fl = f // world
        sh_gu = (q_gu[0][rows], q_gu[1][rows], None)
        sh_d = (q_d[0][:, rank * fl:(rank + 1) * fl].contiguous(), q_d[1][:, rank * fl // 32:(rank + 1) * fl // 32].contiguous(), None)
        _, y = O.decoder_block(x, res.clone(), w_n, sh_gu, sh_d, fmt)
        part = y.float()
        dist.all_reduce(part)  # gloo has no bf16 sum everywhere: the partials are already rounded to bf16, the sum is exact in f32
        if rank == 0:
            _, full = O.decoder_block(x, res.clone(), w_n, q_gu, q_d, fmt)
            err = float((part - full.float()).abs().max())
            out.put((err, float(full.float().abs().max())))
    finally:
        dist.destroy_process_group()


def test_two_rank_split_sums_to_the_single_rank_result():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    err, top = out.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert err <= 2 * 2.0**-8 * top * 1.01, (err, top)


def test_shard_rows_pairs_gate_and_up():
    rows = shard_rows(512, 1, 4)
    assert rows.tolist() == list(range(128, 256)) + list(range(512 + 128, 512 + 256))


def _worker_rows(rank, world, port, out):
    """The row-sharded exchange: each rank normalises and quantizes ITS rows, the ranks all-gather the quantized bytes, every
    rank multiplies all rows by its weight shard, and the summed partials come back split by rows."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        m, h, f, fmt = 256, 128, 256, "mxfp8"
        x = O.randn((m, h), 0, torch.bfloat16)
        res = O.randn((m, h), 1)
        w_n = (1 + 0.1 * O.randn((h,), 2)).to(torch.bfloat16)
        w_gu = O.randn((2 * f, h), 3, torch.bfloat16, scale=h**-0.5)
        w_d = O.randn((h, f), 4, torch.bfloat16, scale=f**-0.5)
        q_gu, q_d = O.quantize(w_gu, fmt), O.quantize(w_d, fmt)
        fl, r = f // world, m // world
        rows = shard_rows(f, rank, world)
        sh_gu = (q_gu[0][rows], q_gu[1][rows], None)
        sh_d = (q_d[0][:, rank * fl:(rank + 1) * fl].contiguous(), q_d[1][:, rank * fl // 32:(rank + 1) * fl // 32].contiguous(), None)
        # this rank's rows: residual add + rmsnorm + quantize; swizzled scale bytes, as the kernels exchange them
        r_loc, h_loc = O.residual_add_rmsnorm(x[rank * r:(rank + 1) * r], res[rank * r:(rank + 1) * r], w_n)
        codes, scales, _ = O.quantize(h_loc, fmt)
        sw = O.swizzle_scales(scales)
        all_codes = [torch.empty_like(codes) for _ in range(world)]
        all_sw = [torch.empty_like(sw) for _ in range(world)]
        dist.all_gather(all_codes, codes)
        dist.all_gather(all_sw, sw)
        codes_full = torch.cat(all_codes)
        sw_full = torch.cat(all_sw)  # r is a multiple of 128: the ranks' swizzled buffers concatenate into the full one
        scales_full = O.unswizzle_scales(sw_full, m, h // 32)
        t = O.gemm_blockscaled((codes_full, scales_full, None), sh_gu, fmt)
        a = O.silu_gate(t[:, :fl], t[:, fl:])
        y = O.gemm_bf16_a(a, sh_d, fmt).float()
        dist.all_reduce(y)  # gloo stands in for the reduce-scatter: sum, then keep this rank's rows
        mine = y[rank * r:(rank + 1) * r]
        r_full, y_full = O.decoder_block(x, res.clone(), w_n, q_gu, q_d, fmt)
        err = float((mine - y_full[rank * r:(rank + 1) * r].float()).abs().max())
        ok_res = torch.equal(r_loc, r_full[rank * r:(rank + 1) * r])
        ok_sw = torch.equal(sw_full, O.swizzle_scales(O.quantize(O.residual_add_rmsnorm(x, res, w_n)[1], fmt)[1]))
        out.put((rank, err, float(y_full.float().abs().max()), ok_res, ok_sw))
    finally:
        dist.destroy_process_group()


def test_row_sharded_exchange_equals_the_single_rank_block():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    out = ctx.Queue()
    procs = [ctx.Process(target=_worker_rows, args=(r, 2, port, out)) for r in range(2)]
    for p in procs:
        p.start()
    results = [out.get(timeout=120) for _ in range(2)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, err, top, ok_res, ok_sw in results:
        assert ok_res and ok_sw, rank
        assert err <= 2 * 2.0**-8 * top * 1.01, (rank, err, top)
