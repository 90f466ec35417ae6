"""Worker of tests/test_gpu_peer_allreduce.py: one process per GPU under torch.distributed.run. Checks the peer all-reduce kernel
against NCCL's all-reduce on the same inputs and the MLP stack's peer_all_reduce mode against its all_reduce mode. Exits with
os._exit so that no process-group teardown can block after collectives were captured in a CUDA graph."""

import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from tilefish_b200 import mlp as MLP  # noqa: E402
from tilefish_b200.collective import PeerAllReduce  # noqa: E402


def main() -> int:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    failures = []

    def expect(cond, what):
        if not cond:
            failures.append(what)

    for multicast, in_switch in ((True, True), (True, False), (False, False)):
        n = 8 * world * 4099  # ragged against every loop stride
        peer = PeerAllReduce(2 * n + 4096, dist.group.WORLD, dev, channels=2, num_ctas=8, multicast=multicast, reduce_in_switch=in_switch)
        if multicast and not peer.multicast_ptr and rank == 0:
            print("no multicast support: the multicast cases run on peer loads", flush=True)
        for call in range(4):
            g = torch.Generator(device=dev).manual_seed(17 * call + rank)
            src = torch.randn(n, generator=g, device=dev).to(torch.bfloat16)
            want = src.float()
            dist.all_reduce(want)  # f32 sum over the ranks, rounded once below: what the kernel computes
            off = 2048 if call % 2 else 0
            v = peer.view(off, (n,))
            v.copy_(src)
            peer.allreduce_(v, channel=call % 2)
            torch.cuda.synchronize()
            if peer.mode == "switch_reduce":
                # the switch's bf16 sum is within one bf16 step of the exact sum, not always the nearest value
                got = v.float()
                expect(bool(((got - want).abs() <= want.abs() * 2.0**-7 + 1e-30).all()),
                       f"switch reduce call {call}: more than one bf16 step from the f32 sum (max diff {float((got - want).abs().max())})")
            else:
                expect(torch.equal(v, want.to(torch.bfloat16)), f"{peer.mode} call {call}: sum differs")
        # replayed from a CUDA graph: the kernel's own call counter keeps the flag values fresh
        v = peer.view(0, (n,))
        src = torch.full((n,), float(rank + 1), device=dev, dtype=torch.bfloat16)
        v.copy_(src)
        peer.allreduce_(v)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            v.copy_(src)
            peer.allreduce_(v)
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        expect(bool((v == world * (world + 1) / 2).all()), f"{peer.mode}: graph replay differs")
        expect(peer.status() == 0, f"{peer.mode}: error word {peer.status()}")

    # the MLP stack: peer_all_reduce against all_reduce (NCCL), same weights and inputs
    h, f, m = 1024, 2048, 512
    for fmt in ("mxfp8", "nvfp4"):
        blocks = []
        for layer in range(2):
            g = torch.Generator(device=dev).manual_seed(100 + layer)
            w_gu = (torch.randn((2 * f, h), generator=g, device=dev) * h**-0.5).to(torch.bfloat16)
            w_d = (torch.randn((h, f), generator=g, device=dev) * f**-0.5).to(torch.bfloat16)
            w_n = (1 + 0.1 * torch.randn(h, generator=g, device=dev)).to(torch.bfloat16)
            blocks.append(MLP.quantize_weights(w_n, w_gu, w_d, fmt, rank=rank, world=world))
        g = torch.Generator(device=dev).manual_seed(5)
        x = torch.randn((m, h), generator=g, device=dev).to(torch.bfloat16)
        outs = {}
        paths = ("multicast_store", "peer_loads", "switch_reduce")
        for comm, chunks, mc in [("all_reduce", 1, None), ("all_reduce", 2, None)] + [("peer_all_reduce", c, pth) for pth in paths for c in (1, 2)]:
            stack = MLP.MlpStack(blocks, group=dist.group.WORLD, chunks=chunks, comm=comm, sm_margin=8, peer_path=mc or "multicast_store")
            res = torch.zeros((m, h), dtype=torch.float32, device=dev)
            outs[(comm, chunks, mc)] = stack(x, res).float()
            if comm == "peer_all_reduce" and chunks == 2:
                res2 = torch.zeros((m, h), dtype=torch.float32, device=dev)
                cap = stack.capture(x.clone(), res2)
                res2.zero_()
                y2 = cap.replay().float()
                torch.cuda.synchronize()
                expect(torch.equal(y2, outs[(comm, chunks, mc)]), f"{fmt}: captured peer stack ({mc}) differs from eager")
                expect(stack._peer.status() == 0, f"{fmt}: error word after the stack")
        for chunks in (1, 2):
            ref = outs[("all_reduce", chunks, None)]
            if world == 2:  # one f32 add, one rounding on both sides
                for pth in ("multicast_store", "peer_loads"):
                    expect(torch.equal(outs[("peer_all_reduce", chunks, pth)], ref), f"{fmt} chunks={chunks}: {pth} differs from NCCL")
            # the switch's sum differs from NCCL's in the last bit: after block 1 that requantizes block 2's input (nvfp4: with
            # another global scale), so the runs agree to quantization noise
            y = outs[("peer_all_reduce", chunks, "switch_reduce")]
            rel = float((y - ref).norm() / ref.norm())
            expect(rel < (0.04 if fmt == "mxfp8" else 0.15), f"{fmt} chunks={chunks} switch_reduce: rel {rel}")
    # the fused exchange kernel (sum + residual add + rmsnorm + quantize + gather in one launch per block and chunk) against the
    # all-reduce stack: mxfp8 has no tensor-wide scale, so sharding the normalisation by rows must not change a byte (peer loads
    # sum in f32 and round once, as NCCL does for two ranks); nvfp4 row blocks get their own global scales: quantization noise
    h, f, m = 1024, 2048, 1024
    for fmt in ("mxfp8", "nvfp4"):
        blocks = []
        for layer in range(3):
            g = torch.Generator(device=dev).manual_seed(200 + layer)
            w_gu = (torch.randn((2 * f, h), generator=g, device=dev) * h**-0.5).to(torch.bfloat16)
            w_d = (torch.randn((h, f), generator=g, device=dev) * f**-0.5).to(torch.bfloat16)
            w_n = (1 + 0.1 * torch.randn(h, generator=g, device=dev)).to(torch.bfloat16)
            blocks.append(MLP.quantize_weights(w_n, w_gu, w_d, fmt, rank=rank, world=world))
        g = torch.Generator(device=dev).manual_seed(9)
        x = torch.randn((m, h), generator=g, device=dev).to(torch.bfloat16)
        for chunks in (1, 2):
            # the reference with the same row sharding: mxfp8 = the all-reduce stack (no tensor-wide scale); nvfp4 = the row-sharded
            # stack over NCCL collectives (every rank's row block has the global scale of its own amax there too)
            res_ref = torch.zeros((m, h), dtype=torch.float32, device=dev)
            ref = MLP.MlpStack(blocks, group=dist.group.WORLD, chunks=chunks, comm="all_reduce" if fmt == "mxfp8" else "scatter_gather")(x, res_ref).float()
            for path in ("multicast_store", "peer_loads", "switch_reduce"):
                stack = MLP.MlpStack(blocks, group=dist.group.WORLD, chunks=chunks, comm="fused_exchange", sm_margin=16, peer_path=path)
                res = torch.zeros((m, h), dtype=torch.float32, device=dev)
                y = stack(x, res).float()
                torch.cuda.synchronize()
                rel = float((y - ref).norm() / ref.norm())
                if path != "switch_reduce" and world == 2:
                    expect(torch.equal(y, ref) and torch.equal(res, res_ref), f"fused {fmt} chunks={chunks} {path}: differs from the all-reduce stack (rel {rel})")
                else:
                    # the switch's sums differ in the last bit, which requantizes everything downstream: quantization noise
                    expect(rel < (0.1 if fmt == "mxfp8" else 0.35), f"fused {fmt} chunks={chunks} {path}: rel {rel}")
                if path == "multicast_store":
                    # rows_local: the rank brings and gets back only its rows of every chunk; same bytes as those rows of the full run
                    rows, rr = m // chunks, m // chunks // world
                    mine = torch.cat([torch.arange(ci * rows + rank * rr, ci * rows + (rank + 1) * rr) for ci in range(chunks)]).to(dev)
                    res_l = torch.zeros((m // world, h), dtype=torch.float32, device=dev)
                    y_l = stack(x[mine].contiguous(), res_l, rows_local=True).float()
                    torch.cuda.synchronize()
                    expect(torch.equal(y_l, y[mine]) and torch.equal(res_l, res[mine]), f"fused {fmt} chunks={chunks}: rows_local differs from the full run")
                if chunks == 2 and path == "multicast_store":
                    res2 = torch.zeros((m, h), dtype=torch.float32, device=dev)
                    cap = stack.capture(x.clone(), res2)
                    res2.zero_()
                    y2 = cap.replay().float()
                    torch.cuda.synchronize()
                    expect(torch.equal(y2, y), f"fused {fmt}: captured stack differs from eager")
                expect(stack._peer.status() == 0, f"fused {fmt} {path}: error word")
    if failures:
        print(f"rank {rank} FAILED: " + "; ".join(failures), flush=True)
    else:
        print(f"rank {rank} ok", flush=True)
    t = torch.tensor([len(failures)], device=dev)
    dist.all_reduce(t)
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(1 if int(t.item()) else 0)


if __name__ == "__main__":
    main()
