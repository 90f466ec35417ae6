"""Worker of tests/test_gpu_peer_allreduce.py: one process per GPU under torch.distributed.run, any world size from 2 to 8.

What is checked, and against what:

* the all-reduce kernel against the f32 sum of the ranks' inputs IN RANK ORDER, rounded to bf16 once (computed here from the
  all-gathered inputs): bit-exact for the two peer-load paths at any world size; the switch's own reduction within one bf16 step;
* the tensor-parallel MLP stack (``peer_all_reduce`` and ``fused_exchange``, every data path, mxfp8 and nvfp4, one and two row
  chunks, eager and from a replayed CUDA graph) against the CPU ORACLE of the same computation (``oracle.blockscaled.tp_mlp_stack``:
  per-rank weight shards, bf16 partial results, f32 sum in rank order rounded once, per-chunk / per-rank-row-block nvfp4 global
  scales). Bounds for the two-block stack, from what two B200s measured (in brackets): the two paths that sum in f32 over peer
  loads: mxfp8 max|d| <= 2**-4 max|ref| [0.035], relative Frobenius error <= 1e-2 [0.0023]; nvfp4 max|d| <= 2**-3 [0.082], relative
  Frobenius <= 2e-2 [0.0073] (about 1 % of the elements differ: a one-ulp difference of a bf16 activation can flip an e2m1 code or move
  a block scale by one e4m3 step). The switch's own reduction returns sums that are one bf16 step off in a fifth of the elements,
  which requantizes everything downstream: nvfp4 relative Frobenius <= 0.12 [0.070], max|d| <= 2**-2 [0.10]. Each run is also
  compared with the UNQUANTIZED f32 stack and the figure is printed: that distance (the quantization error itself) is the same for
  the switch's sums as for the exact ones, which is why the switch path is offered at all; it is not the default;
* variants that must agree bit for bit do (the two peer-load paths; for mxfp8 also row-sharded against replicated normalisation);
* the row-sharded quantizer with the tensor-wide nvfp4 scale against the single-GPU quantization of the whole tensor: the same bytes.

Teardown: every stack releases its symmetric memory (``close()``), captured graphs are dropped first, then the ranks meet at a barrier.
The process still leaves through ``os._exit`` after that: destroying an NCCL process group whose collectives had been captured in a
CUDA graph blocked on this torch / NCCL pair, and the teardown is not re-run here to find out whether it still does.
"""

import gc
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

from oracle import blockscaled as O  # noqa: E402  (the checker; the product path never imports it)
from tilefish_b200 import kernels as K  # noqa: E402
from tilefish_b200 import mlp as MLP  # noqa: E402
from tilefish_b200.collective import PeerAllReduce, quantize_rows_sharded  # noqa: E402

LAYERS = 2
# (format, switch reduction?) -> (max|d| / max|ref|, relative Frobenius error) against the oracle, for the LAYERS-block stack
BOUNDS = {("mxfp8", False): (2.0**-4, 1e-2), ("nvfp4", False): (2.0**-3, 2e-2), ("mxfp8", True): (2.0**-3, 6e-2), ("nvfp4", True): (2.0**-2, 0.12)}


def rank_order_sum(src, world):
    """bf16( ((0 + x0) + x1) + ... ) of the ranks' bf16 tensors, on this rank's GPU."""
    parts = [torch.empty_like(src) for _ in range(world)]
    dist.all_gather(parts, src)
    acc = torch.zeros_like(src, dtype=torch.float32)
    for p in parts:
        acc = acc + p.float()
    return acc.to(torch.bfloat16), acc


def check_allreduce_kernel(rank, world, dev, expect):
    for multicast, in_switch in ((True, True), (True, False), (False, False)):
        n = 8 * world * 4099  # ragged against every loop stride
        peer = PeerAllReduce(2 * n + 4096, dist.group.WORLD, dev, channels=2, num_ctas=8, multicast=multicast, reduce_in_switch=in_switch)
        if multicast and not peer.multicast_ptr and rank == 0:
            print("no multicast support: the multicast cases run on peer loads", flush=True)
        for call in range(4):
            g = torch.Generator(device=dev).manual_seed(17 * call + rank)
            src = torch.randn(n, generator=g, device=dev).to(torch.bfloat16)
            want, want_f32 = rank_order_sum(src, world)
            off = 2048 if call % 2 else 0
            v = peer.view(off, (n,))
            v.copy_(src)
            peer.allreduce_(v, channel=call % 2)
            torch.cuda.synchronize()
            if peer.mode == "switch_reduce":
                # the switch's bf16 sum is within one bf16 step of the exact sum, not always the nearest value
                got = v.float()
                expect(bool(((got - want_f32).abs() <= want_f32.abs() * 2.0**-7 + 1e-30).all()),
                       f"switch reduce call {call}: more than one bf16 step from the f32 sum (max diff {float((got - want_f32).abs().max())})")
            else:
                expect(torch.equal(v, want), f"{peer.mode} call {call}: differs from the rank-order f32 sum")
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
        del graph, v
        peer.close()


def make_layers(h, f, fmt, rank, world, dev, seed):
    """(this rank's quantized shards on the GPU, the oracle's full quantized weights on the CPU) from the same seeded bf16 weights."""
    shards, full = [], []
    for layer in range(LAYERS):
        w_gu = O.randn((2 * f, h), seed + 10 * layer, torch.bfloat16, scale=h**-0.5)
        w_d = O.randn((h, f), seed + 10 * layer + 1, torch.bfloat16, scale=f**-0.5)
        w_n = (1 + 0.1 * O.randn((h,), seed + 10 * layer + 2)).to(torch.bfloat16)
        shards.append(MLP.quantize_weights(w_n.to(dev), w_gu.to(dev), w_d.to(dev), fmt, rank=rank, world=world))
        if rank == 0:
            full.append((w_n, O.quantize(w_gu, fmt), O.quantize(w_d, fmt)))
    return shards, full


def oracle_on_rank0(rank, dev, x, res0, full, fmt, world, norm, spans):
    """The oracle's (residual, y) computed on rank 0's host and broadcast to every rank's GPU."""
    m, h = x.shape
    y = torch.empty((m, h), dtype=torch.bfloat16, device=dev)
    r = torch.empty((m, h), dtype=torch.float32, device=dev)
    if rank == 0:
        r_ref, y_ref = O.tp_mlp_stack(x, res0, full, fmt, world, norm=norm, spans=spans)
        y.copy_(y_ref)
        r.copy_(r_ref)
    dist.broadcast(y, 0)
    dist.broadcast(r, 0)
    return r, y


def check_stacks_against_the_oracle(rank, world, dev, expect, report):
    h, f = 1024, 2048
    m = 256 * world
    for fmt in ("mxfp8", "nvfp4"):
        shards, full = make_layers(h, f, fmt, rank, world, dev, seed=100)
        x = O.randn((m, h), 5, torch.bfloat16)
        res0 = O.randn((m, h), 6)
        results = {}
        truth = torch.empty((m, h), dtype=torch.float32, device=dev)
        if rank == 0:
            truth.copy_(O.mlp_stack_unquantized(x, res0, full, fmt)[1])
        dist.broadcast(truth, 0)
        for chunks in (1, 2):
            rows = m // chunks
            spans = [(i * rows, (i + 1) * rows) for i in range(chunks)]
            oracle = {norm: oracle_on_rank0(rank, dev, x, res0, full, fmt, world, norm, spans) for norm in ("replicated", "row_sharded")}
            for comm, norm in (("peer_all_reduce", "replicated"), ("fused_exchange", "row_sharded")):
                r_ref, y_ref = oracle[norm]
                for path in ("multicast_store", "peer_loads", "switch_reduce"):
                    stack = MLP.MlpStack(shards, group=dist.group.WORLD, chunks=chunks, comm=comm, sm_margin=16, peer_path=path)
                    res = res0.to(dev)
                    y = stack(x.to(dev), res)
                    torch.cuda.synchronize()
                    stack.check()
                    c = O.compare(y.cpu(), y_ref.cpu())
                    cr = O.compare(res.cpu(), r_ref.cpu())
                    report(f"{fmt} {comm} {path} chunks={chunks}: y max_rel {c['max_rel']:.2e} rel_fro {c['rel_fro']:.2e} frac_diff {c['frac_diff']:.3f}; "
                           f"residual rel_fro {cr['rel_fro']:.2e}")
                    ct = O.compare(y.cpu().float(), truth.cpu())
                    report(f"{fmt} {comm} {path} chunks={chunks}: distance from the unquantized f32 stack: rel_fro {ct['rel_fro']:.3e}")
                    max_bound, fro_bound = BOUNDS[(fmt, path == "switch_reduce")]
                    expect(c["max_rel"] <= max_bound and c["rel_fro"] <= fro_bound, f"{fmt} {comm} {path} chunks={chunks}: off the oracle: {c}")
                    expect(cr["rel_fro"] <= fro_bound, f"{fmt} {comm} {path} chunks={chunks}: residual stream off the oracle: {cr}")
                    results[(comm, path, chunks)] = (y.clone(), res.clone())
                    if comm == "fused_exchange" and path != "switch_reduce":
                        # GEMM-2 delivering its partial results into the summing rank's buffer gives the same bytes as the exchange kernel pulling them
                        expect(not stack.delivered, f"{fmt} {path} chunks={chunks}: the default is to pull the partial results")
                        push = MLP.MlpStack(shards, group=dist.group.WORLD, chunks=chunks, comm=comm, sm_margin=16, peer_path=path, deliver_partials=True)
                        res_p = res0.to(dev)
                        y_p = push(x.to(dev), res_p)
                        torch.cuda.synchronize()
                        push.check()
                        expect(push.delivered and len(shards) > 1 and torch.equal(y_p, y) and torch.equal(res_p, res),
                               f"{fmt} {path} chunks={chunks}: delivered and pulled partial results give different bytes")
                        push.close()
                        del push
                    if chunks == 2 and path == "multicast_store":
                        res2 = res0.to(dev)
                        cap = stack.capture(x.to(dev), res2)
                        res2.copy_(res0.to(dev))
                        y2 = cap.replay(check=True).clone()
                        torch.cuda.synchronize()
                        expect(torch.equal(y2, y) and torch.equal(res2, res), f"{fmt} {comm}: captured stack differs from eager")
                        cap.release()
                        del cap
                    if comm == "fused_exchange" and path == "multicast_store":
                        # rows_local: the rank brings and gets back only its rows of every chunk; same bytes as those rows of the full run
                        rr = rows // world
                        mine = torch.cat([torch.arange(ci * rows + rank * rr, ci * rows + (rank + 1) * rr) for ci in range(chunks)])
                        res_l = res0[mine].to(dev)
                        y_l = stack(x[mine].contiguous().to(dev), res_l, rows_local=True)
                        torch.cuda.synchronize()
                        expect(torch.equal(y_l, y[mine.to(dev)]) and torch.equal(res_l, res[mine.to(dev)]), f"fused {fmt} chunks={chunks}: rows_local differs from the full run")
                    stack.close()
                    del stack
            # the two peer-load paths form the same rank-order f32 sum: the same bytes at any world size
            for comm in ("peer_all_reduce", "fused_exchange"):
                a, b = results[(comm, "multicast_store", chunks)], results[(comm, "peer_loads", chunks)]
                expect(torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]), f"{fmt} {comm} chunks={chunks}: multicast_store and peer_loads differ")
            if fmt == "mxfp8":  # no tensor-wide scale: sharding the normalisation by rows changes no byte
                a, b = results[("peer_all_reduce", "peer_loads", chunks)], results[("fused_exchange", "peer_loads", chunks)]
                expect(torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]), f"mxfp8 chunks={chunks}: fused exchange differs from the all-reduce stack")
            if world == 2:  # NCCL's two-rank sum is one f32 add, rounded once: the same bytes as the rank-order sum
                nccl = MLP.MlpStack(shards, group=dist.group.WORLD, chunks=chunks, comm="all_reduce")
                res = res0.to(dev)
                y = nccl(x.to(dev), res)
                torch.cuda.synchronize()
                a = results[("peer_all_reduce", "peer_loads", chunks)]
                expect(torch.equal(y, a[0]) and torch.equal(res, a[1]), f"{fmt} chunks={chunks}: this library's all-reduce stack differs from the NCCL stack")
                nccl.close()
                del nccl
        del shards, results
        gc.collect()


def check_row_sharded_quantize(rank, world, dev, expect):
    """Quantize and rmsnorm shard by rows with no exchange, but for the nvfp4 global scale: with the 4-byte max all-reduce the shard's
    bytes are the single-GPU quantizer's bytes for those rows."""
    m, k = 256 * world, 2048
    x = O.outlier_input(m, k, seed=3)
    rr = m // world
    mine = x[rank * rr:(rank + 1) * rr].to(dev)
    for fmt in ("mxfp8", "mxfp4", "nvfp4"):
        q = quantize_rows_sharded(mine, fmt, dist.group.WORLD, layout="plain")
        codes, scales, gs = O.quantize(x, fmt)
        expect(torch.equal(q.codes.cpu(), codes[rank * rr:(rank + 1) * rr]) and torch.equal(q.plain_scales().cpu(), scales[rank * rr:(rank + 1) * rr]),
               f"row-sharded {fmt} quantize differs from the whole-tensor quantization")
        if gs is not None:
            expect(q.global_scale.cpu().view(torch.int32).item() == gs.view(torch.int32).item(), "row-sharded nvfp4: global scale differs from the whole tensor's")


def main() -> int:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    K.require_cuda()
    failures = []

    def expect(cond, what):
        if not cond:
            failures.append(what)

    def report(text):
        if rank == 0:
            print("PARITY " + text, flush=True)

    check_allreduce_kernel(rank, world, dev, expect)
    check_row_sharded_quantize(rank, world, dev, expect)
    check_stacks_against_the_oracle(rank, world, dev, expect, report)

    if failures:
        print(f"rank {rank} FAILED: " + "; ".join(failures), flush=True)
    else:
        print(f"rank {rank} ok", flush=True)
    t = torch.tensor([len(failures)], device=dev)
    dist.all_reduce(t)
    bad = int(t.item())
    del t
    gc.collect()
    torch.cuda.synchronize()
    dist.barrier()  # nobody leaves while a peer may still touch its memory; every symmetric buffer was released by close()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(1 if bad else 0)


if __name__ == "__main__":
    main()
