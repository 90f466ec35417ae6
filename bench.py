"""Benchmark of the quantized-inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

One step = one forward pass of the tensor-parallel MLP stack of the last benchmark configuration: 32 decoder blocks shaped
like Llama-3-70B's MLP (H = 8192, F = 28672, SiLU-gated), NVFP4 weights quantized from seeded N(0, 1/sqrt(fan_in)) bf16,
M = 4096 tokens of x ~ N(0, 1): residual_add_rmsnorm -> quantize -> gemm (+ SiLU-gate epilogue) -> quantize -> gemm ->
(N > 1: one bf16 NCCL all-reduce) per block. ``value`` is tokens/s with x resident in HBM; ``e2e`` is the same step through the
public API with x in pinned host memory and the result copied back, both copies inside the timed region. The total work is
fixed as N grows (``scaling: strong``). At N = 1 the line also carries the two single-kernel headline metrics: quantize GB/s
(M = 65536, K = 4096, every format) and block-scaled GEMM TFLOP/s (M = 4096, N = 6144, K = 2560, MXFP8 and NVFP4).

``--impl reference`` times the CPU restatement of the same block (oracle/blockscaled.py, torch on all host threads) on a
bounded sample of the workload; the reference project itself cannot run this path (it only types BlockScaled tensors).
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

H, F, LAYERS, M_TOKENS, FMT = 8192, 28672, 32, 4096, "nvfp4"
WORKLOAD = f"tp_mlp_stack: {LAYERS} layers H={H} F={F} {FMT} weights, M={M_TOKENS} (prefill)"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=LAYERS, help="development only: fewer layers (the line then says so)")
    ap.add_argument("--tokens", type=int, default=M_TOKENS, help="development only")
    ap.add_argument("--no-extras", action="store_true", help="skip the single-kernel quantize / GEMM measurements")
    ap.add_argument("--kernel", default=None, choices=["gemm1", "quantize-mxfp8", "quantize-mxfp4", "quantize-nvfp4", "rmsnorm", "decode", "exchange"],
                    help="profiling aid: launch only this kernel three times on a reduced case (what the ncu summaries under profiles/ capture) and exit")
    ap.add_argument("--comm", default=None, choices=["all_reduce", "peer_all_reduce", "fused_exchange", "scatter_gather"],
                    help="tensor-parallel exchange per block (default: fused_exchange = sum + rmsnorm + quantize + gather in one kernel of this library; peer_all_reduce = this library's all-reduce kernel; all_reduce = NCCL; scatter_gather = reduce-scatter + all-gather of the quantized activation, "
                         "fewer bytes but four collectives per block: measured slower on 8 B200s, where the exchange is latency-bound)")
    ap.add_argument("--ar-ctas", type=int, default=None, help="SMs the GEMMs leave free while a row chunk's exchange runs beside them; with peer_all_reduce / fused_exchange also that kernel's CTAs (default: 16; fused_exchange 24 on 2 GPUs, 32 otherwise)")
    ap.add_argument("--peer-path", default="switch_reduce", choices=["multicast_store", "switch_reduce", "peer_loads"],
                    help="data path of peer_all_reduce: the switch's own reduction (default: fewest bytes; its bf16 sum is within one bf16 step of the exact sum, as "
                         "NCCL's NVLS all-reduce), f32 sum over peer loads + multicast store (exact, rounded once), or peer loads only")
    ap.add_argument("--sweep-exchange", action="store_true",
                    help="N > 1, instead of the benchmark: time the step (one CUDA graph) for every exchange mode / row-chunk count / CTA count over the "
                         "same weights, and a bare 64 MiB all-reduce by NCCL and by the peer kernel's three paths; one JSON line (profiles/tp_exchange_modes_*)")
    ap.add_argument("--pdl", type=int, default=None, choices=[0, 1],
                    help="programmatic dependent launch of this library's kernels (tf_set_programmatic_launch); default: the library's default")
    ap.add_argument("--chunks", type=int, default=None, help="row chunks whose all-reduces overlap the other chunk's GEMMs (default: 2 when N > 1)")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ----------------------------------------------------------------------------------------------------------------------
# CPU arm: the oracle's decoder block on a bounded sample
# ----------------------------------------------------------------------------------------------------------------------
_CPU_WEIGHTS: dict = {}


def cpu_block_seconds(rows: int, repeats: int = 1):
    """Seconds for ONE decoder block on ``rows`` tokens with the CPU oracle (weights already dequantized to f32: the values
    do not change the time, so seeded random f32 stands in for them), best of ``repeats``."""
    import torch

    from oracle import blockscaled as O

    g = torch.Generator().manual_seed(0)
    if not _CPU_WEIGHTS:
        _CPU_WEIGHTS["w_gu"] = torch.randn((2 * F, H), generator=g) * H**-0.5
        _CPU_WEIGHTS["w_d"] = torch.randn((H, F), generator=g) * F**-0.5
    w_gu, w_d = _CPU_WEIGHTS["w_gu"], _CPU_WEIGHTS["w_d"]
    w_n = torch.ones(H, dtype=torch.bfloat16)
    x = torch.randn((rows, H), generator=g).to(torch.bfloat16)
    best = float("inf")
    for _ in range(repeats):
        res = torch.zeros((rows, H))
        t0 = time.perf_counter()
        r, h = O.residual_add_rmsnorm(x, res, w_n)
        qh = O.quantize(h, FMT)
        t = O.f32_to_bf16(O.dequantize(qh[0], qh[1], FMT, qh[2]) @ w_gu.t())
        a = O.silu_gate(t[:, :F], t[:, F:])
        qa = O.quantize(a, FMT)
        y = O.f32_to_bf16(O.dequantize(qa[0], qa[1], FMT, qa[2]) @ w_d.t())
        best = min(best, time.perf_counter() - t0)
        del r, h, qh, t, a, qa, y
    return best


def run_reference(args, rank: int) -> None:
    if rank != 0:
        return
    import torch

    rows = 128
    cpu_block_seconds(rows)  # warm-up (also pages the weights in)
    for _ in range(max(0, min(args.warmup, 2) - 1)):
        cpu_block_seconds(rows)
    times = [cpu_block_seconds(rows) for _ in range(min(args.steps, 5))]
    t_block = statistics.median(times)
    t_step = t_block * LAYERS * (M_TOKENS / rows)  # the full step, scaled linearly in rows and layers
    value = M_TOKENS / t_step
    cores = torch.get_num_threads()
    sample = f"{rows} of {M_TOKENS} rows x 1 of {LAYERS} layers per timed run (f32 matmuls of dequantized operands), scaled linearly"
    line = {
        "impl": "reference", "metric": "mlp_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": len(times),
        "warmup": args.warmup, "ms_per_step": t_step * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOAD, "note": "CPU restatement (oracle) of the block; the reference types this path but cannot run it"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index: int) -> None:
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in out.strip().splitlines():
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        # samples under load are the upper half of the clock samples' power... keep it simple: median of all samples
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def event_ms(fn, iters: int, torch, flush=None):
    """Median device time of fn() over ``iters`` launches, CUDA events on the current stream, L2 flushed between launches."""
    ts = []
    for _ in range(iters):
        if flush is not None:
            flush.zero_()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        ts.append(a.elapsed_time(b))
    return statistics.median(ts)


def extras(torch, K, pk):
    """Single-kernel headline metrics at N = 1: quantize GB/s (sweep point M = 65536) and block-scaled GEMM TFLOP/s."""
    out = {"quantize": {}, "gemm": {}}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    m, k = 65536, 4096
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((m, k), generator=g, device="cuda")
    x = torch.where(torch.rand((m, k), generator=g, device="cuda") < 0.01, x * 100, x).to(torch.bfloat16)
    gs = K.nvfp4_global_scale(x)
    for fmt, bpe in (("mxfp8", 2 + 1 + 1 / 32), ("mxfp4", 2 + 0.5 + 1 / 32), ("nvfp4", 2 + 0.5 + 1 / 16)):
        fn = (lambda f=fmt: K.quantize(x, f, global_scale=gs if f == "nvfp4" else None))
        for _ in range(3):
            fn()
        ms = event_ms(fn, 10, torch, flush)
        gbs = m * k * bpe / ms / 1e6
        out["quantize"][fmt] = {"GBps": round(gbs, 1), "us": round(ms * 1e3, 1), "frac_of_hbm_peak": round(gbs / pk["hbm_gbs"], 3), "shape": [m, k]}
    ms = event_ms(lambda: K.nvfp4_global_scale(x, out=gs), 10, torch, flush)
    out["quantize"]["nvfp4_amax_pass"] = {"GBps": round(m * k * 2 / ms / 1e6, 1), "us": round(ms * 1e3, 1)}
    out["quantize"]["sweep"] = {}
    for ms_rows in (1, 128, 8192):  # the smaller points of the sweep: launch-latency bound up to M = 128
        xs = x[:ms_rows]
        row = {}
        for fmt, bpe in (("mxfp8", 2 + 1 + 1 / 32), ("mxfp4", 2 + 0.5 + 1 / 32), ("nvfp4", 2 + 0.5 + 1 / 16)):
            fn = (lambda f=fmt: K.quantize(xs, f, global_scale=gs if f == "nvfp4" else None))
            for _ in range(3):
                fn()
            t = event_ms(fn, 10, torch, flush if ms_rows >= 8192 else None)
            row[fmt] = {"us": round(t * 1e3, 1), "GBps": round(ms_rows * k * bpe / t / 1e6, 1)}
        out["quantize"]["sweep"][f"M={ms_rows}"] = row
    del x
    m, n, k = 4096, 6144, 2560
    a = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn((n, k), generator=g, device="cuda") * k**-0.5).to(torch.bfloat16)
    for fmt, mult in (("mxfp8", 2), ("nvfp4", 4)):
        qa, qb = K.quantize(a, fmt), K.quantize(w, fmt)
        o = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        fn = (lambda: K.gemm_blockscaled(qa, qb, out=o))
        for _ in range(3):
            fn()
        # back-to-back launches so that host launch latency is hidden; operands (tens of MB) stay in L2 by design of the shape
        iters = 20
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        e.synchronize()
        ms = s.elapsed_time(e) / iters
        tf = 2 * m * n * k / ms / 1e9
        ms_q = event_ms(lambda: K.quantize(a, fmt), 5, torch)
        small = {}
        for sm_rows in (1, 16, 128):  # weight-streaming regime: report time and the rate the weights are read at
            qs = K.quantize(a[:sm_rows], fmt)
            os_ = torch.empty((sm_rows, n), dtype=torch.bfloat16, device="cuda")
            need = K.gemm_workspace_bytes(sm_rows, n, k, fmt)
            ws = torch.empty(max(need, 1), dtype=torch.uint8, device="cuda")
            gfn = (lambda: K.gemm_blockscaled(qs, qb, out=os_, workspace=ws))
            for _ in range(3):
                gfn()
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                for _ in range(20):
                    gfn()
            gr.replay()
            s2, e2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s2.record()
            gr.replay()
            e2.record()
            e2.synchronize()
            us = s2.elapsed_time(e2) / 20 * 1e3
            small[f"M={sm_rows}"] = {"us": round(us, 2), "weights_GBps": round(qb.nbytes() / us / 1e3, 1), "TFLOPs": round(2 * sm_rows * n * k / us / 1e6, 2)}
        out["gemm"][fmt + "_small_m"] = small
        out["gemm"][fmt] = {"TFLOPs": round(tf, 1), "us": round(ms * 1e3, 1), "a_quantize_us": round(ms_q * 1e3, 1), "shape": [m, n, k],
                            "frac_of_peak": round(tf / (mult * pk["bf16_tflops"]), 3), "peak": f"{mult} x bf16 burst {pk['bf16_tflops']} ({pk['source']})",
                            "frac_of_nominal": round(tf / (2250.0 * mult), 3)}
    return out


def finish_ranks(world: int) -> None:
    """End of a multi-rank run: destroying the NCCL process group after its collectives were captured into a CUDA graph
    blocks forever (observed on this stack), so the ranks meet at a barrier, flush and leave without tearing NCCL down."""
    if world <= 1:
        return
    import torch
    import torch.distributed as dist

    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def extras_mlp(torch, K, pk):
    """The other two MLP configurations, through the typed API and CUDA-graph replay: the README decoder block (H = 2560,
    F = 3072, MXFP8; exported plan, replayed and captured) at M = 1, 32, 512, 8192, and the decode shape of the stack
    (M = 64, 4 of the 32 layers timed, all 32 reported by scaling)."""
    import tempfile

    import tilefish_b200 as tilefish
    from tilefish_b200 import Dim, InOut, Tensor, bf16, const, f32, mxfp8
    from tilefish_b200 import mlp as MLP
    from tilefish_b200 import runtime

    out = {"readme_block_mxfp8": {}, "decode_stack_nvfp4": {}}
    Mb, Hb, Fb = Dim("M", buckets=[1, 32, 512, 8192]), Dim("H", 2560), Dim("F", 3072)

    @tilefish.kernel
    def residual_add_rmsnorm(x: Tensor[Mb, Hb, bf16], residual: InOut[Tensor[Mb, Hb, f32]], w: Tensor[Hb, bf16], *, eps: const[f32] = 1e-6) -> Tensor[Mb, Hb, bf16]:
        r = residual + x.to(f32)
        residual[...] = r
        rstd = tilefish.rsqrt(tilefish.mean(r * r, axis=-1, keepdims=True) + eps)
        return (r * rstd * w.to(f32)).to(bf16)

    @tilefish.library("gemm_gu", acc=f32)
    def gemm_gu(a: Tensor[Mb, Hb, bf16], b: Tensor[2 * Fb, Hb, mxfp8]) -> Tensor[Mb, 2 * Fb, bf16]: ...

    @tilefish.library("gemm_d", acc=f32)
    def gemm_d(a: Tensor[Mb, Fb, bf16], b: Tensor[Hb, Fb, mxfp8]) -> Tensor[Mb, Hb, bf16]: ...

    @tilefish.graph(inputs=("x",), weights=("w_n", "w_gu", "w_d"))
    def block(x: Tensor[Mb, Hb, bf16], residual: InOut[Tensor[Mb, Hb, f32]], w_n: Tensor[Hb, bf16], w_gu: Tensor[2 * Fb, Hb, mxfp8], w_d: Tensor[Hb, Fb, mxfp8]):
        h = residual_add_rmsnorm(x, residual, w_n)
        g, u = gemm_gu(h, w_gu).split(Fb, axis=-1)
        return gemm_d((tilefish.silu(g.to(f32)) * u.to(f32)).to(bf16), w_d)

    g = torch.Generator(device="cuda").manual_seed(4)
    w_n = (1 + 0.1 * torch.randn(2560, generator=g, device="cuda")).to(torch.bfloat16)
    q_gu = K.quantize((torch.randn((6144, 2560), generator=g, device="cuda") * 2560**-0.5).to(torch.bfloat16), "mxfp8")
    q_d = K.quantize((torch.randn((2560, 3072), generator=g, device="cuda") * 3072**-0.5).to(torch.bfloat16), "mxfp8")
    weight_bytes = q_gu.nbytes() + q_d.nbytes()
    with tempfile.TemporaryDirectory() as d:
        exp = runtime.export(block, d)
        for m in (1, 32, 512, 8192):
            x = torch.randn((m, 2560), generator=g, device="cuda").to(torch.bfloat16)
            res = torch.zeros((m, 2560), device="cuda")
            cap = tilefish.capture(block, x, res, w_n, q_gu, q_d, plan=exp.directory, pin=exp.digest)
            for _ in range(3):
                cap.replay()
            iters = 50 if m <= 512 else 10
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s.record()
            for _ in range(iters):
                cap.replay()
            e.record()
            e.synchronize()
            us = s.elapsed_time(e) / iters * 1e3
            roof = max(6 * 2560 * 3072 * m / (2 * pk["bf16_tflops"] * 1e12), weight_bytes / (pk["hbm_gbs"] * 1e9)) * 1e6
            out["readme_block_mxfp8"][f"M={m}"] = {"tokens_per_s": round(m / us * 1e6, 1), "us_per_step": round(us, 2), "roofline_us": round(roof, 2),
                                                   "frac_of_roofline": round(roof / us, 3)}
        out["readme_block_mxfp8"]["note"] = ("exported plan replayed as one captured CUDA graph (3 launches: rmsnorm+quantize, gemm+SiLU gate+quantize, gemm); "
                                             "roofline = max(6HF*M / (2 x bf16 burst), weight bytes / HBM peak)")
    # decode: M = 64 through the 70B-shaped stack (4 layers timed)
    layers = []
    for layer in range(4):
        gg = torch.Generator(device="cuda").manual_seed(2000 + layer)
        w_gu = (torch.randn((2 * F, H), generator=gg, device="cuda") * H**-0.5).to(torch.bfloat16)
        w_d = (torch.randn((H, F), generator=gg, device="cuda") * F**-0.5).to(torch.bfloat16)
        layers.append(MLP.quantize_weights(torch.ones(H, dtype=torch.bfloat16, device="cuda"), w_gu, w_d, FMT))
        del w_gu, w_d
    stack = MLP.MlpStack(layers)
    x = torch.randn((64, H), generator=g, device="cuda").to(torch.bfloat16)
    res = torch.zeros((64, H), device="cuda")
    cap = stack.capture(x, res)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    ts = []
    for _ in range(10):
        flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        cap.replay()
        e.record()
        e.synchronize()
        ts.append(s.elapsed_time(e))
    ms_layer = statistics.median(ts) / 4
    wbytes = stack.weight_bytes() / 4
    out["decode_stack_nvfp4"] = {"M": 64, "us_per_layer": round(ms_layer * 1e3, 1), "tokens_per_s_32_layers": round(64 / (ms_layer * 32 / 1e3), 1),
                                 "weight_stream_GBps": round(wbytes / ms_layer / 1e6, 1), "frac_of_hbm_peak": round(wbytes / ms_layer / 1e6 / pk["hbm_gbs"], 3),
                                 "note": "4 of 32 layers timed as one captured graph, L2 flushed between replays; HBM-bound (396 MB of weights per layer)"}
    return out


def run_single_kernel(name: str, pdl=None) -> None:
    """Three launches of one kernel on a case of a few hundred MB (larger than L2, small enough for a multi-pass ncu capture)."""
    import torch

    from tilefish_b200 import kernels as K

    K.require_cuda()
    if pdl is not None:
        K.set_programmatic_launch(bool(pdl))
    g = torch.Generator(device="cuda").manual_seed(0)
    if name == "gemm1":  # the dominant kernel at half the benchmark's width: M = 4096, F = 14336, K = 8192, nvfp4, SiLU-gate epilogue
        m, f, k = 4096, F // 2, H
        qa = K.quantize(torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16), FMT)
        qb = K.quantize((torch.randn((2 * f, k), generator=g, device="cuda") * k**-0.5).to(torch.bfloat16), FMT)
        out = torch.empty((m, f), dtype=torch.bfloat16, device="cuda")
        amax = torch.zeros(1, device="cuda")
        fn = lambda: K.gemm_blockscaled(qa, qb, epilogue="silu_gate", out=out, amax_out=amax)  # noqa: E731
    elif name == "decode":  # two blocks of the stack at M = 64 (weights stream once per block): the launch list of the decode path
        from tilefish_b200 import mlp as MLP

        blocks = []
        for layer in range(2):
            w_gu = (torch.randn((2 * F, H), generator=g, device="cuda") * H**-0.5).to(torch.bfloat16)
            w_d = (torch.randn((H, F), generator=g, device="cuda") * F**-0.5).to(torch.bfloat16)
            blocks.append(MLP.quantize_weights(torch.ones(H, dtype=torch.bfloat16, device="cuda"), w_gu, w_d, FMT))
            del w_gu, w_d
        stack = MLP.MlpStack(blocks)
        x = torch.randn((64, H), generator=g, device="cuda").to(torch.bfloat16)
        res = torch.zeros((64, H), device="cuda")
        fn = lambda: stack(x, res)  # noqa: E731
    elif name == "exchange":  # the fused exchange kernel on one GPU (a single rank: nothing to sum; residual add + rmsnorm + amax + nvfp4 quantize)
        from tilefish_b200.collective import PeerAllReduce

        rows = 8192
        part_b, codes_b, scales_b = rows * H * 2, rows * H // 2, K.scale_bytes(FMT, rows, H)
        peer = PeerAllReduce(part_b + codes_b + scales_b + 256, None, torch.device("cuda"), channels=1, num_ctas=148)
        peer.buffer[:part_b].view(torch.bfloat16).copy_(torch.randn(rows * H, generator=g, device="cuda").to(torch.bfloat16))
        res = torch.zeros((rows, H), device="cuda")
        w = torch.ones(H, dtype=torch.bfloat16, device="cuda")
        scratch = torch.empty((rows, H), dtype=torch.bfloat16, device="cuda")
        amax = torch.zeros(1, device="cuda")

        def fn():
            amax.zero_()
            peer.norm_exchange_(partial_offset=0, codes_offset=part_b, scales_offset=part_b + codes_b, gs_offset=part_b + codes_b + scales_b, rows_total=rows,
                                d=H, sum_peers=False, residual_rows=res, w=w, h_scratch=scratch, amax=amax, eps=1e-6, fmt=FMT)
    elif name == "rmsnorm":
        x = torch.randn((8192, H), generator=g, device="cuda").to(torch.bfloat16)
        res = torch.zeros((8192, H), device="cuda")
        w = torch.ones(H, dtype=torch.bfloat16, device="cuda")
        out = torch.empty_like(x)
        fn = lambda: K.residual_add_rmsnorm(x, res, w, out=out)  # noqa: E731
    else:
        fmt = name.split("-")[1]
        x = torch.randn((32768, 4096), generator=g, device="cuda").to(torch.bfloat16)  # 268 MB in
        gs = K.nvfp4_global_scale(x) if fmt == "nvfp4" else None
        fn = lambda: K.quantize(x, fmt, global_scale=gs)  # noqa: E731
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    print(json.dumps({"kernel": name, "launches": 3}))


def exchange_sweep(args, torch, MLP, blocks, group, dev, rank, world, layers, m) -> None:
    """Every exchange variant of the tensor-parallel step over the same weights: per variant the step is captured into one CUDA
    graph and `--steps` replays are timed with CUDA events (max over ranks). Also the bare all-reduce of one [M, H] bf16 tensor."""
    import torch.distributed as dist

    from tilefish_b200.collective import PeerAllReduce

    def timed(fn, n):
        for _ in range(3):
            fn()
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(n):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return round(float(t.item()), 4)

    out = {"sweep": "tp exchange", "n_gpus": world, "layers": layers, "tokens": m, "bare_allreduce_ms": {}, "step_ms": {}}
    n = m * H
    x = torch.randn(n, device=dev).to(torch.bfloat16)
    out["bare_allreduce_ms"]["nccl"] = timed(lambda: dist.all_reduce(x), 20)
    for path in ("switch_reduce", "multicast_store", "peer_loads"):
        for ctas in (16, 32, 64, 128):
            peer = PeerAllReduce(2 * n, group, dev, channels=1, num_ctas=ctas, multicast=path != "peer_loads", reduce_in_switch=path == "switch_reduce")
            v = peer.view(0, (n,))
            v.copy_(x)
            out["bare_allreduce_ms"][f"{peer.mode}/{ctas} CTAs"] = timed(lambda: peer.allreduce_(v), 20)
            if peer.status():
                out["bare_allreduce_ms"][f"{peer.mode}/{ctas} CTAs"] = "bounded wait gave up"
            del peer, v
    del x
    g = torch.Generator().manual_seed(0)
    x_dev = torch.randn((m, H), generator=g).to(torch.bfloat16).to(dev)
    residual = torch.zeros((m, H), dtype=torch.float32, device=dev)
    variants = [("all_reduce", 1, None, 16), ("all_reduce", 2, None, 16)]
    for path in ("switch_reduce", "multicast_store"):
        variants += [("peer_all_reduce", 1, path, 148), ("peer_all_reduce", 1, path, 64), ("peer_all_reduce", 2, path, 16), ("peer_all_reduce", 2, path, 32),
                     ("peer_all_reduce", 2, path, 48)]
        variants += [("fused_exchange", 1, path, 148), ("fused_exchange", 1, path, 64), ("fused_exchange", 2, path, 16), ("fused_exchange", 2, path, 32),
                     ("fused_exchange", 2, path, 48)]
    variants += [("peer_all_reduce", 3, "switch_reduce", 16), ("peer_all_reduce", 4, "switch_reduce", 16), ("peer_all_reduce", 4, "switch_reduce", 8),
                 ("peer_all_reduce", 2, "switch_reduce", 8), ("fused_exchange", 4, "switch_reduce", 32)]
    for comm, chunks, path, ctas in variants:
        stack = MLP.MlpStack(blocks, group=group, chunks=chunks, comm=comm, sm_margin=ctas, peer_path=path or "multicast_store")
        cap = stack.capture(x_dev, residual)

        def step():
            residual.zero_()
            cap.replay()

        key = f"{comm}" + (f"/{path}" if path else "") + f", {chunks} chunk(s), {ctas} CTAs left to the exchange"
        out["step_ms"][key] = timed(step, args.steps)
        if getattr(stack, "_peer", None) is not None and stack._peer.status():
            out["step_ms"][key] = "bounded wait gave up"
        del cap, stack
    if rank == 0:
        print(json.dumps(out), flush=True)


def run_ours(args) -> None:
    import torch

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device (this backend has no CPU path); use --impl reference for the CPU arm")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    group = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)
        group = dist.group.WORLD
    if world != args.gpus:
        raise SystemExit(f"bench.py: --gpus {args.gpus} but WORLD_SIZE={world}")

    from tilefish_b200 import kernels as K
    from tilefish_b200 import mlp as MLP

    K.require_cuda()
    if args.pdl is not None:
        K.set_programmatic_launch(bool(args.pdl))
    pk = peaks()
    layers, m = args.layers, args.tokens

    # ---- weights: seeded per layer, identical on every rank, quantized once and sharded ----
    blocks = []
    for layer in range(layers):
        g = torch.Generator(device=dev).manual_seed(1000 + layer)
        w_gu = (torch.randn((2 * F, H), generator=g, device=dev) * H**-0.5).to(torch.bfloat16)
        w_d = (torch.randn((H, F), generator=g, device=dev) * F**-0.5).to(torch.bfloat16)
        w_n = (1 + 0.1 * torch.randn(H, generator=g, device=dev)).to(torch.bfloat16)
        blocks.append(MLP.quantize_weights(w_n, w_gu, w_d, FMT, rank=rank, world=world))
        del w_gu, w_d
    if args.sweep_exchange:
        if world < 2:
            raise SystemExit("bench.py: --sweep-exchange needs --gpus >= 2")
        exchange_sweep(args, torch, MLP, blocks, group, dev, rank, world, layers, m)
        finish_ranks(world)
        return
    chunks = args.chunks if args.chunks is not None else (2 if world > 1 else 1)
    # default exchange: this library's fused kernel (sum of the partial results + residual add + rmsnorm + quantize + gather in one
    # launch per block and chunk, switch reduction). Measured over the full 32 layers, tokens/s: 8 GPUs 483.9 k (32 CTAs) against
    # 396.9 k with this library's all-reduce kernel and 292 k with NCCL's all-reduce; 2 GPUs 158.2 k (24 CTAs) against 154.9 k and 148.5 k
    comm = args.comm or ("fused_exchange" if world > 1 else "all_reduce")
    if args.ar_ctas is None:
        args.ar_ctas = (24 if world == 2 else 32) if comm == "fused_exchange" else 16
    stack = MLP.MlpStack(blocks, group=group, chunks=chunks, comm=comm, sm_margin=args.ar_ctas, peer_path=args.peer_path)
    torch.cuda.synchronize()

    gx = torch.Generator().manual_seed(0)
    x_all = torch.randn((m, H), generator=gx).to(torch.bfloat16)
    # scatter_gather and fused_exchange keep every token on one rank outside the GEMMs: each rank uploads, normalises and downloads only its own
    # rows, so the job's input and output cross PCIe once in total (m * H * 2 bytes each way over all ranks)
    rows_local = world > 1 and stack.comm in ("scatter_gather", "fused_exchange")
    m_io = m // world if rows_local else m
    x_host = (x_all[rank * m_io:(rank + 1) * m_io] if rows_local else x_all).contiguous().pin_memory()
    out_host = torch.empty((m_io, H), dtype=torch.bfloat16).pin_memory()
    x_dev = x_host.to(dev)
    residual = torch.zeros((m_io, H), dtype=torch.float32, device=dev)

    # per-launch events around the dominant kernel (the first GEMM of every block) inside the timed region
    gemm_events = []
    orig_gemm = K.gemm_blockscaled

    def timed_gemm(a, b, **kw):
        if kw.get("epilogue") != "silu_gate" or not gemm_events_enabled[0]:
            return orig_gemm(a, b, **kw)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        r = orig_gemm(a, b, **kw)
        e.record()
        gemm_events.append((s, e))
        return r

    gemm_events_enabled = [False]
    K.gemm_blockscaled = timed_gemm
    # rmsnorm, 2 x quantize, 2 x gemm per block and row chunk (nvfp4); with peer_all_reduce the exchange is this library's kernel too
    launches_per_step = layers * (6 if (world > 1 and stack.comm == "peer_all_reduce") else 4 if stack.comm == "fused_exchange" else 5) * stack.chunks
    if stack.comm == "fused_exchange":  # per block and chunk: exchange (sum + rmsnorm + quantize + gather), gemm, quantize, gemm; one all-reduce at the end
        launches_per_step += stack.chunks

    def step():
        residual.zero_()
        return stack(x_dev, residual, rows_local=True) if rows_local else stack(x_dev, residual)

    def step_e2e():
        x_dev.copy_(x_host, non_blocking=True)
        residual.zero_()
        y = step_inner()
        out_host.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return out_host

    def step_inner():
        return stack(x_dev, residual, rows_local=True) if rows_local else stack(x_dev, residual)

    def barrier():
        if world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(steps):
            fn()
        e.record()
        barrier()
        ms = s.elapsed_time(e)
        if world > 1:
            import torch.distributed as dist

            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    exchange_note = None
    if world > 1 and args.comm is None and stack.comm in ("peer_all_reduce", "fused_exchange"):
        # the default picked this library's all-reduce: if its symmetric memory cannot be set up on this machine (every rank sees
        # the same refusal), run the NCCL exchange instead and say so in the line
        try:
            step()
        except Exception as e:  # noqa: BLE001
            exchange_note = f"{stack.comm} unavailable ({type(e).__name__}: {str(e)[:120]}); NCCL collectives used"
            stack = MLP.MlpStack(blocks, group=group, chunks=chunks, comm="scatter_gather" if rows_local else "all_reduce", sm_margin=16)
            launches_per_step = layers * 5 * stack.chunks
    for _ in range(max(args.warmup, 3)):
        step()
    use_graph = world > 1
    if use_graph:
        # N > 1: the per-layer kernels are short (tens of microseconds per row chunk at 8 GPUs) and Python cannot enqueue them
        # fast enough, so the whole step (kernels, both chunk streams, the NCCL all-reduces) is one captured CUDA graph.
        # Per-kernel events cannot be recorded inside a replay: the dominant kernel is timed in an instrumented eager pass of
        # the same step right after the timed region.
        torch.cuda.synchronize()
        cap_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(cap_graph):
            y_cap = step()

        def step_fast():
            cap_graph.replay()
            return y_cap

        def step_e2e_fast():
            x_dev.copy_(x_host, non_blocking=True)
            cap_graph.replay()
            out_host.copy_(y_cap, non_blocking=True)
            torch.cuda.current_stream().synchronize()
            return out_host

        for _ in range(3):
            step_fast()
    else:
        step_fast, step_e2e_fast = step, step_e2e
    sampler = ClockSampler(local) if rank == 0 else None
    gemm_events_enabled[0] = not use_graph
    total_ms = timed(step_fast, args.steps)
    gemm_events_enabled[0] = False
    clocks = sampler.stop() if sampler else None
    if use_graph:
        gemm_events_enabled[0] = True
        timed(step, max(2, args.steps // 2))
        gemm_events_enabled[0] = False
    gemm_ms = [s.elapsed_time(e) for s, e in gemm_events]
    for _ in range(2):
        step_e2e_fast()
    e2e_ms = timed(step_e2e_fast, args.steps)
    K.gemm_blockscaled = orig_gemm

    ms_per_step = total_ms / args.steps
    value = m / (ms_per_step / 1e3)
    e2e_value = m / (e2e_ms / args.steps / 1e3)

    # roofline of the dominant kernel: gemm(h, w_gu) with the SiLU-gate epilogue, on this rank's shard
    f_local = F // world
    flops = 2.0 * (m / stack.chunks) * (2 * f_local) * H
    avg_ms = statistics.mean(gemm_ms) if gemm_ms else float("nan")
    achieved = flops / avg_ms / 1e9
    peak = 4 * pk["bf16_tflops_sustained"]
    roofline = {"bound": "tensor", "kernel": "gemm_blockscaled_kernel<nvfp4, 256, silu_gate>", "achieved": round(achieved, 1), "peak": peak,
                "unit": "TFLOP/s", "frac": round(achieved / peak, 4),
                # DRAM read + write of one launch from the ncu capture summarised under profiles/ (242 MB at half width, F = 14336;
                # the traffic is proportional to F): algorithmic bytes of a full-width launch are 518 MB
                "traffic": round(242.3e6 * (2 * f_local) / 28672) if m == M_TOKENS else None, "traffic_unit": "bytes per launch (ncu, scaled from F = 14336)",
                "peak_note": f"4 x sustained bf16 cuBLAS {pk['bf16_tflops_sustained']} TFLOP/s ({pk['source']}); no FP4 peak was measured on this pool. "
                             f"Nominal dense FP4 is 9000: frac_of_nominal = {achieved / 9000.0:.4f}",
                "launches_timed": len(gemm_ms), "avg_launch_ms": round(avg_ms, 4),
                "timing": "CUDA events around each launch " + ("in an instrumented eager pass after the timed region (the timed region replays a CUDA graph)"
                                                               if world > 1 else "inside the timed region")}

    if rank != 0:
        finish_ranks(world)
        return
    line = {
        "metric": "mlp_tokens_per_s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp4 (e2m1 x e4m3 block scales, f32 accumulate, bf16 out)",
        "data": "synthetic", "impl": "ours",
        "config": {"workload": WORKLOAD if (layers, m) == (LAYERS, M_TOKENS) else f"REDUCED {layers} layers M={m} (development run, not the benchmark)",
                   "parallelism": f"tp{world}" + (f", {stack.comm}, {stack.chunks} row chunks on 2 streams (one chunk's exchange under the other's GEMMs)" if world > 1 else ""), "l2": "inputs larger than L2: every step streams all weights (>= 1.5 GB per GPU)"},
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": x_host.numel() * 2 * (world if rows_local else 1),
                "d2h_bytes_per_step": out_host.numel() * 2 * (world if rows_local else 1),
                "io": (f"each rank copies its own {m_io} rows; bytes are the job's total" if rows_local else "every rank copies the full tensors; bytes are per rank"),
                "ms_per_step": round(e2e_ms / args.steps, 4)},
        "gpu_launches": launches_per_step * args.steps,
        "exchange_note": exchange_note,
        "exchange": ({"kernel": "tp_norm_exchange_kernel" if stack.comm == "fused_exchange" else "allreduce_bf16_kernel", "path": stack._peer.mode, "ctas": stack._peer.num_ctas, "error_word": stack._peer.status()}
                     if getattr(stack, "_peer", None) is not None else None),
        "roofline": roofline,
        "clocks": clocks,
    }
    if world == 1:
        if not args.no_extras:
            del stack, blocks
            torch.cuda.empty_cache()
            line["kernels"] = extras(torch, K, pk)
            line["kernels"].update(extras_mlp(torch, K, pk))
        rows = 128
        cpu_block_seconds(rows)
        t_block = cpu_block_seconds(rows, repeats=2)
        cpu_value = M_TOKENS / (t_block * LAYERS * (M_TOKENS / rows))
        line["cpu_baseline"] = {"value": round(cpu_value, 3), "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": f"{rows} of {M_TOKENS} rows x 1 of {LAYERS} layers with the CPU oracle (f32 matmuls of dequantized operands), scaled linearly"}
    print(json.dumps(line), flush=True)
    finish_ranks(world)


def main() -> None:
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.kernel:
        run_single_kernel(args.kernel, args.pdl)
        return
    run_ours(args)


if __name__ == "__main__":
    main()
