"""Benchmark of the quantized-inference hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P bench.py --gpus N ...

One step = one forward pass of the tensor-parallel MLP stack of the last benchmark configuration: 32 decoder blocks shaped
like Llama-3-70B's MLP (H = 8192, F = 28672, SiLU-gated), NVFP4 weights quantized from seeded N(0, 1/sqrt(fan_in)) bf16,
M = 4096 tokens of x ~ N(0, 1): residual_add_rmsnorm -> quantize -> gemm (+ SiLU-gate epilogue) -> quantize -> gemm ->
(N > 1: one exchange of the partial results) per block. ``value`` is tokens/s with x resident in HBM; ``e2e`` is the same step
through the public API with x in pinned host memory and the result copied back, both copies inside the timed region. The total
work is fixed as N grows (``scaling: strong``).

Beside the headline the line carries, at every N: ``parity`` (the first 128 x N rows of the step's real input through two blocks
of the real weights, on the GPUs and with the CPU oracle of the same tensor-parallel computation), ``decode`` (the same stack at
M = 64) and, at N > 1, ``row_sharded_quantize``; at N = 1 also the single-kernel metrics: quantize GB/s (M = 65536, K = 4096,
every format, and the smaller sweep points), block-scaled GEMM TFLOP/s (M = 4096, N = 6144, K = 2560, MXFP8 and NVFP4) against the
FP8 / FP4 peak measured in the same run with the library's block-scaled GEMM (torch._scaled_mm: the denominator only), the README
decoder block through the typed API, and the CPU baseline.

``--impl reference`` times the CPU restatement of the same block (oracle/blockscaled.py, torch on all host threads) on a
bounded sample of the workload; the reference project itself cannot run this path (it only types BlockScaled tensors).
"""

import argparse
import gc
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

H, F, LAYERS, M_TOKENS, M_DECODE, FMT = 8192, 28672, 32, 4096, 64, "nvfp4"
WORKLOAD = f"tp_mlp_stack: {LAYERS} layers H={H} F={F} {FMT} weights, M={M_TOKENS} (prefill)"
BYTES_PER_ELEM = {"mxfp8": 2 + 1 + 1 / 32, "mxfp4": 2 + 0.5 + 1 / 32, "nvfp4": 2 + 0.5 + 1 / 16}


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--layers", type=int, default=LAYERS, help="fewer layers than the benchmark's 32 (the line then says REDUCED)")
    ap.add_argument("--no-extras", action="store_true", help="skip the single-kernel, decode and typed-API measurements")
    ap.add_argument("--no-parity", action="store_true", help="skip the oracle comparison after the timed region")
    ap.add_argument("--kernel", default=None, choices=["gemm1", "gemm-config3", "quantize-mxfp8", "quantize-mxfp4", "quantize-nvfp4", "rmsnorm", "decode", "exchange"],
                    help="profiling aid: launch only this kernel three times on a reduced case and exit")
    ap.add_argument("--comm", default=None, choices=["all_reduce", "peer_all_reduce", "fused_exchange", "scatter_gather"],
                    help="tensor-parallel exchange per block (default: fused_exchange = sum + rmsnorm + quantize + gather in one kernel of this library; "
                         "peer_all_reduce = this library's all-reduce kernel; all_reduce = NCCL; scatter_gather = reduce-scatter + all-gather of the quantized activation)")
    ap.add_argument("--ar-ctas", type=int, default=None,
                    help="SMs the GEMMs leave free while a row chunk's exchange runs beside them; with peer_all_reduce / fused_exchange also that kernel's CTAs")
    ap.add_argument("--peer-path", default="multicast_store", choices=["multicast_store", "switch_reduce", "peer_loads"],
                    help="data path of the exchange kernels: f32 sum over peer loads in rank order, rounded once, written through the switch (default: the bytes "
                         "the oracle computes); the switch's own reduction (fewer bytes, but its bf16 sums are one bf16 step off in a fifth of the elements, "
                         "which moves every quantization downstream); or peer loads only")
    ap.add_argument("--chunks", type=int, default=None, help="row chunks whose exchanges overlap the other chunk's GEMMs (default: 2 when N > 1)")
    ap.add_argument("--deliver-partials", action="store_true",
                    help="fused_exchange: the second GEMM's epilogue delivers each rank's rows of the partial results into that rank's buffer with peer "
                         "stores, instead of the exchange kernel pulling them with bulk copies (the default; same bytes either way)")
    ap.add_argument("--exclusive-gemms", action="store_true",
                    help="fused_exchange: run one row chunk's GEMMs at a time (an event chain) instead of letting the chunks' GEMMs overlap "
                         "(the default; measured 2 %% faster on two GPUs, the same on eight)")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        d = json.load(open(path))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        return os.cpu_count() or 1


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

    cores = host_threads()
    torch.set_num_threads(cores)  # under torch.distributed.run OMP_NUM_THREADS is 1: use the cores this process may run on
    rows = 128
    cpu_block_seconds(rows)  # warm-up (also pages the weights in)
    for _ in range(max(0, min(args.warmup, 2) - 1)):
        cpu_block_seconds(rows)
    times = [cpu_block_seconds(rows) for _ in range(min(args.steps, 5))]
    t_block = statistics.median(times)
    t_step = t_block * LAYERS * (M_TOKENS / rows)  # the full step, scaled linearly in rows and layers
    value = M_TOKENS / t_step
    sample = f"{rows} of {M_TOKENS} rows x 1 of {LAYERS} layers per timed run (f32 matmuls of dequantized operands), scaled linearly"
    line = {
        "impl": "reference", "metric": "mlp_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": args.gpus, "steps": len(times),
        "warmup": args.warmup, "ms_per_step": t_step * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": {"workload": WORKLOAD, "note": "CPU restatement (oracle) of the block; the reference types this path but cannot run it"},
        "cpu_baseline": {"value": value, "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port", "sample": sample},
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
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def graph_us(fns, torch, replays: int = 3, flush=None):
    """Device time per launch, in microseconds: the launches ``fns`` (a list of callables, each enqueuing one kernel or one short chain)
    are captured into ONE CUDA graph, so that no host time sits between them, and the graph is replayed ``replays`` times (the best is
    kept; ``flush`` is zeroed before each replay to empty L2)."""
    for f in fns[:3]:
        f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fns:
            f()
    g.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(replays):
        if flush is not None:
            flush.zero_()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        g.replay()
        e.record()
        e.synchronize()
        best = min(best, s.elapsed_time(e) * 1e3 / len(fns))
    del g
    return best


def scaled_mm_operands(torch, q):
    """A BlockScaledTensor as the operands torch._scaled_mm takes: the codes and the swizzled scale bytes, reinterpreted."""
    if q.fmt == "mxfp8":
        return q.codes.view(torch.float8_e4m3fn), q.scales.view(torch.float8_e8m0fnu)
    return q.codes.view(torch.float4_e2m1fn_x2), q.scales.view(torch.float8_e4m3fn)


def library_gemm_us(torch, qa, qb, launches: int = 10):
    """Microseconds of the vendor library's block-scaled GEMM on the same operands (None when this torch build has no such path)."""
    try:
        a, sa = scaled_mm_operands(torch, qa)
        b, sb = scaled_mm_operands(torch, qb)
        out = torch.empty((qa.shape[0], qb.shape[0]), dtype=torch.bfloat16, device=qa.codes.device)
        return graph_us([lambda: torch._scaled_mm(a, b.t(), sa, sb, out_dtype=torch.bfloat16, out=out)] * launches, torch)
    except Exception:  # noqa: BLE001
        return None


def measured_tensor_peaks(torch, K):
    """The FP8 and FP4 denominators: TFLOP/s of the vendor library's block-scaled GEMM (cuBLASLt through torch._scaled_mm) at 8192^3,
    measured in this run on this GPU. Used as a peak only; no part of the product calls it."""
    out = {}
    g = torch.Generator(device="cuda").manual_seed(7)
    n = 8192
    a = torch.randn((n, n), generator=g, device="cuda").to(torch.bfloat16)
    b = (torch.randn((n, n), generator=g, device="cuda") * n**-0.5).to(torch.bfloat16)
    for fmt in ("mxfp8", "nvfp4"):
        us = library_gemm_us(torch, K.quantize(a, fmt), K.quantize(b, fmt))
        out[fmt] = round(2.0 * n**3 / us / 1e6, 1) if us else None
    return out


def extras(torch, K, pk, tensor_peak):
    """Single-kernel headline metrics at N = 1: quantize GB/s (every sweep point) and block-scaled GEMM TFLOP/s."""
    out = {"quantize": {}, "gemm": {}}
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    m, k = 65536, 4096
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((m, k), generator=g, device="cuda")
    x = torch.where(torch.rand((m, k), generator=g, device="cuda") < 0.01, x * 100, x).to(torch.bfloat16)
    gs = K.nvfp4_global_scale(x)
    for fmt, bpe in BYTES_PER_ELEM.items():
        q = K.quantize(x, fmt, global_scale=gs if fmt == "nvfp4" else None)
        us = graph_us([lambda f=fmt, q=q: K.quantize(x, f, global_scale=gs if f == "nvfp4" else None, out=q)] * 10, torch, flush=flush)
        gbs = m * k * bpe / us / 1e3
        out["quantize"][fmt] = {"GBps": round(gbs, 1), "us": round(us, 1), "frac_of_hbm_peak": round(gbs / pk["hbm_gbs"], 3), "shape": [m, k]}
        del q
    us_amax = graph_us([lambda: K.nvfp4_global_scale(x, out=gs)] * 10, torch, flush=flush)
    out["quantize"]["nvfp4_amax_pass"] = {"GBps": round(m * k * 2 / us_amax / 1e3, 1), "us": round(us_amax, 1), "frac_of_hbm_peak": round(m * k * 2 / us_amax / 1e3 / pk["hbm_gbs"], 3)}
    q = K.quantize(x, "nvfp4")
    us2 = graph_us([lambda: K.quantize(x, "nvfp4", out=q)] * 5, torch, flush=flush)  # global scale computed inside: amax pass + quantize pass
    gbs2 = m * k * (BYTES_PER_ELEM["nvfp4"] + 2) / us2 / 1e3
    out["quantize"]["nvfp4_two_pass"] = {"GBps": round(gbs2, 1), "us": round(us2, 1), "frac_of_hbm_peak": round(gbs2 / pk["hbm_gbs"], 3),
                                         "bytes_per_elem": BYTES_PER_ELEM["nvfp4"] + 2, "note": "amax pass + quantize pass, the tensor read twice"}
    del q
    out["quantize"]["sweep"] = {}
    for rows in (1, 128, 8192):  # launch-latency bound up to M = 128; four rotating inputs so that M = 8192 (64 MB) does not sit in L2
        xs = [x[i * rows:(i + 1) * rows] for i in range(4)]
        row = {}
        for fmt, bpe in BYTES_PER_ELEM.items():
            qs = [K.quantize(t, fmt, global_scale=gs if fmt == "nvfp4" else None) for t in xs]
            fns = [(lambda f=fmt, t=xs[i % 4], q=qs[i % 4]: K.quantize(t, f, global_scale=gs if f == "nvfp4" else None, out=q)) for i in range(20)]
            us = graph_us(fns, torch)
            row[fmt] = {"us": round(us, 2), "GBps": round(rows * k * bpe / us / 1e3, 1)}
        out["quantize"]["sweep"][f"M={rows}"] = row
    out["quantize"]["timing"] = "every figure: launches captured into one CUDA graph (no host time between them), best of 3 replays; L2 flushed before a replay at M = 65536"
    del x, xs
    m, n, k = 4096, 6144, 2560
    a = torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16)
    w = (torch.randn((n, k), generator=g, device="cuda") * k**-0.5).to(torch.bfloat16)
    for fmt in ("mxfp8", "nvfp4"):
        qa, qb = K.quantize(a, fmt), K.quantize(w, fmt)
        o = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
        us = graph_us([lambda: K.gemm_blockscaled(qa, qb, out=o)] * 20, torch)
        tf = 2 * m * n * k / us / 1e6
        us_q = graph_us([lambda: K.quantize(a, fmt, out=qa)] * 20, torch)
        lib_us = library_gemm_us(torch, qa, qb, 20)
        small = {}
        for rows in (1, 16, 128):  # weight-streaming regime: report time and the rate the weights are read at
            qs = K.quantize(a[:rows], fmt)
            os_ = torch.empty((rows, n), dtype=torch.bfloat16, device="cuda")
            ws = torch.empty(max(K.gemm_workspace_bytes(rows, n, k, fmt), 1), dtype=torch.uint8, device="cuda")
            us_s = graph_us([lambda: K.gemm_blockscaled(qs, qb, out=os_, workspace=ws)] * 20, torch)
            small[f"M={rows}"] = {"us": round(us_s, 2), "weights_GBps": round(qb.nbytes() / us_s / 1e3, 1), "TFLOPs": round(2 * rows * n * k / us_s / 1e6, 2)}
        out["gemm"][fmt + "_small_m"] = small
        peak = tensor_peak.get(fmt)
        out["gemm"][fmt] = {"TFLOPs": round(tf, 1), "us": round(us, 2), "a_quantize_us": round(us_q, 2), "shape": [m, n, k],
                            "frac_of_peak": round(tf / peak, 3) if peak else None, "peak": peak,
                            "peak_is": "TFLOP/s of the vendor library's block-scaled GEMM at 8192^3, measured in this run",
                            "library_same_shape_TFLOPs": round(2 * m * n * k / lib_us / 1e6, 1) if lib_us else None,
                            "frac_of_library_same_shape": round(lib_us / us, 3) if lib_us else None,
                            "frac_of_nominal": round(tf / (4500.0 if fmt == "mxfp8" else 9000.0), 3)}
    return out


def cleanup_ranks(world: int, stacks=(), graphs=()) -> None:
    """End of a multi-rank run. Captured graphs are dropped first (they hold the captured exchange kernels and collectives), every stack
    releases its symmetric memory and handles, the ranks meet at a barrier; only then does a rank leave. The process still exits through
    os._exit: destroying an NCCL process group whose collectives had been captured into a CUDA graph blocked on this torch / NCCL pair,
    and that teardown is not attempted again here."""
    import torch

    for g in graphs:
        del g
    for s in stacks:
        if s is not None:
            s.close()
    gc.collect()
    torch.cuda.synchronize()
    if world <= 1:
        return
    import torch.distributed as dist

    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    sys.stderr.flush()
    os._exit(0)


def extras_mlp(torch, K, pk, tensor_peak):
    """The README decoder block (H = 2560, F = 3072, MXFP8) through the typed API: exported plan, replayed as one captured CUDA graph,
    at M = 1, 32, 512, 8192."""
    import tempfile

    import tilefish_b200 as tilefish
    from tilefish_b200 import Dim, InOut, Tensor, bf16, const, f32, mxfp8
    from tilefish_b200 import runtime

    out = {}
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
    fp8_peak = tensor_peak.get("mxfp8") or 2 * pk["bf16_tflops"]
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
            roof = max(6 * 2560 * 3072 * m / (fp8_peak * 1e12), weight_bytes / (pk["hbm_gbs"] * 1e9)) * 1e6
            out[f"M={m}"] = {"tokens_per_s": round(m / us * 1e6, 1), "us_per_step": round(us, 2), "roofline_us": round(roof, 2), "frac_of_roofline": round(roof / us, 3)}
            del cap
        out["note"] = ("exported plan replayed as one captured CUDA graph (3 launches: rmsnorm+quantize, gemm+SiLU gate+quantize, gemm); "
                       "roofline = max(6HF*M / measured FP8 peak, weight bytes / HBM peak)")
        runtime.clear_caches()
    return {"readme_block_mxfp8": out}


def run_single_kernel(name: str) -> None:
    """Three launches of one kernel on a case of a few hundred MB (larger than L2, small enough for a multi-pass profiler capture)."""
    import torch

    from tilefish_b200 import kernels as K

    K.require_cuda()
    g = torch.Generator(device="cuda").manual_seed(0)
    if name == "gemm1":  # the dominant kernel at half the benchmark's width: M = 4096, F = 14336, K = 8192, nvfp4, SiLU-gate epilogue
        m, f, k = 4096, F // 2, H
        qa = K.quantize(torch.randn((m, k), generator=g, device="cuda").to(torch.bfloat16), FMT)
        qb = K.quantize((torch.randn((2 * f, k), generator=g, device="cuda") * k**-0.5).to(torch.bfloat16), FMT)
        out = torch.empty((m, f), dtype=torch.bfloat16, device="cuda")
        amax = torch.zeros(1, device="cuda")
        fn = lambda: K.gemm_blockscaled(qa, qb, epilogue="silu_gate", out=out, amax_out=amax)  # noqa: E731
    elif name == "gemm-config3":  # the third benchmark configuration's GEMM: 4096 x 6144 x 2560, nvfp4
        qa = K.quantize(torch.randn((4096, 2560), generator=g, device="cuda").to(torch.bfloat16), FMT)
        qb = K.quantize((torch.randn((6144, 2560), generator=g, device="cuda") * 2560**-0.5).to(torch.bfloat16), FMT)
        out = torch.empty((4096, 6144), dtype=torch.bfloat16, device="cuda")
        fn = lambda: K.gemm_blockscaled(qa, qb, out=out)  # noqa: E731
    elif name == "decode":  # two blocks of the stack at M = 64 (weights stream once per block): the launch list of the decode path
        from tilefish_b200 import mlp as MLP

        blocks = []
        for layer in range(2):
            w_gu = (torch.randn((2 * F, H), generator=g, device="cuda") * H**-0.5).to(torch.bfloat16)
            w_d = (torch.randn((H, F), generator=g, device="cuda") * F**-0.5).to(torch.bfloat16)
            blocks.append(MLP.quantize_weights(torch.ones(H, dtype=torch.bfloat16, device="cuda"), w_gu, w_d, FMT))
            del w_gu, w_d
        stack = MLP.MlpStack(blocks)
        x = torch.randn((M_DECODE, H), generator=g, device="cuda").to(torch.bfloat16)
        res = torch.zeros((M_DECODE, H), device="cuda")
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


DELIVER_PARTIALS = False  # --deliver-partials sets it
EXCLUSIVE_GEMMS = False  # --exclusive-gemms sets it


def make_stack(MLP, blocks, group, world, comm, chunks, ctas, peer_path):
    return MLP.MlpStack(blocks, group=group, chunks=chunks if world > 1 else 1, comm=comm, sm_margin=ctas, peer_path=peer_path,
                        deliver_partials=DELIVER_PARTIALS, exclusive_gemms=EXCLUSIVE_GEMMS)


def parity_check(torch, K, MLP, blocks, group, world, rank, dev, comm, ctas, peer_path, x_all):
    """The first 128 x N rows of the step's real input through the first two blocks of the real weights: on the GPUs with the exchange the
    benchmark uses (one row chunk), and on rank 0's host with the CPU oracle of the same tensor-parallel computation (per-rank weight
    shards cut from the full quantized weights, bf16 partial results, f32 sum in rank order rounded once, nvfp4 global scales per row
    block as the exchange forms them). Returns the comparison (rank 0) or None."""
    from oracle import blockscaled as O  # the checker only: nothing that is timed or shipped calls it

    layers = min(2, len(blocks))
    rows = 128 * world
    x = x_all[:rows].contiguous()
    res0 = torch.zeros((rows, H), dtype=torch.float32)
    rows_sharded = world > 1 and comm in ("fused_exchange", "scatter_gather")
    stack = make_stack(MLP, blocks[:layers], group, world, comm, 1, ctas, peer_path)
    res = res0.to(dev)
    y = stack(x.to(dev), res)
    torch.cuda.synchronize()
    stack.check()
    y_host, res_host = y.cpu(), res.cpu()
    stack.close()
    del stack, y, res
    out = None
    if rank == 0:
        torch.set_num_threads(host_threads())
        full = []
        for layer in range(layers):
            g = torch.Generator(device=dev).manual_seed(1000 + layer)
            w_gu = (torch.randn((2 * F, H), generator=g, device=dev) * H**-0.5).to(torch.bfloat16)
            w_d = (torch.randn((H, F), generator=g, device=dev) * F**-0.5).to(torch.bfloat16)
            w_n = (1 + 0.1 * torch.randn(H, generator=g, device=dev)).to(torch.bfloat16)
            q = []
            for w in (w_gu, w_d):  # the full weights, quantized by the kernels (bit-exact with the oracle's quantizer: its own tests), plain scales
                t = K.quantize(w, FMT, layout="plain")
                q.append((t.codes.cpu(), t.plain_scales().cpu(), t.global_scale.cpu().reshape(()) if t.global_scale is not None else None))
                del t
            full.append((w_n.cpu(), q[0], q[1]))
            del w_gu, w_d
        t0 = time.perf_counter()
        r_ref, y_ref = O.tp_mlp_stack(x, res0, full, FMT, world, norm="row_sharded" if rows_sharded else "replicated")
        c, cr = O.compare(y_host, y_ref), O.compare(res_host, r_ref)
        # nvfp4, two blocks of the benchmark's shape. Where the GPU's and the host's bf16 activations differ by one ulp (accumulation order over
        # K = 8192 / 28672, the approximate exponential of the SiLU) an e2m1 code can flip or a block scale move by one e4m3 step, so the
        # difference is noise with a heavy tail: its maximum grows with the number of elements compared (measured 0.07-0.16 of max|ref| over
        # 1-4 M elements), its bulk does not. The check therefore rests on the relative Frobenius error (<= 5e-2; measured 0.017-0.021) and on
        # the 99.99th percentile of |d| (<= 2**-3 max|ref|), with the maximum only guarded against a gross error (<= 2**-1). For scale: two runs
        # whose inputs differ by one bf16 ulp are 7e-2 apart, any nvfp4 run is 0.19 from the unquantized arithmetic, and a wrong exchange (a
        # rank's partial result missing) is beyond 0.5. With the switch's own reduction, whose sums are one bf16 step off in a fifth of the
        # elements: 0.12 and 2**-2
        switch = world > 1 and peer_path == "switch_reduce" and comm in ("fused_exchange", "peer_all_reduce")
        fro_bound, tail_bound, max_bound = (0.12, 2.0**-2, 2.0**-1) if switch else (5e-2, 2.0**-3, 2.0**-1)
        dabs = (y_host.float() - y_ref.float()).abs().flatten()
        tail = float(dabs.kthvalue(max(1, int(0.9999 * dabs.numel()))).values) / max(float(y_ref.float().abs().max()), 1e-30)
        out = {"rows": rows, "blocks": layers, "oracle": f"tp_mlp_stack(world={world}, norm={'row_sharded' if rows_sharded else 'replicated'}) on the host",
               "max_rel": round(c["max_rel"], 5), "rel_fro": round(c["rel_fro"], 5), "frac_diff": round(c["frac_diff"], 4), "residual_rel_fro": round(cr["rel_fro"], 6),
               "p9999_rel": round(tail, 5),
               "bound": {"rel_fro": fro_bound, "p9999_rel": tail_bound, "max_rel": max_bound},
               "ok": bool(c["rel_fro"] <= fro_bound and tail <= tail_bound and c["max_rel"] <= max_bound and cr["rel_fro"] <= fro_bound),
               "oracle_seconds": round(time.perf_counter() - t0, 1)}
    return out


def decode_line(torch, K, MLP, blocks, group, world, rank, dev, comm, ctas, peer_path, pk):
    """The same stack at M = 64 (decode): weights stream from HBM once per block, so the roofline is this rank's weight bytes over the HBM peak.
    With N > 1 the 64 rows stay replicated and the partial results (1 MiB per block) go through this library's all-reduce kernel on 8 CTAs: the
    row-sharded exchange of the prefill step needs 128 x N rows per call, which for 64 tokens would be mostly padding. (scatter_gather, the NCCL
    row-sharded mode, pads.)"""
    import torch.distributed as dist

    layers = len(blocks)
    if world > 1 and comm in ("fused_exchange", "peer_all_reduce"):
        comm, ctas = "peer_all_reduce", 8
    fused = world > 1 and comm == "scatter_gather"
    rows = 128 * world if fused else M_DECODE
    stack = make_stack(MLP, blocks, group, world, comm, 1, ctas, peer_path)
    x = torch.zeros((rows, H), dtype=torch.bfloat16, device=dev)
    x[:M_DECODE] = torch.randn((M_DECODE, H), generator=torch.Generator(device=dev).manual_seed(3), device=dev).to(torch.bfloat16)
    res = torch.zeros((rows, H), dtype=torch.float32, device=dev)
    cap = stack.capture(x, res)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    ts = []
    for _ in range(8):
        flush.zero_()
        res.zero_()
        if world > 1:
            dist.barrier()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        cap.replay()
        e.record()
        e.synchronize()
        ts.append(s.elapsed_time(e))
    ms = statistics.median(ts)
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    stack.check()
    wbytes = stack.weight_bytes() / layers
    cap.release()
    stack.close()
    us_layer = ms * 1e3 / layers
    return {"M": M_DECODE, "rows_per_call": rows, "exchange": comm if world > 1 else None, "layers_timed": layers, "us_per_layer": round(us_layer, 1), "tokens_per_s": round(M_DECODE / (ms / 1e3) * (layers / LAYERS), 1),
            "weight_stream_GBps_per_gpu": round(wbytes / us_layer / 1e3, 1), "frac_of_hbm_peak": round(wbytes / us_layer / 1e3 / pk["hbm_gbs"], 3),
            "roofline_us_per_layer": round(wbytes / pk["hbm_gbs"] / 1e3, 1),
            "note": "one captured CUDA graph per step, L2 flushed between replays, median of 8, max over ranks; tokens/s is for 32 layers"}


def row_sharded_quantize_line(torch, K, group, world, rank, dev, pk):
    """Quantize shards by rows with no exchange (nvfp4: one 4-byte max all-reduce for the tensor's global scale): M = 65536 rows over the ranks."""
    import torch.distributed as dist

    from tilefish_b200.collective import quantize_rows_sharded

    m, k = 65536 // world, 4096
    g = torch.Generator(device=dev).manual_seed(rank)
    # rotating inputs larger than L2 in total, so that every call reads its rows from HBM
    n_bufs = max(2, -(-(300 << 20) // (m * k * 2)))
    xs = [torch.randn((m, k), generator=g, device=dev).to(torch.bfloat16) for _ in range(n_bufs)]
    out = {}
    calls = 12
    for fmt, bpe in BYTES_PER_ELEM.items():
        for i in range(3):
            quantize_rows_sharded(xs[i % n_bufs], fmt, group)
        dist.barrier()
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()  # no host time between the calls (the nvfp4 calls carry their 4-byte all-reduce into the graph)
        with torch.cuda.graph(graph):
            for i in range(calls):
                quantize_rows_sharded(xs[i % n_bufs], fmt, group)
        graph.replay()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(3):
            dist.barrier()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            graph.replay()
            e.record()
            e.synchronize()
            best = min(best, s.elapsed_time(e) / calls)
        del graph
        t = torch.tensor([best], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t.item()) * 1e3
        total_bpe = bpe + (2 if fmt == "nvfp4" else 0)
        out[fmt] = {"us": round(us, 1), "aggregate_GBps": round(65536 * k * total_bpe / us / 1e3, 1), "frac_of_n_x_hbm_peak": round(65536 * k * total_bpe / us / 1e3 / (world * pk["hbm_gbs"]), 3)}
    out["note"] = (f"65536 x 4096 rows split over {world} ranks, {calls} calls over {n_bufs} rotating inputs in one CUDA graph (best of 3 replays, max over ranks); "
                   "nvfp4 includes the amax pass and the 4-byte max all-reduce")
    return out


def run_ours(args) -> None:
    import torch

    global DELIVER_PARTIALS, EXCLUSIVE_GEMMS
    DELIVER_PARTIALS = args.deliver_partials
    EXCLUSIVE_GEMMS = args.exclusive_gemms

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
    pk = peaks()
    layers, m = args.layers, M_TOKENS

    # ---- weights: seeded per layer, identical on every rank, quantized once and sharded ----
    blocks = []
    for layer in range(layers):
        g = torch.Generator(device=dev).manual_seed(1000 + layer)
        w_gu = (torch.randn((2 * F, H), generator=g, device=dev) * H**-0.5).to(torch.bfloat16)
        w_d = (torch.randn((H, F), generator=g, device=dev) * F**-0.5).to(torch.bfloat16)
        w_n = (1 + 0.1 * torch.randn(H, generator=g, device=dev)).to(torch.bfloat16)
        blocks.append(MLP.quantize_weights(w_n, w_gu, w_d, FMT, rank=rank, world=world))
        del w_gu, w_d
    chunks = args.chunks if args.chunks is not None else (2 if world > 1 else 1)
    # default exchange: this library's fused kernel (sum of the partial results in rank order + residual add + rmsnorm + quantize + gather in
    # one launch per block and chunk) beside the other chunk's GEMMs: on 16 CTAs at 2 and 4 GPUs, on 32 at 8, where the exchange kernel (256
    # rows per call, each summed over 8 ranks) and not the GEMMs set the pace (measured on B200: 16 / 24 / 32 CTAs -> 10.1 / 9.6 / 9.0 ms per step)
    comm = args.comm or ("fused_exchange" if world > 1 else "all_reduce")
    if args.ar_ctas is None:
        args.ar_ctas = 32 if world >= 8 else 16
    stack = make_stack(MLP, blocks, group, world, comm, chunks, args.ar_ctas, args.peer_path)
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
        y = step()
        out_host.copy_(y, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return out_host

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
        # the default picked this library's exchange kernel: if its symmetric memory cannot be set up on this machine (every rank sees
        # the same refusal), run the NCCL exchange instead and say so in the line
        try:
            step()
        except Exception as e:  # noqa: BLE001
            exchange_note = f"{stack.comm} unavailable ({type(e).__name__}: {str(e)[:120]}); NCCL collectives used"
            comm = "scatter_gather" if rows_local else "all_reduce"
            stack = make_stack(MLP, blocks, group, world, comm, chunks, 16, args.peer_path)
            launches_per_step = layers * 5 * stack.chunks
    for _ in range(max(args.warmup, 3)):
        step()
    use_graph = world > 1
    cap_graph = None
    if use_graph:
        # N > 1: the per-layer kernels are short (tens of microseconds per row chunk at 8 GPUs) and Python cannot enqueue them
        # fast enough, so the whole step (kernels, both chunk streams, the exchanges) is one captured CUDA graph.
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
        def step_queued():
            # The eager pass must not measure the host: at 4 and 8 GPUs the kernels are shorter than Python's enqueue time, and an event
            # recorded on an idle stream starts the clock before the kernel has even been launched. A spin kernel of about 0.1 s holds
            # the streams back while the host enqueues the whole step, so the step then runs from a full queue as in the graph.
            spin = getattr(torch.cuda, "_sleep", None)
            if spin is not None:
                spin(200_000_000)
            return step()

        gemm_events_enabled[0] = True
        timed(step_queued, max(2, args.steps // 2))
        gemm_events_enabled[0] = False
    gemm_ms = [s.elapsed_time(e) for s, e in gemm_events]
    for _ in range(2):
        step_e2e_fast()
    e2e_ms = timed(step_e2e_fast, args.steps)
    K.gemm_blockscaled = orig_gemm
    error_word = stack._peer.status() if getattr(stack, "_peer", None) is not None else None
    exchange = ({"kernel": "tp_norm_exchange_kernel" if stack.comm == "fused_exchange" else "allreduce_bf16_kernel", "path": stack._peer.mode, "ctas": stack._peer.num_ctas,
                 "partials": ("delivered by the second GEMM's epilogue (tf_gemm_blockscaled_scatter)" if getattr(stack, "delivered", False)
                              else "read from the peers by the exchange kernel"),
                 "error_word": error_word} if getattr(stack, "_peer", None) is not None else None)
    stack_comm, stack_chunks = stack.comm, stack.chunks
    # the timed stack's graph and symmetric memory go before the follow-up measurements build their own
    cap_graph = None
    y_cap = None
    stack.close()
    del stack
    gc.collect()

    ms_per_step = total_ms / args.steps
    value = m / (ms_per_step / 1e3)
    e2e_value = m / (e2e_ms / args.steps / 1e3)

    parity = None
    if not args.no_parity:
        parity = parity_check(torch, K, MLP, blocks, group, world, rank, dev, comm, args.ar_ctas, args.peer_path, x_all)
    decode = None
    sharded_q = None
    if not args.no_extras:
        decode = decode_line(torch, K, MLP, blocks[:min(layers, 8)], group, world, rank, dev, comm, args.ar_ctas, args.peer_path, pk)
        if world > 1:
            sharded_q = row_sharded_quantize_line(torch, K, group, world, rank, dev, pk)

    if rank != 0:
        cleanup_ranks(world)
        return
    # N > 1: the per-launch times of the step include the moments when the two row chunks' GEMMs share the SMs. The same kernel on the same
    # operands alone, on the SMs the step leaves it (148 - exchange CTAs), 10 launches in one CUDA graph:
    alone_us = None
    if world > 1 and stack_chunks > 1:
        from tilefish_b200 import _native as N_

        xa = torch.randn((m // stack_chunks, H), generator=torch.Generator(device=dev).manual_seed(11), device=dev).to(torch.bfloat16)
        qa = K.quantize(xa, FMT)
        out_a = torch.empty((m // stack_chunks, F // world), dtype=torch.bfloat16, device=dev)
        am = torch.zeros(1, device=dev)
        N_.check(N_.load().tf_set_sm_margin(args.ar_ctas), "tf_set_sm_margin")
        try:
            alone_us = graph_us([lambda: K.gemm_blockscaled(qa, blocks[0].w_gu, epilogue="silu_gate", out=out_a, amax_out=am)] * 10, torch)
        finally:
            N_.check(N_.load().tf_set_sm_margin(0), "tf_set_sm_margin")
        del xa, qa, out_a
    del blocks
    gc.collect()
    torch.cuda.empty_cache()
    tensor_peak = measured_tensor_peaks(torch, K)

    # roofline of the dominant kernel: gemm(h, w_gu) with the SiLU-gate epilogue, on this rank's shard
    f_local = F // world
    flops = 2.0 * (m / stack_chunks) * (2 * f_local) * H
    avg_ms = statistics.mean(gemm_ms) if gemm_ms else float("nan")
    achieved = flops / avg_ms / 1e9
    peak = tensor_peak.get("nvfp4") or 4 * pk["bf16_tflops_sustained"]
    roofline = {"bound": "tensor", "kernel": "gemm_blockscaled_kernel<nvfp4, 256, silu_gate>", "achieved": round(achieved, 1), "peak": peak,
                "unit": "TFLOP/s", "frac": round(achieved / peak, 4), "traffic": None,
                "peak_note": ("FP4 block-scaled GEMM of the vendor library at 8192^3, measured in this run (burst: that GEMM timed alone)" if tensor_peak.get("nvfp4")
                              else f"4 x sustained bf16 {pk['bf16_tflops_sustained']} TFLOP/s ({pk['source']}): this torch build has no block-scaled library GEMM")
                             + f". Nominal dense FP4 is 9000: frac_of_nominal = {achieved / 9000.0:.4f}; frac of 4 x sustained bf16 = {achieved / (4 * pk['bf16_tflops_sustained']):.4f}",
                "launches_timed": len(gemm_ms), "avg_launch_ms": round(avg_ms, 4),
                **({"alone_on_the_step_s_sms": {"sms": 148 - args.ar_ctas, "us": round(alone_us, 1), "TFLOPs": round(flops / alone_us / 1e6, 1),
                                                "frac": round(flops / alone_us / 1e6 / peak, 4),
                                                "note": "the same kernel and shape alone, 10 launches in one CUDA graph; the in-step figure includes the moments "
                                                        "when both row chunks' GEMMs share the SMs"}} if alone_us else {}),
                "timing": "CUDA events around each launch " + ("in an instrumented eager pass after the timed region (the timed region replays a CUDA graph; the eager "
                                                              "pass is enqueued behind a 0.1 s spin kernel, so that it runs from a full queue)"
                                                               if world > 1 else "inside the timed region")}
    line = {
        "metric": "mlp_tokens_per_s", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": round(ms_per_step, 4), "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "fp4 (e2m1 x e4m3 block scales, f32 accumulate, bf16 out)",
        "data": "synthetic", "impl": "ours",
        "config": {"workload": WORKLOAD if layers == LAYERS else f"REDUCED {layers} layers M={m} (not the benchmark)",
                   "parallelism": f"tp{world}" + (f", {stack_comm}, {stack_chunks} row chunks on 2 streams (one chunk's exchange under the other's GEMMs)" if world > 1 else ""),
                   "l2": "inputs larger than L2: every step streams all weights (>= 1.5 GB per GPU)"},
        "e2e": {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": x_host.numel() * 2 * (world if rows_local else 1),
                "d2h_bytes_per_step": out_host.numel() * 2 * (world if rows_local else 1),
                "io": (f"each rank copies its own {m_io} rows; bytes are the job's total" if rows_local else "every rank copies the full tensors; bytes are per rank"),
                "ms_per_step": round(e2e_ms / args.steps, 4)},
        "gpu_launches": launches_per_step * args.steps,
        "exchange_note": exchange_note,
        "exchange": exchange,
        "parity": parity,
        "roofline": roofline,
        "tensor_peak_measured": tensor_peak,
        "clocks": clocks,
        "decode": decode,
    }
    if sharded_q is not None:
        line["row_sharded_quantize"] = sharded_q
    if world == 1:
        if not args.no_extras:
            line["kernels"] = extras(torch, K, pk, tensor_peak)
            line["kernels"].update(extras_mlp(torch, K, pk, tensor_peak))
        torch.set_num_threads(host_threads())
        rows = 128
        cpu_block_seconds(rows)
        t_block = cpu_block_seconds(rows, repeats=2)
        cpu_value = M_TOKENS / (t_block * LAYERS * (M_TOKENS / rows))
        line["cpu_baseline"] = {"value": round(cpu_value, 3), "unit": "tokens/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": f"{rows} of {M_TOKENS} rows x 1 of {LAYERS} layers with the CPU oracle (f32 matmuls of dequantized operands), scaled linearly"}
    print(json.dumps(line), flush=True)
    cleanup_ranks(world)


def main() -> None:
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if args.kernel:
        run_single_kernel(args.kernel)
        return
    run_ours(args)


if __name__ == "__main__":
    main()
