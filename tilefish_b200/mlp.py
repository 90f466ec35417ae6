"""The decoder-block path built from the kernels: residual_add_rmsnorm -> gemm(x, w_gu) -> SiLU gate -> gemm(a, w_d).

This is what the README ``mlp`` graph of the reference (README.md:81-85, preceded by ``residual_add_rmsnorm`` :53-63)
executes on this backend, single-GPU or tensor-parallel:

* activations are quantized in the weights' format at both GEMMs (the library ``gemm`` takes a bf16 ``a``);
* the split / SiLU gate / multiply of the graph body runs as the first GEMM's epilogue (gate and up column tiles are
  accumulated side by side in tensor memory), so the [M, 2F] intermediate never reaches HBM;
* mxfp8 / mxfp4: the rmsnorm kernel and the first GEMM's epilogue emit the quantized activations directly (two launches
  less, no bf16 intermediate in HBM); nvfp4: the producing kernels also reduce
  max|out| (an atomic max), from which the quantizer derives the tensor's global scale in stream order: no host sync;
* tensor parallel: ``w_gu`` is split by columns of the output (gate rows and the matching up rows per rank), ``w_d`` by K;
  one bf16 all-reduce (NCCL, through torch.distributed) per layer sums the partial results of the second GEMM.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

from . import kernels as K
from .errors import TilefishPreconditionError


@dataclass
class MlpWeights:
    """One decoder block's weights on one device. ``w_gu``: [2F_local, H] (gate rows then up rows); ``w_d``: [H, F_local]."""

    w_n: "object"  # bf16 [H]
    w_gu: K.BlockScaledTensor
    w_d: K.BlockScaledTensor

    @property
    def fmt(self) -> str:
        return self.w_gu.fmt

    def nbytes(self) -> int:
        return self.w_gu.nbytes() + self.w_d.nbytes() + self.w_n.numel() * 2


def quantize_weights(w_n, w_gu, w_d, fmt: str, *, rank: int = 0, world: int = 1) -> MlpWeights:
    """Quantizes the FULL bf16 weights once, then keeps this rank's shard, so that shards hold exactly the bytes of the
    single-GPU weights (codes, scale bytes and the nvfp4 global scales of the full tensors).

    w_gu bf16 [2F, H], w_d bf16 [H, F] on the device. rank r keeps gate rows [rF/n, (r+1)F/n) and the matching up rows of
    w_gu, and columns [rF/n, (r+1)F/n) of w_d; scales are re-swizzled per shard.
    """
    import torch

    two_f, h = w_gu.shape
    f = two_f // 2
    if tuple(w_d.shape) != (h, f):
        raise TilefishPreconditionError(f"w_d: shape {tuple(w_d.shape)}, expected {(h, f)}", kind="shape", arg="w_d")
    if world == 1:
        return MlpWeights(w_n, K.quantize(w_gu, fmt), K.quantize(w_d, fmt))
    if f % world or (f // world) % 128:
        raise TilefishPreconditionError(f"F={f} cannot be split over {world} ranks in multiples of 128", kind="divisible", arg="w_gu")
    fl = f // world
    blk = K.BLOCK[fmt]
    epb = K.ELEMS_PER_BYTE[fmt]
    q_gu = K.quantize(w_gu, fmt, layout="plain")
    rows = torch.cat([torch.arange(rank * fl, (rank + 1) * fl), torch.arange(f + rank * fl, f + (rank + 1) * fl)]).to(w_gu.device)
    gu = K.BlockScaledTensor(fmt, (2 * fl, h), q_gu.codes[rows].contiguous(), K.swizzle_scales(q_gu.plain_scales()[rows].contiguous()),
                             q_gu.global_scale, "swizzled")
    del q_gu
    q_d = K.quantize(w_d, fmt, layout="plain")
    c0, c1 = rank * fl, (rank + 1) * fl
    d = K.BlockScaledTensor(fmt, (h, fl), q_d.codes[:, c0 // epb:c1 // epb].contiguous(),
                            K.swizzle_scales(q_d.plain_scales()[:, c0 // blk:c1 // blk].contiguous()), q_d.global_scale, "swizzled")
    return MlpWeights(w_n, gu, d)


def decoder_block(x, residual, w: MlpWeights, eps: float = 1e-6, *, group=None, scratch: Optional[dict] = None, out=None, reduce=None, amax=None):
    """One block: ``residual += x`` (f32, in place), returns bf16 [M, H] = mlp(rmsnorm(residual) * w_n).

    ``group``: a torch.distributed process group for the tensor-parallel all-reduce (None = single GPU).
    ``reduce``: instead of ``group``, a callable that sums the second GEMM's partial result over the ranks in place
    (``PeerAllReduce.allreduce_`` with ``out`` a view of its symmetric buffer).
    ``scratch``: a dict reused between calls for the two-float amax buffer (nvfp4).
    ``amax``: instead, two f32 on the device that the caller has zeroed (a stack zeroes one buffer for all its blocks at once).
    """
    import torch

    fmt = w.fmt
    if fmt == "nvfp4":
        if amax is None:
            if scratch is None:
                scratch = {}
            amax = scratch.get("amax")
            if amax is None or amax.device != x.device:
                amax = scratch["amax"] = torch.zeros(2, dtype=torch.float32, device=x.device)
            amax.zero_()
        h = K.residual_add_rmsnorm(x, residual, w.w_n, eps, amax_out=amax[0:1])
        hq = K.quantize(h, fmt, amax=amax[0:1])
        a = K.gemm_blockscaled(hq, w.w_gu, epilogue="silu_gate", amax_out=amax[1:2])
        aq = K.quantize(a, fmt, amax=amax[1:2])
    else:
        _, hq = K.residual_add_rmsnorm(x, residual, w.w_n, eps, quantize_to=fmt, want_bf16=False)
        _, aq = K.gemm_blockscaled(hq, w.w_gu, epilogue="silu_gate", quantize_out=True, want_bf16=False)  # `a` never exists in bf16
    y = K.gemm_blockscaled(aq, w.w_d, out=out)
    if reduce is not None:
        reduce(y)
    elif group is not None:
        import torch.distributed as dist

        dist.all_reduce(y, group=group)
    return y


def decoder_block_row_sharded(x_loc, res_loc, w: MlpWeights, eps: float, group, world: int, scratch: dict):
    """One tensor-parallel block with the normalisation sharded by rows: this rank holds rows ``x_loc`` / ``res_loc`` ([R, H],
    R a multiple of 128) of the block's input. It normalises and quantizes its rows, all-gathers the QUANTIZED activation
    (0.56 bytes per element for nvfp4 instead of 2), runs both GEMMs on all rows against its weight shard and reduce-scatters
    the bf16 partial results, so the next block again starts from its own rows. Compared with an all-reduce per block the
    bytes on NVLink drop to (1 + 0.28) / 2 of the all-reduce's, and the rmsnorm work is divided by the group size. Every rank's
    row block keeps the nvfp4 global scale of its own amax (the GEMM takes one global scale per row block)."""
    import torch
    import torch.distributed as dist

    fmt = w.fmt
    r, h = x_loc.shape
    dev = x_loc.device
    key = (r, h, fmt)
    buf = scratch.get(key)
    if buf is None:
        epb = K.ELEMS_PER_BYTE[fmt]
        sbytes = K.scale_bytes(fmt, r, h)
        buf = scratch[key] = {
            "codes": torch.empty((world * r, h // epb), dtype=torch.uint8, device=dev),
            "scales": torch.empty(world * sbytes, dtype=torch.uint8, device=dev),
            "gs": torch.empty(world, dtype=torch.float32, device=dev) if fmt == "nvfp4" else None,
            "amax": torch.zeros(2, dtype=torch.float32, device=dev),
        }
    if fmt == "nvfp4":
        amax = buf["amax"]
        amax.zero_()
        hl = K.residual_add_rmsnorm(x_loc, res_loc, w.w_n, eps, amax_out=amax[0:1])
        hq = K.quantize(hl, fmt, amax=amax[0:1])
        dist.all_gather_into_tensor(buf["gs"], hq.global_scale, group=group)
    else:
        _, hq = K.residual_add_rmsnorm(x_loc, res_loc, w.w_n, eps, quantize_to=fmt, want_bf16=False)
    dist.all_gather_into_tensor(buf["codes"], hq.codes, group=group)
    dist.all_gather_into_tensor(buf["scales"], hq.scales, group=group)
    hq_all = K.BlockScaledTensor(fmt, (world * r, h), buf["codes"], buf["scales"], buf["gs"], "swizzled", gs_rows=r if fmt == "nvfp4" else 0)
    if fmt == "nvfp4":
        a = K.gemm_blockscaled(hq_all, w.w_gu, epilogue="silu_gate", amax_out=amax[1:2])
        aq = K.quantize(a, fmt, amax=amax[1:2])
    else:
        _, aq = K.gemm_blockscaled(hq_all, w.w_gu, epilogue="silu_gate", quantize_out=True, want_bf16=False)
    y = K.gemm_blockscaled(aq, w.w_d)
    out = torch.empty((r, h), dtype=torch.bfloat16, device=dev)
    dist.reduce_scatter_tensor(out, y, group=group)
    return out


class MlpStack:
    """``layers`` decoder blocks applied in sequence: the output of block l is the ``x`` of block l + 1, the f32 residual
    stream is carried in place.

    ``chunks`` > 1 (tensor parallel only) cuts the rows into that many independent chunks, each on its own CUDA stream: rows
    never interact in this stack, so while one chunk's partial results are in the all-reduce, the other chunk's GEMMs run.
    The GEMMs then leave ``sm_margin`` SMs free for the collective's kernel. Every chunk is its own tensor for the nvfp4
    global scales.
    """

    def __init__(self, layers: List[MlpWeights], eps: float = 1e-6, group=None, chunks: int = 1, sm_margin: int = 16,
                 comm: str = "all_reduce", peer_path: str = "multicast_store", deliver_partials: bool = False,
                 exclusive_gemms: bool = False, fuse_few_rows: bool = True) -> None:
        """``comm``: "all_reduce" (one NCCL bf16 all-reduce per block), "peer_all_reduce" (the same exchange by this package's
        own kernel over symmetric memory, see ``collective.PeerAllReduce``; ``sm_margin`` is also its CTA count) or
        "scatter_gather" (rows of the normalisation sharded over the ranks: reduce-scatter of the partial results +
        all-gather of the quantized activations; see ``decoder_block_row_sharded``) or "fused_exchange" (the same row-sharded
        scheme as ONE kernel of this package per block: sum of the partial results, residual add, rmsnorm, quantization and the
        gather of the quantized rows, ``tf_tp_norm_exchange``; ``sm_margin`` is its CTA count). ``deliver_partials``
        (fused_exchange, exact peer paths): the second GEMM's epilogue stores each rank's rows of the partial result straight into
        that rank's buffer (``tf_gemm_blockscaled_scatter``), so the exchange kernel sums local memory only; otherwise (the
        default: measured faster on two GPUs, where the epilogue's 16-byte peer stores slow the GEMM down), and for shapes that
        GEMM splits along K, the exchange kernel pulls its rows from the peers with bulk copies. Same sums, same bytes.
        ``exclusive_gemms`` (fused_exchange with more than one chunk): the chunks' GEMMs run one chunk at a time (an event chain),
        so that only the exchange kernel ever runs beside a GEMM. Off by default: on B200 it measured 2 % slower on two GPUs (the
        tail of one chunk's GEMM no longer overlaps the head of the other's) and the same on eight.
        ``fuse_few_rows`` (one GPU, at most 128 rows, shapes whose second GEMM is split along K: the decode step): the reduction of
        that GEMM's partial sums, the next block's residual add and rmsnorm and the quantization of its result are one launch
        (``tf_rmsnorm_quantize_rows``) instead of three; same bytes."""
        self.layers = layers
        self.exclusive_gemms = bool(exclusive_gemms)
        self.fuse_few_rows = bool(fuse_few_rows)
        self.deliver_partials = bool(deliver_partials)
        self.delivered = False
        self.eps = eps
        self.group = group
        self.chunks = chunks if group is not None else 1
        self.sm_margin = sm_margin
        self.comm = comm if group is not None else "all_reduce"
        if self.comm not in ("all_reduce", "peer_all_reduce", "fused_exchange", "scatter_gather"):
            raise TilefishPreconditionError(f"unknown comm mode {comm!r}", kind="argument", arg="comm")
        self._peer = None
        # how the peer all-reduce moves data: "multicast_store" (sum over peer loads, result written through the switch),
        # "switch_reduce" (the switch also sums: fewer bytes, last bit not always nearest) or "peer_loads" (no multicast at all)
        if peer_path not in ("multicast_store", "switch_reduce", "peer_loads"):
            raise TilefishPreconditionError(f"unknown peer_path {peer_path!r}", kind="argument", arg="peer_path")
        self._peer_path = peer_path
        self._last_reduce = None
        self._scratch: List[dict] = [{} for _ in range(max(1, self.chunks))]
        self._streams = None

    def _amax_slots(self, ci: int, device):
        """Two zeroed f32 per block for chunk ``ci`` (nvfp4 global scales): one buffer, one memset per forward."""
        import torch

        if not self.layers or self.layers[0].fmt != "nvfp4":
            return [None] * len(self.layers)
        buf = self._scratch[ci].get("amax_all")
        if buf is None or buf.device != device or buf.numel() != 2 * len(self.layers):
            buf = self._scratch[ci]["amax_all"] = torch.zeros(2 * len(self.layers), dtype=torch.float32, device=device)
        buf.zero_()
        return [buf[2 * i:2 * i + 2] for i in range(len(self.layers))]

    def forward(self, x, residual, rows_local: bool = False):
        """``rows_local`` (scatter_gather and fused_exchange): ``x`` and ``residual`` are THIS RANK'S rows ([M / n, H]) and so is the result: no
        rank ever holds the other ranks' tokens outside the GEMMs, and the job's input and output cross PCIe once in total."""
        if self._peer is not None:
            # a bounded wait of an earlier forward gave up: everything since then is partial sums. Seen without a synchronization
            # (the copy armed at the end of the previous forward); check() is the synchronizing form
            self._peer.raise_if_failed(f"MlpStack comm={self.comm}")
        if self.comm == "scatter_gather":
            return self._forward_row_sharded(x, residual, rows_local)
        if self.comm == "fused_exchange":
            out = self._forward_fused(x, residual, rows_local)
            self._peer.arm_poll()
            return out
        if rows_local:
            raise TilefishPreconditionError("rows_local needs comm='scatter_gather' or 'fused_exchange'", kind="argument", arg="rows_local")
        if self.comm == "peer_all_reduce" and self._peer_for(x) is not None:
            out = self._forward_peer(x, residual)
            self._peer.arm_poll()
            return out
        if self.chunks <= 1:
            if self.group is None and self._few_rows_applies(x):
                return self._forward_few_rows(x, residual)
            slots = self._amax_slots(0, x.device)
            for w, am in zip(self.layers, slots):
                x = decoder_block(x, residual, w, self.eps, group=self.group, scratch=self._scratch[0], amax=am)
            return x
        return self._forward_chunked(x, residual)

    def _few_rows_applies(self, x) -> bool:
        if not (self.fuse_few_rows and self.layers and x.dim() == 2 and 0 < x.shape[0] <= 128 and x.shape[1] % 32 == 0):
            return False
        w0 = self.layers[0]
        m, h = x.shape
        f = w0.w_d.shape[1]
        same = all(w.fmt == w0.fmt and w.w_d.shape == w0.w_d.shape and w.w_gu.shape == w0.w_gu.shape for w in self.layers)
        return same and w0.w_d.shape[0] == h and K.gemm_splits(m, h, f, w0.fmt) > 1

    def _forward_few_rows(self, x, residual):
        """The decode step on one GPU. Per block: rmsnorm_quantize_rows (fed by the bf16 input, or by the split-K partial sums of the
        previous block's second GEMM) -> gemm + SiLU gate -> (quantize) -> gemm that leaves its partial sums; the last block's
        second GEMM finishes its own sum. Three launches fewer per block than decoder_block, the same bytes."""
        import torch

        m, h = x.shape
        w0 = self.layers[0]
        fmt, f = w0.fmt, w0.w_d.shape[1]
        key = ("few_rows", m, h, f, fmt, str(x.device))
        st = self._scratch[0].get(key)
        if st is None:
            nv = fmt == "nvfp4"
            st = self._scratch[0][key] = {
                # the scale buffer is zeroed once: the kernel never writes its padding
                "hq": K.BlockScaledTensor(fmt, (m, h), torch.empty((m, h // K.ELEMS_PER_BYTE[fmt]), dtype=torch.uint8, device=x.device),
                                          torch.zeros(K.scale_bytes(fmt, m, h), dtype=torch.uint8, device=x.device),
                                          torch.empty(1, dtype=torch.float32, device=x.device) if nv else None, "swizzled"),
                "ws": torch.empty(K.gemm_workspace_bytes(m, h, f, fmt), dtype=torch.uint8, device=x.device),
                "sync": torch.zeros(2 * len(self.layers), dtype=torch.int32, device=x.device) if nv else None,
            }
        if st["sync"] is not None:
            st["sync"].zero_()
        slots = self._amax_slots(0, x.device)
        src, y = x, None
        last = len(self.layers) - 1
        for li, w in enumerate(self.layers):
            hq = K.rmsnorm_quantize_rows(src, residual, w.w_n, self.eps, fmt, st["hq"], sync=st["sync"][2 * li:2 * li + 2] if st["sync"] is not None else None)
            if fmt == "nvfp4":
                a = K.gemm_blockscaled(hq, w.w_gu, epilogue="silu_gate", amax_out=slots[li][1:2])
                aq = K.quantize(a, fmt, amax=slots[li][1:2])
            else:
                _, aq = K.gemm_blockscaled(hq, w.w_gu, epilogue="silu_gate", quantize_out=True, want_bf16=False)
            if li < last:
                src = K.gemm_blockscaled_partials(aq, w.w_d, workspace=st["ws"])
            else:
                y = K.gemm_blockscaled(aq, w.w_d)
        return y

    def _forward_chunked(self, x, residual):
        import torch

        from . import _native as N

        m = x.shape[0]
        c = self.chunks
        bounds = [((m * i // c) + 127) // 128 * 128 if 0 < i < c else m * i // c for i in range(c + 1)]
        bounds = [min(b, m) for b in bounds]
        spans = [(bounds[i], bounds[i + 1]) for i in range(c) if bounds[i + 1] > bounds[i]]
        if len(spans) < 2:
            slots = self._amax_slots(0, x.device)
            for w, am in zip(self.layers, slots):
                x = decoder_block(x, residual, w, self.eps, group=self.group, scratch=self._scratch[0], amax=am)
            return x
        if self._streams is None or len(self._streams) < len(spans):
            self._streams = [torch.cuda.Stream(device=x.device) for _ in spans]
        main = torch.cuda.current_stream()
        out = torch.empty_like(x)
        N.check(N.load().tf_set_sm_margin(self.sm_margin), "tf_set_sm_margin")
        try:
            xs = [x[a:b] for a, b in spans]
            rs = [residual[a:b] for a, b in spans]
            for s in self._streams[:len(spans)]:
                s.wait_stream(main)
            last = len(self.layers) - 1
            slots = []
            for ci in range(len(spans)):
                with torch.cuda.stream(self._streams[ci]):
                    slots.append(self._amax_slots(ci, x.device))
            for li, w in enumerate(self.layers):
                for ci, (a, b) in enumerate(spans):
                    with torch.cuda.stream(self._streams[ci]):
                        xs[ci] = decoder_block(xs[ci], rs[ci], w, self.eps, group=self.group, scratch=self._scratch[ci], out=out[a:b] if li == last else None,
                                               amax=slots[ci][li])
            for s in self._streams[:len(spans)]:
                main.wait_stream(s)
        finally:
            N.check(N.load().tf_set_sm_margin(0), "tf_set_sm_margin")
        return out

    def _peer_for(self, x):
        """The symmetric buffer for activations of ``x``'s size (collective on first use; None for a single-rank group)."""
        import torch.distributed as dist

        if dist.get_world_size(self.group) < 2:
            return None
        need = x.numel() * 2
        if self._peer is None or self._peer.nbytes < need:
            from .collective import PeerAllReduce

            self._peer = PeerAllReduce(need, self.group, x.device, channels=max(1, self.chunks), num_ctas=max(1, self.sm_margin), multicast=self._peer_path != "peer_loads",
                                       reduce_in_switch=self._peer_path == "switch_reduce")
        return self._peer

    def _forward_peer(self, x, residual):
        """All-reduce by this package's kernel: every chunk's second GEMM writes into the chunk's rows of the symmetric buffer,
        the kernel sums them in place and the next block reads them there. The all-reduce kernels of the chunks are chained by
        events into one order that is the same on every rank, so two of them never wait for each other crosswise."""
        import torch

        from . import _native as N

        peer = self._peer
        m, h = x.shape
        c = max(1, self.chunks)
        world = peer.world
        unit = 128
        while (unit * h) % (8 * world):
            unit *= 2
        bounds = [min(m, (m * i // c + unit - 1) // unit * unit) if 0 < i < c else m * i // c for i in range(c + 1)]
        spans = [(bounds[i], bounds[i + 1]) for i in range(c) if bounds[i + 1] > bounds[i]]
        if any(((b - a) * h) % (8 * world) for a, b in spans):
            raise TilefishPreconditionError(f"peer_all_reduce: a chunk of [{m}, {h}] is not a multiple of {8 * world} elements", kind="divisible", arg="x")
        multi = len(spans) > 1
        if multi and (self._streams is None or len(self._streams) < len(spans)):
            self._streams = [torch.cuda.Stream(device=x.device) for _ in spans]
        main = torch.cuda.current_stream()
        streams = self._streams[:len(spans)] if multi else [main]
        out = torch.empty_like(x)
        views = [peer.view(a * h * 2, (b - a, h)) for a, b in spans]
        self._last_reduce = None

        def reducer(ci):
            def reduce(y):
                st = torch.cuda.current_stream()
                if self._last_reduce is not None:
                    st.wait_event(self._last_reduce)
                peer.allreduce_(y, channel=ci)
                ev = torch.cuda.Event()
                ev.record(st)
                self._last_reduce = ev

            return reduce

        if multi:
            N.check(N.load().tf_set_sm_margin(self.sm_margin), "tf_set_sm_margin")
        try:
            xs = [x[a:b] for a, b in spans]
            rs = [residual[a:b] for a, b in spans]
            for s in streams:
                if s is not main:
                    s.wait_stream(main)
            slots = []
            for ci in range(len(spans)):
                with torch.cuda.stream(streams[ci]):
                    slots.append(self._amax_slots(ci, x.device))
            for li, w in enumerate(self.layers):
                for ci in range(len(spans)):
                    with torch.cuda.stream(streams[ci]):
                        xs[ci] = decoder_block(xs[ci], rs[ci], w, self.eps, scratch=self._scratch[ci], out=views[ci], reduce=reducer(ci), amax=slots[ci][li])
            for ci, (a, b) in enumerate(spans):
                with torch.cuda.stream(streams[ci]):
                    out[a:b].copy_(xs[ci])
            for s in streams:
                if s is not main:
                    main.wait_stream(s)
        finally:
            if multi:
                N.check(N.load().tf_set_sm_margin(0), "tf_set_sm_margin")
            self._last_reduce = None
        return out

    def _forward_fused(self, x, residual, rows_local: bool = False):
        """Row-sharded normalisation with this package's fused exchange kernel. Every rank gets the full ``x`` / ``residual`` and
        returns the full result (the residual rows of the other ranks arrive with one all-gather at the end); with
        ``rows_local`` it gets and returns only its own rows (chunk by chunk: rows [rank * r, (rank + 1) * r) of every chunk),
        which is all the kernel ever reads of the input. Per block and row chunk: tf_tp_norm_exchange -> gemm + SiLU gate ->
        (quantize) -> gemm into the symmetric partial buffer."""
        import torch
        import torch.distributed as dist

        from . import _native as N
        from .collective import PeerAllReduce

        world = dist.get_world_size(self.group)
        rank = dist.get_rank(self.group)
        m, h = x.shape
        if rows_local:
            m *= world
        fmt = self.layers[0].fmt
        c = max(1, self.chunks)
        unit = 128 * world
        if m % (unit * c):
            c = 1
        if m % unit or h % 128:
            raise TilefishPreconditionError(f"fused_exchange needs M={m} to be a multiple of 128 x group size ({unit}) and H={h} of 128", kind="divisible", arg="x")
        rows = m // c       # rows of a chunk
        r = rows // world   # rows of a chunk this rank normalises
        epb = K.ELEMS_PER_BYTE[fmt]
        part_b, codes_b, scales_b = rows * h * 2, rows * h // epb, K.scale_bytes(fmt, rows, h)
        chunk_b = (part_b + codes_b + scales_b + 256 + 255) // 256 * 256
        if self._peer is None or self._peer.nbytes < c * chunk_b or self._peer.channels < c:
            self._peer = PeerAllReduce(c * chunk_b, self.group, x.device, channels=c, num_ctas=max(1, self.sm_margin),
                                       multicast=self._peer_path != "peer_loads", reduce_in_switch=self._peer_path == "switch_reduce")
        peer = self._peer
        key = ("fused", rows, h, fmt)
        for ci in range(c):
            while len(self._scratch) <= ci:
                self._scratch.append({})
            if key not in self._scratch[ci]:
                self._scratch[ci][key] = torch.empty((r, h), dtype=torch.bfloat16, device=x.device)
        multi = c > 1
        if multi and (self._streams is None or len(self._streams) < c):
            self._streams = [torch.cuda.Stream(device=x.device) for _ in range(c)]
        main = torch.cuda.current_stream()
        streams = self._streams[:c] if multi else [main]
        out = torch.empty_like(x)
        self._last_reduce = None

        def ordered(fn):  # the exchange kernels of all chunks run in one order that is the same on every rank
            st = torch.cuda.current_stream()
            if self._last_reduce is not None:
                st.wait_event(self._last_reduce)
            fn()
            ev = torch.cuda.Event()
            ev.record(st)
            self._last_reduce = ev

        last_gemms = [None]

        def gemms_begin():
            # One chunk's GEMMs at a time: only the exchange kernel then ever runs beside a GEMM (an option; see the constructor).
            if self.exclusive_gemms and multi and last_gemms[0] is not None:
                torch.cuda.current_stream().wait_event(last_gemms[0])

        def gemms_end():
            if self.exclusive_gemms and multi:
                ev = torch.cuda.Event()
                ev.record(torch.cuda.current_stream())
                last_gemms[0] = ev

        if multi:
            N.check(N.load().tf_set_sm_margin(self.sm_margin), "tf_set_sm_margin")
        try:
            views = []
            for ci in range(c):
                base = ci * chunk_b
                buf = peer.buffer
                views.append({
                    "off": (base, base + part_b, base + part_b + codes_b, base + part_b + codes_b + scales_b),
                    "partial": buf[base:base + part_b].view(torch.bfloat16).view(rows, h),
                    "codes": buf[base + part_b:base + part_b + codes_b].view(rows, h // epb),
                    "scales": buf[base + part_b + codes_b:base + part_b + codes_b + scales_b],
                    "gs": buf[base + part_b + codes_b + scales_b:base + part_b + codes_b + scales_b + 4 * world].view(torch.float32) if fmt == "nvfp4" else None,
                    "res": residual[ci * r:(ci + 1) * r] if rows_local else residual[ci * rows + rank * r:ci * rows + (rank + 1) * r],
                })
            for s in streams:
                if s is not main:
                    s.wait_stream(main)
            slots = []
            for ci in range(c):
                with torch.cuda.stream(streams[ci]):
                    slots.append(self._amax_slots(ci, x.device))
                    if rows_local:  # the first exchange reads this rank's rows only
                        views[ci]["partial"][rank * r:(rank + 1) * r].copy_(x[ci * r:(ci + 1) * r])
                    else:
                        views[ci]["partial"].copy_(x[ci * rows:(ci + 1) * rows])
            # the second GEMM delivers its partial results to the ranks that sum them, when it can (one pass, exact sum)
            f_local = self.layers[0].w_d.shape[1]
            deliver = (self.deliver_partials and world > 1 and self._peer_path != "switch_reduce"
                       and K.gemm_workspace_bytes(rows, h, f_local, fmt, "none") == 0)
            self.delivered = deliver  # what the most recent forward did (tests read it)
            last = len(self.layers) - 1
            for li, w in enumerate(self.layers):
                for ci in range(c):
                    v = views[ci]
                    with torch.cuda.stream(streams[ci]):
                        am = slots[ci][li]
                        ordered(lambda: peer.norm_exchange_(partial_offset=v["off"][0], codes_offset=v["off"][1], scales_offset=v["off"][2], gs_offset=v["off"][3],
                                                            rows_total=rows, d=h, sum_peers=0 if li == 0 else (2 if deliver else 1), residual_rows=v["res"], w=w.w_n,
                                                            h_scratch=self._scratch[ci][key], amax=am[0:1] if am is not None else None, eps=self.eps,
                                                            fmt=fmt, channel=ci))
                        hq = K.BlockScaledTensor(fmt, (rows, h), v["codes"], v["scales"], v["gs"], "swizzled", gs_rows=r if fmt == "nvfp4" else 0)
                        gemms_begin()
                        if fmt == "nvfp4":
                            a = K.gemm_blockscaled(hq, w.w_gu, epilogue="silu_gate", amax_out=am[1:2])
                            aq = K.quantize(a, fmt, amax=am[1:2])
                        else:
                            _, aq = K.gemm_blockscaled(hq, w.w_gu, epilogue="silu_gate", quantize_out=True, want_bf16=False)
                        if deliver and li < last:
                            # rows [o * r, (o + 1) * r) of this rank's partial result go to rank o's region, slot `rank`
                            K.gemm_blockscaled_scatter(aq, w.w_d, [p + v["off"][0] + rank * r * h * 2 for p in peer.buffer_ptrs], r, h)
                        else:
                            K.gemm_blockscaled(aq, w.w_d, out=v["partial"])
                        gemms_end()
            for ci in range(c):
                v = views[ci]
                with torch.cuda.stream(streams[ci]):
                    ordered(lambda: peer.allreduce_(v["partial"], channel=ci))
                    if rows_local:
                        out[ci * r:(ci + 1) * r].copy_(v["partial"][rank * r:(rank + 1) * r])
                    else:
                        out[ci * rows:(ci + 1) * rows].copy_(v["partial"])
                        if world > 1:
                            dist.all_gather_into_tensor(residual[ci * rows:(ci + 1) * rows], v["res"].clone(), group=self.group)
            for s in streams:
                if s is not main:
                    main.wait_stream(s)
        finally:
            if multi:
                N.check(N.load().tf_set_sm_margin(0), "tf_set_sm_margin")
            self._last_reduce = None
        return out

    def _forward_row_sharded(self, x, residual, rows_local: bool = False):
        import torch
        import torch.distributed as dist

        from . import _native as N

        world = dist.get_world_size(self.group)
        rank = dist.get_rank(self.group)
        m, h = x.shape
        if rows_local:
            m *= world
        c = max(1, self.chunks)
        unit = 128 * world
        if m % (unit * c):
            c = 1
        if m % unit:
            raise TilefishPreconditionError(f"scatter_gather needs M={m} to be a multiple of 128 x group size ({unit})", kind="divisible", arg="x")
        rows = m // c       # rows of a chunk
        r = rows // world   # rows of a chunk this rank normalises
        if self._streams is None or len(self._streams) < c:
            self._streams = [torch.cuda.Stream(device=x.device) for _ in range(c)]
        while len(self._scratch) < c:
            self._scratch.append({})
        main = torch.cuda.current_stream()
        out = torch.empty_like(x)
        if c > 1:
            N.check(N.load().tf_set_sm_margin(self.sm_margin), "tf_set_sm_margin")
        try:
            xs, rs = [], []
            for ci in range(c):
                lo = ci * r if rows_local else ci * rows + rank * r
                xs.append(x[lo:lo + r])
                rs.append(residual[lo:lo + r])  # this rank's rows are updated in place; the others arrive with the final all-gather
            streams = self._streams[:c] if c > 1 else [main]
            for st in streams:
                if st is not main:
                    st.wait_stream(main)
            for w in self.layers:
                for ci in range(c):
                    with torch.cuda.stream(streams[ci]):
                        xs[ci] = decoder_block_row_sharded(xs[ci], rs[ci], w, self.eps, self.group, world, self._scratch[ci])
            for ci in range(c):
                with torch.cuda.stream(streams[ci]):
                    if rows_local:
                        out[ci * r:(ci + 1) * r].copy_(xs[ci])
                    else:
                        dist.all_gather_into_tensor(out[ci * rows:(ci + 1) * rows], xs[ci], group=self.group)
                        dist.all_gather_into_tensor(residual[ci * rows:(ci + 1) * rows], rs[ci].clone(), group=self.group)
            for st in streams:
                if st is not main:
                    main.wait_stream(st)
        finally:
            if c > 1:
                N.check(N.load().tf_set_sm_margin(0), "tf_set_sm_margin")
        return out

    __call__ = forward

    def check(self) -> None:
        """Synchronizes and raises ``TilefishRuntimeError`` if a bounded wait of this stack's exchange kernels gave up (their waits on
        the peers are limited to two seconds; after a failure the outputs are partial sums). Recovery: ``reset()`` on every rank."""
        if self._peer is not None:
            self._peer.check()

    def reset(self) -> None:
        """Collective: clears the exchange kernels' state on every rank after a failure (see ``check``)."""
        if self._peer is not None:
            self._peer.reset()

    def close(self) -> None:
        """Releases what the stack holds of the process group: the symmetric buffers and their handles, the side streams and the scratch
        tensors. Every rank calls it (after dropping the CUDA graphs captured from the stack) before the process group is destroyed or
        the process exits."""
        import torch

        torch.cuda.synchronize()
        if self._peer is not None:
            self._peer.close()
        self._peer = None
        self._streams = None
        self._scratch = [{} for _ in range(max(1, self.chunks))]
        self._last_reduce = None

    def capture(self, x, residual, rows_local: bool = False):
        """Captures one ``forward(x, residual)`` into a CUDA graph (after one eager warm-up run, which also sets the kernels'
        attributes). ``x`` and ``residual`` are the graph's fixed input buffers: write new inputs into them, then
        ``replay()``. With tensor parallelism the all-reduces and both row-chunk streams are part of the graph, so a step
        costs one launch on the host: at 4-8 GPUs the per-layer kernels are too short for Python to keep up otherwise."""
        import torch

        self.forward(x, residual, rows_local) if rows_local else self.forward(x, residual)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            out = self.forward(x, residual, rows_local) if rows_local else self.forward(x, residual)
        return CapturedStack(graph, x, residual, out, self)

    def weight_bytes(self) -> int:
        return sum(w.nbytes() for w in self.layers)


class CapturedStack:
    """A captured ``MlpStack.forward``: ``replay()`` relaunches it over the captured ``x`` / ``residual`` buffers and returns ``out``."""

    def __init__(self, graph, x, residual, out, stack=None) -> None:
        self.graph, self.x, self.residual, self.out, self.stack = graph, x, residual, out, stack

    def replay(self, check: bool = False):
        """``check=True``: look (without synchronizing) at the error words the previous replay copied out, and raise if an exchange
        kernel's bounded wait gave up; ``stack.check()`` is the synchronizing form."""
        if check and self.stack is not None and self.stack._peer is not None:
            self.stack._peer.raise_if_failed("captured MlpStack")
        self.graph.replay()
        return self.out

    def release(self) -> None:
        """Drops the CUDA graph (it holds the captured exchange kernels and, with NCCL modes, the captured collectives)."""
        self.graph = None
        self.out = None
