"""The tensor-parallel exchange as this package's own kernel: an in-place bf16 all-reduce over peer-mapped (symmetric) memory.

torch.distributed does the plumbing only: ``torch.distributed._symmetric_memory`` allocates the buffers, exchanges the
handles over the process group and (on NVSwitch machines) binds them to a multicast object. The data path is
``tf_allreduce_bf16`` (csrc/allreduce.cu): sums over plain peer loads (f32, one rounding to nearest even) whose result ``multimem.st`` writes to all ranks through
the switch, or - ``reduce_in_switch=True`` - ``multimem.ld_reduce``, where NVSwitch forms the sum: half the bytes per GPU, but
its bf16 result is within one bf16 step of the exact sum and not always the nearest value (measured on B200). Without a
multicast mapping (or ``multicast=False``) the result is gathered with peer loads as well. The reference has no cross-device exchange; this is the "one all-reduce per layer" of the
tensor-parallel MLP (w_gu split by output columns, w_d by K).
"""

from __future__ import annotations

import ctypes
from typing import Optional

from . import _native as N
from .errors import TilefishPreconditionError, TilefishRuntimeError

STATE_BYTES = 128  # per channel: flag slots, call counter, grid-barrier counters, error word, wait limit (see csrc/allreduce.cu)
ERROR_WORD_OFFSET = 88
WAIT_LIMIT_OFFSET = 96  # nanoseconds, 0 = the kernels' two-second default


class PeerAllReduce:
    """A symmetric bf16 buffer of ``nbytes`` on every rank of ``group`` plus the state the kernel's barriers need.

    The producer (the second GEMM) writes its partial result straight into ``view(...)`` of the buffer; ``allreduce_`` sums it
    over the ranks in place. ``channels``: independent state blocks, one per stream that may have a call in flight.
    Construction is collective (every rank of the group, same arguments).
    """

    def __init__(self, nbytes: int, group, device, *, channels: int = 2, num_ctas: int = 24, multicast: bool = True,
                 reduce_in_switch: bool = False) -> None:
        import torch
        import torch.distributed as dist
        import torch.distributed._symmetric_memory as symm

        self.lib = N.load()
        self.group = group if group is not None else (dist.group.WORLD if dist.is_initialized() else None)
        self.world = dist.get_world_size(self.group) if self.group is not None else 1
        self.rank = dist.get_rank(self.group) if self.group is not None else 0
        if not 1 <= self.world <= 8:
            raise TilefishPreconditionError(f"PeerAllReduce: {self.world} ranks (1..8 supported)", kind="argument", arg="group")
        self.num_ctas = int(num_ctas)
        self.reduce_in_switch = bool(reduce_in_switch)
        self.channels = int(channels)
        self.nbytes = (int(nbytes) + 255) // 256 * 256
        if self.world == 1:
            # a single rank has no peers: ordinary device memory, the same kernels (their barriers then only meet themselves)
            self.buffer = torch.empty(self.nbytes, dtype=torch.uint8, device=device)
            self.state = torch.zeros(self.channels * STATE_BYTES, dtype=torch.uint8, device=device)
            self.multicast_ptr = 0
            u64s = ctypes.c_uint64 * 1
            self._bufs = u64s(self.buffer.data_ptr())
            self._states = [u64s(self.state.data_ptr() + c * STATE_BYTES) for c in range(self.channels)]
            return
        self.buffer = symm.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.state = symm.empty(self.channels * STATE_BYTES, dtype=torch.uint8, device=device)
        self.state.zero_()
        torch.cuda.synchronize(device)
        self._buf_handle = symm.rendezvous(self.buffer, self.group)
        self._state_handle = symm.rendezvous(self.state, self.group)
        dist.barrier(group=self.group)  # every rank's state block is zero before any kernel writes a flag into it
        bufs = [int(p) for p in self._buf_handle.buffer_ptrs]
        states = [int(p) for p in self._state_handle.buffer_ptrs]
        if len(bufs) != self.world or not all(bufs) or not all(states):
            raise TilefishRuntimeError("PeerAllReduce: symmetric memory rendezvous returned no peer pointers")
        # the handles describe the allocation block a tensor lives in: carry the tensor's offset inside it over to every mapping
        boff = self.buffer.data_ptr() - bufs[self.rank]
        soff = self.state.data_ptr() - states[self.rank]
        if boff < 0 or soff < 0 or boff % 16 or soff % 16:
            raise TilefishRuntimeError("PeerAllReduce: this rank's tensor does not lie inside its own symmetric block")
        bufs = [p + boff for p in bufs]
        states = [p + soff for p in states]
        mc = int(self._buf_handle.multicast_ptr) if (multicast and self._buf_handle.has_multicast_support) else 0
        self.multicast_ptr = mc + boff if mc else 0
        u64s = ctypes.c_uint64 * self.world
        self._bufs = u64s(*bufs)
        self._states = [u64s(*[s + c * STATE_BYTES for s in states]) for c in range(self.channels)]

    @property
    def buffer_ptrs(self):
        """The address, on this GPU, of every rank's buffer (entry ``rank`` is this rank's own)."""
        return [int(p) for p in self._bufs]

    @property
    def mode(self) -> str:
        if not self.multicast_ptr:
            return "peer_loads"
        return "switch_reduce" if self.reduce_in_switch else "peer_reduce_multicast_store"

    def view(self, offset_bytes: int, shape):
        """A bf16 tensor over ``shape`` elements of this rank's buffer starting at ``offset_bytes`` (a multiple of 16)."""
        import torch

        n = 1
        for s in shape:
            n *= int(s)
        if offset_bytes % 16 or offset_bytes < 0 or offset_bytes + 2 * n > self.nbytes:
            raise TilefishPreconditionError(f"PeerAllReduce.view: [{offset_bytes}, +{2 * n}) outside the {self.nbytes}-byte buffer", kind="shape", arg="shape")
        return self.buffer[offset_bytes:offset_bytes + 2 * n].view(torch.bfloat16).view(*shape)

    def allreduce_(self, t, channel: int = 0):
        """Sums ``t`` (a contiguous bf16 view into ``self.buffer``; the same view on every rank) over the ranks, in place, on the
        current stream. Calls on one channel must be stream-ordered; all ranks issue the same calls in the same order."""
        import torch

        if self.world == 1:
            return t  # nothing to sum
        off = t.data_ptr() - self.buffer.data_ptr()
        n = t.numel()
        if t.dtype != torch.bfloat16 or not t.is_contiguous() or off < 0 or off + 2 * n > self.nbytes:
            raise TilefishPreconditionError("PeerAllReduce.allreduce_: not a contiguous bf16 view of the symmetric buffer", kind="argument", arg="t")
        if not 0 <= channel < self.channels:
            raise TilefishPreconditionError(f"PeerAllReduce.allreduce_: channel {channel} of {self.channels}", kind="argument", arg="channel")
        N.check(self.lib.tf_allreduce_bf16(self._bufs, self._states[channel], ctypes.c_uint64(self.multicast_ptr), int(self.reduce_in_switch), self.rank, self.world, off, n,
                                          self.num_ctas, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "tf_allreduce_bf16")
        return t

    def norm_exchange_(self, *, partial_offset: int, codes_offset: int, scales_offset: int, gs_offset: int, rows_total: int, d: int, sum_peers: bool,
                       residual_rows, w, h_scratch, amax, eps: float, fmt: str, channel: int = 0) -> None:
        """``tf_tp_norm_exchange`` on the current stream: this rank sums its rows of the partial results at ``partial_offset`` over
        the ranks, adds them into ``residual_rows`` (f32, its rows of the residual stream), normalises with ``w`` and writes the
        quantized rows (codes, swizzled scales, nvfp4 global scale) at the given offsets of EVERY rank's buffer.
        ``sum_peers``: 0 / False (the region holds complete values), 1 / True (pull this rank's rows from every rank's region) or
        2 (the producers delivered their partial results for this rank's rows into this rank's region, one slot per source rank)."""
        import torch

        from . import kernels as K

        if not 0 <= channel < self.channels:
            raise TilefishPreconditionError(f"PeerAllReduce.norm_exchange_: channel {channel} of {self.channels}", kind="argument", arg="channel")
        for name, t, dt in (("residual_rows", residual_rows, torch.float32), ("w", w, torch.bfloat16), ("h_scratch", h_scratch, torch.bfloat16)):
            if t.dtype != dt or not t.is_contiguous() or not t.is_cuda:
                raise TilefishPreconditionError(f"PeerAllReduce.norm_exchange_: {name} must be a contiguous {dt} device tensor", kind="dtype", arg=name)
        rows_local = rows_total // self.world
        if residual_rows.numel() != rows_local * d or h_scratch.numel() < rows_local * d or w.numel() != d:
            raise TilefishPreconditionError("PeerAllReduce.norm_exchange_: residual_rows / h_scratch / w do not match rows_total / world x d", kind="shape",
                                            arg="residual_rows")
        N.check(self.lib.tf_tp_norm_exchange(self._bufs, self._states[channel], ctypes.c_uint64(self.multicast_ptr), int(self.reduce_in_switch), self.rank,
                                            self.world, partial_offset, codes_offset, scales_offset, gs_offset, rows_total, d, int(sum_peers),
                                            residual_rows.data_ptr(), w.data_ptr(), h_scratch.data_ptr(), amax.data_ptr() if amax is not None else None,
                                            float(eps), K.FORMATS[fmt], self.num_ctas, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)),
                "tf_tp_norm_exchange")

    # ---- failure detection -----------------------------------------------------------------------------------------------
    # Every wait of the exchange kernels on a peer is bounded (two seconds). When one runs out (rank skew beyond the limit, a
    # stalled host, a rank that left), the kernel stores a nonzero error word in the channel's state block and returns; the
    # word is sticky, so every later call on that channel returns at once with partial sums. The host must therefore look at
    # the word: ``status()`` / ``check()`` synchronize and read it; ``arm_poll()`` + ``last_error()`` watch it without a
    # synchronization (an asynchronous copy into pinned host memory after a forward, read before the next one).
    def set_wait_limit(self, seconds: float) -> None:
        """How long a wait of the exchange kernels on a peer (or on this rank's own CTAs) may last before the kernel gives up, for this
        rank's later calls on every channel; 0 restores the two-second default. Stream-ordered with the calls around it."""
        import torch

        ns = int(round(float(seconds) * 1e9))
        if ns < 0:
            raise TilefishPreconditionError("PeerAllReduce.set_wait_limit: negative limit", kind="argument", arg="seconds")
        self._wait_limit_ns = ns
        words = self.state.view(torch.int64).view(self.channels, STATE_BYTES // 8)
        words[:, WAIT_LIMIT_OFFSET // 8] = ns

    @staticmethod
    def describe_error(word: int) -> str:
        return {0: "healthy", 1: "a grid barrier of the kernel's own CTAs gave up (not all CTAs were resident: leave that many SMs to the kernel)",
                2: "a peer never arrived within the wait limit (two seconds unless set_wait_limit changed it)"}.get(int(word), f"unknown error word {word}")

    def arm_poll(self) -> None:
        """Enqueues, on the current stream, a copy of the channels' error words into pinned host memory. Capturable in a CUDA graph."""
        import torch

        if getattr(self, "_poll_host", None) is None:
            self._poll_host = torch.zeros(self.channels, dtype=torch.int64).pin_memory()
        words = self.state.view(torch.int64).view(self.channels, STATE_BYTES // 8)[:, ERROR_WORD_OFFSET // 8]
        self._poll_host.copy_(words, non_blocking=True)

    def last_error(self) -> int:
        """The first nonzero error word the most recent completed ``arm_poll`` copy saw (0 when none, or when none was armed). No
        synchronization: the word is sticky, so a failure is seen one poll late at worst."""
        host = getattr(self, "_poll_host", None)
        if host is None:
            return 0
        for w in host.tolist():
            if w:
                return int(w)
        return 0

    def raise_if_failed(self, where: str = "") -> None:
        w = self.last_error()
        if w:
            raise TilefishRuntimeError(f"PeerAllReduce{(' (' + where + ')') if where else ''}: {self.describe_error(w)}; the results since then are partial sums. "
                                       "Stop, call reset() on every rank (a collective) and redo the step")

    def reset(self) -> None:
        """Collective: waits for this rank's work, zeroes its state blocks (flags, call counters, error words) and meets the other ranks, so
        that no rank launches again before every state block is clean."""
        import torch
        import torch.distributed as dist

        torch.cuda.synchronize(self.buffer.device)
        if self.world > 1:
            dist.barrier(group=self.group)  # no peer is still writing flags into this rank's block
        self.state.zero_()
        if getattr(self, "_wait_limit_ns", 0):
            self.set_wait_limit(self._wait_limit_ns * 1e-9)
        if getattr(self, "_poll_host", None) is not None:
            self._poll_host.zero_()
        torch.cuda.synchronize(self.buffer.device)
        if self.world > 1:
            dist.barrier(group=self.group)

    def close(self) -> None:
        """Drops the symmetric tensors and the rendezvous handles (after this rank's work is done). Call it on every rank before the
        process group goes away: a rank must not exit while its memory is still bound to the group's multicast object."""
        import torch

        if getattr(self, "buffer", None) is not None:
            torch.cuda.synchronize(self.buffer.device)
        for name in ("_buf_handle", "_state_handle", "buffer", "state", "_poll_host", "_bufs", "_states"):
            if hasattr(self, name):
                setattr(self, name, None)
        self.multicast_ptr = 0

    def status(self) -> int:
        """0 when healthy; else the first nonzero error word of the channels (1: a local barrier gave up, 2: a peer never
        arrived). Synchronizes the device."""
        import torch

        torch.cuda.synchronize(self.buffer.device)
        words = self.state.cpu().view(torch.int64).view(self.channels, STATE_BYTES // 8)[:, ERROR_WORD_OFFSET // 8]
        for w in words.tolist():
            if w:
                return int(w)
        return 0

    def check(self) -> None:
        s = self.status()
        if s:
            raise TilefishRuntimeError(f"PeerAllReduce: {self.describe_error(s)} (error word {s}); the results since then are partial sums. Stop, call "
                                       "reset() on every rank (a collective) and redo the step")


def peer_all_reduce(group, nbytes: int, device, **kw) -> Optional[PeerAllReduce]:
    """``PeerAllReduce`` for ``group``, or None for a single rank (nothing to exchange)."""
    import torch.distributed as dist

    if group is None or dist.get_world_size(group) < 2:
        return None
    return PeerAllReduce(nbytes, group, device, **kw)


# ---- row-sharded quantize / rmsnorm ---------------------------------------------------------------------------------------------
# Rows are independent in both operators, so each rank of a group works on a contiguous block of rows and nothing is exchanged, with
# one exception: the nvfp4 global scale is a property of the whole tensor. One 4-byte max all-reduce of the ranks' amax makes every
# rank quantize with the tensor's scale, and the shard's codes, scale bytes and global scale are then exactly the bytes the single-GPU
# quantizer produces for those rows. (max commutes with the correctly rounded division by 2688, so the scales themselves are reduced.)
def quantize_rows_sharded(x_rows, fmt: str, group=None, *, layout: str = "swizzled", stream=None):
    """BlockScaled quantization of this rank's rows ``x_rows`` (bf16 [M / n, K]) of a tensor whose rows are spread over ``group``.
    mxfp8 / mxfp4: no communication. nvfp4: the tensor-wide global scale through one 4-byte max all-reduce."""
    import torch.distributed as dist

    from . import kernels as K

    if fmt != "nvfp4":
        return K.quantize(x_rows, fmt, layout=layout, stream=stream)
    gs = K.nvfp4_global_scale(x_rows, stream=stream)
    if group is not None and dist.get_world_size(group) > 1:
        dist.all_reduce(gs, op=dist.ReduceOp.MAX, group=group)
    return K.quantize(x_rows, fmt, layout=layout, global_scale=gs, stream=stream)


def residual_add_rmsnorm_rows_sharded(x_rows, residual_rows, w, eps: float = 1e-6, group=None, *, quantize_to=None):
    """``residual_add_rmsnorm`` on this rank's rows, optionally followed by the quantization of the result with the scales of the WHOLE
    tensor (nvfp4: the kernel reduces this rank's amax, one 4-byte max all-reduce gives the tensor's). Returns ``out`` or ``(out, q)``."""
    import torch
    import torch.distributed as dist

    from . import kernels as K

    if quantize_to is None:
        return K.residual_add_rmsnorm(x_rows, residual_rows, w, eps)
    if quantize_to != "nvfp4":
        return K.residual_add_rmsnorm(x_rows, residual_rows, w, eps, quantize_to=quantize_to)
    amax = torch.zeros(1, dtype=torch.float32, device=x_rows.device)
    out = K.residual_add_rmsnorm(x_rows, residual_rows, w, eps, amax_out=amax)
    if group is not None and dist.get_world_size(group) > 1:
        dist.all_reduce(amax, op=dist.ReduceOp.MAX, group=group)
    return out, K.quantize(out, "nvfp4", amax=amax)

