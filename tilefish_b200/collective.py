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

STATE_BYTES = 128  # per channel: flag slots, call counter, grid-barrier counters, error word (see csrc/allreduce.cu)
ERROR_WORD_OFFSET = 88


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
        quantized rows (codes, swizzled scales, nvfp4 global scale) at the given offsets of EVERY rank's buffer."""
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
                                            self.world, partial_offset, codes_offset, scales_offset, gs_offset, rows_total, d, int(bool(sum_peers)),
                                            residual_rows.data_ptr(), w.data_ptr(), h_scratch.data_ptr(), amax.data_ptr() if amax is not None else None,
                                            float(eps), K.FORMATS[fmt], self.num_ctas, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)),
                "tf_tp_norm_exchange")

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
            raise TilefishRuntimeError(f"PeerAllReduce: a bounded wait gave up (error word {s}); the group's state must be rebuilt")


def peer_all_reduce(group, nbytes: int, device, **kw) -> Optional[PeerAllReduce]:
    """``PeerAllReduce`` for ``group``, or None for a single rank (nothing to exchange)."""
    import torch.distributed as dist

    if group is None or dist.get_world_size(group) < 2:
        return None
    return PeerAllReduce(nbytes, group, device, **kw)
