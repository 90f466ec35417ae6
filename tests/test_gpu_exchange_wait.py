"""Failure detection of the exchange kernels without a fault and without a second GPU: a rank whose peer never arrives.

Both kernels of csrc/allreduce.cu are launched through the raw C ABI as rank 0 of a two-rank group whose "peer" is a second
set of local buffers that nothing ever writes. The rank's own state block carries a 50 ms wait limit. The kernel must return
by itself with error word 2 ("a peer never arrived") in its state block, well inside a second, touch nothing it should not,
and leave the context usable for the next kernels."""

import ctypes
import time

import numpy as np
import pytest
import torch

from oracle import blockscaled as O

pytestmark = pytest.mark.gpu

STATE_BYTES, ERROR_WORD, LIMIT_WORD = 128, 88 // 8, 96 // 8
LIMIT_NS = 50_000_000


@pytest.fixture(scope="module")
def N():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from tilefish_b200 import _native

    _native.load()
    return _native


def lonely_rank(nbytes):
    """Buffers and state blocks of a two-rank group living on one GPU; only rank 0 will ever run."""
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(2)]
    states = [torch.zeros(STATE_BYTES, dtype=torch.uint8, device="cuda") for _ in range(2)]
    states[0].view(torch.int64)[LIMIT_WORD] = LIMIT_NS
    u64s = ctypes.c_uint64 * 2
    return bufs, states, u64s(*[b.data_ptr() for b in bufs]), u64s(*[s.data_ptr() for s in states])


def assert_context_usable(N):
    from tilefish_b200 import kernels as K

    assert N.device_status() == (0, 0)
    x = O.randn((64, 256), 5, torch.bfloat16)
    q = K.quantize(x.cuda(), "mxfp8", layout="plain")
    codes, scales = O.quantize_mx(x, "mxfp8")
    assert np.array_equal(q.codes.cpu().numpy().view(np.uint8), np.asarray(codes).view(np.uint8))
    assert np.array_equal(q.scales.cpu().numpy().view(np.uint8).reshape(-1), np.asarray(scales).view(np.uint8).reshape(-1))


def test_all_reduce_gives_up_on_a_peer_that_never_arrives(N):
    count = 8 * 2 * 4096
    bufs, states, buf_ptrs, state_ptrs = lonely_rank(2 * count)
    bufs[0].view(torch.bfloat16).fill_(1.0)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    N.check(N.load().tf_allreduce_bf16(buf_ptrs, state_ptrs, ctypes.c_uint64(0), 0, 0, 2, 0, count, 4,
                                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "tf_allreduce_bf16")
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert LIMIT_NS * 1e-9 <= elapsed < 1.0, elapsed
    words = states[0].cpu().view(torch.int64)
    assert int(words[ERROR_WORD]) == 2
    # the rank announced itself to the peer, and summed nothing: its buffer is untouched
    assert int(states[1].cpu().view(torch.int32)[0]) != 0
    assert bool((bufs[0].view(torch.bfloat16) == 1.0).all())
    # the word is sticky: the next call on the same state returns at once
    t0 = time.perf_counter()
    N.check(N.load().tf_allreduce_bf16(buf_ptrs, state_ptrs, ctypes.c_uint64(0), 0, 0, 2, 0, count, 4,
                                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "tf_allreduce_bf16")
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < LIMIT_NS * 1e-9
    assert_context_usable(N)


@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
def test_norm_exchange_gives_up_on_a_peer_that_never_arrives(N, fmt):
    from tilefish_b200 import kernels as K

    rows, d = 256, 1024
    partial_off, codes_off, scales_off, gs_off = 0, rows * d * 2, rows * d * 3, rows * d * 3 + 65536
    bufs, states, buf_ptrs, state_ptrs = lonely_rank(rows * d * 3 + 2 * 65536)
    residual = torch.ones(rows // 2, d, dtype=torch.float32, device="cuda")
    w = torch.ones(d, dtype=torch.bfloat16, device="cuda")
    h = torch.zeros(rows // 2, d, dtype=torch.bfloat16, device="cuda")
    amax = torch.zeros(1, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    N.check(N.load().tf_tp_norm_exchange(buf_ptrs, state_ptrs, ctypes.c_uint64(0), 0, 0, 2, partial_off, codes_off, scales_off, gs_off, rows, d, 1,
                                         residual.data_ptr(), w.data_ptr(), h.data_ptr(), ctypes.cast(amax.data_ptr(), ctypes.POINTER(ctypes.c_float)),
                                         1e-6, K.FORMATS[fmt], 8, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)), "tf_tp_norm_exchange")
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    assert LIMIT_NS * 1e-9 <= elapsed < 1.0, elapsed
    assert int(states[0].cpu().view(torch.int64)[ERROR_WORD]) == 2
    assert bool((residual == 1.0).all()), "a rank that gave up must not have updated its residual rows"
    assert_context_usable(N)
