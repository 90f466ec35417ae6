"""tf_gemm_blockscaled_static: the GEMM for hosts that cannot allocate device memory when they call it.

A serving process with a frozen memory pool, or a plugin that only receives its operator's tensors, has no workspace to
give the small-M GEMM (which sums K ranges through scratch memory). This entry point uses a fixed array inside the library
instead. The test drives it through the C ABI exactly as such a host would (raw pointers, no allocation between the calls)
and compares it with the regular entry point, twice in a row with different operands, so that whatever the first call left
in the shared array cannot leak into the second result. Collected last on purpose: if it fails under `-x`, every other test
has already run.
"""

import ctypes

import pytest
import torch

from oracle import blockscaled as O

pytestmark = pytest.mark.gpu


def call_static(N, qa, qb, out, m, n, k, fmt, epi, stream):
    lib = N.load()
    gsa = qa.global_scale.data_ptr() if qa.global_scale is not None else None
    gsb = qb.global_scale.data_ptr() if qb.global_scale is not None else None
    return lib.tf_gemm_blockscaled_static(qa.codes.data_ptr(), qa.scales.data_ptr(), gsa, qb.codes.data_ptr(), qb.scales.data_ptr(), gsb,
                                          out.data_ptr(), n, m, n, k, fmt, epi, None, None, stream)


@pytest.mark.parametrize("fmt_name", ["mxfp8", "nvfp4"])
def test_static_scratch_gemm_matches_the_workspace_gemm_twice_in_a_row(fmt_name):
    from tilefish_b200 import _native as N
    from tilefish_b200 import kernels as K

    K.require_cuda()
    m, n, k = 48, 1024, 8192
    fmt = K.FORMATS[fmt_name]
    need = K.gemm_workspace_bytes(m, n, k, fmt_name)
    assert 0 < need <= N.load().tf_gemm_static_scratch_bytes(), "the shape must use scratch memory and fit the built-in array"
    stream = torch.cuda.current_stream().cuda_stream
    operands = []
    for seed in (1, 2):
        a = O.randn((m, k), seed, torch.bfloat16)
        w = O.randn((n, k), seed + 10, torch.bfloat16, scale=k**-0.5)
        operands.append((K.quantize(a.cuda(), fmt_name), K.quantize(w.cuda(), fmt_name)))
    expected = [K.gemm_blockscaled(qa, qb) for qa, qb in operands]
    outs = [torch.empty((m, n), dtype=torch.bfloat16, device="cuda") for _ in operands]
    # one warm-up call: the first call on a device looks the array's address up and sets the kernel's attributes
    warm = torch.empty((m, n), dtype=torch.bfloat16, device="cuda")
    assert call_static(N, operands[0][0], operands[0][1], warm, m, n, k, fmt, N.EPI_NONE, stream) == N.TF_OK, N.last_error()
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before, _ = torch.cuda.mem_get_info()  # the driver's view: sees a cudaMalloc made inside the library, which torch's allocator cannot
    for (qa, qb), out in zip(operands, outs):  # two calls back to back, nothing allocated in between
        status = call_static(N, qa, qb, out, m, n, k, fmt, N.EPI_NONE, stream)
        assert status == N.TF_OK, N.last_error()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    assert torch.cuda.mem_get_info()[0] == free_before, "device memory was allocated (or freed) during the two calls"
    for out, ref in zip(outs, expected):
        assert torch.equal(out, ref), "same kernels, same summation order: the bytes must be identical"
    assert not torch.equal(outs[0], outs[1])
    assert N.device_status() == (0, 0)


def test_static_scratch_gemm_refuses_what_does_not_fit():
    from tilefish_b200 import _native as N
    from tilefish_b200 import kernels as K

    K.require_cuda()
    m, n, k = 256, 8192, 32768  # split-K with a workspace larger than the built-in array
    need = K.gemm_workspace_bytes(m, n, k, "mxfp8")
    cap = N.load().tf_gemm_static_scratch_bytes()
    if need <= cap:
        pytest.skip("this device splits the problem differently")
    one = torch.zeros(16, dtype=torch.uint8, device="cuda")
    status = N.load().tf_gemm_blockscaled_static(one.data_ptr(), one.data_ptr(), None, one.data_ptr(), one.data_ptr(), None, one.data_ptr(), n, m, n, k,
                                                 N.FMT_MXFP8, N.EPI_NONE, None, None, None)
    assert status == N.TF_ERR_WORKSPACE
    assert "built-in scratch holds" in N.last_error()
