"""The exchange kernel's data paths at 4 and 8 ranks, on ONE GPU, without any kernel waiting on another.

Every "rank" is a set of local buffers; the ranks' kernels run one after the other through the raw C ABI, each as rank r of a
world of 4 or 8. The cross-rank flag barriers are satisfied beforehand: the flag slots of the rank's state block are preset to a
value far ahead of any call counter, so no launch waits for a launch that has not run (nothing here spins on a peer). What is
checked is everything else: the bulk-copy ring with 4 or 8 sources per segment, the rank-order f32 sum rounded once, pulled
(sum_peers = 1) against delivered (sum_peers = 2) partial results, residual add, rmsnorm, the row block's own nvfp4 global scale and
the gather of codes / swizzled scales / global scales into every rank's buffer, bit for bit against the stand-alone kernels."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

STATE_BYTES = 128
AHEAD = 0x7FFFFFF0  # a flag value every barrier of the first calls sees as "already arrived"


@pytest.fixture(scope="module")
def K():
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    from tilefish_b200 import kernels

    kernels.require_cuda()
    return kernels


@pytest.mark.parametrize("world", [4, 8])
@pytest.mark.parametrize("fmt", ["nvfp4", "mxfp8"])
@pytest.mark.parametrize("delivered", [False, True])
def test_every_rank_of_a_world_run_in_turn(K, world, fmt, delivered):
    from tilefish_b200 import _native as N

    lib = N.load()
    d, r = 8192, 128
    rows = r * world
    epb = K.ELEMS_PER_BYTE[fmt]
    part_b, codes_b, scales_b = rows * d * 2, rows * d // epb, K.scale_bytes(fmt, rows, d)
    offs = (0, part_b, part_b + codes_b, part_b + codes_b + scales_b)
    nbytes = offs[3] + 256
    g = torch.Generator(device="cuda").manual_seed(world * 10 + (1 if delivered else 0))
    parts = [(torch.randn((rows, d), generator=g, device="cuda") * (1 + 0.25 * k)).to(torch.bfloat16) for k in range(world)]
    residual = torch.randn((rows, d), generator=g, device="cuda")
    w = (1 + 0.1 * torch.randn(d, generator=g, device="cuda")).to(torch.bfloat16)

    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device="cuda") for _ in range(world)]
    for o in range(world):
        region = bufs[o][:part_b].view(torch.bfloat16).view(rows, d)
        if delivered:  # slot s of owner o: rank s's partial results for owner o's rows
            for s in range(world):
                region[s * r:(s + 1) * r] = parts[s][o * r:(o + 1) * r]
        else:  # every rank's buffer holds that rank's partial results for all rows
            region.copy_(parts[o])
    states = torch.zeros((world, STATE_BYTES), dtype=torch.uint8, device="cuda")
    states.view(torch.int32).view(world, STATE_BYTES // 4)[:, :8] = AHEAD
    u64s = ctypes.c_uint64 * world
    buf_ptrs = u64s(*[b.data_ptr() for b in bufs])
    state_ptrs = u64s(*[states[k].data_ptr() for k in range(world)])
    res_dev = residual.clone()
    scratch = torch.empty((r, d), dtype=torch.bfloat16, device="cuda")
    amax = torch.zeros(world, dtype=torch.float32, device="cuda")
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for rank in range(world):
        N.check(lib.tf_tp_norm_exchange(buf_ptrs, state_ptrs, ctypes.c_uint64(0), 0, rank, world, offs[0], offs[1], offs[2], offs[3], rows, d,
                                        2 if delivered else 1, res_dev[rank * r:(rank + 1) * r].data_ptr(), w.data_ptr(), scratch.data_ptr(),
                                        ctypes.cast(amax[rank:rank + 1].data_ptr(), ctypes.POINTER(ctypes.c_float)), 1e-6, K.FORMATS[fmt], 8, stream),
                "tf_tp_norm_exchange")
    torch.cuda.synchronize()
    words = states.cpu().view(torch.int64).view(world, STATE_BYTES // 8)
    assert [int(x) for x in words[:, 88 // 8]] == [0] * world, "an exchange kernel reported an error word"

    # what the stand-alone kernels give: the rank-order f32 sum rounded once, then residual_add_rmsnorm and the quantizer per row block
    acc = parts[0].float()
    for k in range(1, world):
        acc = acc + parts[k].float()
    summed = acc.to(torch.bfloat16)
    res_ref = residual.clone()
    h = K.residual_add_rmsnorm(summed, res_ref, w, eps=1e-6)
    assert torch.equal(res_dev, res_ref), "residual stream"
    for check in (0, world - 1):  # every rank's buffer received every rank's rows
        buf = bufs[check]
        codes = buf[offs[1]:offs[1] + codes_b].view(rows, d // epb)
        scales = buf[offs[2]:offs[2] + scales_b]
        gs = buf[offs[3]:offs[3] + 4 * world].view(torch.float32)
        per_tile = scales_b // world  # one 128-row tile row of the swizzled layout per rank
        for rank in range(world):
            q = K.quantize(h[rank * r:(rank + 1) * r].contiguous(), fmt)
            assert torch.equal(codes[rank * r:(rank + 1) * r], q.codes), f"codes of rank {rank}'s rows in buffer {check}"
            assert torch.equal(scales[rank * per_tile:(rank + 1) * per_tile], q.scales.reshape(-1)), f"scales of rank {rank}'s rows in buffer {check}"
            if fmt == "nvfp4":
                assert gs[rank].view(torch.int32).item() == q.global_scale.view(torch.int32).item(), f"global scale of rank {rank}"
