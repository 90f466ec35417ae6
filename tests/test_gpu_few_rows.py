"""The few-rows (decode) step: residual add + rmsnorm + quantization in one launch, fed by a bf16 tensor or by the partial sums of a
split-K GEMM. Everything is compared bit for bit with the separate launches it replaces (which the other GPU tests hold against the
CPU oracle), and the stack built from it with the oracle's stack."""

import pytest
import torch

from oracle import blockscaled as O

pytestmark = pytest.mark.gpu

FMTS = ["mxfp8", "mxfp4", "nvfp4"]


@pytest.fixture(scope="module")
def K():
    from tilefish_b200 import kernels

    kernels.require_cuda()
    return kernels


def fresh_q(K, fmt, m, d):
    return K.BlockScaledTensor(fmt, (m, d), torch.empty((m, d // K.ELEMS_PER_BYTE[fmt]), dtype=torch.uint8, device="cuda"),
                               torch.zeros(K.scale_bytes(fmt, m, d), dtype=torch.uint8, device="cuda"),
                               torch.empty(1, dtype=torch.float32, device="cuda") if fmt == "nvfp4" else None, "swizzled")


def separate(K, x, res, w, eps, fmt):
    """residual_add_rmsnorm, then quantize: the launches the fused one replaces."""
    if fmt == "nvfp4":
        amax = torch.zeros(1, device="cuda")
        h = K.residual_add_rmsnorm(x, res, w, eps, amax_out=amax)
        return h, K.quantize(h, fmt, amax=amax)
    h, q = K.residual_add_rmsnorm(x, res, w, eps, quantize_to=fmt)
    return h, q


def same_q(a, b):
    assert torch.equal(a.codes, b.codes), "codes differ"
    assert torch.equal(a.scales, b.scales), "swizzled scale bytes differ"
    if a.global_scale is not None:
        assert a.global_scale.view(torch.int32).item() == b.global_scale.view(torch.int32).item(), "global scale differs"


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("m,d", [(1, 64), (5, 2560), (64, 8192), (128, 4096), (3, 32768), (148, 256)])
def test_fused_rows_equal_the_separate_launches(K, fmt, m, d):
    g = torch.Generator().manual_seed(m * 131 + d)
    x = torch.randn((m, d), generator=g).to(torch.bfloat16).cuda()
    res0 = torch.randn((m, d), generator=g).cuda()
    w = (1 + 0.1 * torch.randn(d, generator=g)).to(torch.bfloat16).cuda()
    res_a, res_b = res0.clone(), res0.clone()
    h_ref, q_ref = separate(K, x, res_a, w, 1e-6, fmt)
    out = torch.empty_like(x)
    sync = torch.zeros(2, dtype=torch.int32, device="cuda")
    q = K.rmsnorm_quantize_rows(x, res_b, w, 1e-6, fmt, fresh_q(K, fmt, m, d), sync=sync if fmt == "nvfp4" else None, out=out)
    torch.cuda.synchronize()
    assert torch.equal(res_a, res_b), "residual differs"
    assert torch.equal(out, h_ref), "bf16 result differs"
    same_q(q, q_ref)
    if fmt == "nvfp4":
        assert sync[1].item() == m  # every row's CTA arrived once


@pytest.mark.parametrize("fmt", FMTS)
@pytest.mark.parametrize("m,n,k", [(1, 2560, 6144), (64, 8192, 28672), (16, 512, 8192)])
def test_fused_rows_from_split_k_partial_sums(K, fmt, m, n, k):
    if K.gemm_splits(m, n, k, fmt) <= 1:
        pytest.skip("the planner does not split this shape")
    g = torch.Generator().manual_seed(k + m)
    a = K.quantize(torch.randn((m, k), generator=g).to(torch.bfloat16).cuda(), fmt)
    b = K.quantize((torch.randn((n, k), generator=g) * k**-0.5).to(torch.bfloat16).cuda(), fmt)
    res0 = torch.randn((m, n), generator=g).cuda()
    w = (1 + 0.1 * torch.randn(n, generator=g)).to(torch.bfloat16).cuda()
    y = K.gemm_blockscaled(a, b)  # both passes
    res_a, res_b = res0.clone(), res0.clone()
    h_ref, q_ref = separate(K, y, res_a, w, 1e-6, fmt)
    part = K.gemm_blockscaled_partials(a, b)
    assert part.splits == K.gemm_splits(m, n, k, fmt) and part.shape == (m, n)
    out = torch.empty_like(y)
    sync = torch.zeros(2, dtype=torch.int32, device="cuda")
    q = K.rmsnorm_quantize_rows(part, res_b, w, 1e-6, fmt, fresh_q(K, fmt, m, n), sync=sync if fmt == "nvfp4" else None, out=out)
    torch.cuda.synchronize()
    assert torch.equal(res_a, res_b), "residual differs"
    assert torch.equal(out, h_ref), "bf16 result differs"
    same_q(q, q_ref)


@pytest.mark.parametrize("fmt", ["mxfp8", "nvfp4"])
@pytest.mark.parametrize("m", [1, 64])
def test_stack_with_fused_rows_equals_the_block_by_block_stack_and_the_oracle(K, fmt, m):
    from tilefish_b200 import mlp as MLP

    h, f, layers = 1024, 8192, 3
    g = torch.Generator().manual_seed(5)
    blocks, host = [], []
    for _ in range(layers):
        w_gu = (torch.randn((2 * f, h), generator=g) * h**-0.5).to(torch.bfloat16)
        w_d = (torch.randn((h, f), generator=g) * f**-0.5).to(torch.bfloat16)
        w_n = (1 + 0.1 * torch.randn(h, generator=g)).to(torch.bfloat16)
        host.append((w_n, w_gu, w_d))
        blocks.append(MLP.quantize_weights(w_n.cuda(), w_gu.cuda(), w_d.cuda(), fmt))
    if K.gemm_splits(m, h, f, fmt) <= 1:
        pytest.skip("the planner does not split this shape")
    x = torch.randn((m, h), generator=g).to(torch.bfloat16)
    fused, plain = MLP.MlpStack(blocks), MLP.MlpStack(blocks, fuse_few_rows=False)
    assert fused._few_rows_applies(x.cuda())
    r1 = torch.zeros((m, h), device="cuda")
    r2 = torch.zeros((m, h), device="cuda")
    y1 = fused(x.cuda(), r1)
    y2 = plain(x.cuda(), r2)
    y1b = fused(x.cuda(), torch.zeros((m, h), device="cuda"))  # the cached buffers and the zeroed sync words serve a second call
    torch.cuda.synchronize()
    assert torch.equal(y1, y2) and torch.equal(r1, r2) and torch.equal(y1, y1b)
    # and the oracle's stack, at the tolerances of the other MLP tests
    xr, rr = x.clone(), torch.zeros((m, h))
    for w_n, w_gu, w_d in host:
        rr, xr = O.decoder_block(xr, rr, w_n, O.quantize(w_gu, fmt), O.quantize(w_d, fmt), fmt)
    got, ref = y1.cpu().float(), xr.float()
    assert float((got - ref).norm() / ref.norm()) <= 5e-2  # three blocks; measured 0.036 for nvfp4
    assert float((r1.cpu() - rr).norm() / rr.norm()) <= 1e-2


def test_refusals(K):
    from tilefish_b200.errors import TilefishError

    m, d = 200, 256  # more rows than SMs
    x = torch.zeros((m, d), dtype=torch.bfloat16, device="cuda")
    res = torch.zeros((m, d), device="cuda")
    w = torch.ones(d, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(TilefishError):
        K.rmsnorm_quantize_rows(x, res, w, 1e-6, "mxfp8", fresh_q(K, "mxfp8", m, d))
    a = K.quantize(torch.zeros((512, 256), dtype=torch.bfloat16, device="cuda"), "mxfp8")
    b = K.quantize(torch.zeros((256, 256), dtype=torch.bfloat16, device="cuda"), "mxfp8")
    with pytest.raises(TilefishError):  # not split along K
        K.gemm_blockscaled_partials(a, b)
