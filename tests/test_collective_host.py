"""Host-side logic of the exchange classes that needs no GPU: the error word of a bounded wait becomes an exception that says what
happened and what to do, and the non-synchronizing poll reads the sticky word."""

import pytest
import torch

from tilefish_b200 import TilefishRuntimeError
from tilefish_b200.collective import PeerAllReduce


def _bare(channels=2):
    peer = object.__new__(PeerAllReduce)
    peer.channels = channels
    peer._poll_host = torch.zeros(channels, dtype=torch.int64)
    return peer


def test_error_words_map_to_exceptions():
    assert PeerAllReduce.describe_error(0) == "healthy"
    assert "peer never arrived" in PeerAllReduce.describe_error(2) and "grid barrier" in PeerAllReduce.describe_error(1)
    peer = _bare()
    assert peer.last_error() == 0
    peer.raise_if_failed("step 3")  # healthy: no exception
    peer._poll_host[1] = 2
    assert peer.last_error() == 2
    with pytest.raises(TilefishRuntimeError, match=r"step 3.*peer never arrived.*reset\(\)"):
        peer.raise_if_failed("step 3")
    peer._poll_host[0] = 1  # the first nonzero channel wins
    with pytest.raises(TilefishRuntimeError, match="grid barrier"):
        peer.raise_if_failed()


def test_stack_surfaces_a_failed_exchange_before_the_next_forward():
    from tilefish_b200 import mlp as MLP

    stack = MLP.MlpStack([], comm="all_reduce")
    stack._peer = _bare()
    stack._peer._poll_host[0] = 2
    with pytest.raises(TilefishRuntimeError, match="MlpStack comm="):
        stack.forward(None, None)
    cap = MLP.CapturedStack(None, None, None, None, stack)
    with pytest.raises(TilefishRuntimeError, match="captured MlpStack"):
        cap.replay(check=True)


def test_few_rows_path_is_chosen_only_where_it_applies(monkeypatch):
    """MlpStack takes the one-launch decode step only on one GPU, for at most 128 rows, equal blocks and a second GEMM that the planner
    splits along K; the decision needs no GPU (the planner's answer is stubbed)."""
    from types import SimpleNamespace

    from tilefish_b200 import kernels as K
    from tilefish_b200 import mlp as MLP

    def block(h=8192, f=28672, fmt="nvfp4"):
        return SimpleNamespace(fmt=fmt, w_d=SimpleNamespace(shape=(h, f)), w_gu=SimpleNamespace(shape=(2 * f, h)))

    asked = []

    def splits(m, n, k, fmt, epilogue="none"):
        asked.append((m, n, k, fmt))
        return 4 if m <= 64 else 1

    monkeypatch.setattr(K, "gemm_splits", splits)
    x = SimpleNamespace(shape=(64, 8192), dim=lambda: 2)
    stack = MLP.MlpStack([block(), block()])
    assert stack._few_rows_applies(x) and asked[-1] == (64, 8192, 28672, "nvfp4")
    assert not stack._few_rows_applies(SimpleNamespace(shape=(128, 8192), dim=lambda: 2))  # the planner does not split 128 rows here
    assert not stack._few_rows_applies(SimpleNamespace(shape=(256, 8192), dim=lambda: 2))  # more rows than the kernel takes
    assert not stack._few_rows_applies(SimpleNamespace(shape=(64, 8200), dim=lambda: 2))   # H not a multiple of 32
    assert not MLP.MlpStack([block(), block(f=14336)])._few_rows_applies(x)               # blocks of different shapes
    assert not MLP.MlpStack([block(), block()], fuse_few_rows=False)._few_rows_applies(x)
    assert not MLP.MlpStack([])._few_rows_applies(x)


def test_row_kernels_refuse_host_tensors():
    """No CPU path: a host tensor is refused before anything is launched."""
    from tilefish_b200 import TilefishPreconditionError
    from tilefish_b200 import kernels as K

    res = torch.zeros((4, 64))
    w = torch.ones(64, dtype=torch.bfloat16)
    q = K.BlockScaledTensor("mxfp8", (4, 64), torch.empty((4, 64), dtype=torch.uint8), torch.zeros(512, dtype=torch.uint8), None, "swizzled")
    with pytest.raises(TilefishPreconditionError, match="CUDA only"):
        K.rmsnorm_quantize_rows(torch.zeros((4, 64), dtype=torch.bfloat16), res, w, 1e-6, "mxfp8", q)
    with pytest.raises(TilefishPreconditionError, match="CUDA only"):
        K.residual_add_rmsnorm(torch.zeros((4, 64), dtype=torch.bfloat16), res, w)
