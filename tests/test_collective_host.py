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
