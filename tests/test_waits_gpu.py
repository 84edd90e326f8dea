"""A bounded wait that runs out: the kernel returns, says so through the status word, the stream drains and the library
keeps working. Nothing here faults or hangs the GPU: the wait is on a counter nobody feeds, with its limit set to a few
milliseconds."""

import numpy as np
import pytest
import torch

from dromos_b200 import abi
from oracle import dromos_oracle as O
from tests import util

pytestmark = pytest.mark.gpu


def test_wait_for_arrivals_gives_up_and_reports(lx, monkeypatch):
    monkeypatch.setenv("LX_B200_WAIT_MS", "20")
    assert lx.lx_b200_last_error() == 0
    counter = torch.zeros(4, dtype=torch.int32, device="cuda")
    t0 = torch.cuda.Event(enable_timing=True)
    t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    assert lx.lx_b200_wait_arrivals(counter.data_ptr(), 3, util.stream_ptr()) == 0  # nobody will ever add the three arrivals
    t1.record()
    torch.cuda.synchronize()  # the stream drains: the wait gave up
    assert 15.0 <= t0.elapsed_time(t1) <= 500.0
    assert lx.lx_b200_last_error() == 5, "the wait that ran out was not reported"
    assert lx.lx_b200_last_error() == 0, "the status word was not cleared"
    assert int(counter[0].item()) == 0  # a wait that gives up takes nothing
    # a wait that IS fed returns at once and takes its arrivals
    counter[0] = 5
    assert lx.lx_b200_wait_arrivals(counter.data_ptr(), 3, util.stream_ptr()) == 0
    torch.cuda.synchronize()
    assert int(counter[0].item()) == 2 and lx.lx_b200_last_error() == 0
    # and the library still multiplies correctly afterwards
    N, K, M = 256, 1024, 3
    w_bits = util.bf16_normal((N, K), 0.02, 1)
    wt = util.make_weight(w_bits, O.W_FP8)
    dw = util.DeviceWeight(wt)
    x = util.bf16_normal((M, K), 1.0, 2)
    y = torch.full((M, N), float("nan"), device="cuda")
    assert util.gemv(lx, util.dev(x), abi.BF16, K, dw, y, abi.F32, N, M, N, K) == 0
    util.check_status(lx)
    util.assert_close(util.host(y), O.gemv_reference(O.bf16_bits_to_f32(x).astype(np.float64), wt), what="after a timed-out wait")
