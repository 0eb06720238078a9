"""The bounded waits of the fused kernel: a wait that runs out makes the kernel return, not hang.

The failure is made without faulting anything: the diagnostic build is told to issue no load at all
(``withhold_loads``), so its first wait (for the query tile) meets its time limit, set to one
millisecond here.  The kernel must come back with bit 0 of the status word set, the host check must
raise, and the next ordinary call on the same context must be correct.
"""

from __future__ import annotations

import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from fusedindextopk_b200 import _lib, operator  # noqa: E402
from fusedindextopk_b200.api import PrefillCase  # noqa: E402
from fusedindextopk_b200.correctness import validate_topk_indices  # noqa: E402
from fusedindextopk_b200.inputs import inputs_to, make_workload_inputs  # noqa: E402

pytestmark = pytest.mark.gpu


def test_expired_wait_sets_the_status_bit_and_the_context_stays_usable():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    device = torch.device("cuda:0")
    host = make_workload_inputs("c0", query_tokens=8, context_tokens=8192)
    gpu = inputs_to(host, device)
    tensors = (gpu.q, gpu.kv, gpu.kv_scales, gpu.weights, gpu.k_start, gpu.k_end)
    ws = operator.make_workspace(8, 8192, device)
    operator.run_sample_thresholds(ws, *tensors)
    trace = torch.zeros((148, 32), dtype=torch.int64, device=device)   # selects the diagnostic build

    started = torch.cuda.Event(enable_timing=True)
    ended = torch.cuda.Event(enable_timing=True)
    started.record()
    operator.run_fused_topk(ws, *tensors, trace=trace, wait_limit_ns=1_000_000, withhold_loads=True)
    ended.record()
    torch.cuda.synchronize()
    assert started.elapsed_time(ended) < 500.0, "the kernel must return soon after the limit"
    assert int(ws.status.item()) & _lib.STATUS_WAIT_EXPIRED
    with pytest.raises(_lib.ItkError):
        ws.check_status()

    ws.status.zero_()
    ids = operator.run_operator(ws, *tensors)
    torch.cuda.synchronize()
    ws.check_status()
    assert int(ws.failure_flags.sum()) == 0
    validate_topk_indices(ids.unsqueeze(1).contiguous().cpu(), PrefillCase("after-expiry", 8, 8192, 2048, 0))
