"""The no-allocation entry point against the ordinary one.

Some hosts cannot allocate device memory where they run the operator (an engine that owns the
whole device through its own pool, a plugin with a budget fixed at start-up, code that must not
trigger an allocation-induced synchronisation).  ``itk_fused_topk_static`` serves them: the
spill scratch comes from an array inside the library instead of from the caller.  This test
calls it through the C ABI twice in a row, on two different inputs, and requires the same
exact Top-2048 sets as ``itk_fused_topk`` with a caller-provided spill.  It is collected last
on purpose, and passes alone in a fresh process as well as after the other tests.
"""

from __future__ import annotations

import ctypes
import math
import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from fusedindextopk_b200 import _lib, operator  # noqa: E402
from fusedindextopk_b200.inputs import inputs_to, make_workload_inputs  # noqa: E402

pytestmark = pytest.mark.gpu


def _fused_args(ws, gpu, out_ids, flags, spill):
    args = _lib.FusedArgs()
    args.q, args.kv, args.kv_scales, args.weights = (_lib.ptr(t) for t in (gpu.q, gpu.kv, gpu.kv_scales, gpu.weights))
    args.k_start, args.k_end = _lib.ptr(gpu.k_start), _lib.ptr(gpu.k_end)
    args.thresholds = _lib.ptr(ws.thresholds)
    args.out_ids = _lib.ptr(out_ids)
    args.failure_flags = _lib.ptr(flags)
    args.spill = _lib.ptr(spill)
    args.status = _lib.ptr(ws.status)
    args.rows, args.keys = ws.rows, ws.keys
    args.key_lo, args.key_hi, args.shards = 0, ws.keys, 1
    args.block_begin, args.block_stride, args.num_blocks = 0, 1, (ws.rows + 3) // 4
    return args


def test_static_spill_variant_matches_the_allocating_entry_point():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    device = torch.device("cuda:0")
    library = _lib.load_library()
    stream = _lib.current_stream(torch, device)
    rows, keys = 64, 16384
    for call, (fixture, threshold) in enumerate((("A", None), ("B", -math.inf))):
        # fixture B with threshold -inf floods the candidate segments, so the spill is really used
        host = make_workload_inputs("c1", query_tokens=rows, context_tokens=keys if call == 0 else 8192, fixture_id=fixture)
        gpu = inputs_to(host, device)
        ws = operator.make_workspace(rows, host.case.context_tokens, device)
        tensors = (gpu.q, gpu.kv, gpu.kv_scales, gpu.weights, gpu.k_start, gpu.k_end)
        if threshold is None:
            operator.run_sample_thresholds(ws, *tensors)
        else:
            ws.thresholds.fill_(threshold)
        want_ids = torch.full((rows, 2048), -5, dtype=torch.int32, device=device)
        want_flags = torch.full((rows,), 9, dtype=torch.uint8, device=device)
        got_ids = torch.full((rows, 2048), -6, dtype=torch.int32, device=device)
        got_flags = torch.full((rows,), 8, dtype=torch.uint8, device=device)
        _lib.check(library.itk_fused_topk(ctypes.byref(_fused_args(ws, gpu, want_ids, want_flags, ws.spill_pairs)), stream))
        _lib.check(library.itk_fused_topk_static(ctypes.byref(_fused_args(ws, gpu, got_ids, got_flags, None)), stream))
        torch.cuda.synchronize()
        ws.check_status()
        assert torch.equal(got_flags, want_flags)
        assert int(want_flags.sum()) == 0
        assert torch.equal(got_ids.sort(dim=-1).values, want_ids.sort(dim=-1).values)
        assert int((got_ids >= 0).sum()) == rows * 2048


def test_static_variant_rejects_what_it_cannot_hold():
    library = _lib.load_library()
    args = _lib.FusedArgs()
    args.rows = _lib.STATIC_MAX_ROWS + 1
    args.shards = 1
    assert library.itk_fused_topk_static(ctypes.byref(args), None) == -1
    assert b"at most 256 query rows" in library.itk_last_error()
    args.rows = 8
    args.spill = 1234
    assert library.itk_fused_topk_static(ctypes.byref(args), None) == -1
    assert b"spill = null" in library.itk_last_error()
