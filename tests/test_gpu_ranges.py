"""Non-causal key ranges and odd shapes through the public callable (GPU).

The reference's standard inputs are causal prefill ranges; the operator contract
(`kernel/csrc/long_fused_bindings.cpp:119-153`) takes any `[k_start, k_end)` per row.
Seeded random windows and arbitrary ranges, with shapes that exercise ragged query
blocks, key counts that are not tile multiples, intra-GPU key shards and the CUDA-graph
replay of repeated calls.  The result must be an exact Top-K of the kernel's own dense
scores inside the row's range.
"""

from __future__ import annotations

import math
import random
import sys
from pathlib import Path

import pytest
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

from fusedindextopk_b200 import fused_index_topk, operator  # noqa: E402
from fusedindextopk_b200.inputs import inputs_to, make_workload_inputs  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def device():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda:0")


def _assert_exact(ids, logits, k_start, k_end, keys):
    out, scores = ids.cpu(), logits.cpu()
    for row in range(out.shape[0]):
        lo, hi = max(int(k_start[row]), 0), min(int(k_end[row]), keys)
        valid = max(hi - lo, 0)
        got = out[row][out[row] >= 0]
        assert got.numel() == min(valid, 2048), f"row {row}: {got.numel()} ids, want {min(valid, 2048)}"
        assert got.unique().numel() == got.numel(), f"row {row}: duplicate ids"
        if got.numel() == 0:
            continue
        assert int(got.min()) >= lo and int(got.max()) < hi, f"row {row}: id outside [{lo},{hi})"
        chosen = torch.zeros(keys, dtype=torch.bool)
        chosen[got.long()] = True
        inside = torch.zeros(keys, dtype=torch.bool)
        inside[lo:hi] = True
        rest = scores[row][inside & ~chosen]
        if rest.numel():
            assert float(scores[row][chosen].min()) >= float(rest.max()), f"row {row}: a better key was left out"


@pytest.mark.parametrize("seed", [3, 7, 11])
def test_random_ranges_and_shapes_are_exact(device, seed):
    rng = random.Random(seed)
    for _ in range(6):
        rows = rng.choice([1, 3, 5, 13, 31, 64, 100, 257])
        keys = rng.choice([2048, 2049, 3000, 5000, 8192, 12345, 20000, 40000])
        workload = rng.choice(["c0", "c1", "c3", "c4"])
        host = make_workload_inputs(workload, query_tokens=rows, context_tokens=keys, seed=rng.randrange(1 << 20))
        generator = torch.Generator().manual_seed(rng.randrange(1 << 30))
        mode = rng.choice(["causal", "window", "random"])
        if mode == "window":
            width = rng.randrange(1, keys + 1)
            start = torch.randint(0, keys - width + 1, (rows,), dtype=torch.int32, generator=generator)
            host.k_start, host.k_end = start, (start + width).to(torch.int32)
        elif mode == "random":
            a = torch.randint(0, keys + 1, (rows,), dtype=torch.int32, generator=generator)
            b = torch.randint(0, keys + 1, (rows,), dtype=torch.int32, generator=generator)
            host.k_start, host.k_end = torch.minimum(a, b), torch.maximum(a, b)
        gpu = inputs_to(host, device)
        tensors = (gpu.q, gpu.kv, gpu.kv_scales, gpu.weights, gpu.k_start, gpu.k_end)
        first = fused_index_topk(gpu.q, (gpu.kv, gpu.kv_scales), gpu.weights, gpu.k_start, gpu.k_end).clone()
        again = fused_index_topk(gpu.q, (gpu.kv, gpu.kv_scales), gpu.weights, gpu.k_start, gpu.k_end).clone()
        plain = operator.make_workspace(rows, keys, device, key_shards=1)
        operator.run_sample_thresholds(plain, *tensors)
        logits = torch.full((rows, keys), -math.inf, device=device)
        operator.run_fused_topk(plain, *tensors, diag_logits=logits, force_compute=True)
        torch.cuda.synchronize()
        plain.check_status()
        _assert_exact(first, logits, host.k_start, host.k_end, keys)
        _assert_exact(again, logits, host.k_start, host.k_end, keys)


def test_largest_key_count_the_library_accepts(device):
    """262144 keys (the 16-bit segment-relative candidate id limit), beyond the reference's 163840."""

    from fusedindextopk_b200 import _lib

    rows, keys = 6, _lib.MAX_KEYS
    host = make_workload_inputs("c1", query_tokens=rows, context_tokens=keys, seed=12)
    gpu = inputs_to(host, device)
    tensors = (gpu.q, gpu.kv, gpu.kv_scales, gpu.weights, gpu.k_start, gpu.k_end)
    ids = fused_index_topk(gpu.q, (gpu.kv, gpu.kv_scales), gpu.weights, gpu.k_start, gpu.k_end).clone()
    plain = operator.make_workspace(rows, keys, device, key_shards=1)
    assert plain.plan.sample_elements == 2048
    operator.run_sample_thresholds(plain, *tensors)
    logits = torch.full((rows, keys), -math.inf, device=device)
    operator.run_fused_topk(plain, *tensors, diag_logits=logits, force_compute=True)
    torch.cuda.synchronize()
    plain.check_status()
    _assert_exact(ids, logits, host.k_start, host.k_end, keys)
    with pytest.raises(ValueError):
        too_many = torch.empty((keys + 128, 128), dtype=torch.float8_e4m3fn, device=device)
        fused_index_topk(gpu.q, (too_many, torch.ones(keys + 128, device=device)), gpu.weights, gpu.k_start, gpu.k_end)
