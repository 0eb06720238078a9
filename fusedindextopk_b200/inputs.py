"""Seeded synthetic operator inputs.

Two recipes live here.

``make_prefill_inputs`` is the reference's own standard recipe
(``src/fused_index_topk/inputs.py:55-181``): bf16 normal sources scaled by
``1/sqrt(128)``, KV quantised row-wise to e4m3 with an fp32 scale
``max(amax,1e-4)/448``, Q cast directly to e4m3, fp32 weights ``N(0,1)/sqrt(64)``,
``k_start = 0`` and ``k_end[i] = N-Q+i+1``.  Generated on the CPU it yields the
same bytes as the reference's generator (pinned by a golden test).

``make_workload_inputs`` builds the five benchmark workloads (c0 .. c4 and the
short-Q variant of c3).  They stand in for the reference's real-corpus replay
tensors, which are not redistributed.  Everything is generated on the CPU with
named, independent ``torch.Generator`` streams so that the CPU oracle and the
GPU kernels see identical bytes; the stream seeds follow the reference's
derivation ``sha256("index-topk-prefill-v2:{seed}:{fixture}:{stream}")``.

The operator takes no query scale, so the per-(query, head) e4m3 scale of the
quantised queries is folded into ``weights`` before the call:
``weights[q,h] = w[q,h] * q_scale[q,h]``.
"""

from __future__ import annotations

import hashlib
import math
from dataclasses import dataclass
from typing import Any

from .api import PrefillCase, PrefillInputs

E4M3_MAX = 448.0
_REFERENCE_STREAMS = ("kv", "q", "weights")
_WORKLOAD_STREAMS = ("kv", "q", "weights", "kv_amp", "sinks", "tie_ids", "amp_rows")


def stream_seed(seed: int, fixture_id: str, stream: str) -> int:
    """63-bit seed of one named RNG stream of one fixture."""

    if fixture_id not in {"A", "B"}:
        raise ValueError("fixture_id must be 'A' or 'B'")
    material = f"index-topk-prefill-v2:{seed}:{fixture_id}:{stream}".encode()
    return int.from_bytes(hashlib.sha256(material).digest()[:8], "big") & ((1 << 63) - 1)


def input_stream_seeds(seed: int, fixture_id: str) -> dict[str, int]:
    """Seeds of the three streams the reference recipe uses."""

    return {name: stream_seed(seed, fixture_id, name) for name in _REFERENCE_STREAMS}


def _generator(torch: Any, seed: int) -> Any:
    generator = torch.Generator(device="cpu")
    generator.manual_seed(seed)
    return generator


def quantize_rows_e4m3(source: Any) -> tuple[Any, Any]:
    """Quantise the last dimension of ``source`` to e4m3 with one fp32 scale per row.

    ``scale = max(amax, 1e-4) / 448`` and ``value = (x / scale)`` rounded to
    e4m3 (``src/fused_index_topk/inputs.py:76-90``).
    """

    import torch

    scales = source.abs().float().amax(dim=-1).clamp_min(1e-4) / E4M3_MAX
    values = (source.float() / scales.unsqueeze(-1)).to(torch.float8_e4m3fn)
    return values.contiguous(), scales.contiguous()


def causal_ranges(torch: Any, query_tokens: int, context_tokens: int, device: Any = "cpu"):
    """``k_start = 0`` and end-exclusive ``k_end[i] = N - Q + i + 1`` as int32."""

    k_start = torch.zeros(query_tokens, device=device, dtype=torch.int32)
    k_end = torch.arange(
        context_tokens - query_tokens + 1, context_tokens + 1, device=device, dtype=torch.int32
    )
    return k_start, k_end


def make_prefill_inputs(case: PrefillCase, device: Any = "cpu", *, fixture_id: str = "A") -> PrefillInputs:
    """The reference's standard recipe, generated on the CPU, then moved to ``device``."""

    import torch

    if case.batch_size != 1 or not case.causal:
        raise ValueError("the prefill contract supports batch_size=1 causal cases only")
    if case.query_tokens <= 0 or case.context_tokens < case.query_tokens:
        raise ValueError("need 0 < query_tokens <= context_tokens")
    seeds = input_stream_seeds(case.seed, fixture_id)
    kv_source = torch.randn(
        (case.context_tokens, case.head_dim), dtype=torch.bfloat16,
        generator=_generator(torch, seeds["kv"]),
    ) / math.sqrt(case.head_dim)
    kv, kv_scales = quantize_rows_e4m3(kv_source)
    q = (
        torch.randn(
            (case.query_tokens, case.indexer_heads, case.head_dim), dtype=torch.bfloat16,
            generator=_generator(torch, seeds["q"]),
        ) / math.sqrt(case.head_dim)
    ).to(torch.float8_e4m3fn).contiguous()
    weights = (
        torch.randn(
            (case.query_tokens, case.indexer_heads), dtype=torch.float32,
            generator=_generator(torch, seeds["weights"]),
        ) / math.sqrt(case.indexer_heads)
    ).contiguous()
    k_start, k_end = causal_ranges(torch, case.query_tokens, case.context_tokens)
    target = torch.device(device)
    return PrefillInputs(
        case=case,
        q=q.to(target), kv=kv.to(target), kv_scales=kv_scales.to(target),
        weights=weights.to(target), k_start=k_start.to(target), k_end=k_end.to(target),
        generation_context_tokens=case.context_tokens,
        fixture_id=fixture_id,
        stream_seeds=seeds,
    )


@dataclass(frozen=True)
class Workload:
    """Shape and generator switches of one benchmark workload."""

    name: str
    query_tokens: int
    context_tokens: int
    sink_keys: int = 0
    tie_vectors: int = 0
    amplified_row_fraction: float = 0.0
    description: str = ""


WORKLOADS: dict[str, Workload] = {
    "c0": Workload("c0", 8, 8192, description="CPU plumbing case"),
    "c1": Workload("c1", 4096, 16384, sink_keys=16, description="single-request prefill"),
    "c2": Workload("c2", 4096, 65536, sink_keys=16, description="long-context prefill"),
    "c3": Workload("c3", 4096, 163840, sink_keys=16, description="max-context prefill"),
    "c3s": Workload("c3s", 64, 131072, sink_keys=16, description="short-Q long context"),
    "c4": Workload("c4", 512, 32768, tie_vectors=16, amplified_row_fraction=0.10,
                   description="tie / repair stress"),
}


def workload_case(workload: Workload, seed: int = 0, top_k: int = 2048) -> PrefillCase:
    return PrefillCase(
        case_id=f"{workload.name}_q{workload.query_tokens}_n{workload.context_tokens}",
        query_tokens=workload.query_tokens,
        context_tokens=workload.context_tokens,
        top_k=top_k,
        seed=seed,
    )


def make_workload_inputs(
    workload: Workload | str,
    *,
    seed: int = 0,
    fixture_id: str = "A",
    device: Any = "cpu",
    query_tokens: int | None = None,
    context_tokens: int | None = None,
) -> PrefillInputs:
    """Generate one benchmark workload; ``query_tokens``/``context_tokens`` scale it down.

    * queries: ``N(0,1)`` per element, quantised per (query, head) row; the
      row scale is folded into the weights;
    * keys: ``N(0,1) * LogNormal(0, 0.5)`` with one amplitude per token,
      quantised per token;
    * ``sink_keys`` keys at positions uniform over the first 1 % of the
      context get 8x amplitude before quantisation (heavy-tailed scores);
    * ``tie_vectors = V``: keys are drawn from only ``V`` distinct quantised
      vectors (uniform assignment, scale tied to the vector) and the
      unfolded weights are the constant ``64**-0.5``, which makes scores tie
      exactly; ``amplified_row_fraction`` of the query rows get 4x amplitude.
    """

    import torch

    if isinstance(workload, str):
        workload = WORKLOADS[workload]
    if query_tokens is not None or context_tokens is not None:
        workload = Workload(
            workload.name,
            int(query_tokens if query_tokens is not None else workload.query_tokens),
            int(context_tokens if context_tokens is not None else workload.context_tokens),
            workload.sink_keys, workload.tie_vectors, workload.amplified_row_fraction,
            workload.description,
        )
    case = workload_case(workload, seed)
    rows, keys, heads, dim = case.query_tokens, case.context_tokens, case.indexer_heads, case.head_dim
    if rows <= 0 or keys < rows:
        raise ValueError("need 0 < query_tokens <= context_tokens")
    seeds = {name: stream_seed(seed, fixture_id, name) for name in _WORKLOAD_STREAMS}

    # keys
    if workload.tie_vectors:
        base = torch.randn((workload.tie_vectors, dim), generator=_generator(torch, seeds["kv"]))
        amplitude = torch.exp(
            0.5 * torch.randn((workload.tie_vectors, 1), generator=_generator(torch, seeds["kv_amp"]))
        )
        base_values, base_scales = quantize_rows_e4m3(base * amplitude)
        assignment = torch.randint(
            0, workload.tie_vectors, (keys,), generator=_generator(torch, seeds["tie_ids"])
        )
        kv = base_values.view(torch.uint8)[assignment].view(torch.float8_e4m3fn).contiguous()
        kv_scales = base_scales[assignment].contiguous()
    else:
        source = torch.randn((keys, dim), generator=_generator(torch, seeds["kv"]))
        amplitude = torch.exp(
            0.5 * torch.randn((keys, 1), generator=_generator(torch, seeds["kv_amp"]))
        )
        source = source * amplitude
        if workload.sink_keys:
            span = max(1, keys // 100)
            positions = torch.randint(
                0, span, (workload.sink_keys,), generator=_generator(torch, seeds["sinks"])
            )
            source[positions] *= 8.0
        kv, kv_scales = quantize_rows_e4m3(source)

    # queries and weights
    q_source = torch.randn((rows, heads, dim), generator=_generator(torch, seeds["q"]))
    if workload.amplified_row_fraction > 0:
        chosen = torch.rand(rows, generator=_generator(torch, seeds["amp_rows"]))
        q_source[chosen < workload.amplified_row_fraction] *= 4.0
    q, q_scales = quantize_rows_e4m3(q_source)
    del q_source
    if workload.tie_vectors:
        raw_weights = torch.full((rows, heads), float(heads) ** -0.5, dtype=torch.float32)
    else:
        raw_weights = torch.randn((rows, heads), generator=_generator(torch, seeds["weights"]))
        raw_weights = raw_weights * (float(heads) ** -0.5) * (float(dim) ** -0.5)
    weights = (raw_weights * q_scales).to(torch.float32).contiguous()

    k_start, k_end = causal_ranges(torch, rows, keys)
    target = torch.device(device)
    return PrefillInputs(
        case=case,
        q=q.to(target), kv=kv.to(target), kv_scales=kv_scales.to(target),
        weights=weights.to(target), k_start=k_start.to(target), k_end=k_end.to(target),
        generation_context_tokens=keys,
        fixture_id=fixture_id,
        stream_seeds=seeds,
        recipe_version="b200-workload-fp8-v1",
        recipe_metadata={
            "workload": workload.name,
            "sink_keys": workload.sink_keys,
            "tie_vectors": workload.tie_vectors,
            "amplified_row_fraction": workload.amplified_row_fraction,
            "q_scale_folded_into_weights": True,
        },
    )


def inputs_to(inputs: PrefillInputs, device: Any, *, non_blocking: bool = False) -> PrefillInputs:
    """Copy of ``inputs`` whose six tensors live on ``device``."""

    from dataclasses import replace

    moved = {
        name: getattr(inputs, name).to(device, non_blocking=non_blocking)
        for name in ("q", "kv", "kv_scales", "weights", "k_start", "k_end")
    }
    return replace(inputs, **moved)
