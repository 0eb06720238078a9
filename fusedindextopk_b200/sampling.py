"""Host-side arithmetic of the sampled-threshold prepass.

Three small integer/float64 functions decide, before any kernel runs, how many
keys are sampled, which descending rank of the sampled scores becomes the
per-row threshold, and which key positions are sampled.  They restate

* ``production_sample_elements`` / ``long_context_sample_elements``
  (``src/fused_index_topk/kernel/plugin.py:42-64``),
* ``guarded_sample_rank`` (``src/fused_index_topk/kernel/sampling.py:25-46``),
* ``common_random_sample_ids`` (``src/fused_index_topk/kernel/sampling.py:49-64``)
  and the seed mix at ``src/fused_index_topk/kernel/plugin.py:31,194``.

The threshold only steers how much work the fused kernel keeps on chip; the
selected Top-K set never depends on it.
"""

from __future__ import annotations

import math
from typing import Any

TOP_K = 2048
TARGET_CANDIDATES = 2816
REPAIR_CHUNK_ELEMENTS = 16384
MAX_CONTEXT = 163840
SAMPLING_SEED_XOR = 0x4655534544523549


def long_context_sample_elements(context_tokens: int) -> int:
    """Sample size for contexts above one repair chunk (N > 16384)."""

    if context_tokens <= REPAIR_CHUNK_ELEMENTS:
        raise ValueError("long-context sampling requires N > 16384")
    if context_tokens <= 32768:
        wanted = 512
    elif context_tokens <= 65536:
        wanted = 1024
    else:
        # three samples per 256 keys, rounded up to whole 256-sample groups
        proportional = (context_tokens * 3 + 255) // 256
        wanted = max(1024, (proportional + 255) // 256 * 256)
    return min(context_tokens, wanted)


def production_sample_elements(context_tokens: int) -> int:
    """Sample size S(N) of the released schedule: 512 below 16 K, 256 at 16 K."""

    if context_tokens == REPAIR_CHUNK_ELEMENTS:
        return 256
    if context_tokens < REPAIR_CHUNK_ELEMENTS:
        return min(context_tokens, 512)
    return long_context_sample_elements(context_tokens)


def guarded_sample_rank(
    sample_elements: int,
    context_tokens: int,
    *,
    target_candidates: int = 3072,
    guard_sigmas: float = 2.0,
) -> int:
    """Descending rank (1-based) of the sampled score used as threshold.

    With ``p = target/N`` the number of sampled keys inside the true top
    ``target`` is Binomial(S, p); the rank is its mean plus ``guard_sigmas``
    standard deviations, clamped to ``[1, S]``, so that the threshold errs on
    the low (more candidates) side.
    """

    if not 0 < target_candidates <= context_tokens:
        raise ValueError("target_candidates must lie in [1, context_tokens]")
    if not 0 < sample_elements <= context_tokens:
        raise ValueError("sample_elements must lie in [1, context_tokens]")
    if guard_sigmas < 0 or not math.isfinite(guard_sigmas):
        raise ValueError("guard_sigmas must be finite and non-negative")
    p = target_candidates / context_tokens
    mean = sample_elements * p
    sigma = math.sqrt(sample_elements * p * (1.0 - p))
    return max(1, min(sample_elements, math.ceil(mean + guard_sigmas * sigma)))


def sampling_seed(case_seed: int) -> int:
    """Seed of the sample-position stream, derived from the case seed."""

    return (int(case_seed) ^ SAMPLING_SEED_XOR) & ((1 << 63) - 1)


def common_random_sample_ids(
    torch: Any,
    context_tokens: int,
    sample_elements: int,
    *,
    seed: int,
    device: Any,
) -> Any:
    """First S entries of a seeded CPU permutation of ``range(N)``, sorted, int32."""

    generator = torch.Generator(device="cpu")
    generator.manual_seed(int(seed))
    permutation = torch.randperm(
        context_tokens, generator=generator, device="cpu", dtype=torch.int64
    )
    chosen = torch.sort(permutation[:sample_elements]).values
    return chosen.to(device=device, dtype=torch.int32).contiguous()
