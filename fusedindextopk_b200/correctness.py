"""Output-contract and exact-Top-K checks for the operator's ``[Q,1,K]`` indices.

Same entry points, argument meaning and error behaviour as the reference's
``src/fused_index_topk/correctness.py`` (``validate_topk_indices`` :278-362,
``compare_topk_indices`` :365-478, ``build_score_threshold_oracle`` :15-173),
written independently:

* the output contract: int32, contiguous, shape ``[Q,1,K]``; row ``i`` may use
  ids in ``[0, N-Q+i+1)`` only, each at most once, exactly
  ``min(K, N-Q+i+1)`` of them, and ``-1`` in every remaining slot;
* the tie rule (``exact_score_threshold``): an exact Top-K is a set only up to
  keys whose score equals the K-th largest score.  A row is exact when it
  holds every key scoring above that cutoff, none scoring below it, and as
  many keys at the cutoff as are needed to reach K.

``score_threshold_check`` applies the tie rule directly to dense scores and
``tolerance_set_report`` does the accounting for comparisons against scores
that are only known to a tolerance.
"""

from __future__ import annotations

from collections.abc import Mapping
from typing import Any

from .api import PrefillCase


class CorrectnessError(AssertionError):
    """An operator result violates the output contract or is not an exact Top-K."""


# --------------------------------------------------------------------------- helpers


def _is_torch(value: object) -> bool:
    return type(value).__module__.split(".")[0] == "torch" and hasattr(value, "device")


def _dtype_name(value: object) -> str:
    dtype = getattr(value, "dtype", None)
    if dtype is None:
        raise CorrectnessError("indices must expose a dtype attribute")
    return str(dtype).lower().rsplit(".", 1)[-1]


def _contiguous(value: object) -> bool:
    probe = getattr(value, "is_contiguous", None)
    if callable(probe):
        return bool(probe())
    flags = getattr(value, "flags", None)
    if flags is not None and hasattr(flags, "c_contiguous"):
        return bool(flags.c_contiguous)
    raise CorrectnessError("indices must expose is_contiguous() or C-contiguous flags")


def _check_header(indices: object, case: PrefillCase, name: str) -> None:
    if not case.causal:
        raise CorrectnessError("the correctness contract requires a causal Prefill case")
    shape = getattr(indices, "shape", None)
    if shape is None:
        raise CorrectnessError("indices must expose a shape attribute")
    actual = tuple(int(extent) for extent in shape)
    wanted = (case.query_tokens, 1, case.top_k)
    if actual != wanted:
        raise CorrectnessError(f"{name} shape must be {wanted}, received {actual}")
    if _dtype_name(indices) != "int32":
        raise CorrectnessError(f"{name} dtype must be int32")
    if not _contiguous(indices):
        raise CorrectnessError(f"{name} must be contiguous")


def _row_sets(indices: object, case: PrefillCase, name: str) -> list[frozenset[int]]:
    """Generic (nested-list) validation; returns the set of valid ids per row."""

    _check_header(indices, case, name)
    data: Any = indices
    for hop in ("detach", "cpu"):
        method = getattr(data, hop, None)
        if callable(method):
            data = method()
    if not callable(getattr(data, "tolist", None)):
        raise CorrectnessError("indices must expose tolist()")
    nested = data.tolist()
    if not isinstance(nested, list) or len(nested) != case.query_tokens:
        raise CorrectnessError(f"{name}.tolist() is inconsistent with its shape")
    sets: list[frozenset[int]] = []
    for row_index, groups in enumerate(nested):
        if not isinstance(groups, list) or len(groups) != 1:
            raise CorrectnessError(f"{name} row {row_index} must contain one index group")
        row = groups[0]
        if not isinstance(row, list) or len(row) != case.top_k:
            raise CorrectnessError(f"{name} row {row_index} has an invalid materialized width")
        if any(isinstance(item, bool) or not isinstance(item, int) for item in row):
            raise CorrectnessError(f"{name} row {row_index} contains a non-integer ID")
        causal_end = case.query_start + row_index + 1
        bad_negative = [item for item in row if item < -1]
        if bad_negative:
            raise CorrectnessError(
                f"{name} row {row_index} contains invalid negative IDs: {bad_negative[:4]}"
            )
        kept = [item for item in row if item != -1]
        wanted = min(case.top_k, causal_end)
        if len(kept) != wanted:
            raise CorrectnessError(
                f"{name} row {row_index} expected {wanted} valid IDs and "
                f"{case.top_k - wanted} -1 slots, received {len(kept)} valid IDs"
            )
        outside = [item for item in kept if item >= causal_end]
        if outside:
            raise CorrectnessError(
                f"{name} row {row_index} contains IDs outside [0, {causal_end}): {outside[:4]}"
            )
        unique = frozenset(kept)
        if len(unique) != len(kept):
            raise CorrectnessError(f"{name} row {row_index} contains duplicate valid IDs")
        sets.append(unique)
    return sets


def _causal_ends(torch: Any, case: PrefillCase, device: Any) -> Any:
    return torch.arange(
        case.query_start + 1, case.context_tokens + 1, device=device, dtype=torch.int64
    )


def _validate_tensor(indices: Any, case: PrefillCase, name: str) -> dict[str, Any]:
    """Vectorised validation of a torch tensor (CPU or CUDA)."""

    import torch

    _check_header(indices, case, name)
    rows = indices[:, 0, :]
    if bool((rows < -1).any()):
        raise CorrectnessError(f"{name} contains a negative ID other than -1")
    present = rows >= 0
    ends = _causal_ends(torch, case, rows.device)
    wanted = ends.clamp(max=case.top_k)
    counts = present.sum(dim=1)
    wrong = (counts != wanted).nonzero()
    if wrong.numel():
        row = int(wrong[0])
        raise CorrectnessError(
            f"{name} row {row} expected {int(wanted[row])} valid IDs, received {int(counts[row])}"
        )
    outside = (present & (rows.to(torch.int64) >= ends[:, None])).nonzero()
    if outside.numel():
        row, column = int(outside[0, 0]), int(outside[0, 1])
        raise CorrectnessError(
            f"{name} row {row} ID {int(rows[row, column])} is outside [0, {int(ends[row])})"
        )
    big = torch.iinfo(torch.int32).max
    ordered = torch.sort(torch.where(present, rows, torch.full_like(rows, big)), dim=1).values
    repeated = ((ordered[:, 1:] == ordered[:, :-1]) & (ordered[:, 1:] != big)).nonzero()
    if repeated.numel():
        raise CorrectnessError(f"{name} row {int(repeated[0, 0])} contains duplicate valid IDs")
    total = int(counts.sum())
    return _summary(case, total)


def _summary(case: PrefillCase, valid_total: int) -> dict[str, Any]:
    return {
        "status": "passed",
        "rows": case.query_tokens,
        "top_k": case.top_k,
        "valid_ids": valid_total,
        "padding_ids": case.query_tokens * case.top_k - valid_total,
        "dtype": "int32",
        "contiguous": True,
    }


# --------------------------------------------------------------------------- public API


def validate_topk_indices(indices: object, case: PrefillCase, *, name: str = "indices") -> dict[str, Any]:
    """Check shape, dtype, layout, causal bounds, ``-1`` padding and uniqueness."""

    if _is_torch(indices):
        return _validate_tensor(indices, case, name)
    sets = _row_sets(indices, case, name)
    return _summary(case, sum(len(row) for row in sets))


def _tensor_row_sets(torch: Any, tensor: Any, row: int) -> frozenset[int]:
    values = tensor[row, 0].to(device="cpu", dtype=torch.int64).tolist()
    return frozenset(int(item) for item in values if item >= 0)


def _judge_differing_row(
    row: int,
    actual: frozenset[int],
    expected: frozenset[int],
    cutoff_tie_rows: Mapping[int, Mapping[str, Any]] | None,
) -> None:
    tie = None if cutoff_tie_rows is None else cutoff_tie_rows.get(row)
    if tie is None:
        raise CorrectnessError(
            f"candidate row {row} differs from baseline; "
            f"missing={sorted(expected - actual)[:8]}, unexpected={sorted(actual - expected)[:8]}"
        )
    boundary = frozenset(int(item) for item in tie["boundary_ids"])
    above = expected - boundary
    lost = sorted(above - actual)
    below = sorted(actual - above - boundary)
    needed = int(tie["required_boundary_selections"])
    taken = len(actual & boundary)
    if lost or below or taken != needed:
        raise CorrectnessError(
            f"candidate row {row} is not an exact score-threshold TopK; "
            f"missing_above_cutoff={lost[:8]}, below_cutoff={below[:8]}, "
            f"selected_at_cutoff={taken}, required_at_cutoff={needed}"
        )


def compare_topk_indices(
    candidate: object,
    baseline: object,
    case: PrefillCase,
    *,
    cutoff_tie_rows: Mapping[int, Mapping[str, Any]] | None = None,
) -> dict[str, Any]:
    """Compare two results as unordered per-row id sets.

    A row that differs is accepted only when ``cutoff_tie_rows`` describes a
    cutoff tie for it and the candidate merely substitutes keys scoring exactly
    at the cutoff.
    """

    mode = (
        "unordered_exact_topk_score_threshold" if cutoff_tie_rows is not None
        else "unordered_exact_id_set"
    )
    substituted = 0
    if _is_torch(candidate) and _is_torch(baseline):
        import torch

        _validate_tensor(candidate, case, "candidate")
        _validate_tensor(baseline, case, "baseline")
        big = torch.iinfo(torch.int32).max

        def canonical(tensor: Any) -> Any:
            rows = tensor[:, 0, :]
            return torch.sort(torch.where(rows >= 0, rows, torch.full_like(rows, big)), dim=1).values

        differing = (canonical(candidate) != canonical(baseline)).any(dim=1).nonzero().flatten().tolist()
        for row in differing:
            _judge_differing_row(
                int(row),
                _tensor_row_sets(torch, candidate, int(row)),
                _tensor_row_sets(torch, baseline, int(row)),
                cutoff_tie_rows,
            )
        substituted = len(differing)
    else:
        actual_sets = _row_sets(candidate, case, "candidate")
        expected_sets = _row_sets(baseline, case, "baseline")
        for row, (actual, expected) in enumerate(zip(actual_sets, expected_sets)):
            if actual != expected:
                _judge_differing_row(row, actual, expected, cutoff_tie_rows)
                substituted += 1
    return {
        "status": "passed",
        "rows_compared": case.query_tokens,
        "comparison": mode,
        "cutoff_tie_rows_available": len(cutoff_tie_rows or {}),
        "cutoff_tie_rows_substituted": substituted,
    }


def build_score_threshold_oracle(
    scores: object, baseline_indices: object, case: PrefillCase
) -> tuple[dict[str, Any], dict[int, dict[str, Any]]]:
    """Derive the tie description of every row whose K-th and (K+1)-th scores tie.

    ``scores`` is the dense fp32 ``[Q,N]`` matrix (``-inf`` outside the causal
    range) that produced ``baseline_indices``.  The baseline itself is checked
    against the tie rule on the way.
    """

    import torch

    if not isinstance(scores, torch.Tensor):
        raise CorrectnessError("baseline scores must be a torch.Tensor")
    wanted = (case.query_tokens, case.context_tokens)
    if tuple(scores.shape) != wanted:
        raise CorrectnessError(
            f"baseline scores shape must be {wanted}, received {tuple(scores.shape)}"
        )
    if scores.dtype != torch.float32:
        raise CorrectnessError("baseline scores must use float32")
    validate_topk_indices(baseline_indices, case, name="baseline cutoff oracle")

    ends = _causal_ends(torch, case, scores.device)
    eligible = ends > case.top_k
    checked = int(eligible.sum())
    skipped = case.query_tokens - checked
    if checked == 0:
        return (
            {
                "status": "passed", "policy": "exact_score_threshold", "rows_checked": 0,
                "reference_selection_rows_validated": 0,
                "rows_skipped_valid_count_le_k": skipped, "rows_with_cutoff_ties": 0,
                "minimum_cutoff_margin": None, "minimum_positive_cutoff_margin": None,
                "tie_rows": [],
            },
            {},
        )
    if case.context_tokens <= case.top_k:
        raise CorrectnessError("eligible cutoff rows require N > K")
    leading = torch.topk(scores, case.top_k + 1, dim=-1, largest=True, sorted=True).values[eligible]
    cutoff = leading[:, case.top_k - 1]
    runner_up = leading[:, case.top_k]
    if not bool(torch.isfinite(cutoff).all() and torch.isfinite(runner_up).all()):
        raise CorrectnessError("eligible TopK cutoff scores must be finite")
    margin = cutoff - runner_up
    if bool((margin < 0).any()):
        raise CorrectnessError("TopK cutoff values are not monotonically ordered")
    row_ids = eligible.nonzero().flatten()
    chosen = baseline_indices[:, 0, :][eligible].to(torch.int64)
    chosen_scores = scores[eligible].gather(1, chosen)
    low = (chosen_scores < cutoff[:, None]).nonzero()
    if low.numel():
        raise CorrectnessError(
            f"exact reference row {int(row_ids[int(low[0, 0])])} selected an ID below the TopK cutoff"
        )
    above_total = (leading[:, : case.top_k] > cutoff[:, None]).sum(dim=1)
    above_chosen = (chosen_scores > cutoff[:, None]).sum(dim=1)
    short = (above_total != above_chosen).nonzero()
    if short.numel():
        raise CorrectnessError(
            f"exact reference row {int(row_ids[int(short[0])])} omitted an ID above the TopK cutoff"
        )

    tie_rows: dict[int, dict[str, Any]] = {}
    reports: list[dict[str, Any]] = []
    for position in (margin == 0).nonzero().flatten().tolist():
        row = int(row_ids[position])
        end = int(ends[row])
        value = cutoff[position]
        live = scores[row, :end]
        at_cutoff = (live == value).nonzero().flatten().to("cpu", torch.int64).tolist()
        greater = int((live > value).sum())
        needed = case.top_k - greater
        picked = _tensor_row_sets(torch, baseline_indices, row)
        at_cutoff_set = set(at_cutoff)
        if len(picked) != case.top_k:
            raise CorrectnessError(f"baseline cutoff oracle row {row} has invalid width")
        if len(picked - at_cutoff_set) != greater:
            raise CorrectnessError(
                f"baseline cutoff oracle row {row} omitted a score above the cutoff"
            )
        if len(picked & at_cutoff_set) != needed:
            raise CorrectnessError(
                f"baseline cutoff oracle row {row} selected an invalid number of tied IDs"
            )
        if len(at_cutoff) <= needed:
            raise CorrectnessError(
                f"baseline cutoff oracle row {row} was marked tied without alternatives"
            )
        tie_rows[row] = {
            "boundary_ids": tuple(int(item) for item in at_cutoff),
            "required_boundary_selections": needed,
            "strictly_greater_count": greater,
        }
        reports.append(
            {
                "row": row, "causal_end": end, "cutoff_score": float(value),
                "boundary_candidate_count": len(at_cutoff),
                "required_boundary_selections": needed,
                "strictly_greater_count": greater,
            }
        )
    positive = margin[margin > 0]
    summary = {
        "status": "passed",
        "policy": "exact_score_threshold",
        "rows_checked": checked,
        "reference_selection_rows_validated": checked,
        "rows_skipped_valid_count_le_k": skipped,
        "minimum_cutoff_margin": float(margin.min()),
        "minimum_positive_cutoff_margin": float(positive.min()) if positive.numel() else None,
        "rows_with_cutoff_ties": len(tie_rows),
        "tie_rows": reports,
    }
    return summary, tie_rows


def score_threshold_check(indices: Any, scores: Any, case: PrefillCase, *, name: str = "indices") -> dict[str, Any]:
    """Apply the tie rule directly: is ``indices`` an exact Top-K of ``scores``?

    ``scores`` is dense fp32 ``[Q,N]`` with ``-inf`` outside each row's causal
    range.  For every row with more than K valid keys the selection must hold
    all keys above the K-th largest score, none below it, and K ids in total
    (the contract check guarantees the count and uniqueness).  Bit-exact: no
    tolerance is involved.
    """

    import torch

    validate_topk_indices(indices, case, name=name)
    ends = _causal_ends(torch, case, scores.device)
    eligible = (ends > case.top_k).nonzero().flatten()
    tie_rows = 0
    tie_row_ids: list[int] = []
    if eligible.numel():
        live = scores[eligible]
        cutoff = torch.topk(live, case.top_k, dim=-1, sorted=True).values[:, -1]
        chosen = indices[:, 0, :][eligible].to(torch.int64)
        chosen_scores = live.gather(1, chosen)
        low = (chosen_scores < cutoff[:, None]).nonzero()
        if low.numel():
            row = int(eligible[int(low[0, 0])])
            key = int(chosen[int(low[0, 0]), int(low[0, 1])])
            raise CorrectnessError(f"{name} row {row} selected ID {key} below the TopK cutoff")
        above_total = (live > cutoff[:, None]).sum(dim=1)
        above_chosen = (chosen_scores > cutoff[:, None]).sum(dim=1)
        short = (above_total != above_chosen).nonzero()
        if short.numel():
            row = int(eligible[int(short[0])])
            raise CorrectnessError(f"{name} row {row} omitted an ID above the TopK cutoff")
        at_cutoff = (live == cutoff[:, None]).sum(dim=1)
        tied = at_cutoff > (case.top_k - above_total)
        tie_rows = int(tied.sum())
        tie_row_ids = eligible[tied].tolist()
    return {
        "status": "passed",
        "policy": "exact_score_threshold",
        "rows_checked": int(eligible.numel()),
        "rows_with_cutoff_ties": tie_rows,
        # rows in which more keys share the cutoff score than fit: any of them completes an exact Top-K,
        # so two exact results may differ there
        "cutoff_tie_rows": tie_row_ids,
    }


def tolerance_set_report(
    indices: Any, oracle_scores: Any, case: PrefillCase, *, relative_tolerance: float = 1e-3, rows: Any = None
) -> dict[str, Any]:
    """Account for set differences against scores that are only known to a tolerance.

    ``oracle_scores`` come from a different arithmetic than the kernel's, so a
    key whose oracle score lies within ``relative_tolerance * rowmax`` of the
    oracle's K-th value may legitimately fall on either side of the cutoff.
    Every id the candidate has but the oracle's Top-K lacks (and vice versa)
    must lie inside that window; they are counted and returned.  An id
    outside the window raises.

    ``rows`` (int64 tensor) names the query rows of ``case`` that ``indices`` and
    ``oracle_scores`` hold, for checks on a sample of a large problem; without it
    they hold every row (and the output contract is validated first).
    """

    import torch

    if rows is None:
        validate_topk_indices(indices, case, name="indices")
        ends = _causal_ends(torch, case, oracle_scores.device)
    else:
        ends = _causal_ends(torch, case, oracle_scores.device)[rows.to(oracle_scores.device)]
    eligible = (ends > case.top_k).nonzero().flatten()
    rows_differing = 0
    swapped = 0
    worst = 0.0
    if eligible.numel():
        live = oracle_scores[eligible]
        cutoff = torch.topk(live, case.top_k, dim=-1, sorted=True).values[:, -1]
        finite = torch.where(torch.isfinite(live), live, torch.zeros_like(live))
        window = relative_tolerance * finite.abs().amax(dim=1)
        chosen = indices[:, 0, :][eligible].to(torch.int64)
        member = torch.zeros_like(live, dtype=torch.bool)
        member.scatter_(1, chosen, True)
        should = live >= cutoff[:, None]
        # ids the candidate holds although the oracle scores them below the cutoff
        extra = member & (live < cutoff[:, None])
        # ids above the oracle cutoff that the candidate lacks
        lost = (~member) & (live > cutoff[:, None])
        distance = (live - cutoff[:, None]).abs()
        offending = (extra | lost) & (distance > window[:, None])
        if bool(offending.any()):
            where = offending.nonzero()[0]
            row = int(eligible[int(where[0])])
            raise CorrectnessError(
                f"row {row} key {int(where[1])} differs from the oracle Top-K by "
                f"{float(distance[int(where[0]), int(where[1])]):.3e}, outside the tolerance window "
                f"{float(window[int(where[0])]):.3e}"
            )
        per_row = (extra | lost).sum(dim=1)
        rows_differing = int((per_row > 0).sum())
        swapped = int(extra.sum())
        if swapped or int(lost.sum()):
            worst = float((distance * (extra | lost)).max())
        del should
    return {
        "status": "passed",
        "rows_checked": int(eligible.numel()),
        "rows_with_set_difference": rows_differing,
        "ids_swapped_within_tolerance": swapped,
        "largest_swapped_distance": worst,
        "relative_tolerance": relative_tolerance,
    }


validate_indices = validate_topk_indices
compare_with_baseline = compare_topk_indices
