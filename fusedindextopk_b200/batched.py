"""Several sequences in one operator call (variable lengths, packed layout).

The reference serves one contiguous sequence per call and rejects
``batch_size > 1`` (``src/fused_index_topk/inputs.py:31-32``).  The operator's
per-row key ranges ``[k_start, k_end)`` already allow more: pack the keys of all
sequences into one ``[sum N_b, 128]`` array and the query rows into one
``[sum Q_b, 64, 128]`` array, give every row the range of its own sequence
(causal inside it), and one launch of the persistent kernel scores the whole
batch; each row only visits the 128-key tiles its range touches.  The returned
ids are positions in the packed array; ``local_ids=True`` rebases them to the
row's sequence.

The layout follows the usual variable-length convention: ``cu_seqlens_q`` and
``cu_seqlens_k`` are int32 ``[B+1]`` prefix sums (first entry 0).  The queries of
a sequence are its LAST ``Q_b`` tokens, as in the single-sequence contract
(``k_end[i] = N_b - Q_b + i + 1`` relative to the sequence start).

Limits: the packed key count obeys the single-call limit (262144); sequences
shorter than 2048 keys return all their visible keys and ``-1`` padding, like
short single sequences do.
"""

from __future__ import annotations

from typing import Any, Sequence

from . import _lib


def pack_sequences(tensors: Sequence[Any]) -> tuple[Any, Any]:
    """Concatenate per-sequence tensors along dim 0; returns ``(packed, cu_seqlens int32 [B+1])``."""

    import torch

    if not tensors:
        raise ValueError("need at least one sequence")
    lengths = torch.tensor([0] + [int(t.shape[0]) for t in tensors], dtype=torch.int64)
    packed = torch.cat(list(tensors), dim=0).contiguous()
    return packed, torch.cumsum(lengths, dim=0).to(torch.int32).to(packed.device)


def varlen_ranges(cu_seqlens_q: Any, cu_seqlens_k: Any, *, causal: bool = True) -> tuple[Any, Any, Any]:
    """``(k_start, k_end, key_offset)`` int32 ``[sum Q_b]`` in packed key positions, on the inputs' device."""

    import torch

    if cu_seqlens_q.dtype != torch.int32 or cu_seqlens_k.dtype != torch.int32:
        raise ValueError("cu_seqlens_q and cu_seqlens_k must be int32")
    if cu_seqlens_q.dim() != 1 or cu_seqlens_q.shape != cu_seqlens_k.shape or cu_seqlens_q.numel() < 2:
        raise ValueError("cu_seqlens_q and cu_seqlens_k must both be [B+1] with B >= 1")
    starts_q, starts_k = cu_seqlens_q.long(), cu_seqlens_k.long()
    rows_per, keys_per = starts_q[1:] - starts_q[:-1], starts_k[1:] - starts_k[:-1]
    if int(starts_q[0]) != 0 or int(starts_k[0]) != 0:
        raise ValueError("cu_seqlens must start at 0")
    if bool((rows_per <= 0).any()) or bool((keys_per < rows_per).any()):
        raise ValueError("every sequence needs 0 < Q_b <= N_b")
    sequence = torch.repeat_interleave(torch.arange(rows_per.numel(), device=rows_per.device), rows_per)
    local_row = torch.arange(int(starts_q[-1]), device=rows_per.device) - starts_q[:-1][sequence]
    key_offset = starts_k[:-1][sequence]
    if causal:
        visible = keys_per[sequence] - rows_per[sequence] + local_row + 1
    else:
        visible = keys_per[sequence]
    return key_offset.to(torch.int32), (key_offset + visible).to(torch.int32), key_offset.to(torch.int32)


def fused_index_topk_varlen(q: Any, kv_pair: tuple[Any, Any], weights: Any, cu_seqlens_q: Any, cu_seqlens_k: Any,
                            top_k: int = _lib.TOP_K, *, causal: bool = True, local_ids: bool = True, **kwargs) -> Any:
    """Exact Top-K ids per query row of a packed batch, int32 ``[sum Q_b, K]``, ``-1`` padded.

    ``q`` is ``[sum Q_b, 64, 128]`` e4m3, ``kv_pair = (kv [sum N_b,128] e4m3, kv_scales [sum N_b])``,
    ``weights`` ``[sum Q_b, 64]``.  With ``local_ids`` the ids count from the start of the row's
    own sequence, otherwise they are positions in the packed key array.
    """

    import torch

    from .operator import fused_index_topk

    device = q.device
    k_start, k_end, key_offset = varlen_ranges(cu_seqlens_q.to(device), cu_seqlens_k.to(device), causal=causal)
    if int(k_start.numel()) != int(q.shape[0]):
        raise ValueError("cu_seqlens_q does not add up to the number of query rows")
    if int(cu_seqlens_k[-1]) != int(kv_pair[0].shape[0]):
        raise ValueError("cu_seqlens_k does not add up to the number of keys")
    ids = fused_index_topk(q, kv_pair, weights, k_start, k_end, top_k=top_k, **kwargs)
    if not local_ids:
        return ids
    return torch.where(ids >= 0, ids - key_offset.unsqueeze(-1), ids)


__all__ = ["fused_index_topk_varlen", "pack_sequences", "varlen_ranges"]
