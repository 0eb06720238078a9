"""On-device e4m3 quantisation of the operator's inputs (the step before the operator).

The reference prepares its FP8 inputs with torch expressions before the operator
is called: ``quantize_contiguous_index_kv`` for the index keys
(``src/fused_index_topk/inputs.py:76-90``) and, for activations quantised per
128-element group, a per-row scale that the caller must fold into the head
weights because the operator has no query-scale argument
(``src/fused_index_topk/contract.py:152-185``).  The functions here keep those
names' meaning and results (bit-identical for finite inputs) but run as one
pass over HBM in ``libitk_b200.so`` (``itk_quantize_rows_e4m3``).

* ``quantize_contiguous_index_kv(source)``: ``[N,128]`` fp32/bf16 ->
  ``([N,128] float8_e4m3fn, [N] float32)``;
* ``quantize_queries(source, weights)``: ``[Q,64,128]`` fp32/bf16 and ``[Q,64]``
  fp32 -> ``([Q,64,128] float8_e4m3fn, [Q,64] float32 weights * row scale)``;
* ``fused_index_topk_from_activations``: both of the above, then the operator.
"""

from __future__ import annotations

from typing import Any

from . import _lib

SOURCE_F32 = 0
SOURCE_BF16 = 1


def _source_code(torch: Any, tensor: Any) -> int:
    if tensor.dtype == torch.float32:
        return SOURCE_F32
    if tensor.dtype == torch.bfloat16:
        return SOURCE_BF16
    raise TypeError(f"source must be float32 or bfloat16, got {tensor.dtype}")


def _check_source(torch: Any, source: Any, what: str) -> None:
    if not source.is_cuda:
        raise ValueError(f"{what} must be a CUDA tensor (there is no CPU path)")
    if not source.is_contiguous():
        raise ValueError(f"{what} must be contiguous")
    if source.shape[-1] != _lib.HEAD_DIM:
        raise ValueError(f"{what} rows must have {_lib.HEAD_DIM} elements")


def quantize_rows(source: Any, *, fold: Any = None, out: Any = None, out_scales: Any = None,
                  out_folded: Any = None, want_scales: bool = True):
    """Quantise every ``[..., 128]`` row; returns ``(values, scales, folded)``.

    ``fold`` (fp32, one entry per row) is multiplied by the row scales into
    ``folded``; without it ``folded`` is ``None``.  ``scales`` is ``None`` when
    ``want_scales`` is false and a fold takes them instead.
    """

    import torch

    _check_source(torch, source, "source")
    rows = source.numel() // _lib.HEAD_DIM
    if rows == 0:
        raise ValueError("source has no rows")
    device = source.device
    values = out if out is not None else torch.empty(source.shape, dtype=torch.float8_e4m3fn, device=device)
    if values.shape != source.shape or values.dtype != torch.float8_e4m3fn or not values.is_contiguous():
        raise ValueError("out must be a contiguous float8_e4m3fn tensor of the source's shape")
    scales = None
    if want_scales or fold is None:
        scales = out_scales if out_scales is not None else torch.empty(source.shape[:-1], dtype=torch.float32, device=device)
        if scales.numel() != rows or scales.dtype != torch.float32 or not scales.is_contiguous():
            raise ValueError("out_scales must be a contiguous float32 tensor with one entry per row")
    folded = None
    if fold is not None:
        if fold.dtype != torch.float32 or fold.numel() != rows or not fold.is_contiguous() or fold.device != device:
            raise ValueError("fold must be a contiguous float32 tensor with one entry per row on the source's device")
        folded = out_folded if out_folded is not None else torch.empty_like(fold)
        if folded.dtype != torch.float32 or folded.numel() != rows or not folded.is_contiguous():
            raise ValueError("out_folded must be a contiguous float32 tensor with one entry per row")
    with torch.cuda.device(device):
        _lib.check(_lib.load_library().itk_quantize_rows_e4m3(
            _lib.ptr(source), _source_code(torch, source), _lib.ptr(fold), _lib.ptr(folded), _lib.ptr(values),
            _lib.ptr(scales), rows, _lib.current_stream(torch, device),
        ))
    return values, scales, folded


def quantize_contiguous_index_kv(source: Any) -> tuple[Any, Any]:
    """``[N,128]`` fp32/bf16 keys -> ``(kv e4m3 [N,128], kv_scales fp32 [N])``."""

    if source.ndim != 2:
        raise ValueError("contiguous index KV must be rank two")
    values, scales, _ = quantize_rows(source)
    return values, scales


def quantize_queries(source: Any, weights: Any) -> tuple[Any, Any]:
    """``[Q,64,128]`` queries and ``[Q,64]`` weights -> ``(q e4m3, weights * q_scale)``."""

    if source.ndim != 3 or source.shape[1] != _lib.HEADS:
        raise ValueError(f"queries must be [Q,{_lib.HEADS},{_lib.HEAD_DIM}]")
    if tuple(weights.shape) != tuple(source.shape[:2]):
        raise ValueError("weights must be [Q,64]")
    values, _, folded = quantize_rows(source, fold=weights, want_scales=False)
    return values, folded


def fused_index_topk_from_activations(q_source: Any, kv_source: Any, weights: Any, k_start: Any, k_end: Any,
                                      top_k: int = _lib.TOP_K, **kwargs):
    """Quantise queries and keys on the device, then run the operator on the result."""

    from .operator import fused_index_topk

    q, folded = quantize_queries(q_source, weights)
    kv, kv_scales = quantize_contiguous_index_kv(kv_source)
    return fused_index_topk(q, (kv, kv_scales), folded, k_start, k_end, top_k=top_k, **kwargs)


__all__ = [
    "SOURCE_BF16", "SOURCE_F32", "fused_index_topk_from_activations", "quantize_contiguous_index_kv",
    "quantize_queries", "quantize_rows",
]
