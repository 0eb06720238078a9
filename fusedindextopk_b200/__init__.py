"""B200-native fused lightning-indexer score + exact Top-2048 operator.

Public surface:

* ``fused_index_topk(q, (kv, kv_scales), weights, k_start, k_end, top_k=2048)``
  -> int32 ``[Q, K]`` exact unordered Top-K key ids (``-1`` padded);
* ``create_variant(options)`` -> the operator as a plugin with
  ``descriptor / supports / fingerprint_metadata / prepare``;
* ``make_workspace`` and the ``run_*`` stage functions for callers that manage
  their own buffers.

Importing the package initialises neither torch nor CUDA; the CUDA library
(``libitk_b200.so``, built by ``python -m fusedindextopk_b200.build``) is loaded
on first use and there is no fallback when it is absent.
"""

from __future__ import annotations

__version__ = "0.1.0"

from .api import (  # noqa: F401
    ExecutionContext,
    PrefillCase,
    PrefillInputs,
    PreparedGraph,
    RunMode,
    StageNode,
    StageSpec,
    VariantDescriptor,
    VariantPlugin,
    execute_graph,
)


def fused_index_topk(*args, **kwargs):
    from .operator import fused_index_topk as implementation

    return implementation(*args, **kwargs)


def fused_index_topk_host(*args, **kwargs):
    from .operator import fused_index_topk_host as implementation

    return implementation(*args, **kwargs)


def make_workspace(*args, **kwargs):
    from .operator import make_workspace as implementation

    return implementation(*args, **kwargs)


def create_variant(options=None):
    from .plugin import create_variant as implementation

    return implementation(options)


__all__ = [
    "ExecutionContext", "PrefillCase", "PrefillInputs", "PreparedGraph", "RunMode", "StageNode", "StageSpec",
    "VariantDescriptor", "VariantPlugin", "create_variant", "execute_graph", "fused_index_topk",
    "fused_index_topk_host", "make_workspace",
]
