"""The unfused checking variant: dense scores, then ``torch.topk``.

The reference validates every candidate against an unfused variant that
materialises the dense ``[Q,N]`` fp32 logits and selects with ``torch.topk``
(``src/fused_index_topk/variants/deepgemm_torch.py``, stages as in
``variants/common.py:19-52,133-152``); its scorer is DeepGEMM, which is not
available on B200 boxes without its JIT.  This variant has the same graph shape
(``indexer`` -> ``topk`` -> ``output``, artifacts ``logits`` and ``indices``), with
the scores written by the fused kernel's diagnostic output (every in-range key,
``-inf`` outside ``[k_start,k_end)``) and the selection left to ``torch.topk``.

It is a harness component (what the reference's ``CaseLifecycle`` builds its
oracle from when this package is checked under the reference harness,
``src/fused_index_topk/lifecycle.py:240-291``), not an operator path: nothing in ``operator.py`` or ``plugin.py`` uses it,
it allocates 4*Q*N bytes, and it exists to give an independent selection over
identical fp32 scores.
"""

from __future__ import annotations

import math
from typing import Any, Mapping

from . import _lib, operator
from .api import (
    API_VERSION,
    PrefillCase,
    PrefillInputs,
    PreparedGraph,
    RunMode,
    StageNode,
    StageSpec,
    VariantDescriptor,
)


class DenseScoresTorchTopK:
    """``mode="unfused"`` variant: dense fp32 logits on the device + ``torch.topk``."""

    descriptor = VariantDescriptor(
        plugin_id="b200_dense_scores_torch_topk",
        display_name="Dense scores + torch.topk",
        api_version=API_VERSION,
        implementation_version="0.1.0",
        mode="unfused",
        description="Dense fp32 logits from the diagnostic output of the score kernel, torch.topk, int32 output stage",
        implementation="b200-native-scores+torch-topk",
        exact_topk=True,
        source_revision="fusedindextopk-b200-0.1",
        supported_arches=("sm100",),
        tags=("prefill", "sm100", "checking-variant", "dense-logits"),
    )

    def __init__(self, options: Mapping[str, Any] | None = None) -> None:
        self.options = dict(options or {})
        if self.options:
            raise ValueError(f"unknown options: {sorted(self.options)}")

    def supports(self, case: PrefillCase) -> bool:
        return (
            case.batch_size == 1 and case.causal and case.indexer_heads == _lib.HEADS
            and case.head_dim == _lib.HEAD_DIM and 0 < case.query_tokens <= case.context_tokens
            and 0 < case.top_k <= case.context_tokens <= _lib.MAX_KEYS
        )

    def fingerprint_metadata(self) -> Mapping[str, Any]:
        return {"algorithm": "dense-logits-torch-topk", "options": self.options, "dense_logits_materialized": True}

    def prepare(self, case: PrefillCase, inputs: PrefillInputs, *, options: Mapping[str, Any],
                mode: RunMode) -> PreparedGraph:
        del mode
        if not self.supports(case):
            raise ValueError(f"unsupported case: {case}")
        if options and dict(options) != self.options:
            raise ValueError("variant options changed after construction")
        import torch

        device = inputs.q.device
        ws = operator.make_workspace(case.query_tokens, case.context_tokens, device, seed=case.seed, key_shards=1)
        logits = torch.empty((case.query_tokens, case.context_tokens), device=device, dtype=torch.float32)

        def run_indexer(context: Any, artifacts: dict) -> None:
            del context
            standard: PrefillInputs = artifacts["inputs"]
            tensors = (standard.q, standard.kv, standard.kv_scales, standard.weights, standard.k_start, standard.k_end)
            operator.validate_operator_inputs(*tensors)
            logits.fill_(-math.inf)
            # no candidate passes a +inf threshold: the launch only writes the dense scores
            ws.thresholds.fill_(math.inf)
            operator.run_fused_topk(ws, *tensors, diag_logits=logits, force_compute=True)
            artifacts["logits"] = logits

        def run_topk(context: Any, artifacts: dict) -> None:
            del context
            values, ids = torch.topk(artifacts["logits"], case.top_k, dim=-1, sorted=False)
            artifacts["topk_values"] = values
            artifacts["topk_ids"] = ids

        def run_output(context: Any, artifacts: dict) -> None:
            del context
            standard: PrefillInputs = artifacts["inputs"]
            values, ids = artifacts["topk_values"], artifacts["topk_ids"]
            valid = torch.isfinite(values) & (ids >= 0) & (ids < standard.k_end.unsqueeze(-1))
            chosen = torch.where(valid, ids, torch.full_like(ids, -1))
            artifacts["indices"] = chosen.to(torch.int32).unsqueeze(1).contiguous()

        def node(stage_id, dependencies, consumes, produces, ops, description, kernels, run):
            return StageNode(
                StageSpec(stage_id=stage_id, dependencies=dependencies, consumes=consumes, produces=produces,
                          semantic_ops=ops, description=description, kernel_regexes=kernels),
                run,
            )

        nodes = (
            node("indexer", (), ("inputs",), ("logits",), ("indexer",),
                 "Dense fp32 logits of every in-range key, -inf elsewhere", ("itk_fused_kernel",), run_indexer),
            node("topk", ("indexer",), ("logits",), ("topk_values", "topk_ids"), ("topk",),
                 "torch.topk over the dense logits, unordered", ("topk", "gatherTopK", "sort"), run_topk),
            node("output", ("topk",), ("inputs", "topk_values", "topk_ids"), ("indices",), ("output",),
                 "Finite scores inside [0,k_end) keep their id, everything else becomes -1; int32 [Q,1,K]",
                 ("elementwise",), run_output),
        )
        return PreparedGraph(
            descriptor=self.descriptor, nodes=nodes, initial_artifacts={"inputs": inputs},
            terminal_artifact="indices",
            metadata={"algorithm": "dense-logits-torch-topk", "dense_logits_materialized": True,
                      "logits_bytes": int(logits.numel()) * 4},
        )


def create_dense_variant(options: Mapping[str, Any] | None = None) -> DenseScoresTorchTopK:
    return DenseScoresTorchTopK(options)


__all__ = ["DenseScoresTorchTopK", "create_dense_variant"]
