"""One case from A/B fixtures through oracle, candidate preparation and exactness checks.

The reference owns every GPU check through one lifecycle object
(``src/fused_index_topk/lifecycle.py:63-418``): two fixtures A and B of the same
shape and different content; an exact oracle per fixture from an unfused variant
that exposes its dense logits (contract check + cutoff-tie oracle); the candidate
prepared ONCE on fixture A and then executed on A and on B through the
``inputs`` artifact, so that a plugin which hides a precomputed answer in
``prepare`` fails on B; and a content hash of all six input tensors of both
fixtures taken before anything runs and re-checked after every phase, so that a
stage that writes into its inputs is caught.  ``CaseLifecycle`` here has the same
phases, method names and error texts, built on this package's variants:
``variants.DenseScoresTorchTopK`` as the default oracle variant and
``plugin.FusedIndexTopK`` as the usual candidate.  ``check_variant`` runs the
whole sequence and returns the record.
"""

from __future__ import annotations

import hashlib
import json
from dataclasses import asdict, dataclass
from typing import Any, Callable, Mapping, Sequence

from .api import ExecutionContext, PrefillCase, PrefillInputs, PreparedGraph, RunMode
from .correctness import build_score_threshold_oracle, compare_topk_indices, validate_topk_indices

FIXTURE_IDS = ("A", "B")
INPUT_NAMES = ("q", "kv", "kv_scales", "weights", "k_start", "k_end")
InputFactory = Callable[[PrefillCase, Any, str], PrefillInputs]


def canonical_hash(value: Any) -> str:
    """SHA-256 of the canonical JSON form (sorted keys, no whitespace)."""

    text = json.dumps(value, sort_keys=True, separators=(",", ":"), default=str)
    return hashlib.sha256(text.encode()).hexdigest()


def input_content_fingerprint(inputs: PrefillInputs) -> dict[str, Any]:
    """Per-tensor dtype, shape and SHA-256 of the logical bytes, plus one digest over all six."""

    import torch

    manifest: dict[str, Any] = {}
    for name in INPUT_NAMES:
        tensor = getattr(inputs, name)
        host = tensor.detach().contiguous().view(torch.uint8).cpu()
        manifest[name] = {
            "dtype": str(tensor.dtype).replace("torch.", ""),
            "shape": [int(extent) for extent in tensor.shape],
            "sha256": hashlib.sha256(host.numpy().tobytes()).hexdigest(),
        }
    return {"sha256": canonical_hash(manifest), "manifest": manifest}


def _input_versions(inputs: PrefillInputs) -> dict[str, int | None]:
    return {name: getattr(getattr(inputs, name), "_version", None) for name in INPUT_NAMES}


def _synchronize(torch: Any) -> None:
    # the lifecycle's bookkeeping also runs with CPU stand-in variants (tests of the gates themselves)
    if torch.cuda.is_available():
        torch.cuda.synchronize()


def validate_graph(graph: PreparedGraph) -> tuple[Any, ...]:
    """Stage ids unique, dependencies and consumed artifacts produced earlier, terminal produced."""

    seen_stages: set[str] = set()
    available = set(graph.initial_artifacts)
    for node in graph.nodes:
        spec = node.spec
        if spec.stage_id in seen_stages:
            raise ValueError(f"duplicate stage_id {spec.stage_id!r}")
        missing = [name for name in spec.dependencies if name not in seen_stages]
        if missing:
            raise ValueError(f"stage {spec.stage_id!r} depends on later or unknown stages {missing}")
        absent = [name for name in spec.consumes if name not in available]
        if absent:
            raise ValueError(f"stage {spec.stage_id!r} consumes artifacts nothing produced: {absent}")
        seen_stages.add(spec.stage_id)
        available.update(spec.produces)
    if graph.terminal_artifact not in available:
        raise ValueError(f"no stage produces the terminal artifact {graph.terminal_artifact!r}")
    return tuple(graph.nodes)


def graph_fingerprint(graph: PreparedGraph) -> str:
    """Digest of the descriptor and the stage specifications (not of buffers or closures)."""

    return canonical_hash({
        "descriptor": asdict(graph.descriptor),
        "terminal_artifact": graph.terminal_artifact,
        "stages": [asdict(node.spec) for node in graph.nodes],
    })


@dataclass
class FixtureState:
    fixture_id: str
    inputs: PrefillInputs
    content_before: Mapping[str, Any]
    versions_before: Mapping[str, int | None]

    @property
    def content_hash(self) -> str:
        return str(self.content_before["sha256"])


@dataclass
class OracleState:
    fixture_id: str
    indices: Any
    output_check: Mapping[str, Any]
    cutoff_tie_check: Mapping[str, Any]
    cutoff_tie_rows: Mapping[int, Mapping[str, Any]]


class CaseLifecycle:
    """Fixtures A/B, per-fixture oracle, one candidate preparation, checks on A and B."""

    def __init__(self, *, case: PrefillCase, reference: Any = None, reference_options: Mapping[str, Any] | None = None,
                 mode: RunMode = RunMode.CORRECTNESS, device: Any = "cuda",
                 input_factory: InputFactory | None = None) -> None:
        if reference is None:
            from .variants import DenseScoresTorchTopK

            reference = DenseScoresTorchTopK()
        self.case = case
        self.reference = reference
        self.reference_options = dict(reference_options or {})
        self.mode = mode
        self.device = device
        self.input_factory = input_factory
        self.fixtures: dict[str, FixtureState] = {}
        self.oracles: dict[str, OracleState] = {}
        self.reference_graph_fingerprint: str | None = None
        self.candidate_graph: PreparedGraph | None = None
        self.candidate_nodes: tuple[Any, ...] = ()
        self.integrity_checks: list[dict[str, Any]] = []
        self._create_fixtures()

    # ------------------------------------------------------------------ fixtures and integrity

    def _create_fixtures(self) -> None:
        from .inputs import make_prefill_inputs

        for fixture_id in FIXTURE_IDS:
            if self.input_factory is None:
                inputs = make_prefill_inputs(self.case, device=self.device, fixture_id=fixture_id)
            else:
                inputs = self.input_factory(self.case, self.device, fixture_id)
                if inputs.case != self.case:
                    raise ValueError("input factory returned inputs for a different case")
                if inputs.fixture_id != fixture_id:
                    raise ValueError("input factory returned the wrong A/B fixture identifier")
            self.fixtures[fixture_id] = FixtureState(
                fixture_id=fixture_id, inputs=inputs,
                content_before=input_content_fingerprint(inputs), versions_before=_input_versions(inputs),
            )
        if len({fixture.content_hash for fixture in self.fixtures.values()}) != len(FIXTURE_IDS):
            raise RuntimeError("A/B fixtures must have different tensor content")

    @property
    def input_content_hash(self) -> str:
        return canonical_hash({name: self.fixtures[name].content_hash for name in FIXTURE_IDS})

    def verify_input_integrity(self, phase: str) -> dict[str, Any]:
        """Re-hash every input tensor of both fixtures; any change since creation is an error."""

        report: dict[str, Any] = {}
        for fixture_id, fixture in self.fixtures.items():
            current = input_content_fingerprint(fixture.inputs)
            if current["sha256"] != fixture.content_hash:
                raise RuntimeError(f"fixture {fixture_id} tensor content changed during {phase}")
            if _input_versions(fixture.inputs) != fixture.versions_before:
                raise RuntimeError(f"fixture {fixture_id} version counters changed during {phase}")
            report[fixture_id] = {
                "sha256_before": fixture.content_hash, "sha256_after": current["sha256"], "versions_unchanged": True,
            }
        result = {"status": "passed", "phase": phase, "fixtures": report}
        self.integrity_checks.append(result)
        return result

    # ------------------------------------------------------------------ graph handling

    def _prepare(self, plugin: Any, options: Mapping[str, Any], *, fixture_id: str = "A"):
        if not plugin.supports(self.case):
            raise ValueError(f"variant {plugin.descriptor.plugin_id!r} does not support {self.case.case_id}")
        graph = plugin.prepare(self.case, self.fixtures[fixture_id].inputs, options=dict(options), mode=self.mode)
        if graph.descriptor.plugin_id != plugin.descriptor.plugin_id:
            raise ValueError("prepared graph descriptor does not match the loaded plugin")
        if "inputs" not in graph.initial_artifacts:
            raise ValueError("prepared graph must expose standard inputs as initial_artifacts['inputs']")
        return graph, validate_graph(graph)

    def bound_artifacts(self, graph: PreparedGraph, fixture_id: str) -> dict[str, Any]:
        if fixture_id not in self.fixtures:
            raise ValueError(f"unknown fixture_id {fixture_id!r}")
        artifacts = dict(graph.initial_artifacts)
        artifacts["inputs"] = self.fixtures[fixture_id].inputs
        return artifacts

    def execute(self, graph: PreparedGraph, nodes: Sequence[Any], *, fixture_id: str, iteration: int,
                validate_produced: bool = False) -> dict[str, Any]:
        import torch

        stream = torch.cuda.current_stream() if torch.cuda.is_available() else None
        context = ExecutionContext(case=self.case, mode=self.mode, iteration=iteration, stream=stream)
        artifacts = self.bound_artifacts(graph, fixture_id)
        with torch.inference_mode():
            for node in nodes:
                node.run(context, artifacts)
                if validate_produced:
                    absent = [name for name in node.spec.produces if name not in artifacts]
                    if absent:
                        raise RuntimeError(f"stage {node.spec.stage_id!r} did not produce {absent}")
        return artifacts

    # ------------------------------------------------------------------ oracle, candidate, checks

    def build_oracles(self) -> dict[str, Any]:
        """Exact A and B answers from the reference variant, before the candidate is prepared."""

        import torch

        graph, nodes = self._prepare(self.reference, self.reference_options)
        self.reference_graph_fingerprint = graph_fingerprint(graph)
        record: dict[str, Any] = {}
        for iteration, fixture_id in enumerate(FIXTURE_IDS):
            outputs = self.execute(graph, nodes, fixture_id=fixture_id, iteration=iteration, validate_produced=True)
            _synchronize(torch)
            if "logits" not in outputs:
                raise RuntimeError("fusion-v1 exactness oracle must expose realized FP32 reference logits")
            indices = outputs[graph.terminal_artifact].clone()
            output_check = validate_topk_indices(indices, self.case, name=f"fixture {fixture_id} exact reference")
            tie_check, tie_rows = build_score_threshold_oracle(outputs["logits"], indices, self.case)
            self.oracles[fixture_id] = OracleState(
                fixture_id=fixture_id, indices=indices, output_check=output_check,
                cutoff_tie_check=tie_check, cutoff_tie_rows=tie_rows,
            )
            record[fixture_id] = {
                "contract_check": output_check,
                "cutoff_tie_check": tie_check,
                "reference_indices_bytes": int(indices.numel()) * int(indices.element_size()),
            }
            del outputs
        self.verify_input_integrity("before_candidate")
        return {"status": "passed", "graph_fingerprint": self.reference_graph_fingerprint, "fixtures": record}

    def prepare_candidate(self, plugin: Any, options: Mapping[str, Any] | None = None) -> PreparedGraph:
        if not self.oracles:
            raise RuntimeError("build_oracles() must run before candidate preparation")
        import torch

        graph, nodes = self._prepare(plugin, dict(options or {}))
        _synchronize(torch)
        self.verify_input_integrity("candidate_prepare")
        self.candidate_graph, self.candidate_nodes = graph, nodes
        return graph

    def validate_outputs(self, outputs: Mapping[str, Any], *, fixture_id: str, name: str) -> dict[str, Any]:
        """The terminal contract, then the fixture's exact oracle under the cutoff-tie rule."""

        if self.candidate_graph is None:
            raise RuntimeError("prepare_candidate() must run before output validation")
        if fixture_id not in self.oracles:
            raise ValueError(f"unknown fixture_id {fixture_id!r}")
        oracle = self.oracles[fixture_id]
        indices = outputs[self.candidate_graph.terminal_artifact]
        return {
            "contract_check": validate_topk_indices(indices, self.case, name=name),
            "exact_reference_check": compare_topk_indices(
                indices, oracle.indices, self.case, cutoff_tie_rows=oracle.cutoff_tie_rows
            ),
        }

    def check_candidate(self, *, phase: str, order: Sequence[str] = FIXTURE_IDS, start_iteration: int = 0) -> dict[str, Any]:
        if self.candidate_graph is None:
            raise RuntimeError("prepare_candidate() must run before candidate checks")
        import torch

        checks: dict[str, Any] = {}
        for offset, fixture_id in enumerate(order):
            outputs = self.execute(self.candidate_graph, self.candidate_nodes, fixture_id=fixture_id,
                                   iteration=start_iteration + offset, validate_produced=True)
            _synchronize(torch)
            verdict = self.validate_outputs(outputs, fixture_id=fixture_id, name=f"{phase} fixture {fixture_id} candidate")
            checks[f"{offset}:{fixture_id}"] = {"fixture_id": fixture_id, **verdict}
            del outputs
        integrity = self.verify_input_integrity(phase)
        return {"status": "passed", "phase": phase, "order": list(order), "checks": checks, "input_integrity": integrity}

    def warmup_candidate(self, iterations: int) -> None:
        if iterations < 0:
            raise ValueError("warmup iterations must be non-negative")
        if self.candidate_graph is None:
            raise RuntimeError("prepare_candidate() must run before warmup")
        import torch

        for iteration in range(iterations):
            outputs = self.execute(self.candidate_graph, self.candidate_nodes,
                                   fixture_id=FIXTURE_IDS[iteration % len(FIXTURE_IDS)], iteration=iteration)
            if self.candidate_graph.terminal_artifact not in outputs:
                raise RuntimeError("warmup graph did not produce its terminal artifact")
        _synchronize(torch)

    def metadata(self) -> dict[str, Any]:
        return {
            "schema_version": 1,
            "case": asdict(self.case),
            "fixture_order": list(FIXTURE_IDS),
            "fixtures": {name: {"content": fixture.content_before} for name, fixture in self.fixtures.items()},
            "input_content_hash": self.input_content_hash,
            "reference_graph_fingerprint": self.reference_graph_fingerprint,
            "candidate_graph_fingerprint": (
                graph_fingerprint(self.candidate_graph) if self.candidate_graph is not None else None
            ),
            "integrity_checks": list(self.integrity_checks),
            "anti_precompute_gate": {
                "candidate_prepare_fixture": "A",
                "required_execution_fixtures": ["A", "B"],
                "same_shape_different_content": True,
            },
        }


def check_variant(case: PrefillCase, candidate: Any = None, *, options: Mapping[str, Any] | None = None,
                  reference: Any = None, device: Any = "cuda", input_factory: InputFactory | None = None,
                  warmup: int = 2) -> dict[str, Any]:
    """Oracle, prepare on A, check A then B, warm up on both, check B then A; returns the record."""

    if candidate is None:
        from .plugin import create_variant

        candidate = create_variant(options)
    life = CaseLifecycle(case=case, reference=reference, device=device, input_factory=input_factory)
    oracle = life.build_oracles()
    life.prepare_candidate(candidate, options)
    first = life.check_candidate(phase="after_prepare")
    life.warmup_candidate(warmup)
    second = life.check_candidate(phase="after_warmup", order=("B", "A"), start_iteration=warmup + 2)
    return {"status": "passed", "oracle": oracle, "checks": [first, second], "lifecycle": life.metadata()}


__all__ = [
    "CaseLifecycle", "FIXTURE_IDS", "FixtureState", "OracleState", "canonical_hash", "check_variant",
    "graph_fingerprint", "input_content_fingerprint", "validate_graph",
]
