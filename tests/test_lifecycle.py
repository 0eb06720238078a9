"""The A/B lifecycle: its gates on CPU stand-in variants (an honest one, one that precomputes
in prepare, one that writes into its inputs), and on the GPU the real candidate against the
dense-score checking variant."""

from __future__ import annotations

import pytest
import torch

from fusedindextopk_b200 import lifecycle
from fusedindextopk_b200.api import (
    API_VERSION, PrefillCase, PreparedGraph, RunMode, StageNode, StageSpec, VariantDescriptor,
)
from fusedindextopk_b200.correctness import CorrectnessError


def _descriptor(plugin_id: str) -> VariantDescriptor:
    return VariantDescriptor(
        plugin_id=plugin_id, display_name=plugin_id, api_version=API_VERSION, implementation_version="0",
        mode="unfused", description="cpu stand-in", implementation="torch-cpu", exact_topk=True,
    )


def _dense_logits(inputs):
    """Plain float32 scores on the CPU: only good enough to drive the lifecycle's bookkeeping."""

    q = inputs.q.float()
    kv = inputs.kv.float()
    dots = torch.relu(torch.einsum("qhd,nd->qhn", q, kv))
    logits = (dots * inputs.weights[:, :, None]).sum(dim=1) * inputs.kv_scales[None, :]
    position = torch.arange(kv.shape[0])[None, :]
    inside = (position >= inputs.k_start[:, None]) & (position < inputs.k_end[:, None])
    return torch.where(inside, logits, torch.full_like(logits, -float("inf"))).contiguous()


class CpuVariant:
    """Dense logits + torch.topk on the CPU, with switches for the two kinds of cheating."""

    def __init__(self, plugin_id="cpu_dense", *, precompute=False, scribble=False, hide_inputs=False):
        self.descriptor = _descriptor(plugin_id)
        self.precompute, self.scribble, self.hide_inputs = precompute, scribble, hide_inputs

    def supports(self, case):
        return True

    def fingerprint_metadata(self):
        return {}

    def prepare(self, case, inputs, *, options, mode):
        frozen = _dense_logits(inputs) if self.precompute else None

        def run_scores(context, artifacts):
            current = artifacts["inputs"]
            artifacts["logits"] = frozen if frozen is not None else _dense_logits(current)
            if self.scribble:
                current.weights[0, 0] += 1.0

        def run_select(context, artifacts):
            values, ids = torch.topk(artifacts["logits"], case.top_k, dim=-1, sorted=False)
            chosen = torch.where(torch.isfinite(values), ids, torch.full_like(ids, -1))
            artifacts["indices"] = chosen.to(torch.int32).unsqueeze(1).contiguous()

        nodes = (
            StageNode(StageSpec(stage_id="scores", dependencies=(), consumes=("inputs",), produces=("logits",),
                                semantic_ops=("indexer",), description="", kernel_regexes=()), run_scores),
            StageNode(StageSpec(stage_id="select", dependencies=("scores",), consumes=("logits",),
                                produces=("indices",), semantic_ops=("topk", "output"), description="",
                                kernel_regexes=()), run_select),
        )
        initial = {} if self.hide_inputs else {"inputs": inputs}
        return PreparedGraph(descriptor=self.descriptor, nodes=nodes, initial_artifacts=initial,
                             terminal_artifact="indices", metadata={})


CASE = PrefillCase("life-q6-n96", 6, 96, top_k=16, seed=4)


def _life(**kwargs):
    return lifecycle.CaseLifecycle(case=CASE, reference=CpuVariant("oracle"), device="cpu", **kwargs)


def test_honest_variant_passes_both_fixtures_and_keeps_inputs_intact():
    record = lifecycle.check_variant(CASE, CpuVariant("honest"), reference=CpuVariant("oracle"), device="cpu")
    assert record["status"] == "passed"
    assert [check["order"] for check in record["checks"]] == [["A", "B"], ["B", "A"]]
    meta = record["lifecycle"]
    assert meta["anti_precompute_gate"]["required_execution_fixtures"] == ["A", "B"]
    assert [item["phase"] for item in meta["integrity_checks"]] == [
        "before_candidate", "candidate_prepare", "after_prepare", "after_warmup"]
    assert meta["reference_graph_fingerprint"] != meta["candidate_graph_fingerprint"]
    fixtures = meta["fixtures"]
    assert fixtures["A"]["content"]["sha256"] != fixtures["B"]["content"]["sha256"]


def test_a_variant_that_precomputes_in_prepare_fails_on_fixture_b():
    life = _life()
    life.build_oracles()
    life.prepare_candidate(CpuVariant("cheat", precompute=True))
    with pytest.raises(CorrectnessError):
        life.check_candidate(phase="after_prepare")
    # fixture A alone would have passed: the gate is the second fixture
    life.check_candidate(phase="only_a", order=("A",))


def test_a_variant_that_writes_into_its_inputs_is_caught():
    life = _life()
    life.build_oracles()
    life.prepare_candidate(CpuVariant("scribbler", scribble=True))
    with pytest.raises(RuntimeError, match="tensor content changed during after_prepare"):
        life.check_candidate(phase="after_prepare")


def test_phase_order_and_graph_shape_are_enforced():
    life = _life()
    with pytest.raises(RuntimeError, match="build_oracles"):
        life.prepare_candidate(CpuVariant("early"))
    with pytest.raises(RuntimeError, match="prepare_candidate"):
        life.check_candidate(phase="x")
    life.build_oracles()
    with pytest.raises(ValueError, match="initial_artifacts"):
        life.prepare_candidate(CpuVariant("hidden", hide_inputs=True))

    class WrongId(CpuVariant):
        def prepare(self, case, inputs, *, options, mode):
            graph = super().prepare(case, inputs, options=options, mode=mode)
            return PreparedGraph(descriptor=_descriptor("someone_else"), nodes=graph.nodes,
                                 initial_artifacts=graph.initial_artifacts, terminal_artifact="indices", metadata={})

    with pytest.raises(ValueError, match="descriptor does not match"):
        life.prepare_candidate(WrongId("me"))


def test_factory_results_are_checked_and_identical_fixtures_rejected():
    from fusedindextopk_b200.inputs import make_prefill_inputs

    def same_content(case, device, fixture_id):
        made = make_prefill_inputs(case, device=device, fixture_id="A")
        made.fixture_id = fixture_id
        return made

    with pytest.raises(RuntimeError, match="different tensor content"):
        _life(input_factory=same_content)
    with pytest.raises(ValueError, match="wrong A/B fixture"):
        _life(input_factory=lambda case, device, fixture_id: make_prefill_inputs(case, device=device, fixture_id="A"))


def test_graph_validation_messages():
    variant = CpuVariant("g")
    life = _life()
    graph = variant.prepare(CASE, life.fixtures["A"].inputs, options={}, mode=RunMode.CORRECTNESS)
    assert len(lifecycle.validate_graph(graph)) == 2
    backwards = PreparedGraph(descriptor=graph.descriptor, nodes=graph.nodes[::-1],
                              initial_artifacts=graph.initial_artifacts, terminal_artifact="indices", metadata={})
    with pytest.raises(ValueError, match="depends on later or unknown stages"):
        lifecycle.validate_graph(backwards)
    no_terminal = PreparedGraph(descriptor=graph.descriptor, nodes=graph.nodes[:1],
                                initial_artifacts=graph.initial_artifacts, terminal_artifact="indices", metadata={})
    with pytest.raises(ValueError, match="terminal artifact"):
        lifecycle.validate_graph(no_terminal)
    assert lifecycle.graph_fingerprint(graph) == lifecycle.graph_fingerprint(graph)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,keys", [(64, 8192), (256, 16384)])
def test_fused_operator_passes_the_lifecycle_against_the_dense_variant(rows, keys):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    case = PrefillCase(f"prefill_q{rows}_n{keys}", rows, keys, top_k=2048, seed=0)
    record = lifecycle.check_variant(case, device="cuda:0")
    assert record["status"] == "passed"
    for check in record["checks"]:
        for verdict in check["checks"].values():
            assert verdict["contract_check"]["status"] == "passed"
            assert verdict["exact_reference_check"]["status"] == "passed"
    assert len(record["lifecycle"]["integrity_checks"]) == 4


@pytest.mark.gpu
def test_replay_factory_feeds_the_lifecycle(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fusedindextopk_b200 import replay
    from fusedindextopk_b200.inputs import make_workload_inputs

    items = [(split, make_workload_inputs("c4", query_tokens=64, context_tokens=8192, fixture_id=fixture))
             for split in replay.REPLAY_SPLITS for fixture in ("A", "B")]
    manifest = replay.write_replay_dataset(tmp_path / "set", "life-set", items)
    factory = replay.ReplayInputFactory(manifest, split="test_hard")
    case = factory.cases()[0]
    record = lifecycle.check_variant(case, device="cuda:0", input_factory=factory)
    assert record["status"] == "passed"
    ties = [record["oracle"]["fixtures"][name]["cutoff_tie_check"] for name in ("A", "B")]
    assert all(item["status"] == "passed" for item in ties)
