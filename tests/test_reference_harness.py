"""The plugin under the reference's own harness code.

The reference loads operator variants through its registry
(``src/fused_index_topk/registry.py:58-101``: factory lookup, ``isinstance`` check of the descriptor
against ITS ``VariantDescriptor``, API major version, mode, ``exact_topk``), validates prepared graphs
(``graph.py``) and checks a candidate with its A/B lifecycle (``lifecycle.py:240-347``: oracle from an
unfused variant on fixtures A and B, candidate prepared once on A, checked on A, B, A, input content
hashes re-verified after every phase).  These tests run exactly that code on this package's plugin.
They need the reference's Python package to be importable (see ``conftest.py``) and skip otherwise.
"""

from __future__ import annotations

import sys
import tomllib
from pathlib import Path
from types import SimpleNamespace

import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))

reference_registry = pytest.importorskip("fused_index_topk.registry", reason="the reference package is not importable")

from fused_index_topk import api as reference_api  # noqa: E402
from fused_index_topk.graph import validate_graph  # noqa: E402

from fusedindextopk_b200 import api  # noqa: E402

FACTORY = "fusedindextopk_b200.plugin:create_variant"
DENSE_FACTORY = "fusedindextopk_b200.variants:create_dense_variant"
# the tensor contract the reference's lab configuration states (configs/fused_index_topk_h20.json, "workload")
WORKLOAD = SimpleNamespace(q_dtype="float8_e4m3fn", kv_dtype="float8_e4m3fn", kv_scale_dtype="float32",
                           weight_dtype="float32", range_dtype="int32")


def test_this_package_speaks_the_reference_classes():
    assert api.reference_api is reference_api
    assert api.VariantDescriptor is reference_api.VariantDescriptor
    assert api.PreparedGraph is reference_api.PreparedGraph


def test_reference_registry_loads_the_plugin():
    plugin = reference_registry.load_variant(FACTORY)
    assert isinstance(plugin.descriptor, reference_api.VariantDescriptor)
    assert plugin.descriptor.mode == "fused" and plugin.descriptor.exact_topk
    assert plugin.descriptor.api_version.split(".")[0] == "1"
    assert plugin.descriptor.supported_arches == ("sm100",)
    case = reference_api.PrefillCase("shape", 4096, 16384, 2048, 0)
    assert plugin.supports(case)
    assert isinstance(plugin.fingerprint_metadata(), dict)
    # configured options go through the same door
    configured = reference_registry.load_variant(FACTORY, options={"sample_guard_sigmas": 2.5})
    assert configured.fingerprint_metadata()["options"]["sample_guard_sigmas"] == 2.5
    with pytest.raises(ValueError):
        reference_registry.load_variant(FACTORY, options={"no_such_option": 1})


def test_reference_registry_loads_the_dense_checking_variant():
    plugin = reference_registry.load_variant(DENSE_FACTORY)
    assert plugin.descriptor.mode == "unfused" and plugin.descriptor.exact_topk


def test_entry_point_is_declared_in_the_group_the_registry_scans():
    project = tomllib.loads((ROOT / "pyproject.toml").read_text())
    group = project["project"]["entry-points"][reference_registry.ENTRY_POINT_GROUP]
    assert group["fused_index_topk_b200"] == FACTORY


@pytest.mark.gpu
@pytest.mark.parametrize("rows,keys", [(64, 8192), (32, 32768)])
def test_plugin_passes_the_reference_lifecycle(rows, keys):
    torch = pytest.importorskip("torch")
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fused_index_topk.lifecycle import CaseLifecycle

    case = reference_api.PrefillCase(f"q{rows}-n{keys}", rows, keys, 2048, 0)
    candidate = reference_registry.load_variant(FACTORY)
    life = CaseLifecycle(case=case, workload=WORKLOAD, reference=reference_registry.load_variant(DENSE_FACTORY),
                         reference_options={}, mode=reference_api.RunMode.CORRECTNESS, device="cuda:0")
    oracle = life.build_oracles()
    assert oracle["status"] == "passed"
    graph = life.prepare_candidate(candidate, {})
    assert len(validate_graph(graph)) == len(graph.nodes) == 3   # sample threshold, fused top-k, repair
    record = life.check_candidate(phase="check", order=("A", "B", "A"))
    assert record["status"] == "passed" and record["order"] == ["A", "B", "A"]
    for check in record["checks"].values():
        assert check["contract_check"]["status"] == "passed"
        assert check["exact_reference_check"]["status"] == "passed"
    meta = life.metadata()
    assert meta["anti_precompute_gate"]["required_execution_fixtures"] == ["A", "B"]
    assert meta["candidate_graph_fingerprint"] and meta["reference_graph_fingerprint"]
