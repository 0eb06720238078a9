"""The replay file format: bytes and manifest verdicts pinned against the reference's own
writer and validator, round trips through the factory, and (GPU) a replayed fixture through
the operator."""

from __future__ import annotations

import json

import pytest
import torch

from fusedindextopk_b200 import replay
from fusedindextopk_b200.api import PrefillCase
from fusedindextopk_b200.inputs import make_prefill_inputs, make_workload_inputs


def _tensors(inputs):
    return {name: getattr(inputs, name) for name in replay.REPLAY_TENSOR_NAMES}


def test_saved_file_is_byte_identical_to_the_reference_writer(golden, tmp_path):
    case = PrefillCase("golden-q6-n96", 6, 96, top_k=96, seed=0)
    made = make_prefill_inputs(case, device="cpu", fixture_id="A")
    saved = replay.save_replay_tensors(
        tmp_path / "item.safetensors", _tensors(made), metadata={"case_id": case.case_id}
    )
    assert saved["bytes"] == golden["replay"]["saved_bytes"]
    assert saved["sha256"] == golden["replay"]["saved_sha256"]
    assert replay.sha256_file(tmp_path / "item.safetensors") == saved["sha256"]


def test_manifest_verdicts_match_the_reference_validator(golden):
    assert len(golden["replay"]["manifests"]) >= 14
    for name, entry in golden["replay"]["manifests"].items():
        want = entry["verdict"]
        if "summary" in want:
            assert replay.validate_replay_manifest(entry["manifest"]) == want["summary"], name
        else:
            with pytest.raises(ValueError) as caught:
                replay.validate_replay_manifest(entry["manifest"])
            assert str(caught.value) == want["error"], name


def test_save_rejects_wrong_tensor_sets(tmp_path):
    made = make_prefill_inputs(PrefillCase("t", 2, 32, top_k=32, seed=1), device="cpu")
    tensors = _tensors(made)
    tensors.pop("weights")
    tensors["extra"] = made.k_end
    with pytest.raises(ValueError, match=r"missing=\['weights'\] extra=\['extra'\]"):
        replay.save_replay_tensors(tmp_path / "x.safetensors", tensors)
    assert not list(tmp_path.iterdir())      # nothing half-written is left behind


def _dataset(tmp_path):
    items = []
    for split, (rows, keys) in zip(replay.REPLAY_SPLITS, ((4, 256), (8, 128), (4, 512))):
        for fixture in ("A", "B"):
            made = make_workload_inputs("c1", query_tokens=rows, context_tokens=keys, fixture_id=fixture, seed=3)
            items.append((split, made))
    return replay.write_replay_dataset(tmp_path / "set", "unit-test-set", items), items


def test_factory_round_trips_every_tensor_bit_for_bit(tmp_path):
    manifest_path, items = _dataset(tmp_path)
    for split, made in items:
        factory = replay.ReplayInputFactory(manifest_path, split=split)
        cases = factory.cases(seed=3)
        assert [case.case_id for case in cases] == [made.case.case_id]
        assert cases[0] == made.case
        loaded = factory(made.case, "cpu", made.fixture_id)
        for name in replay.REPLAY_TENSOR_NAMES:
            got, want = getattr(loaded, name), getattr(made, name)
            assert got.dtype == want.dtype and got.shape == want.shape
            assert torch.equal(got.view(torch.uint8), want.view(torch.uint8)), name
        assert loaded.recipe_metadata["generation_order"] == "frozen_replay_load"
        assert loaded.recipe_metadata["replay_split"] == split
        assert loaded.recipe_version == "dsv32-real-replay-v1"


def test_factory_refuses_tampered_files_shape_mismatches_and_unknown_cases(tmp_path):
    manifest_path, items = _dataset(tmp_path)
    split, made = items[0]
    factory = replay.ReplayInputFactory(manifest_path, split=split)
    with pytest.raises(KeyError):
        factory(PrefillCase("nope", 4, 256, top_k=2048, seed=0), "cpu", "A")
    wrong = PrefillCase(made.case.case_id, 4, 512, top_k=made.case.top_k, seed=0)
    with pytest.raises(ValueError, match="replay case mismatch for context_tokens"):
        factory(wrong, "cpu", "A")
    with pytest.raises(ValueError, match="invalid replay split"):
        replay.ReplayInputFactory(manifest_path, split="train")
    manifest = json.loads(manifest_path.read_text())
    target = manifest_path.parent / manifest["items"][0]["path"]
    data = bytearray(target.read_bytes())
    data[-1] ^= 1
    target.write_bytes(bytes(data))
    with pytest.raises(RuntimeError, match="checksum mismatch"):
        replay.ReplayInputFactory(manifest_path, split=split)(made.case, "cpu", "A")


@pytest.mark.gpu
def test_replayed_fixture_gives_the_same_ids_as_the_generated_one(tmp_path):
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from fusedindextopk_b200.inputs import inputs_to
    from fusedindextopk_b200.operator import fused_index_topk

    device = torch.device("cuda:0")
    items = []
    for split in replay.REPLAY_SPLITS:
        for fixture in ("A", "B"):
            items.append((split, make_workload_inputs("c1", query_tokens=64, context_tokens=8192, fixture_id=fixture)))
    manifest_path = replay.write_replay_dataset(tmp_path / "set", "gpu-set", items)
    factory = replay.ReplayInputFactory(manifest_path, split="test_hard")
    case = factory.cases()[0]
    for fixture in ("A", "B"):
        loaded = factory(case, device, fixture)
        assert loaded.q.is_cuda and loaded.q.dtype == torch.float8_e4m3fn
        direct = inputs_to(next(m for s, m in items if s == "test_hard" and m.fixture_id == fixture), device)
        got = fused_index_topk(loaded.q, (loaded.kv, loaded.kv_scales), loaded.weights, loaded.k_start, loaded.k_end)
        want = fused_index_topk(direct.q, (direct.kv, direct.kv_scales), direct.weights, direct.k_start, direct.k_end)
        assert torch.equal(got.sort(dim=-1).values, want.sort(dim=-1).values)
