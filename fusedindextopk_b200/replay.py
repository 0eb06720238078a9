"""Replay sets: the operator's six input tensors frozen on disk.

The reference measures on tensors captured from a real model and replays them from
``.safetensors`` files listed in a JSON manifest (``src/fused_index_topk/replay.py:20-300``).
Those captures are not redistributed; whoever holds them, or makes new ones, can run
them here, because this module speaks the same format:

* a file per (split, case, fixture) with exactly ``q, kv, kv_scales, weights, k_start, k_end``;
* a manifest (``schema_version`` 1, ``frozen`` true, ``dataset_id``, ``items``) whose items carry
  ``item_id``, ``split`` (all of ``tuning``, ``test_normal``, ``test_hard`` must occur),
  ``case_id``, ``fixture_id`` (``A``/``B``), a relative ``path``, the file's ``sha256`` and the
  ``case`` shape.

Files written by one side load on the other, and a manifest gets the same verdict, word
for word, from both validators: golden tests pin the bytes written here and the messages
raised here against the reference's.  Tensors bound for a CUDA device are staged through
pinned memory and copied asynchronously on the current stream.
"""

from __future__ import annotations

import hashlib
import json
import os
import tempfile
from dataclasses import asdict
from pathlib import Path
from typing import Any, Iterator, Mapping

from .api import PrefillCase, PrefillInputs

REPLAY_SCHEMA_VERSION = 1
REPLAY_TENSOR_NAMES = ("q", "kv", "kv_scales", "weights", "k_start", "k_end")
REPLAY_SPLITS = ("tuning", "test_normal", "test_hard")
_SHAPE_FIELDS = ("query_tokens", "context_tokens", "top_k", "indexer_heads", "head_dim")
_KV_RECIPE = "dsv32-act-quant-group128-fp8-e4m3fn"
_HEX = frozenset("0123456789abcdef")


def sha256_file(path: str | os.PathLike[str]) -> str:
    """Hex SHA-256 of a file."""

    with open(path, "rb") as handle:
        return hashlib.file_digest(handle, "sha256").hexdigest()


def _inside(path: object) -> Path:
    relative = Path(str(path))
    if relative.is_absolute() or ".." in relative.parts:
        raise ValueError(f"replay item path must be a safe relative path: {relative}")
    return relative


def _item_faults(item: Any, ids: set, keys: set) -> Iterator[str]:
    """The complaints about one manifest item, in the order the reference raises them."""

    if not isinstance(item, Mapping):
        yield "each replay item must be an object"
        return
    name, split, case_id, fixture = (str(item.get(k, "")) for k in ("item_id", "split", "case_id", "fixture_id"))
    if not name or name in ids:
        yield f"missing or duplicate replay item_id: {name!r}"
    if split not in REPLAY_SPLITS:
        yield f"invalid replay split: {split!r}"
    if fixture not in ("A", "B"):
        yield f"invalid fixture_id: {fixture!r}"
    if not case_id:
        yield "replay item requires case_id"
    if (split, case_id, fixture) in keys:
        yield f"duplicate replay fixture key: {(split, case_id, fixture)}"
    _inside(item.get("path"))
    digest = str(item.get("sha256", ""))
    if len(digest) != 64 or not set(digest) <= _HEX:
        yield f"invalid sha256 for replay item {name!r}"
    shape = item.get("case")
    if not isinstance(shape, Mapping):
        yield f"replay item {name!r} requires case metadata"
        return
    for field in _SHAPE_FIELDS:
        if int(shape.get(field, 0)) <= 0:
            yield f"invalid {field} for replay item {name!r}"


def validate_replay_manifest(value: Mapping[str, Any]) -> dict[str, Any]:
    """Summary of a well-formed manifest; the first fault raises ``ValueError``."""

    items = value.get("items")
    header = (
        (int(value.get("schema_version", -1)) == REPLAY_SCHEMA_VERSION, "unsupported replay manifest schema_version"),
        (bool(value.get("dataset_id")), "replay manifest requires dataset_id"),
        (value.get("frozen") is True, "formal replay manifests must be frozen"),
        (isinstance(items, list) and bool(items), "replay manifest requires a non-empty items list"),
    )
    for fine, complaint in header:
        if not fine:
            raise ValueError(complaint)
    ids: set[str] = set()
    keys: set[tuple[str, str, str]] = set()
    for item in items:
        for complaint in _item_faults(item, ids, keys):
            raise ValueError(complaint)
        ids.add(str(item["item_id"]))
        keys.add((str(item["split"]), str(item["case_id"]), str(item["fixture_id"])))
    present = {split for split, _, _ in keys}
    if present != set(REPLAY_SPLITS):
        raise ValueError(f"replay manifest is missing splits: {sorted(set(REPLAY_SPLITS) - present)}")
    return {"status": "passed", "schema_version": REPLAY_SCHEMA_VERSION, "dataset_id": str(value["dataset_id"]),
            "items": len(items), "splits": sorted(present)}


def save_replay_tensors(path: str | os.PathLike[str], tensors: Mapping[str, Any], *,
                        metadata: Mapping[str, str] | None = None) -> dict[str, Any]:
    """Write the six CPU tensors to ``path`` (via a temporary file beside it); returns path, size, SHA-256."""

    from safetensors.torch import save_file

    wanted, given = set(REPLAY_TENSOR_NAMES), set(tensors)
    if given != wanted:
        raise ValueError(f"replay tensors mismatch: missing={sorted(wanted - given)} extra={sorted(given - wanted)}")
    for name in REPLAY_TENSOR_NAMES:
        if tensors[name].device.type != "cpu":
            raise ValueError(f"replay tensor {name} must be on CPU before serialization")
    target = Path(path)
    target.parent.mkdir(parents=True, exist_ok=True)
    descriptor, scratch = tempfile.mkstemp(prefix=f".{target.name}.", suffix=".tmp", dir=target.parent)
    os.close(descriptor)
    try:
        save_file({name: tensors[name].contiguous() for name in REPLAY_TENSOR_NAMES}, scratch,
                  metadata=dict(metadata or {}))
        os.chmod(scratch, 0o644)
        os.replace(scratch, target)
    finally:
        Path(scratch).unlink(missing_ok=True)
    return {"path": str(target), "bytes": target.stat().st_size, "sha256": sha256_file(target)}


def replay_case_metadata(case: PrefillCase) -> dict[str, Any]:
    """The shape record stored beside every manifest item."""

    return asdict(case)


class ReplayInputFactory:
    """``factory(case, device, fixture_id) -> PrefillInputs`` over one split of a frozen set."""

    def __init__(self, manifest_path: str | os.PathLike[str], *, split: str, verify_sha256: bool = True) -> None:
        self.manifest_path = Path(manifest_path).resolve()
        self.root = self.manifest_path.parent
        self.manifest = json.loads(self.manifest_path.read_text(encoding="utf-8"))
        validate_replay_manifest(self.manifest)
        if split not in REPLAY_SPLITS:
            raise ValueError(f"invalid replay split: {split!r}")
        self.split = split
        self.verify_sha256 = verify_sha256
        self._checked: set[Path] = set()
        self._items = {(str(item["case_id"]), str(item["fixture_id"])): item
                       for item in self.manifest["items"] if item["split"] == split}

    def _checked_file(self, item: Mapping[str, Any]) -> Path:
        path = (self.root / _inside(item["path"])).resolve()
        if not path.is_relative_to(self.root):
            raise ValueError(f"replay item escapes dataset root: {path}")
        if self.verify_sha256 and path not in self._checked:
            found = sha256_file(path)
            if found != item["sha256"]:
                raise RuntimeError(f"replay item checksum mismatch for {path}: expected={item['sha256']} actual={found}")
            self._checked.add(path)
        return path

    def __call__(self, case: PrefillCase, device: str | Any, fixture_id: str) -> PrefillInputs:
        import torch
        from safetensors.torch import load_file

        try:
            item = self._items[(case.case_id, fixture_id)]
        except KeyError:
            raise KeyError(f"replay split {self.split!r} has no {fixture_id} fixture for {case.case_id!r}") from None
        for field in _SHAPE_FIELDS:
            if int(item["case"][field]) != int(getattr(case, field)):
                raise ValueError(f"replay case mismatch for {field}: manifest={item['case'][field]} "
                                 f"runtime={getattr(case, field)}")
        stored = load_file(self._checked_file(item), device="cpu")
        if set(stored) != set(REPLAY_TENSOR_NAMES):
            raise ValueError(f"replay file has unexpected tensors: {sorted(stored)}")

        target = torch.device(device)
        if target.type == "cuda":
            pinned = {name: stored[name].contiguous().pin_memory() for name in REPLAY_TENSOR_NAMES}
            tensors = {name: torch.empty_like(value, device=target) for name, value in pinned.items()}
            for name, value in pinned.items():
                tensors[name].copy_(value, non_blocking=True)
            torch.cuda.current_stream(target).synchronize()   # the pinned buffers are released on return
        else:
            tensors = {name: stored[name].to(target).contiguous() for name in REPLAY_TENSOR_NAMES}
        provenance = {
            "dataset_id": self.manifest["dataset_id"],
            "dataset_manifest": str(self.manifest_path),
            "dataset_manifest_sha256": sha256_file(self.manifest_path),
            "replay_split": self.split,
            "replay_item_id": item["item_id"],
            "replay_file": item["path"],
            "replay_file_sha256": item["sha256"],
            "capture": dict(item.get("capture", {})),
            "score_statistics": dict(item.get("score_statistics", {})),
            "generation_order": "frozen_replay_load",
            "kv_quantization": item.get("kv_quantization", _KV_RECIPE),
        }
        return PrefillInputs(case=case, generation_context_tokens=case.context_tokens, fixture_id=fixture_id,
                             stream_seeds={}, recipe_metadata=provenance,
                             recipe_version=str(self.manifest.get("recipe_version", "dsv32-real-replay-v1")), **tensors)

    def cases(self, *, seed: int = 0) -> tuple[PrefillCase, ...]:
        """The split's cases that have both fixtures, shortest context first."""

        shapes: dict[str, Mapping[str, Any]] = {}
        have: dict[str, set[str]] = {}
        for (case_id, fixture_id), item in self._items.items():
            shapes[case_id] = item["case"]
            have.setdefault(case_id, set()).add(fixture_id)
        partial = sorted(case_id for case_id, fixtures in have.items() if fixtures != {"A", "B"})
        if partial:
            raise ValueError(f"replay cases without complete A/B fixtures: {partial}")
        def shaped(case_id: str) -> PrefillCase:
            shape = shapes[case_id]
            numbers = {name: int(shape[name]) for name in (*_SHAPE_FIELDS, "batch_size") if name in shape}
            return PrefillCase(case_id=case_id, seed=seed, causal=bool(shape.get("causal", True)), **numbers)

        return tuple(shaped(case_id)
                     for case_id in sorted(shapes, key=lambda name: (int(shapes[name]["context_tokens"]), name)))


def write_replay_dataset(root: str | os.PathLike[str], dataset_id: str,
                         items: list[tuple[str, PrefillInputs]], *, recipe_version: str | None = None) -> Path:
    """Freeze ``(split, inputs)`` pairs under ``root`` and return the manifest path.

    For replay sets made from this package's own workloads or from tensors captured
    elsewhere and wrapped in ``PrefillInputs``.
    """

    base = Path(root)
    records = []
    for split, inputs in items:
        case = inputs.case
        relative = Path(split) / f"{case.case_id}-{inputs.fixture_id}.safetensors"
        # a single metadata key: the writer orders several keys differently from process to process,
        # which would make the file's SHA-256 irreproducible
        saved = save_replay_tensors(base / relative, {name: getattr(inputs, name).cpu() for name in REPLAY_TENSOR_NAMES},
                                    metadata={"item": f"{case.case_id}:{inputs.fixture_id}"})
        records.append({
            "item_id": f"{split}/{case.case_id}/{inputs.fixture_id}", "split": split, "case_id": case.case_id,
            "fixture_id": inputs.fixture_id, "path": str(relative), "sha256": saved["sha256"], "bytes": saved["bytes"],
            "case": replay_case_metadata(case),
            "kv_quantization": str(dict(inputs.recipe_metadata).get("kv_quantization", _KV_RECIPE)),
        })
    manifest = {"schema_version": REPLAY_SCHEMA_VERSION, "dataset_id": dataset_id, "frozen": True, "items": records}
    if recipe_version is not None:
        manifest["recipe_version"] = recipe_version
    validate_replay_manifest(manifest)
    base.mkdir(parents=True, exist_ok=True)
    (base / "manifest.json").write_text(json.dumps(manifest, indent=1, sort_keys=True) + "\n")
    return base / "manifest.json"


__all__ = [
    "REPLAY_SCHEMA_VERSION", "REPLAY_SPLITS", "REPLAY_TENSOR_NAMES", "ReplayInputFactory", "replay_case_metadata",
    "save_replay_tensors", "sha256_file", "validate_replay_manifest", "write_replay_dataset",
]
