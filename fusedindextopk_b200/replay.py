"""Frozen replay inputs: safetensors files with the six operator tensors plus a manifest.

The reference replays captured real workloads through the same operator contract
(``src/fused_index_topk/replay.py:20-300``).  Its captures are not redistributed,
but anyone who holds them (or makes new ones) can run them on this operator: this
module reads and writes the same on-disk format

* one ``.safetensors`` file per (split, case, fixture) holding exactly
  ``q, kv, kv_scales, weights, k_start, k_end``;
* a JSON manifest, ``schema_version`` 1, ``frozen`` true, a ``dataset_id`` and an
  ``items`` list; every item names ``item_id``, ``split`` (``tuning``,
  ``test_normal`` or ``test_hard``; all three must occur), ``case_id``,
  ``fixture_id`` (``A``/``B``), a relative ``path``, the file's ``sha256`` and the
  ``case`` shape (query/context tokens, top_k, heads, head_dim)

with the same names, checks and error behaviour, so that files written by either
side load on the other (a golden test pins the bytes written here against the
bytes the reference writes for the same tensors).

On a CUDA target the tensors are staged through pinned host memory and copied
with asynchronous transfers on the current stream.
"""

from __future__ import annotations

import hashlib
import json
import os
import tempfile
from dataclasses import asdict
from pathlib import Path
from typing import Any, Mapping

from .api import PrefillCase, PrefillInputs

REPLAY_SCHEMA_VERSION = 1
REPLAY_TENSOR_NAMES = ("q", "kv", "kv_scales", "weights", "k_start", "k_end")
REPLAY_SPLITS = ("tuning", "test_normal", "test_hard")
_CASE_FIELDS = ("query_tokens", "context_tokens", "top_k", "indexer_heads", "head_dim")
_DEFAULT_KV_QUANTIZATION = "dsv32-act-quant-group128-fp8-e4m3fn"


def sha256_file(path: str | os.PathLike[str]) -> str:
    """Hex SHA-256 of a file, read in 16 MiB pieces."""

    digest = hashlib.sha256()
    with open(path, "rb") as handle:
        while True:
            block = handle.read(1 << 24)
            if not block:
                break
            digest.update(block)
    return digest.hexdigest()


def _relative_item_path(value: object) -> Path:
    path = Path(str(value))
    if path.is_absolute() or ".." in path.parts:
        raise ValueError(f"replay item path must be a safe relative path: {path}")
    return path


def _is_sha256(text: str) -> bool:
    return len(text) == 64 and all(character in "0123456789abcdef" for character in text)


def validate_replay_manifest(value: Mapping[str, Any]) -> dict[str, Any]:
    """Check the portable part of a manifest; raises ``ValueError`` with the reference's wording."""

    if int(value.get("schema_version", -1)) != REPLAY_SCHEMA_VERSION:
        raise ValueError("unsupported replay manifest schema_version")
    if not value.get("dataset_id"):
        raise ValueError("replay manifest requires dataset_id")
    if value.get("frozen") is not True:
        raise ValueError("formal replay manifests must be frozen")
    items = value.get("items")
    if not isinstance(items, list) or not items:
        raise ValueError("replay manifest requires a non-empty items list")

    seen_ids: set[str] = set()
    seen_keys: set[tuple[str, str, str]] = set()
    seen_splits: set[str] = set()
    for item in items:
        if not isinstance(item, Mapping):
            raise ValueError("each replay item must be an object")
        item_id = str(item.get("item_id", ""))
        split = str(item.get("split", ""))
        case_id = str(item.get("case_id", ""))
        fixture_id = str(item.get("fixture_id", ""))
        if not item_id or item_id in seen_ids:
            raise ValueError(f"missing or duplicate replay item_id: {item_id!r}")
        if split not in REPLAY_SPLITS:
            raise ValueError(f"invalid replay split: {split!r}")
        if fixture_id not in ("A", "B"):
            raise ValueError(f"invalid fixture_id: {fixture_id!r}")
        if not case_id:
            raise ValueError("replay item requires case_id")
        if (split, case_id, fixture_id) in seen_keys:
            raise ValueError(f"duplicate replay fixture key: {(split, case_id, fixture_id)}")
        _relative_item_path(item.get("path"))
        if not _is_sha256(str(item.get("sha256", ""))):
            raise ValueError(f"invalid sha256 for replay item {item_id!r}")
        case = item.get("case")
        if not isinstance(case, Mapping):
            raise ValueError(f"replay item {item_id!r} requires case metadata")
        for name in _CASE_FIELDS:
            if int(case.get(name, 0)) <= 0:
                raise ValueError(f"invalid {name} for replay item {item_id!r}")
        seen_ids.add(item_id)
        seen_keys.add((split, case_id, fixture_id))
        seen_splits.add(split)

    absent = set(REPLAY_SPLITS) - seen_splits
    if absent:
        raise ValueError(f"replay manifest is missing splits: {sorted(absent)}")
    return {
        "status": "passed",
        "schema_version": REPLAY_SCHEMA_VERSION,
        "dataset_id": str(value["dataset_id"]),
        "items": len(items),
        "splits": sorted(seen_splits),
    }


def save_replay_tensors(path: str | os.PathLike[str], tensors: Mapping[str, Any], *,
                        metadata: Mapping[str, str] | None = None) -> dict[str, Any]:
    """Write the six CPU tensors to ``path`` atomically; returns path, size and SHA-256."""

    from safetensors.torch import save_file

    names = set(tensors)
    if names != set(REPLAY_TENSOR_NAMES):
        missing = sorted(set(REPLAY_TENSOR_NAMES) - names)
        extra = sorted(names - set(REPLAY_TENSOR_NAMES))
        raise ValueError(f"replay tensors mismatch: missing={missing} extra={extra}")
    ordered: dict[str, Any] = {}
    for name in REPLAY_TENSOR_NAMES:
        tensor = tensors[name]
        if tensor.device.type != "cpu":
            raise ValueError(f"replay tensor {name} must be on CPU before serialization")
        ordered[name] = tensor.contiguous()

    target = Path(path)
    target.parent.mkdir(parents=True, exist_ok=True)
    handle, scratch_name = tempfile.mkstemp(prefix=f".{target.name}.", suffix=".tmp", dir=target.parent)
    os.close(handle)
    scratch = Path(scratch_name)
    try:
        save_file(ordered, scratch, metadata=dict(metadata or {}))
        os.chmod(scratch, 0o644)
        os.replace(scratch, target)
    except BaseException:
        scratch.unlink(missing_ok=True)
        raise
    return {"path": str(target), "bytes": target.stat().st_size, "sha256": sha256_file(target)}


def replay_case_metadata(case: PrefillCase) -> dict[str, Any]:
    """The shape record stored beside every manifest item."""

    return asdict(case)


def _to_device(torch: Any, tensor: Any, device: Any) -> tuple[Any, Any]:
    """``(tensor on device, pinned staging buffer or None)``; CUDA copies are asynchronous."""

    if device.type != "cuda":
        return tensor.to(device).contiguous(), None
    staged = tensor.contiguous().pin_memory()
    moved = torch.empty(staged.shape, dtype=staged.dtype, device=device)
    moved.copy_(staged, non_blocking=True)
    return moved, staged


class ReplayInputFactory:
    """``factory(case, device, fixture_id) -> PrefillInputs`` for one split of a frozen dataset."""

    def __init__(self, manifest_path: str | os.PathLike[str], *, split: str, verify_sha256: bool = True) -> None:
        self.manifest_path = Path(manifest_path).resolve()
        self.root = self.manifest_path.parent
        with self.manifest_path.open("r", encoding="utf-8") as handle:
            self.manifest = json.load(handle)
        validate_replay_manifest(self.manifest)
        if split not in REPLAY_SPLITS:
            raise ValueError(f"invalid replay split: {split!r}")
        self.split = split
        self.verify_sha256 = verify_sha256
        self._verified: set[Path] = set()
        self._items = {
            (str(item["case_id"]), str(item["fixture_id"])): item
            for item in self.manifest["items"] if item["split"] == split
        }

    def _item(self, case: PrefillCase, fixture_id: str) -> Mapping[str, Any]:
        key = (case.case_id, fixture_id)
        if key not in self._items:
            raise KeyError(f"replay split {self.split!r} has no {fixture_id} fixture for {case.case_id!r}")
        item = self._items[key]
        for name in _CASE_FIELDS:
            if int(item["case"][name]) != int(getattr(case, name)):
                raise ValueError(
                    f"replay case mismatch for {name}: manifest={item['case'][name]} runtime={getattr(case, name)}"
                )
        return item

    def __call__(self, case: PrefillCase, device: str | Any, fixture_id: str) -> PrefillInputs:
        import torch
        from safetensors.torch import load_file

        item = self._item(case, fixture_id)
        path = (self.root / _relative_item_path(item["path"])).resolve()
        if not path.is_relative_to(self.root):
            raise ValueError(f"replay item escapes dataset root: {path}")
        if self.verify_sha256 and path not in self._verified:
            actual = sha256_file(path)
            if actual != item["sha256"]:
                raise RuntimeError(
                    f"replay item checksum mismatch for {path}: expected={item['sha256']} actual={actual}"
                )
            self._verified.add(path)
        payload = load_file(path, device="cpu")
        if set(payload) != set(REPLAY_TENSOR_NAMES):
            raise ValueError(f"replay file has unexpected tensors: {sorted(payload)}")

        target = torch.device(device)
        loaded: dict[str, Any] = {}
        staging = []
        for name in REPLAY_TENSOR_NAMES:
            loaded[name], pinned = _to_device(torch, payload[name], target)
            if pinned is not None:
                staging.append(pinned)
        if staging:
            torch.cuda.current_stream(target).synchronize()   # the pinned staging buffers may go now

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
            "kv_quantization": item.get("kv_quantization", _DEFAULT_KV_QUANTIZATION),
        }
        return PrefillInputs(
            case=case,
            generation_context_tokens=case.context_tokens,
            fixture_id=fixture_id,
            stream_seeds={},
            recipe_version=str(self.manifest.get("recipe_version", "dsv32-real-replay-v1")),
            recipe_metadata=provenance,
            **loaded,
        )

    def cases(self, *, seed: int = 0) -> tuple[PrefillCase, ...]:
        """Cases of the split that have both fixtures, by context length then id."""

        shapes: dict[str, Mapping[str, Any]] = {}
        fixtures: dict[str, set[str]] = {}
        for (case_id, fixture_id), item in self._items.items():
            shapes[case_id] = item["case"]
            fixtures.setdefault(case_id, set()).add(fixture_id)
        incomplete = sorted(case_id for case_id, have in fixtures.items() if have != {"A", "B"})
        if incomplete:
            raise ValueError(f"replay cases without complete A/B fixtures: {incomplete}")
        ordered = sorted(shapes, key=lambda case_id: (int(shapes[case_id]["context_tokens"]), case_id))
        return tuple(
            PrefillCase(
                case_id=case_id,
                query_tokens=int(shapes[case_id]["query_tokens"]),
                context_tokens=int(shapes[case_id]["context_tokens"]),
                top_k=int(shapes[case_id]["top_k"]),
                seed=seed,
                batch_size=int(shapes[case_id].get("batch_size", 1)),
                indexer_heads=int(shapes[case_id]["indexer_heads"]),
                head_dim=int(shapes[case_id]["head_dim"]),
                causal=bool(shapes[case_id].get("causal", True)),
            )
            for case_id in ordered
        )


def write_replay_dataset(root: str | os.PathLike[str], dataset_id: str,
                         items: list[tuple[str, PrefillInputs]], *, recipe_version: str | None = None) -> Path:
    """Write ``(split, inputs)`` pairs as a frozen dataset under ``root``; returns the manifest path.

    Convenience for making replay sets from this package's own workloads (or from
    tensors captured elsewhere and wrapped in ``PrefillInputs``); the reference has
    a capture script for this, which is outside the operator path.
    """

    base = Path(root)
    records = []
    for split, inputs in items:
        case = inputs.case
        relative = Path(split) / f"{case.case_id}-{inputs.fixture_id}.safetensors"
        saved = save_replay_tensors(
            base / relative,
            {name: getattr(inputs, name).cpu() for name in REPLAY_TENSOR_NAMES},
            # one key: the safetensors writer orders several metadata keys differently from
            # process to process, which would make the file's SHA-256 irreproducible
            metadata={"item": f"{case.case_id}:{inputs.fixture_id}"},
        )
        records.append({
            "item_id": f"{split}/{case.case_id}/{inputs.fixture_id}",
            "split": split, "case_id": case.case_id, "fixture_id": inputs.fixture_id,
            "path": str(relative), "sha256": saved["sha256"], "bytes": saved["bytes"],
            "case": replay_case_metadata(case),
            "kv_quantization": str(dict(inputs.recipe_metadata).get("kv_quantization", _DEFAULT_KV_QUANTIZATION)),
        })
    manifest = {"schema_version": REPLAY_SCHEMA_VERSION, "dataset_id": dataset_id, "frozen": True, "items": records}
    if recipe_version is not None:
        manifest["recipe_version"] = recipe_version
    validate_replay_manifest(manifest)
    manifest_path = base / "manifest.json"
    manifest_path.parent.mkdir(parents=True, exist_ok=True)
    manifest_path.write_text(json.dumps(manifest, indent=1, sort_keys=True) + "\n")
    return manifest_path


__all__ = [
    "REPLAY_SCHEMA_VERSION", "REPLAY_SPLITS", "REPLAY_TENSOR_NAMES", "ReplayInputFactory", "replay_case_metadata",
    "save_replay_tensors", "sha256_file", "validate_replay_manifest", "write_replay_dataset",
]
