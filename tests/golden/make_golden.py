"""Regenerate ``reference_golden.json`` from the reference's own Python layer.

Run where the reference checkout is available (it is not on the GPU box):

    python tests/golden/make_golden.py /path/to/reference

The reference's CUDA kernels and its DeepGEMM scorer cannot run without their
GPU and third-party dependency, but its pure-Python host layer imports on a
CPU.  This script calls that layer (sample schedule, guarded rank, sample
positions, RNG stream seeds, the standard input recipe, the row-wise key
quantisation, the replay file format and manifest checks, the output-contract
validator and the cutoff-tie oracle) and records inputs and outputs as small
fixtures; the tests replay them against this package's own implementations.
"""

from __future__ import annotations

import hashlib
import json
import sys
from pathlib import Path


def _digest(tensor) -> str:
    import torch

    return hashlib.sha256(tensor.contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def main(reference_root: str) -> None:
    sys.path.insert(0, str(Path(reference_root) / "src"))
    import torch
    from fused_index_topk.api import PrefillCase
    from fused_index_topk.correctness import (
        CorrectnessError,
        build_score_threshold_oracle,
        compare_topk_indices,
        validate_topk_indices,
    )
    from fused_index_topk.inputs import (
        input_stream_seeds,
        make_prefill_inputs,
        quantize_contiguous_index_kv,
    )
    from fused_index_topk.kernel.plugin import (
        _SAMPLING_SEED_XOR,
        _TARGET_CANDIDATES,
        production_sample_elements,
    )
    from fused_index_topk.kernel.sampling import common_random_sample_ids, guarded_sample_rank

    golden: dict = {"source": "EdgePro001/FusedIndexTopK v0.3.0 python host layer"}

    # 1. sample schedule + guarded rank + sample positions
    schedule = []
    for context in (8192, 12288, 16384, 16512, 32768, 40000, 65536, 98304, 131072, 163840):
        samples = production_sample_elements(context)
        rank = guarded_sample_rank(
            samples, context, target_candidates=_TARGET_CANDIDATES, guard_sigmas=2.0
        )
        rank_loose = guarded_sample_rank(samples, context, target_candidates=3072, guard_sigmas=0.5)
        seed = (0 ^ _SAMPLING_SEED_XOR) & ((1 << 63) - 1)
        ids = common_random_sample_ids(torch, context, samples, seed=seed, device="cpu")
        schedule.append(
            {
                "context_tokens": context,
                "sample_elements": samples,
                "sample_rank": rank,
                "sample_rank_target3072_guard0p5": rank_loose,
                "sampling_seed": seed,
                "sample_ids_sha256": _digest(ids),
                "sample_ids_head": ids[:8].tolist(),
                "sample_ids_tail": ids[-4:].tolist(),
            }
        )
    golden["sampling"] = schedule

    # 2. RNG stream seeds
    golden["stream_seeds"] = {
        f"{seed}:{fixture}": input_stream_seeds(seed, fixture)
        for seed in (0, 1, 20260803)
        for fixture in ("A", "B")
    }

    # 3. the standard input recipe, generated on the CPU
    recipe = []
    for rows, keys, seed, fixture in ((6, 96, 0, "A"), (8, 8192, 0, "A"), (8, 8192, 0, "B"), (64, 512, 7, "B")):
        case = PrefillCase(f"golden-q{rows}-n{keys}", rows, keys, top_k=min(2048, keys), seed=seed)
        made = make_prefill_inputs(case, device="cpu", fixture_id=fixture)
        recipe.append(
            {
                "query_tokens": rows, "context_tokens": keys, "seed": seed, "fixture_id": fixture,
                "sha256": {
                    name: _digest(getattr(made, name))
                    for name in ("q", "kv", "kv_scales", "weights", "k_start", "k_end")
                },
                "kv_scales_head": made.kv_scales[:4].tolist(),
                "weights_head": made.weights[0, :4].tolist(),
            }
        )
    golden["input_recipe"] = recipe

    # 4. cutoff-tie oracle and tie-aware comparison on small dense score matrices
    tie_cases = []
    generator = torch.Generator().manual_seed(1234)
    for rows, keys, top_k, levels in ((4, 12, 3, 5), (6, 40, 8, 6), (5, 64, 16, 4), (8, 33, 5, 50)):
        case = PrefillCase("tie", rows, keys, top_k=top_k, seed=0)
        values = torch.randint(0, levels, (rows, keys), generator=generator).float()
        position = torch.arange(keys)[None, :]
        ends = torch.arange(keys - rows + 1, keys + 1)[:, None]
        scores = torch.where(position < ends, values, torch.full_like(values, -float("inf")))
        top_values, top_ids = torch.topk(scores, top_k, dim=-1, sorted=False)
        baseline = torch.where(torch.isfinite(top_values), top_ids, torch.full_like(top_ids, -1))
        baseline = baseline.to(torch.int32).unsqueeze(1).contiguous()
        summary, tie_rows = build_score_threshold_oracle(scores, baseline, case)
        # a candidate that swaps one tied id per tied row, and one that takes a low id
        swapped = baseline.clone()
        broken = baseline.clone()
        for row, tie in tie_rows.items():
            chosen = set(int(v) for v in baseline[row, 0].tolist())
            spare = [b for b in tie["boundary_ids"] if b not in chosen]
            used = [b for b in tie["boundary_ids"] if b in chosen]
            if spare and used:
                column = baseline[row, 0].tolist().index(used[0])
                swapped[row, 0, column] = spare[0]
        verdict_swapped = compare_topk_indices(swapped, baseline, case, cutoff_tie_rows=tie_rows)
        # replace a strictly-above-cutoff id by an unselected one -> must be rejected
        rejected = None
        for row in range(rows):
            end = keys - rows + row + 1
            if end <= top_k:
                continue
            chosen = set(int(v) for v in baseline[row, 0].tolist() if v >= 0)
            live = scores[row, :end]
            cutoff = torch.topk(live, top_k).values[-1]
            above = [i for i in chosen if live[i] > cutoff]
            spare = [i for i in range(end) if i not in chosen]
            if above and spare:
                column = baseline[row, 0].tolist().index(above[0])
                broken[row, 0, column] = spare[0]
                try:
                    compare_topk_indices(broken, baseline, case, cutoff_tie_rows=tie_rows)
                    rejected = False
                except CorrectnessError:
                    rejected = True
                break
        tie_cases.append(
            {
                "rows": rows, "keys": keys, "top_k": top_k,
                "scores": [[None if v == -float("inf") else v for v in r] for r in scores.tolist()],
                "baseline": baseline.tolist(),
                "summary": summary,
                "tie_rows": {str(k): {kk: list(vv) if isinstance(vv, tuple) else vv for kk, vv in v.items()}
                             for k, v in tie_rows.items()},
                "swapped": swapped.tolist(),
                "swapped_verdict": verdict_swapped,
                "broken": broken.tolist(),
                "broken_rejected": rejected,
            }
        )
    golden["tie_oracle"] = tie_cases

    # 5. output-contract validator messages
    case = PrefillCase("small", 3, 3, top_k=4, seed=1)
    good = torch.tensor([[[0, -1, -1, -1]], [[1, 0, -1, -1]], [[2, 0, 1, -1]]], dtype=torch.int32)
    contract = {"good_summary": validate_topk_indices(good, case), "violations": []}
    for label, data in (
        ("duplicate", [[[0, -1, -1, -1]], [[1, 1, -1, -1]], [[2, 0, 1, -1]]]),
        ("outside", [[[1, -1, -1, -1]], [[1, 0, -1, -1]], [[2, 0, 1, -1]]]),
        ("count", [[[0, -1, -1, -1]], [[1, 0, -1, -1]], [[2, 0, -1, -1]]]),
        ("negative", [[[0, -2, -1, -1]], [[1, 0, -1, -1]], [[2, 0, 1, -1]]]),
    ):
        try:
            validate_topk_indices(torch.tensor(data, dtype=torch.int32), case)
            message = None
        except CorrectnessError as error:
            message = str(error)
        contract["violations"].append({"label": label, "data": data, "message": message})
    golden["output_contract"] = contract

    # 6. row-wise e4m3 quantisation of the index keys (fp32 and bf16 sources, edge rows)
    quantize = []
    for label, dtype, seed in (("float32", torch.float32, 11), ("bfloat16", torch.bfloat16, 12)):
        generator = torch.Generator().manual_seed(seed)
        source = torch.randn((20, 128), generator=generator) * torch.exp(
            2.0 * torch.randn((20, 1), generator=generator)
        )
        source[0] = 0.0                                   # amax floor 1e-4
        source[1] = source[1] * 1e-7                      # below the floor: codes near zero
        source[2] = source[2] * 1e6
        source[3, ::2] = -0.0
        source[4] = 0.0
        source[4, 0] = 448.0                              # scale exactly 1: ties land on code midpoints
        source[4, 1:9] = torch.tensor([17.0, 19.0, -21.0, 2.0 ** -10, 3 * 2.0 ** -10, -416.0 - 16.0, 0.0107421875, 1.0625])
        source = source.to(dtype).contiguous()
        values, scales = quantize_contiguous_index_kv(source)
        quantize.append(
            {
                "dtype": label,
                "rows": int(source.shape[0]),
                "source_hex": source.view(torch.uint8).numpy().tobytes().hex(),
                "values_hex": values.view(torch.uint8).numpy().tobytes().hex(),
                "scales_hex": scales.view(torch.uint8).numpy().tobytes().hex(),
            }
        )
    golden["quantize_index_kv"] = quantize

    # 7. replay format: bytes of a saved fixture and manifest validation verdicts
    import copy
    import tempfile

    from fused_index_topk.replay import save_replay_tensors, validate_replay_manifest

    case = PrefillCase("golden-q6-n96", 6, 96, top_k=96, seed=0)
    made = make_prefill_inputs(case, device="cpu", fixture_id="A")
    with tempfile.TemporaryDirectory() as scratch:
        saved = save_replay_tensors(
            Path(scratch) / "item.safetensors",
            {name: getattr(made, name) for name in ("q", "kv", "kv_scales", "weights", "k_start", "k_end")},
            # one key only: the writer's metadata map has no fixed order across processes
            metadata={"case_id": case.case_id},
        )
    shape = {"query_tokens": 6, "context_tokens": 96, "top_k": 96, "indexer_heads": 64, "head_dim": 128}
    good = {
        "schema_version": 1, "dataset_id": "golden", "frozen": True,
        "items": [
            {"item_id": f"{split}-{fixture}", "split": split, "case_id": "golden-q6-n96", "fixture_id": fixture,
             "path": f"{split}/{fixture}.safetensors", "sha256": "0" * 64, "case": shape}
            for split in ("tuning", "test_normal", "test_hard") for fixture in ("A", "B")
        ],
    }

    def verdict(manifest):
        try:
            return {"summary": validate_replay_manifest(manifest)}
        except ValueError as error:
            return {"error": str(error)}

    def broken(edit):
        manifest = copy.deepcopy(good)
        edit(manifest)
        return manifest

    manifests = {
        "good": good,
        "schema": broken(lambda m: m.update(schema_version=2)),
        "not_frozen": broken(lambda m: m.update(frozen=False)),
        "no_dataset": broken(lambda m: m.update(dataset_id="")),
        "no_items": broken(lambda m: m.update(items=[])),
        "duplicate_item": broken(lambda m: m["items"][1].update(item_id=m["items"][0]["item_id"])),
        "bad_split": broken(lambda m: m["items"][0].update(split="train")),
        "bad_fixture": broken(lambda m: m["items"][0].update(fixture_id="C")),
        "duplicate_key": broken(lambda m: m["items"][1].update(fixture_id="A")),
        "absolute_path": broken(lambda m: m["items"][0].update(path="/etc/passwd")),
        "parent_path": broken(lambda m: m["items"][0].update(path="../x.safetensors")),
        "bad_sha": broken(lambda m: m["items"][0].update(sha256="xyz")),
        "bad_shape": broken(lambda m: m["items"][0]["case"].update(top_k=0)),
        "missing_split": broken(lambda m: m.update(items=[i for i in m["items"] if i["split"] != "test_hard"])),
    }
    golden["replay"] = {
        "saved_bytes": saved["bytes"],
        "saved_sha256": saved["sha256"],
        "manifests": {name: {"manifest": value, "verdict": verdict(value)} for name, value in manifests.items()},
    }

    target = Path(__file__).resolve().parent / "reference_golden.json"
    target.write_text(json.dumps(golden, indent=1, sort_keys=True) + "\n")
    print(f"wrote {target} ({target.stat().st_size} bytes)")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of the reference repository>")
    main(sys.argv[1])
