"""Run by tests/test_gpu_two_ranks.py under torch.distributed.run, one process per GPU.

Every rank checks its shard of the benchmark's two partitionings on its own GPU: query-row shards
(c1 at full size, c2 and c3 with fewer rows) by exactness on the diagnostic build's own scores, and the
key-range shards of c3s (per-rank Top-2048 pairs, NCCL all-gather, merge) against the one-GPU result.
"""
import os, sys, math
from pathlib import Path
sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import torch, torch.distributed as dist
from fusedindextopk_b200 import operator, fused_index_topk, distributed as shards
from fusedindextopk_b200.inputs import inputs_to, make_workload_inputs
rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
torch.cuda.set_device(local); dev = torch.device("cuda", local)
dist.init_process_group("nccl", device_id=dev)
for workload, rows, keys in (("c1", 4096, 16384), ("c2", 1024, 65536), ("c3", 512, 163840)):
    full = make_workload_inputs(workload, query_tokens=rows, context_tokens=keys)
    host, _ = shards.shard_rows(full, rank, world)
    g = inputs_to(host, dev)
    t = (g.q, g.kv, g.kv_scales, g.weights, g.k_start, g.k_end)
    r = host.case.query_tokens
    for _ in range(3):
        ids = fused_index_topk(t[0], (t[1], t[2]), t[3], t[4], t[5]).clone()
    diag = operator.make_workspace(r, keys, dev, key_shards=1)
    logits = torch.full((r, keys), -math.inf, device=dev)
    operator.run_sample_thresholds(diag, *t); operator.run_fused_topk(diag, *t, diag_logits=logits, force_compute=True)
    torch.cuda.synchronize()
    chosen = torch.zeros_like(logits, dtype=torch.bool); chosen.scatter_(1, ids.long().clamp_min(0), True)
    inside = torch.where(chosen, logits, torch.full_like(logits, math.inf)).amin(1)
    outside = torch.where(chosen, torch.full_like(logits, -math.inf), logits).amax(1)
    ok = bool((inside >= outside).all()) and bool((chosen.sum(1) == 2048).all()) and int((ids < 0).sum()) == 0
    print(f"rank {rank}/{world} {workload} rows {r} x {keys}: exact on own scores {ok}", flush=True)
    assert ok
# key range (c3s)
full = make_workload_inputs("c3s")
gfull = inputs_to(full, dev)
want = fused_index_topk(gfull.q, (gfull.kv, gfull.kv_scales), gfull.weights, gfull.k_start, gfull.k_end).clone()
local_in, offset = shards.shard_keys(full, rank, world)
gl = inputs_to(local_in, dev)
ws = operator.make_workspace(local_in.case.query_tokens, local_in.case.context_tokens, dev, with_pairs=True)
pairs, counts = shards.gpu_local_pairs(ws, gl, offset)
gp, gc = shards.dist_all_gather(pairs), shards.dist_all_gather(counts)
merged = torch.empty((full.case.query_tokens, 2048), dtype=torch.int32, device=dev)
shards.gpu_merge(gp, gc, merged)
torch.cuda.synchronize()
same = (merged.sort(dim=-1).values == want.sort(dim=-1).values).all(dim=1)
print(f"rank {rank}/{world} c3s key-range merge: {int(same.sum())}/{same.numel()} rows equal to the one-GPU sets", flush=True)
assert int(same.sum()) >= same.numel() - 2
dist.destroy_process_group()
