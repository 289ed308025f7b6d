"""Expert-parallel routing on two CPU ranks over gloo: the numpy restatement of the device
algorithm (slot plan, slab exchange, owner-side expert projections, ordered combine; also with a layer's
rows in 2 and 3 chunks, each with its own share of every slab and its own announced row counts) must give
each rank exactly the bits the single-rank MoE block gives for the same rows."""
import os
import subprocess
import sys

import numpy as np

CHILD = r'''
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, sys.argv[3])
from oracle import engine, fjo

rank, world = int(sys.argv[1]), int(sys.argv[2])
dist.init_process_group("gloo", rank=rank, world_size=world)
cfg = dict(layers=1, hidden=128, q_heads=2, kv_heads=1, head_dim=64, experts=8, top_k=3, expert_intermediate=64, vocab=64,
           group_size=64, router_bits=8, eps=1e-6, theta=1e7, max_rows=8)
weights = engine.random_moe_weights(cfg, 5)
L = weights["layers"][0]
per = cfg["experts"] // world
local = {name: tuple(np.ascontiguousarray(t[rank * per:(rank + 1) * per]) for t in L[name]) for name in ("gate", "up", "down")}

def exchange(slabs):
    t = torch.from_numpy(np.ascontiguousarray(slabs).view(np.uint8).reshape(world, -1).copy())
    gathered = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(gathered, t)
    mine = np.stack([g.numpy()[rank] for g in gathered])            # [source, bytes addressed to me]
    return mine.view(slabs.dtype).reshape(slabs.shape)

rng = np.random.default_rng(40 + rank)
for rows in ([5, 8][rank], [3, 0][rank]):                            # the second round leaves rank 1 without rows
    normed = fjo.encode(rng.standard_normal((rows, cfg["hidden"])).astype(np.float32), fjo.BF16)
    residual = fjo.encode(rng.standard_normal((rows, cfg["hidden"])).astype(np.float32), fjo.BF16)
    want = engine.MoeOracle(cfg, weights, 2, 16).moe(normed, residual, L)[0] if rows else None
    for chunks in (1, 2, 3):                                         # 2 and 3: the chunked slot layout of the direct exchange
        got = engine.ep_moe_layer(rank, world, cfg, normed, residual, local, L["router"], exchange, chunks=chunks)
        if rows:
            assert np.array_equal(got, want), f"rank {rank}: expert-parallel block ({chunks} chunks) differs from the single-rank block"
dist.barrier()
dist.destroy_process_group()
print("EP_GLOO_OK", rank)
'''


def test_expert_parallel_block_on_two_gloo_ranks(tmp_path):
    script = tmp_path / "ep_gloo_child.py"
    script.write_text(CHILD)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29653")
    procs = [subprocess.Popen([sys.executable, str(script), str(rank), "2", root], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for rank in range(2)]
    for rank, p in enumerate(procs):
        try:
            out, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        assert p.returncode == 0 and "EP_GLOO_OK" in out, f"rank {rank}:\n{out[-3000:]}"
