"""One rank of the two-GPU expert-parallel check (started by tests/test_gpu_moe.py). Each rank runs
its own lanes through the expert-parallel model and, on the same GPU, through a single-GPU model
holding all experts; the logits must agree bit for bit. Ranks leave only between steps."""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch.distributed as dist  # noqa: E402

import forja_b200 as fb  # noqa: E402
from oracle import engine  # noqa: E402  (weight generator only)
from tests.test_gpu_moe import upload_moe  # noqa: E402

CFG = dict(layers=2, hidden=512, q_heads=8, kv_heads=1, head_dim=128, experts=16, top_k=4, expert_intermediate=192, vocab=1024,
           group_size=64, router_bits=8, eps=1e-6, theta=1e7, max_rows=64,
           grouped_min_routes=1 << 30)  # per-route projections on both sides: the comparison below is bit for bit


def main():
    rank, world = int(sys.argv[1]), int(sys.argv[2])
    dist.init_process_group("gloo", rank=rank, world_size=world)
    be = fb.CudaBackend(rank)

    def exchange(mine):
        box = [mine]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    ep = fb.ExpertParallel(be, rank, world, exchange)
    weights = engine.random_moe_weights(CFG, 11)
    local = {"embed": weights["embed"], "final_norm": weights["final_norm"], "lm_head": weights["lm_head"], "layers": []}
    per = CFG["experts"] // world
    for layer in weights["layers"]:
        entry = dict(layer)
        for name in ("gate", "up", "down"):
            entry[name] = tuple(np.ascontiguousarray(t[rank * per:(rank + 1) * per]) for t in layer[name])
        local["layers"].append(entry)

    prompts = [[3, 17, 1, 8], [21, 2, 9]][rank]
    steps, page, lanes = 4, 16, len(prompts)
    table_pages = max((n + steps + page - 1) // page for n in prompts) + 2
    physical = sum((n + steps + page - 1) // page for n in prompts) + 3
    rng = np.random.default_rng(100 + rank)
    ids = [rng.integers(0, CFG["vocab"], n).astype(np.uint32) for n in prompts]

    def gather(obj):
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    for max_rows in (64, 300):  # slab capacity 256 (padded exchange, no host round trip) and 1200 (row counts exchanged first)
        run_case(be, ep, rank, dict(CFG, max_rows=max_rows), weights, local, prompts, steps, page, lanes, table_pages, physical, ids)
    # rows returned as bf16: half the bytes on the way back, logits within the bf16 bound instead of bit-identical
    run_case(be, ep, rank, dict(CFG, max_rows=300, ep_return_bf16=1), weights, local, prompts, steps, page, lanes, table_pages, physical, ids, exact=False)
    # the direct exchange (peer stores over NVLink and flags instead of NCCL): the same three cases, then one with the
    # bucketed expert kernels reading the slabs through the per-source row counts
    for max_rows in (64, 300):
        run_case(be, ep, rank, dict(CFG, max_rows=max_rows), weights, local, prompts, steps, page, lanes, table_pages, physical, ids, gather=gather)
    run_case(be, ep, rank, dict(CFG, max_rows=300, ep_return_bf16=1), weights, local, prompts, steps, page, lanes, table_pages, physical, ids, exact=False, gather=gather)
    run_case(be, ep, rank, dict(CFG, max_rows=300, grouped_min_routes=0), weights, local, prompts, steps, page, lanes, table_pages, physical, ids, exact=False, gather=gather)
    # results written back by the owners instead of read by the origins (what 4 and more ranks do by default)
    run_case(be, ep, rank, dict(CFG, max_rows=300), weights, local, prompts, steps, page, lanes, table_pages, physical, ids, gather=gather, return_mode=2)
    run_case(be, ep, rank, dict(CFG, max_rows=64, ep_chunks=2), weights, local, prompts, steps, page, lanes, table_pages, physical, ids, gather=gather, return_mode=2)
    # every layer's rows in 3 chunks that pass through dispatch, experts and return one behind the other on their own streams
    run_case(be, ep, rank, dict(CFG, max_rows=64, ep_chunks=3), weights, local, prompts, steps, page, lanes, table_pages, physical, ids, gather=gather)
    run_case(be, ep, rank, dict(CFG, max_rows=300, ep_chunks=2, grouped_min_routes=0), weights, local, prompts, steps, page, lanes, table_pages, physical, ids, exact=False, gather=gather)
    dist.barrier()
    ep.close()
    dist.destroy_process_group()
    print("EP_OK", rank)


def run_case(be, ep, rank, cfg, weights, local, prompts, steps, page, lanes, table_pages, physical, ids, exact=True, gather=None, return_mode=0):
    def build(w, group):
        pool = fb.KvPool(be, page, physical, lanes, table_pages)
        assert all(s == 0 for s in pool.reserve(list(range(lanes)), [n + steps + 1 for n in prompts]))
        embed, final_norm, lm_head, layers = upload_moe(be, w)
        return pool, fb.MoeModel(be, pool, cfg, embed, final_norm, lm_head, layers, ep=group)

    pool_ep, model_ep = build(local, ep)
    pool_one, model_one = build(weights, None)
    if gather is not None:
        assert model_ep.connect_peers(gather), f"rank {rank}: the peers' buffers could not be mapped"
        model_ep.set_return_mode(return_mode)
        model_ep.set_wait_polls(1 << 23)  # a few seconds: the other rank also runs its single-GPU twin between steps
    logits_ep, logits_one = be.alloc(fb.BF16, (lanes, cfg["vocab"])), be.alloc(fb.BF16, (lanes, cfg["vocab"]))

    def both(starts, counts, tokens):
        pool_ep.pack_step(starts, counts)
        got = model_ep.step(tokens, lanes=lanes, logits=logits_ep)
        pool_one.pack_step(starts, counts)
        want = model_one.step(tokens, lanes=lanes, logits=logits_one)
        a, b = be.read(logits_ep), be.read(logits_one)
        if exact:
            assert np.array_equal(a, b), f"rank {rank}: expert-parallel logits differ from the single-GPU path"
            assert got.tolist() == want.tolist()
        else:
            fa, fb_ = (a.astype(np.uint32) << 16).view(np.float32), (b.astype(np.uint32) << 16).view(np.float32)
            err = float(np.max(np.abs(fa - fb_)) / np.max(np.abs(fb_)))
            assert err <= 2e-2, f"rank {rank}: bf16-return logits off by {err:.3e} (max-abs rel)"
        return want

    tokens = both([0] * lanes, prompts, np.concatenate(ids))
    positions = list(prompts)
    for _ in range(steps):
        tokens = both(positions, [1] * lanes, tokens)
        positions = [p + 1 for p in positions]
    # a step in which rank 1 has nothing to run still serves rank 0's routes
    if rank == 0:
        both(positions, [1] * lanes, tokens)
    else:
        pool_ep.pack_step(positions, [0] * lanes)
        model_ep.step(None, want_tokens=False, lanes=lanes)
    be.synchronize()
    dist.barrier()
    model_ep.close(); model_one.close(); pool_ep.close(); pool_one.close()


if __name__ == "__main__":
    main()
