"""Benchmarks of the rows next to the headline decode path: the sparse-MoE step with expert
parallelism (Qwen3-30B-A3B shape), the isolated q4 projection and the isolated paged attention.
`python -m forja_b200.benchmarks moe --gpus N` (under torch.distributed.run for N > 1, one rank per
GPU) prints one JSON line on rank 0. Weights and KV contents are synthetic (counter-based generator
on the device); timing is CUDA events on the backend's stream, maximum over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import forja_b200 as fb  # noqa: E402

PAGE = 16
MOE = dict(layers=48, hidden=2048, q_heads=32, kv_heads=4, head_dim=128, experts=128, top_k=8, expert_intermediate=768, vocab=151936,
           group_size=64, router_bits=8, eps=1e-6, theta=1e7)


def quant_tensor(be, shape_n, k, bits, seed):
    """Random MLX-affine tensor on the device: uniform codes, scales near 0.006, biases centring the groups."""
    lead = tuple(shape_n) if isinstance(shape_n, (tuple, list)) else (shape_n,)
    packed = be.alloc(fb.U32, lead + (k * bits // 32,))
    scales = be.alloc(fb.BF16, lead + (k // 64,))
    biases = be.alloc(fb.BF16, lead + (k // 64,))
    spread = 0.006 if bits == 4 else 0.006 / 16
    centre = (2 ** bits - 1) / 2.0
    be.fill_random(packed, seed)
    be.fill_random(scales, seed + 1, mean=spread, std=spread * 0.15)
    be.fill_random(biases, seed + 2, mean=-centre * spread, std=spread * 0.5)
    return packed, scales, biases


def gain(be, n, seed):
    t = be.alloc(fb.BF16, (n,))
    be.fill_random(t, seed, mean=1.0, std=0.02)
    return t


def build_moe(be, pool, cfg, ep, rank, world):
    per = cfg["experts"] // world
    H, I, d = cfg["hidden"], cfg["expert_intermediate"], cfg["head_dim"]
    qd, kd = cfg["q_heads"] * d, cfg["kv_heads"] * d
    seed = 1000  # replicated tensors use the same seeds on every rank; expert slices differ by rank
    embed = quant_tensor(be, cfg["vocab"], H, 4, seed)
    lm_head = quant_tensor(be, cfg["vocab"], H, 4, seed + 10)
    final_norm = gain(be, H, seed + 20)
    layers = []
    for layer in range(cfg["layers"]):
        s = seed + 100 * (layer + 1)
        layers.append({
            "input_norm": gain(be, H, s), "q_norm": gain(be, d, s + 1), "k_norm": gain(be, d, s + 2), "post_norm": gain(be, H, s + 3),
            "qkv": quant_tensor(be, qd + 2 * kd, H, 4, s + 10), "o": quant_tensor(be, H, qd, 4, s + 20),
            "router": quant_tensor(be, cfg["experts"], H, cfg["router_bits"], s + 30),
            "gate": quant_tensor(be, (per, I), H, 4, s + 40 + 7919 * rank), "up": quant_tensor(be, (per, I), H, 4, s + 50 + 7919 * rank),
            "down": quant_tensor(be, (per, H), I, 4, s + 60 + 7919 * rank)})
    return fb.MoeModel(be, pool, cfg, embed, final_norm, lm_head, layers, ep=ep)


class MoeLanes:
    """Continuous batch of one rank: prompts uniform 512-4096 prefilled in 512-token pieces under a
    per-step prompt budget (the library's scheduler policy), then 64-256 decode steps; a finished
    lane is refilled with the next request."""

    def __init__(self, pool, lanes, seed, prompt_budget, prefill_limit, prompt_range, decode_only):
        self.pool, self.n = pool, lanes
        self.rng = np.random.default_rng(seed)
        self.prompt_range, self.decode_only = prompt_range, decode_only
        self.policy = fb.SchedulerPolicy([1, lanes] if lanes > 1 else [1], lanes, prefill_limit, prompt_budget, prompt_budget).with_prompt_chunk_multiple(512)
        self.length = np.zeros(lanes, np.int64)       # tokens already in the cache
        self.prompt_left = np.zeros(lanes, np.int64)
        self.decode_left = np.zeros(lanes, np.int64)
        for lane in range(lanes):
            self.refill(lane)

    def refill(self, lane):
        prompt = int(self.rng.integers(self.prompt_range[0], self.prompt_range[1] + 1))
        budget = int(self.rng.integers(64, 257))
        self.pool.reserve([lane], [prompt + budget + 1], want_status=False)
        if self.decode_only:  # the prompt is taken as already cached (KV planes hold random contents)
            self.length[lane], self.prompt_left[lane] = prompt, 0
        else:
            self.length[lane], self.prompt_left[lane] = 0, prompt
            self.policy.ready_prompt(lane, prompt)
        self.decode_left[lane] = budget

    def plan(self):
        """(starts, tokens) of this step."""
        tokens = np.zeros(self.n, np.uint32)
        decoding = (self.prompt_left == 0) & (self.decode_left > 0)
        tokens[decoding] = 1
        for lane, spend in self.policy.prompt_batch(bool(decoding.any())):
            tokens[lane] = spend
        return self.length.astype(np.uint32), tokens

    def advance(self, tokens):
        done = []
        for lane in np.nonzero(tokens)[0].tolist():
            t = int(tokens[lane])
            self.length[lane] += t
            if self.prompt_left[lane] > 0:
                self.prompt_left[lane] -= t
            else:
                self.decode_left[lane] -= 1
                if self.decode_left[lane] == 0:
                    done.append(lane)
        if done:
            self.pool.release(done)
            for lane in done:
                self.refill(lane)


def run_moe(args):
    """With --micro-batches R > 1 every GPU runs R independent half-size (1/R) continuous batches, each on its own
    backend (stream), pool, model and expert-parallel group and stepped by its own host thread, so that one batch's
    exchange with the experts' owners overlaps the other batch's attention and expert work."""
    import threading
    rank, world = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))
    local_rank = int(os.environ.get("LOCAL_RANK", 0))
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = dict(MOE)
    if args.layers:
        cfg["layers"] = args.layers
    R = max(1, args.micro_batches)
    lanes = args.lanes // world // R
    budget = args.prompt_budget // R
    cfg["max_rows"] = lanes + (0 if args.decode_only else budget)
    cfg["grouped_min_routes"] = args.grouped_min_routes
    cfg["stream_rows_per_expert"] = args.stream_rows_per_expert
    cfg["ep_return_bf16"] = int(args.ep_bf16_return)
    cfg["ep_chunks"] = args.ep_chunks
    if R > 1 and world > 1 and args.nccl and cfg["max_rows"] * cfg["top_k"] <= 1024:
        # Small steps exchange padded slabs without a host round trip, so each thread queues dozens of NCCL groups ahead; with two
        # communicators per GPU issued in whatever order the threads happen to run, such a run stopped making progress on 8 GPUs
        # (ended by its timeout). The exchange with a host round trip per layer keeps one group per communicator in flight.
        raise SystemExit("--micro-batches > 1 needs steps of more than 1024 routes per micro-batch (row counts exchanged per layer); use it with prompt work, not with --decode-only at this size")

    def exchange(mine):
        box = [mine]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    def gather(obj):
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    direct = False
    table_pages = (args.prompt_max + 256 + 1 + PAGE - 1) // PAGE + 1
    parts = []
    for r in range(R):  # built one after the other: the rendezvous of every expert-parallel group goes through the same gloo group
        be = fb.CudaBackend(local_rank)
        ep = fb.ExpertParallel(be, rank, world, exchange) if world > 1 else None
        pool = fb.KvPool(be, PAGE, lanes * table_pages + 8, lanes, table_pages)
        model = build_moe(be, pool, cfg, ep, rank, world)
        if world > 1 and not args.nccl:
            direct = model.connect_peers(gather)
            model.set_return_mode(args.ep_return_mode)
        if args.uniform_routing:
            model.uniform_routing(True)
        state = MoeLanes(pool, lanes, args.seed + rank * R + r, budget, args.prefill_limit, (args.prompt_min, args.prompt_max), args.decode_only)
        parts.append({"be": be, "ep": ep, "pool": pool, "model": model, "state": state, "rng": np.random.default_rng(args.seed + 77 + rank * R + r)})
    gate = threading.Barrier(R)
    results = [None] * R
    failures = []

    def worker(i):
        try:
            part = parts[i]
            be, pool, model, state, rng = part["be"], part["pool"], part["model"], part["state"], part["rng"]
            t0, t1 = be.timer(), be.timer()
            processed = kernels = 0
            phase_ms = [0.0] * 4
            if args.phases:
                model.phase_timing(True)
            for step in range(args.warmup + args.steps):
                if step == args.warmup:
                    be.synchronize()
                    gate.wait()
                    if i == 0 and dist is not None:
                        dist.barrier()
                    gate.wait()
                    be.timer_record(t0)
                    processed, kernels = 0, 0
                starts, tokens = state.plan()
                rows = int(tokens.sum())
                pool.pack_step(starts, tokens)
                ids = rng.integers(0, cfg["vocab"], rows).astype(np.uint32) if rows else None
                model.step(ids, want_tokens=rows > 0, lanes=lanes)
                kernels += model.stats()["kernels"]
                if args.phases and step >= args.warmup:
                    phase_ms = [a + b for a, b in zip(phase_ms, model.phase_ms())]
                state.advance(tokens)
                processed += rows
            be.timer_record(t1)
            be.synchronize()
            if args.phases and direct:
                print(json.dumps({"rank": rank, "micro_batch": i, "rows_received_per_layer_last_step": model.received_rows().sum(axis=1).tolist()}), flush=True)
            results[i] = (be.timer_elapsed_ns(t0, t1) * 1e-9, processed, kernels, phase_ms)
        except BaseException as error:  # noqa: BLE001 - reported by the main thread
            failures.append(error)
            gate.abort()

    threads = [threading.Thread(target=worker, args=(i,)) for i in range(R)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if failures:
        raise failures[0]
    elapsed = max(r[0] for r in results)
    total = sum(r[1] for r in results)
    kernels = sum(r[2] for r in results)
    if dist is not None:
        import torch
        box = torch.tensor([elapsed, float(total), float(kernels)], dtype=torch.float64)
        gathered = [torch.zeros_like(box) for _ in range(world)]
        dist.all_gather(gathered, box)
        elapsed = max(float(g[0]) for g in gathered)
        total = int(sum(float(g[1]) for g in gathered))
        kernels = int(sum(float(g[2]) for g in gathered))
        dist.barrier()
    if args.phases:
        for i, r in enumerate(results):
            print(json.dumps({"rank": rank, "micro_batch": i, "ms_per_step_by_phase": {name: v / args.steps for name, v in zip(
                ("attention_and_router", "dispatch", "experts", "return_and_combine"), r[3])}}), flush=True)
    if rank == 0:
        print(json.dumps({
            "metric": "moe step tok/s (prompt + generated tokens)", "value": total / elapsed, "unit": "tok/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True, "scaling": "strong", "dtype": "bf16 activations, q4 weights",
            "data": "synthetic", "gpu_launches": kernels,
            "config": {"workload": "qwen3-30b-a3b-arch q4 sparse-MoE continuous batching" + (" (decode only)" if args.decode_only else " (chunked prefill + decode)"),
                       "lanes_total": args.lanes, "lanes_per_gpu": lanes * R, "micro_batches_per_gpu": R, "layers": cfg["layers"], "prompt_tokens": [args.prompt_min, args.prompt_max],
                       "prompt_budget_per_gpu_step": 0 if args.decode_only else budget * R,
                       "parallelism": ("experts sharded over %d GPUs, %s per MoE layer (rows return as %s); lanes data-parallel" % (
                           world, "peer stores and loads over NVLink with flags" if direct else "NCCL send/recv all-to-all", "bf16" if args.ep_bf16_return else "f32")) if world > 1 else "single GPU"}}))
    for part in parts:
        part["model"].close()
        part["pool"].close()
        if part["ep"] is not None:
            part["ep"].close()
    if dist is not None:
        dist.destroy_process_group()


def moe_ep_block(rank, world, local_rank, exchange, barrier, max_over_ranks, sum_over_ranks, lanes_total=256, steps=8, warmup=3, layers=0, seed=0,
                 prompt_budget=2048, prompt_range=(512, 4096), prefill_limit=4, all_gather=None):
    """One measurement of the sparse-MoE continuous-batching step (Qwen3-30B-A3B shape, q4 weights, bf16 activations) with the
    experts sharded over `world` ranks: `lanes_total` lanes split evenly over the ranks (strong scaling over the lanes), every
    rank prefilling up to `prompt_budget` prompt tokens per step beside its decode rows. `exchange(obj)` broadcasts rank 0's
    object (the NCCL id of the expert-parallel group), `barrier()` aligns the ranks, `max_over_ranks(x)` / `sum_over_ranks(x)`
    reduce a float; `all_gather(obj) -> list`, when given, lets the ranks map each other's buffers so that the exchange runs as
    peer stores over NVLink instead of NCCL (MoeModel.connect_peers). Timed with CUDA events on the backend's stream between
    barriers, maximum over ranks; two further steps run with per-phase events for the split. Returns the block on every rank."""
    cfg = dict(MOE)
    if layers:
        cfg["layers"] = layers
    lanes = max(1, lanes_total // world)
    cfg["max_rows"] = lanes + prompt_budget
    cfg["grouped_min_routes"] = 0
    cfg["stream_rows_per_expert"] = 0
    cfg["ep_return_bf16"] = 0
    be = fb.CudaBackend(local_rank)
    ep = fb.ExpertParallel(be, rank, world, exchange) if world > 1 else None
    table_pages = (prompt_range[1] + 256 + 1 + PAGE - 1) // PAGE + 1
    pool = fb.KvPool(be, PAGE, lanes * table_pages + 8, lanes, table_pages)
    model = build_moe(be, pool, cfg, ep, rank, world)
    direct = bool(world > 1 and all_gather is not None and model.connect_peers(all_gather))
    state = MoeLanes(pool, lanes, seed + rank, prompt_budget, prefill_limit, prompt_range, False)
    rng = np.random.default_rng(seed + 77 + rank)
    t0, t1 = be.timer(), be.timer()

    def one_step():
        starts, tokens = state.plan()
        rows = int(tokens.sum())
        pool.pack_step(starts, tokens)
        ids = rng.integers(0, cfg["vocab"], rows).astype(np.uint32) if rows else None
        model.step(ids, want_tokens=rows > 0, lanes=lanes)
        state.advance(tokens)
        return rows, model.stats()["kernels"]

    for _ in range(warmup):
        one_step()
    be.synchronize()
    barrier()
    be.timer_record(t0)
    processed = kernels = 0
    for _ in range(steps):
        rows, launched = one_step()
        processed += rows
        kernels += launched
    be.timer_record(t1)
    be.synchronize()
    barrier()
    elapsed = max_over_ranks(be.timer_elapsed_ns(t0, t1) * 1e-9)
    total = sum_over_ranks(float(processed))
    model.phase_timing(True)
    phase_ms, phase_steps = [0.0] * 4, 2
    for _ in range(phase_steps):
        one_step()
        phase_ms = [a + b for a, b in zip(phase_ms, model.phase_ms())]
    model.phase_timing(False)
    names = ("attention_and_router", "dispatch", "experts", "return_and_combine")
    phases = {name: max_over_ranks(v / phase_steps) for name, v in zip(names, phase_ms)}
    # the smallest value over the ranks: a rank that arrives early at an exchange waits there for the others, so the spread of
    # the two exchange phases is mostly the imbalance of the compute phases before them
    phases_min = {name: -max_over_ranks(-v / phase_steps) for name, v in zip(names, phase_ms)}
    # how evenly the router of this random-weight model spreads the rows over the ranks: per layer, the busiest rank's
    # received rows over the mean (every rank waits for the busiest one at that layer's return)
    imbalance = None
    if direct:
        mine = model.received_rows().sum(axis=1).astype(np.float64)
        busiest = np.array([max_over_ranks(float(v)) for v in mine])
        mean = np.array([sum_over_ranks(float(v)) for v in mine]) / world
        ratio = busiest / np.maximum(mean, 1.0)
        imbalance = {"mean": float(ratio.mean()), "max": float(ratio.max())}
    # the same steps with the router's choice replaced by an even spread over the experts (what a trained, load-balanced
    # router approximates): separates the cost of the exchange from the cost of waiting for the busiest rank
    model.uniform_routing(True)
    for _ in range(2):
        one_step()
    be.synchronize()
    barrier()
    be.timer_record(t0)
    even_rows = 0
    for _ in range(steps):
        rows, _ = one_step()
        even_rows += rows
    be.timer_record(t1)
    be.synchronize()
    barrier()
    even_elapsed = max_over_ranks(be.timer_elapsed_ns(t0, t1) * 1e-9)
    even_total = sum_over_ranks(float(even_rows))
    model.uniform_routing(False)
    rows_per_step = total / steps / world
    remote = (world - 1) / world
    block = {
        "workload": "qwen3-30b-a3b-arch q4 sparse-MoE continuous batching (chunked prefill + decode), %d layers, 128 experts top-8" % cfg["layers"],
        "n_gpus": world, "scaling": "strong over the lanes (%d lanes in total, %d per GPU); prompt budget %d tokens per GPU and step" % (lanes_total, lanes, prompt_budget),
        "tok_s": total / elapsed, "ms_per_step": elapsed / steps * 1e3, "steps": steps, "warmup": warmup, "rows_per_gpu_step": rows_per_step,
        "phase_ms_per_step_max_over_ranks": phases, "phase_ms_per_step_min_over_ranks": phases_min,
        "exchange_mb_per_layer_and_gpu": {"dispatch_bf16": rows_per_step * cfg["top_k"] * remote * cfg["hidden"] * 2 / 1e6,
                                          "return_f32": rows_per_step * cfg["top_k"] * remote * cfg["hidden"] * 4 / 1e6},
        "rows_received_busiest_rank_over_mean_per_layer": imbalance,
        "with_even_routing": {"tok_s": even_total / even_elapsed, "ms_per_step": even_elapsed / steps * 1e3,
                              "what": "router's choice replaced by an even spread over the experts (fj_moe_uniform_routing); not the headline"},
        "gpu_launches": int(sum_over_ranks(float(kernels))),
        "parallelism": ("experts sharded over %d GPUs, %s per MoE layer, lanes data-parallel" %
                        (world, "rows stored straight into the owner's memory over NVLink by the dispatching kernel, results read from the owner's memory by the combine, flags instead of a host round trip" if direct
                         else "NCCL send/recv all-to-all")) if world > 1 else "single GPU",
    }
    model.close()
    pool.close()
    if ep is not None:
        ep.close()
    be.close()
    return block


def load_peaks():
    try:
        with open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")) as f:
            peaks = json.load(f)
        return float(peaks.get("hbm_gbs", 6650.0)), float(peaks.get("bf16_tflops", 1590.0)), "measured"
    except (OSError, ValueError):
        return 6650.0, 1590.0, "fallback"


def timed(be, commands, dispatches, reps=3):
    """Best device time per dispatch over `reps` submissions of a command list (CUDA events around the submission)."""
    be.submit(commands).wait()
    best = float("inf")
    for _ in range(reps):
        sub = be.submit(commands)
        sub.wait()
        best = min(best, sub.gpu_time_ns() / dispatches)
    return best


def run_q4(args):
    """Isolated MLX q4 projection (config 4): weights uniform nibbles, scales/biases N(0, 0.01), activations N(0, 1).
    Each dispatch uses its own copy of the weights so that every launch streams them from HBM."""
    from forja_b200.backend import CommandList, Op
    be = fb.CudaBackend(0)
    hbm, tflops, source = load_peaks()
    shapes = {"qkv": (2048, 6144), "o": (4096, 2048), "expert": (2048, 768), "lm_head": (2048, 151936)}
    for name in args.shapes.split(","):
        k, n = shapes[name]
        wbytes = 0.5625 * n * k
        copies = max(2, min(args.copies, int((768 << 20) // wbytes) + 1))
        packed = be.alloc(fb.U32, (copies, n, k // 8)); be.fill_random(packed, 1)
        scales = be.alloc(fb.BF16, (copies, n, k // 64)); be.fill_random(scales, 2, std=0.01)
        biases = be.alloc(fb.BF16, (copies, n, k // 64)); be.fill_random(biases, 3, std=0.01)
        for m in [int(v) for v in args.m.split(",")]:
            x = be.alloc(fb.BF16, (m, k)); be.fill_random(x, 4)
            out = be.alloc(fb.BF16, (m, n))
            cl = CommandList()
            used = copies if m <= 64 else min(copies, 4)
            for c in range(used):
                cl.dispatch(Op.QuantMatmul(4, 64), [x, packed.narrow(0, c, 1).reshape((n, k // 8)), scales.narrow(0, c, 1).reshape((n, k // 64)),
                                                    biases.narrow(0, c, 1).reshape((n, k // 64))], out)
            ns = timed(be, cl, used)
            print(json.dumps({"workload": "q4 projection", "shape": name, "k": k, "n": n, "m": m, "us_per_launch": ns / 1e3, "weight_gbs": wbytes / ns,
                              "frac_of_hbm_peak": wbytes / ns / hbm, "tflops": 2.0 * m * k * n / ns / 1e3, "frac_of_bf16_peak": 2.0 * m * k * n / ns / 1e3 / tflops,
                              "peak_source": source}), flush=True)
            be.release(x); be.release(out)
        for t in (packed, scales, biases):
            be.release(t)


def run_gemm(args):
    from forja_b200.backend import CommandList, Op
    be = fb.CudaBackend(0)
    _, tflops, source = load_peaks()
    for shape in args.shapes.split(","):
        m, k, n = (int(v) for v in shape.split("x"))
        x = be.alloc(fb.BF16, (m, k)); w = be.alloc(fb.BF16, (n, k)); out = be.alloc(fb.BF16, (m, n))
        be.fill_random(x, 1); be.fill_random(w, 2, std=0.05)
        cl = CommandList()
        for _ in range(args.reps):
            cl.dispatch(Op.Matmul(), [x, w.permute([1, 0])], out)
        ns = timed(be, cl, args.reps)
        print(json.dumps({"workload": "bf16 matmul (weight [n, k] through a transposed view)", "m": m, "k": k, "n": n, "us_per_launch": ns / 1e3,
                          "tflops": 2.0 * m * k * n / ns / 1e3, "frac_of_bf16_peak": 2.0 * m * k * n / ns / 1e3 / tflops, "peak_source": source,
                          "tcgen05_wait_giveups": be.tcgen05_wait_giveups()}), flush=True)
        for t in (x, w, out):
            be.release(t)


def run_sample(args):
    """Op::Sample on [rows, vocab] bf16 logits (N(0, spread)): device time per dispatch for a few parameter settings."""
    from forja_b200.backend import CommandList, Op
    be = fb.CudaBackend(0)
    logits = be.alloc(fb.BF16, (args.rows, args.vocab))
    be.fill_random(logits, 3, std=args.spread)
    out = be.alloc(fb.U32, (args.rows,))
    bits = lambda v: int(np.array([v], np.float32).view(np.uint32)[0])
    for name, temperature, top_k, top_p in (("greedy", 0.0, 0, 1.0), ("top-k 40, top-p 0.95", 0.8, 40, 0.95), ("top-p 0.9 over the row", 1.0, 0, 0.9),
                                            ("temperature only", 1.0, 0, 1.0)):
        params = be.tensor_from(np.array([bits(temperature), top_k, bits(top_p), 11, 22], np.uint32), fb.U32)
        cl = CommandList()
        for rep in range(args.reps):
            cl.dispatch(Op.Sample(rep), [logits, params], out)
        ns = timed(be, cl, args.reps)
        print(json.dumps({"workload": "Op::Sample, one CTA per row", "rows": args.rows, "vocab": args.vocab, "setting": name, "us_per_dispatch": ns / 1e3}), flush=True)
        be.release(params)


def run_attention(args):
    """Isolated paged GQA attention (config 3): 32 q / 4 kv heads, head_dim 128, page 16, permuted page tables, bf16 N(0, 1).
    decode: `lanes` sequences with kv lengths log-uniform 64-32768, one query token each (one ragged launch);
    prefill: one 512-token chunk per sequence at a random chunk-aligned start."""
    from forja_b200.backend import CommandList, Op
    be = fb.CudaBackend(0)
    hbm, tflops, source = load_peaks()
    rng = np.random.default_rng(args.seed)
    hq, kvh, d, page = 32, 4, 128, PAGE
    scale = float(1.0 / np.sqrt(d))
    if args.mode == "decode":
        lengths = np.round(np.exp(rng.uniform(np.log(64), np.log(args.kv_max), args.lanes))).astype(np.int64)
        q_lens = np.ones(args.lanes, np.int64)
        starts = lengths - 1
    else:
        chunks = rng.integers(0, max(args.kv_max // 512, 1), args.lanes)
        starts = chunks * 512
        q_lens = np.full(args.lanes, 512, np.int64)
        lengths = starts + q_lens
    pages = (lengths + page - 1) // page
    physical = int(pages.sum()) + 8
    kpool = be.alloc(fb.BF16, (physical, page, kvh, d)); be.fill_random(kpool, 11)
    vpool = be.alloc(fb.BF16, (physical, page, kvh, d)); be.fill_random(vpool, 12)
    generations = be.tensor_from(np.ones(physical, np.uint32), fb.U32)
    order = rng.permutation(physical)
    cl = CommandList()
    cursor = 0
    keep = []
    for lane in range(args.lanes):
        table = np.zeros((int(pages[lane]), 2), np.uint32)
        table[:, 0] = order[cursor:cursor + int(pages[lane])]
        table[:, 1] = 1
        cursor += int(pages[lane])
        t = be.tensor_from(table, fb.U32)
        q = be.alloc(fb.BF16, (int(q_lens[lane]), hq, d)); be.fill_random(q, 100 + lane)
        out = be.alloc(fb.BF16, (int(q_lens[lane]), hq, d))
        keep += [t, q, out]
        cl.dispatch(Op.PagedSdpa(scale, True, int(starts[lane]), int(lengths[lane]), page), [q.permute([1, 0, 2]), kpool, vpool, t, generations], out.permute([1, 0, 2]))
    ns = timed(be, cl, 1)
    kv_bytes = float((lengths * kvh * d * 2 * 2).sum())
    qo_bytes = float((q_lens * hq * d * 2 * 2).sum())
    # causal flops: every query row attends min(key_length, q_start + row + 1) keys, 4 d flops per (row, key, head)
    attended = sum(float(np.minimum(lengths[i], starts[i] + np.arange(q_lens[i]) + 1).sum()) for i in range(args.lanes))
    flops = attended * hq * d * 4.0
    print(json.dumps({"workload": "paged GQA attention " + args.mode, "lanes": args.lanes, "q_heads": hq, "kv_heads": kvh, "head_dim": d, "kv_tokens": int(lengths.sum()),
                      "us": ns / 1e3, "algorithmic_gbs": (kv_bytes + qo_bytes) / ns, "frac_of_hbm_peak": (kv_bytes + qo_bytes) / ns / hbm,
                      "tflops": flops / ns / 1e3, "frac_of_bf16_peak": flops / ns / 1e3 / tflops, "peak_source": source, "kernel_launches": be.kernel_launch_count()}), flush=True)


def main():
    ap = argparse.ArgumentParser(description=__doc__)
    sub = ap.add_subparsers(dest="command", required=True)
    moe = sub.add_parser("moe")
    moe.add_argument("--gpus", type=int, default=1, help="informational; the rank count comes from the launcher's environment")
    moe.add_argument("--lanes", type=int, default=256)
    moe.add_argument("--steps", type=int, default=16)
    moe.add_argument("--warmup", type=int, default=3)
    moe.add_argument("--layers", type=int, default=0)
    moe.add_argument("--seed", type=int, default=0)
    moe.add_argument("--prompt-min", type=int, default=512)
    moe.add_argument("--prompt-max", type=int, default=4096)
    moe.add_argument("--prompt-budget", type=int, default=2048)
    moe.add_argument("--prefill-limit", type=int, default=4)
    moe.add_argument("--decode-only", action="store_true")
    moe.add_argument("--ep-bf16-return", action="store_true", help="expert parallelism: per-route rows come back as bf16 instead of f32")
    moe.add_argument("--ep-chunks", type=int, default=1, help="direct exchange: chunks per layer that overlap their transfers with each other's expert work")
    moe.add_argument("--ep-return-mode", type=int, default=0, help="direct exchange: 0 or 1 = origins read the results, 2 = owners write them")
    moe.add_argument("--uniform-routing", action="store_true", help="measurement aid: spread every row's experts evenly instead of using the (random-weight) router's choice")
    moe.add_argument("--nccl", action="store_true", help="expert parallelism through NCCL send/recv instead of the direct exchange over NVLink")
    moe.add_argument("--micro-batches", type=int, default=1, help="independent continuous batches per GPU, stepped concurrently (each gets 1/R of the lanes and of the prompt budget)")
    moe.add_argument("--phases", action="store_true", help="also print the time of the timed steps split by phase (CUDA events inside the step)")
    moe.add_argument("--grouped-min-routes", type=int, default=0, help="0 = library default")
    moe.add_argument("--stream-rows-per-expert", type=int, default=0, help="0 = library default")
    q4 = sub.add_parser("q4")
    q4.add_argument("--shapes", default="qkv,o,expert,lm_head")
    q4.add_argument("--m", default="1,8,64,512,4096")
    q4.add_argument("--copies", type=int, default=64)
    gemm = sub.add_parser("gemm")
    gemm.add_argument("--shapes", default="2048x2048x5120,4096x4096x4096,8192x2048x8192")
    gemm.add_argument("--reps", type=int, default=10)
    attn = sub.add_parser("attention")
    attn.add_argument("--mode", default="decode", choices=["decode", "prefill"])
    attn.add_argument("--lanes", type=int, default=256)
    attn.add_argument("--kv-max", type=int, default=32768)
    attn.add_argument("--seed", type=int, default=0)
    sample = sub.add_parser("sample")
    sample.add_argument("--rows", type=int, default=128)
    sample.add_argument("--vocab", type=int, default=151936)
    sample.add_argument("--spread", type=float, default=3.0)
    sample.add_argument("--reps", type=int, default=5)
    args = ap.parse_args()
    {"moe": run_moe, "q4": run_q4, "gemm": run_gemm, "attention": run_attention, "sample": run_sample}[args.command](args)


if __name__ == "__main__":
    main()
