"""Benchmark of the continuous-batching decode step (the hot path) on B200.

Workload (fits one GPU): Qwen3-0.6B architecture, bf16, random-init weights; 128 sequences whose
context lengths are log-uniform over 128..8192 tokens, page size 16, greedy decode; a sequence that
reaches its token budget leaves and a new request takes its lane (continuous batching). Contexts
are synthetic: the KV planes are pre-filled with seeded N(0, 1) values, so a newly admitted
request finds its context rows already in its pages and the timed region is pure decode.

One "step" = one forward step over every active lane. `value` is decode tokens per second with
all inputs resident on the device (tokens fed back on the device, no host synchronisation inside
the timed region); `e2e` is the same loop driven through the C ABI with host buffers: every step
uploads token ids and lane descriptors and reads the greedy tokens back before the next step.

usage: python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference]
For N > 1 launch with torch.distributed.run: each rank owns one GPU, runs its own 128 lanes
(independent replicas over sequences, no data-path collective) and rank 0 prints one JSON line.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

BF16, U32 = 2, 4
QWEN3_06B = dict(dtype=BF16, layers=28, hidden=1024, q_heads=16, kv_heads=8, head_dim=128, intermediate=3072, vocab=151936, qk_norm=1,
                 eps=1e-6, theta=1e6, max_rows=128)
PAGE = 16
CTX_MIN, CTX_MAX = 128, 8192
BUDGET_MIN, BUDGET_MAX = 64, 256


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--lanes", type=int, default=128)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--pool-pages", type=int, default=36000, help="physical KV pages per GPU (36000 pages = 66 GB of planes)")
    ap.add_argument("--ctx-max", type=int, default=CTX_MAX, help="largest context length (lower it for profiler captures)")
    ap.add_argument("--layers", type=int, default=0, help="override the layer count (profiler captures only; 0 = the model's 28)")
    ap.add_argument("--repeats", type=int, default=0, help="how often the block of --steps steps is timed (the median block is reported); 0 = 9 for blocks up to 64 steps, else 3, else 1")
    ap.add_argument("--no-moe", action="store_true", help="skip the sharded sparse-MoE block")
    ap.add_argument("--moe-lanes", type=int, default=256, help="lanes of the sparse-MoE block, in total over all GPUs")
    ap.add_argument("--moe-steps", type=int, default=8)
    ap.add_argument("--moe-layers", type=int, default=0, help="0 = the model's 48")
    ap.add_argument("--moe-nccl", action="store_true", help="sharded MoE block: exchange through NCCL send/recv instead of peer stores over NVLink")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph-replay", action="store_true", help="launch every decode step kernel by kernel instead of replaying its recorded CUDA graph")
    return ap.parse_args()


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even f32 -> bf16 bit patterns (finite inputs)."""
    u = np.ascontiguousarray(x, np.float32).view(np.uint32)
    return ((u + 0x7FFF + ((u >> 16) & 1)) >> 16).astype(np.uint16)


class Requests:
    """Seeded stream of synthetic requests: (context length, new-token budget)."""

    def __init__(self, seed, ctx_max):
        self.rng = np.random.default_rng(seed)
        self.ctx_max = ctx_max

    def next(self):
        ctx = int(round(float(np.exp(self.rng.uniform(np.log(CTX_MIN), np.log(self.ctx_max))))))
        budget = int(self.rng.integers(BUDGET_MIN, BUDGET_MAX + 1))
        return ctx, budget


class Lanes:
    """Host bookkeeping of the continuous batch. Admission runs through the product scheduler
    (SchedulerPolicy over fj_sched_*: FIFO with at most 8 bypasses by smaller requests, page
    reservation = ceil((context + budget) / page), crates/forja-serve/src/scheduler.rs:109-152):
    every request that finishes is replaced in the waiting line by the next one of the seeded
    stream, and whatever the scheduler admits against the free pages takes the lowest free lanes.
    The device allocator is deterministic, so the host knows the free-page count without reading
    anything back."""

    def __init__(self, pool, requests, lanes, pool_pages):
        import forja_b200 as fb
        self.pool, self.requests, self.n = pool, requests, lanes
        self.free_pages = pool_pages
        self.length = np.zeros(lanes, np.uint32)
        self.remaining = np.zeros(lanes, np.int64)
        self.pages = np.zeros(lanes, np.int64)
        self.request_of = [None] * lanes
        self.waiting = {}
        self.next_id = 0
        self.admitted = 0
        buckets = sorted({1 << i for i in range(lanes.bit_length())} | {lanes})
        self.sched = fb.SchedulerPolicy(buckets, active_limit=lanes, prefill_limit=lanes, prompt_budget=PAGE, idle_prompt_budget=PAGE)
        for _ in range(lanes):
            self.enqueue()
        self.admit()

    def enqueue(self):
        ctx, budget = self.requests.next()
        self.waiting[self.next_id] = (ctx, budget)
        self.sched.enqueue(self.next_id, ctx + budget)
        self.next_id += 1

    def admit(self):
        ids, self.free_pages = self.sched.admit_pages(PAGE, self.free_pages)
        free_lanes = [lane for lane in range(self.n) if self.request_of[lane] is None]
        lanes, tokens = [], []
        for rid, lane in zip(ids, free_lanes):
            ctx, budget = self.waiting.pop(rid)
            self.pages[lane], self.length[lane], self.remaining[lane] = (ctx + budget + PAGE - 1) // PAGE, ctx, budget
            self.request_of[lane] = rid
            lanes.append(lane)
            tokens.append(ctx + budget)
            self.admitted += 1
        if lanes:
            self.pool.reserve(lanes, tokens, want_status=False)

    def descriptors(self):
        active = self.remaining > 0
        return self.length.copy(), active.astype(np.uint32)

    def advance(self):
        """After a step: every active lane grew by one token; finished lanes release their pages."""
        active = self.remaining > 0
        self.length[active] += 1
        self.remaining[active] -= 1
        done = np.nonzero(active & (self.remaining == 0))[0]
        if done.size:
            self.pool.release(done.tolist())
            for lane in done.tolist():
                self.free_pages += int(self.pages[lane])
                self.pages[lane] = 0
                self.sched.complete(self.request_of[lane])
                self.request_of[lane] = None
                self.enqueue()
            self.admit()
        return int(active.sum())


def attention_bytes(lengths, cfg):
    """Algorithmic bytes of one paged decode-attention launch (one layer): q rows + K/V rows of
    every attended token + 12 B per page of table/generation reads + 4 B + output rows
    (the reference's KernelCost, crates/forja-core/src/cost/attention.rs:38-90)."""
    hq, kvh, d, esz = cfg["q_heads"], cfg["kv_heads"], cfg["head_dim"], 2
    total = 0
    for L in lengths:
        total += hq * d * esz + kvh * int(L) * 2 * d * esz + 12 * ((int(L) + PAGE - 1) // PAGE) + 4 + hq * d * esz
    return total


def start_clock_sampler(path, device):
    query = "index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown," \
            "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    try:
        return subprocess.Popen(["nvidia-smi", "-i", str(device), f"--query-gpu={query}", "--format=csv,noheader,nounits", "-lms", "200"],
                                stdout=open(path, "w"), stderr=subprocess.DEVNULL)
    except OSError:
        return None


def read_clock_samples(path):
    sm, sm_max, reasons = [], 0.0, set()
    try:
        for line in open(path):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                sm_max = max(sm_max, float(parts[2]))
            except ValueError:
                continue
            for name, value in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                if value.lower().startswith("active"):
                    reasons.add(name)
    except OSError:
        pass
    busy = sorted(s for s in sm if s > 0)
    top = busy[len(busy) // 2:] if busy else []  # samples under load: upper half
    return {"sm_mhz": float(np.median(top)) if top else None, "sm_max_mhz": sm_max or None, "reasons": sorted(reasons), "samples": len(sm)}


def random_weights_bf16(cfg, seed):
    """Random-init N(0, 0.02) weights, norm gains 1 + N(0, 0.02), as bf16 bit patterns."""
    rng = np.random.default_rng(seed)
    H, I, V, d = cfg["hidden"], cfg["intermediate"], cfg["vocab"], cfg["head_dim"]
    qd, kd = cfg["q_heads"] * d, cfg["kv_heads"] * d
    mat = lambda r, c: f32_to_bf16_bits(rng.standard_normal((r, c), dtype=np.float32) * np.float32(0.02))
    gain = lambda n: f32_to_bf16_bits(np.float32(1.0) + rng.standard_normal(n, dtype=np.float32) * np.float32(0.02))
    weights = {"embed": mat(V, H), "final_norm": gain(H), "layers": []}
    for _ in range(cfg["layers"]):
        weights["layers"].append({"input_norm": gain(H), "wq": mat(qd, H), "wk": mat(kd, H), "wv": mat(kd, H), "q_norm": gain(d), "k_norm": gain(d),
                                  "wo": mat(H, qd), "post_norm": gain(H), "w_gate": mat(I, H), "w_up": mat(I, H), "w_down": mat(H, I)})
    return weights


def dist_setup(n_gpus):
    """torch.distributed is plumbing only: rendezvous, barrier and the max over ranks."""
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local, dist


def reduce_max_sum(dist, local, elapsed_s, tokens, extra):
    """max of elapsed over ranks, sums of the token counts and of each entry of `extra`."""
    if dist is None:
        return elapsed_s, tokens, extra
    import torch
    t = torch.tensor([elapsed_s], dtype=torch.float64, device=f"cuda:{local}")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    s = torch.tensor([float(tokens)] + [float(v) for v in extra], dtype=torch.float64, device=f"cuda:{local}")
    dist.all_reduce(s, op=dist.ReduceOp.SUM)
    vals = s.tolist()
    return float(t.item()), vals[0], vals[1:]


def barrier(dist, be):
    be.synchronize()
    if dist is not None:
        dist.barrier()


def run_native(args):
    import forja_b200 as fb
    rank, world, local, dist = dist_setup(args.gpus)
    be = fb.CudaBackend(local)  # raises when the CUDA library or device is missing: no fallback
    cfg = dict(QWEN3_06B)
    if args.layers:
        cfg["layers"] = args.layers
    cfg["max_rows"] = args.lanes
    table_pages = (args.ctx_max + BUDGET_MAX + PAGE - 1) // PAGE
    pool = fb.KvPool(be, PAGE, args.pool_pages, args.lanes, table_pages)
    weights = random_weights_bf16(cfg, args.seed)
    up = lambda a: be.tensor_from(a, fb.BF16)
    model = fb.DenseModel(be, pool, cfg, up(weights["embed"]), up(weights["final_norm"]), [{k: up(v) for k, v in layer.items()} for layer in weights["layers"]])
    del weights
    model.fill_kv(args.seed + 17 * rank)
    model.graph_replay(not args.no_graph_replay)
    lanes = Lanes(pool, Requests(args.seed * 1000 + rank, args.ctx_max), args.lanes, args.pool_pages)

    repeats = args.repeats if args.repeats > 0 else (9 if args.steps <= 64 else (3 if args.steps <= 256 else 1))

    def step_device():
        starts, tokens = lanes.descriptors()
        pool.pack_step(starts, tokens)
        model.step(None, want_tokens=False)
        return starts, tokens

    # The clock sampler starts before the warm-up: nvidia-smi's own start-up (NVML initialisation) can stall
    # kernel launches for about a second, which must not land inside a timed region. It keeps sampling
    # through both timed regions.
    clocks_dir = tempfile.mkdtemp(prefix="fj_bench_clocks_")
    clocks_path = os.path.join(clocks_dir, f"clocks_rank{rank}.csv")
    sampler = start_clock_sampler(clocks_path, local)
    if sampler is not None:
        deadline = time.perf_counter() + 5.0
        while time.perf_counter() < deadline and not (os.path.exists(clocks_path) and os.path.getsize(clocks_path) > 200):
            time.sleep(0.05)

    # first token of every lane comes from the host once; afterwards tokens feed back on the device
    starts, tokens = lanes.descriptors()
    pool.pack_step(starts, tokens)
    seed_tokens = np.random.default_rng(args.seed).integers(0, cfg["vocab"], int(tokens.sum())).astype(np.uint32)
    model.step(seed_tokens, want_tokens=False)
    lanes.advance()
    for _ in range(max(args.warmup - 1, 0)):
        step_device()
        lanes.advance()

    # ---- timed region 1: device-resident decode --------------------------------------------
    # The block of `steps` steps is timed `repeats` times back to back on the running batch (each
    # bracketed by barrier + synchronise, CUDA events on the backend's stream, max over ranks);
    # the line reports the median block, so one disturbed block does not decide the number.
    t_begin, t_end = be.timer(), be.timer()
    model.attention_time()
    blocks = []
    launches = 0
    attn_bytes, profiled_steps = 0, 0
    for rep in range(repeats):
        barrier(dist, be)
        launches0 = be.kernel_launch_count()
        be.timer_record(t_begin)
        block_tokens, block_kv = 0, 0
        for step in range(args.steps):
            # the attention launches of every 8th step are bracketed by CUDA events on the kernel's
            # stream; bracketing all of them costs about a millisecond per step in pipeline bubbles
            sampled = step % 8 == 0
            model.profile_attention(sampled)
            starts, tokens = step_device()
            active = starts[tokens > 0] + 1
            if sampled:
                attn_bytes += attention_bytes(active, cfg)
                profiled_steps += 1
            block_kv += int(active.sum())
            block_tokens += lanes.advance()
        be.timer_record(t_end)
        barrier(dist, be)
        block_elapsed = be.timer_elapsed_ns(t_begin, t_end) * 1e-9
        launches = be.kernel_launch_count() - launches0
        block_elapsed, block_tokens_all, (block_kv_all,) = reduce_max_sum(dist, local, block_elapsed, block_tokens, [block_kv])
        blocks.append((block_elapsed, block_tokens_all, block_kv_all))
    order = sorted(range(repeats), key=lambda i: blocks[i][1] / blocks[i][0])
    elapsed, total_tokens, kv_tokens = blocks[order[repeats // 2]]
    kv_tokens /= world
    attn_ns, attn_launches = model.attention_time()
    model.profile_attention(False)
    stats = model.stats()

    # ---- timed region 2: end to end through the C ABI with host buffers ----------------------
    e2e_steps = args.steps
    host_tokens = np.zeros(args.lanes, np.uint32)
    for _ in range(min(args.warmup, 3)):  # the host-fed form of the step warms up outside the timed region
        starts, tokens = lanes.descriptors()
        pool.pack_step(starts, tokens)
        host_tokens = model.step(host_tokens[tokens > 0], want_tokens=True, lanes=args.lanes)
        lanes.advance()
    barrier(dist, be)
    h2d = d2h = 0
    e2e_tokens = e2e_kv_tokens = 0
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        starts, tokens = lanes.descriptors()
        pool.pack_step(starts, tokens)                       # host -> device: 2 x lanes x 4 B lane descriptors
        ids = host_tokens[tokens > 0]
        out = model.step(ids, want_tokens=True, lanes=args.lanes)  # host -> device ids, device -> host greedy tokens (synchronises)
        host_tokens = out
        e2e_kv_tokens += int((starts[tokens > 0] + 1).sum())
        h2d += starts.nbytes + tokens.nbytes + ids.nbytes
        d2h += out.nbytes
        e2e_tokens += lanes.advance()
    be.synchronize()
    e2e_elapsed = time.perf_counter() - t0
    if sampler is not None:
        sampler.terminate()
        sampler.wait()
    clocks = read_clock_samples(clocks_path)

    e2e_elapsed, _, (e2e_tok_sum,) = reduce_max_sum(dist, local, e2e_elapsed, 0, [e2e_tokens])
    graph_stats = model.graph_stats()
    giveups = int(be.tcgen05_wait_giveups())
    parity = parity_check(args, cfg, be, pool, model, lanes, host_tokens) if world == 1 and not args.no_cpu_baseline else None
    # the dense model and its 66 GB of KV planes go before the sparse model comes
    model.close()
    pool.close()
    moe = None if args.no_moe else moe_ep(args, rank, world, local, dist)
    if rank != 0:
        return None
    peaks = load_peaks()
    # attn_bytes sums one launch per step; every step launches the kernel once per layer on the same lanes
    achieved = (attn_bytes * cfg["layers"] / 1e9) / (attn_ns * 1e-9) if attn_ns else None
    per_launch_bytes = attn_bytes / max(profiled_steps, 1)
    result = {
        "metric": "ragged decode tok/s", "value": total_tokens / elapsed, "unit": "tok/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "repeats": repeats,
        "block_tok_s": [round(b[1] / b[0], 1) for b in blocks],
        "ms_per_step": elapsed / args.steps * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "qwen3-0.6b-arch bf16 continuous-batching decode, 128 lanes, ctx log-uniform 128-%d, page 16" % args.ctx_max,
                   "lanes_per_gpu": args.lanes, "layers": cfg["layers"], "pool_pages": args.pool_pages, "admitted_requests": lanes.admitted,
                   "mean_kv_tokens_per_step": kv_tokens / args.steps, "parallelism": "independent replicas over sequences (no collective)",
                   "l2": "inputs larger than L2: each step streams the KV of every lane (tens of GB) and 1.19 GB of weights"},
        "clocks": clocks,
        "e2e": {"value": e2e_tok_sum / e2e_elapsed, "unit": "tok/s", "h2d_bytes_per_step": h2d / e2e_steps, "d2h_bytes_per_step": d2h / e2e_steps,
                "ms_per_step": e2e_elapsed / e2e_steps * 1e3, "mean_kv_tokens_per_step": e2e_kv_tokens / e2e_steps},
        "gpu_launches": int(launches),
        "health": {"tcgen05_wait_giveups": giveups},
        "graph_replay": graph_stats,
        "roofline": {"kernel": "attn_decode_mma_kernel (paged GQA decode attention, split-K)", "bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": (achieved / peaks["hbm_gbs"]) if achieved else None, "peak_source": peaks["source"],
                     "algorithmic_bytes_per_launch": per_launch_bytes, "launches": int(attn_launches), "avg_launch_us": attn_ns / max(attn_launches, 1) * 1e-3,
                     "attention_share_of_step": (attn_ns * 1e-9 / max(profiled_steps, 1)) / (elapsed / args.steps) if elapsed else None, "profiled_steps": profiled_steps, "work_items_last_step": stats["attn_work_items"],
                     "traffic": ncu_traffic_per_launch(per_launch_bytes)},
    }
    step_bytes = 2 * sum_weight_params(cfg) + (kv_tokens / args.steps) * cfg["layers"] * cfg["kv_heads"] * cfg["head_dim"] * 2 * 2
    result["step_roofline"] = {"algorithmic_gb_per_step": step_bytes / 1e9, "achieved_gbs": step_bytes / 1e9 / (elapsed / args.steps),
                               "frac_of_hbm_peak": step_bytes / 1e9 / (elapsed / args.steps) / peaks["hbm_gbs"]}
    if moe is not None:
        result["moe_ep"] = moe
    if parity is not None:
        result["parity_check"] = parity
    if world == 1 and not args.no_cpu_baseline:
        result["cpu_baseline"] = cpu_baseline(args, cfg)
    return result


def moe_ep(args, rank, world, local, dist):
    """The sharded sparse-MoE step (Qwen3-30B-A3B shape) beside the headline: 256 lanes in total, experts sharded over
    the ranks and the rows exchanged per MoE layer by peer stores and loads over NVLink (fj_moe_ep_* / fj_moe_step; NCCL
    send/recv with --moe-nccl), so that the scaling run carries its
    1/2/4/8-GPU numbers. Every rank takes part; the block reports whole-job tokens per second (maximum over ranks of the
    device time) and the step's phases."""
    from forja_b200 import benchmarks

    def exchange(mine):
        box = [mine]
        dist.broadcast_object_list(box, src=0)
        return box[0]

    def barrier_all():
        if dist is not None:
            dist.barrier()

    def gather(obj):
        out = [None] * world
        dist.all_gather_object(out, obj)
        return out

    def reduce(value, op):
        if dist is None:
            return value
        import torch
        t = torch.tensor([value], dtype=torch.float64, device=f"cuda:{local}")
        dist.all_reduce(t, op=op)
        return float(t.item())

    try:
        return benchmarks.moe_ep_block(rank, world, local, exchange, barrier_all, lambda v: reduce(v, dist.ReduceOp.MAX if dist else None),
                                       lambda v: reduce(v, dist.ReduceOp.SUM if dist else None), lanes_total=args.moe_lanes, steps=args.moe_steps, warmup=3,
                                       layers=args.moe_layers, seed=args.seed, all_gather=None if (dist is None or args.moe_nccl) else gather)
    except Exception as error:  # noqa: BLE001 - the headline line is still printed; the failure is reported in the block
        return {"error": f"{type(error).__name__}: {error}"}


def parity_check(args, cfg, be, pool, model, lanes, host_tokens):
    """After the timed regions, outside them: one more decode step of the running batch on the GPU with the
    logits kept, and the lane with the shortest context replayed on the CPU port from the very cache rows
    the GPU holds for it (read back page by page) and the same bf16 weights. Reports the logits' max-abs
    relative difference and whether the greedy tokens agree. Bound: 2e-2, or twice the comparison's noise
    floor where that is larger (the CPU port against itself with its projection sums re-associated: at 28
    bf16 layers that alone moves the logits by 1e-2 to 3e-2 of their maximum). The oracle is the checker
    here, not the thing measured."""
    import forja_b200 as fb
    from oracle import engine, fjo
    starts, tokens = lanes.descriptors()
    active = np.nonzero(tokens)[0]
    if active.size == 0:
        return None
    lane = int(active[np.argmin(starts[active])])
    start = int(starts[lane])
    table = pool.table(lane)
    bound = int((table[:, 1] != 0xFFFFFFFF).sum())
    bits = random_weights_bf16(cfg, args.seed)
    ref = engine.DenseOracle(cfg, None, bound + 1, PAGE, weight_bits=bits)
    reordered = engine.ReorderedDenseOracle(cfg, None, bound + 1, PAGE, weight_bits=bits)
    own_table, generations = engine.copy_lane_cache(ref, model.kv_pages, table, start, compact=True)
    for mine, theirs in zip(reordered.k_planes + reordered.v_planes, ref.k_planes + ref.v_planes):
        mine[:] = theirs
    logits = be.alloc(fb.BF16, (args.lanes, cfg["vocab"]))
    pool.pack_step(starts, tokens)
    got_tokens = model.step(host_tokens[tokens > 0], want_tokens=True, lanes=args.lanes, logits=logits)
    lanes.advance()
    got = fjo.decode(be.read(logits)[lane], fjo.BF16)
    fjo.set_threads(fjo.max_threads())
    want, want_token = ref.forward_lane([int(host_tokens[lane])], start, own_table, generations)
    other, _ = reordered.forward_lane([int(host_tokens[lane])], start, own_table, generations)
    fjo.set_threads(1)
    err = float(np.max(np.abs(got - want)) / np.max(np.abs(want)))
    noise = float(np.max(np.abs(other - want)) / np.max(np.abs(want)))
    return {"lane": lane, "context": start, "max_abs_rel": err, "noise_floor_max_abs_rel": noise,
            "bound": "max(2e-2, 2 x noise floor); noise floor = the CPU port against itself with re-associated projection sums",
            "within_bound": bool(err <= max(2e-2, 2.0 * noise)),
            "token_equal": bool(int(got_tokens[lane]) == want_token), "gpu_token": int(got_tokens[lane]), "cpu_token": int(want_token),
            "logit_gap_of_the_two_tokens_rel": float(abs(got[int(got_tokens[lane])] - got[want_token]) / np.max(np.abs(got)))}


def sum_weight_params(cfg):
    qd, kd = cfg["q_heads"] * cfg["head_dim"], cfg["kv_heads"] * cfg["head_dim"]
    per_layer = cfg["hidden"] * (qd + 2 * kd) + cfg["hidden"] * qd + 3 * cfg["hidden"] * cfg["intermediate"]
    return cfg["layers"] * per_layer + cfg["vocab"] * cfg["hidden"]


def load_peaks():
    """Roofline denominators: the driver-measured copy bandwidth of this pool's B200s, else the
    earlier pool measurement."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        data = json.load(open(path))
        return {"hbm_gbs": float(data["hbm_gbs"]), "source": "measured (MEASURED_PEAKS.json)"}
    except (OSError, KeyError, ValueError):
        return {"hbm_gbs": 6650.0, "source": "fallback (earlier pool measurement)"}


# DRAM traffic of the decode-attention kernel relative to its algorithmic bytes, from the ncu
# capture summarised in profiles/attn_decode_mma_small_case_ncu.md: dram__bytes_read.sum +
# dram__bytes_write.sum = 408.3 MB for a launch of 403.9 MB algorithmic bytes. The kernel reads
# every page once, so traffic scales with the attended tokens of the launch.
NCU_TRAFFIC_RATIO = 1.011


def ncu_traffic_per_launch(algorithmic_bytes):
    return None if NCU_TRAFFIC_RATIO is None else algorithmic_bytes * NCU_TRAFFIC_RATIO


def cpu_sample(args, cfg, n_lanes, threads, appended_tokens):
    """Builds the CPU port (the oracle engine, test infrastructure) on a sample of the workload:
    `n_lanes` requests drawn from the same length distribution, synthetic N(0,1) KV contexts. Every
    lane's page table has room for its context plus `appended_tokens` decode steps."""
    from oracle import engine, fjo
    fjo.set_threads(threads)
    requests = Requests(args.seed * 1000, args.ctx_max)
    sample = [requests.next() for _ in range(args.lanes)]
    pick = [sample[i] for i in np.linspace(0, args.lanes - 1, n_lanes).astype(int)]
    pages = [(ctx + appended_tokens + PAGE - 1) // PAGE for ctx, _ in pick]
    physical = sum(pages) + 1
    ref = engine.DenseOracle(cfg, None, physical, PAGE, weight_bits=random_weights_bf16(cfg, args.seed))
    rng = np.random.default_rng(args.seed)
    block = f32_to_bf16_bits(rng.standard_normal(1 << 20, dtype=np.float32))
    for plane in ref.k_planes + ref.v_planes:
        flat = plane.reshape(-1)
        flat[:] = np.resize(block, flat.size)
    generations = np.ones(physical, np.uint32)
    tables, cursor = [], 0
    for n in pages:
        t = np.zeros((n, 2), np.uint32)
        t[:, 0] = np.arange(cursor, cursor + n)
        t[:, 1] = 1
        tables.append(t)
        cursor += n
    return ref, pick, tables, generations


def cpu_decode_step(ref, pick, tables, generations, offset, n_lanes=None):
    """One decode step of the sampled lanes on the CPU port: lane i appends one token at position
    ctx_i + offset. Returns the tokens produced."""
    tokens = 0
    for (ctx, _), table in list(zip(pick, tables))[:n_lanes]:
        ref.forward_lane([(ctx * 7 + offset) % ref.cfg["vocab"]], ctx + offset, table, generations)
        tokens += 1
    return tokens


CPU_BASELINE_STEPS = 5  # timed steps per thread count (median reported), after one untimed step


def cpu_baseline(args, cfg):
    """Times the CPU port on this box's host cores on a bounded sample of the workload: decode steps
    of a few lanes of the same request stream through all layers, once with every host thread
    (OpenMP over rows/columns; `value`) and once on one core (`one_core`: forja-cpu itself is
    single-threaded, crates/forja-cpu/src/lib.rs:20-24). Median of CPU_BASELINE_STEPS steps each,
    after one untimed step. A reported baseline, not the optimisation target."""
    from oracle import fjo
    threads = fjo.max_threads()
    ref, pick, tables, generations = cpu_sample(args, cfg, 2, threads, 2 * (CPU_BASELINE_STEPS + 1))

    def median_rate(n_lanes, first_offset):
        cpu_decode_step(ref, pick, tables, generations, first_offset, n_lanes)
        rates = []
        for s in range(CPU_BASELINE_STEPS):
            t0 = time.perf_counter()
            tokens = cpu_decode_step(ref, pick, tables, generations, first_offset + 1 + s, n_lanes)
            rates.append(tokens / (time.perf_counter() - t0))
        return float(np.median(rates)), float(np.max(rates))

    all_median, all_best = median_rate(2, 0)
    fjo.set_threads(1)
    one_median, one_best = median_rate(1, CPU_BASELINE_STEPS + 1)
    contexts = [c for c, _ in pick]
    return {"value": all_median, "unit": "tok/s", "cores": threads, "kind": "port", "best": all_best,
            "one_core": {"value": one_median, "unit": "tok/s", "cores": 1, "best": one_best,
                         "sample": f"median of {CPU_BASELINE_STEPS} decode steps of 1 lane (context {contexts[0]}) after 1 untimed step"},
            "sample": f"median of {CPU_BASELINE_STEPS} decode steps of 2 lanes (contexts {contexts}) of the same request stream after 1 untimed step, all "
                      f"{cfg['layers']} layers, C++ restatement of forja-cpu with OpenMP over rows/columns"}


REFERENCE_BUDGET_S = 150.0


def run_reference(args):
    """Reference arm: forja's own CPU backend cannot be built here (Rust, no toolchain), so the CPU
    port (oracle restatement of crates/forja-cpu) is timed on the host cores with every thread it
    can use. Each step decodes a bounded sample of the workload: one lane of the same request stream
    through all layers. Steps and warm-up are the requested ones unless they would not fit in
    REFERENCE_BUDGET_S seconds."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    from oracle import fjo
    cfg = dict(QWEN3_06B)
    if args.layers:
        cfg["layers"] = args.layers
    threads = fjo.max_threads()
    n_lanes = 1
    # positions used: ctx + 0 (probe), ctx + 1 .. ctx + warmup + steps; the table holds one more
    ref, pick, tables, generations = cpu_sample(args, cfg, n_lanes, threads, 2 + args.warmup + args.steps)
    t0 = time.perf_counter()
    cpu_decode_step(ref, pick, tables, generations, 0)
    one = max(time.perf_counter() - t0, 1e-3)
    fit = int(REFERENCE_BUDGET_S / one)
    steps = max(1, min(args.steps, fit - args.warmup))
    warmup = min(args.warmup, max(0, fit - steps))
    for w in range(warmup):
        cpu_decode_step(ref, pick, tables, generations, 1 + w)
    tokens, durations = 0, []
    t_all = time.perf_counter()
    for s in range(steps):
        t0 = time.perf_counter()
        tokens += cpu_decode_step(ref, pick, tables, generations, 1 + warmup + s)
        durations.append(time.perf_counter() - t0)
    elapsed = time.perf_counter() - t_all
    fjo.set_threads(1)
    value = tokens / elapsed
    sample = f"each step decodes {n_lanes} lane (context {pick[0][0]}) of the same request stream through all {cfg['layers']} layers; {steps} timed steps"
    return {"impl": "reference", "metric": "ragged decode tok/s", "value": value, "unit": "tok/s", "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
            "ms_per_step": elapsed / steps * 1e3, "median_ms_per_step": float(np.median(durations)) * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "qwen3-0.6b-arch bf16 continuous-batching decode, 128 lanes, ctx log-uniform 128-%d, page 16" % args.ctx_max,
                       "note": "forja-cpu restated in C++ (the Rust reference cannot be compiled on this box); steps requested %d" % args.steps},
            "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}


def main():
    args = parse_args()
    result = run_reference(args) if args.impl == "reference" else run_native(args)
    try:  # leave the process group before the line is printed, so nothing follows it on the terminal
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            dist.destroy_process_group()
    except Exception:  # noqa: BLE001 - teardown only
        pass
    if result is not None:
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
