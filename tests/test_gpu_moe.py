"""Sparse-MoE decoder step (fj_moe_*) against the CPU oracle's replay of the reference op order
(engines/qwen3-coder/src/lib.rs:886-947, :505-603), and expert parallelism over two GPUs against the
single-GPU path. Tolerance: bf16 / 4-bit logits within max-abs rel 2e-2; greedy tokens equal or a
near-tie (reduced-precision rule of the reference, docs/engines.md:108-111)."""
import os
import subprocess
import sys

import numpy as np
import pytest

import forja_b200 as fb
from oracle import engine, fjo
from tests.gpu_util import backend, down, max_abs_rel

pytestmark = pytest.mark.gpu

TINY = dict(layers=2, hidden=256, q_heads=4, kv_heads=2, head_dim=64, experts=8, top_k=2, expert_intermediate=128, vocab=512,
            group_size=64, router_bits=8, eps=1e-6, theta=1e7, max_rows=160)
# head_dim 128 with 8 query heads per KV head: the decode steps run the tensor-core attention and,
# with at most 16 rows, the streaming q4 projection kernels
CODER_LIKE = dict(layers=2, hidden=512, q_heads=8, kv_heads=1, head_dim=128, experts=16, top_k=4, expert_intermediate=192, vocab=1024,
                  group_size=64, router_bits=8, eps=1e-6, theta=1e7, max_rows=96)


def upload_moe(be, weights):
    def triple(t):
        return (be.tensor_from(t[0], fb.U32), be.tensor_from(t[1], fb.BF16), be.tensor_from(t[2], fb.BF16))

    layers = []
    for layer in weights["layers"]:
        entry = {k: be.tensor_from(layer[k], fb.BF16) for k in ("input_norm", "q_norm", "k_norm", "post_norm")}
        entry.update({k: triple(layer[k]) for k in ("qkv", "o", "router", "gate", "up", "down")})
        layers.append(entry)
    return triple(weights["embed"]), be.tensor_from(weights["final_norm"], fb.BF16), triple(weights["lm_head"]), layers


def near_tie_flips(tokens, ref_tokens, got_logits):
    flips = 0
    for lane, (got, want) in enumerate(zip(tokens.tolist(), ref_tokens)):
        if got != want:
            row = got_logits[lane]
            assert abs(row[got] - row[want]) <= 2e-2 * np.max(np.abs(row)), "token differs without a near-tie"
            flips += 1
    return flips


# the long prompts put more than 64 routes into one step: routes bucketed by expert (streamed 16-row tiles, or tile GEMMs from
# 72 rows per expert on); the rest: one pass per route
@pytest.mark.parametrize("cfg,prompts,steps", [(TINY, [5, 23, 9], 5), (CODER_LIKE, [3, 17, 1, 8], 6), (TINY, [70, 40, 9], 3), (CODER_LIKE, [40, 33], 2)])
def test_moe_step_matches_oracle(cfg, prompts, steps):
    """Two claims, checked separately. (1) Routing: every layer's top-k expert set on the GPU equals the oracle's,
    except where the oracle's own decision was a near-tie (the last routed expert ahead of the first one left out
    by less than 3 % of the row's largest router logit): the q8 router sums in another order on the GPU and its
    input is bf16, so such ties may resolve the other way (the reference documents the effect,
    engines/olmoe/README.md:157-165). (2) Values: with the GPU's routing handed to the oracle, logits agree within
    max-abs rel 2e-2 and greedy tokens are equal or a near-tie of the logits."""
    rng = np.random.default_rng(3)
    be = backend()
    page, lanes = 16, len(prompts)
    table_pages = max((n + steps + page - 1) // page for n in prompts) + 1
    physical = sum((n + steps + page - 1) // page for n in prompts) + 3
    pool = fb.KvPool(be, page, physical, lanes, table_pages)
    assert all(s == 0 for s in pool.reserve(list(range(lanes)), [n + steps for n in prompts]))
    weights = engine.random_moe_weights(cfg, 11)
    embed, final_norm, lm_head, layers = upload_moe(be, weights)
    model = fb.MoeModel(be, pool, cfg, embed, final_norm, lm_head, layers)
    model.capture_routes(True)
    ref = engine.MoeOracle(cfg, weights, physical, page)
    tables = [pool.table(lane) for lane in range(lanes)]
    generations = pool.generations()
    ids = [rng.integers(0, cfg["vocab"], n).astype(np.uint32) for n in prompts]
    logits = be.alloc(fb.BF16, (lanes, cfg["vocab"]))
    fjo.set_threads(fjo.max_threads())
    decisions = disagreements = flips = 0

    def replay(step_tokens, starts, counts, where):
        """Runs the oracle for every lane of the step that just ran on the GPU, with the GPU's routing."""
        nonlocal decisions, disagreements
        rows = int(sum(counts))
        routes = [model.routes(layer, rows)[0] for layer in range(cfg["layers"])]
        got = down(logits)
        out_tokens, offset = [], 0
        for lane in range(lanes):
            n = counts[lane]
            forced = [r[offset:offset + n] for r in routes]
            want, tok = ref.forward_lane(step_tokens[lane], starts[lane], tables[lane], generations, forced_routes=forced)
            offset += n
            decisions += n * cfg["layers"]
            for layer, row, margin in ref.route_disagreements:
                assert margin < 0.03, f"{where} lane {lane} layer {layer} row {row}: experts differ although the oracle's margin was {margin:.3f}"
            disagreements += len(ref.route_disagreements)
            err = max_abs_rel(got[lane], want)
            assert err <= 2e-2, f"{where} lane {lane}: logits max-abs rel {err:.3e}"
            out_tokens.append(tok)
        return got, out_tokens

    pool.pack_step([0] * lanes, prompts)
    tokens = model.step(np.concatenate(ids), lanes=lanes, logits=logits)
    got, ref_tokens = replay(ids, [0] * lanes, prompts, "prefill")
    flips += near_tie_flips(tokens, ref_tokens, got)
    positions = list(prompts)
    for step in range(steps):
        pool.pack_step(positions, [1] * lanes)
        tokens = model.step(np.array(ref_tokens, np.uint32), lanes=lanes, logits=logits)  # teacher-forced
        got, ref_tokens = replay([[t] for t in ref_tokens], positions, [1] * lanes, f"step {step}")
        flips += near_tie_flips(tokens, ref_tokens, got)
        positions = [p + 1 for p in positions]
    fjo.set_threads(1)
    assert flips <= max(1, int(0.05 * lanes * (steps + 1)))
    # every disagreement above was individually checked to be a near-tie of the oracle; this bounds how many there may be
    assert disagreements <= max(4, int(0.05 * decisions)), f"{disagreements} of {decisions} routing decisions differ"
    print(f"routing decisions {decisions}, resolved differently at near-ties {disagreements}, token near-tie flips {flips}")
    assert model.stats()["kernels"] > 0
    model.close()
    pool.close()


def test_device_wait_of_the_direct_exchange_gives_up_and_reports():
    """The receiver of the direct exchange polls a flag in its own memory with a bound. Here nothing ever sets the flag:
    the kernel has to return by itself, report the exchange number it waited for, and leave the context usable."""
    be = backend()
    assert be._lib.fj_ep_wait_selftest(be._h, 3000) == fb.backend.TIMEOUT
    x = be.tensor_from(np.arange(8, dtype=np.float32), fb.F32)
    assert be.read(x).tolist() == list(range(8))


def test_expert_parallel_step_equals_single_gpu_bits():
    """Two ranks, one GPU each, experts split in half: every rank's logits must equal, bit for bit,
    what one GPU computes for the same lanes (each route runs the same arithmetic either way)."""
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", MASTER_ADDR="127.0.0.1", MASTER_PORT="29741")
    script = os.path.join(os.path.dirname(__file__), "ep_child.py")
    procs = [subprocess.Popen([sys.executable, script, str(rank), "2"], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for rank in range(2)]
    outputs = []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=600)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
        outputs.append(out)
    for rank, (p, out) in enumerate(zip(procs, outputs)):
        assert p.returncode == 0, f"rank {rank} failed:\n{out[-4000:]}"
        assert "EP_OK" in out, out[-2000:]
