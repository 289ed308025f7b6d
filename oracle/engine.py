"""Dense decoder step composed from oracle operators in the reference engines' op order
(Qwen3: engines/qwen3/src/lib.rs:391-452, 734-811; SmolLM2: engines/smollm2/src/optimized.rs:97-245).

TEST INFRASTRUCTURE ONLY (part of the CPU oracle): used by the parity tests, the smoke check and
the CPU-baseline leg of the benchmark. Every dispatch of the reference is one oracle call, so each
intermediate is rounded to the activation dtype exactly where the reference materialises it.
"""
from __future__ import annotations

import numpy as np

from . import fjo


def random_dense_weights(cfg: dict, seed: int = 0):
    """Random-init weights N(0, 0.02), norm gains 1 + N(0, 0.02) (the reference's random-weight
    recipe offsets norm tensors by 1.0, crates/forja-host/tests/smollm2.rs:46-52). Values are
    rounded to bf16-representable numbers so f32 and bf16 conventions coincide
    (EmbeddingConfig::promoted_bf16, crates/forja-sdk/src/nn.rs:211-219). Returns f32 arrays."""
    rng = np.random.default_rng(seed)
    H, I, V, d = cfg["hidden"], cfg["intermediate"], cfg["vocab"], cfg["head_dim"]
    qd, kd = cfg["q_heads"] * d, cfg["kv_heads"] * d

    def mat(rows, cols):
        return fjo.decode(fjo.encode((rng.standard_normal((rows, cols)) * 0.02).astype(np.float32), fjo.BF16), fjo.BF16)

    def gain(n):
        return fjo.decode(fjo.encode((1.0 + rng.standard_normal(n) * 0.02).astype(np.float32), fjo.BF16), fjo.BF16)

    weights = {"embed": mat(V, H), "final_norm": gain(H), "layers": []}
    for _ in range(cfg["layers"]):
        layer = {"input_norm": gain(H), "wq": mat(qd, H), "wk": mat(kd, H), "wv": mat(kd, H), "wo": mat(H, qd), "post_norm": gain(H),
                 "w_gate": mat(I, H), "w_up": mat(I, H), "w_down": mat(H, I)}
        if cfg["qk_norm"]:
            layer["q_norm"], layer["k_norm"] = gain(d), gain(d)
        weights["layers"].append(layer)
    return weights


class DenseOracle:
    """Reference-order forward step over paged KV. ``dt`` is the activation/weight/KV dtype code."""

    def __init__(self, cfg: dict, weights: dict, physical_pages: int, page_tokens: int, weight_bits: dict = None):
        """``weights``: f32 arrays (encoded here to the storage dtype); or ``weight_bits``: the same
        dictionary already in storage form (bf16 bit patterns as uint16), used as it is."""
        self.cfg, self.dt, self.page_tokens = cfg, cfg["dtype"], page_tokens
        if weight_bits is not None:
            self.w = weight_bits
        else:
            enc = lambda a: fjo.encode(a, self.dt)
            self.w = {"embed": enc(weights["embed"]), "final_norm": enc(weights["final_norm"]),
                      "layers": [{k: enc(v) for k, v in layer.items()} for layer in weights["layers"]]}
        kd = cfg["kv_heads"] * cfg["head_dim"]
        self.k_planes = [np.zeros((physical_pages, page_tokens, kd), fjo.NP_OF[self.dt]) for _ in range(cfg["layers"])]
        self.v_planes = [np.zeros((physical_pages, page_tokens, kd), fjo.NP_OF[self.dt]) for _ in range(cfg["layers"])]
        self.scale = float(np.float32(1.0) / np.sqrt(np.float32(cfg["head_dim"])))

    def _linear(self, x, w):
        return fjo.matmul(x, self.dt, w, self.dt, self.dt, right_transposed=True)

    def forward_lane(self, token_ids, start: int, table: np.ndarray, generations: np.ndarray):
        """One lane: ``token_ids`` appended at ``start``. Returns (logits of the last row as f32,
        greedy token). table: [table_pages, 2], generations: [physical_pages]."""
        cfg, dt = self.cfg, self.dt
        T, d, hq, kvh = len(token_ids), cfg["head_dim"], cfg["q_heads"], cfg["kv_heads"]
        eps, theta = cfg["eps"], cfg["theta"]
        hidden = fjo.embed(self.w["embed"], dt, np.asarray(token_ids, np.uint32))
        positions_u32 = np.arange(start, start + T, dtype=np.uint32)
        positions_f32 = positions_u32.astype(np.float32)
        first = self.w["layers"][0]
        normed = fjo.prog_rms_norm(hidden, dt, first["input_norm"], dt, eps) if cfg["qk_norm"] else fjo.rms_norm(hidden, dt, first["input_norm"], dt, eps)
        for li, L in enumerate(self.w["layers"]):
            q = self._linear(normed, L["wq"]).reshape(T, hq, d)
            k = self._linear(normed, L["wk"]).reshape(T, kvh, d)
            v = self._linear(normed, L["wv"]).reshape(T, kvh, d)
            if cfg["qk_norm"]:
                q = fjo.prog_qk_norm_rope(q, dt, L["q_norm"], dt, positions_f32, eps, theta)
                k = fjo.prog_qk_norm_rope(k, dt, L["k_norm"], dt, positions_f32, eps, theta)
            else:
                q = fjo.rope(q, dt, positions_u32, theta)
                k = fjo.rope(k, dt, positions_u32, theta)
            fjo.paged_copy_in(k.reshape(T, kvh * d), dt, self.k_planes[li], dt, table, generations, start, self.page_tokens)
            fjo.paged_copy_in(v.reshape(T, kvh * d), dt, self.v_planes[li], dt, table, generations, start, self.page_tokens)
            P = self.k_planes[li].shape[0]
            attended = fjo.paged_sdpa(np.ascontiguousarray(q.transpose(1, 0, 2)), dt, self.k_planes[li].reshape(P, self.page_tokens, kvh, d), dt,
                                      self.v_planes[li].reshape(P, self.page_tokens, kvh, d), dt, table, generations, start + T, start, self.scale, True,
                                      self.page_tokens)
            attended = np.ascontiguousarray(attended.transpose(1, 0, 2)).reshape(T, hq * d)
            attention = self._linear(attended, L["wo"])
            if cfg["qk_norm"]:
                hidden, normed = fjo.prog_residual_norm(hidden, attention, dt, L["post_norm"], dt, eps)
            else:
                hidden = fjo.prog_add(hidden, attention, dt)
                normed = fjo.rms_norm(hidden, dt, L["post_norm"], dt, eps)
            gate, up = self._linear(normed, L["w_gate"]), self._linear(normed, L["w_up"])
            projected = self._linear(fjo.prog_silu_mul(gate, up, dt), L["w_down"])
            if li + 1 < len(self.w["layers"]):
                nxt = self.w["layers"][li + 1]["input_norm"]
                if cfg["qk_norm"]:
                    hidden, normed = fjo.prog_residual_norm(hidden, projected, dt, nxt, dt, eps)
                else:
                    hidden = fjo.prog_add(hidden, projected, dt)
                    normed = fjo.rms_norm(hidden, dt, nxt, dt, eps)
            else:
                hidden = fjo.prog_add(hidden, projected, dt)
        last = hidden[T - 1:T]
        final = fjo.prog_rms_norm(last, dt, self.w["final_norm"], dt, eps) if cfg["qk_norm"] else fjo.rms_norm(last, dt, self.w["final_norm"], dt, eps)
        logits = self._linear(final, self.w["embed"])
        token = int(fjo.argmax(logits, dt)[0])
        return fjo.decode(logits, dt)[0], token


class ReorderedDenseOracle(DenseOracle):
    """The same step with one liberty taken: every projection sums its products in blocked (BLAS) order instead
    of sequentially in index order. Accumulation stays f32 and every rounding point stays where it is, so this
    is what any implementation that does not copy the reference's scalar summation order can hope to match.
    The distance between this oracle and DenseOracle on the same inputs is the noise floor of the comparison:
    a deep bf16 model amplifies last-place differences of the sums through the bf16 roundings that follow."""

    def _linear(self, x, w):
        cache = self.__dict__.setdefault("_f32_weights", {})
        wf = cache.get(id(w))
        if wf is None:
            wf = cache[id(w)] = fjo.decode(w, self.dt)
        return fjo.encode((fjo.decode(x, self.dt) @ wf.T).astype(np.float32), self.dt)


def random_moe_weights(cfg: dict, seed: int = 0):
    """Random MLX-affine weights for the sparse-MoE decoder: uniformly random codes, positive scales
    and biases that centre every group near zero. Returns numpy arrays: quantised tensors as
    (packed u32, scales bf16 bits, biases bf16 bits) triples, norm gains as bf16 bit arrays."""
    rng = np.random.default_rng(seed)
    H, I, V, d, E = cfg["hidden"], cfg["expert_intermediate"], cfg["vocab"], cfg["head_dim"], cfg["experts"]
    qd, kd, G = cfg["q_heads"] * d, cfg["kv_heads"] * d, cfg["group_size"]

    def quant(shape_n, k, bits=4, spread=0.006):
        lead = shape_n if isinstance(shape_n, tuple) else (shape_n,)
        packed = rng.integers(0, 2 ** 32, lead + (k * bits // 32,), dtype=np.uint64).astype(np.uint32)
        scales = (np.abs(rng.standard_normal(lead + (k // G,))) * spread + spread * 0.25).astype(np.float32)
        if bits == 8:
            scales = scales / 16.0
        centre = (2 ** bits - 1) / 2.0
        biases = (-centre * scales + rng.standard_normal(lead + (k // G,)) * spread * 0.5).astype(np.float32)
        return packed, fjo.encode(scales, fjo.BF16), fjo.encode(biases, fjo.BF16)

    def gain(n):
        return fjo.encode((1.0 + rng.standard_normal(n) * 0.02).astype(np.float32), fjo.BF16)

    weights = {"embed": quant(V, H, spread=0.02), "final_norm": gain(H), "lm_head": quant(V, H), "layers": []}
    for _ in range(cfg["layers"]):
        weights["layers"].append({
            "input_norm": gain(H), "q_norm": gain(d), "k_norm": gain(d), "post_norm": gain(H),
            "qkv": quant(qd + 2 * kd, H), "o": quant(H, qd), "router": quant(E, H, bits=cfg["router_bits"], spread=0.02),
            "gate": quant((E, I), H), "up": quant((E, I), H), "down": quant((E, H), I)})
    return weights


class MoeOracle:
    """Reference-order forward step of the sparse-MoE decoder over paged KV (Qwen3-Coder,
    engines/qwen3-coder/src/lib.rs:886-947 and :505-603), one lane at a time. Activations bf16;
    router logits, routing weights and the inputs of the fused epilogues f32 (an epilogue of the
    reference sees the f32 accumulator and its output is rounded once)."""

    def __init__(self, cfg: dict, weights: dict, physical_pages: int, page_tokens: int):
        self.cfg, self.w, self.page_tokens = cfg, weights, page_tokens
        kd = cfg["kv_heads"] * cfg["head_dim"]
        self.k_planes = [np.zeros((physical_pages, page_tokens, kd), np.uint16) for _ in range(cfg["layers"])]
        self.v_planes = [np.zeros((physical_pages, page_tokens, kd), np.uint16) for _ in range(cfg["layers"])]
        self.scale = float(np.float32(1.0) / np.sqrt(np.float32(cfg["head_dim"])))

    def _q(self, x, triple, bits=4, out_dt=None):
        return fjo.quant_matmul(x, fjo.BF16, triple[0], triple[1], triple[2], fjo.BF16, bits, self.cfg["group_size"], fjo.BF16 if out_dt is None else out_dt)

    def moe(self, normed, residual, L, forced_experts=None):
        """Returns (new residual stream, router logits f32, expert ids, routing weights). With
        ``forced_experts`` [rows, top_k] the block uses that routing (weights from its own logits:
        exp(v_i - v_first) / sum over the forced set) and keeps its own choice in ``self.own_experts``."""
        cfg, G = self.cfg, self.cfg["group_size"]
        logits = self._q(normed, L["router"], bits=cfg["router_bits"], out_dt=fjo.F32)
        weights, experts = fjo.top_k(logits, fjo.F32, cfg["top_k"], True)
        self.own_experts = experts
        if forced_experts is not None:
            experts = np.ascontiguousarray(forced_experts, np.uint32)
            picked = np.take_along_axis(logits.astype(np.float32), experts.astype(np.int64), axis=-1)
            e = np.exp((picked - picked[:, :1]).astype(np.float32)).astype(np.float32)
            weights = (e / e.sum(axis=-1, keepdims=True, dtype=np.float32)).astype(np.float32)
        gate = fjo.gather_quant_matmul(normed, fjo.BF16, *L["gate"], fjo.BF16, experts, 4, G, out_dt=fjo.F32)
        up = fjo.gather_quant_matmul(normed, fjo.BF16, *L["up"], fjo.BF16, experts, 4, G, out_dt=fjo.F32)
        act = fjo.prog_silu_mul(gate, up, fjo.F32, out_dt=fjo.BF16)
        mixed = fjo.gather_quant_weighted_sum(act, fjo.BF16, *L["down"], fjo.BF16, experts, weights, fjo.F32, 4, G, fjo.F32)
        out = fjo.prog_add(mixed, fjo.decode(residual, fjo.BF16), fjo.F32, out_dt=fjo.BF16)
        return out, logits, experts, weights

    def forward_lane(self, token_ids, start: int, table: np.ndarray, generations: np.ndarray, forced_routes=None):
        """``forced_routes``: per layer, expert ids [T, top_k] to use instead of the oracle's own top-k.
        ``self.route_disagreements`` then lists (layer, row, relative margin of the oracle's own decision)
        for every row whose forced expert set differs from the oracle's."""
        cfg, dt = self.cfg, fjo.BF16
        self.route_disagreements = []
        T, d, hq, kvh = len(token_ids), cfg["head_dim"], cfg["q_heads"], cfg["kv_heads"]
        eps, theta, G = cfg["eps"], cfg["theta"], cfg["group_size"]
        hidden = fjo.quant_embed(*self.w["embed"], fjo.BF16, np.asarray(token_ids, np.uint32), 4, G, dt)
        # smallest gap, relative to the largest |logit| of the row, between the last routed expert and the first one
        # left out, over all rows and layers of this call: tells a caller how close the routing was to a tie
        self.last_min_margin = float("inf")
        positions = np.arange(start, start + T, dtype=np.uint32).astype(np.float32)
        normed = fjo.rms_norm(hidden, dt, self.w["layers"][0]["input_norm"], dt, eps)
        for li, L in enumerate(self.w["layers"]):
            qkv = self._q(normed, L["qkv"])
            q = np.ascontiguousarray(qkv[:, :hq * d]).reshape(T, hq, d)
            k = np.ascontiguousarray(qkv[:, hq * d:(hq + kvh) * d]).reshape(T, kvh, d)
            v = np.ascontiguousarray(qkv[:, (hq + kvh) * d:]).reshape(T, kvh, d)
            q = fjo.prog_qk_norm_rope(q, dt, L["q_norm"], dt, positions, eps, theta)
            k = fjo.prog_qk_norm_rope(k, dt, L["k_norm"], dt, positions, eps, theta)
            fjo.paged_copy_in(k.reshape(T, kvh * d), dt, self.k_planes[li], dt, table, generations, start, self.page_tokens)
            fjo.paged_copy_in(v.reshape(T, kvh * d), dt, self.v_planes[li], dt, table, generations, start, self.page_tokens)
            P = self.k_planes[li].shape[0]
            attended = fjo.paged_sdpa(np.ascontiguousarray(q.transpose(1, 0, 2)), dt, self.k_planes[li].reshape(P, self.page_tokens, kvh, d), dt,
                                      self.v_planes[li].reshape(P, self.page_tokens, kvh, d), dt, table, generations, start + T, start, self.scale, True,
                                      self.page_tokens)
            attended = np.ascontiguousarray(attended.transpose(1, 0, 2)).reshape(T, hq * d)
            hidden, normed = fjo.prog_residual_norm(hidden, self._q(attended, L["o"]), dt, L["post_norm"], dt, eps)
            forced = None if forced_routes is None else forced_routes[li]
            hidden, router_logits, _, _ = self.moe(normed, hidden, L, forced)
            ranked = np.sort(router_logits.astype(np.float32), axis=-1)[:, ::-1]
            k = cfg["top_k"]
            gaps = (ranked[:, k - 1] - ranked[:, k]) / np.maximum(np.abs(ranked).max(axis=-1), 1e-30)
            self.last_min_margin = min(self.last_min_margin, float(gaps.min()))
            if forced is not None:
                for row in range(T):
                    if set(int(v) for v in forced[row]) != set(int(v) for v in self.own_experts[row]):
                        self.route_disagreements.append((li, row, float(gaps[row])))
            nxt = self.w["layers"][li + 1]["input_norm"] if li + 1 < len(self.w["layers"]) else self.w["final_norm"]
            normed = fjo.prog_rms_norm(hidden, dt, nxt, dt, eps)
        logits = self._q(normed[T - 1:T], self.w["lm_head"])
        return fjo.decode(logits, dt)[0], int(fjo.argmax(logits, dt)[0])


class Bf16WeightMoeOracle(MoeOracle):
    """MoeOracle with one liberty taken in the 4-bit projections of the attention block and the lm_head: the
    dequantised weight s * q + b (f32, as the reference forms it, crates/forja-cpu/src/lib.rs:878-962) is rounded
    to bf16 before the products, which is what a tensor-core GEMM over 16-bit operands has to do, and the sums run
    in blocked (BLAS) order. Accumulation stays f32 and every other rounding point stays in place. The distance
    between this oracle and MoeOracle on the same inputs and routing is the floor of a comparison against such a
    GEMM: each projection moves by about 2e-3 normwise, and a layer amplifies that."""

    def _q(self, x, triple, bits=4, out_dt=None):
        if bits != 4:
            return super()._q(x, triple, bits, out_dt)
        cache = self.__dict__.setdefault("_bf16_weights", {})
        wf = cache.get(id(triple[0]))
        if wf is None:
            packed, G = triple[0], self.cfg["group_size"]
            q = ((packed[..., None] >> (np.arange(8, dtype=np.uint32) * 4)) & 15).reshape(packed.shape[0], -1).astype(np.float32)
            s = np.repeat(fjo.decode(triple[1], fjo.BF16), G, axis=-1)
            b = np.repeat(fjo.decode(triple[2], fjo.BF16), G, axis=-1)
            wf = cache[id(triple[0])] = fjo.decode(fjo.encode((s * q).astype(np.float32) + b, fjo.BF16), fjo.BF16)
        y = (fjo.decode(x, fjo.BF16) @ wf.T).astype(np.float32)
        return y if out_dt == fjo.F32 else fjo.encode(y, fjo.BF16)


def ep_moe_layer(rank: int, world: int, cfg: dict, normed, residual, L_local: dict, router, exchange, chunks: int = 1):
    """Expert-parallel form of MoeOracle.moe for one rank, restating the device algorithm in numpy:
    slots are handed out per destination in (row, j) order, slabs are exchanged, the owner computes
    gate/up/silu/down for every received slot, results return as f32 and the origin adds
    residual + sum_j w_j * down_j in ascending j (product rounded, then added).
    ``L_local`` holds this rank's expert slice; ``exchange(array)`` takes [world, ...] slabs and
    returns the slabs addressed to this rank, [world, ...] indexed by source.
    ``chunks`` > 1 restates the layout of the direct exchange with a layer's rows in several chunks:
    chunk c covers rows [c * ceil(rows / chunks), ...) of this rank, owns slots
    [c * cap_c, (c + 1) * cap_c) of every slab (cap_c = ceil(max_rows / chunks) * top_k) and announces
    how many of them it filled per destination (the payload of the device's flags); the owner visits
    exactly the announced slots of every (chunk, source)."""
    G, K, H, I = cfg["group_size"], cfg["top_k"], cfg["hidden"], cfg["expert_intermediate"]
    per = cfg["experts"] // world
    rows = normed.shape[0]
    chunks = max(1, int(chunks))
    cap_c = (cfg["max_rows"] + chunks - 1) // chunks * K
    cap = chunks * cap_c
    rows_c = (rows + chunks - 1) // chunks
    logits = fjo.quant_matmul(normed, fjo.BF16, *router, fjo.BF16, cfg["router_bits"], G, fjo.F32)
    weights, experts = fjo.top_k(logits, fjo.F32, K, True) if rows else (np.zeros((0, K), np.float32), np.zeros((0, K), np.uint32))
    send_rows = np.zeros((world, cap, H), np.uint16)
    send_experts = np.full((world, cap), per, np.uint32)
    send_counts = np.zeros((world, chunks), np.uint32)  # [destination][chunk]
    route_slot = np.zeros((rows, K), np.int64)
    for r in range(rows):
        c = r // rows_c
        for j in range(K):
            dest = int(experts[r, j]) // per
            slot = c * cap_c + int(send_counts[dest, c])
            assert send_counts[dest, c] < cap_c
            send_counts[dest, c] += 1
            route_slot[r, j] = dest * cap + slot
            send_rows[dest, slot] = normed[r]
            send_experts[dest, slot] = int(experts[r, j]) - dest * per
    recv_rows, recv_experts, recv_counts = exchange(send_rows), exchange(send_experts), exchange(send_counts)
    down = np.zeros((world, cap, H), np.float32)
    for c in range(chunks):
        for src in range(world):
            live = c * cap_c + np.arange(int(recv_counts[src, c]))
            if live.size == 0:
                continue
            assert np.all(recv_experts[src, live] < per)
            x = np.ascontiguousarray(recv_rows[src, live])
            ids = np.ascontiguousarray(recv_experts[src, live]).reshape(-1, 1)
            gate = fjo.gather_quant_matmul(x, fjo.BF16, *L_local["gate"], fjo.BF16, ids, 4, G, out_dt=fjo.F32)
            up = fjo.gather_quant_matmul(x, fjo.BF16, *L_local["up"], fjo.BF16, ids, 4, G, out_dt=fjo.F32)
            act = fjo.prog_silu_mul(gate, up, fjo.F32, out_dt=fjo.BF16).reshape(live.size, I)
            down[src, live] = fjo.gather_quant_matmul(act, fjo.BF16, *L_local["down"], fjo.BF16, ids, 4, G, out_dt=fjo.F32).reshape(live.size, H)
    returned = exchange(down).reshape(world * cap, H)
    out = np.zeros((rows, H), np.uint16)
    res = fjo.decode(residual, fjo.BF16) if rows else np.zeros((0, H), np.float32)
    for r in range(rows):
        total = np.zeros(H, np.float32)
        for j in range(K):
            total = (total + (weights[r, j] * returned[route_slot[r, j]]).astype(np.float32)).astype(np.float32)
        out[r] = fjo.encode((total + res[r]).astype(np.float32), fjo.BF16)
    return out


def copy_lane_cache(oracle, read_pages, table: np.ndarray, tokens: int, compact: bool = False):
    """Copies the K/V rows a lane holds on the device into ``oracle``'s planes, page by page, so that
    the CPU replay of that lane starts from the very cache contents the device kernel reads.
    ``read_pages(layer, plane, first_page, count)`` returns [count, page_tokens, kv_dim] storage values
    (plane 0 = K, 1 = V); ``table`` is the lane's page table [table_pages, 2]; ``tokens`` = rows in use.
    ``compact``: the oracle's planes hold only this lane (its i-th bound page becomes oracle page i), for
    device pools too large to mirror on the host. Returns (table, generations) to replay the lane with."""
    bound = int((table[:, 1] != 0xFFFFFFFF).sum())
    used = (tokens + oracle.page_tokens - 1) // oracle.page_tokens
    pages = [int(p) for p in table[:used, 0]]
    runs, i = [], 0
    while i < len(pages):  # runs of consecutive physical pages: one device read each
        j = i
        while j + 1 < len(pages) and pages[j + 1] == pages[j] + 1:
            j += 1
        runs.append((i, pages[i], j - i + 1))
        i = j + 1
    for layer in range(oracle.cfg["layers"]):
        for plane, planes in ((0, oracle.k_planes), (1, oracle.v_planes)):
            for index, first, count in runs:
                dst = index if compact else first
                planes[layer][dst:dst + count] = read_pages(layer, plane, first, count)
    if not compact:
        return table, None
    own = table.copy()
    own[:bound, 0] = np.arange(bound, dtype=np.uint32)
    generations = np.zeros(oracle.k_planes[0].shape[0], np.uint32)
    generations[:bound] = table[:bound, 1]
    return own, generations
