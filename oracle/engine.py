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

    def __init__(self, cfg: dict, weights: dict, physical_pages: int, page_tokens: int):
        self.cfg, self.dt, self.page_tokens = cfg, cfg["dtype"], page_tokens
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
