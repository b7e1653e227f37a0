"""NumPy restatement of the reference's decoder forward.  TEST INFRASTRUCTURE ONLY.

Follows crates/quantibbler-server/src/engine/mod.rs: transformer (:878-945), norm_apply
(:837-851), rms_norm_into (:1154-1160), rope_rotate (:1169-1184), gqa_attention_scalar
(:1074-1121, through oracle.gqa_attention_scalar), logits (:788-800) and
sampler.rs:5-16 (greedy).  The linears go through oracle.layer_apply, which is pinned to
the reference's vectors; the whole forward is pinned by the reference's model-level golden
(tests/fixtures/parity-tiny: logits of eight teacher-forced positions, budget 1e-2 as in
crates/quantibbler-server/tests/parity_tiny.rs:26), read through the model-directory reader.
"""

from __future__ import annotations

import numpy as np

import oracle


def _bf16(a):
    return oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits(np.asarray(a, np.float32)))


def rms_norm(x, w, eps, serving):
    x = np.asarray(x, np.float32)
    if serving == "bfloat16":
        x = _bf16(x)
    ss = np.float32(0.0)
    for v in x:  # sequential float32 sum, as the iterator sum in the reference
        ss = np.float32(ss + v * v)
    ss = np.float32(ss / np.float32(len(x)))
    inv = np.float32(1.0) / np.sqrt(np.float32(ss + np.float32(eps)))
    out = (x * inv * w).astype(np.float32)
    return _bf16(out) if serving == "bfloat16" else out


def per_head_norm(v, w, head_dim, eps, serving):
    """One head_dim weight vector applied to every head's slice (engine/mod.rs:854-873)."""
    v = np.asarray(v, np.float32)
    return np.concatenate([rms_norm(v[i:i + head_dim], w, eps, serving)
                           for i in range(0, len(v), head_dim)])


def rope_rotate(v, head_dim, pos, theta):
    v = np.array(v, np.float32, copy=True)
    half = head_dim // 2
    for head in range(len(v) // head_dim):
        base = head * head_dim
        for i in range(half):
            inv_freq = float(theta) ** (-(2.0 * i) / head_dim)
            s, c = np.float32(np.sin(pos * inv_freq)), np.float32(np.cos(pos * inv_freq))
            a, b = v[base + i], v[base + half + i]
            v[base + i] = a * c - b * s
            v[base + half + i] = b * c + a * s
    return v


def apply(layer, x, serving):
    return oracle.layer_apply(layer["ub_rows"], layer["vb_t_rows"], layer["dout"], layer["din"],
                              layer["r"], layer["s1"], layer["s2"], layer.get("bias"), x,
                              serving=serving)


class Session:
    """One sequence: weights + an append-only KV cache (KvCache, engine/mod.rs:1189-1209)."""

    def __init__(self, cfg, weights, kv_round=None, reduce=None):
        # ``reduce``: sums a rank's partial o / down output over the tensor-parallel ranks (the
        # one all-reduce per sub-block); None on a single rank
        self.cfg, self.w, self.reduce = cfg, weights, reduce or (lambda part: part)
        self.keys = [[] for _ in range(cfg.n_layers)]
        self.vals = [[] for _ in range(cfg.n_layers)]
        self.kv_round = kv_round  # optional storage rounding of the cache (bfloat16 cache)

    def transformer(self, x):
        cfg, sv = self.cfg, self.cfg.serving
        pos = len(self.keys[0])
        h = np.asarray(x, np.float32)
        for b, lw in enumerate(self.w["layers"]):
            normed = rms_norm(h, lw["input_norm"], cfg.rms_eps, sv)
            q, k, v = (apply(lw[n], normed, sv) for n in ("q", "k", "v"))
            if "q_norm" in lw and "k_norm" in lw:   # per_head_norm, engine/mod.rs:854-873,908-911
                q = per_head_norm(q, lw["q_norm"], cfg.head_dim, cfg.rms_eps, sv)
                k = per_head_norm(k, lw["k_norm"], cfg.head_dim, cfg.rms_eps, sv)
            q = rope_rotate(q, cfg.head_dim, pos, cfg.rope_theta)
            k = rope_rotate(k, cfg.head_dim, pos, cfg.rope_theta)
            if self.kv_round:
                k, v = self.kv_round(k), self.kv_round(v)
            self.keys[b].append(k)
            self.vals[b].append(v)
            attn = oracle.gqa_attention_scalar(q, np.stack(self.keys[b]), np.stack(self.vals[b]),
                                               cfg.n_heads, cfg.n_kv_heads, cfg.head_dim)
            h = (self.reduce(apply(lw["o"], attn, sv)) + h).astype(np.float32)
            normed = rms_norm(h, lw["post_norm"], cfg.rms_eps, sv)
            g, u = apply(lw["gate"], normed, sv), apply(lw["up"], normed, sv)
            hidden = (g * u / (np.float32(1.0) + np.exp(-g))).astype(np.float32)
            h = (self.reduce(apply(lw["down"], hidden, sv)) + h).astype(np.float32)
        return rms_norm(h, self.w["final_norm"], cfg.rms_eps, sv)

    def logits(self, hidden):
        return (self.w["lm_head"].astype(np.float32) @ hidden.astype(np.float32)).astype(np.float32)

    def step(self, token):
        hidden = self.transformer(self.w["embedding"][token])
        lg = self.logits(hidden)
        return int(np.argmax(lg)), lg  # np.argmax returns the first maximum, like greedy()


def generate(cfg, weights, prompt_tokens, max_tokens, eos_token_id=None):
    """engine/mod.rs:1377-1500 (decode_start, push_token, decode_step, generate) without the
    text-side stop strings: returns (completion tokens, finish reason)."""
    if len(prompt_tokens) == 0:
        raise ValueError("prompt tokenized to zero tokens")
    s = Session(cfg, weights)
    for tok in prompt_tokens:
        nxt, _ = s.step(int(tok))
    out = []
    while True:
        if eos_token_id is not None and nxt == eos_token_id:
            return out, "stop"
        out.append(nxt)
        if len(out) >= max_tokens:
            return out, "length"
        nxt, _ = s.step(nxt)
