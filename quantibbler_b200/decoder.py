"""A Llama-shaped decoder built from the factorized-linear and attention kernels.

Mirrors the control flow of the reference's ``ModelWeights::transformer`` /
``Engine::decode_step`` (crates/quantibbler-server/src/engine/mod.rs:878-945,
:1461-1476) for batched single-token decode with device-resident state: per block
RMSNorm -> q,k,v -> RoPE -> KV append -> GQA attention -> o + residual -> RMSNorm ->
gate,up -> SwiGLU -> down + residual; final norm, LM head, greedy (first maximum).

Every operation is one C-ABI call that only launches kernels on the current stream, so a
whole step can be captured in a CUDA graph and replayed.  Under tensor parallelism each
rank holds its shard (``tp.shard_model``) and the two partial sums per block are completed
by ``torch.distributed.all_reduce`` (NCCL) on the output buffers.
"""

from __future__ import annotations

import ctypes
from dataclasses import dataclass

import numpy as np

from . import _lib, tp
from ._lib import QK_BF16, QK_F32, KernelError, check
from .gpu import (DecodeStep, GpuContext, LayerPlan, PackedLayer, apply_prefill_many,
                  apply_prefill_many_gated, make_feed)

LINEARS = ("q", "k", "v", "o", "gate", "up", "down")


@dataclass
class DecoderConfig:
    n_layers: int
    d_model: int
    n_heads: int
    n_kv_heads: int
    head_dim: int
    d_ff: int
    vocab: int
    rms_eps: float = 1e-5
    rope_theta: float = 10000.0
    serving: str = "float32"       # ServingDtype of the linears and norms
    kv_dtype: str = "bfloat16"     # storage of the KV cache
    max_seq: int = 4096
    max_batch: int = 1
    n_splits: int = 0              # key splits of the decode attention (0 = choose)
    # bfloat16 serving: batches this large take the tensor-core GEMM (measured per step on the
    # Llama-3-8B shape, GEMM against the per-token GEMV forms: batch 5 5.69 / 4.95 ms, 6 5.86 /
    # 5.81, 7 6.03 / 6.49, 8 5.38 / 6.14, 10 5.69 / 6.74, 12 5.73 / 7.47, 15 6.08 / 11.98)
    gemm_min_batch: int = 7
    fused_allreduce: bool = True   # tensor parallel: the all-reduce happens inside the norm, over peer memory
    fused_allreduce_max_bytes: int = 1 << 20   # ... while a rank pushes at most this much per all-reduce
    # Batches up to this size build the digit tables of the linears' inputs where each vector is
    # produced (fed plans) and read gate/up through the SwiGLU inside the down projection.  Both
    # measured slower than the plain sequence on the Llama-3-8B shape at batch 1 (5.4 against
    # 4.8 ms per step), so the default is off.
    feed_max_batch: int = 0
    # Batches up to this size run all transformer blocks of a step as ONE cooperative kernel
    # (gpu.DecodeStep: a grid barrier between phases instead of a kernel boundary; the same
    # bits as the separate launches).  Measured slower than the launches on the Llama-3-8B shape
    # (5.1 against 4.4 ms per step), so the default is off.  Needs head_dim 128, a bfloat16
    # cache, no q/k norms, one GPU and a model narrow enough for its shared memory; other
    # configurations keep the separate launches.
    fused_step_max_batch: int = 0
    # RoPE, cache append, attention and combine of a step in one launch instead of three
    # (bfloat16 cache, head_dim 128; the same bits).  Pays at small batches, where the step is a
    # chain of short launches (batch 1: 4.43 -> 4.36 ms); at batch 64 the combine by the last
    # split of each head group costs more than the two launches it saves (10.96 -> 11.40 ms).
    fused_attention: bool = True
    fused_attention_max_batch: int = 8
    # Batches up to this size let the down projection read gate and up through the SwiGLU itself
    # (the activation is evaluated where the projection's digit table is built) instead of a
    # SwiGLU launch of its own: one kernel boundary less per block, the same bits (measured up
    # to batch 12, where it still pays: 8.04 -> 7.88 ms per step; from batch 16 on bfloat16
    # serving takes the GEMM path, which has its own activation pass).
    gated_down_max_batch: int = 15
    # Batches up to this size (one GPU) let q,k,v and gate,up apply the RMSNorm in front of them
    # themselves (every block of the first stage forms the norm of the 4096-entry stream, which
    # costs it about a microsecond) instead of a norm launch of its own, which costs the step
    # about ten: two kernel boundaries less per block, the same bits.
    # (measured per step, norm inside against a norm launch: batch 5 4.61 / 4.94 ms, batch 6
    # 5.47 / 5.74; from batch 7 the tensor-core GEMM takes over.)  Under tensor parallelism,
    # where these plans also carry the all-reduce, the limit is norm_fused_max_batch_tp.
    norm_fused_max_batch: int = 6
    norm_fused_max_batch_tp: int = 4
    prefill_min_tokens: int = 16   # generate(): prompts this long go through the trunk in one pass
    prefill_chunk: int = 2048      # ... in pieces of at most this many positions


def rope_table(cfg: DecoderConfig) -> np.ndarray:
    """cos/sin per (position, i) as the reference forms them: the angle in float64, the
    results cast to float32 (engine/mod.rs:1169-1184)."""
    half = cfg.head_dim // 2
    inv_freq = cfg.rope_theta ** (-(2.0 * np.arange(half, dtype=np.float64)) / cfg.head_dim)
    ang = np.arange(cfg.max_seq, dtype=np.float64)[:, None] * inv_freq[None, :]
    return np.stack([np.cos(ang), np.sin(ang)], axis=-1).astype(np.float32)


def random_layer(rng, dout, din, r, with_bias=False) -> dict:
    """Synthetic factorized linear as the benchmark's configurations prescribe: Bernoulli(0.5)
    factors, scales |N(0,1)|*0.02 + 1e-3."""
    ub = rng.integers(0, 256, size=(dout, (r + 7) // 8), dtype=np.uint8)
    vbt = rng.integers(0, 256, size=(r, (din + 7) // 8), dtype=np.uint8)
    if r % 8:
        ub[:, -1] &= (1 << (r % 8)) - 1
    if din % 8:
        vbt[:, -1] &= (1 << (din % 8)) - 1
    return dict(ub_rows=ub, vb_t_rows=vbt, dout=dout, din=din, r=r,
                s1=(np.abs(rng.standard_normal(dout)) * 0.02 + 1e-3).astype(np.float32),
                s2=(np.abs(rng.standard_normal(din)) * 0.02 + 1e-3).astype(np.float32),
                bias=(rng.standard_normal(dout) * 0.01).astype(np.float32) if with_bias else None)


def random_model(cfg: DecoderConfig, ranks: dict, seed: int = 0, device_tables: bool = False) -> dict:
    """Random-init weights of the configured architecture (no checkpoint is involved).
    With ``device_tables`` the embedding and LM head are drawn on the GPU (bfloat16
    N(0, 0.02)), which is what a 128k-entry vocabulary needs to stay quick."""
    rng = np.random.default_rng(seed)
    d, hd = cfg.d_model, cfg.head_dim
    shapes = {"q": (cfg.n_heads * hd, d), "k": (cfg.n_kv_heads * hd, d),
              "v": (cfg.n_kv_heads * hd, d), "o": (d, cfg.n_heads * hd),
              "gate": (cfg.d_ff, d), "up": (cfg.d_ff, d), "down": (d, cfg.d_ff)}
    layers = []
    for _ in range(cfg.n_layers):
        lw = {name: random_layer(rng, shapes[name][0], shapes[name][1], ranks[name])
              for name in LINEARS}
        lw["input_norm"] = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32)
        lw["post_norm"] = (1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32)
        layers.append(lw)

    def bf16_valued(a):
        u = a.astype(np.float32).view(np.uint32).astype(np.uint64)
        u = ((u + 0x7FFF + ((u >> 16) & 1)) >> 16) << 16
        return u.astype(np.uint32).view(np.float32)

    if device_tables:
        import torch
        gen = torch.Generator(device="cuda").manual_seed(seed)
        emb = (torch.randn(cfg.vocab, d, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
        head = (torch.randn(cfg.vocab, d, device="cuda", generator=gen) * 0.02).to(torch.bfloat16)
    else:
        emb = bf16_valued(rng.standard_normal((cfg.vocab, d)) * 0.02)
        head = bf16_valued(rng.standard_normal((cfg.vocab, d)) * 0.02)
    return dict(layers=layers,
                final_norm=(1.0 + 0.1 * rng.standard_normal(d)).astype(np.float32),
                embedding=emb, lm_head=head, vocab_offset=0)


def check_cache_capacity(positions, n_steps: int, max_seq: int) -> None:
    """Refuse work that would run past the KV cache: a token at position p needs row p of a
    cache of ``max_seq`` rows, and ``n_steps`` further steps reach position p + n_steps - 1.
    The reference's cache grows on demand (engine/mod.rs:1189-1209); this one is a fixed
    allocation, so the host refuses instead (the device skips and reports such a token too)."""
    pos = [int(p) for p in positions]
    if not pos:
        return
    if min(pos) < 0:
        raise ValueError(f"negative position {min(pos)}")
    last = max(pos) + max(int(n_steps), 1) - 1
    if last >= int(max_seq):
        raise ValueError(f"position {last} does not fit the KV cache of {max_seq} positions "
                         f"(start {max(pos)}, {n_steps} steps)")


def _p(t) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


class Decoder:
    """Batched greedy decode on one GPU (one tensor-parallel rank)."""

    def __init__(self, ctx: GpuContext, cfg: DecoderConfig, weights: dict | None, tp_rank: int = 0,
                 tp_size: int = 1, group=None, share_from: "Decoder | None" = None):
        """``share_from``: another decoder of the same model and tensor-parallel rank (it may
        differ in ``max_batch`` and ``max_seq``) whose device-resident weights this one uses
        instead of uploading its own; ``weights`` may then be None."""
        import torch
        self.torch, self.ctx, self.cfg = torch, ctx, cfg
        self.tp_rank, self.tp_size, self.group = tp_rank, tp_size, group
        if share_from is not None:
            w = {"layers": [dict() for _ in range(cfg.n_layers)],
                 "vocab_offset": share_from.vocab_offset}
        else:
            w = tp.shard_model(weights, cfg, tp_rank, tp_size)
        self.vocab_offset = int(w.get("vocab_offset", 0))
        dev = torch.device("cuda", torch.cuda.current_device())
        ctx.set_stream(torch.cuda.current_stream().cuda_stream)  # order with torch's own work
        B, d, hd = cfg.max_batch, cfg.d_model, cfg.head_dim
        self.h_loc, self.kv_loc = cfg.n_heads // tp_size, cfg.n_kv_heads // tp_size
        self.ff_loc, self.v_loc = cfg.d_ff // tp_size, cfg.vocab // tp_size
        self.serving_tag = QK_F32 if cfg.serving == "float32" else QK_BF16
        self.kv_tag = QK_F32 if cfg.kv_dtype == "float32" else QK_BF16
        f32 = dict(dtype=torch.float32, device=dev)
        i32 = dict(dtype=torch.int32, device=dev)

        def dev_f32(a):
            if isinstance(a, torch.Tensor):
                return a.to(dev, torch.float32).contiguous()
            return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dev)

        def dev_bf16(a):
            if isinstance(a, torch.Tensor):
                return a.to(dev, torch.bfloat16).contiguous()
            return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(dev).to(
                torch.bfloat16)

        # activations (static: the step is captured in a CUDA graph)
        self.x = torch.zeros(B, d, **f32)
        self.x2 = torch.zeros(B, d, **f32)   # the residual stream alternates between x and x2
        self.h = torch.zeros(B, d, **f32)
        self.q = torch.zeros(B, self.h_loc * hd, **f32)
        self.k = torch.zeros(B, self.kv_loc * hd, **f32)
        self.v = torch.zeros(B, self.kv_loc * hd, **f32)
        self.attn = torch.zeros(B, self.h_loc * hd, **f32)
        # per-head q/k norms (one head_dim vector each, engine/mod.rs:854-873) write here; the
        # RoPE and the attention then read these instead of the projections' outputs
        self.has_qk_norm = (share_from.has_qk_norm if share_from is not None else
                            any("q_norm" in lw and "k_norm" in lw for lw in w["layers"]))
        self.qn = torch.zeros(B, self.h_loc * hd, **f32) if self.has_qk_norm else self.q
        self.kn = torch.zeros(B, self.kv_loc * hd, **f32) if self.has_qk_norm else self.k
        # o / down outputs (one partial per rank under TP).  With the fused all-reduce the two
        # are separate buffers in symmetric memory that every peer can read.
        self.delta = torch.zeros(B, d, **f32)
        self.delta_attn = self.delta_mlp = self.delta
        self.fused_ar = False
        self.allreduce_in_plans = False   # (the row-parallel sums happen inside the GEMV plans)
        # The fused form is a one-shot push: every rank stores its whole partial to every peer.
        # That wins while the pushed bytes are few (measured: batch 1 at 2 and 8 ranks, batch 64
        # at 2 ranks) and loses to NCCL's bandwidth-optimal schedule when they are many (batch
        # 64 at 8 ranks: 7 MB per rank and all-reduce, 9.1 against 8.7 ms per step).
        if tp_size > 1 and cfg.fused_allreduce and B * d * 4 * (tp_size - 1) <= cfg.fused_allreduce_max_bytes:
            self._setup_fused_allreduce(B, d)
        self.g = torch.zeros(B, self.ff_loc, **f32)
        self.u = torch.zeros(B, self.ff_loc, **f32)
        self.a = torch.zeros(B, self.ff_loc, **f32)
        self.logits = torch.zeros(B, self.v_loc, **f32)
        self.best_val = torch.zeros(B, **f32)
        self.best_idx = torch.zeros(B, **i32)
        self.token_ids = torch.zeros(B, **i32)
        self.positions = torch.zeros(B, **i32)
        self.kv_len = torch.ones(B, **i32)
        self.seq_index = torch.arange(B, **i32)
        kv_t = torch.float32 if cfg.kv_dtype == "float32" else torch.bfloat16
        self.cache_k = [torch.zeros(B, self.kv_loc, cfg.max_seq, hd, dtype=kv_t, device=dev)
                        for _ in range(cfg.n_layers)]
        self.cache_v = [torch.zeros(B, self.kv_loc, cfg.max_seq, hd, dtype=kv_t, device=dev)
                        for _ in range(cfg.n_layers)]
        # Key splits: about 256 blocks of 128 threads per launch (two per SM is what stays
        # resident) in chunks of at least ~64 keys.  Measured per step on the Llama-3-8B
        # shape at 2048 keys, by batch (best split count: ms against the former "eight blocks
        # per SM" rule): 4 (8: 4.18 against 4.64 at 32), 8 (4: 6.13 against 6.56 at 19), 12
        # (4: 7.57 against 7.78 at 13), 16 (2: 5.95 against 6.25 at 10), 32 (2: 7.14 against
        # 7.32 at 5), 64 (3: 9.75, 2: 9.81); more splits mean more partial results for the
        # combine and more blocks that each stage a query tile for few keys.
        # (a step of one or two sequences is a chain of latencies, not a stream: sixteen splits
        # leave the last block of a head group half as many partial results to combine as
        # thirty-two, measured 3.85 against 3.95 ms per step)
        per_split = max(1, B * self.kv_loc)
        want = -(-256 // per_split)
        if per_split >= 512:
            want = 3
        elif per_split >= 128:
            want = max(2, want)
        most = 16 if per_split <= 16 else 32
        self.n_splits = cfg.n_splits or max(1, min(most, want, max(1, cfg.max_seq // 64)))
        # (the one-launch form is the tensor-core attention; a context switched to the scalar
        # kernel keeps the separate launches)
        self.fused_attention = (cfg.fused_attention and B <= cfg.fused_attention_max_batch
                                and cfg.kv_dtype == "bfloat16" and hd == 128
                                and ctx.set_decode_attention_kernel(-1) != 0)
        scratch = max(_lib.lib().qk_decode_attention_scratch(B, self.h_loc, hd, self.n_splits),
                      _lib.lib().qk_decode_attention_rope_scratch(B, self.h_loc, self.kv_loc, hd, self.n_splits))
        self.att_scratch = torch.zeros(scratch // 4 + 4, **f32)
        self.cos_sin = dev_f32(rope_table(cfg))
        self.emb_tag = QK_BF16 if cfg.serving == "bfloat16" else QK_F32
        if share_from is not None:
            o = share_from
            if (o.cfg.serving, o.tp_rank, o.tp_size, o.cfg.n_layers) != (cfg.serving, tp_rank,
                                                                         tp_size, cfg.n_layers):
                raise ValueError("decoders that share weights must agree in serving dtype, "
                                 "tensor-parallel rank and size, and layer count")
            self.embedding, self.lm_head, self.final_norm = o.embedding, o.lm_head, o.final_norm
        else:
            self.embedding = dev_bf16(w["embedding"]) if cfg.serving == "bfloat16" else dev_f32(
                w["embedding"])
            # the LM head is stored in bfloat16 (benchmark configuration 4) unless serving is float32
            self.lm_head = dev_bf16(w["lm_head"]) if cfg.serving == "bfloat16" else dev_f32(
                w["lm_head"])
            self.final_norm = dev_f32(w["final_norm"])
        self.norms, self.layers, self.plans, self.qk_norms = [], [], [], []
        for li, lw in enumerate(w["layers"]):
            if share_from is not None:
                self.norms.append(share_from.norms[li])
                self.qk_norms.append(share_from.qk_norms[li])
                L = share_from.layers[li]
            else:
                self.norms.append((dev_f32(lw["input_norm"]), dev_f32(lw["post_norm"])))
                if "q_norm" in lw and "k_norm" in lw:
                    self.qk_norms.append((dev_f32(lw["q_norm"]), dev_f32(lw["k_norm"])))
                elif self.has_qk_norm:
                    raise ValueError("q/k norms must be present in every block or in none")
                else:
                    self.qk_norms.append(None)
                L = {n: self._upload(ctx, lw[n], n) for n in LINEARS}
            self.layers.append(L)

            def rows(t, b):
                return t[b].data_ptr()

            def inst(names, src, dsts):
                return [(L[n], rows(src, b), rows(dst, b)) for b in range(B)
                        for n, dst in zip(names, dsts)]

            fed = cfg.serving in ("float32", "bfloat16") and B <= cfg.feed_max_batch
            gemm = cfg.serving == "bfloat16" and B >= cfg.gemm_min_batch
            self.gated_down = fed or (cfg.serving in ("float32", "bfloat16") and not gemm
                                      and B <= cfg.gated_down_max_batch)
            plan = {"o": LayerPlan(ctx, inst(["o"], self.attn, [self.delta_attn]))}
            if self.gated_down:   # down reads SwiGLU(gate, up) directly: no separate activation pass
                plan["down"] = LayerPlan(ctx, [(L["down"], rows(self.g, b), rows(self.u, b),
                                                rows(self.delta_mlp, b)) for b in range(B)], gated=True)
            else:
                plan["down"] = LayerPlan(ctx, inst(["down"], self.a, [self.delta_mlp]))
            same_kv = all(getattr(L["k"], f) == getattr(L["v"], f) for f in ("dout", "din", "r"))
            try:
                # q, k and v in one pair of launches although q differs in shape: possible
                # while the plan is small enough for the few-instance kernel form
                plan["qkv"] = LayerPlan(ctx, inst(["q", "k", "v"], self.h, [self.q, self.k, self.v]))
            except KernelError:
                plan["q"] = LayerPlan(ctx, inst(["q"], self.h, [self.q]))
                if same_kv:
                    plan["kv"] = LayerPlan(ctx, inst(["k", "v"], self.h, [self.k, self.v]))
                else:
                    plan["k"] = LayerPlan(ctx, inst(["k"], self.h, [self.k]))
                    plan["v"] = LayerPlan(ctx, inst(["v"], self.h, [self.v]))
            same_gu = all(getattr(L["gate"], f) == getattr(L["up"], f)
                          for f in ("dout", "din", "r"))
            if same_gu:
                plan["gu"] = LayerPlan(ctx, inst(["gate", "up"], self.h, [self.g, self.u]))
            else:
                plan["gate"] = LayerPlan(ctx, inst(["gate"], self.h, [self.g]))
                plan["up"] = LayerPlan(ctx, inst(["up"], self.h, [self.u]))
            # (under tensor parallelism the norms are also where the row-parallel outputs are summed
            # over the ranks: with the all-reduce over peer memory the plans do that themselves)
            if ((B <= cfg.norm_fused_max_batch if tp_size == 1
                 else B <= cfg.norm_fused_max_batch_tp and self.fused_ar and d <= 4096)
                    and not fed and not gemm
                    and cfg.serving in ("float32", "bfloat16") and "qkv" in plan and "gu" in plan):
                # the first norm of a block reads the stream from x and leaves it in x2, the second
                # the other way round; what they add is the output of the linear before them
                def normed(names, src, dsts, residual, weight, x_out):
                    p = LayerPlan(ctx, inst(names, src, dsts))
                    k = len(names)
                    p.set_norm([None if residual is None else rows(residual, b) for b in range(B) for _ in names],
                               weight.data_ptr(), cfg.rms_eps,
                               [rows(x_out, b) if j == 0 else None for b in range(B) for j in range(k)])
                    return p
                try:
                    in_w, post_w = self.norms[li]
                    sharded = tp_size > 1
                    qkv_n = normed(["q", "k", "v"], self.x, [self.q, self.k, self.v],
                                   None if (li == 0 or sharded) else self.delta_mlp, in_w, self.x2)
                    gu_n = normed(["gate", "up"], self.x2, [self.g, self.u], None if sharded else self.delta_attn,
                                  post_w, self.x)
                    if sharded:
                        # o pushes into inbox 0 and gate,up gathers from it; down pushes into inbox 1
                        # and the next block's q,k,v gathers from it (the last block's down output
                        # goes through the all-reduce of the final norm instead)
                        ar = dict(rank=tp_rank, world=tp_size, total_words=B * d, d=d,
                                  state_ptr=self._ar_state.data_ptr())
                        own = lambda which: [int(self._peer_inbox[which][tp_rank])]
                        every = lambda which: [int(a) for a in self._peer_inbox[which]]
                        gu_n.set_allreduce(True, own(0), tokens=[b for b in range(B) for _ in range(2)], **ar)
                        if li > 0:
                            qkv_n.set_allreduce(True, own(1), tokens=[b for b in range(B) for _ in range(3)], **ar)
                        plan["o"].set_allreduce(False, every(0), tokens=list(range(B)), **ar)
                        if li + 1 < cfg.n_layers:
                            plan["down"].set_allreduce(False, every(1), tokens=list(range(B)), **ar)
                        self.allreduce_in_plans = True
                    plan["qkv_normed"], plan["gu_normed"] = qkv_n, gu_n
                except KernelError:
                    if tp_size > 1:
                        raise   # (half-configured plans must not be used)
                    pass   # (a stream too wide for the normed form: the separate norm stays)
            self.plans.append(plan)
        self.step_kernel = None
        if (B <= cfg.fused_step_max_batch and tp_size == 1 and not self.has_qk_norm and hd == 128
                and cfg.kv_dtype == "bfloat16"):
            blocks = [dict(L, input_norm=self.norms[li][0].data_ptr(), post_norm=self.norms[li][1].data_ptr(),
                           cache_k=self.cache_k[li].data_ptr(), cache_v=self.cache_v[li].data_ptr())
                      for li, L in enumerate(self.layers)]
            bufs = dict(x=self.x, x2=self.x2, q=self.q, k=self.k, v=self.v, attn=self.attn,
                        delta_attn=self.delta_attn, delta_mlp=self.delta_mlp, gate=self.g, up=self.u,
                        att_scratch=self.att_scratch, cos_sin=self.cos_sin, positions=self.positions,
                        seq_index=self.seq_index, kv_len=self.kv_len)
            try:
                self.step_kernel = DecodeStep(
                    ctx, blocks, {n: t.data_ptr() for n, t in bufs.items()}, self.serving_tag, self.kv_tag,
                    cfg.rms_eps, n_tokens=B, d_model=d, n_heads=self.h_loc, n_kv_heads=self.kv_loc,
                    head_dim=hd, d_ff=self.ff_loc, s_max=cfg.max_seq, n_seq=B, n_splits=self.n_splits)
            except KernelError:
                self.step_kernel = None   # e.g. a model too wide for the kernel's shared memory
        # a large enough batch is a real contraction: the tcgen05 GEMM expands each weight bit
        # once for all tokens, the GEMV forms would do it once per token
        self.use_gemm = cfg.serving == "bfloat16" and B >= cfg.gemm_min_batch
        # A small batch is bound by what every GEMV block does before it can multiply (scan the
        # input, build its digit table).  Fed plans move that to the kernel that produces the
        # vector, once per vector: the norm feeds q,k,v and gate,up, the attention combine feeds
        # o, the SwiGLU feeds down.
        self.fed = (not self.use_gemm) and B <= cfg.feed_max_batch
        self.feeds = []
        if self.fed:
            for plan in self.plans:
                def group(keys):
                    pairs = []
                    for key, per_token in keys:
                        if key in plan:
                            pairs.append((plan[key], per_token))
                    return make_feed(pairs)
                self.feeds.append({
                    "qkv": group([("qkv", 3), ("q", 1), ("kv", 2), ("k", 1), ("v", 1)]),
                    "o": group([("o", 1)]),
                    "gu": group([("gu", 2), ("gate", 1), ("up", 1)]),
                    "down": group([("down", 1)])})
        self.graph = None
        self.kernels_per_step = None
        self._host_positions = [0] * B

    # ------------------------------------------------------------------ tensor parallel
    def _upload(self, ctx, layer: dict, name: str) -> PackedLayer:
        """One linear onto the device: from its container streams where the dict still holds
        them (a whole layer of a model directory; the device separates the rows), else from
        row bitplanes (synthetic weights, tensor-parallel shards)."""
        if "ub_packed" in layer and "ub_rows" not in layer:
            return PackedLayer.from_container(ctx, layer["ub_packed"], layer["vb_packed"],
                                              layer["dout"], layer["din"], layer["r"],
                                              layer["s1"], layer["s2"], layer.get("bias"),
                                              serving=self.cfg.serving, name=name)
        return PackedLayer(ctx, layer["ub_rows"], layer["vb_t_rows"], layer["dout"], layer["din"],
                           layer["r"], layer["s1"], layer["s2"], layer.get("bias"),
                           serving=self.cfg.serving, name=name)

    def _setup_fused_allreduce(self, B: int, d: int) -> None:
        """Two inboxes in symmetric memory (every rank maps every peer's copy) for
        ``qk_allreduce_rmsnorm``.  If the peers cannot be mapped the decoder keeps the NCCL
        all-reduce and says so in ``fused_ar``."""
        torch = self.torch
        try:
            import torch.distributed._symmetric_memory as symm
            dev = torch.device("cuda", torch.cuda.current_device())
            # [inbox][source rank][token][channel][value, tag]
            self._sym_inbox = symm.empty((2, self.tp_size, B, d, 2), dtype=torch.int32, device=dev)
            self._sym_inbox.zero_()
            handle = symm.rendezvous(self._sym_inbox, self.group)
            bases = list(handle.buffer_ptrs)
        except Exception as exc:  # no peer access on this box: NCCL stays
            self.fused_ar_error = repr(exc)
            return
        torch.cuda.synchronize()
        torch.distributed.barrier(group=self.group)   # every inbox is zero before anyone sends
        inbox_bytes = self.tp_size * B * d * 8
        self._peer_inbox = [np.array([b + which * inbox_bytes for b in bases], dtype=np.uint64)
                            for which in (0, 1)]
        self._ar_state = torch.zeros(2, dtype=torch.int32, device=dev)
        self.delta_attn = torch.zeros(B, d, dtype=torch.float32, device=dev)
        self.delta_mlp = torch.zeros(B, d, dtype=torch.float32, device=dev)
        self.fused_ar = True

    def _all_reduce(self, t):
        if self.tp_size > 1 and not self.fused_ar:
            self.torch.distributed.all_reduce(t, group=self.group)

    def _norm(self, pending, weight, feed=None, x_in=None, x_out=None) -> None:
        """x_out = x_in + pending partial outputs (summed over the ranks); h = RMSNorm(x_out) *
        weight.  ``pending``: None, 0 (attention block's o output) or 1 (MLP block's down output).
        ``feed``: the fed plans that read h (their digit tables are written here; with x_out
        another buffer than x_in several blocks per token share that work)."""
        lib, c, cfg = _lib.lib(), self.ctx.handle, self.cfg
        B, d = cfg.max_batch, cfg.d_model
        x_in = self.x if x_in is None else x_in
        x_out = x_in if x_out is None else x_out
        fp = ctypes.byref(feed) if feed is not None else None
        if pending is not None and self.fused_ar:
            partial = self.delta_attn if pending == 0 else self.delta_mlp
            check(lib.qk_allreduce_rmsnorm_feed(
                c, _p(partial), self._peer_inbox[pending].ctypes.data, _p(self._ar_state),
                self.tp_rank, self.tp_size, _p(x_in), _p(weight), B, d, cfg.rms_eps,
                self.serving_tag, _p(x_out), _p(self.h), fp))
            return
        residual = None if pending is None else _p(self.delta_attn if pending == 0 else self.delta_mlp)
        check(lib.qk_rmsnorm_feed(c, _p(x_in), residual, _p(weight), B, d, cfg.rms_eps,
                                  self.serving_tag, _p(x_out), _p(self.h), fp))

    # ------------------------------------------------------------------ one step

    def _linears(self, li: int, names, src, dsts) -> None:
        """The named linears of layer ``li`` from ``src`` into ``dsts`` for the whole batch."""
        B = self.cfg.max_batch
        if self.use_gemm:
            apply_prefill_many([self.layers[li][n] for n in names], src.data_ptr(), B,
                               [dst.data_ptr() for dst in dsts])
            return
        plan = self.plans[li]
        joint = {("q", "k", "v"): "qkv", ("k", "v"): "kv", ("gate", "up"): "gu"}.get(tuple(names))
        if joint in plan:
            plan[joint].apply()
        elif tuple(names) == ("q", "k", "v"):
            self._linears(li, ["q"], src, dsts[:1])
            self._linears(li, ["k", "v"], src, dsts[1:])
        else:
            for name in names:
                plan[name].apply()

    def step(self) -> None:
        """One decode step for the whole batch: reads ``token_ids``/``positions``/``kv_len``,
        appends to the KV cache, leaves the greedy tokens in ``best_idx``."""
        lib, c, cfg, h = _lib.lib(), self.ctx.handle, self.cfg, self.ctx
        B, d, hd = cfg.max_batch, cfg.d_model, cfg.head_dim
        check(lib.qk_embed(c, _p(self.embedding), self.emb_tag, _p(self.token_ids), B, d, cfg.vocab,
                           _p(self.x)))
        pending = None
        xa, xb = self.x, self.x2   # every norm reads the residual stream from xa and writes it to xb
        if self.step_kernel is not None:
            # all blocks in one kernel; it leaves the stream in x and the last down output in delta_mlp
            self.step_kernel.run()
            pending = 1
        for li in range(cfg.n_layers if self.step_kernel is None else 0):
            in_w, post_w = self.norms[li]
            feeds = self.feeds[li] if self.fed else None
            normed = (not self.use_gemm) and "qkv_normed" in self.plans[li]
            if normed:   # (norm and q,k,v in one pair of launches)
                self.plans[li]["qkv_normed"].apply()
            else:
                self._norm(pending, in_w, feeds["qkv"] if feeds else None, xa, xb)
                self._linears(li, ["q", "k", "v"], self.h, [self.q, self.k, self.v])
            xa, xb = xb, xa
            if self.qk_norms[li] is not None:
                # every head is one row of head_dim values; x_out = x rewrites the projection
                # unchanged (the kernel's usual in-place form)
                for src, dst, wgt, heads in ((self.q, self.qn, self.qk_norms[li][0], self.h_loc),
                                             (self.k, self.kn, self.qk_norms[li][1], self.kv_loc)):
                    check(lib.qk_rmsnorm(c, _p(src), None, _p(wgt), B * heads, hd, cfg.rms_eps,
                                         self.serving_tag, _p(src), _p(dst)))
            if self.fused_attention and not feeds:
                # RoPE, cache append, attention and combine in one launch
                check(lib.qk_decode_attention_rope(
                    c, _p(self.qn), _p(self.kn), _p(self.v), _p(self.cos_sin), _p(self.positions),
                    _p(self.seq_index), _p(self.cache_k[li]), _p(self.cache_v[li]), self.kv_tag,
                    _p(self.kv_len), B, self.h_loc, self.kv_loc, hd, cfg.max_seq, B, self.n_splits,
                    _p(self.att_scratch), _p(self.attn)))
            else:
                check(lib.qk_rope_cache(c, _p(self.qn), _p(self.kn), _p(self.v), _p(self.cos_sin),
                                        _p(self.positions), _p(self.seq_index), _p(self.cache_k[li]),
                                        _p(self.cache_v[li]), self.kv_tag, B, self.h_loc, self.kv_loc,
                                        hd, cfg.max_seq, B))
                check(lib.qk_decode_attention_feed(
                    c, _p(self.qn), _p(self.cache_k[li]), _p(self.cache_v[li]), self.kv_tag,
                    _p(self.kv_len), B, self.h_loc, self.kv_loc, hd, cfg.max_seq, self.n_splits,
                    _p(self.att_scratch), _p(self.attn), self.serving_tag,
                    ctypes.byref(feeds["o"]) if feeds else None))
            self._linears(li, ["o"], self.attn, [self.delta_attn])
            self._all_reduce(self.delta_attn)
            if normed:
                self.plans[li]["gu_normed"].apply()
            else:
                self._norm(0, post_w, feeds["gu"] if feeds else None, xa, xb)
                self._linears(li, ["gate", "up"], self.h, [self.g, self.u])
            xa, xb = xb, xa
            if feeds:   # (the fed down plan needs no activation vector, only its digit table)
                check(lib.qk_swiglu_feed(c, _p(self.g), _p(self.u), B, self.ff_loc, self.serving_tag,
                                         ctypes.byref(feeds["down"])))
            elif not self.gated_down and not self.use_gemm:
                check(lib.qk_swiglu(c, _p(self.g), _p(self.u), B * self.ff_loc, _p(self.a)))
            if self.use_gemm:   # (the SwiGLU inside the GEMM's scaling kernel)
                apply_prefill_many_gated([self.layers[li]["down"]], self.g.data_ptr(), self.u.data_ptr(), B,
                                         [self.delta_mlp.data_ptr()])
            else:
                self._linears(li, ["down"], self.a, [self.delta_mlp])
            self._all_reduce(self.delta_mlp)
            pending = 1
        self._norm(pending, self.final_norm, None, xa, xb)
        head_tag = QK_BF16 if cfg.serving == "bfloat16" else QK_F32
        check(lib.qk_lm_head(c, _p(self.h), _p(self.lm_head), head_tag, B, self.v_loc, d,
                             self.v_loc, _p(self.logits)))
        check(lib.qk_argmax_first(c, _p(self.logits), B, self.v_loc, self.v_loc, self.vocab_offset,
                                  _p(self.best_val), _p(self.best_idx)))
        if self.tp_size > 1:
            self._gather_argmax(self.best_val, self.best_idx)

    # ------------------------------------------------------------------ batched prefill
    def _prefill_buffers(self, n_tokens: int) -> dict:
        """Activation buffers for ``n_tokens`` positions at once (kept and reused)."""
        torch, cfg = self.torch, self.cfg
        have = getattr(self, "_pf", None)
        if have is not None and have["cap"] >= n_tokens:
            return have
        dev = self.x.device
        f32 = dict(dtype=torch.float32, device=dev)
        hd, d = cfg.head_dim, cfg.d_model
        T = n_tokens
        pf = dict(cap=T, x=torch.zeros(T, d, **f32), h=torch.zeros(T, d, **f32),
                  q=torch.zeros(T, self.h_loc * hd, **f32), k=torch.zeros(T, self.kv_loc * hd, **f32),
                  v=torch.zeros(T, self.kv_loc * hd, **f32), attn=torch.zeros(T, self.h_loc * hd, **f32),
                  delta=torch.zeros(T, d, **f32), g=torch.zeros(T, self.ff_loc, **f32),
                  u=torch.zeros(T, self.ff_loc, **f32), a=torch.zeros(T, self.ff_loc, **f32),
                  ids=torch.zeros(T, dtype=torch.int32, device=dev),
                  pos=torch.zeros(T, dtype=torch.int32, device=dev),
                  seq=torch.zeros(T, dtype=torch.int32, device=dev))
        if self.has_qk_norm:
            pf["qn"], pf["kn"] = torch.zeros_like(pf["q"]), torch.zeros_like(pf["k"])
        else:
            pf["qn"], pf["kn"] = pf["q"], pf["k"]
        self._pf = pf
        return pf

    def _prefill_linears(self, li: int, names, src, dsts, n_tokens: int) -> None:
        """The named linears of layer ``li`` on ``n_tokens`` rows of ``src``: the tensor-core GEMM
        for bfloat16 serving (every weight bit expanded once for all rows), otherwise one GEMV
        instance per row (many rows run in the persistent streaming form)."""
        layers = [self.layers[li][n] for n in names]
        if self.cfg.serving == "bfloat16" and n_tokens >= self.cfg.gemm_min_batch:
            apply_prefill_many(layers, src.data_ptr(), n_tokens, [t.data_ptr() for t in dsts])
        else:
            for layer, dst in zip(layers, dsts):
                layer.apply_device(src.data_ptr(), n_tokens, dst.data_ptr())

    def prefill(self, tokens, seq: int = 0, first_position: int = 0) -> None:
        """All of ``tokens`` (consecutive positions ``first_position ...`` of sequence slot ``seq``)
        through the trunk in one pass per ``prefill_chunk`` positions: the batched form of the
        reference's prompt loop (engine/mod.rs:1393-1413, one ``transformer`` call per prompt
        token).  Appends the keys and values of every position to the cache and leaves the
        greedy token of the last position in ``best_idx[seq]``; ``advance()`` + ``step()`` then
        continue the sequence.  Only the last position goes through the final norm and the head."""
        torch, lib, c, cfg = self.torch, _lib.lib(), self.ctx.handle, self.cfg
        toks = [int(t) for t in tokens]
        if not toks:
            raise ValueError("prefill needs at least one token")
        if not 0 <= seq < cfg.max_batch:
            raise ValueError(f"sequence slot {seq} outside the batch of {cfg.max_batch}")
        check_cache_capacity([first_position], len(toks), cfg.max_seq)
        B, d, hd = cfg.max_batch, cfg.d_model, cfg.head_dim
        handle = self.ctx.stream
        # (handles 0 and 1 are the legacy default stream, which torch wraps itself)
        stream = torch.cuda.ExternalStream(handle) if handle > 2 else torch.cuda.default_stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for c0 in range(0, len(toks), cfg.prefill_chunk):
                part = toks[c0:c0 + cfg.prefill_chunk]
                T, p0 = len(part), first_position + c0
                pf = self._prefill_buffers(min(len(toks), cfg.prefill_chunk))
                pf["ids"][:T].copy_(torch.tensor(part, dtype=torch.int32), non_blocking=False)
                pf["pos"][:T].copy_(torch.arange(p0, p0 + T, dtype=torch.int32))
                pf["seq"][:T].fill_(seq)
                check(lib.qk_embed(c, _p(self.embedding), self.emb_tag, _p(pf["ids"]), T, d, cfg.vocab,
                                   _p(pf["x"])))
                pending = None
                for li in range(cfg.n_layers):
                    in_w, post_w = self.norms[li]
                    check(lib.qk_rmsnorm(c, _p(pf["x"]), pending, _p(in_w), T, d, cfg.rms_eps,
                                         self.serving_tag, _p(pf["x"]), _p(pf["h"])))
                    self._prefill_linears(li, ["q", "k", "v"], pf["h"], [pf["q"], pf["k"], pf["v"]], T)
                    if self.qk_norms[li] is not None:
                        for src, dst, wgt, heads in ((pf["q"], pf["qn"], self.qk_norms[li][0], self.h_loc),
                                                     (pf["k"], pf["kn"], self.qk_norms[li][1], self.kv_loc)):
                            check(lib.qk_rmsnorm(c, _p(src), None, _p(wgt), T * heads, hd, cfg.rms_eps,
                                                 self.serving_tag, _p(src), _p(dst)))
                    check(lib.qk_rope_cache(c, _p(pf["qn"]), _p(pf["kn"]), _p(pf["v"]), _p(self.cos_sin),
                                            _p(pf["pos"]), _p(pf["seq"]), _p(self.cache_k[li]),
                                            _p(self.cache_v[li]), self.kv_tag, T, self.h_loc,
                                            self.kv_loc, hd, cfg.max_seq, B))
                    check(lib.qk_prefill_attention(c, _p(pf["qn"]), _p(self.cache_k[li]),
                                                   _p(self.cache_v[li]), self.kv_tag, seq, p0, T,
                                                   self.h_loc, self.kv_loc, hd, cfg.max_seq,
                                                   _p(pf["attn"])))
                    self._prefill_linears(li, ["o"], pf["attn"], [pf["delta"]], T)
                    if self.tp_size > 1:
                        torch.distributed.all_reduce(pf["delta"][:T], group=self.group)
                    check(lib.qk_rmsnorm(c, _p(pf["x"]), _p(pf["delta"]), _p(post_w), T, d, cfg.rms_eps,
                                         self.serving_tag, _p(pf["x"]), _p(pf["h"])))
                    self._prefill_linears(li, ["gate", "up"], pf["h"], [pf["g"], pf["u"]], T)
                    if cfg.serving == "bfloat16" and T >= cfg.gemm_min_batch:
                        apply_prefill_many_gated([self.layers[li]["down"]], pf["g"].data_ptr(), pf["u"].data_ptr(),
                                                 T, [pf["delta"].data_ptr()])
                    else:
                        check(lib.qk_swiglu(c, _p(pf["g"]), _p(pf["u"]), T * self.ff_loc, _p(pf["a"])))
                        self._prefill_linears(li, ["down"], pf["a"], [pf["delta"]], T)
                    if self.tp_size > 1:
                        torch.distributed.all_reduce(pf["delta"][:T], group=self.group)
                    pending = _p(pf["delta"])
            # the last position alone: final norm, head, greedy choice
            last_x, last_delta = pf["x"][T - 1:T], pf["delta"][T - 1:T]
            check(lib.qk_rmsnorm(c, _p(last_x), _p(last_delta) if pending is not None else None,
                                 _p(self.final_norm), 1, d, cfg.rms_eps, self.serving_tag, _p(last_x),
                                 _p(self.h[seq:seq + 1])))
            head_tag = QK_BF16 if cfg.serving == "bfloat16" else QK_F32
            check(lib.qk_lm_head(c, _p(self.h[seq:seq + 1]), _p(self.lm_head), head_tag, 1, self.v_loc, d,
                                 self.v_loc, _p(self.logits[seq:seq + 1])))
            check(lib.qk_argmax_first(c, _p(self.logits[seq:seq + 1]), 1, self.v_loc, self.v_loc,
                                      self.vocab_offset, _p(self.best_val[seq:seq + 1]),
                                      _p(self.best_idx[seq:seq + 1])))
            if self.tp_size > 1:
                self._gather_argmax(self.best_val[seq:seq + 1], self.best_idx[seq:seq + 1])
            last = first_position + len(toks) - 1
            self.token_ids[seq:seq + 1].fill_(toks[-1])
            self.positions[seq:seq + 1].fill_(last)
            self.kv_len[seq:seq + 1].fill_(last + 1)
        stream.synchronize()
        torch.cuda.current_stream().wait_stream(stream)
        self._host_positions[seq] = last
        self.ctx.synchronize()

    def _gather_argmax(self, best_val, best_idx) -> None:
        """Vocabulary-parallel head: the first maximum over the ranks' shard winners."""
        torch = self.torch
        vals = [torch.empty_like(best_val) for _ in range(self.tp_size)]
        idxs = [torch.empty_like(best_idx) for _ in range(self.tp_size)]
        torch.distributed.all_gather(vals, best_val, group=self.group)
        torch.distributed.all_gather(idxs, best_idx, group=self.group)
        v = torch.stack(vals)              # [ranks, n]; shards are in vocabulary order,
        win = torch.argmax(v, dim=0)       # and argmax returns the first maximum
        best_idx.copy_(torch.stack(idxs).gather(0, win[None])[0])

    def advance(self) -> None:
        """Feed the greedy tokens back and move every sequence one position on."""
        self.token_ids.copy_(self.best_idx)
        self.positions.add_(1)
        self.kv_len.add_(1)

    def capture(self) -> None:
        """Record step() + advance() into a CUDA graph (after a few eager warm-up steps)."""
        torch = self.torch
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        saved = [t.clone() for t in (self.token_ids, self.positions, self.kv_len)]
        with torch.cuda.stream(stream):
            self.ctx.set_stream(stream.cuda_stream)
            for _ in range(2):
                self.step()
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        n0 = self.ctx.launch_count
        with torch.cuda.graph(graph, stream=stream):  # the context already launches on `stream`
            self.step()
            self.advance()
        self.kernels_per_step = self.ctx.launch_count - n0   # this library's kernels in the graph
        for t, s in zip((self.token_ids, self.positions, self.kv_len), saved):
            t.copy_(s)
        torch.cuda.synchronize()
        self.graph = graph

    def start(self, token_ids, positions) -> None:
        torch = self.torch
        check_cache_capacity(positions, 1, self.cfg.max_seq)
        self._host_positions = [int(p) for p in positions]
        self.token_ids.copy_(torch.as_tensor(token_ids, dtype=torch.int32))
        self.positions.copy_(torch.as_tensor(positions, dtype=torch.int32))
        self.kv_len.copy_(self.positions + 1)

    def decode(self, n_steps: int) -> np.ndarray:
        """Greedy decode; returns the [n_steps, batch] generated ids."""
        check_cache_capacity(self._host_positions, n_steps, self.cfg.max_seq)
        self._host_positions = [p + n_steps for p in self._host_positions]
        out = []
        for _ in range(n_steps):
            if self.graph is not None:
                self.graph.replay()
            else:
                self.step()
                self.advance()
            out.append(self.token_ids.clone())
        self.torch.cuda.synchronize()
        self.ctx.synchronize()   # also reports a device-side wait that gave up or a skipped token
        return self.torch.stack(out).cpu().numpy()

    def generate(self, prompt_tokens, max_tokens: int, eos_token_id: int | None = None) -> dict:
        """Greedy generation for one sequence, with the control flow of the reference's
        ``Engine::decode_start`` / ``push_token`` / ``decode_step`` / ``generate``
        (engine/mod.rs:1377-1500): the prompt goes through the trunk one position at a time
        over the device-resident KV cache, the first token is the argmax at the last prompt
        position, EOS ends the generation without being part of it (finish ``"stop"``), and
        the completion ends at ``max_tokens`` tokens (finish ``"length"``; as in the
        reference the first token is kept even when ``max_tokens`` is 0).  ``prompt_ms`` is the
        prefill span rounded up to a whole millisecond, at least 1.  Stop strings are text-side
        (they need the tokenizer) and stay with the caller.
        """
        import math
        import time
        prompt = [int(t) for t in prompt_tokens]
        if not prompt:
            raise ValueError("prompt tokenized to zero tokens")
        if self.cfg.max_batch != 1:
            raise ValueError("generate serves one sequence: build the decoder with max_batch=1")
        if len(prompt) + max(int(max_tokens), 1) > self.cfg.max_seq:
            raise ValueError(f"prompt of {len(prompt)} tokens plus {max_tokens} new tokens does "
                             f"not fit the KV cache of {self.cfg.max_seq} positions")
        for tok in prompt:
            if not 0 <= tok < self.cfg.vocab:
                raise ValueError(f"token id {tok} out of range (vocab_size {self.cfg.vocab})")
        started = time.perf_counter()
        if len(prompt) >= self.cfg.prefill_min_tokens:
            self.prefill(prompt, seq=0, first_position=0)   # the whole prompt in one pass
        else:
            for pos, tok in enumerate(prompt):
                self.start([tok], [pos])
                self.step()
        self.ctx.synchronize()
        prompt_ms = max(1, math.ceil((time.perf_counter() - started) * 1000.0))
        out, finish = [], None
        while finish is None:
            nxt = int(self.best_idx[0].item())
            if eos_token_id is not None and nxt == int(eos_token_id):
                finish = "stop"
                break
            out.append(nxt)
            if len(out) >= int(max_tokens):
                finish = "length"
                break
            self.advance()
            self.step()
        self.ctx.synchronize()
        return {"prompt_tokens": len(prompt), "completion_tokens": out, "finish": finish,
                "prompt_ms": prompt_ms}
