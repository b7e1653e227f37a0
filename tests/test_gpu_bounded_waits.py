"""Failure paths that end in a status, not in a fault: a device-side wait that runs out,
and a token that does not fit the KV cache.  Neither test makes the GPU fault, trap or hang:
the wait is a bounded poll of ordinary memory that nothing writes, the out-of-range token is
skipped by a bounds check."""

import ctypes

import numpy as np
import pytest

from quantibbler_b200 import _lib
from quantibbler_b200._lib import DeviceError, KernelError

pytestmark = pytest.mark.gpu


def _p(t):
    return ctypes.c_void_p(t.data_ptr())


def test_fused_allreduce_wait_runs_out_and_the_context_stays_usable(gpu_ctx):
    """qk_allreduce_rmsnorm as rank 0 of 2 on ONE GPU: the "peer" inbox is another local buffer
    and nobody ever writes this rank's inbox, so the poll for rank 1's words can only run out.
    With the poll limit set to a few thousand rounds that takes milliseconds; the kernel
    returns, qk_gpu_synchronize reports QK_ERR_TIMEOUT, and the same context then runs an
    ordinary norm correctly."""
    import torch
    lib, c = _lib.lib(), gpu_ctx.handle
    n_tokens, d, world = 3, 256, 2
    rng = np.random.default_rng(0)
    x = torch.from_numpy(rng.standard_normal((n_tokens, d)).astype(np.float32)).cuda()
    partial = torch.from_numpy(rng.standard_normal((n_tokens, d)).astype(np.float32)).cuda()
    w = torch.ones(d, device="cuda")
    x_out = torch.zeros_like(x)
    y = torch.full_like(x, float("nan"))
    inboxes = torch.zeros(world, world, n_tokens, d, 2, dtype=torch.int32, device="cuda")
    state = torch.zeros(2, dtype=torch.int32, device="cuda")
    ptrs = np.array([inboxes[r].data_ptr() for r in range(world)], dtype=np.uint64)
    torch.cuda.synchronize()
    prev = gpu_ctx.set_wait_limit(4000)
    try:
        _lib.check(lib.qk_allreduce_rmsnorm(c, _p(partial), ptrs.ctypes.data, _p(state), 0, world,
                                            _p(x), _p(w), n_tokens, d, 1e-5, _lib.QK_F32,
                                            _p(x_out), _p(y)))
        with pytest.raises(DeviceError, match="inbox of a fused all-reduce"):
            gpu_ctx.synchronize()
    finally:
        gpu_ctx.set_wait_limit(prev)
    # what the kernel did before giving up: it pushed its tagged partial to the peer's inbox,
    # counted the call, and left y unwritten
    torch.cuda.synchronize()
    sent = inboxes[1, 0].cpu().numpy()          # rank 1's inbox, slot of source rank 0
    assert np.array_equal(sent[..., 0].view(np.float32), partial.cpu().numpy())
    assert (sent[..., 1] == 1).all()
    assert int(state[0]) == 1 and int(state[1]) == 0
    assert torch.isnan(y).all()
    # the error word was cleared by the failing synchronize: the context works on
    gpu_ctx.synchronize()
    _lib.check(lib.qk_rmsnorm(c, _p(x), None, _p(w), n_tokens, d, 1e-5, _lib.QK_F32, None, _p(y)))
    gpu_ctx.synchronize()
    xn = x.cpu().numpy().astype(np.float64)
    want = xn / np.sqrt((xn * xn).mean(axis=1, keepdims=True) + 1e-5)
    assert np.abs(y.cpu().numpy() - want).max() <= 1e-5


def test_single_rank_allreduce_is_the_plain_norm(gpu_ctx):
    # world = 1: nothing to wait for; x_out = x + partial, y = norm
    import torch
    lib, c = _lib.lib(), gpu_ctx.handle
    n_tokens, d = 2, 192
    rng = np.random.default_rng(1)
    x = torch.from_numpy(rng.standard_normal((n_tokens, d)).astype(np.float32)).cuda()
    partial = torch.from_numpy(rng.standard_normal((n_tokens, d)).astype(np.float32)).cuda()
    w = torch.from_numpy((1 + 0.1 * rng.standard_normal(d)).astype(np.float32)).cuda()
    x_out, y = torch.zeros_like(x), torch.zeros_like(x)
    inbox = torch.zeros(1, n_tokens, d, 2, dtype=torch.int32, device="cuda")
    state = torch.zeros(2, dtype=torch.int32, device="cuda")
    ptrs = np.array([inbox.data_ptr()], dtype=np.uint64)
    torch.cuda.synchronize()
    for step in (1, 2):
        _lib.check(lib.qk_allreduce_rmsnorm(c, _p(partial), ptrs.ctypes.data, _p(state), 0, 1, _p(x),
                                            _p(w), n_tokens, d, 1e-5, _lib.QK_F32, _p(x_out), _p(y)))
        gpu_ctx.synchronize()
        assert int(state[0]) == step
    h = (x + partial).cpu().numpy().astype(np.float64)
    assert np.array_equal(x_out.cpu().numpy(), (x + partial).cpu().numpy())
    want = h / np.sqrt((h * h).mean(axis=1, keepdims=True) + 1e-5) * w.cpu().numpy()
    assert np.abs(y.cpu().numpy() - want).max() <= 1e-5


def test_token_outside_the_cache_is_skipped_and_reported(gpu_ctx):
    """A position past the cache's last row (a graph replayed too often) must neither write
    into a neighbour's rows nor read past the RoPE table: the token is skipped and the next
    synchronize says so."""
    import torch
    lib, c = _lib.lib(), gpu_ctx.handle
    n_seq, n_heads, n_kv, d, s_max = 2, 2, 1, 16, 8
    rng = np.random.default_rng(2)
    q = torch.from_numpy(rng.standard_normal((n_seq, n_heads * d)).astype(np.float32)).cuda()
    k = torch.from_numpy(rng.standard_normal((n_seq, n_kv * d)).astype(np.float32)).cuda()
    v = torch.from_numpy(rng.standard_normal((n_seq, n_kv * d)).astype(np.float32)).cuda()
    cos_sin = torch.zeros(s_max, d // 2, 2, device="cuda")
    cos_sin[..., 0] = 1.0
    cache_k = torch.zeros(n_seq, n_kv, s_max, d, device="cuda")
    cache_v = torch.zeros_like(cache_k)
    seq_index = torch.arange(n_seq, dtype=torch.int32, device="cuda")

    def run(positions):
        pos = torch.tensor(positions, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        _lib.check(lib.qk_rope_cache(c, _p(q), _p(k), _p(v), _p(cos_sin), _p(pos), _p(seq_index),
                                     _p(cache_k), _p(cache_v), _lib.QK_F32, n_seq, n_heads, n_kv,
                                     d, s_max, n_seq))

    run([s_max - 1, 3])
    gpu_ctx.synchronize()                       # both in range: no complaint
    assert np.array_equal(cache_v[0, 0, s_max - 1].cpu().numpy(), v[0].cpu().numpy())
    before_k, before_v = cache_k.clone(), cache_v.clone()
    run([s_max, 4])                             # sequence 0 is one past the end
    with pytest.raises(KernelError, match="outside the KV cache"):
        gpu_ctx.synchronize()
    torch.cuda.synchronize()
    # sequence 0 wrote nothing (in particular not into sequence 1's first row); sequence 1 did
    assert np.array_equal(cache_k[0].cpu().numpy(), before_k[0].cpu().numpy())
    assert np.array_equal(cache_v[1, 0, 4].cpu().numpy(), v[1].cpu().numpy())
    assert np.array_equal(cache_v[1, 0, 0].cpu().numpy(), before_v[1, 0, 0].cpu().numpy())
    gpu_ctx.synchronize()                       # reported once, then clear


def test_decode_attention_clamps_the_length_to_the_cache(gpu_ctx):
    # kv_len beyond s_max reads the s_max rows that exist, nothing more
    import torch
    lib, c = _lib.lib(), gpu_ctx.handle
    B, H, KV, d, S = 1, 4, 2, 64, 40
    rng = np.random.default_rng(3)
    q = torch.from_numpy(rng.standard_normal((B, H, d)).astype(np.float32)).cuda()
    k = torch.from_numpy(rng.standard_normal((B, KV, S, d)).astype(np.float32)).cuda()
    v = torch.from_numpy(rng.standard_normal((B, KV, S, d)).astype(np.float32)).cuda()
    outs = []
    for length in (S, S + 1000):
        kv_len = torch.tensor([length], dtype=torch.int32, device="cuda")
        out = torch.zeros(B, H, d, device="cuda")
        scratch = torch.zeros(lib.qk_decode_attention_scratch(B, H, d, 2) // 4 + 4, device="cuda")
        torch.cuda.synchronize()
        _lib.check(lib.qk_decode_attention(c, _p(q), _p(k), _p(v), _lib.QK_F32, _p(kv_len), B, H, KV,
                                           d, S, 2, _p(scratch), _p(out)))
        gpu_ctx.synchronize()
        outs.append(out.cpu().numpy())
    assert np.array_equal(outs[0], outs[1])


def test_grid_barrier_of_the_whole_step_kernel_runs_out_and_recovers(gpu_ctx):
    """The whole-step decode kernel separates its phases by a grid barrier whose poll is bounded.
    With the limit set to a single poll, blocks give up at the first barrier they reach before
    the others: the kernel still runs to its end (every block keeps arriving, so the barrier
    count stays whole), the step's results are meaningless, qk_gpu_synchronize reports
    QK_ERR_TIMEOUT - and the same decoder, the same barrier counter, then decodes correctly."""
    from quantibbler_b200.decoder import Decoder, DecoderConfig, random_model
    ranks = {"q": 72, "k": 40, "v": 40, "o": 100, "gate": 130, "up": 130, "down": 90}
    cfg = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=2, head_dim=128, d_ff=640, vocab=192,
               max_seq=64, max_batch=1, kv_dtype="bfloat16", serving="bfloat16", n_splits=2)
    weights = random_model(DecoderConfig(**cfg), ranks, seed=5)
    fused = Decoder(gpu_ctx, DecoderConfig(fused_step_max_batch=1, **cfg), weights)
    plain = Decoder(gpu_ctx, DecoderConfig(**cfg), weights)
    assert fused.step_kernel is not None
    fused.start([7], [0])
    prev = gpu_ctx.set_wait_limit(1)
    try:
        fused.step()
        with pytest.raises(DeviceError, match="grid barrier of the whole-step decode kernel"):
            gpu_ctx.synchronize()
    finally:
        gpu_ctx.set_wait_limit(prev)
    gpu_ctx.synchronize()   # the error word was cleared
    fused.start([7], [0])
    plain.start([7], [0])
    assert np.array_equal(fused.decode(10), plain.decode(10))


def test_allreduce_inside_plans_on_one_gpu_and_its_wait_running_out(gpu_ctx):
    """The all-reduce inside the plans with both "ranks" on ONE GPU, one after the other (no
    kernel waits for another: rank 1's push plan runs to completion before rank 0's gathering
    plan starts): a row-parallel plan pushes its outputs, tagged, into both inboxes; the normed
    plan that follows sums what arrived in rank order as the residual of its norm.  Expected:
    the bits of the all-reduce + norm kernel followed by the plain plan.  Then the same
    gathering plan with nothing pushed for the next all-reduce: its polls run out (limit 4000),
    the launch ends, qk_gpu_synchronize reports QK_ERR_TIMEOUT, the context works on."""
    import torch
    from quantibbler_b200.gpu import LayerPlan, PackedLayer
    from tests.conftest import make_layer
    lib, c = _lib.lib(), gpu_ctx.handle
    d, n_tok, world = 512, 2, 2
    rng = np.random.default_rng(3)
    Lo = [make_layer(d, 384, 40, seed=30 + r) for r in range(world)]      # each rank's row-parallel o
    Lq = make_layer(200, d, 48, seed=40)                                   # what follows the norm
    o = [PackedLayer(gpu_ctx, L["ub_rows"], L["vb_t_rows"], d, 384, 40, L["s1"], L["s2"], None, serving="float32")
         for L in Lo]
    q = PackedLayer(gpu_ctx, Lq["ub_rows"], Lq["vb_t_rows"], 200, d, 48, Lq["s1"], Lq["s2"], None, serving="float32")
    attn = [torch.from_numpy(rng.standard_normal((n_tok, 384)).astype(np.float32)).cuda() for _ in range(world)]
    x = torch.from_numpy(rng.standard_normal((n_tok, d)).astype(np.float32)).cuda()
    w = torch.from_numpy((1 + 0.1 * rng.standard_normal(d)).astype(np.float32)).cuda()
    # reference: partial outputs stored, all-reduce + norm kernel per rank would give x + p0 + p1
    part = [torch.zeros(n_tok, d, device="cuda") for _ in range(world)]
    for r in range(world):
        LayerPlan(gpu_ctx, [(o[r], attn[r][b].data_ptr(), part[r][b].data_ptr()) for b in range(n_tok)]).apply()
    gpu_ctx.synchronize()
    h_ref = x + (torch.zeros_like(x) + part[0] + part[1])   # the kernels' order: 0 + p0 + p1, then x + sum
    hn = torch.zeros_like(x)
    _lib.check(lib.qk_rmsnorm(c, _p(h_ref), None, _p(w), n_tok, d, 1e-5, _lib.QK_F32, None, _p(hn)))
    y_ref = torch.zeros(n_tok, 200, device="cuda")
    LayerPlan(gpu_ctx, [(q, hn[b].data_ptr(), y_ref[b].data_ptr()) for b in range(n_tok)]).apply()
    gpu_ctx.synchronize()
    # the same through the inboxes
    inbox = torch.zeros(world, world, n_tok, d, 2, dtype=torch.int32, device="cuda")   # [owner][source]...
    states = [torch.zeros(2, dtype=torch.int32, device="cuda") for _ in range(world)]
    bases = [inbox[r].data_ptr() for r in range(world)]
    dummy = torch.zeros(n_tok, d, device="cuda")
    push = []
    for r in range(world):
        p = LayerPlan(gpu_ctx, [(o[r], attn[r][b].data_ptr(), dummy[b].data_ptr()) for b in range(n_tok)])
        p.set_allreduce(False, bases, r, world, n_tok * d, list(range(n_tok)), d, states[r].data_ptr())
        push.append(p)
    x_out = torch.zeros_like(x)
    y = torch.full((n_tok, 200), float("nan"), device="cuda")
    gather = LayerPlan(gpu_ctx, [(q, x[b].data_ptr(), y[b].data_ptr()) for b in range(n_tok)])
    gather.set_norm([None] * n_tok, w.data_ptr(), 1e-5, [x_out[b].data_ptr() for b in range(n_tok)])
    gather.set_allreduce(True, [bases[0]], 0, world, n_tok * d, list(range(n_tok)), d, states[0].data_ptr())
    torch.cuda.synchronize()
    for p in push:
        p.apply()
    gpu_ctx.synchronize()
    gather.apply()
    gpu_ctx.synchronize()
    assert torch.equal(x_out, h_ref)
    assert torch.equal(y, y_ref)
    assert int(states[0][0]) == 1 and int(states[0][1]) == 0
    # all-reduce number 2: nobody pushes, so the gathering plan's polls can only run out
    prev = gpu_ctx.set_wait_limit(4000)
    try:
        gather.apply()
        with pytest.raises(DeviceError, match="all-reduce"):
            gpu_ctx.synchronize()
    finally:
        gpu_ctx.set_wait_limit(prev)
    gpu_ctx.synchronize()   # (the error word was cleared by the failing synchronize)
    y2 = torch.zeros(n_tok, 200, device="cuda")
    LayerPlan(gpu_ctx, [(q, hn[b].data_ptr(), y2[b].data_ptr()) for b in range(n_tok)]).apply()
    gpu_ctx.synchronize()
    assert torch.equal(y2, y_ref)
