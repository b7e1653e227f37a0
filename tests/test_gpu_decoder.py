"""GPU parity of the decoder path (norm, RoPE, KV cache, decode attention, SwiGLU, head,
greedy) against the NumPy restatement of the reference's transformer forward."""

import numpy as np
import pytest

import oracle
from oracle import decoder_np
from quantibbler_b200.decoder import Decoder, DecoderConfig, random_model

pytestmark = pytest.mark.gpu

@pytest.fixture(autouse=True)
def _restore_stream(gpu_ctx):
    yield
    gpu_ctx.set_stream(None)


RANKS = {n: 24 for n in ("q", "k", "v", "o", "gate", "up", "down")}


def tiny_cfg(**kw):
    base = dict(n_layers=2, d_model=64, n_heads=4, n_kv_heads=2, head_dim=16, d_ff=128, vocab=128,
                max_seq=32, max_batch=3, kv_dtype="float32", serving="float32")
    base.update(kw)
    return DecoderConfig(**base)


def reference_run(cfg, weights, first_tokens, n_steps, kv_round=None):
    toks, logits = [], []
    for t0 in first_tokens:
        s = decoder_np.Session(cfg, weights, kv_round=kv_round)
        tok, seq_t, seq_l = int(t0), [], []
        for _ in range(n_steps):
            tok, lg = s.step(tok)
            seq_t.append(tok)
            seq_l.append(lg)
        toks.append(seq_t)
        logits.append(seq_l)
    return np.array(toks).T, np.array(logits).transpose(1, 0, 2)  # [steps, batch(, vocab)]


@pytest.mark.parametrize("serving,kv_dtype", [("float32", "float32"), ("float32", "bfloat16"),
                                              ("bfloat16", "bfloat16")])
def test_decoder_matches_reference_forward(gpu_ctx, serving, kv_dtype):
    cfg = tiny_cfg(serving=serving, kv_dtype=kv_dtype)
    weights = random_model(cfg, RANKS, seed=3)
    first = [5, 77, 120]
    kv_round = decoder_np._bf16 if kv_dtype == "bfloat16" else None
    want_t, want_l = reference_run(cfg, weights, first, 6, kv_round)
    dec = Decoder(gpu_ctx, cfg, weights)
    dec.start(first, [0, 0, 0])
    got_l = []
    got_t = []
    for _ in range(6):
        dec.step()
        got_l.append(dec.logits.cpu().numpy().copy())
        dec.advance()
        got_t.append(dec.token_ids.cpu().numpy().copy())
    got_l, got_t = np.array(got_l), np.array(got_t)
    # teacher-force check on step 0 (identical inputs): tight; later steps may diverge only
    # if a greedy choice flips, which these seeds do not do
    tol = 2e-4 if serving == "float32" else 3e-2
    scale = np.abs(want_l).max()
    assert np.abs(got_l[0] - want_l[0]).max() <= tol * scale
    assert np.array_equal(got_t, want_t)
    assert np.abs(got_l - want_l).max() <= 5 * tol * scale


def test_graph_capture_replays_the_eager_step(gpu_ctx):
    import torch
    cfg = tiny_cfg()
    weights = random_model(cfg, RANKS, seed=4)
    eager = Decoder(gpu_ctx, cfg, weights)
    eager.start([1, 2, 3], [0, 0, 0])
    want = eager.decode(8)
    torch.cuda.synchronize()
    graphed = Decoder(gpu_ctx, cfg, weights)
    graphed.capture()
    graphed.start([1, 2, 3], [0, 0, 0])
    got = graphed.decode(8)
    assert np.array_equal(got, want)
    gpu_ctx.set_stream(None)


def test_decode_attention_against_exact_oracle(gpu_ctx):
    # config-3-like: 4 sequences of different lengths, GQA 8/2, bf16 cache
    import ctypes
    import torch
    from oracle import attention_np as anp
    from quantibbler_b200 import _lib
    rng = np.random.default_rng(0)
    B, H, KV, d, S = 4, 8, 2, 128, 700
    lens = np.array([700, 1, 333, 64], np.int32)
    q = rng.standard_normal((B, H, d)).astype(np.float32)
    k = decoder_np._bf16(rng.standard_normal((B, KV, S, d)).astype(np.float32))
    v = decoder_np._bf16(rng.standard_normal((B, KV, S, d)).astype(np.float32))
    tq = torch.from_numpy(q).cuda()
    tk = torch.from_numpy(k).cuda().to(torch.bfloat16)
    tv = torch.from_numpy(v).cuda().to(torch.bfloat16)
    tl = torch.from_numpy(lens).cuda()
    out = torch.zeros(B, H, d, device="cuda")
    n_splits = 5
    scratch = torch.zeros(_lib.lib().qk_decode_attention_scratch(B, H, d, n_splits) // 4 + 4,
                          device="cuda")
    torch.cuda.synchronize()
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    _lib.check(_lib.lib().qk_decode_attention(gpu_ctx.handle, p(tq), p(tk), p(tv), _lib.QK_BF16,
                                              p(tl), B, H, KV, d, S, n_splits, p(scratch), p(out)))
    gpu_ctx.synchronize()
    got = out.cpu().numpy()
    for b in range(B):
        n = lens[b]
        want = anp.attention_exact(q[b][None, :, None, :], k[b][None, :, :n], v[b][None, :, :n],
                                   causal=True)[0, :, 0]
        assert np.abs(got[b] - want).max() <= 1e-5 * max(1.0, np.abs(want).max()), b


def test_lm_head_and_first_max(gpu_ctx):
    import ctypes
    import torch
    from quantibbler_b200 import _lib
    rng = np.random.default_rng(1)
    T, V, d = 5, 1000, 256
    h = rng.standard_normal((T, d)).astype(np.float32)
    w = decoder_np._bf16(rng.standard_normal((V, d)).astype(np.float32))
    th = torch.from_numpy(h).cuda()
    tw = torch.from_numpy(w).cuda().to(torch.bfloat16)
    logits = torch.zeros(T, V, device="cuda")
    val = torch.zeros(T, device="cuda")
    idx = torch.zeros(T, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    lib = _lib.lib()
    _lib.check(lib.qk_lm_head(gpu_ctx.handle, p(th), p(tw), _lib.QK_BF16, T, V, d, V, p(logits)))
    gpu_ctx.synchronize()
    want = h.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(logits.cpu().numpy() - want).max() <= 1e-5 * np.abs(want).max()
    # ties: the first maximum wins (sampler.rs:5-16)
    lg = logits.clone()
    lg[0, 10] = lg[0, 700] = 1e9
    lg[1, :] = 0.0
    torch.cuda.synchronize()
    _lib.check(lib.qk_argmax_first(gpu_ctx.handle, p(lg), T, V, V, 100, p(val), p(idx)))
    gpu_ctx.synchronize()
    got = idx.cpu().numpy()
    assert got[0] == 110 and got[1] == 100
    assert np.array_equal(got[2:], np.argmax(lg.cpu().numpy()[2:], axis=1) + 100)


@pytest.mark.parametrize("tokens,vocab,d", [(8, 1000, 256), (13, 777, 128), (64, 2048, 512),
                                            (70, 300, 64)])
def test_lm_head_batched_tensor_core_form(gpu_ctx, tokens, vocab, d):
    """Eight tokens or more take the bf16 tensor-core kernel that reads the head once; the
    hidden state is arbitrary float32 (not bfloat16-valued), which the hi/lo split covers."""
    import ctypes
    import torch
    from quantibbler_b200 import _lib
    rng = np.random.default_rng(tokens + vocab)
    h = rng.standard_normal((tokens, d)).astype(np.float32)
    w = decoder_np._bf16(rng.standard_normal((vocab, d)).astype(np.float32))
    th = torch.from_numpy(h).cuda()
    tw = torch.from_numpy(w).cuda().to(torch.bfloat16)
    stride = vocab + 5
    logits = torch.full((tokens, stride), -7.0, device="cuda")
    torch.cuda.synchronize()
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    _lib.check(_lib.lib().qk_lm_head(gpu_ctx.handle, p(th), p(tw), _lib.QK_BF16, tokens, vocab, d,
                                     stride, p(logits)))
    gpu_ctx.synchronize()
    got = logits.cpu().numpy()
    want = h.astype(np.float64) @ w.astype(np.float64).T
    assert np.abs(got[:, :vocab] - want).max() <= 2e-5 * np.abs(want).max()
    assert (got[:, vocab:] == -7.0).all()


def test_large_batch_takes_the_tensor_core_gemm_and_lm_head(gpu_ctx):
    """bfloat16 serving with a batch of 16: every linear goes through the tcgen05 GEMM and
    the head through the batched tensor-core kernel; the result must agree with the GEMV
    forms (same rounding points) and replay identically from a CUDA graph."""
    import torch
    cfg = tiny_cfg(serving="bfloat16", kv_dtype="bfloat16", max_batch=16)
    weights = random_model(cfg, RANKS, seed=9)
    first = [(7 * i + 3) % cfg.vocab for i in range(16)]
    gemm = Decoder(gpu_ctx, cfg, weights)
    assert gemm.use_gemm
    gemv = Decoder(gpu_ctx, tiny_cfg(serving="bfloat16", kv_dtype="bfloat16", max_batch=16,
                                     gemm_min_batch=10 ** 6), weights)
    assert not gemv.use_gemm
    for dec in (gemm, gemv):
        dec.start(first, [0] * 16)
    for _ in range(4):
        for dec in (gemm, gemv):
            dec.step()
        gpu_ctx.synchronize()
        a, b = gemm.logits.cpu().numpy(), gemv.logits.cpu().numpy()
        assert np.abs(a - b).max() <= 3e-2 * np.abs(b).max()
        assert np.array_equal(gemm.best_idx.cpu().numpy(), gemv.best_idx.cpu().numpy())
        for dec in (gemm, gemv):
            dec.advance()
    want_t, _ = reference_run(cfg, weights, first[:3], 2, decoder_np._bf16)
    eager_tokens = gemm.decode(3)
    graph = Decoder(gpu_ctx, cfg, weights)
    graph.capture()
    graph.start(first, [0] * 16)
    got = graph.decode(2)
    assert np.array_equal(got[:, :3], want_t)
    del eager_tokens


@pytest.mark.parametrize("heads,kv_heads", [(8, 8), (8, 2), (16, 1), (12, 2)])
def test_decode_attention_tensor_core_kernel(gpu_ctx, heads, kv_heads):
    """bfloat16 cache, head_dim 128: the bf16 tensor-core kernel against the exact oracle and
    against the scalar kernel, for MHA, GQA groups of 4 and 6, and a group of 16 (two blocks
    of eight heads per kv head); ragged lengths including one key and a length that is not a
    multiple of the 16-key step."""
    import ctypes
    import torch
    from oracle import attention_np as anp
    from quantibbler_b200 import _lib
    rng = np.random.default_rng(heads * 10 + kv_heads)
    B, d, S = 3, 128, 533
    lens = np.array([533, 1, 250], np.int32)
    q = rng.standard_normal((B, heads, d)).astype(np.float32)
    k = decoder_np._bf16(rng.standard_normal((B, kv_heads, S, d)).astype(np.float32))
    v = decoder_np._bf16(rng.standard_normal((B, kv_heads, S, d)).astype(np.float32))
    tq = torch.from_numpy(q).cuda()
    tk = torch.from_numpy(k).cuda().to(torch.bfloat16)
    tv = torch.from_numpy(v).cuda().to(torch.bfloat16)
    tl = torch.from_numpy(lens).cuda()
    lib = _lib.lib()
    n_splits = 3
    scratch = torch.zeros(lib.qk_decode_attention_scratch(B, heads, d, n_splits) // 4 + 4, device="cuda")
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    outs = []
    for which in (1, 0):
        out = torch.zeros(B, heads, d, device="cuda")
        torch.cuda.synchronize()
        before = lib.qk_set_decode_attention_kernel(gpu_ctx.handle, which)
        try:
            _lib.check(lib.qk_decode_attention(gpu_ctx.handle, p(tq), p(tk), p(tv), _lib.QK_BF16, p(tl),
                                               B, heads, kv_heads, d, S, n_splits, p(scratch), p(out)))
            gpu_ctx.synchronize()
        finally:
            lib.qk_set_decode_attention_kernel(gpu_ctx.handle, before)
        outs.append(out.cpu().numpy())
    tc, scalar = outs
    group = heads // kv_heads
    for b in range(B):
        n = lens[b]
        want = anp.attention_exact(q[b][None, :, None, :], k[b][None, :, :n], v[b][None, :, :n],
                                   causal=True)[0, :, 0]
        assert np.abs(tc[b] - want).max() <= 1e-5 * max(1.0, np.abs(want).max()), (b, group)
    assert np.abs(tc - scalar).max() <= 2e-5


@pytest.mark.parametrize("case", [
    # (query heads, kv heads, head_dim, cache dtype, new tokens, first position)
    (8, 2, 128, "bfloat16", 70, 37),     # GQA group 4: one CTA per 16 positions
    (4, 4, 128, "bfloat16", 100, 0),     # MHA: four position blocks per CTA
    (4, 2, 128, "bfloat16", 33, 5),      # group 2
    (8, 1, 128, "bfloat16", 17, 200),    # group 8: two CTAs per kv head
    (4, 2, 32, "float32", 21, 3),        # any other shape: the plain kernel
    (6, 2, 128, "bfloat16", 19, 0)])     # group 3: the plain kernel as well
def test_prefill_attention_against_exact_oracle(gpu_ctx, case):
    """Causal attention of a run of new positions against the cache (bottom-right alignment,
    gpu_attention.rs:451-570 / engine/mod.rs:1074-1121 per position): the tensor-core kernel and
    the plain kernel against the float64 oracle under the exact face's 1e-5 gate."""
    import ctypes
    import torch
    from oracle import attention_np as anp
    from quantibbler_b200 import _lib
    heads, kv_heads, d, kv_dtype, T, p0 = case
    rng = np.random.default_rng(sum(case[:3]) + T)
    n_seq, seq, s_max = 2, 1, p0 + T + 9
    q = rng.standard_normal((T, heads, d)).astype(np.float32)
    k = rng.standard_normal((n_seq, kv_heads, s_max, d)).astype(np.float32)
    v = rng.standard_normal((n_seq, kv_heads, s_max, d)).astype(np.float32)
    if kv_dtype == "bfloat16":
        k, v = decoder_np._bf16(k), decoder_np._bf16(v)
    tq = torch.from_numpy(q).cuda()
    tdt = torch.bfloat16 if kv_dtype == "bfloat16" else torch.float32
    tk, tv = torch.from_numpy(k).cuda().to(tdt), torch.from_numpy(v).cuda().to(tdt)
    out = torch.full((T, heads, d), float("nan"), device="cuda")
    torch.cuda.synchronize()
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    tag = _lib.QK_BF16 if kv_dtype == "bfloat16" else _lib.QK_F32
    _lib.check(_lib.lib().qk_prefill_attention(gpu_ctx.handle, p(tq), p(tk), p(tv), tag, seq, p0, T,
                                               heads, kv_heads, d, s_max, p(out)))
    gpu_ctx.synchronize()
    got = out.cpu().numpy()
    n_keys = p0 + T
    want = anp.attention_exact(q.transpose(1, 0, 2)[None], k[seq][None, :, :n_keys],
                               v[seq][None, :, :n_keys], causal=True)[0].transpose(1, 0, 2)
    assert np.isfinite(got).all()
    assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("cfg_kw,tol", [
    (dict(), 2e-4),                                                      # small heads, float32 everywhere
    (dict(n_heads=8, n_kv_heads=2, head_dim=128, d_model=256, kv_dtype="bfloat16"), 2e-4),
    (dict(n_heads=8, n_kv_heads=2, head_dim=128, d_model=256, kv_dtype="bfloat16",
          serving="bfloat16"), 3e-2)])
def test_batched_prefill_matches_the_token_by_token_path(gpu_ctx, cfg_kw, tol):
    """Decoder.prefill puts the whole prompt through the trunk at once (tensor-core GEMM for
    bfloat16 serving, one GEMV instance per position otherwise; tensor-core causal attention
    for a bfloat16 cache with head_dim 128).  The logits of the last prompt position and the
    tokens decoded after it must be those of the reference's one-position-at-a-time loop
    (engine/mod.rs:1393-1413), here run on the device and through the NumPy restatement."""
    cfg = tiny_cfg(max_batch=2, max_seq=96, **cfg_kw)
    weights = random_model(cfg, RANKS, seed=21)
    rng = np.random.default_rng(5)
    prompt = [int(t) for t in rng.integers(0, cfg.vocab, 45)]
    # token by token on the device, in slot 1 of the batch
    step = Decoder(gpu_ctx, cfg, weights)
    for pos, tok in enumerate(prompt):
        step.start([0, tok], [0, pos])
        step.step()
    gpu_ctx.synchronize()
    want_logits = step.logits.cpu().numpy()[1].copy()
    # the same prompt in one pass (two chunks: 32 + 13 positions)
    cfg2 = tiny_cfg(max_batch=2, max_seq=96, prefill_chunk=32, **cfg_kw)
    fast = Decoder(gpu_ctx, cfg2, weights)
    fast.prefill(prompt, seq=1)
    got_logits = fast.logits.cpu().numpy()[1].copy()
    scale = np.abs(want_logits).max()
    assert np.abs(got_logits - want_logits).max() <= tol * scale
    # the NumPy restatement of the reference's loop
    kv_round = decoder_np._bf16 if cfg.kv_dtype == "bfloat16" else None
    session = decoder_np.Session(cfg, weights, kv_round=kv_round)
    for tok in prompt:
        _, ref_logits = session.step(tok)
    assert np.abs(got_logits - ref_logits).max() <= 5 * tol * np.abs(ref_logits).max()
    # the cache the prefill left behind continues like the stepped one
    top2 = np.sort(want_logits)[-2:]
    if top2[1] - top2[0] > 10 * tol * scale:
        assert int(fast.best_idx[1]) == int(step.best_idx[1])
        for dec in (step, fast):
            dec.advance()
            dec.step()
        gpu_ctx.synchronize()
        a, b = fast.logits.cpu().numpy()[1], step.logits.cpu().numpy()[1]
        assert np.abs(a - b).max() <= 2 * tol * np.abs(b).max()


def test_generate_uses_the_batched_prefill_for_long_prompts(gpu_ctx):
    cfg = tiny_cfg(max_batch=1, max_seq=128)
    weights = random_model(cfg, RANKS, seed=22)
    prompt = [int(t) for t in np.random.default_rng(6).integers(1, cfg.vocab, 40)]
    want, finish = decoder_np.generate(cfg, weights, prompt, 6)
    dec = Decoder(gpu_ctx, cfg, weights)
    assert len(prompt) >= cfg.prefill_min_tokens
    got = dec.generate(prompt, 6)
    assert got["completion_tokens"] == want and got["finish"] == finish
    with pytest.raises(ValueError, match="does not fit the KV cache"):
        dec.prefill([1] * 200)


@pytest.mark.parametrize("serving", ["float32", "bfloat16"])
def test_fed_plans_reproduce_the_plain_step(gpu_ctx, serving):
    """With fed plans the digit tables of the linears' inputs are written by the kernels that
    produce those inputs (norm, attention combine, SwiGLU; several blocks per token share the
    work) and stage 1 hands over to stage 2 through its last block.  The tables are the same
    numbers and the accumulation is exact, so logits and tokens must be the plain step's bits."""
    kv = "float32" if serving == "float32" else "bfloat16"
    weights = random_model(tiny_cfg(serving=serving, kv_dtype=kv), RANKS, seed=31)
    plain = Decoder(gpu_ctx, tiny_cfg(serving=serving, kv_dtype=kv), weights)
    fed = Decoder(gpu_ctx, tiny_cfg(serving=serving, kv_dtype=kv, feed_max_batch=4), weights)
    assert fed.fed and not plain.fed
    first = [9, 41, 100]
    for dec in (plain, fed):
        dec.start(first, [0, 0, 0])
    for _ in range(5):
        for dec in (plain, fed):
            dec.step()
        gpu_ctx.synchronize()
        a, b = fed.logits.cpu().numpy(), plain.logits.cpu().numpy()
        # the SwiGLU is evaluated by two kernels (fed: inside the feeding kernel): same
        # float32 expression, so the same bits
        assert np.array_equal(a, b)
        for dec in (plain, fed):
            dec.advance()
    graph = Decoder(gpu_ctx, tiny_cfg(serving=serving, kv_dtype=kv, feed_max_batch=4), weights)
    graph.capture()
    graph.start(first, [0, 0, 0])
    eager = Decoder(gpu_ctx, tiny_cfg(serving=serving, kv_dtype=kv), weights)
    eager.start(first, [0, 0, 0])
    assert np.array_equal(graph.decode(6), eager.decode(6))


def step_cfg(**kw):
    """A small model inside what the whole-step kernel takes: head_dim 128, bfloat16 cache,
    ragged ranks and widths (several k-steps, partial row groups), four key splits."""
    base = dict(n_layers=3, d_model=256, n_heads=4, n_kv_heads=2, head_dim=128, d_ff=640, vocab=192,
                max_seq=96, max_batch=2, kv_dtype="bfloat16", serving="bfloat16", n_splits=4)
    base.update(kw)
    return DecoderConfig(**base)


STEP_RANKS = {"q": 72, "k": 40, "v": 40, "o": 100, "gate": 130, "up": 130, "down": 90}


@pytest.mark.parametrize("serving,batch", [("bfloat16", 1), ("bfloat16", 2), ("float32", 1), ("float32", 3)])
def test_whole_step_kernel_reproduces_the_step_of_separate_launches(gpu_ctx, serving, batch):
    """All blocks of a step in one cooperative kernel (norms, RoPE, cache append, combine and
    SwiGLU folded into its phases) against the same step made of separate launches: the same
    exact integer sums and the same device functions in the same order, so logits, tokens and
    cache contents must agree bit for bit - over enough steps that the appended position
    crosses from one key split into the next - and stay within the usual tolerance of the
    forward oracle."""
    cfg = step_cfg(serving=serving, max_batch=batch)
    weights = random_model(cfg, STEP_RANKS, seed=77)
    plain = Decoder(gpu_ctx, step_cfg(serving=serving, max_batch=batch), weights)
    fused = Decoder(gpu_ctx, step_cfg(serving=serving, max_batch=batch, fused_step_max_batch=batch), weights)
    assert fused.step_kernel is not None and plain.step_kernel is None
    first = [9, 41, 7][:batch]
    want_t, want_l = reference_run(cfg, weights, first, 4, decoder_np._bf16)
    for dec in (plain, fused):
        dec.start(first, [0] * batch)
    tol = 2e-4 if serving == "float32" else 3e-2
    for step in range(30):
        for dec in (plain, fused):
            dec.step()
        gpu_ctx.synchronize()
        a, b = fused.logits.cpu().numpy(), plain.logits.cpu().numpy()
        assert np.array_equal(a, b), step
        if step < 4:
            assert np.abs(a - want_l[step]).max() <= 5 * tol * np.abs(want_l).max()
        for dec in (plain, fused):
            dec.advance()
        assert np.array_equal(fused.token_ids.cpu().numpy(), plain.token_ids.cpu().numpy())
        if step < 4:
            assert np.array_equal(fused.token_ids.cpu().numpy(), want_t[step])
    for li in range(cfg.n_layers):
        assert torch_equal(fused.cache_k[li], plain.cache_k[li]) and torch_equal(fused.cache_v[li], plain.cache_v[li])
    # captured in a graph (a cooperative launch inside a CUDA graph) it replays the same tokens
    graph = Decoder(gpu_ctx, step_cfg(serving=serving, max_batch=batch, fused_step_max_batch=batch), weights)
    graph.capture()
    graph.start(first, [0] * batch)
    eager = Decoder(gpu_ctx, step_cfg(serving=serving, max_batch=batch, fused_step_max_batch=batch), weights)
    eager.start(first, [0] * batch)
    assert np.array_equal(graph.decode(12), eager.decode(12))
    gpu_ctx.set_stream(None)


def torch_equal(a, b):
    import torch
    return bool(torch.equal(a, b))


def test_whole_step_kernel_is_refused_outside_its_limits(gpu_ctx):
    """head_dim other than 128, a float32 cache or too many tokens keep the separate launches."""
    weights = random_model(tiny_cfg(), RANKS, seed=5)
    dec = Decoder(gpu_ctx, tiny_cfg(fused_step_max_batch=4), weights)   # head_dim 16, float32 cache
    assert dec.step_kernel is None
    cfg = step_cfg(max_batch=9, fused_step_max_batch=9)   # more tokens than the kernel takes
    dec = Decoder(gpu_ctx, cfg, random_model(cfg, STEP_RANKS, seed=6))
    assert dec.step_kernel is None


@pytest.mark.parametrize("serving", ["float32", "bfloat16"])
def test_one_launch_attention_reproduces_the_three_launches(gpu_ctx, serving):
    """RoPE + cache append + split attention + combine in one kernel (the rotation in the
    fragment loader, the append by the block whose keys include the new position, the combine
    by the last split to finish) against rope_cache + decode_attention + combine: the same
    device functions, so logits, tokens and cache contents must be identical - over enough
    steps that the appended position crosses from one key split into the next."""
    cfg = step_cfg(serving=serving, max_batch=2)
    weights = random_model(cfg, STEP_RANKS, seed=78)
    three = Decoder(gpu_ctx, step_cfg(serving=serving, max_batch=2, fused_attention=False), weights)
    one = Decoder(gpu_ctx, step_cfg(serving=serving, max_batch=2), weights)
    assert one.fused_attention and not three.fused_attention
    for dec in (three, one):
        dec.start([9, 41], [0, 5])
    for step in range(30):
        for dec in (three, one):
            dec.step()
        gpu_ctx.synchronize()
        assert np.array_equal(one.logits.cpu().numpy(), three.logits.cpu().numpy()), step
        for dec in (three, one):
            dec.advance()
    # (sequence 1 started at position 5 over rows nobody wrote: both caches hold zeros there)
    for li in range(cfg.n_layers):
        assert torch_equal(one.cache_k[li], three.cache_k[li]) and torch_equal(one.cache_v[li], three.cache_v[li])


@pytest.mark.parametrize("batch", [2, 6])
@pytest.mark.parametrize("serving", ["float32", "bfloat16"])
def test_norm_and_swiglu_inside_the_linears_reproduce_the_separate_launches(gpu_ctx, serving, batch):
    """At small batches q,k,v and gate,up form the RMSNorm of the residual stream themselves
    (every block of their first stage, with the norm kernel's thread count and summation
    order; one block also writes the updated stream) and the down projection reads gate and up
    through the SwiGLU: three launches less per block.  Logits and residual stream must be the
    bits of the separate norm and SwiGLU kernels."""
    base = dict(serving=serving, max_batch=batch)
    weights = random_model(step_cfg(**base), STEP_RANKS, seed=79)
    apart = Decoder(gpu_ctx, step_cfg(norm_fused_max_batch=0, gated_down_max_batch=0, **base), weights)
    fused = Decoder(gpu_ctx, step_cfg(**base), weights)
    assert "qkv_normed" in fused.plans[0] and "gu_normed" in fused.plans[0] and fused.gated_down
    assert "qkv_normed" not in apart.plans[0] and not apart.gated_down
    for dec in (apart, fused):
        dec.start([3, 77, 5, 120, 9, 64][:batch], [0, 2, 1, 0, 3, 2][:batch])
    for step in range(6):
        for dec in (apart, fused):
            dec.step()
        gpu_ctx.synchronize()
        assert np.array_equal(fused.logits.cpu().numpy(), apart.logits.cpu().numpy()), step
        assert torch_equal(fused.x, apart.x) and torch_equal(fused.x2, apart.x2), step
        for dec in (apart, fused):
            dec.advance()


def test_normed_plan_is_refused_outside_its_form(gpu_ctx):
    """A stream wider than the norm kernel's sixteen entries per thread, an in-place update of
    the stream and a gated plan are refused with the plan left as it was."""
    import torch
    from quantibbler_b200.decoder import random_layer
    from quantibbler_b200.gpu import KernelError, LayerPlan, PackedLayer
    rng = np.random.default_rng(5)
    for dout, din, r in ((64, 8704, 32),):
        spec = random_layer(rng, dout, din, r)
        layer = PackedLayer(gpu_ctx, spec["ub_rows"], spec["vb_t_rows"], dout, din, r, spec["s1"], spec["s2"],
                            None, serving="float32")
        x, x2, y, w = (torch.zeros(n, device="cuda") for n in (din, din, dout, din))
        plan = LayerPlan(gpu_ctx, [(layer, x.data_ptr(), y.data_ptr())])
        with pytest.raises(KernelError):
            plan.set_norm([None], w.data_ptr(), 1e-5, [x2.data_ptr()])
    spec = random_layer(rng, 64, 512, 32)
    layer = PackedLayer(gpu_ctx, spec["ub_rows"], spec["vb_t_rows"], 64, 512, 32, spec["s1"], spec["s2"], None,
                        serving="float32")
    x, u, y, w = (torch.ones(n, device="cuda") for n in (512, 512, 64, 512))
    plan = LayerPlan(gpu_ctx, [(layer, x.data_ptr(), y.data_ptr())])
    with pytest.raises(KernelError):
        plan.set_norm([None], w.data_ptr(), 1e-5, [x.data_ptr()])       # in place
    gated = LayerPlan(gpu_ctx, [(layer, x.data_ptr(), u.data_ptr(), y.data_ptr())], gated=True)
    with pytest.raises(KernelError):
        gated.set_norm([None], w.data_ptr(), 1e-5, [None])
    plan.apply()   # still the plain plan
    gpu_ctx.synchronize()
    assert torch.isfinite(y).all()
