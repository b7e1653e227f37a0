"""GPU parity of the tensor-core prefill GEMM against the per-token reference apply."""

import numpy as np
import pytest

import oracle
from conftest import make_layer
from quantibbler_b200.gpu import PackedLayer

pytestmark = pytest.mark.gpu


def run_case(ctx, dout, din, r, n_tokens, seed, with_bias):
    import torch
    L = make_layer(dout, din, r, seed=seed, with_bias=with_bias)
    layer = PackedLayer(ctx, L["ub_rows"], L["vb_t_rows"], dout, din, r, L["s1"], L["s2"],
                        L["bias"], serving="bfloat16")
    rng = np.random.default_rng(seed + 1)
    xs = rng.standard_normal((n_tokens, din)).astype(np.float32)
    x = torch.from_numpy(xs).cuda()
    y = torch.full((n_tokens, dout), float("nan"), device="cuda")
    torch.cuda.synchronize()
    layer.apply_prefill(x.data_ptr(), n_tokens, y.data_ptr())
    ctx.synchronize()   # the call is asynchronous; this also reports an expired in-kernel wait
    got = y.cpu().numpy()
    assert np.isfinite(got).all()
    check = range(n_tokens) if n_tokens <= 16 else [0, 1, n_tokens // 2, n_tokens - 2, n_tokens - 1]
    for t in check:
        want = oracle.layer_apply(L["ub_rows"], L["vb_t_rows"], dout, din, r, L["s1"], L["s2"],
                                  L["bias"], xs[t], serving="bfloat16")
        # exact float64 two-stage product for the backward scale
        z = oracle.bf16_bits_to_f32(oracle.f32_to_bf16_bits((L["s2"] * xs[t]).astype(np.float32)))
        tt = oracle.unpack_signs(L["vb_t_rows"], din) @ z.astype(np.float64)
        scale = np.abs(L["s1"].astype(np.float64)) * np.abs(tt).sum()
        err = np.abs(got[t].astype(np.float64) - want)
        assert (err / np.maximum(scale, 1e-300)).max() <= 2e-2, t   # bf16 backward bound, two stages
        assert err.max() <= 2e-2 * np.abs(want).max(), t
    # the decode path computes the same layer: the two must agree to bf16 rounding
    one = layer.apply(xs[0])
    assert np.abs(one - got[0]).max() <= 2e-2 * np.abs(one).max()
    layer.close()
    return got


@pytest.mark.parametrize("shape", [(256, 64, 64, 128), (300, 1100, 515, 200), (96, 160, 72, 7),
                                   (1024, 4096, 1024, 256)])
def test_prefill_matches_reference(gpu_ctx, shape):
    dout, din, r, n_tokens = shape
    got = run_case(gpu_ctx, dout, din, r, n_tokens, seed=dout + n_tokens, with_bias=dout % 2 == 0)
    again = run_case(gpu_ctx, dout, din, r, n_tokens, seed=dout + n_tokens, with_bias=dout % 2 == 0)
    assert np.array_equal(got, again)


@pytest.mark.parametrize("shape", [(14336, 4096, 2560), (4096, 14336, 2560)],
                         ids=["gate_up", "down"])
def test_prefill_at_config1(gpu_ctx, shape):
    """benchmark configuration 1 at full size: the Llama-3-8B MLP shapes at rank 2560 on 2048 tokens
    (the case the prefill benchmark times, with tiles split between CTAs); five tokens are
    checked against the oracle's per-token bfloat16 apply."""
    dout, din, r = shape
    run_case(gpu_ctx, dout, din, r, 2048, seed=dout // 7, with_bias=False)


def test_prefill_needs_bf16_serving(gpu_ctx):
    L = make_layer(32, 64, 16, seed=1)
    layer = PackedLayer(gpu_ctx, L["ub_rows"], L["vb_t_rows"], 32, 64, 16, L["s1"], L["s2"])
    with pytest.raises(ValueError, match="bfloat16 serving"):
        layer.apply_prefill(0, 4, 0)


def test_several_layers_in_one_call(gpu_ctx):
    """q, k, v style: three layers of different ranks and widths on the same input through
    one launch per stage; each must agree with its own single-layer call (the work is dealt
    out differently, so split tiles add their partial sums in another order: equal up to one
    bfloat16 rounding of an intermediate) and with the oracle."""
    import torch
    from quantibbler_b200.gpu import apply_prefill_many
    din, n_tokens = 320, 150
    shapes = [(260, 70), (96, 33), (512, 200)]
    rng = np.random.default_rng(3)
    xs = rng.standard_normal((n_tokens, din)).astype(np.float32)
    x = torch.from_numpy(xs).cuda()
    params, layers, ys = [], [], []
    for i, (dout, r) in enumerate(shapes):
        L = make_layer(dout, din, r, seed=40 + i, with_bias=i == 1)
        params.append(L)
        layers.append(PackedLayer(gpu_ctx, L["ub_rows"], L["vb_t_rows"], dout, din, r, L["s1"], L["s2"],
                                  L["bias"], serving="bfloat16"))
        ys.append(torch.full((n_tokens, dout), float("nan"), device="cuda"))
    torch.cuda.synchronize()
    apply_prefill_many(layers, x.data_ptr(), n_tokens, [y.data_ptr() for y in ys])
    gpu_ctx.synchronize()
    for (dout, r), L, layer, y in zip(shapes, params, layers, ys):
        got = y.cpu().numpy()
        assert np.isfinite(got).all()
        single = torch.zeros(n_tokens, dout, device="cuda")
        layer.apply_prefill(x.data_ptr(), n_tokens, single.data_ptr())
        gpu_ctx.synchronize()
        ref = single.cpu().numpy()
        assert np.abs(got - ref).max() <= 1e-2 * np.abs(ref).max()
        assert np.mean(got == ref) >= 0.99
        for t in (0, n_tokens - 1):
            want = oracle.layer_apply(L["ub_rows"], L["vb_t_rows"], dout, din, r, L["s1"], L["s2"],
                                      L["bias"], xs[t], serving="bfloat16")
            assert np.abs(got[t] - want).max() <= 2e-2 * np.abs(want).max()
        layer.close()
    with pytest.raises(ValueError, match="share their input"):
        a = make_layer(32, 64, 16, seed=1)
        b = make_layer(32, 128, 16, seed=2)
        la = PackedLayer(gpu_ctx, a["ub_rows"], a["vb_t_rows"], 32, 64, 16, a["s1"], a["s2"], None, serving="bfloat16")
        lb = PackedLayer(gpu_ctx, b["ub_rows"], b["vb_t_rows"], 32, 128, 16, b["s1"], b["s2"], None, serving="bfloat16")
        apply_prefill_many([la, lb], 0, 4, [0, 0])


@pytest.mark.parametrize("shape", [(96, 320, 40, 150), (200, 333, 64, 37), (256, 1024, 128, 9)])
def test_gated_prefill_equals_swiglu_then_prefill(gpu_ctx, shape):
    """The down projection behind the SwiGLU (engine/mod.rs:931-935): the activation formed
    inside the GEMM's scaling kernel must give the bits of the SwiGLU kernel followed by the
    plain call (the same expression, the same roundings), for widths on and off the vector
    path."""
    import torch
    from quantibbler_b200 import _lib
    from quantibbler_b200._lib import check
    from quantibbler_b200.gpu import apply_prefill_many, apply_prefill_many_gated
    dout, din, r, n_tokens = shape
    L = make_layer(dout, din, r, seed=din + r, with_bias=True)
    layer = PackedLayer(gpu_ctx, L["ub_rows"], L["vb_t_rows"], dout, din, r, L["s1"], L["s2"], L["bias"],
                        serving="bfloat16")
    gen = torch.Generator(device="cuda").manual_seed(din)
    gate = torch.randn(n_tokens, din, device="cuda", generator=gen) * 2
    up = torch.randn(n_tokens, din, device="cuda", generator=gen)
    act = torch.zeros_like(gate)
    apart = torch.zeros(n_tokens, dout, device="cuda")
    fused = torch.full((n_tokens, dout), float("nan"), device="cuda")
    torch.cuda.synchronize()
    check(_lib.lib().qk_swiglu(gpu_ctx.handle, gate.data_ptr(), up.data_ptr(), n_tokens * din, act.data_ptr()))
    apply_prefill_many([layer], act.data_ptr(), n_tokens, [apart.data_ptr()])
    apply_prefill_many_gated([layer], gate.data_ptr(), up.data_ptr(), n_tokens, [fused.data_ptr()])
    gpu_ctx.synchronize()
    assert np.array_equal(fused.cpu().numpy(), apart.cpu().numpy())
    # and against the restatement on one token
    a0 = act[0].cpu().numpy()
    want = oracle.layer_apply(L["ub_rows"], L["vb_t_rows"], dout, din, r, L["s1"], L["s2"], L["bias"], a0,
                              serving="bfloat16")
    assert np.abs(fused[0].cpu().numpy() - want).max() <= 2e-2 * np.abs(want).max()
    with pytest.raises(ValueError, match="gate and up"):
        apply_prefill_many_gated([layer], gate.data_ptr(), 0, n_tokens, [fused.data_ptr()])
    layer.close()
