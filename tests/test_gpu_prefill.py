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


def test_prefill_needs_bf16_serving(gpu_ctx):
    L = make_layer(32, 64, 16, seed=1)
    layer = PackedLayer(gpu_ctx, L["ub_rows"], L["vb_t_rows"], 32, 64, 16, L["s1"], L["s2"])
    with pytest.raises(ValueError, match="bfloat16 serving"):
        layer.apply_prefill(0, 4, 0)
