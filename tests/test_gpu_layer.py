"""GPU parity of the device-resident factorized linear through the C ABI."""

import ctypes

import numpy as np
import pytest

import oracle
from conftest import golden, make_layer
from quantibbler_b200._lib import KernelError
from quantibbler_b200.gpu import PackedLayer, apply_group

pytestmark = pytest.mark.gpu

# crates/quantibbler-kernels/tests/parity.rs:795,806: backward bounds on sum|v_k|
F32_BACKWARD = 1e-6
BF16_BACKWARD = 1e-2


def backward_scale(L):
    """Upper bound of sum_k |term| for each output of the two-stage product."""
    z = np.abs(L["s2"].astype(np.float64) * L["x"].astype(np.float64))
    t_abs = np.full(L["r"], z.sum())             # |t_j| <= sum|z|
    return np.abs(L["s1"].astype(np.float64)) * t_abs.sum()  # |y_i| <= s1_i * sum_j |t_j|


def exact_layer(L):
    z = (L["s2"] * L["x"]).astype(np.float32).astype(np.float64)
    t = oracle.unpack_signs(L["vb_t_rows"], L["din"]) @ z
    u = oracle.unpack_signs(L["ub_rows"], L["r"]) @ t
    y = u * L["s1"].astype(np.float64)
    if L["bias"] is not None:
        y = y + L["bias"]
    return y, t


@pytest.fixture(params=[1, 0], ids=["bitslice", "signselect"])
def kernel_ctx(gpu_ctx, request):
    prev = gpu_ctx.set_gemv_kernel(request.param)
    yield gpu_ctx
    gpu_ctx.set_gemv_kernel(prev)


def check_layer(ctx, L, serving, expect_bit_identical=True):
    layer = PackedLayer(ctx, L["ub_rows"], L["vb_t_rows"], L["dout"], L["din"], L["r"], L["s1"],
                        L["s2"], L["bias"], serving=serving)
    y = layer.apply(L["x"])
    want = oracle.layer_apply(L["ub_rows"], L["vb_t_rows"], L["dout"], L["din"], L["r"], L["s1"],
                              L["s2"], L["bias"], L["x"], serving=serving)
    exact, t = exact_layer(L)
    # stage-wise backward bound: each output's error is measured against the magnitude
    # scale of the terms that were summed to make it
    term_scale = np.abs(L["s1"].astype(np.float64)) * np.abs(t).sum()
    tol = F32_BACKWARD if serving == "float32" else BF16_BACKWARD
    # two chained products: stage-1 error propagates through stage 2
    err = np.abs(y.astype(np.float64) - want.astype(np.float64))
    assert (err / np.maximum(term_scale, 1e-300)).max() <= 2 * tol, serving
    # the benchmark's bound: max error relative to the largest reference output
    rel = err.max() / np.abs(want).max()
    assert rel <= (2e-3 if serving == "float32" else 2e-2), (serving, rel)
    # run-to-run bit identity
    assert np.array_equal(layer.apply(L["x"]), y)
    if ctx.set_gemv_kernel(-1) == 1 and serving == "float32":
        # the bit-sliced kernel sums exactly, so it reproduces the reference's float64
        # stages to the last float32 bit except where u sits on a rounding boundary
        ulp = np.spacing(np.abs(want).astype(np.float32)).astype(np.float64)
        # (where rows cancel, the reference's own float64 loop is only good to 1e-12 of the
        # term scale: fast.rs:10-18)
        assert (err <= 2 * ulp + 1e-12 * term_scale).all()
        if expect_bit_identical:
            assert np.mean(y == want) >= 0.9
    layer.close()
    return y, want


@pytest.mark.parametrize("serving", ["float32", "bfloat16"])
@pytest.mark.parametrize("key", ["small", "odd", "mid"])
def test_golden_layers(kernel_ctx, key, serving):
    gpu_ctx = kernel_ctx
    g = golden("layer")
    m = g.meta[key]
    L = dict(ub_rows=g[key + "_ub_rows"], vb_t_rows=g[key + "_vb_t_rows"], s1=g[key + "_s1"],
             s2=g[key + "_s2"], x=g[key + "_x"], bias=g[key + "_bias"] if m["bias"] else None,
             dout=m["dout"], din=m["din"], r=m["r"])
    y, want = check_layer(gpu_ctx, L, serving)
    gold = g[key + ("_y_f32" if serving == "float32" else "_y_bf16")]
    assert np.array_equal(want, gold)


@pytest.mark.parametrize("serving", ["float32", "bfloat16"])
def test_config0_layer_against_reference_vector(kernel_ctx, serving):
    gpu_ctx = kernel_ctx
    g = golden("layer")
    m = g.meta["config0"]
    L = make_layer(m["dout"], m["din"], m["r"], m["seed"])
    layer = PackedLayer(gpu_ctx, L["ub_rows"], L["vb_t_rows"], L["dout"], L["din"], L["r"],
                        L["s1"], L["s2"], None, serving=serving)
    y = layer.apply(L["x"])
    gold = g["config0_y_f32" if serving == "float32" else "config0_y_bf16"]
    rel = np.abs(y.astype(np.float64) - gold).max() / np.abs(gold).max()
    assert rel <= (2e-5 if serving == "float32" else 2e-2), rel
    if serving == "float32":
        t = g["config0_t_f64"]
        scale = np.abs(L["s1"].astype(np.float64)) * np.abs(t).sum()
        assert (np.abs(y - gold) / scale).max() <= 2 * F32_BACKWARD


@pytest.mark.parametrize("shape", [(1, 1, 1), (8, 8, 8), (33, 129, 17), (300, 4097, 130),
                                   (64, 14336, 96), (4096, 300, 1102)])
def test_odd_shapes(kernel_ctx, shape):
    gpu_ctx = kernel_ctx
    dout, din, r = shape
    L = make_layer(dout, din, r, seed=dout + din + r, with_bias=(dout % 2 == 0))
    check_layer(gpu_ctx, L, "float32")
    check_layer(gpu_ctx, L, "bfloat16")


def test_dirty_pad_bits_are_ignored(kernel_ctx):
    gpu_ctx = kernel_ctx
    # crates/quantibbler-kernels/tests/fixtures/packed_matvec.json (packed_dirty): bits
    # beyond n_bits in the last byte of a row must not change any result
    L = make_layer(24, 21, 13, seed=77)
    clean = PackedLayer(gpu_ctx, L["ub_rows"], L["vb_t_rows"], 24, 21, 13, L["s1"], L["s2"])
    ub_dirty = L["ub_rows"].copy()
    ub_dirty[:, -1] |= 0xE0
    vbt_dirty = L["vb_t_rows"].copy()
    vbt_dirty[:, -1] |= 0xE0
    dirty = PackedLayer(gpu_ctx, ub_dirty, vbt_dirty, 24, 21, 13, L["s1"], L["s2"])
    assert np.array_equal(clean.apply(L["x"]), dirty.apply(L["x"]))


def test_group_apply_matches_single(gpu_ctx):
    import torch
    n = 5
    layers, xs, want = [], [], []
    for i in range(n):
        L = make_layer(128, 256, 64, seed=100 + i, with_bias=True)
        layer = PackedLayer(gpu_ctx, L["ub_rows"], L["vb_t_rows"], 128, 256, 64, L["s1"], L["s2"],
                            L["bias"])
        layers.append(layer)
        xs.append(L["x"])
        want.append(layer.apply(L["x"]))
    x = torch.from_numpy(np.stack(xs)).cuda()
    y = torch.zeros(n, 128, device="cuda")
    torch.cuda.synchronize()
    apply_group(gpu_ctx, layers, x.data_ptr(), y.data_ptr())
    gpu_ctx.synchronize()
    assert np.array_equal(y.cpu().numpy(), np.stack(want))


@pytest.mark.parametrize("serving", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(96, 160, 72), (130, 1100, 515)])
def test_fused_layer_kernel_matches_two_stage_path(gpu_ctx, shape, serving):
    # with at least one instance per SM the two stages run fused in one block per layer;
    # both paths accumulate in integers, so they must agree bit for bit
    import torch
    from quantibbler_b200.gpu import LayerGroup
    dout, din, r = shape
    n = 160
    layers, xs, want = [], [], []
    for i in range(n):
        L = make_layer(dout, din, r, seed=500 + i % 7, with_bias=(i % 2 == 0))
        layer = PackedLayer(gpu_ctx, L["ub_rows"], L["vb_t_rows"], dout, din, r, L["s1"],
                            L["s2"], L["bias"], serving=serving)
        layers.append(layer)
        x = (L["x"] * (1 + i)).astype(np.float32)
        xs.append(x)
        if i < 7:
            want.append(layer.apply(x))
            ref = oracle.layer_apply(L["ub_rows"], L["vb_t_rows"], dout, din, r, L["s1"],
                                     L["s2"], L["bias"], x, serving=serving)
            tol = 2e-5 if serving == "float32" else 2e-2
            assert np.abs(want[-1] - ref).max() <= tol * np.abs(ref).max()
    x = torch.from_numpy(np.stack(xs)).cuda()
    y = torch.zeros(n, dout, device="cuda")
    torch.cuda.synchronize()
    group = LayerGroup(gpu_ctx, layers, x.data_ptr(), y.data_ptr())
    group.apply()
    gpu_ctx.synchronize()
    got = y.cpu().numpy()
    for i in range(7):
        assert np.array_equal(got[i], want[i]), i
    first = got.copy()
    group.apply()
    gpu_ctx.synchronize()
    assert np.array_equal(y.cpu().numpy(), first)


@pytest.mark.parametrize("serving", ["float32", "bfloat16"])
def test_benchmarked_launch_shape_at_config0(gpu_ctx, serving):
    """The launch bench.py times: one grouped apply of at least 2 x 148 config-0 instances
    (4096 x 4096, rank 1024), which is the size at which the library picks the form it uses for
    many independent layers.  Eight instances are checked against the oracle under the same
    gates as a single layer, one of them against the reference's own config-0 vector."""
    import torch
    from quantibbler_b200.gpu import LayerGroup
    g = golden("layer")
    m = g.meta["config0"]
    dout, din, r = m["dout"], m["din"], m["r"]
    assert (dout, din, r) == (4096, 4096, 1024)
    n_distinct, n_inst = 8, 304
    specs = [make_layer(dout, din, r, m["seed"])]
    rng = np.random.default_rng(20)
    for i in range(1, n_distinct):
        specs.append(dict(
            ub_rows=rng.integers(0, 256, size=(dout, r // 8), dtype=np.uint8),
            vb_t_rows=rng.integers(0, 256, size=(r, din // 8), dtype=np.uint8),
            s1=(np.abs(rng.standard_normal(dout)) * 0.02 + 1e-3).astype(np.float32),
            s2=(np.abs(rng.standard_normal(din)) * 0.02 + 1e-3).astype(np.float32),
            bias=(rng.standard_normal(dout) * 0.1).astype(np.float32) if i % 2 else None,
            dout=dout, din=din, r=r))
    layers = [PackedLayer(gpu_ctx, s["ub_rows"], s["vb_t_rows"], dout, din, r, s["s1"], s["s2"],
                          s.get("bias"), serving=serving) for s in specs]
    xs = rng.standard_normal((n_inst, din)).astype(np.float32)
    xs[0] = specs[0]["x"]
    x = torch.from_numpy(xs).cuda()
    y = torch.full((n_inst, dout), float("nan"), device="cuda")
    torch.cuda.synchronize()
    group = LayerGroup(gpu_ctx, [layers[i % n_distinct] for i in range(n_inst)], x.data_ptr(),
                       y.data_ptr())
    launches0 = gpu_ctx.launch_count
    group.apply()
    gpu_ctx.synchronize()
    assert gpu_ctx.launch_count - launches0 == 1    # the single-launch form, as in the benchmark
    got = y.cpu().numpy()
    assert np.isfinite(got).all()
    tol = F32_BACKWARD if serving == "float32" else BF16_BACKWARD
    for i in (0, 1, 2, 3, 150, 297, 302, 303):
        s = dict(specs[i % n_distinct], x=xs[i])
        want = oracle.layer_apply(s["ub_rows"], s["vb_t_rows"], dout, din, r, s["s1"], s["s2"],
                                  s.get("bias"), xs[i], serving=serving)
        if s.get("bias") is None:
            s["bias"] = None
        _, t = exact_layer(s)
        term_scale = np.abs(s["s1"].astype(np.float64)) * np.abs(t).sum()
        err = np.abs(got[i].astype(np.float64) - want.astype(np.float64))
        assert (err / term_scale).max() <= 2 * tol, (i, serving)
        assert err.max() <= (2e-3 if serving == "float32" else 2e-2) * np.abs(want).max(), i
        if serving == "float32":
            ulp = np.spacing(np.abs(want).astype(np.float32)).astype(np.float64)
            assert (err <= 2 * ulp + 1e-12 * term_scale).all(), i
            assert np.mean(got[i] == want) >= 0.9, i
        # the same instance through the single-layer call (another kernel form, also exact
        # integer accumulation): identical bits
        assert np.array_equal(layers[i % n_distinct].apply(xs[i]), got[i]), i
    gold = g["config0_y_f32" if serving == "float32" else "config0_y_bf16"]
    rel = np.abs(got[0].astype(np.float64) - gold).max() / np.abs(gold).max()
    assert rel <= (2e-5 if serving == "float32" else 2e-2), rel
    group.apply()
    gpu_ctx.synchronize()
    assert np.array_equal(y.cpu().numpy(), got)     # run-to-run bit identity
    group.close()
    for layer in layers:
        layer.close()


@pytest.mark.parametrize("serving", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape,n_inst", [((1100, 700, 1102), 150), ((200, 2100, 70), 149),
                                          ((64, 512, 64), 300), ((4096, 4096, 431), 148)])
def test_streaming_form_matches_the_other_kernel_forms(gpu_ctx, shape, n_inst, serving):
    """With at least one instance per SM a group runs in the persistent streaming form (ring
    of chunks, producer and table-builder warps).  Row-group counts that are not a multiple of
    its 16 consumer warps, a single k-step, CTAs with one, two or three instances: all forms
    accumulate exactly in integers, so the outputs must be the same bits as the
    one-block-per-instance form (selector 5) and as the single-layer call."""
    import torch
    from quantibbler_b200.gpu import LayerGroup
    dout, din, r = shape
    n_distinct = 5
    specs = [make_layer(dout, din, r, seed=700 + i, with_bias=(i % 2 == 1)) for i in range(n_distinct)]
    layers = [PackedLayer(gpu_ctx, s["ub_rows"], s["vb_t_rows"], dout, din, r, s["s1"], s["s2"],
                          s["bias"], serving=serving) for s in specs]
    rng = np.random.default_rng(n_inst)
    xs = (rng.standard_normal((n_inst, din)) * rng.uniform(0.01, 100, (n_inst, 1))).astype(np.float32)
    x = torch.from_numpy(xs).cuda()
    y = torch.full((n_inst, dout), float("nan"), device="cuda")
    torch.cuda.synchronize()
    group = LayerGroup(gpu_ctx, [layers[i % n_distinct] for i in range(n_inst)], x.data_ptr(),
                       y.data_ptr())
    group.apply()
    gpu_ctx.synchronize()
    got = y.cpu().numpy()
    assert np.isfinite(got).all()
    prev = gpu_ctx.set_gemv_kernel(5)
    try:
        y.fill_(float("nan"))
        group.apply()
        gpu_ctx.synchronize()
        assert np.array_equal(y.cpu().numpy(), got)
    finally:
        gpu_ctx.set_gemv_kernel(prev)
    for i in (0, 1, n_inst // 2, n_inst - 1):
        assert np.array_equal(layers[i % n_distinct].apply(xs[i]), got[i]), i
        s = specs[i % n_distinct]
        want = oracle.layer_apply(s["ub_rows"], s["vb_t_rows"], dout, din, r, s["s1"], s["s2"],
                                  s["bias"], xs[i], serving=serving)
        assert np.abs(got[i] - want).max() <= (2e-5 if serving == "float32" else 2e-2) * np.abs(want).max()
    group.apply()
    gpu_ctx.synchronize()
    assert np.array_equal(y.cpu().numpy(), got)
    group.close()
    for layer in layers:
        layer.close()


def test_streaming_form_nonfinite_and_zero_inputs(gpu_ctx):
    import torch
    from quantibbler_b200.gpu import LayerGroup
    L = make_layer(128, 300, 96, seed=31)
    layer = PackedLayer(gpu_ctx, L["ub_rows"], L["vb_t_rows"], 128, 300, 96, L["s1"], L["s2"])
    n_inst = 150
    xs = np.tile(L["x"], (n_inst, 1)).astype(np.float32)
    xs[3, 7] = np.inf
    xs[9, 0] = np.nan
    xs[11] = 0.0
    x = torch.from_numpy(xs).cuda()
    y = torch.zeros(n_inst, 128, device="cuda")
    torch.cuda.synchronize()
    group = LayerGroup(gpu_ctx, [layer] * n_inst, x.data_ptr(), y.data_ptr())
    group.apply()
    gpu_ctx.synchronize()
    got = y.cpu().numpy()
    assert np.isnan(got[3]).all() and np.isnan(got[9]).all()
    assert np.array_equal(got[11], np.zeros(128, np.float32))
    assert np.array_equal(got[0], layer.apply(L["x"]))
    assert np.array_equal(got[149], got[0])
    group.close()


@pytest.mark.parametrize("serving", ["float32", "bfloat16"])
def test_plan_of_mixed_shapes_and_gated_input(gpu_ctx, serving):
    """q beside k and v in one plan although their shapes differ, and a plan whose input is
    SwiGLU(gate, up): both must give the bits of the plain single-layer calls."""
    import torch
    from quantibbler_b200.gpu import LayerPlan
    din = 1100
    shapes = [(520, 300), (130, 70), (130, 70)]   # (dout, r): "q", "k", "v"
    specs = [make_layer(dout, din, r, seed=60 + i, with_bias=(i == 1)) for i, (dout, r) in enumerate(shapes)]
    layers = [PackedLayer(gpu_ctx, s["ub_rows"], s["vb_t_rows"], s["dout"], din, s["r"], s["s1"],
                          s["s2"], s["bias"], serving=serving) for s in specs]
    rng = np.random.default_rng(8)
    n_tok = 2
    xs = rng.standard_normal((n_tok, din)).astype(np.float32)
    x = torch.from_numpy(xs).cuda()
    outs = [torch.full((n_tok, s["dout"]), float("nan"), device="cuda") for s in specs]
    torch.cuda.synchronize()
    plan = LayerPlan(gpu_ctx, [(layers[i], x[b].data_ptr(), outs[i][b].data_ptr())
                               for b in range(n_tok) for i in range(3)])
    plan.apply()
    gpu_ctx.synchronize()
    for i in range(3):
        for b in range(n_tok):
            assert np.array_equal(outs[i][b].cpu().numpy(), layers[i].apply(xs[b])), (i, b)
    # gated: "down" applied to SwiGLU(gate, up)
    L = make_layer(96, 700, 130, seed=70)
    down = PackedLayer(gpu_ctx, L["ub_rows"], L["vb_t_rows"], 96, 700, 130, L["s1"], L["s2"], None,
                       serving=serving)
    gate = rng.standard_normal((n_tok, 700)).astype(np.float32) * 3
    up = rng.standard_normal((n_tok, 700)).astype(np.float32)
    tg, tu = torch.from_numpy(gate).cuda(), torch.from_numpy(up).cuda()
    y = torch.full((n_tok, 96), float("nan"), device="cuda")
    torch.cuda.synchronize()
    gated = LayerPlan(gpu_ctx, [(down, tg[b].data_ptr(), tu[b].data_ptr(), y[b].data_ptr())
                                for b in range(n_tok)], gated=True)
    gated.apply()
    gpu_ctx.synchronize()
    act = (tg * tu / (1.0 + torch.exp(-tg))).cpu().numpy()   # float32, the order the kernels use
    for b in range(n_tok):
        want = down.apply(act[b])
        got = y[b].cpu().numpy()
        # torch's exp and the device's expf may differ in the last bit of an activation
        assert np.abs(got - want).max() <= 1e-5 * np.abs(want).max() + (2e-2 * np.abs(want).max() if serving == "bfloat16" else 0)
        ref = oracle.layer_apply(L["ub_rows"], L["vb_t_rows"], 96, 700, 130, L["s1"], L["s2"], None,
                                 act[b], serving=serving)
        assert np.abs(got - ref).max() <= (2e-5 if serving == "float32" else 2e-2) * np.abs(ref).max()
    # too many instances of different shapes do not fit the few-instance form
    with pytest.raises(ValueError, match="few-instance form"):
        big = [(layers[i % 3], x[0].data_ptr(), outs[i % 3][0].data_ptr()) for i in range(3000)]
        LayerPlan(gpu_ctx, big)


def test_multi_token_apply(gpu_ctx):
    import torch
    L = make_layer(96, 160, 72, seed=11, with_bias=True)
    layer = PackedLayer(gpu_ctx, L["ub_rows"], L["vb_t_rows"], 96, 160, 72, L["s1"], L["s2"],
                        L["bias"])
    rng = np.random.default_rng(4)
    xs = rng.standard_normal((7, 160)).astype(np.float32)
    want = np.stack([layer.apply(x) for x in xs])
    x = torch.from_numpy(xs).cuda()
    y = torch.zeros(7, 96, device="cuda")
    torch.cuda.synchronize()
    layer.apply_device(x.data_ptr(), 7, y.data_ptr())
    gpu_ctx.synchronize()
    assert np.array_equal(y.cpu().numpy(), want)


def test_nonfinite_input_gives_nan(gpu_ctx):
    L = make_layer(32, 40, 16, seed=5)
    layer = PackedLayer(gpu_ctx, L["ub_rows"], L["vb_t_rows"], 32, 40, 16, L["s1"], L["s2"])
    x = L["x"].copy()
    x[3] = np.inf
    assert np.isnan(layer.apply(x)).all()
    x[3] = np.nan
    assert np.isnan(layer.apply(x)).all()
    assert np.array_equal(layer.apply(np.zeros(40, np.float32)), np.zeros(32, np.float32))


def test_extreme_dynamic_range(gpu_ctx):
    # one huge entry among tiny ones: the fixed-point grid is set by the largest entry
    L = make_layer(64, 512, 48, seed=9)
    x = (L["x"] * 1e-6).astype(np.float32)
    x[7] = 3.0e4
    L["x"] = x
    # rows cancel almost completely here, so the reference's float64 loop is itself only
    # accurate to ~1e-12 of the term scale and bit identity is not expected
    check_layer(gpu_ctx, L, "float32", expect_bit_identical=False)


def test_layer_validation(gpu_ctx):
    L = make_layer(16, 24, 8, seed=1)
    with pytest.raises(ValueError, match="bitplane length mismatch after repack"):
        PackedLayer(gpu_ctx, L["ub_rows"][:-1], L["vb_t_rows"], 16, 24, 8, L["s1"], L["s2"])
    layer = PackedLayer(gpu_ctx, L["ub_rows"], L["vb_t_rows"], 16, 24, 8, L["s1"], L["s2"])
    with pytest.raises(ValueError, match="expects input dim 24, got 23"):
        layer.apply(np.zeros(23, np.float32))


def test_host_layer_group_matches_per_layer_host_apply(gpu_ctx):
    # one upload, the group's launches, one download: same numbers as PackedLayer.apply per layer
    import torch
    from quantibbler_b200.gpu import HostLayerGroup
    specs = [make_layer(192, 256, 64, seed=900 + i) for i in range(9)]
    layers = [PackedLayer(gpu_ctx, s["ub_rows"], s["vb_t_rows"], 192, 256, 64, s["s1"], s["s2"],
                          None) for s in specs]
    x_host = torch.from_numpy(np.stack([s["x"] for s in specs])).pin_memory()
    y_host = torch.empty((9, 192), dtype=torch.float32).pin_memory()
    step = HostLayerGroup(gpu_ctx, layers)
    for _ in range(2):       # the device buffers are reused
        y_host.zero_()
        step.apply(x_host, y_host)
        for i, layer in enumerate(layers):
            assert np.array_equal(y_host[i].numpy(), layer.apply(specs[i]["x"])), i
    pageable = torch.empty((9, 192), dtype=torch.float32)
    step.apply(x_host.clone(), pageable)            # ordinary host memory works too
    assert np.array_equal(pageable.numpy(), y_host.numpy())
    with pytest.raises(KernelError, match="host buffers must be"):
        step.apply(x_host[:3], y_host)
    step.close()


@pytest.mark.parametrize("serving", ["float32", "bfloat16"])
@pytest.mark.parametrize("din", [8192, 9000, 14336])
def test_long_input_vector_in_the_few_instance_form(gpu_ctx, serving, din):
    """A single instance over a long input (8192 entries and more, the down projection's kind):
    its digit table is built once, by a thread-block cluster that shares out the k-steps, and the
    stage's blocks only stream.  Ragged lengths (a partial k-step, a partial last CTA), plain and
    through the SwiGLU, against the oracle; non-finite input gives NaN."""
    import torch
    from quantibbler_b200.gpu import LayerPlan
    dout, r = 200, 150
    L = make_layer(dout, din, r, seed=din % 97, with_bias=True)
    y, want = check_layer(gpu_ctx, L, serving, expect_bit_identical=False)
    layer = PackedLayer(gpu_ctx, L["ub_rows"], L["vb_t_rows"], dout, din, r, L["s1"], L["s2"], L["bias"],
                        serving=serving)
    rng = np.random.default_rng(din)
    gate = (rng.standard_normal(din) * 3).astype(np.float32)
    up = rng.standard_normal(din).astype(np.float32)
    tg, tu = torch.from_numpy(gate).cuda(), torch.from_numpy(up).cuda()
    out = torch.full((dout,), float("nan"), device="cuda")
    torch.cuda.synchronize()
    gated = LayerPlan(gpu_ctx, [(layer, tg.data_ptr(), tu.data_ptr(), out.data_ptr())], gated=True)
    gated.apply()
    gpu_ctx.synchronize()
    act = (tg * tu / (1.0 + torch.exp(-tg))).cpu().numpy()
    ref = oracle.layer_apply(L["ub_rows"], L["vb_t_rows"], dout, din, r, L["s1"], L["s2"], L["bias"], act,
                             serving=serving)
    got = out.cpu().numpy()
    assert np.abs(got - ref).max() <= (2e-5 if serving == "float32" else 2e-2) * np.abs(ref).max()
    bad = L["x"].copy()
    bad[din - 3] = np.inf
    assert np.isnan(layer.apply(bad)).all()
    layer.close()


@pytest.mark.parametrize("shape", [(5, 7), (4, 16), (9, 35), (300, 129), (257, 1000), (4096, 1024),
                                   (1, 1), (130, 515)])
def test_container_repack_on_the_device(gpu_ctx, shape):
    # engine/mod.rs:258-289: rows of the matrix and rows of its transpose from the container's
    # unpadded bit stream, byte for byte what the host functions and the restatement give
    n_rows, r = shape
    rng = np.random.default_rng(n_rows * 131 + r)
    bits = rng.random((n_rows, r)) < 0.5
    stream = np.packbits(bits.ravel(), bitorder="little")
    assert np.array_equal(gpu_ctx.container_to_rows(stream, n_rows, r),
                          oracle.container_to_rows(stream, n_rows, r))
    assert np.array_equal(gpu_ctx.container_to_rows(stream, n_rows, r, transposed=True),
                          oracle.container_to_rows_transposed(stream, n_rows, r))
    # a wrong length is refused with the host function's text
    with pytest.raises(KernelError, match="container stream holds"):
        gpu_ctx.container_to_rows(np.append(stream, np.uint8(0)), n_rows, r)


@pytest.mark.parametrize("serving", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(96, 160, 72), (130, 1100, 515), (1024, 4096, 1000)])
def test_layer_from_container_streams_equals_layer_from_rows(gpu_ctx, shape, serving):
    # the same layer, bit for bit, whether the host or the device separates the rows
    dout, din, r = shape
    L = make_layer(dout, din, r, seed=dout + r, with_bias=True)
    ub_stream = np.packbits(L["ub"].ravel(), bitorder="little")   # dout x r, no padding
    vb_stream = np.packbits(L["vb"].ravel(), bitorder="little")   # din x r
    a = PackedLayer(gpu_ctx, L["ub_rows"], L["vb_t_rows"], dout, din, r, L["s1"], L["s2"],
                    L["bias"], serving=serving)
    b = PackedLayer.from_container(gpu_ctx, ub_stream, vb_stream, dout, din, r, L["s1"], L["s2"],
                                   L["bias"], serving=serving)
    x = np.stack([L["x"], -0.5 * L["x"][::-1]])
    ya = np.stack([a.apply(v) for v in x])
    yb = np.stack([b.apply(v) for v in x])
    assert np.array_equal(ya, yb)
    want = oracle.layer_apply(L["ub_rows"], L["vb_t_rows"], dout, din, r, L["s1"], L["s2"],
                              L["bias"], x[0], serving=serving)
    assert np.abs(yb[0] - want).max() <= (2e-3 if serving == "float32" else 2e-2) * np.abs(want).max()
    with pytest.raises(KernelError, match="container stream holds"):
        PackedLayer.from_container(gpu_ctx, ub_stream[:-1], vb_stream, dout, din, r, L["s1"],
                                   L["s2"], L["bias"], serving=serving)
    a.close()
    b.close()
