"""The allocation-free layer apply (qk_layer_apply_noalloc) against qk_layer_apply.

Some hosts cannot let this library call cudaMalloc: a server that has already given the
rest of device memory to its KV cache, or a request thread that must stay clear of
cudaMalloc's device-wide synchronisation.  For them one entry point keeps its
intermediates in an array built into the library.  It must give exactly what the
allocating entry point gives (both sum in integers, so the comparison is bit for bit), on
repeated calls that reuse the array, and must refuse layers that do not fit it.

The file name sorts last so that a run which stops at the first failure has already run
every other test.
"""

import ctypes

import numpy as np
import pytest

from conftest import make_layer
from quantibbler_b200 import _lib
from quantibbler_b200.gpu import GpuContext, PackedLayer, apply_noalloc

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("serving", ["float32", "bfloat16"])
def test_noalloc_matches_allocating_apply_on_consecutive_calls(serving):
    import torch
    ctx = GpuContext.init()
    try:
        shapes = [(300, 1100, 515), (4096, 4096, 1024)]
        for dout, din, r in shapes:
            L = make_layer(dout, din, r, seed=dout + r, with_bias=True)
            layer = PackedLayer(ctx, L["ub_rows"], L["vb_t_rows"], dout, din, r, L["s1"], L["s2"],
                                L["bias"], serving=serving)
            rng = np.random.default_rng(din)
            for call in range(2):  # the second call reuses the array the first one wrote
                x = torch.from_numpy(rng.standard_normal(din).astype(np.float32)).cuda()
                want = torch.zeros(dout, device="cuda")
                got = torch.full((dout,), float("nan"), device="cuda")
                torch.cuda.synchronize()
                layer.apply_device(x.data_ptr(), 1, want.data_ptr())
                ctx.synchronize()
                apply_noalloc(layer, x.data_ptr(), got.data_ptr())
                ctx.synchronize()
                assert torch.equal(got, want), (dout, din, r, call)
            layer.close()
    finally:
        ctx.close()


def test_noalloc_refuses_what_does_not_fit():
    ctx = GpuContext.init()
    try:
        L = make_layer(16, 16392, 8, seed=1)  # din above the limit
        layer = PackedLayer(ctx, L["ub_rows"], L["vb_t_rows"], 16, 16392, 8, L["s1"], L["s2"])
        with pytest.raises(ValueError, match="exceeds the built-in scratch"):
            apply_noalloc(layer, 0, 0)
        status = _lib.lib().qk_layer_apply_noalloc(None, layer.handle, None, None)
        assert status == _lib.QK_ERR_VALUE and "existing context" in _lib.last_error()
    finally:
        ctx.close()
