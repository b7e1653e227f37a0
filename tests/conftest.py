import json
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


class Golden:
    """One golden family: arrays from <name>.npz, scalars from <name>.json."""

    def __init__(self, name):
        self.arrays = np.load(os.path.join(GOLDEN, name + ".npz"))
        with open(os.path.join(GOLDEN, name + ".json")) as f:
            self.meta = json.load(f)

    def __getitem__(self, key):
        return self.arrays[key]

    def has(self, key):
        return key in self.arrays.files

    def cases(self, prefix=""):
        return sorted(k for k in self.meta if k.startswith(prefix))


_cache = {}


def golden(name):
    if name not in _cache:
        _cache[name] = Golden(name)
    return _cache[name]


@pytest.fixture(scope="session")
def gpu_ctx():
    from quantibbler_b200.gpu import GpuContext
    ctx = GpuContext.init()
    yield ctx
    ctx.close()


def make_layer(dout, din, r, seed, with_bias=False):
    """The generator tests/golden/make_golden.py used for the layer family."""
    rng = np.random.default_rng(seed)
    ub = rng.random((dout, r)) < 0.5
    vb = rng.random((din, r)) < 0.5
    s1 = (np.abs(rng.standard_normal(dout)) * 0.02 + 1e-3).astype(np.float32)
    s2 = (np.abs(rng.standard_normal(din)) * 0.02 + 1e-3).astype(np.float32)
    x = rng.standard_normal(din).astype(np.float32)
    bias = (rng.standard_normal(dout) * 0.1).astype(np.float32) if with_bias else None
    ub_rows = np.packbits(ub, axis=1, bitorder="little")
    vb_t_rows = np.packbits(vb.T, axis=1, bitorder="little")
    return dict(ub_rows=ub_rows, vb_t_rows=vb_t_rows, s1=s1, s2=s2, x=x, bias=bias,
                dout=dout, din=din, r=r, ub=ub, vb=vb)
