"""One context called from several host threads at once.

The reference's server calls the kernels from its request threads, up to
``--max-concurrency`` (default 4) at a time, through ``&self`` methods of one ``GpuContext``
(crates/quantibbler-server/src/engine/mod.rs:299-309,1021-1023).  The library serialises the
calls of a context internally, and the last error text is per thread.  Here four threads mix
products, the resident layer apply, exact and Sage attention and deliberately refused calls
on one context; every result must equal the one a single thread gets, and a refusal's text
must be the caller's own.
"""

import threading

import numpy as np
import pytest

from conftest import make_layer
from quantibbler_b200 import kernels
from quantibbler_b200._lib import KernelError
from quantibbler_b200.gpu import AttentionShape, PackedLayer

pytestmark = pytest.mark.gpu


def test_four_threads_share_one_context(gpu_ctx):
    rng = np.random.default_rng(77)
    jobs = []

    # float64 device product (GpuContext::packed_matvec)
    packed = rng.integers(0, 256, size=(300, 40), dtype=np.uint8)
    vec = rng.standard_normal(320)
    jobs.append(lambda: gpu_ctx.packed_matvec(packed, 300, 320, vec))
    # dtype-tagged matmul through the Python face (default context of the library)
    mat = rng.standard_normal((320, 5)).astype(np.float32)
    jobs.append(lambda: kernels.packed_matmul_dtype(packed, 320, mat, "float32"))
    # resident factorized layer
    lay = make_layer(192, 256, 64, seed=78, with_bias=True)
    layer = PackedLayer(gpu_ctx, lay["ub_rows"], lay["vb_t_rows"], 192, 256, 64, lay["s1"],
                        lay["s2"], lay["bias"])
    x = rng.standard_normal(256).astype(np.float32)
    jobs.append(lambda: layer.apply(x))
    # exact and Sage attention
    sh = AttentionShape(1, 4, 2, 96, 96, 32, 32)
    q = rng.standard_normal((1, 4, 96, 32)).astype(np.float32)
    k = rng.standard_normal((1, 2, 96, 32)).astype(np.float32)
    v = rng.standard_normal((1, 2, 96, 32)).astype(np.float32)
    jobs.append(lambda: gpu_ctx.attention(sh, q, k, v, True))
    jobs.append(lambda: gpu_ctx.attention_sage(sh, q, k, v, True, 32))

    serial = [job() for job in jobs]
    failures = []
    barrier = threading.Barrier(4)

    def worker(tid):
        try:
            barrier.wait(timeout=30)
            for it in range(12):
                j = (tid + it) % len(jobs)
                got = jobs[j]()
                if not np.array_equal(got, serial[j]):
                    failures.append(f"thread {tid} job {j} iteration {it}: result differs")
                # a refused call: the text must be this thread's, whatever the others do
                n = 7 + tid
                try:
                    gpu_ctx.packed_matvec(packed, 300, 320, vec[:n])
                    failures.append(f"thread {tid}: the short vector was accepted")
                except KernelError as e:
                    if str(e) != f"vec must have length 320, got {n}":
                        failures.append(f"thread {tid}: foreign error text {e}")
        except Exception as e:  # noqa: BLE001
            failures.append(f"thread {tid}: {type(e).__name__}: {e}")

    threads = [threading.Thread(target=worker, args=(t,)) for t in range(4)]
    for t in threads:
        t.start()
    for t in threads:
        t.join(timeout=120)
    assert not any(t.is_alive() for t in threads), "a thread did not finish"
    assert not failures, failures[:5]
    layer.close()
