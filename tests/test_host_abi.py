"""Host side of the C-ABI library: it loads, exports what the header declares, and its
integer core and error texts match the reference.  No GPU needed, no compute calls."""

import ctypes
import os
import re

import numpy as np
import pytest

from conftest import ROOT, golden
from quantibbler_b200 import _build, _lib, kernels
from quantibbler_b200._lib import DeviceError, KernelError


def header_symbols():
    text = open(os.path.join(ROOT, "include", "qk_kernels.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(qk_[a-z0-9_]+)\s*\(", text)))


def test_library_builds_and_exports_every_declared_symbol():
    path = _build.build()
    handle = ctypes.CDLL(path)
    declared = header_symbols()
    assert len(declared) >= 25
    for name in declared:
        assert hasattr(handle, name), f"{name} declared in qk_kernels.h but not exported"
    assert sorted(_lib.exported_symbols()) == declared


def test_pack_unpack_golden_bytes():
    g = golden("bitplanes")
    for key in g.cases("pack"):
        factor, packed = g[key + "_factor"], g[key + "_packed"]
        n_bits = g.meta[key]["n_bits"]
        if factor.ndim < 2 or factor.shape[-1] != n_bits:
            continue
        got = kernels.pack_bits(factor)
        assert got.dtype == np.uint8 and np.array_equal(got, packed), key
        assert np.array_equal(kernels.pack_bits(factor.astype(np.float64)), packed)
        back = kernels.unpack_bits(packed, n_bits, "int8")
        assert back.dtype == np.int8 and np.array_equal(back, factor)
        assert kernels.unpack_bits(packed, n_bits, "float64").dtype == np.float64


def test_pack_any_dimensionality_and_degenerate_shapes():
    rng = np.random.default_rng(1)
    f = rng.choice(np.array([-1, 1], dtype=np.int8), size=(2, 3, 11))
    p = kernels.pack_bits(f)
    assert p.shape == (6, 2)
    assert np.array_equal(kernels.unpack_bits(p, 11), f.reshape(6, 11))
    assert kernels.pack_bits(np.zeros((2, 0), np.int8)).shape == (2, 0)
    assert kernels.pack_bits(np.zeros((0, 7), np.int8)).shape == (0, 1)
    assert kernels.unpack_bits(np.zeros((3, 0), np.uint8), 0).shape == (3, 0)


def test_error_texts_match_reference():
    # crates/quantibbler-kernels/tests/parity.rs:1062-1081 pins these as values
    with pytest.raises(ValueError, match=r"pack_bits expects values in \{-1, \+1\}; got 0 at row 1, "
                                         r"column 2"):
        kernels.pack_bits(np.array([[1, -1, 1], [1, 1, 0]], dtype=np.int8))
    with pytest.raises(ValueError, match=r"got 1\.0001$"):
        kernels.pack_bits(np.array([[1.0, 1.0001]]))
    with pytest.raises(ValueError, match=r"got 2\.0$"):
        kernels.pack_bits(np.array([[2.0, 1.0]]))
    with pytest.raises(ValueError, match=r"n_bits=17 exceeds the packed width 2 \(16 bits\)"):
        kernels.unpack_bits(np.zeros((1, 2), np.uint8), 17)
    with pytest.raises(ValueError, match=r"unpack_bits dtype must be 'int8' or 'float64'"):
        kernels.unpack_bits(np.zeros((1, 2), np.uint8), 9, "int32")
    lib = _lib.lib()
    n_words = ctypes.c_size_t()
    assert lib.qk_validate_packed(6, 3, 13, ctypes.byref(n_words)) == 0 and n_words.value == 2
    assert lib.qk_validate_packed(5, 3, 13, ctypes.byref(n_words)) == _lib.QK_ERR_VALUE
    assert _lib.last_error() == "packed length 5 does not match 3 rows x 2 bitplanes"
    assert lib.qk_validate_packed(4, 2, 0, ctypes.byref(n_words)) == _lib.QK_ERR_VALUE
    assert _lib.last_error() == "n_bits=0 with non-empty packed rows"
    tag = ctypes.c_int32()
    assert lib.qk_dtype_from_name(b"float16", ctypes.byref(tag)) == _lib.QK_ERR_VALUE
    assert _lib.last_error() == ('unknown kernel dtype "float16"; expected one of "float64", '
                                 '"float32", "bfloat16"')
    for i, name in enumerate(["float64", "float32", "bfloat16"]):
        assert lib.qk_dtype_from_name(name.encode(), ctypes.byref(tag)) == 0 and tag.value == i
        assert lib.qk_dtype_name(i) == name.encode()


def test_product_validation_happens_before_any_device_work():
    # these are refused on the host, so they raise ValueError even without a GPU
    p = np.zeros((6, 2), np.uint8)
    with pytest.raises(ValueError, match=r"vec must have length 13, got 12"):
        kernels.packed_matvec(p, 13, np.zeros(12))
    with pytest.raises(ValueError, match=r"packed length 12 does not match 6 rows x 3 bitplanes"):
        kernels.packed_matvec(p, 17, np.zeros(17))
    with pytest.raises(ValueError, match=r"mat length 25 is not a multiple of n_bits 13"):
        kernels.packed_matmul(p, 13, np.zeros((5, 5)))
    with pytest.raises(ValueError, match=r'unknown kernel dtype "half"'):
        kernels.packed_matvec_dtype(p, 13, np.zeros(13), "half")
    # zero-size work returns zeros without touching a device (gpu.rs:139-143)
    assert kernels.packed_matvec(np.zeros((0, 2), np.uint8), 13, np.zeros(13)).shape == (0,)
    assert np.array_equal(kernels.packed_matvec(np.zeros((3, 0), np.uint8), 0, np.zeros(0)),
                          np.zeros(3))


def test_sign_estimate_host():
    g = golden("bitplanes")
    x = g["sign0_x"]
    assert np.array_equal(kernels.sign_estimate(x), g["sign0_x_signs"].ravel())


def test_container_repack_host():
    import oracle
    rng = np.random.default_rng(8)
    lib = _lib.lib()
    for n_rows, r in [(5, 7), (4, 16), (9, 35)]:
        bits = rng.random((n_rows, r)) < 0.5
        stream = np.packbits(bits.ravel(), bitorder="little")
        out = np.zeros(n_rows * ((r + 7) // 8), np.uint8)
        assert lib.qk_container_to_rows(stream.ctypes.data, stream.size, n_rows, r,
                                        out.ctypes.data, out.size) == 0
        assert np.array_equal(out.reshape(n_rows, -1), oracle.container_to_rows(stream, n_rows, r))
        out_t = np.zeros(r * ((n_rows + 7) // 8), np.uint8)
        assert lib.qk_container_to_rows_transposed(stream.ctypes.data, stream.size, n_rows, r,
                                                   out_t.ctypes.data, out_t.size) == 0
        assert np.array_equal(out_t.reshape(r, -1),
                              oracle.container_to_rows_transposed(stream, n_rows, r))


def test_init_failure_is_typed_and_carries_the_hint():
    # crates/quantibbler-kernels/tests/gpu_attention_parity.rs:183-204: an impossible device
    # index must give a typed error that embeds the staging hint, with or without hardware
    from quantibbler_b200.gpu import GpuContext, gpu_init_hint
    with pytest.raises(DeviceError) as info:
        GpuContext.init_at(2**40)
    assert gpu_init_hint() in str(info.value)
    assert "CUDA" in gpu_init_hint() and "no CPU fallback" in gpu_init_hint()


def test_drop_in_module_exposes_the_reference_names():
    import quantibbler_kernels as qk
    for name in ["backend_version", "pack_bits", "unpack_bits", "sign_estimate", "packed_matvec",
                 "packed_matmul", "packed_matvec_dtype", "packed_matmul_dtype", "joint_itq"]:
        assert callable(getattr(qk, name)), name
    assert isinstance(qk.backend_version(), str)
    assert issubclass(KernelError, ValueError)


def test_joint_itq_golden_signs_iterations_and_flags():
    # crates/quantibbler-kernels/tests/fixtures/joint_itq.json (parity.rs reads it) and seeded
    # cases run through the reference's NumPy face: int8 signs are pinned exactly
    g = golden("joint_itq")
    for key in g.cases("itq"):
        meta = g.meta[key]
        u_t, v_t, n_iter, converged = kernels.joint_itq(g[key + "_u_hat"], g[key + "_v_hat"],
                                                        **meta["kwargs"])
        assert u_t.dtype == np.int8 and v_t.dtype == np.int8
        assert np.array_equal(u_t, g[key + "_u_t"]), meta["scenario"]
        assert np.array_equal(v_t, g[key + "_v_t"]), meta["scenario"]
        assert (n_iter, converged) == (meta["n_iter"], meta["converged"]), meta["scenario"]


def test_joint_itq_matches_oracle_at_compressor_sizes_and_preserves_product():
    # tests/test_kernels_parity.py:273-292 of the reference: every entry is +-1 and the result
    # is a rotation of the inputs' signs, deterministic in the seed
    from oracle import itq_np
    rng = np.random.default_rng(31)
    u_hat = rng.standard_normal((600, 48)) @ rng.standard_normal((48, 48))
    v_hat = rng.standard_normal((420, 48))
    want = itq_np.joint_itq(u_hat, v_hat, max_iter=12, seed=42, return_margin=True)
    got = kernels.joint_itq(u_hat, v_hat, max_iter=12, seed=42)
    assert got[2:] == want[2:4]
    differ = np.concatenate([got[0], got[1]]) != np.concatenate([want[0], want[1]])
    # a sign may differ only where Z R vanishes to rounding (the two SVDs differ in the last bits)
    assert np.all(np.abs(want[4][differ]) < 1e-9)
    assert differ.sum() <= 2
    assert set(np.unique(got[0])) <= {-1, 1} and set(np.unique(got[1])) <= {-1, 1}
    again = kernels.joint_itq(u_hat, v_hat, max_iter=12, seed=42)
    assert np.array_equal(again[0], got[0]) and np.array_equal(again[1], got[1])
    other = kernels.joint_itq(u_hat, v_hat, max_iter=12, seed=7)
    assert not np.array_equal(other[0], got[0])
    # defaults of the PyO3 face: 50 iterations, tolerance 1e-12, seed 0
    a = kernels.joint_itq(u_hat[:40, :6].copy(), v_hat[:30, :6].copy())
    b = kernels.joint_itq(u_hat[:40, :6].copy(), v_hat[:30, :6].copy(), max_iter=50, tol=1e-12,
                          seed=0)
    assert a[2:] == b[2:] and np.array_equal(a[0], b[0]) and np.array_equal(a[1], b[1])


def test_joint_itq_refusals():
    # core.rs:337-346, lib.rs:211-216
    u = np.zeros((4, 3))
    with pytest.raises(KernelError, match="joint_itq rank mismatch: u_hat r=3, v_hat r=2"):
        kernels.joint_itq(u, np.zeros((4, 2)))
    with pytest.raises(KernelError, match="joint_itq expects non-empty factors"):
        kernels.joint_itq(np.zeros((4, 0)), np.zeros((2, 0)))
    with pytest.raises(KernelError, match="joint_itq expects non-empty factors"):
        kernels.joint_itq(np.zeros((0, 3)), np.zeros((0, 3)))
    with pytest.raises(OverflowError):
        kernels.joint_itq(u, u, max_iter=-1)
    with pytest.raises(TypeError):
        kernels.joint_itq(u.astype(np.float32), u)
    lib = _lib.lib()
    out = np.zeros(12, dtype=np.int8)
    n_iter, conv = ctypes.c_size_t(), ctypes.c_int32()
    rc = lib.qk_joint_itq(u.ctypes.data, 11, u.ctypes.data, 12, 4, 4, 3, 5, 1e-12, 0,
                          out.ctypes.data, out.ctypes.data, ctypes.byref(n_iter),
                          ctypes.byref(conv))
    assert rc == _lib.QK_ERR_VALUE
    assert lib.qk_last_error().decode() == "joint_itq shape mismatch: u_hat 4x2, v_hat 4x3"
    # all-zero factors: Z R = 0 everywhere, every sign is +1 (x >= 0), as in the reference
    u_t, v_t, _, _ = kernels.joint_itq(u, u, max_iter=2)
    assert np.all(u_t == 1) and np.all(v_t == 1)


def test_public_header_is_plain_c(tmp_path):
    # the boundary is a C ABI: the header must compile as C99 and as C++ on its own
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    src = tmp_path / "hdr.c"
    src.write_text('#include "qk_kernels.h"\nint main(void) { return 0; }\n')
    inc = os.path.join(ROOT, "include")
    for flags in (["-std=c99", "-pedantic"], ["-x", "c++", "-std=c++17"]):
        res = subprocess.run([gcc, *flags, "-Wall", "-Werror", "-fsyntax-only", "-I", inc, str(src)],
                             capture_output=True, text=True)
        assert res.returncode == 0, res.stderr


def test_c_program_links_and_calls_the_host_entry_points(tmp_path):
    # tests/abi/host_abi.c is a plain C99 caller: it is what a compiled host links against
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    _lib.lib()                      # builds the library only if it is missing
    lib_path = _build.LIB_PATH
    exe = tmp_path / "host_abi"
    res = subprocess.run(
        [gcc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"),
         os.path.join(ROOT, "tests", "abi", "host_abi.c"), "-L", os.path.dirname(lib_path),
         "-lqk_kernels", f"-Wl,-rpath,{os.path.dirname(lib_path)}", "-o", str(exe)],
        capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode == 0, run.stderr
    assert "host ABI ok" in run.stdout


def _build_c_program(tmp_path, name):
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    _lib.lib()                      # builds the library only if it is missing
    lib_path = _build.LIB_PATH
    exe = tmp_path / name
    res = subprocess.run(
        [gcc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-I", os.path.join(ROOT, "include"),
         os.path.join(ROOT, "tests", "abi", name + ".c"), "-L", os.path.dirname(lib_path),
         "-lqk_kernels", "-lm", f"-Wl,-rpath,{os.path.dirname(lib_path)}", "-o", str(exe)],
        capture_output=True, text=True)
    assert res.returncode == 0, res.stderr
    return exe


def test_gpu_c_program_expectations_match_the_oracle(tmp_path):
    # tests/abi/gpu_abi.c prints the checksums of its own expected values before it looks for
    # a device: they must be the oracle's on the same inputs (rebuilt in tests/abi_inputs.py)
    import subprocess

    import abi_inputs
    exe = _build_c_program(tmp_path, "gpu_abi")
    run = subprocess.run([str(exe)], capture_output=True, text=True, timeout=120)
    assert run.returncode in (0, 77), run.stdout + run.stderr   # 77: no usable device
    printed = dict(line.rsplit(" ", 1) for line in run.stdout.splitlines()
                   if line.startswith("expected "))
    want_mv, want_y = abi_inputs.expected_checksums()
    assert float(printed["expected matvec checksum"]) == want_mv
    assert float(printed["expected layer checksum"]) == want_y
    if run.returncode == 77:
        assert "no CPU fallback" in run.stdout


def test_prefill_work_split_invariants():
    """How the tensor-core GEMM deals (tile, k-chunk) units out to its CTAs: every unit goes to
    exactly one CTA, the runs are contiguous and in order, the grid never exceeds the SMs, and
    when there are few tiles every tile goes to a whole number of CTAs in equal parts (at most
    seven unless a run would then exceed sixteen k-chunks)."""
    import ctypes
    lib = _lib.lib()

    def split(tiles, ks, sms=148):
        n = len(tiles)
        t = (ctypes.c_size_t * n)(*tiles)
        k = (ctypes.c_size_t * n)(*ks)
        out = (ctypes.c_uint32 * 200)()
        got = ctypes.c_size_t()
        assert lib.qk_prefill_work_split(n, t, k, sms, out, 200, ctypes.byref(got)) == 0
        return list(out[:got.value + 1])

    rng = np.random.default_rng(11)
    cases = [([9, 4, 4], [64, 64, 64]), ([32, 8, 8], [18, 7, 7]), ([28], [64]), ([14], [224]),
             ([9], [64]), ([224, 224], [27, 27]), ([1], [3]), ([1], [4096]), ([72, 32, 32], [64, 64, 64])]
    for _ in range(200):
        n = int(rng.integers(1, 5))
        cases.append(([int(rng.integers(1, 60)) for _ in range(n)], [int(rng.integers(1, 300)) for _ in range(n)]))
    for tiles, ks in cases:
        for sms in (148, 132, 16):
            b = split(tiles, ks, sms)
            units = sum(t * k for t, k in zip(tiles, ks))
            n_ctas = len(b) - 1
            assert b[0] == 0 and b[-1] == units and 1 <= n_ctas <= sms, (tiles, ks, sms)
            assert all(lo < hi for lo, hi in zip(b, b[1:])), (tiles, ks, sms)   # no empty CTA, in order
            # tile borders in unit space
            borders, at = {0}, 0
            for t, k in zip(tiles, ks):
                for _ in range(t):
                    at += k
                    borders.add(at)
            if 2 * sum(tiles) <= max(1, min(sms, units // 8)) and set(b) >= borders:
                # the aligned form: a tile's sharers have runs that differ by at most one chunk
                at = 0
                for t, k in zip(tiles, ks):
                    for _ in range(t):
                        runs = [hi - lo for lo, hi in zip(b, b[1:]) if at <= lo < at + k]
                        assert sum(runs) == k and max(runs) - min(runs) <= 1, (tiles, ks, sms)
                        assert len(runs) <= 7 or -(-k // 7) > 16, (tiles, ks, sms, len(runs))
                        at += k
    # the decode shapes of the Llama-3-8B-like stack at 64 tokens take the aligned form
    b = split([9, 4, 4], [64, 64, 64])
    assert len(b) - 1 == 17 * 7 and all(hi - lo in (9, 10) for lo, hi in zip(b, b[1:]))
    # refusals
    t1, k1 = (ctypes.c_size_t * 1)(4), (ctypes.c_size_t * 1)(8)
    out, got = (ctypes.c_uint32 * 2)(), ctypes.c_size_t()
    assert lib.qk_prefill_work_split(1, t1, k1, 148, out, 2, ctypes.byref(got)) == _lib.QK_ERR_VALUE
    assert "are needed" in _lib.last_error()
    assert lib.qk_prefill_work_split(0, t1, k1, 148, out, 2, ctypes.byref(got)) == _lib.QK_ERR_VALUE
