"""The inputs and expected values of tests/abi/gpu_abi.c, rebuilt in Python.

The C program draws its inputs from a 64-bit linear congruential generator; this module
draws the same stream and computes the expected results with the oracle, so that the C
file's own arithmetic can be checked on a machine without a GPU (it prints two checksums
before it looks for a device)."""

import numpy as np

import oracle

ROWS, BITS, DOUT, DIN, RANK = 37, 75, 48, 80, 24
_MASK = (1 << 64) - 1


class Lcg:
    def __init__(self):
        self.state = 0x243F6A8885A308D3

    def next(self) -> int:
        self.state = (self.state * 6364136223846793005 + 1442695040888963407) & _MASK
        return self.state >> 33

    def unit(self) -> float:
        return self.next() / 2147483648.0 * 2.0 - 1.0

    def rows(self, n_rows, n_bits):
        words = (n_bits + 7) // 8
        out = np.zeros((n_rows, words), np.uint8)
        for i in range(n_rows):
            for j in range(words):
                b = self.next() & 0xFF
                valid = n_bits - 8 * j
                if valid < 8:
                    b &= (1 << valid) - 1
                out[i, j] = b
        return out


def expected_checksums():
    g = Lcg()
    packed = g.rows(ROWS, BITS)
    vec = np.array([g.unit() for _ in range(BITS)], np.float64)
    ub_rows = g.rows(DOUT, RANK)
    vb_t_rows = g.rows(RANK, DIN)
    s1 = np.array([np.float32(0.001 + 0.02 * abs(g.unit())) for _ in range(DOUT)], np.float32)
    s2 = np.array([np.float32(0.001 + 0.02 * abs(g.unit())) for _ in range(DIN)], np.float32)
    bias = np.array([np.float32(0.1 * g.unit()) for _ in range(DOUT)], np.float32)
    x = np.array([np.float32(g.unit()) for _ in range(DIN)], np.float32)
    mv = oracle.packed_matvec(packed, BITS, vec, "float64")
    y = oracle.layer_apply(ub_rows, vb_t_rows, DOUT, DIN, RANK, s1, s2, bias, x)
    sum_mv = 0.0
    for i, v in enumerate(mv.tolist()):
        sum_mv += v * (i + 1)
    sum_y = 0.0
    for i, v in enumerate(y.astype(np.float64).tolist()):
        sum_y += v * (i + 1)
    return sum_mv, sum_y
