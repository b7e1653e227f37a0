// The table-free ("direct") product of packed sign rows with a few vector columns, as device
// code shared by the small-plan GEMV kernel and by the whole-step decode kernel.
//
// One or a few tokens through a layer (single-token decode): the cost of a stage is not its
// weight bits but the chain of dependent steps a block runs before it can multiply.  The
// bit-sliced form's chain is: read the vector, reduce max|v|, quantise, build the digit table,
// multiply, recombine.  This form has no table and no reduction over the vector:
//   * the weight bits are expanded to bfloat16 +-1 in registers, two bits per A-fragment
//     register (a field extract, a multiply that moves the two bits to the sign positions of
//     the two halves, one LOP3), for mma.sync.m16n8k16 with float32 accumulation;
//   * the vector is the B operand, as up to eight columns: under bfloat16 serving one column
//     per token, z = bf16(s2 * x) (exactly the operands and the float32 accumulation of the
//     reference's apply_bf16, engine/mod.rs:449-460); under float32 serving three columns per
//     token, the bfloat16 terms hi + mid + lo that reproduce the float32 value to 2^-25,
//     added up after the contraction.
// Accumulation is float32 in an order that depends on the shape alone (k-steps dealt to four
// k-lanes, the k-lanes' partial sums added in order), so results are reproducible and the
// same wherever this code is used; against the exact sum the error stays inside the
// reference's float32 bound (1e-6 * sum|v_k|, tests/parity.rs:795).  It is NOT the bit-sliced
// form's exact integer sum, which is why only callers that opt in use it.
//
// Geometry: a block of 512 threads = 16 warps = 4 k-lanes x 4 row tiles works on one row group
// (64 rows) at a time.  Warp w owns tile w % 4 of the group and the k-steps w / 4, w / 4 + 4, ...
// and streams its 1 KB tiles through a private four-deep cp.async ring.
#pragma once

#include <cstdint>

namespace qk_direct {

constexpr int kThreads = 512;
constexpr int kKLanes = 4, kTiles = 4;   // kThreads / 32 = kKLanes * kTiles
constexpr int kStages = 4;               // ring depth per warp, in tiles
constexpr int kTileBytes = 1024, kChunkBytes = kTiles * kTileBytes;
constexpr int kGroupRows = 64, kStepBits = 512;
constexpr int kMaxCols = 8;              // columns of the MMA's B operand
constexpr int kPadShift = 7;             // 4 elements of padding per 128: the four t-lanes hit different banks

__host__ __device__ inline uint32_t padded_index(uint32_t k) { return k + 4 * (k >> kPadShift); }
// Elements between two columns of the staged vector (a multiple of 16; the +16 lets
// consecutive columns start on different banks).
__host__ __device__ inline uint32_t column_stride(uint32_t n_steps) {
    return padded_index(n_steps * kStepBits) + 16;
}
__host__ __device__ inline size_t ring_bytes() { return (size_t)(kThreads / 32) * kStages * kTileBytes; }
__host__ __device__ inline size_t red_bytes() { return (size_t)kKLanes * kGroupRows * kMaxCols * sizeof(float); }
// Shared memory of a block whose widest input has n_steps k-steps and n_cols columns.
__host__ __device__ inline size_t smem_bytes(uint32_t n_steps, uint32_t n_cols) {
    return (size_t)n_cols * column_stride(n_steps) * 2 + ring_bytes() + red_bytes();
}

struct Smem {
    uint16_t *cols;   // [n_cols][stride] bfloat16
    uint8_t *ring;    // [warp][kStages][kTileBytes]
    float *red;       // [k-lane][row 0..63][column 0..7]
    uint32_t stride;
};
__device__ __forceinline__ Smem carve(uint8_t *base, uint32_t n_steps_max, uint32_t n_cols_max) {
    Smem s;
    s.stride = column_stride(n_steps_max);
    s.cols = reinterpret_cast<uint16_t *>(base);
    s.ring = base + (size_t)n_cols_max * s.stride * 2;
    s.red = reinterpret_cast<float *>(s.ring + ring_bytes());
    return s;
}

__device__ __forceinline__ void cp16(void *smem, const void *gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem)),
                 "l"(gmem)
                 : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void mma_bf16_f32(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Bits `pos`, `pos + 1` of w as two bfloat16 values (+1.0 for a set bit, -1.0 otherwise), the
// lower bit in the low half.
__device__ __forceinline__ uint32_t signs_bf16x2(uint32_t w, int pos) {
    const uint32_t two = (w >> pos) & 3u;
    // bit 0 -> bit 15 (and bit 30), bit 1 -> bit 31 (and bit 16): keep the two sign positions
    return ((two * 0x40008000u) & 0x80008000u) ^ 0xBF80BF80u;
}
__device__ __forceinline__ float round_to_bf16(float v) {
    uint32_t u = __float_as_uint(v);
    if ((u & 0x7fffffffu) > 0x7f800000u) return __uint_as_float((u | 0x00400000u) & 0xffff0000u);
    u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;
    return __uint_as_float(u);
}
__device__ __forceinline__ uint16_t bf16_bits(float v) { return (uint16_t)(__float_as_uint(round_to_bf16(v)) >> 16); }

// Columns per token: one (the value rounded to bfloat16) or three (its bfloat16 split).
template <bool kRoundBf16> struct Terms { static constexpr int kN = kRoundBf16 ? 1 : 3; };

// Puts element k of token `tok`'s vector into the staged columns.
template <bool kRoundBf16>
__device__ __forceinline__ void stage_value(const Smem &s, uint32_t tok, uint32_t k, float v) {
    const uint32_t at = padded_index(k);
    uint16_t *col = s.cols + (size_t)tok * Terms<kRoundBf16>::kN * s.stride + at;
    if (kRoundBf16) {
        col[0] = bf16_bits(v);
    } else {
        const uint16_t hi = bf16_bits(v);
        const float r1 = v - __uint_as_float((uint32_t)hi << 16);
        const uint16_t mid = bf16_bits(r1);
        const float r2 = r1 - __uint_as_float((uint32_t)mid << 16);
        col[0] = hi;
        col[s.stride] = mid;
        col[2 * s.stride] = bf16_bits(r2);
    }
}

// Four consecutive elements k .. k + 3 (k a multiple of 4) of token `tok`'s vector.
template <bool kRoundBf16>
__device__ __forceinline__ void stage_four(const Smem &s, uint32_t tok, uint32_t k, float4 v) {
    const uint32_t at = padded_index(k);  // k .. k + 3 share a padding group
    uint16_t *col = s.cols + (size_t)tok * Terms<kRoundBf16>::kN * s.stride + at;
    const float in[4] = {v.x, v.y, v.z, v.w};
    uint16_t hi[4], mid[4], lo[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        hi[e] = bf16_bits(in[e]);
        if (!kRoundBf16) {
            const float r1 = in[e] - __uint_as_float((uint32_t)hi[e] << 16);
            mid[e] = bf16_bits(r1);
            lo[e] = bf16_bits(r1 - __uint_as_float((uint32_t)mid[e] << 16));
        }
    }
    *reinterpret_cast<uint2 *>(col) = make_uint2(hi[0] | ((uint32_t)hi[1] << 16), hi[2] | ((uint32_t)hi[3] << 16));
    if (!kRoundBf16) {
        *reinterpret_cast<uint2 *>(col + s.stride) =
            make_uint2(mid[0] | ((uint32_t)mid[1] << 16), mid[2] | ((uint32_t)mid[3] << 16));
        *reinterpret_cast<uint2 *>(col + 2 * s.stride) =
            make_uint2(lo[0] | ((uint32_t)lo[1] << 16), lo[2] | ((uint32_t)lo[3] << 16));
    }
}

// Stages token `tok`'s vector of n_bits elements (zero beyond, up to n_steps k-steps).  All of a
// thread's loads are issued before any value is used, so the whole vector costs one memory
// round trip per 4096 elements (scalar form) or per 16384 (vector form), not one per element.
//   value(k)  -> float   element k, k < n_bits
//   value4(k) -> float4  elements k .. k + 3; only called when `vector_ok` (n_bits a multiple
//                        of 4 and the sources 16-byte aligned), with k + 3 < n_bits
template <bool kRoundBf16, class Value, class Value4>
__device__ __forceinline__ void stage_vector(const Smem &s, uint32_t tok, uint32_t n_bits, uint32_t n_steps,
                                             bool vector_ok, Value value, Value4 value4) {
    const uint32_t padded = n_steps * kStepBits;
    constexpr int kBatch = 8;
    if (vector_ok) {
        for (uint32_t base = 0; base < padded; base += kBatch * 4 * kThreads) {
            float4 v[kBatch];
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
                const uint32_t k = base + 4 * (threadIdx.x + i * kThreads);
                v[i] = k < n_bits ? value4(k) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
                const uint32_t k = base + 4 * (threadIdx.x + i * kThreads);
                if (k < padded) stage_four<kRoundBf16>(s, tok, k, v[i]);
            }
        }
    } else {
        for (uint32_t base = 0; base < padded; base += kBatch * kThreads) {
            float v[kBatch];
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
                const uint32_t k = base + threadIdx.x + i * kThreads;
                v[i] = k < n_bits ? value(k) : 0.f;
            }
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
                const uint32_t k = base + threadIdx.x + i * kThreads;
                if (k < padded) stage_value<kRoundBf16>(s, tok, k, v[i]);
            }
        }
    }
}

// One row group of one packed factor: tiles of 16 rows x 512 bits, four per 4 KB chunk,
// chunks ordered [group][k-step].
struct Work {
    const uint8_t *tiles;
    uint32_t n_steps, group;
};

// This warp's share of the k-steps.
__device__ __forceinline__ uint32_t warp_items(uint32_t n_steps) {
    const uint32_t kl = (threadIdx.x / 32) / kTiles;
    return kl < n_steps ? (n_steps - kl + kKLanes - 1) / kKLanes : 0;
}
__device__ __forceinline__ void issue_tile(const Smem &s, const Work &w, uint32_t i, uint32_t n_items) {
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t m = warp % kTiles, kl = warp / kTiles;
    if (i < n_items) {
        uint4 *dst = reinterpret_cast<uint4 *>(s.ring + ((size_t)warp * kStages + i % kStages) * kTileBytes) + lane;
        const uint4 *from = reinterpret_cast<const uint4 *>(w.tiles) +
                            ((size_t)w.group * w.n_steps + kl + (size_t)i * kKLanes) * (kChunkBytes / 16) +
                            m * (kTileBytes / 16) + lane;
        cp16(dst, from);            // row g:     bits 128 t .. 128 t + 127 of the k-step
        cp16(dst + 32, from + 32);  // row g + 8
    }
    cp_commit();  // (an empty group keeps the group count in step with i)
}
// Starts the first copies of a row group.  The weight bits depend on nothing a kernel or an
// earlier phase computes, so this may run before the wait for the input vector.
__device__ __forceinline__ void prefetch(const Smem &s, const Work &w) {
    const uint32_t n_items = warp_items(w.n_steps);
#pragma unroll
    for (int st = 0; st < kStages - 1; ++st) issue_tile(s, w, st, n_items);
}

// Multiplies the row group with the staged columns (n_cols <= 8) and leaves, for every row of
// the group and column c, the k-lanes' partial sums in s.red.  prefetch(s, w) must have been
// called by every thread, and the columns must be staged and visible (a block barrier after the
// staging).  Ends with a block barrier: s.red is complete, the ring is free.
__device__ __forceinline__ void multiply(const Smem &s, const Work &w, uint32_t n_cols) {
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t m = warp % kTiles, kl = warp / kTiles;
    const uint32_t g = lane / 4, t = lane % 4;
    const uint32_t n_items = warp_items(w.n_steps);
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    // lane (g, t) feeds column g of B (columns beyond n_cols are zero)
    const uint16_t *my_col = s.cols + (size_t)min(g, n_cols - 1) * s.stride;
    const bool live_col = g < n_cols;
    const uint4 *ring = reinterpret_cast<const uint4 *>(s.ring + (size_t)warp * kStages * kTileBytes) + lane;
    for (uint32_t i = 0; i < n_items; ++i) {
        issue_tile(s, w, i + kStages - 1, n_items);
        cp_wait<kStages - 1>();
        const uint4 *stage = ring + (size_t)(i % kStages) * (kTileBytes / 16);
        const uint4 lo = stage[0], hi = stage[32];
        const uint32_t ks = kl + i * kKLanes;
        const uint16_t *bsrc = my_col + padded_index(ks * kStepBits + 128 * t);  // the lane's 128 k
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t wg = q == 0 ? lo.x : q == 1 ? lo.y : q == 2 ? lo.z : lo.w;
            const uint32_t wh = q == 0 ? hi.x : q == 1 ? hi.y : q == 2 ? hi.z : hi.w;
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
                // this MMA contracts the lane's k 32 q + 4 jj .. + 3 (and the other t-lanes'
                // counterparts): B holds the column's four values there
                uint2 b = *reinterpret_cast<const uint2 *>(bsrc + 32 * q + 4 * jj);
                if (!live_col) b = make_uint2(0u, 0u);
                mma_bf16_f32(acc, signs_bf16x2(wg, 4 * jj), signs_bf16x2(wh, 4 * jj),
                             signs_bf16x2(wg, 4 * jj + 2), signs_bf16x2(wh, 4 * jj + 2), b.x, b.y);
            }
        }
    }
    cp_wait<0>();
    // lane (g, t) holds columns 2t, 2t + 1 of rows g (acc[0..1]) and g + 8 (acc[2..3])
    float *mine = s.red + ((size_t)kl * kGroupRows + m * 16 + g) * kMaxCols + 2 * t;
    *reinterpret_cast<float2 *>(mine) = make_float2(acc[0], acc[1]);
    *reinterpret_cast<float2 *>(mine + 8 * kMaxCols) = make_float2(acc[2], acc[3]);
    __syncthreads();
}
// Row `row` (0..63) of the group against token `tok`: the terms' columns added, then the
// k-lanes in order.
template <bool kRoundBf16>
__device__ __forceinline__ float gather(const Smem &s, uint32_t row, uint32_t tok) {
    constexpr int kN = Terms<kRoundBf16>::kN;
    float sum = 0.f;
#pragma unroll
    for (int kl = 0; kl < kKLanes; ++kl) {
        const float *c = s.red + ((size_t)kl * kGroupRows + row) * kMaxCols + tok * kN;
        sum += kN == 1 ? c[0] : (c[0] + c[1]) + c[2];
    }
    return sum;
}

}  // namespace qk_direct
