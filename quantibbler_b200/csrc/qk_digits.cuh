// The digit-table form of a vector: what the bit-sliced GEMV kernels multiply the weight
// bits with.  Shared by the GEMV kernels (which build tables in shared memory) and by the
// kernels that produce a vector for them (norm, SwiGLU, attention combine), which can write
// the table of their output straight to global memory so that the GEMV blocks only stream.
//
// A vector v is put on a fixed-point grid, v_k ~ q_k * 2^-shift with |q_k| < 2^47 relative
// to max|v|, and q_k * 2^(7-i), i = k mod 8, is split into eight balanced base-256 digits.
// Table layout (uint2 units): record ((ks*4 + q)*4 + ip)*4 + t of k-step ks holds, for digit
// column n, the B-fragment pair of lane (g = n, t) of the MMA that consumes word q under the
// masks 2*ip (b0) and 2*ip+1 (b1); byte j of b0/b1 belongs to k = 512*ks + 128*t + 32*q + 8*j + i.
#pragma once

#include <cstdint>

namespace {

constexpr int kStepBits = 512;      // bits of one row inside one tile
constexpr int kQBits = 46;          // |q_k| < 2^(kQBits+1)

struct StageMeta {
    long long total;  // sum_k q_k
    int shift;        // v_k ~ q_k * 2^-shift
    int nonfinite;    // the input held a NaN or an infinity
};

// What a producing kernel needs to know to write the table of one consumer: z_k = in_scale_k *
// v_k (float32 product, rounded to bfloat16 under bfloat16 serving) for k < n_bits.
struct FeedTarget {
    const float *in_scale;  // s2 of the consuming linear (may be null)
    uint2 *digits;
    StageMeta *meta;
    uint32_t n_bits, n_steps;
};

__device__ __forceinline__ float round_bf16(float v) {
    uint32_t u = __float_as_uint(v);
    if ((u & 0x7fffffffu) > 0x7f800000u) return __uint_as_float((u | 0x00400000u) & 0xffff0000u);
    u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;
    return __uint_as_float(u);
}

// Fixed-point grid of a vector whose largest magnitude is m: |v| * 2^shift < 2^(kQBits+1).
struct FixedPoint {
    int shift;
    bool direct;   // 2^shift is a normal double
    double pow2;
    __device__ __forceinline__ long long quant(double v) const {
        return __double2ll_rn(direct ? v * pow2 : ldexp(v, shift));
    }
};
__device__ __forceinline__ FixedPoint fixed_point_of(double m) {
    int e = 0;
    if (m > 0.0) {
        int biased = (__double2hiint(m) >> 20) & 0x7ff;  // m = f * 2^e, f in [0.5, 1)
        if (biased) e = biased - 1022; else frexp(m, &e);
    }
    FixedPoint fp;
    fp.shift = kQBits + 1 - e;
    fp.direct = fp.shift > -1000 && fp.shift < 1000;
    fp.pow2 = fp.direct ? __hiloint2double((1023 + fp.shift) << 20, 0) : 0.0;
    return fp;
}

// Record rec = (qw*4 + ip)*4 + t of k-step ks: the eight uint2 B-fragment pairs (one per
// digit column) built from the eight vector entries k = 512*ks + 128*t + 32*qw + 8*j + i,
// i in {2*ip, 2*ip+1}, j in 0..3.  q8[which*4 + j] holds their fixed-point values.
__device__ __forceinline__ void build_record(const long long (&q8)[8], uint32_t ip, uint4 *dst) {
    // Balanced base-256 digits without a carry loop: adding 128 to every byte position and
    // flipping each byte's top bit turns the two's-complement bytes into digits in
    // [-128, 127] with sum_n d_n 256^n equal to the value.
    const unsigned long long bias = 0x8080808080808080ull;
    uint32_t w[2][4][2];  // [which][j][low digits 0-3 / high digits 4-7]
#pragma unroll
    for (int which = 0; which < 2; ++which)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            unsigned long long u =
                (((unsigned long long)q8[which * 4 + j] << (7 - (2 * ip + which))) + bias) ^ bias;
            w[which][j][0] = (uint32_t)u;
            w[which][j][1] = (uint32_t)(u >> 32);
        }
    // 4x4 byte transposes: word n of the result holds digit n of the four entries j = 0..3
    uint32_t out[2][8];
#pragma unroll
    for (int which = 0; which < 2; ++which)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const uint32_t a = w[which][0][half], b2 = w[which][1][half];
            const uint32_t c = w[which][2][half], d = w[which][3][half];
            const uint32_t t0 = __byte_perm(a, b2, 0x5140), t1 = __byte_perm(c, d, 0x5140);
            const uint32_t t2 = __byte_perm(a, b2, 0x7362), t3 = __byte_perm(c, d, 0x7362);
            out[which][half * 4 + 0] = __byte_perm(t0, t1, 0x5410);
            out[which][half * 4 + 1] = __byte_perm(t0, t1, 0x7632);
            out[which][half * 4 + 2] = __byte_perm(t2, t3, 0x5410);
            out[which][half * 4 + 3] = __byte_perm(t2, t3, 0x7632);
        }
#pragma unroll
    for (int n = 0; n < 8; n += 2)
        dst[n / 2] = make_uint4(out[0][n], out[1][n], out[0][n + 1], out[1][n + 1]);
}


// The table of one vector, built by a whole block (any size up to 1024 threads) and written
// to `table` (shared or global memory).  entry(k) is element k as float64, zero beyond the
// vector.  red_max, red_sum: 32 entries of shared memory each; red_bad: one int.  Ends with a
// __syncthreads(); thread 0 writes *meta_out.
// Several blocks may share one table: block `part` of `n_parts` scans the whole vector (the
// scale and the sum need all of it, and scanning is cheap) but assembles and stores only its
// own share of the records, which is where the work is; part 0 writes the stage record.
template <typename Entry>
__device__ __forceinline__ void block_build_table(Entry entry, uint32_t n_steps, uint4 *table,
                                                  StageMeta *meta_out, double *red_max,
                                                  long long *red_sum, int *red_bad,
                                                  uint32_t part = 0, uint32_t n_parts = 1) {
    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32, n_warps = (blockDim.x + 31) / 32;
    const uint32_t n_records = n_steps * 64;
    auto record_entry = [&](uint32_t r, int e) -> double {
        const uint32_t ks = r / 64, rec = r % 64;
        const uint32_t tt = rec % 4, ip = (rec / 4) % 4, qw = rec / 16;
        return entry(ks * kStepBits + 128 * tt + 32 * qw + 8 * (e % 4) + 2 * ip + e / 4);
    };
    double mx = 0.0;
    int bad = 0;
    for (uint32_t r = tid; r < n_records; r += blockDim.x)
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const double a = fabs(record_entry(r, e));
            if (!(a <= 1.7e308)) bad = 1;  // NaN or infinity
            mx = fmax(mx, a);
        }
    for (int off = 16; off > 0; off >>= 1) mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if (tid == 0) *red_bad = 0;
    if (lane == 0) red_max[warp] = mx;
    __syncthreads();
    if (bad) *red_bad = 1;
    __syncthreads();
    double m = red_max[0];
    for (uint32_t w = 1; w < n_warps; ++w) m = fmax(m, red_max[w]);
    const int nonfinite = *red_bad;
    const FixedPoint fp = fixed_point_of(nonfinite ? 0.0 : m);
    long long total = 0;
    const uint32_t r_lo = (uint32_t)((uint64_t)n_records * part / n_parts);
    const uint32_t r_hi = (uint32_t)((uint64_t)n_records * (part + 1) / n_parts);
    for (uint32_t r = tid; r < n_records; r += blockDim.x) {
        const bool mine = r >= r_lo && r < r_hi;
        if (!mine && part != 0) continue;  // only part 0 needs the sum over everything
        long long q8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            q8[e] = nonfinite ? 0 : fp.quant(record_entry(r, e));
            total += q8[e];
        }
        if (mine) build_record(q8, (r % 64 / 4) % 4, table + (size_t)r * 4);
    }
    for (int off = 16; off > 0; off >>= 1) total += __shfl_xor_sync(0xffffffffu, total, off);
    if (lane == 0) red_sum[warp] = total;
    __syncthreads();
    if (tid == 0 && part == 0) {
        long long sum = 0;
        for (uint32_t w = 0; w < n_warps; ++w) sum += red_sum[w];
        meta_out->total = sum;
        meta_out->shift = fp.shift;
        meta_out->nonfinite = nonfinite;
    }
    __syncthreads();
}

// ---- the same table without floating-point arithmetic --------------------------------
// fp.quant(v) = round-to-nearest-even(v * 2^shift) of a finite value given by its bits:
// v = (-1)^neg * mant * 2^exp_lsb.  The conversions and the float64 multiply of the
// arithmetic form are slow, dependent instructions; shifts are not.  The result is the same
// integer: v * 2^shift is exact in float64 (a power-of-two scaling), so its rounding to an
// integer is the rounding of mant * 2^(exp_lsb + shift).
__device__ __forceinline__ long long quant_bits(unsigned long long mant, int exp_lsb, bool neg, int shift) {
    const int sh = exp_lsb + shift;
    unsigned long long q;
    if (sh >= 0) {
        q = mant << (sh < 63 ? sh : 63);  // (|q| < 2^48 by the choice of shift whenever mant != 0)
    } else {
        const int r = -sh;
        if (r >= 56) {
            q = 0;  // mant < 2^53: below a quarter
        } else {
            q = mant >> r;
            const unsigned long long rem = mant & ((1ull << r) - 1), half = 1ull << (r - 1);
            if (rem > half || (rem == half && (q & 1))) ++q;
        }
    }
    return neg ? -(long long)q : (long long)q;
}
template <typename T> struct FloatBits;
template <> struct FloatBits<float> {
    // |v| as an unsigned integer that orders like |v|; anything at or above `kBad` is NaN or infinity
    static constexpr unsigned long long kBad = 0x7f800000ull;
    __device__ static unsigned long long magnitude(float v) { return __float_as_uint(v) & 0x7fffffffu; }
    __device__ static double as_double(unsigned long long mag) { return (double)__uint_as_float((uint32_t)mag); }
    __device__ static long long quant(float v, int shift) {
        const uint32_t u = __float_as_uint(v), ex = (u >> 23) & 0xffu;
        const uint32_t mant = (u & 0x7fffffu) | (ex ? 0x800000u : 0u);
        const int sh = (int)(ex ? ex : 1u) - 150 + shift;
        if (sh >= 0) {  // the usual case (a value within 2^23 of the largest): a plain shift
            const long long q = (long long)((unsigned long long)mant << (sh < 63 ? sh : 63));
            return (u >> 31) ? -q : q;
        }
        return quant_bits(mant, (int)(ex ? ex : 1u) - 150, (u >> 31) != 0, shift);
    }
};
template <> struct FloatBits<double> {
    // the arithmetic form calls a value above 1.7e308 non-finite
    static constexpr unsigned long long kBad = 0x7FEE42D130773B77ull;  // the bits after those of 1.7e308
    __device__ static unsigned long long magnitude(double v) {
        return (unsigned long long)__double_as_longlong(v) & 0x7fffffffffffffffull;
    }
    __device__ static double as_double(unsigned long long mag) { return __longlong_as_double((long long)mag); }
    __device__ static long long quant(double v, int shift) {
        const unsigned long long u = (unsigned long long)__double_as_longlong(v);
        const uint32_t ex = (uint32_t)(u >> 52) & 0x7ffu;
        return quant_bits((u & 0xfffffffffffffull) | (ex ? 1ull << 52 : 0ull), (int)(ex ? ex : 1u) - 1075,
                          (u >> 63) != 0, shift);
    }
};

// block_build_table for a vector that lies in shared memory (vec[k], k < n_bits; zero beyond):
// the same table and the same stage record, by integer arithmetic on the bits of the values.
// red_max, red_sum: 32 eight-byte entries of shared memory each; red_bad: one int.
template <typename T>
__device__ __forceinline__ void block_build_table_bits(const T *vec, uint32_t n_bits, uint32_t n_steps, uint4 *table,
                                                       StageMeta *meta_out, unsigned long long *red_max,
                                                       long long *red_sum, int *red_bad) {
    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32, n_warps = (blockDim.x + 31) / 32;
    unsigned long long mx = 0;
    for (uint32_t k = tid; k < n_bits; k += blockDim.x) {
        const unsigned long long mag = FloatBits<T>::magnitude(vec[k]);
        mx = mag > mx ? mag : mx;
    }
    for (int off = 16; off > 0; off >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, mx, off);
        mx = other > mx ? other : mx;
    }
    if (lane == 0) red_max[warp] = mx;
    __syncthreads();
    mx = red_max[0];
    for (uint32_t w = 1; w < n_warps; ++w) mx = red_max[w] > mx ? red_max[w] : mx;
    const int nonfinite = mx >= FloatBits<T>::kBad;
    const FixedPoint fp = fixed_point_of(nonfinite ? 0.0 : FloatBits<T>::as_double(mx));
    long long total = 0;
    const uint32_t n_records = n_steps * 64;
    for (uint32_t r = tid; r < n_records; r += blockDim.x) {
        const uint32_t ks = r / 64, rec = r % 64;
        const uint32_t tt = rec % 4, ip = (rec / 4) % 4, qw = rec / 16;
        long long q8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const uint32_t k = ks * kStepBits + 128 * tt + 32 * qw + 8 * (e % 4) + 2 * ip + e / 4;
            q8[e] = (nonfinite || k >= n_bits) ? 0 : FloatBits<T>::quant(vec[k], fp.shift);
            total += q8[e];
        }
        build_record(q8, ip, table + (size_t)r * 4);
    }
    for (int off = 16; off > 0; off >>= 1) total += __shfl_xor_sync(0xffffffffu, total, off);
    if (lane == 0) red_sum[warp] = total;
    __syncthreads();
    if (tid == 0) {
        long long sum = 0;
        for (uint32_t w = 0; w < n_warps; ++w) sum += red_sum[w];
        meta_out->total = sum;
        meta_out->shift = fp.shift;
        meta_out->nonfinite = nonfinite;
    }
    __syncthreads();
}

}  // namespace
