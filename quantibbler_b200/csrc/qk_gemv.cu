// Decode GEMV over packed +-1 factors and the device-resident factorized linear
//   y = s1 * (Ub (Vb^T (s2 * x))) + bias.
//
// Replaces, for device-resident operation, crates/quantibbler-server/src/engine/mod.rs
// :342-381 (PackedLayer::from_layer) and :393-480 (apply / apply_bf16), whose inner
// loop is crates/quantibbler-kernels/src/core.rs:202-221 (accumulate_row).
//
// Why the main kernel uses the INT8 tensor pipe.  At HBM speed a B200 SM receives about
// 185 weight bits per clock, but it can issue only 128 lane-instructions per clock, so
// any kernel that spends an instruction per weight (sign select + add) is issue-bound
// far below the memory roofline.  The bit-sliced kernel spends 0.3 instructions per
// weight and is exact:
//   * sum_k s_k v_k = 2 * sum_{bit_k = 1} v_k - sum_k v_k, so only the 0/1 weights matter;
//   * v is converted once per call to fixed point, v_k ~ q_k * 2^-sh with |q_k| < 2^47,
//     and q_k * 2^(7-i) (i = k mod 8) is split into eight balanced base-256 digits;
//   * a 32-bit word of weight bits ANDed with 0x01010101 << i is four unsigned bytes
//     holding bit * 2^i: a ready-made A fragment of mma.sync.m16n8k32.u8.s8 with no
//     unpacking.  The eight digit columns are the N dimension, so one MMA retires
//     16 rows x 32 weights against all digits, accumulating exactly in int32;
//   * the eight int32 column sums recombine as sum_n c_n 256^n = 128 * sum bit_k q_k.
// Integer accumulation is associative, so results do not depend on the order of
// summation and are bit-reproducible.  The only roundings are the fixed-point
// conversion (relative 2^-47 of max|v|) and one rounding of the final sum: closer to
// the exact sum than the reference's own float64 left-to-right loop.
//
// Data layout in HBM (built once by qk_layer_create):
//   * tiles: the factor's rows are cut into groups of 64 rows and k-steps of 512 bits.
//     One (group, k-step) pair is a 4 KB chunk holding four 16-row x 512-bit tiles;
//     chunks are stored group-major then k-step-major, which is exactly the order a
//     warp consumes them in, so every warp streams one contiguous byte range.  Inside
//     a tile, the 16-byte piece of row (g + 8*h) at byte offset 16*t sits at piece
//     index h*32 + 4*g + t, so lane (g,t) of a warp moves its own eight pieces of a
//     chunk with eight fully coalesced 512-byte warp transfers.  Rows are padded to a
//     multiple of 64 and bits to a multiple of 512 with zeros.
//   * rows: the reference's per-row bitplanes padded to 16-byte rows; only the
//     sign-select kernel reads it.
//
// Rounding points follow the reference: fp32 serving forms z = s2*x in float32 and
// keeps t and u in float64 between the stages; bf16 serving rounds z, t and u to
// bfloat16 exactly where apply_bf16 does.
#include <cmath>
#include <cstring>
#include <type_traits>

#include "qk_common.h"
#include "qk_digits.cuh"

namespace {

// ------------------------------------------------------------------ shared helpers

// One (layer, token) instance of one stage.
struct StageParams {
    const uint8_t *w_rows;   // padded per-row bitplanes (sign-select kernel)
    const uint8_t *w_tiles;  // 16 x 512 tiles (tensor-core kernel)
    const void *in;          // float[n_bits] (stage 1) or the previous stage's output
    const float *in_scale;   // s2 or null
    void *out;               // intermediate (float or double) or float y
    const float *out_scale;  // s1 or null
    const float *out_bias;   // bias or null
    uint2 *digits;           // tensor-core kernel: digit table of the input vector
    StageMeta *meta;
    const float *in_gate_up; // not null: the input is SwiGLU(in, in_gate_up) = g * u / (1 + e^-g)
    uint32_t n_rows, n_bits; // this instance's shape (the few-instance form mixes shapes)
    // "fed" plans: the digit table of a stage's input is written by whoever produces that
    // input, so the GEMV blocks only stream.  For stage 1 that is the kernel before it (norm,
    // SwiGLU, attention combine); for stage 2 it is stage 1 itself: the last of its blocks to
    // finish (counted by `ticket`) turns t into next_digits / next_meta.
    uint2 *next_digits;
    StageMeta *next_meta;
    uint32_t *ticket;
    // "normed" plans (stage 1 of the few-instance form): `in` is the residual stream x and the
    // stage's input is RMSNorm(x + in_residual) * norm_w, formed in the block itself exactly as
    // the stand-alone norm kernel forms it (same thread count, same order of the sum).  Block 0
    // of an instance with x_out writes the updated stream x + in_residual there.
    const float *norm_w;
    const float *in_residual;
    float *x_out;
    float norm_eps;
    // Tensor parallel, the all-reduce inside the plans (few-instance form).  A row-parallel
    // linear's last stage PUSHES each output it has finished, tagged with the number of this
    // all-reduce, into the inbox of every rank (ar_push[p], peer memory; its own included)
    // instead of storing it.  The normed plan that follows takes as its residual the sum, in
    // rank order, of what has arrived in this rank's inbox (ar_inbox): every block of its first
    // stage polls the words it needs (bounded; error bit 2 on expiry).  An inbox word is
    // {value, all-reduce number}, read and written as one 64-bit access; word
    // (source rank * ar_total + ar_offset + channel) belongs to this instance's token.
    unsigned long long *ar_push[8];
    const unsigned long long *ar_inbox;
    uint32_t *ar_state;   // [0] all-reduces completed, [1] ticket of the consuming launch's blocks
    int *ar_error;
    uint32_t ar_rank, ar_world, ar_total, ar_offset, ar_poll_limit;
};

// ------------------------------------------------------------------ sign-select kernel
constexpr int kWarpsPerBlock = 8;
constexpr int kRowsPerWarp = 4;
constexpr int kChunkBits = 4096;  // 32 lanes x 128 bits

// (bit b of w) ? v : -v: the weight bit is moved onto the sign position and flips
// the sign of v when it is 0.  Compiles to one shift and one three-input logic op.
__device__ __forceinline__ float signed_term(uint32_t w, int b, float v) {
    uint32_t t = w << (31 - b);
    return __uint_as_float(__float_as_uint(v) ^ (~t & 0x80000000u));
}

// out[i] = epilogue(sum_k sign(i,k) * prologue(in[k])), float32 lane partials combined by
// a fixed butterfly.  grid.x tiles the rows, grid.y indexes the instance.
template <bool kRoundBf16>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
gemv_signselect_kernel(const StageParams *__restrict__ many, uint32_t n_rows, uint32_t n_bits,
                       uint32_t stride) {
    qk::pdl_launch();
    qk::pdl_wait();
    extern __shared__ float vs[];  // permuted copy of the input vector, zero padded
    const StageParams p = many[blockIdx.y];
    const float *in = static_cast<const float *>(p.in);
    float *out = static_cast<float *>(p.out);
    const uint32_t n_chunks = (n_bits + kChunkBits - 1) / kChunkBits;
    // element k of chunk c is used by lane l = (k/128)%32 as its e = k%128-th weight
    for (uint32_t k = threadIdx.x; k < n_chunks * kChunkBits; k += blockDim.x) {
        float v = 0.f;
        if (k < n_bits) {
            v = in[k];
            if (p.in_scale) v = p.in_scale[k] * v;
            if (kRoundBf16) v = round_bf16(v);
        }
        uint32_t c = k / kChunkBits, l = (k / 128) % 32, e = k % 128;
        vs[((c * 32 + e / 4) * 32 + l) * 4 + (e % 4)] = v;
    }
    __syncthreads();

    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t row0 = (blockIdx.x * kWarpsPerBlock + warp) * kRowsPerWarp;
    if (row0 >= n_rows) return;
    float acc[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) acc[r] = 0.f;

    for (uint32_t c = 0; c < n_chunks; ++c) {
        const uint32_t byte_off = (c * 32 + lane) * 16;
        if (byte_off >= stride) continue;  // vector entries there are zero as well
        uint4 w[kRowsPerWarp];
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            w[r] = make_uint4(0, 0, 0, 0);
            if (row0 + r < n_rows)
                w[r] = *reinterpret_cast<const uint4 *>(p.w_rows + (size_t)(row0 + r) * stride +
                                                        byte_off);
        }
        const float4 *vrow = reinterpret_cast<const float4 *>(vs) + (size_t)c * 32 * 32 + lane;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                float4 v = vrow[(q * 8 + g) * 32];
#pragma unroll
                for (int r = 0; r < kRowsPerWarp; ++r) {
                    uint32_t word = q == 0 ? w[r].x : q == 1 ? w[r].y : q == 2 ? w[r].z : w[r].w;
                    acc[r] += signed_term(word, 4 * g + 0, v.x);
                    acc[r] += signed_term(word, 4 * g + 1, v.y);
                    acc[r] += signed_term(word, 4 * g + 2, v.z);
                    acc[r] += signed_term(word, 4 * g + 3, v.w);
                }
            }
        }
    }
    // Pad positions hold weight bit 0 (-1) against vector entry +0.0: they add -0.0,
    // which leaves every partial sum unchanged.
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
        float a = acc[r];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
        if (lane == 0 && row0 + r < n_rows) {
            if (kRoundBf16) a = round_bf16(a);
            if (p.out_scale) a = a * p.out_scale[row0 + r];
            if (p.out_bias) a = a + p.out_bias[row0 + r];
            out[row0 + r] = a;
        }
    }
}

// ------------------------------------------------------------------ tensor-core kernel
constexpr int kTileRows = 16;
constexpr int kTileBytes = 1024;
constexpr int kTilesPerWarp = 4;    // row tiles of a group; they share every B fragment (the tile
                                    // layout kernels and the chunk size assume four)
constexpr int kGroupRows = kTileRows * kTilesPerWarp;
constexpr int kChunkBytes = kTileBytes * kTilesPerWarp;
constexpr int kStages = 2;          // ring depth per warp (cp.async)

__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    uint32_t sa = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
    asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// One element of a stage's input vector as float64 (zero beyond n_bits).
//   kInDouble: the input is the float64 intermediate of the previous stage.
template <bool kInDouble, bool kRoundBf16>
__device__ __forceinline__ double load_input(const StageParams &p, uint32_t k, uint32_t n_bits) {
    if (k >= n_bits) return 0.0;
    if (kInDouble) return static_cast<const double *>(p.in)[k];  // rounded by its producer
    float v = static_cast<const float *>(p.in)[k];
    if (p.in_gate_up) v = v * p.in_gate_up[k] / (1.0f + expf(-v));  // the SwiGLU between gate/up and down
    if (p.in_scale) v = p.in_scale[k] * v;  // float32 product, as the reference forms z
    if (kRoundBf16) v = round_bf16(v);
    return (double)v;
}

// kN entries of the input at once, k0, k0 + stride, ...: first every load (unconditional, the
// index clamped into the vector), then the arithmetic.  A loop over load_input() keeps each
// load behind its own bounds check, which the compiler cannot hoist a load across: the entries
// then cost one memory latency EACH, and that, not the arithmetic, is what a digit table built
// from global memory used to wait for.  Same values as load_input().
//   kNorm: 1 = the entries go through the RMSNorm first (StageParams::norm_w), norm_inv being
//   1 / sqrt(mean square + eps) of the whole vector; 2 = they do if the instance has a norm
//   weight (decided at run time, one copy of the code).
template <bool kInDouble, bool kRoundBf16, int kN, typename Out, int kNorm = 0, typename Index>
__device__ __forceinline__ void load_inputs(const StageParams &p, Index index_of, uint32_t n_bits, bool live,
                                            Out (&out)[kN], float norm_inv = 0.f) {
    constexpr bool kNormed = kNorm != 0;
    const bool normed = kNorm == 1 || (kNorm == 2 && p.norm_w != nullptr);
    uint32_t k[kN];
#pragma unroll
    for (int e = 0; e < kN; ++e) k[e] = index_of(e);
    if (kInDouble) {
        double raw[kN];
#pragma unroll
        for (int e = 0; e < kN; ++e) raw[e] = static_cast<const double *>(p.in)[min(k[e], n_bits - 1)];
#pragma unroll
        for (int e = 0; e < kN; ++e) out[e] = (live && k[e] < n_bits) ? (Out)raw[e] : (Out)0;
        return;
    }
    const bool gated = p.in_gate_up != nullptr, scaled = p.in_scale != nullptr;
    const float *up = gated ? p.in_gate_up : static_cast<const float *>(p.in);  // (a valid address either way)
    const float *sc = scaled ? p.in_scale : static_cast<const float *>(p.in);
    const bool residual = normed && p.in_residual != nullptr;
    const float *res = residual ? p.in_residual : static_cast<const float *>(p.in);
    const float *nwp = normed ? p.norm_w : static_cast<const float *>(p.in);
    float v[kN], u[kN], w[kN], rr[kNormed ? kN : 1], nw[kNormed ? kN : 1];
#pragma unroll
    for (int e = 0; e < kN; ++e) {
        const uint32_t kc = min(k[e], n_bits - 1);
        v[e] = static_cast<const float *>(p.in)[kc];
        u[e] = up[kc];
        w[e] = sc[kc];
        if (kNormed) {
            rr[e] = res[kc];
            nw[e] = nwp[kc];
        }
    }
#pragma unroll
    for (int e = 0; e < kN; ++e) {
        float x = v[e];
        if (kNormed && normed) {  // (the roundings of the norm kernel under bfloat16 serving)
            if (residual) x += rr[e];
            if (kRoundBf16) x = round_bf16(x);
            x = x * norm_inv * nw[e];
            if (kRoundBf16) x = round_bf16(x);
        }
        if (gated) x = x * u[e] / (1.0f + expf(-x));  // the SwiGLU between gate/up and down
        if (scaled) x = w[e] * x;                      // float32 product, as the reference forms z
        if (kRoundBf16) x = round_bf16(x);
        out[e] = (live && k[e] < n_bits) ? (Out)x : (Out)0;  // (float or, exactly, double)
    }
}
// ... the eight entries of record r of the digit table (see digit_table_kernel for the layout)
template <bool kInDouble, bool kRoundBf16, typename Out>
__device__ __forceinline__ void load_record(const StageParams &p, uint32_t r, uint32_t n_records, uint32_t n_bits,
                                            Out (&out)[8], float norm_inv = 0.f) {
    const uint32_t ks = r / 64, rec = r % 64;
    const uint32_t base = ks * kStepBits + 128 * (rec % 4) + 32 * (rec / 16) + 2 * ((rec / 4) % 4);
    auto index_of = [&](int e) { return base + 8 * (e % 4) + e / 4; };
    if (!kInDouble && p.norm_w)
        load_inputs<kInDouble, kRoundBf16, 8, Out, 1>(p, index_of, n_bits, r < n_records, out, norm_inv);
    else
        load_inputs<kInDouble, kRoundBf16, 8, Out>(p, index_of, n_bits, r < n_records, out);
}

// Converts one instance's input vector to its digit table.
//   kInDouble: the input is the float64 intermediate of the previous stage.
// Table layout (uint2 units): record ((ks*4 + q)*4 + ip)*4 + t holds, for digit column n,
// the B fragment pair of lane (g = n, t) for the MMA that consumes word q of k-step ks
// under masks 2*ip (b0) and 2*ip+1 (b1); byte j of b0/b1 belongs to
// k = 512*ks + 128*t + 32*q + 8*j + i.
// grid.x covers the k-steps four at a time (one record per thread), grid.y is the instance.
// Every block first walks the whole vector - evaluating each entry once (scale, SwiGLU,
// rounding) into shared memory and reducing max|v| - so blocks need no communication; block 0
// of each instance also forms sum_k q_k.  A thread then builds one record for all eight digit
// columns from its eight entries and writes 64 contiguous bytes.  All of it is integer
// arithmetic on the bits of the values (FloatBits: the same integers as the float64 form); a
// float32 input never becomes a double.  Dynamic shared memory: n_steps * 512 entries.
constexpr int kTableThreads = 256;
//   kCache = false: a vector too long for shared memory is evaluated again where it is needed.
template <bool kInDouble, bool kRoundBf16, bool kCache = true>
__global__ void __launch_bounds__(kTableThreads)
digit_table_kernel(const StageParams *__restrict__ many, uint32_t n_bits, uint32_t n_steps) {
    using T = typename std::conditional<kInDouble, double, float>::type;
    qk::pdl_launch();
    const StageParams p = many[blockIdx.y];
    // (the scale vector depends on no other kernel: its first touch, cold in caches and TLB,
    // need not wait for the one before this)
    if (!kInDouble && p.in_scale)
        for (uint32_t line = threadIdx.x; line * 32 < n_bits; line += kTableThreads)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(p.in_scale + line * 32));
    qk::pdl_wait();
    extern __shared__ __align__(16) uint8_t table_vec_raw[];
    T *vec = reinterpret_cast<T *>(table_vec_raw);  // the evaluated entries, zero beyond n_bits
    __shared__ unsigned long long red_max[kTableThreads / 32];
    __shared__ long long red_sum[kTableThreads / 32];
    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t n_padded = n_steps * kStepBits;

    // (eight entries per thread and round: their loads are in flight together)
    constexpr int kScan = 8;
    unsigned long long mx = 0;
    for (uint32_t k0 = tid; k0 < n_padded; k0 += kTableThreads * kScan) {
        T vals[kScan];
        load_inputs<kInDouble, kRoundBf16, kScan, T>(p, [&](int u) { return k0 + kTableThreads * u; }, n_bits, true, vals);
#pragma unroll
        for (int u = 0; u < kScan; ++u) {
            const uint32_t k = k0 + kTableThreads * u;
            if (kCache && k < n_padded) vec[k] = vals[u];
            const unsigned long long mag = FloatBits<T>::magnitude(vals[u]);
            mx = mag > mx ? mag : mx;
        }
    }
    for (int off = 16; off > 0; off >>= 1) {
        const unsigned long long other = __shfl_xor_sync(0xffffffffu, mx, off);
        mx = other > mx ? other : mx;
    }
    if (lane == 0) red_max[warp] = mx;
    __syncthreads();  // (also: vec is complete)
    mx = red_max[0];
#pragma unroll
    for (int w = 1; w < kTableThreads / 32; ++w) mx = red_max[w] > mx ? red_max[w] : mx;
    const bool nonfinite = mx >= FloatBits<T>::kBad;  // NaN or infinity somewhere
    const FixedPoint fp = fixed_point_of(nonfinite ? 0.0 : FloatBits<T>::as_double(mx));

    if (blockIdx.x == 0) {
        long long total = 0;
        if (!nonfinite && kCache)
            for (uint32_t k = tid; k < n_bits; k += kTableThreads) total += FloatBits<T>::quant(vec[k], fp.shift);
        if (!nonfinite && !kCache)
            for (uint32_t k0 = tid; k0 < n_bits; k0 += kTableThreads * kScan) {
                T vals[kScan];
                load_inputs<kInDouble, kRoundBf16, kScan, T>(p, [&](int u) { return k0 + kTableThreads * u; }, n_bits, true,
                                                             vals);
#pragma unroll
                for (int u = 0; u < kScan; ++u) total += FloatBits<T>::quant(vals[u], fp.shift);
            }
        for (int off = 16; off > 0; off >>= 1) total += __shfl_xor_sync(0xffffffffu, total, off);
        if (lane == 0) red_sum[warp] = total;
        __syncthreads();
        if (tid == 0) {
            long long sum = 0;
            for (int w = 0; w < kTableThreads / 32; ++w) sum += red_sum[w];
            p.meta->total = sum;
            p.meta->shift = fp.shift;
            p.meta->nonfinite = nonfinite;
        }
    }

    const uint32_t ks = blockIdx.x * (kTableThreads / 64) + tid / 64;
    if (ks >= n_steps) return;
    const uint32_t rec = tid % 64;  // (qw*4 + ip)*4 + t
    const uint32_t tt = rec % 4, ip = (rec / 4) % 4, qw = rec / 16;
    T entries[8];
    if (kCache) {
#pragma unroll
        for (int e = 0; e < 8; ++e)
            entries[e] = vec[ks * kStepBits + 128 * tt + 32 * qw + 8 * (e % 4) + 2 * ip + e / 4];
    } else {
        load_record<kInDouble, kRoundBf16, T>(p, ks * 64 + rec, n_steps * 64, n_bits, entries);
    }
    long long q8[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) q8[e] = nonfinite ? 0 : FloatBits<T>::quant(entries[e], fp.shift);
    build_record(q8, ip, reinterpret_cast<uint4 *>(p.digits + ((size_t)ks * 64 + rec) * 8));
}
// The same table by a thread-block CLUSTER per instance (float32 input, at most 32 k-steps):
// CTA c of the cluster owns k-steps 4c .. 4c + 3, evaluates only ITS 2048 entries (coalesced
// loads; scale, SwiGLU, rounding; into shared memory), and the CTAs agree on max|v| and on
// sum q_k through each other's shared memory: every CTA pushes its maximum into a slot of
// every CTA, a cluster barrier, every CTA reads its own slots; the partial sums go to CTA 0 the
// same way.  Nothing is evaluated twice, which is what the one-vector-per-block form above
// spends its time on (each of its blocks walks the whole vector).
template <bool kRoundBf16>
__global__ void __launch_bounds__(256)
digit_table_cluster_kernel(const StageParams *__restrict__ many, uint32_t n_bits, uint32_t n_steps) {
    qk::pdl_launch();
    const StageParams p = many[blockIdx.y];
    uint32_t rank, n_rank;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(rank));
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(n_rank));
    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32, k_lo = rank * 4 * kStepBits;
    // (the scale vector depends on no other kernel: its first touch need not wait)
    if (p.in_scale && tid < 64 && k_lo + tid * 32 < n_bits)
        asm volatile("prefetch.global.L2 [%0];" ::"l"(p.in_scale + k_lo + tid * 32));
    qk::pdl_wait();
    __shared__ float zs[4 * kStepBits];
    __shared__ uint32_t cl_max[8], red_u[8];
    __shared__ long long cl_total[8], red_s[8];
    auto swz = [](uint32_t k) { return k ^ (((k >> 7) & 3) << 3) ^ ((k >> 5) & 1); };
    auto cluster_sync = [] {
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    };
    auto remote = [](const void *local, uint32_t cta) {  // the same shared-memory word in CTA `cta`
        uint32_t r;
        asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(cta));
        return r;
    };

    float vals[8];
    load_inputs<false, kRoundBf16, 8, float>(p, [&](int e) { return k_lo + tid + 256 * e; }, n_bits, true, vals);
    uint32_t mx = 0;
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        zs[swz(tid + 256 * e)] = vals[e];
        mx = max(mx, __float_as_uint(vals[e]) & 0x7fffffffu);
    }
    for (int off = 16; off > 0; off >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if (lane == 0) red_u[warp] = mx;
    __syncthreads();  // (also: zs is complete)
    if (tid < n_rank) {
        uint32_t bm = red_u[0];
#pragma unroll
        for (int w = 1; w < 8; ++w) bm = max(bm, red_u[w]);
        asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote(&cl_max[rank], tid)), "r"(bm) : "memory");
    }
    cluster_sync();
    mx = cl_max[0];
    for (uint32_t c = 1; c < n_rank; ++c) mx = max(mx, cl_max[c]);
    const bool nonfinite = mx >= 0x7f800000u;  // NaN or infinity somewhere in the vector
    const FixedPoint fp = fixed_point_of(nonfinite ? 0.0 : (double)__uint_as_float(mx));

    const uint32_t ks = rank * 4 + tid / 64, rec = tid % 64;
    long long total = 0;
    if (ks < n_steps) {
        const uint32_t base = (tid / 64) * kStepBits + 128 * (rec % 4) + 32 * (rec / 16) + 2 * ((rec / 4) % 4);
        long long q8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            q8[e] = nonfinite ? 0 : fp.quant((double)zs[swz(base + 8 * (e % 4) + e / 4)]);
            total += q8[e];
        }
        build_record(q8, (rec / 4) % 4, reinterpret_cast<uint4 *>(p.digits + ((size_t)ks * 64 + rec) * 8));
    }
    for (int off = 16; off > 0; off >>= 1) total += __shfl_xor_sync(0xffffffffu, total, off);
    if (lane == 0) red_s[warp] = total;
    __syncthreads();
    if (tid == 0) {
        long long bt = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) bt += red_s[w];
        asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(remote(&cl_total[rank], 0)), "l"(bt) : "memory");
    }
    cluster_sync();  // (nobody leaves while a peer may still write into its shared memory)
    if (rank == 0 && tid == 0) {
        long long sum = 0;
        for (uint32_t c = 0; c < n_rank; ++c) sum += cl_total[c];
        p.meta->total = sum;
        p.meta->shift = fp.shift;
        p.meta->nonfinite = nonfinite;
    }
}

// Launches it for n_inst instances of one stage.
template <bool kFinal>
qk_status launch_digit_table(qk_ctx *c, const StageParams *many, size_t n_inst, size_t n_bits, size_t n_steps,
                             bool bf16) {
    if (!kFinal && qk::ceil_div(n_steps, (size_t)4) <= 8 && n_inst <= 65535) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)qk::ceil_div(n_steps, (size_t)4), (unsigned)n_inst);
        cfg.blockDim = dim3(256);
        cfg.dynamicSmemBytes = 0;
        cfg.stream = c->stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = c->pdl ? 1 : 0;
        attr[1].id = cudaLaunchAttributeClusterDimension;
        attr[1].val.clusterDim.x = cfg.gridDim.x;
        attr[1].val.clusterDim.y = 1;
        attr[1].val.clusterDim.z = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 2;
        QK_CUDA(cudaLaunchKernelEx(&cfg, bf16 ? digit_table_cluster_kernel<true> : digit_table_cluster_kernel<false>,
                                   many, (uint32_t)n_bits, (uint32_t)n_steps));
        c->launches++;
        return QK_OK;
    }
    const size_t smem = n_steps * kStepBits * (kFinal ? 8 : 4);  // (stage 2 reads the float64 intermediate)
    const bool cache = smem <= 200 * 1024;
    auto table = cache ? (bf16 ? digit_table_kernel<kFinal, true, true> : digit_table_kernel<kFinal, false, true>)
                       : (bf16 ? digit_table_kernel<kFinal, true, false> : digit_table_kernel<kFinal, false, false>);
    if (cache && smem > 48 * 1024)
        QK_CUDA(cudaFuncSetAttribute(table, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 tgrid((unsigned)qk::ceil_div(n_steps, kTableThreads / 64), (unsigned)n_inst);
    (void)qk::launch_pdl(c->pdl, table, tgrid, dim3(kTableThreads), cache ? smem : 0, c->stream, many,
                         (uint32_t)n_bits, (uint32_t)n_steps);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    return QK_OK;
}

// Starts this warp's first kStages-1 chunks of a stage (item i of a warp goes to ring slot
// i % kStages; here the items are the contiguous chunks of the warp's row groups).
__device__ __forceinline__ void ring_prologue(const StageParams &p, uint8_t *ring_smem,
                                              uint32_t n_groups, uint32_t n_steps,
                                              uint32_t block_in_instance,
                                              uint32_t groups_per_warp) {
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t group_begin =
        min(n_groups, (block_in_instance * (blockDim.x / 32) + warp) * groups_per_warp);
    const uint32_t group_end = min(n_groups, group_begin + groups_per_warp);
    const uint32_t n_items = (group_end - group_begin) * n_steps;
    uint4 *ring = reinterpret_cast<uint4 *>(ring_smem + (size_t)warp * kStages * kChunkBytes) + lane;
    const uint4 *src = reinterpret_cast<const uint4 *>(p.w_tiles) + lane;
#pragma unroll
    for (int i = 0; i < kStages - 1; ++i) {
        if ((uint32_t)i < n_items) {
            uint4 *dst = ring + (size_t)i * (kChunkBytes / 16);
            const uint4 *from = src + (size_t)(group_begin * n_steps + i) * (kChunkBytes / 16);
#pragma unroll
            for (int piece = 0; piece < 8; ++piece) cp_async16(dst + piece * 32, from + piece * 32);
        }
        cp_async_commit();
    }
}

// out[row] = epilogue((2 * sum_{bit=1} q_k - sum q_k) * 2^-shift).
//   kFinal = false: writes the float64 intermediate t;  true: y = float(u)*s1 + bias.
//   kSmemDigits: the block builds the instance's digit table in shared memory itself,
//   straight from the input vector (no separate kernel, no table in global memory);
//   otherwise the table made by digit_table_kernel is read through L1 (only for inputs
//   too wide for shared memory).
// grid.y is the instance; the instance's row groups are dealt to the grid.x * (warps per
// block) warps in contiguous runs of `groups_per_warp`, so each warp reads one contiguous
// range of chunks.  Every lane copies exactly the eight 16-byte pieces it will consume
// itself through a private cp.async ring, so the ring needs no barrier of any kind.
// Measured on B200: with the table in shared memory, 16 warps per SM and a two-deep ring
// the loop runs at 92% of what the INT8 tensor pipe plus the mask ALU work allow.
//   kInSmem / kOutSmem: the input vector is read from / the result written to shared memory
//   as float64 (the fused kernel keeps t on the SM between the two stages).
// table_smem: the digit table (kSmemDigits); ring_smem: warps x kStages x 4 KB.
// prologue_issued: the caller already started this warp's first kStages-1 chunks with
// ring_prologue (the fused kernel does so before the stage boundary barrier).
// kSplitK: the block owns ONE row group (block_in_instance is the group) and its warps
// share the group's k-steps (warp w takes k-steps w, w+W, ...); the partial int32 sums are
// added through red_smem ([warps][16][32] ints) and warps 0..3 finish one 16-row tile each.
// This is the low-latency form for a single small layer: every chunk of the factor is in
// flight at once instead of eight per warp in sequence.
template <bool kRoundBf16, bool kFinal, bool kSmemDigits, bool kInSmem, bool kOutSmem,
          bool kSplitK = false>
__device__ __forceinline__ void
bitslice_stage(const StageParams &p, uint8_t *table_smem, uint8_t *ring_smem,
               const double *in_smem, double *out_smem, uint32_t n_rows, uint32_t n_bits,
               uint32_t n_groups, uint32_t n_steps, uint32_t block_in_instance,
               uint32_t groups_per_warp, bool prologue_issued, int *red_smem = nullptr) {
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t warps_per_block = blockDim.x / 32;
    const uint32_t g = lane / 4, t = lane % 4;
    auto input = [&](uint32_t k) -> double {
        if (kInSmem) return k < n_bits ? in_smem[k] : 0.0;
        return load_input<kFinal, kRoundBf16>(p, k, n_bits);
    };
    const uint32_t group_begin =
        kSplitK ? block_in_instance
                : min(n_groups, (block_in_instance * warps_per_block + warp) * groups_per_warp);
    const uint32_t group_end = kSplitK ? group_begin + 1 : min(n_groups, group_begin + groups_per_warp);
    // the chunks this warp consumes, as items 0..n_items-1
    const uint32_t n_items =
        kSplitK ? (warp < n_steps ? (n_steps - warp + warps_per_block - 1) / warps_per_block : 0)
                : (group_end - group_begin) * n_steps;
    auto chunk_of = [&](uint32_t i) -> uint32_t {
        return kSplitK ? group_begin * n_steps + warp + i * warps_per_block
                       : group_begin * n_steps + i;
    };

    uint4 *ring = reinterpret_cast<uint4 *>(ring_smem + (size_t)warp * kStages * kChunkBytes) + lane;
    const uint4 *src = reinterpret_cast<const uint4 *>(p.w_tiles) + lane;
    auto issue = [&](uint32_t i) {  // item i goes to ring slot i % kStages
        if (i < n_items) {
            uint4 *dst = ring + (size_t)(i % kStages) * (kChunkBytes / 16);
            const uint4 *from = src + (size_t)chunk_of(i) * (kChunkBytes / 16);
#pragma unroll
            for (int piece = 0; piece < 8; ++piece) cp_async16(dst + piece * 32, from + piece * 32);
        }
        cp_async_commit();  // an empty group keeps the group count in step with i
    };
    if (!prologue_issued) {
        // (the few-instance form fills every slot of its ring before it waits for the kernel
        // before it: a warp has one or two chunks, and both are then on their way; the slot of
        // an item is refilled only after the item has been multiplied)
#pragma unroll
        for (int s = 0; s < (kSplitK ? kStages : kStages - 1); ++s) issue(s);
    }
    if (kSplitK) {
        // The few-instance form is a chain of latencies, and one of its links is the first
        // touch of the small constant vectors (s2, the norm weight, s1, bias: a few KB each in
        // allocations of their own, cold in the caches and in the TLB).  They depend on no
        // other kernel either: ask for them before the wait.
        auto ask = [](const float *v, uint32_t first, uint32_t n, uint32_t t, uint32_t t_n) {
            // floats first .. first + n of v, one 128-byte line per thread t of t_n
            for (uint32_t line = t; line * 32 < n; line += t_n)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(v + first + line * 32));
        };
        const uint32_t quarter = blockDim.x / 4, tq = threadIdx.x % quarter;
        const uint32_t row0 = block_in_instance * kGroupRows;
        const uint32_t rows = min((uint32_t)kGroupRows, n_rows - min(n_rows, row0));
        switch (threadIdx.x / quarter) {
            case 0: if (!kFinal && p.in_scale) ask(p.in_scale, 0, n_bits, tq, quarter); break;
            case 1: if (!kFinal && p.norm_w) ask(p.norm_w, 0, n_bits, tq, quarter); break;
            case 2: if (kFinal && p.out_scale) ask(p.out_scale, row0, rows, tq, quarter); break;
            default: if (kFinal && p.out_bias) ask(p.out_bias, row0, rows, tq, quarter); break;
        }
    }
    // The weight bits depend on no other kernel, the input vector does: from here on the
    // kernel before this one on the stream must be complete.
    qk::pdl_wait();
    // ---- a normed plan's stage 1: the norm's scale over the whole vector, as rmsnorm_kernel
    // forms it (512 threads, element i of a thread's sixteen is tid + 512 i, warp sums by
    // shuffles, then the warps' sums in order), and the updated residual stream
    float norm_inv = 0.f;
    // the number of the all-reduce this launch sends (last stage) or receives (first stage)
    const uint32_t ar_step = (kSplitK && (kFinal ? p.ar_world != 0 : p.ar_inbox != nullptr)) ? *p.ar_state + 1 : 0;
    float hk[8];  // a normed instance's entries tid + 512 i after the residual add (rounded), i < 8
    bool hk_valid = false;
    if (!kFinal && !kInSmem && p.norm_w) {
        __shared__ float norm_red[16];
        const float *xs = static_cast<const float *>(p.in);
        const bool writer = p.x_out && block_in_instance == 0;
        // (eight of a thread's sixteen elements at a time: their loads go out together; the
        // second eight only exist beyond 4096 entries, and adding their zeros changes nothing)
        const float *rs = p.in_residual ? p.in_residual : xs;
        float ss = 0.f;
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
            if (half * 8u * 512u >= n_bits) break;
            float hx[8], hr[8];
#pragma unroll
            for (int rr = 0; rr < 8; ++rr) {
                const uint32_t i = min(threadIdx.x + (8 * half + rr) * 512, n_bits - 1);
                hx[rr] = xs[i];
                hr[rr] = rs[i];
            }
            const bool gathered = kSplitK && p.ar_inbox != nullptr;  // (only for vectors of at most 4096 entries)
            if (gathered) {
                // the residual is the sum over the ranks, in rank order, of what they pushed
                // into this rank's inbox for this all-reduce
#pragma unroll
                for (int rr = 0; rr < 8; ++rr) hr[rr] = 0.f;
                bool all_ready = true;
                for (uint32_t r = 0; r < p.ar_world; ++r) {
                    const unsigned long long *src = p.ar_inbox + (size_t)r * p.ar_total + p.ar_offset;
                    float got[8];
                    bool ready = false;
                    for (uint32_t tries = 0; tries < p.ar_poll_limit && !ready; ++tries) {
                        ready = true;
#pragma unroll
                        for (int rr = 0; rr < 8; ++rr) {
                            const uint32_t i = threadIdx.x + rr * 512;
                            unsigned long long word = (unsigned long long)ar_step << 32;
                            if (i < n_bits)
                                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(word) : "l"(src + i) : "memory");
                            got[rr] = __uint_as_float((uint32_t)word);
                            if ((uint32_t)(word >> 32) != ar_step) ready = false;
                        }
                    }
                    if (!ready) all_ready = false;
#pragma unroll
                    for (int rr = 0; rr < 8; ++rr) hr[rr] += got[rr];
                }
                if (!all_ready && p.ar_error) atomicOr(p.ar_error, 2);  // (reported at the next synchronise)
            }
            const bool add = gathered || p.in_residual != nullptr;
#pragma unroll
            for (int rr = 0; rr < 8; ++rr) {
                const uint32_t i = threadIdx.x + (8 * half + rr) * 512;
                float h = 0.f;
                if (i < n_bits) {
                    h = hx[rr];
                    if (add) h += hr[rr];
                    if (writer) p.x_out[i] = h;
                    if (kRoundBf16) h = round_bf16(h);
                }
                if (half == 0) hk[rr] = h;
                ss += h * h;
            }
        }
        hk_valid = n_bits <= 8u * 512u && blockDim.x == 512;
        for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        if (lane == 0) norm_red[warp] = ss;
        __syncthreads();
        float total = 0.f;
        for (uint32_t w = 0; w < warps_per_block; ++w) total += norm_red[w];
        norm_inv = 1.0f / sqrtf(total / (float)n_bits + p.norm_eps);
    }
    // ---- the digit table of this instance (the weight ring is already filling)
    __shared__ double red_max[16];
    __shared__ long long red_sum[16];
    StageMeta meta;
    if (kSmemDigits && kSplitK && !kInSmem && !kFinal && red_smem &&
        n_steps * kStepBits * 4 <= warps_per_block * 16 * 32 * 4) {
        // The few-instance form's first stage.  A record's eight entries lie 8 and 128 floats
        // apart: fetched from global memory record by record, a warp's load touches eight lines
        // for 128 useful bytes, and the block spends microseconds in the load/store unit.  The
        // vector is evaluated once instead, with coalesced loads (scale, norm, SwiGLU,
        // rounding), into the buffer the k-split reduction uses later, and the records read
        // it from there (the index is swizzled so that a warp's 32 reads fall into 32 banks).
        float *zs = reinterpret_cast<float *>(red_smem);
        auto swz = [](uint32_t k) { return k ^ (((k >> 7) & 3) << 3) ^ ((k >> 5) & 1); };
        const uint32_t n_records = n_steps * 64, n_padded = n_steps * kStepBits;
        double mx = 0.0;
        int bad = 0;
        for (uint32_t k0 = threadIdx.x; k0 < n_padded; k0 += 8 * blockDim.x) {
            float vals[8];
            if (hk_valid) {
                // a normed instance: the thread still holds its entries from the norm (the same
                // elements tid + 512 e), so neither the stream nor the residual - which may have
                // come out of the all-reduce inbox - is read again
                const float *nwp = p.norm_w, *scp = p.in_scale ? p.in_scale : p.norm_w;
                float nw[8], sc[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const uint32_t kc = min(k0 + e * 512, n_bits - 1);
                    nw[e] = nwp[kc];
                    sc[e] = scp[kc];
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    float x = hk[e] * norm_inv * nw[e];
                    if (kRoundBf16) x = round_bf16(x);
                    if (p.in_scale) x = sc[e] * x;
                    if (kRoundBf16) x = round_bf16(x);
                    vals[e] = k0 + e * 512 < n_bits ? x : 0.f;
                }
            } else {
                load_inputs<false, kRoundBf16, 8, float, 2>(p, [&](int e) { return k0 + e * blockDim.x; }, n_bits,
                                                            true, vals, norm_inv);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const uint32_t k = k0 + e * blockDim.x;
                if (k < n_padded) zs[swz(k)] = vals[e];
                const double a = fabs((double)vals[e]);
                if (!(a <= 1.7e308)) bad = 1;  // NaN or infinity
                mx = fmax(mx, a);
            }
        }
        for (int off = 16; off > 0; off >>= 1) mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        if (lane == 0) red_max[warp] = mx;
        meta.nonfinite = __syncthreads_or(bad);  // (also: zs is complete)
        double m = red_max[0];
        for (uint32_t w = 1; w < warps_per_block; ++w) m = fmax(m, red_max[w]);
        const FixedPoint fp = fixed_point_of(meta.nonfinite ? 0.0 : m);
        meta.shift = fp.shift;
        long long total = 0;
        uint4 *table = reinterpret_cast<uint4 *>(table_smem);
        for (uint32_t r = threadIdx.x; r < n_records; r += blockDim.x) {
            const uint32_t ks = r / 64, rec = r % 64;
            const uint32_t base = ks * kStepBits + 128 * (rec % 4) + 32 * (rec / 16) + 2 * ((rec / 4) % 4);
            long long q8[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                q8[e] = meta.nonfinite ? 0 : fp.quant((double)zs[swz(base + 8 * (e % 4) + e / 4)]);
                total += q8[e];
            }
            build_record(q8, (rec / 4) % 4, table + (size_t)r * 4);
        }
        for (int off = 16; off > 0; off >>= 1) total += __shfl_xor_sync(0xffffffffu, total, off);
        if (lane == 0) red_sum[warp] = total;
        __syncthreads();  // the table and the partial totals are complete (zs is free again)
        total = 0;
        for (uint32_t w = 0; w < warps_per_block; ++w) total += red_sum[w];
        meta.total = total;
    } else if (kSmemDigits) {
        // Each thread owns whole records (eight vector entries each).  The first two
        // records of a thread stay in registers between the max pass and the
        // quantisation, so the input is read from memory once.
        constexpr int kCached = 2;
        const uint32_t n_records = n_steps * 64;
        auto record_entry = [&](uint32_t r, int e) -> double {
            const uint32_t ks = r / 64, rec = r % 64;
            const uint32_t tt = rec % 4, ip = (rec / 4) % 4, qw = rec / 16;
            return input(ks * kStepBits + 128 * tt + 32 * qw + 8 * (e % 4) + 2 * ip + e / 4);
        };
        // (from global memory a record's eight loads go out together: load_inputs)
        auto record = [&](uint32_t r, double (&entries)[8]) {
            if (kInSmem) {
#pragma unroll
                for (int e = 0; e < 8; ++e) entries[e] = r < n_records ? record_entry(r, e) : 0.0;
            } else {
                load_record<kFinal, kRoundBf16, double>(p, r, n_records, n_bits, entries, norm_inv);
            }
        };
        double cached[kCached][8];
        double mx = 0.0;
        int bad = 0;
#pragma unroll
        for (int sl = 0; sl < kCached; ++sl) record(threadIdx.x + sl * blockDim.x, cached[sl]);
#pragma unroll
        for (int sl = 0; sl < kCached; ++sl)
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                double a = fabs(cached[sl][e]);
                if (!(a <= 1.7e308)) bad = 1;  // NaN or infinity
                mx = fmax(mx, a);
            }
        for (uint32_t r = threadIdx.x + kCached * blockDim.x; r < n_records; r += blockDim.x) {
            double entries[8];
            record(r, entries);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                double a = fabs(entries[e]);
                if (!(a <= 1.7e308)) bad = 1;
                mx = fmax(mx, a);
            }
        }
        for (int off = 16; off > 0; off >>= 1)
            mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        if (lane == 0) red_max[warp] = mx;
        meta.nonfinite = __syncthreads_or(bad);
        double m = red_max[0];
        for (uint32_t w = 1; w < warps_per_block; ++w) m = fmax(m, red_max[w]);
        const FixedPoint fp = fixed_point_of(meta.nonfinite ? 0.0 : m);
        meta.shift = fp.shift;
        long long total = 0;
        uint4 *table = reinterpret_cast<uint4 *>(table_smem);
#pragma unroll
        for (int sl = 0; sl < kCached; ++sl) {
            const uint32_t r = threadIdx.x + sl * blockDim.x;
            if (r < n_records) {
                long long q8[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    q8[e] = meta.nonfinite ? 0 : fp.quant(cached[sl][e]);
                    total += q8[e];
                }
                build_record(q8, (r % 64 / 4) % 4, table + (size_t)r * 4);
            }
        }
        for (uint32_t r = threadIdx.x + kCached * blockDim.x; r < n_records; r += blockDim.x) {
            double entries[8];
            record(r, entries);
            long long q8[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                q8[e] = meta.nonfinite ? 0 : fp.quant(entries[e]);
                total += q8[e];
            }
            build_record(q8, (r % 64 / 4) % 4, table + (size_t)r * 4);
        }
        for (int off = 16; off > 0; off >>= 1) total += __shfl_xor_sync(0xffffffffu, total, off);
        if (lane == 0) red_sum[warp] = total;
        __syncthreads();  // the table and the partial totals are complete
        total = 0;
        for (uint32_t w = 0; w < warps_per_block; ++w) total += red_sum[w];
        meta.total = total;
    } else {
        meta = *p.meta;
    }

    int acc[kTilesPerWarp][4];
#pragma unroll
    for (int m = 0; m < kTilesPerWarp; ++m)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[m][e] = 0;
    const uint2 *dig =
        (kSmemDigits ? reinterpret_cast<const uint2 *>(table_smem) : p.digits) + t * 8 + g;
    const long long th = meta.total >> 26;
    const long long tl = (meta.total & ((1ll << 26) - 1)) << 6;
    const int sh0 = 16 * (t & 1);
    // 2^(-shift-6) as a double (one multiply per row instead of a call to ldexp)
    const int oexp = -meta.shift - 6;
    const bool odirect = oexp > -1000 && oexp < 1000;
    const double oscale = odirect ? __hiloint2double((1023 + oexp) << 20, 0) : 0.0;

    // Exact recombination of one 16-row tile.  Lane (g,t) holds digit columns 2t and 2t+1
    // of rows g (a[0..1]) and g+8 (a[2..3]).  With X = sum_n c_n 256^n = 128 * S and
    // T = sum q_k, the row's value is (X - 64 T) / 64 * 2^-shift.  X is kept as
    // hi * 2^32 + lo (digits 4..7 and 0..3) and 64 T as th * 2^32 + tl, so the subtraction
    // is exact in int64 and only the last conversion rounds.
    auto finish_tile = [&](const int (&a)[4], uint32_t group, int m) {
        long long pg = ((long long)a[0] << sh0) + ((long long)a[1] << (sh0 + 8));
        long long ph = ((long long)a[2] << sh0) + ((long long)a[3] << (sh0 + 8));
        pg += __shfl_xor_sync(0xffffffffu, pg, 1);  // t=0,1: low half; t=2,3: high half
        ph += __shfl_xor_sync(0xffffffffu, ph, 1);
        const long long og = __shfl_xor_sync(0xffffffffu, pg, 2);
        const long long oh = __shfl_xor_sync(0xffffffffu, ph, 2);
        const uint32_t row = group * kGroupRows + m * kTileRows + g + 8 * t;
        if (t < 2 && row < n_rows) {
            const long long lo = t == 0 ? pg : ph, hi = t == 0 ? og : oh;
            double val = (double)(hi - th) * 4294967296.0 + (double)(lo - tl);
            val = odirect ? val * oscale : ldexp(val, oexp);
            if (meta.nonfinite) val = nan("");
            if (kRoundBf16) val = (double)round_bf16((float)val);
            if (kOutSmem) {
                out_smem[row] = val;
            } else if (kFinal) {
                float y = (float)val;
                if (p.out_scale) y = y * p.out_scale[row];
                if (p.out_bias) y = y + p.out_bias[row];
                if (kSplitK && p.ar_world) {
                    // this rank's part of a row-parallel output: into every rank's inbox
                    const unsigned long long word =
                        (unsigned long long)__float_as_uint(y) | ((unsigned long long)ar_step << 32);
                    const size_t at = (size_t)p.ar_rank * p.ar_total + p.ar_offset + row;
                    for (uint32_t peer = 0; peer < p.ar_world; ++peer)
                        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(p.ar_push[peer] + at), "l"(word)
                                     : "memory");
                } else {
                    static_cast<float *>(p.out)[row] = y;
                }
            } else {
                static_cast<double *>(p.out)[row] = val;
            }
        }
    };

    // The same for two tiles at once: lanes t = 0,1 take the rows of tile m, lanes t = 2,3 those
    // of tile m + 1, so every lane converts one row and the exchange needs three shuffles of a
    // 64-bit value per tile instead of four.
    auto finish_pair = [&](const int (&a)[4], const int (&b2)[4], uint32_t group, int m) {
        long long pg[2], ph[2];
        pg[0] = ((long long)a[0] << sh0) + ((long long)a[1] << (sh0 + 8));
        ph[0] = ((long long)a[2] << sh0) + ((long long)a[3] << (sh0 + 8));
        pg[1] = ((long long)b2[0] << sh0) + ((long long)b2[1] << (sh0 + 8));
        ph[1] = ((long long)b2[2] << sh0) + ((long long)b2[3] << (sh0 + 8));
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            pg[k] += __shfl_xor_sync(0xffffffffu, pg[k], 1);  // t=0,1: low half; t=2,3: high half
            ph[k] += __shfl_xor_sync(0xffffffffu, ph[k], 1);
        }
        const bool first = t < 2;
        const long long other_g = __shfl_xor_sync(0xffffffffu, first ? pg[1] : pg[0], 2);
        const long long other_h = __shfl_xor_sync(0xffffffffu, first ? ph[1] : ph[0], 2);
        const long long mine_g = first ? pg[0] : pg[1], mine_h = first ? ph[0] : ph[1];
        const bool upper = (t & 1) != 0;  // row g (t even) or g + 8 (t odd) of the lane's tile
        const long long lo = first ? (upper ? mine_h : mine_g) : (upper ? other_h : other_g);
        const long long hi = first ? (upper ? other_h : other_g) : (upper ? mine_h : mine_g);
        const uint32_t row = group * kGroupRows + (m + (first ? 0 : 1)) * kTileRows + g + (upper ? 8 : 0);
        if (row < n_rows) {
            double val = (double)(hi - th) * 4294967296.0 + (double)(lo - tl);
            val = odirect ? val * oscale : ldexp(val, oexp);
            if (meta.nonfinite) val = nan("");
            if (kRoundBf16) val = (double)round_bf16((float)val);
            if (kOutSmem) {
                out_smem[row] = val;
            } else if (kFinal) {
                float y = (float)val;
                if (p.out_scale) y = y * p.out_scale[row];
                if (p.out_bias) y = y + p.out_bias[row];
                static_cast<float *>(p.out)[row] = y;
            } else {
                static_cast<double *>(p.out)[row] = val;
            }
        }
    };

    uint32_t ks = kSplitK ? warp : 0, group = group_begin;
    for (uint32_t i = 0; i < n_items; ++i) {
        if (!kSplitK) issue(i + kStages - 1);  // refills the slot consumed one iteration ago
        cp_async_wait<kStages - 1>();          // this lane's pieces of item i have landed
        const uint4 *stage = ring + (size_t)(i % kStages) * (kChunkBytes / 16);
        uint4 cur[kTilesPerWarp][2];
#pragma unroll
        for (int m = 0; m < kTilesPerWarp; ++m) {
            cur[m][0] = stage[m * 64];
            cur[m][1] = stage[m * 64 + 32];
        }
        const uint2 *dk = dig + (size_t)ks * 512;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int ip = 0; ip < 4; ++ip) {
                const uint2 b = kSmemDigits ? dk[(q * 4 + ip) * 32] : __ldg(dk + (q * 4 + ip) * 32);
                const uint32_t m0 = 0x01010101u << (2 * ip), m1 = m0 << 1;
#pragma unroll
                for (int m = 0; m < kTilesPerWarp; ++m) {
                    const uint32_t wg = q == 0 ? cur[m][0].x : q == 1 ? cur[m][0].y
                                      : q == 2 ? cur[m][0].z : cur[m][0].w;
                    const uint32_t wh = q == 0 ? cur[m][1].x : q == 1 ? cur[m][1].y
                                      : q == 2 ? cur[m][1].z : cur[m][1].w;
                    mma_u8s8(acc[m], wg & m0, wh & m0, wg & m1, wh & m1, b.x, b.y);
                }
            }
        }
        if (kSplitK) {
            issue(i + kStages);  // (item i sits in registers and has been multiplied: its slot is free)
            ks += warps_per_block;
            continue;
        }
        if (++ks < n_steps) continue;
        ks = 0;
        // ---- the group's rows are complete: two tiles at a time (finish_pair)
#pragma unroll
        for (int m = 0; m < kTilesPerWarp; m += 2) {
            finish_pair(acc[m], acc[m + 1], group, m);
            acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0;
            acc[m + 1][0] = acc[m + 1][1] = acc[m + 1][2] = acc[m + 1][3] = 0;
        }
        ++group;
    }
    if (kSplitK) {
        // add the warps' partial sums (integers: the order does not matter)
#pragma unroll
        for (int m = 0; m < kTilesPerWarp; ++m)
#pragma unroll
            for (int e = 0; e < 4; ++e) red_smem[(warp * 16 + m * 4 + e) * 32 + lane] = acc[m][e];
        __syncthreads();
        if (warp < kTilesPerWarp) {
            int sum[4] = {0, 0, 0, 0};
            for (uint32_t w = 0; w < warps_per_block; ++w)
#pragma unroll
                for (int e = 0; e < 4; ++e) sum[e] += red_smem[(w * 16 + warp * 4 + e) * 32 + lane];
            finish_tile(sum, group_begin, (int)warp);
        }
    }
    cp_async_wait<0>();
}

// One stage of the factorized linear.  grid.y is the instance, grid.x the blocks that
// share its row groups.  smem: [digit table][ring].
template <bool kRoundBf16, bool kFinal, bool kSmemDigits>
__global__ void __launch_bounds__(512, 1)
gemv_bitslice_kernel(const StageParams *__restrict__ many, uint32_t n_rows, uint32_t n_bits,
                     uint32_t n_groups, uint32_t n_steps, uint32_t groups_per_warp) {
    qk::pdl_launch();  // (bitslice_stage waits for the kernel before, after its weight prologue)
    extern __shared__ __align__(128) uint8_t smem_dyn[];
    const StageParams p = many[blockIdx.y];
    uint8_t *ring = smem_dyn + (kSmemDigits ? (size_t)n_steps * 4096 : 0);
    bitslice_stage<kRoundBf16, kFinal, kSmemDigits, false, false>(
        p, smem_dyn, ring, nullptr, nullptr, n_rows, n_bits, n_groups, n_steps, blockIdx.x,
        groups_per_warp, false);
}

// Low-latency form for few instances: one block per (row group, instance), the block's
// warps share the group's k-steps.  smem: [digit table][ring][reduction buffer].
// The instances of one launch may differ in shape (q beside k and v): every instance brings
// its own n_rows and n_bits, the grid covers the largest group count and the shared memory
// the longest table; blocks beyond an instance's last row group have nothing to do.
//   kFed: the digit table and the stage record of the input are already in global memory
//   (p.digits, p.meta), written by the kernel that produced the input; the block builds
//   nothing, needs no shared memory for a table, and starts multiplying as soon as its first
//   chunks have landed.  A stage-1 instance with a ticket then hands over to stage 2: the last
//   of its blocks to finish builds the table of t.  smem: [ring][reduction buffer].
template <bool kRoundBf16, bool kFinal, bool kFed = false>
__global__ void __launch_bounds__(512)
gemv_bitslice_splitk_kernel(const StageParams *__restrict__ many) {
    qk::pdl_launch();  // (bitslice_stage waits for the kernel before, after its weight prologue)
    extern __shared__ __align__(128) uint8_t smem_dyn[];
    const StageParams p = many[blockIdx.y];
    const uint32_t n_rows = p.n_rows, n_bits = p.n_bits;
    const uint32_t n_groups = (n_rows + kGroupRows - 1) / kGroupRows;
    const uint32_t n_steps = (n_bits + kStepBits - 1) / kStepBits;
    // A launch that receives an all-reduce counts its blocks: the last one to finish records
    // that the all-reduce is done (every block has read the number by then).
    auto all_reduce_done = [&] {
        if (kFinal || kFed || !p.ar_inbox) return;
        __syncthreads();
        if (threadIdx.x == 0) {
            const uint32_t step = *p.ar_state + 1;
            __threadfence();
            if (atomicAdd(p.ar_state + 1, 1u) == gridDim.x * gridDim.y - 1) {
                p.ar_state[1] = 0;
                p.ar_state[0] = step;
            }
        }
    };
    if (blockIdx.x >= n_groups) {
        qk::pdl_wait();
        all_reduce_done();
        return;
    }
    uint8_t *ring = smem_dyn + (kFed ? 0 : (size_t)n_steps * 4096);
    int *red = reinterpret_cast<int *>(ring + (size_t)(blockDim.x / 32) * kStages * kChunkBytes);
    bitslice_stage<kRoundBf16, kFinal, !kFed, false, false, true>(
        p, smem_dyn, ring, nullptr, nullptr, n_rows, n_bits, n_groups, n_steps, blockIdx.x, 1, false,
        red);
    all_reduce_done();
    if (kFed && !kFinal && p.ticket) {
        // hand-over to stage 2: whoever finishes last has all of t in front of it
        __shared__ double tail_max[32];
        __shared__ long long tail_sum[32];
        __shared__ int tail_bad, tail_last;
        __threadfence();  // this block's rows of t are visible to the device
        __syncthreads();
        if (threadIdx.x == 0) {
            const uint32_t ticket = atomicAdd(p.ticket, 1u);
            tail_last = ticket == n_groups - 1;
            if (tail_last) *p.ticket = 0;  // every block has drawn: ready for the next launch
        }
        __syncthreads();
        if (tail_last) {
            __threadfence();
            const double *t_in = static_cast<const double *>(p.out);
            block_build_table([&](uint32_t k) { return k < n_rows ? __ldcg(t_in + k) : 0.0; },
                              (n_rows + kStepBits - 1) / kStepBits, reinterpret_cast<uint4 *>(p.next_digits),
                              p.next_meta, tail_max, tail_sum, &tail_bad);
        }
    }
}

// Both stages of one layer instance in one block: t = Vb^T z stays in shared memory as
// float64, the second digit table is built from it there, and each warp starts fetching
// its first chunks of the second factor before the stage boundary barrier.  Used whenever
// one block per instance is the right grain (many independent instances per launch).
// smem: [t: r doubles][table (the larger of the two stages)][ring].
template <bool kRoundBf16>
__global__ void __launch_bounds__(512, 1)
layer_bitslice_fused_kernel(const StageParams *__restrict__ stage1,
                            const StageParams *__restrict__ stage2, uint32_t r, uint32_t din,
                            uint32_t dout, uint32_t t_bytes, uint32_t table_bytes, uint32_t gpw1,
                            uint32_t gpw2) {
    qk::pdl_launch();
    extern __shared__ __align__(128) uint8_t smem_dyn[];
    double *t_smem = reinterpret_cast<double *>(smem_dyn);
    uint8_t *table = smem_dyn + t_bytes, *ring = table + table_bytes;
    const StageParams p1 = stage1[blockIdx.x], p2 = stage2[blockIdx.x];
    const uint32_t groups2 = (dout + kGroupRows - 1) / kGroupRows;
    const uint32_t steps2 = (r + kStepBits - 1) / kStepBits;
    bitslice_stage<kRoundBf16, false, true, false, true>(
        p1, table, ring, nullptr, t_smem, r, din, (r + kGroupRows - 1) / kGroupRows,
        (din + kStepBits - 1) / kStepBits, 0, gpw1, false);
    // this warp's ring slots are free again: start on the second factor right away
    ring_prologue(p2, ring, groups2, steps2, 0, gpw2);
    __syncthreads();  // every row of t is in shared memory; the table can be rebuilt
    bitslice_stage<kRoundBf16, true, true, true, false>(p2, table, ring, t_smem, nullptr, dout, r,
                                                        groups2, steps2, 0, gpw2, true);
}

// ------------------------------------------------------------------ persistent streaming form
// Many independent layer instances per launch (a stack of layers, or one layer for many
// requests): one CTA per SM stays resident and walks over its share of the instances with
// two kinds of warps, so that the stream of weight bits from HBM never stops for a layer
// boundary, a table build or a stage boundary.
//   * consumer warps (16): the mask-and-MMA loop of bitslice_stage and nothing else.  A warp
//     owns whole row groups.  Its 4 KB chunks arrive in a private two-slot ring by bulk copies
//     (cp.async.bulk completing on an mbarrier) that the warp starts itself, one instruction
//     from one lane: the moment a chunk has been read into registers its slot is refilled
//     with the chunk two ahead.  The sequence of a warp's chunks depends on no data, so the
//     prefetch runs on across stage and layer boundaries.
//   * builder warps (3): turn the input vector of the NEXT instance into its digit table
//     while the consumers stream the current one, and turn t into the second table as soon
//     as the consumers have finished stage 1.
// The stages are software-pipelined over the instances, J1(0) J1(1) J2(0) J1(2) J2(1) ...,
// so that a whole stage of other work lies between the end of J1(i) (t complete) and the
// start of J2(i) (which needs the table made from t): nobody waits in the steady state.
// Two table buffers per stage and two t buffers suffice; their reuse is ordered by the
// barriers themselves (see the notes at the waits).  Every wait is bounded: a role that runs
// out of polls raises the CTA's abort flag, every other role sees it in its own wait, all
// leave, and the launch reports bit 8 of the context's error word.
constexpr int kPsConsumers = 16;
constexpr int kPsBuilders = 3;
constexpr int kPsBuilderWarp0 = kPsConsumers;
constexpr int kPsThreads = (kPsConsumers + kPsBuilders) * 32;
constexpr int kPsDepth = 2;  // ring slots per consumer warp
constexpr int kPsTilePtrs = 48;  // instances per CTA whose tile addresses are kept in shared memory
constexpr uint32_t kPsWaitLimitDefault = 1u << 22;

struct PsArgs {
    const StageParams *stage1, *stage2;  // [n_inst] each
    uint32_t n_inst;
    uint32_t r, din, dout;
    uint32_t wait_limit;
    int *error;
};

__device__ __forceinline__ uint32_t ps_smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void ps_mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ps_smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void ps_mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ps_smem_u32(bar)) : "memory");
}
// One lane's bounded wait; false when the polls ran out or another role gave up.
__device__ __forceinline__ bool ps_wait_lane(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                             uint32_t limit) {
    const uint32_t addr = ps_smem_u32(bar);
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            " selp.u32 %0, 1, 0, p;\n}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if ((i & 63u) == 63u && *abort_flag) return false;
    }
    return false;
}
// The warp's verdict (all 32 lanes call it): every lane has either seen the phase or run out.
__device__ __forceinline__ bool ps_wait_warp(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                             uint32_t limit) {
    return __all_sync(0xffffffffu, ps_wait_lane(bar, parity, abort_flag, limit)) != 0;
}

// Digit table of one stage's input, built by the builder threads (tid 0 .. 32*kPsBuilders-1).
//   input(k): element k as float64 (zero beyond the vector).  red: kPsBuilders doubles, long
//   longs and ints of shared memory for the group's reductions; named barrier 2 keeps the
//   group in step.
template <typename Input>
__device__ __forceinline__ void ps_build_table(Input input, uint32_t n_steps, uint4 *table,
                                               StageMeta *meta_out, double *red_max,
                                               long long *red_sum, int *red_bad, uint32_t tid) {
    constexpr uint32_t kGroupThreads = kPsBuilders * 32;
    const uint32_t warp = tid / 32, lane = tid % 32;
    const uint32_t n_records = n_steps * 64;
    auto record_entry = [&](uint32_t r, int e) -> double {
        const uint32_t ks = r / 64, rec = r % 64;
        const uint32_t tt = rec % 4, ip = (rec / 4) % 4, qw = rec / 16;
        return input(ks * kStepBits + 128 * tt + 32 * qw + 8 * (e % 4) + 2 * ip + e / 4);
    };
    double mx = 0.0;
    int bad = 0;
    for (uint32_t r = tid; r < n_records; r += kGroupThreads)
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const double a = fabs(record_entry(r, e));
            if (!(a <= 1.7e308)) bad = 1;  // NaN or infinity
            mx = fmax(mx, a);
        }
    for (int off = 16; off > 0; off >>= 1) {
        mx = fmax(mx, __shfl_xor_sync(0xffffffffu, mx, off));
        bad |= __shfl_xor_sync(0xffffffffu, bad, off);
    }
    if (lane == 0) {
        red_max[warp] = mx;
        red_bad[warp] = bad;
    }
    asm volatile("bar.sync 2, %0;" ::"r"(kGroupThreads) : "memory");
    double m = red_max[0];
    int nonfinite = red_bad[0];
#pragma unroll
    for (int w = 1; w < kPsBuilders; ++w) {
        m = fmax(m, red_max[w]);
        nonfinite |= red_bad[w];
    }
    const FixedPoint fp = fixed_point_of(nonfinite ? 0.0 : m);
    long long total = 0;
    for (uint32_t r = tid; r < n_records; r += kGroupThreads) {
        long long q8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            q8[e] = nonfinite ? 0 : fp.quant(record_entry(r, e));
            total += q8[e];
        }
        build_record(q8, (r % 64 / 4) % 4, table + (size_t)r * 4);
    }
    for (int off = 16; off > 0; off >>= 1) total += __shfl_xor_sync(0xffffffffu, total, off);
    if (lane == 0) red_sum[warp] = total;
    asm volatile("bar.sync 2, %0;" ::"r"(kGroupThreads) : "memory");
    if (tid == 0) {
        long long sum = 0;
#pragma unroll
        for (int w = 0; w < kPsBuilders; ++w) sum += red_sum[w];
        meta_out->total = sum;
        meta_out->shift = fp.shift;
        meta_out->nonfinite = nonfinite;
    }
    // (the caller's arrival on the table's barrier publishes table and meta)
}

// Where a consumer warp is in its sequence of chunks.  Job t of a CTA with n instances:
//   t = 0: J1(0);  t = 2n-1: J2(n-1);  otherwise t odd: J1((t+1)/2), t even: J2(t/2 - 1)
// which is the order J1(0) J1(1) J2(0) J1(2) J2(1) ... J2(n-1).  Within a job the warp takes
// the row groups warp, warp + 16, ..., and within a group the k-steps in order.
struct PsCursor {
    uint32_t job, group, ks;
};
struct PsShape {
    uint32_t n_mine, groups[2], steps[2];
};
__device__ __forceinline__ void ps_job(const PsShape &sh, uint32_t job, uint32_t *stage, uint32_t *inst) {
    if (job == 0) {
        *stage = 0;
        *inst = 0;
    } else if (job == 2 * sh.n_mine - 1) {
        *stage = 1;
        *inst = sh.n_mine - 1;
    } else if (job & 1) {
        *stage = 0;
        *inst = (job + 1) / 2;
    } else {
        *stage = 1;
        *inst = job / 2 - 1;
    }
}
// First chunk of the first job from `job` on in which this warp owns a row group.
__device__ __forceinline__ bool ps_seek(const PsShape &sh, uint32_t warp, PsCursor *c) {
    while (c->job < 2 * sh.n_mine) {
        uint32_t stage, inst;
        ps_job(sh, c->job, &stage, &inst);
        if (warp < sh.groups[stage]) {
            c->group = warp;
            c->ks = 0;
            return true;
        }
        ++c->job;
    }
    return false;
}
__device__ __forceinline__ bool ps_next(const PsShape &sh, uint32_t warp, PsCursor *c) {
    uint32_t stage, inst;
    ps_job(sh, c->job, &stage, &inst);
    if (++c->ks < sh.steps[stage]) return true;
    c->ks = 0;
    c->group += kPsConsumers;
    if (c->group < sh.groups[stage]) return true;
    ++c->job;
    return ps_seek(sh, warp, c);
}

template <bool kRoundBf16>
__global__ void __launch_bounds__(kPsThreads, 1)
layer_stream_kernel(const PsArgs a, uint32_t t_bytes, uint32_t table1_bytes, uint32_t table2_bytes) {
    qk::pdl_launch();
    extern __shared__ __align__(128) uint8_t smem_dyn[];
    // [rings: warp x depth x 4 KB][table1 x2][table2 x2][t x2][meta x4][barriers][reduction scratch][abort]
    uint8_t *ring = smem_dyn;
    uint8_t *table1 = ring + (size_t)kPsConsumers * kPsDepth * kChunkBytes;
    uint8_t *table2 = table1 + 2 * (size_t)table1_bytes;
    uint8_t *t_base = table2 + 2 * (size_t)table2_bytes;
    StageMeta *meta = reinterpret_cast<StageMeta *>(t_base + 2 * (size_t)t_bytes);  // [stage][buffer]
    uint64_t *full = reinterpret_cast<uint64_t *>(meta + 4);  // [warp][depth]
    uint64_t *t1_full = full + kPsConsumers * kPsDepth;       // [2] table of stage 1, buffer b, is ready
    uint64_t *tt_full = t1_full + 2;                          // [2] t buffer b is complete
    uint64_t *t2_full = tt_full + 2;                          // [2] table of stage 2, buffer b, is ready
    double *red_max = reinterpret_cast<double *>(t2_full + 2);
    long long *red_sum = reinterpret_cast<long long *>(red_max + kPsBuilders);
    int *red_bad = reinterpret_cast<int *>(red_sum + kPsBuilders);
    volatile int *abort_flag = red_bad + kPsBuilders;
    // where the weight tiles of this CTA's instances lie, [stage][instance], so that starting
    // a copy costs no global load (instances beyond the table are looked up in global memory)
    __shared__ const uint8_t *tiles_of[2][kPsTilePtrs];

    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t limit = a.wait_limit;
    PsShape sh;
    // this CTA's instances: blockIdx.x, blockIdx.x + gridDim.x, ...
    sh.n_mine = a.n_inst > blockIdx.x ? (a.n_inst - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
    sh.groups[0] = (a.r + kGroupRows - 1) / kGroupRows;
    sh.steps[0] = (a.din + kStepBits - 1) / kStepBits;
    sh.groups[1] = (a.dout + kGroupRows - 1) / kGroupRows;
    sh.steps[1] = (a.r + kStepBits - 1) / kStepBits;

    if (threadIdx.x == 0) {
        for (int b = 0; b < 2; ++b) {
            ps_mbar_init(&t1_full[b], kPsBuilders);
            // every consumer warp that owns a row group of stage 1 reports its rows of t
            ps_mbar_init(&tt_full[b], min((uint32_t)kPsConsumers, sh.groups[0]));
            ps_mbar_init(&t2_full[b], kPsBuilders);
        }
        abort_flag[0] = 0;
        abort_flag[1] = 0;  // stays zero: the flag of waits that must not be cut short
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (uint32_t i = threadIdx.x; i < min(sh.n_mine, (uint32_t)kPsTilePtrs); i += blockDim.x) {
        const size_t at = blockIdx.x + (size_t)i * gridDim.x;
        tiles_of[0][i] = a.stage1[at].w_tiles;
        tiles_of[1][i] = a.stage2[at].w_tiles;
    }
    __syncthreads();

    if (warp < kPsConsumers) {
        // ------------------------------------------------------------ consumers
        const uint32_t g = lane / 4, t = lane % 4;
        uint8_t *my_ring = ring + (size_t)warp * kPsDepth * kChunkBytes;
        // the chunk a cursor points at: weight bits only, known without any input
        // Every lane copies exactly the eight 16-byte pieces of a chunk that it will read itself
        // (cp.async, one commit group per chunk), so the ring needs no barrier of any kind.
        auto issue = [&](const PsCursor &c, uint32_t slot) {
            uint32_t stage, inst;
            ps_job(sh, c.job, &stage, &inst);
            const uint8_t *tiles;
            if (inst < (uint32_t)kPsTilePtrs) {
                tiles = tiles_of[stage][inst];
            } else {
                const size_t at = blockIdx.x + (size_t)inst * gridDim.x;
                tiles = stage == 0 ? a.stage1[at].w_tiles : a.stage2[at].w_tiles;
            }
            const uint4 *from = reinterpret_cast<const uint4 *>(
                                    tiles + ((size_t)c.group * sh.steps[stage] + c.ks) * kChunkBytes) + lane;
            uint4 *dst = reinterpret_cast<uint4 *>(my_ring + (size_t)slot * kChunkBytes) + lane;
#pragma unroll
            for (int piece = 0; piece < 8; ++piece) cp_async16(dst + piece * 32, from + piece * 32);
        };
        PsCursor fetch{0, 0, 0}, cur{0, 0, 0};
        bool more = ps_seek(sh, warp, &fetch);
        uint32_t n_issued = 0;
        for (; n_issued < (uint32_t)kPsDepth; ++n_issued) {
            if (more) {
                issue(fetch, n_issued);
                more = ps_next(sh, warp, &fetch);
            }
            cp_async_commit();  // (an empty group keeps the group count in step with the chunks)
        }
        qk::pdl_wait();  // from here on: inputs, which come from the kernel before this one
        bool ok = true, have = ps_seek(sh, warp, &cur);
        uint32_t n_done = 0, job_ready = 0xffffffffu;
        StageMeta mt{};
        const uint2 *dig = nullptr;
        StageParams p{};
        int acc[kTilesPerWarp][4];
        while (have && ok) {
            uint32_t stage, inst;
            ps_job(sh, cur.job, &stage, &inst);
            const uint32_t b = inst & 1, n_steps = sh.steps[stage];
            if (job_ready != cur.job) {
                // first chunk of a job: its table (built a whole stage ago in the steady state)
                if (!ps_wait_warp(stage == 0 ? &t1_full[b] : &t2_full[b], (inst >> 1) & 1, abort_flag, limit)) {
                    ok = false;
                    break;
                }
                mt = meta[stage * 2 + b];
                dig = reinterpret_cast<const uint2 *>(stage == 0 ? table1 + (size_t)b * table1_bytes
                                                                 : table2 + (size_t)b * table2_bytes) + t * 8 + g;
                p = stage == 0 ? a.stage1[blockIdx.x + (size_t)inst * gridDim.x]
                               : a.stage2[blockIdx.x + (size_t)inst * gridDim.x];
                job_ready = cur.job;
            }
            if (cur.ks == 0) {
#pragma unroll
                for (int m = 0; m < kTilesPerWarp; ++m) acc[m][0] = acc[m][1] = acc[m][2] = acc[m][3] = 0;
            }
            const uint32_t slot = n_done % kPsDepth;
            cp_async_wait<kPsDepth - 1>();  // this lane's pieces of the chunk have landed
            const uint4 *stage_ptr = reinterpret_cast<const uint4 *>(my_ring + (size_t)slot * kChunkBytes) + lane;
            uint4 chunk[kTilesPerWarp][2];
#pragma unroll
            for (int m = 0; m < kTilesPerWarp; ++m) {
                chunk[m][0] = stage_ptr[m * 64];
                chunk[m][1] = stage_ptr[m * 64 + 32];
            }
            // the chunk is in registers: refill its slot with the chunk kPsDepth ahead (a lane
            // overwrites only pieces it has just read itself)
            if (more) {
                issue(fetch, slot);
                more = ps_next(sh, warp, &fetch);
            }
            cp_async_commit();
            const uint2 *dk = dig + (size_t)cur.ks * 512;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
#pragma unroll
                for (int ip = 0; ip < 4; ++ip) {
                    const uint2 bq = dk[(q * 4 + ip) * 32];
                    const uint32_t m0 = 0x01010101u << (2 * ip), m1 = m0 << 1;
#pragma unroll
                    for (int m = 0; m < kTilesPerWarp; ++m) {
                        const uint32_t wg = q == 0 ? chunk[m][0].x : q == 1 ? chunk[m][0].y
                                          : q == 2 ? chunk[m][0].z : chunk[m][0].w;
                        const uint32_t wh = q == 0 ? chunk[m][1].x : q == 1 ? chunk[m][1].y
                                          : q == 2 ? chunk[m][1].z : chunk[m][1].w;
                        mma_u8s8(acc[m], wg & m0, wh & m0, wg & m1, wh & m1, bq.x, bq.y);
                    }
                }
            }
            ++n_done;
            const bool group_done = cur.ks + 1 == n_steps;
            const uint32_t group = cur.group, job = cur.job;
            have = ps_next(sh, warp, &cur);
            if (!group_done) continue;
            // ---- exact recombination (see bitslice_stage): X = sum_n c_n 256^n = 128 S, value =
            // (X - 64 T) / 64 * 2^-shift with X = hi 2^32 + lo and 64 T = th 2^32 + tl.  Two
            // tiles are finished at a time: lanes t = 0,1 take the rows of the first, lanes
            // t = 2,3 those of the second, so every lane converts one row.
            {
                const uint32_t n_rows = stage == 0 ? a.r : a.dout;
                double *out_smem = reinterpret_cast<double *>(t_base + (size_t)b * t_bytes);
                const long long th = mt.total >> 26;
                const long long tl = (mt.total & ((1ll << 26) - 1)) << 6;
                const int sh0 = 16 * (t & 1);
                const int oexp = -mt.shift - 6;
                const bool odirect = oexp > -1000 && oexp < 1000;
                const double oscale = odirect ? __hiloint2double((1023 + oexp) << 20, 0) : 0.0;
#pragma unroll
                for (int pair = 0; pair < kTilesPerWarp / 2; ++pair) {
                    long long pg[2], ph[2];
#pragma unroll
                    for (int k = 0; k < 2; ++k) {
                        const int(&c4)[4] = acc[2 * pair + k];
                        pg[k] = ((long long)c4[0] << sh0) + ((long long)c4[1] << (sh0 + 8));
                        ph[k] = ((long long)c4[2] << sh0) + ((long long)c4[3] << (sh0 + 8));
                        pg[k] += __shfl_xor_sync(0xffffffffu, pg[k], 1);  // t=0,1: low half; t=2,3: high half
                        ph[k] += __shfl_xor_sync(0xffffffffu, ph[k], 1);
                    }
                    // lanes t<2 keep tile 2*pair (they hold its low half and get the high half from
                    // t+2); lanes t>=2 keep tile 2*pair+1 (they hold its high half and get the low)
                    const bool first = t < 2;
                    const long long send_g = first ? pg[1] : pg[0], send_h = first ? ph[1] : ph[0];
                    const long long other_g = __shfl_xor_sync(0xffffffffu, send_g, 2);
                    const long long other_h = __shfl_xor_sync(0xffffffffu, send_h, 2);
                    const long long mine_g = first ? pg[0] : pg[1], mine_h = first ? ph[0] : ph[1];
                    const bool upper = (t & 1) != 0;  // row g (t even) or g + 8 (t odd) of the lane's tile
                    const long long lo = first ? (upper ? mine_h : mine_g) : (upper ? other_h : other_g);
                    const long long hi = first ? (upper ? other_h : other_g) : (upper ? mine_h : mine_g);
                    const int m = 2 * pair + (first ? 0 : 1);
                    const uint32_t row = group * kGroupRows + m * kTileRows + g + (upper ? 8 : 0);
                    if (row < n_rows) {
                        double val = (double)(hi - th) * 4294967296.0 + (double)(lo - tl);
                        val = odirect ? val * oscale : ldexp(val, oexp);
                        if (mt.nonfinite) val = nan("");
                        if (kRoundBf16) val = (double)round_bf16((float)val);
                        if (stage == 1) {
                            float y = (float)val;
                            if (p.out_scale) y = y * p.out_scale[row];
                            if (p.out_bias) y = y + p.out_bias[row];
                            static_cast<float *>(p.out)[row] = y;
                        } else {
                            out_smem[row] = val;
                        }
                    }
                }
            }
            // the warp's last row group of a stage-1 job: its rows of t are written
            if (stage == 0 && (!have || cur.job != job)) {
                __syncwarp();
                if (lane == 0) ps_mbar_arrive(&tt_full[b]);
            }
        }
        cp_async_wait<0>();  // nothing of this warp is in flight when the CTA ends
        if (!ok) *abort_flag = 1;
    } else {
        // ------------------------------------------------------------ builders
        qk::pdl_wait();
        const uint32_t tid = threadIdx.x - kPsBuilderWarp0 * 32;
        auto build1 = [&](uint32_t i) {
            const uint32_t b = i & 1;
            const StageParams p = a.stage1[blockIdx.x + (size_t)i * gridDim.x];
            const uint32_t n_bits = a.din;
            ps_build_table([&](uint32_t k) { return load_input<false, kRoundBf16>(p, k, n_bits); }, sh.steps[0],
                           reinterpret_cast<uint4 *>(table1 + (size_t)b * table1_bytes), &meta[b], red_max,
                           red_sum, red_bad, tid);
            __syncwarp();
            if (lane == 0) ps_mbar_arrive(&t1_full[b]);
        };
        bool ok = true;
        // table1 buffer i&1 was last read by J1(i-2); J1(i-2) had finished before T2(i-2)
        // started (tt_full), and T2(i-2) precedes T1(i) in this loop: no extra barrier.
        if (sh.n_mine > 0) build1(0);
        for (uint32_t i = 0; i < sh.n_mine && ok; ++i) {
            if (i + 1 < sh.n_mine) build1(i + 1);
            const uint32_t b = i & 1;
            // all consumers have written their rows of t(i) ...
            bool seen = ps_wait_warp(&tt_full[b], (i >> 1) & 1, abort_flag, limit);
            // ... and the builder warps agree on it before any of them meets the others at the
            // group's barrier inside the build
            uint32_t all;
            asm volatile(
                "{\n .reg .pred p, q;\n setp.ne.b32 p, %1, 0;\n"
                " barrier.cta.red.and.pred q, 3, %2, p;\n selp.u32 %0, 1, 0, q;\n}"
                : "=r"(all)
                : "r"((uint32_t)seen), "r"((uint32_t)(kPsBuilders * 32))
                : "memory");
            if (!all) {
                ok = false;
                break;
            }
            // table2 buffer b was last read by J2(i-2), which every consumer had finished
            // before it began J1(i); t buffer b is next written by J1(i+2), which follows J2(i),
            // and J2(i) starts only after this build has arrived on t2_full.
            const double *t_in = reinterpret_cast<const double *>(t_base + (size_t)b * t_bytes);
            const uint32_t n_bits = a.r;
            ps_build_table([&](uint32_t k) { return k < n_bits ? t_in[k] : 0.0; }, sh.steps[1],
                           reinterpret_cast<uint4 *>(table2 + (size_t)b * table2_bytes), &meta[2 + b],
                           red_max, red_sum, red_bad, tid);
            __syncwarp();
            if (lane == 0) ps_mbar_arrive(&t2_full[b]);
        }
        if (!ok) *abort_flag = 1;
    }
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicOr(a.error, 8);
}

// ------------------------------------------------------------------ layer construction
// Copy host-layout rows (row_words bytes each) into 16-byte padded rows, clearing the
// pad bits of the last byte.
__global__ void pad_rows_kernel(const uint8_t *__restrict__ src, uint8_t *__restrict__ dst,
                                uint32_t n_rows, uint32_t n_bits, uint32_t row_words,
                                uint32_t stride) {
    uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (uint64_t)n_rows * stride) return;
    uint32_t i = (uint32_t)(gid / stride), b = (uint32_t)(gid % stride);
    uint8_t v = 0;
    if (b < row_words) {
        v = src[(size_t)i * row_words + b];
        uint32_t valid = n_bits - b * 8;  // bits of this byte that are real
        if (valid < 8) v &= (uint8_t)((1u << valid) - 1u);
    }
    dst[gid] = v;
}

// Container bit stream -> padded rows on the device (engine/mod.rs:258-273,
// container_to_rows): the stream holds the n_rows x r sign matrix row-major with no padding
// between rows, bit b of the stream in byte b / 8 at bit b % 8; row i of the result starts at
// a byte and ends with zero bits.  One thread per 16-byte piece of the padded result.
__global__ void stream_rows_kernel(const uint8_t *__restrict__ stream, size_t stream_len,
                                   uint8_t *__restrict__ dst, uint32_t n_rows, uint32_t r,
                                   uint32_t stride) {
    const uint32_t pieces = stride / 16;
    uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (uint64_t)n_rows * pieces) return;
    const uint32_t i = (uint32_t)(gid / pieces), p = (uint32_t)(gid % pieces);
    uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (uint32_t q = 0; q < 16; ++q) {
        const uint32_t j = p * 128 + q * 8;  // first column of this byte
        if (j >= r) break;
        const uint64_t bit = (uint64_t)i * r + j;
        const size_t at = (size_t)(bit >> 3);
        uint32_t two = stream[at];
        if (at + 1 < stream_len) two |= (uint32_t)stream[at + 1] << 8;
        uint32_t v = (two >> (uint32_t)(bit & 7)) & 0xffu;
        if (r - j < 8) v &= (1u << (r - j)) - 1u;
        w[q >> 2] |= v << (8 * (q & 3));
    }
    reinterpret_cast<uint4 *>(dst)[gid] = make_uint4(w[0], w[1], w[2], w[3]);
}

// The same for the transposed factor (engine/mod.rs:275-289, container_to_rows_transposed):
// the stream holds the din x r matrix row-major; row k of the result is column k, i.e. bit j
// of row k is stream bit j * r + k.  One thread per 16-byte piece (128 values of j); threads
// next to each other take neighbouring k, so a warp's 32 reads of one j fall into 4-5 bytes.
__global__ void stream_rows_transposed_kernel(const uint8_t *__restrict__ stream,
                                              uint8_t *__restrict__ dst, uint32_t din, uint32_t r,
                                              uint32_t stride) {
    const uint32_t pieces = stride / 16;
    uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (uint64_t)r * pieces) return;
    const uint32_t k = (uint32_t)(gid % r), p = (uint32_t)(gid / r);
    uint32_t w[4] = {0, 0, 0, 0};
    for (uint32_t q = 0; q < 128; ++q) {
        const uint32_t j = p * 128 + q;
        if (j >= din) break;
        const uint64_t bit = (uint64_t)j * r + k;
        w[q >> 5] |= (uint32_t)((stream[bit >> 3] >> (uint32_t)(bit & 7)) & 1u) << (q & 31);
    }
    reinterpret_cast<uint4 *>(dst + (size_t)k * stride)[p] = make_uint4(w[0], w[1], w[2], w[3]);
}

// Padded rows -> 4 KB chunks of four 16 x 512 tiles (one thread per 16-byte piece).
__global__ void tile_rows_kernel(const uint8_t *__restrict__ rows, uint8_t *__restrict__ tiles,
                                 uint32_t n_rows, uint32_t stride, uint32_t n_groups,
                                 uint32_t n_steps) {
    uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (uint64_t)n_groups * n_steps * 256) return;
    uint64_t chunk = gid / 256;
    uint32_t within = (uint32_t)(gid % 256);
    uint32_t grp = (uint32_t)(chunk / n_steps), ks = (uint32_t)(chunk % n_steps);
    uint32_t m = within / 64, half = (within % 64) / 32, lane = within % 32;
    uint32_t g = lane / 4, t = lane % 4;
    uint32_t row = grp * kGroupRows + m * kTileRows + g + 8 * half;
    uint32_t off = ks * 64 + t * 16;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (row < n_rows && off < stride)
        v = *reinterpret_cast<const uint4 *>(rows + (size_t)row * stride + off);
    reinterpret_cast<uint4 *>(tiles)[gid] = v;
}

size_t signselect_smem(size_t n_bits) {
    return qk::ceil_div(n_bits, kChunkBits) * kChunkBits * sizeof(float);
}

// ------------------------------------------------------------------ launches
struct StageShape {
    size_t n_rows, n_bits, row_stride, n_groups, n_steps;
};

StageShape stage1_shape(const qk_layer *l) {
    return {l->r, l->din, l->vbt_stride, qk::ceil_div(l->r, kGroupRows),
            qk::ceil_div(l->din, kStepBits)};
}
StageShape stage2_shape(const qk_layer *l) {
    return {l->dout, l->r, l->ub_stride, qk::ceil_div(l->dout, kGroupRows),
            qk::ceil_div(l->r, kStepBits)};
}

qk_status launch_signselect(qk_ctx *c, const StageParams *many, size_t n_inst, const StageShape &s,
                            bool bf16) {
    size_t smem = signselect_smem(s.n_bits);
    dim3 grid((unsigned)qk::ceil_div(s.n_rows, kWarpsPerBlock * kRowsPerWarp), (unsigned)n_inst);
    auto kern = bf16 ? gemv_signselect_kernel<true> : gemv_signselect_kernel<false>;
    if (smem > 48 * 1024)
        QK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    (void)qk::launch_pdl(c->pdl, kern, grid, dim3(kWarpsPerBlock * 32), smem, c->stream, many,
                         (uint32_t)s.n_rows, (uint32_t)s.n_bits, (uint32_t)s.row_stride);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    return QK_OK;
}

// How one stage is cut into blocks and warps.
struct StagePlan {
    bool smem_digits;
    size_t warps_per_block, gpw, blocks, smem;
};

constexpr size_t kSmemBudget = 224 * 1024;
constexpr size_t kRingPerWarp = (size_t)kStages * kChunkBytes;

StagePlan plan_stage(const qk_ctx *c, const StageShape &s, size_t n_inst) {
    // Shared memory: the digit table (4 KB per k-step) plus a ring of kStages chunks per
    // warp.  Prefer 16 warps per block (one block per SM); use fewer warps when the table
    // is large, and read the table through L1 when it does not fit at all.
    StagePlan pl;
    const size_t table_bytes = s.n_steps * 4096;
    pl.smem_digits = table_bytes + 4 * kRingPerWarp <= kSmemBudget;
    pl.warps_per_block = 16;
    if (pl.smem_digits)
        while (table_bytes + pl.warps_per_block * kRingPerWarp > kSmemBudget)
            pl.warps_per_block -= 4;
    // Deal the row groups to warps: about eight chunks per warp keeps the ring in steady
    // state; with few instances, spread each one over more and smaller blocks instead.
    pl.gpw = s.n_steps >= 8 ? 1 : 8 / s.n_steps;
    if (pl.gpw > s.n_groups) pl.gpw = s.n_groups;
    pl.blocks = qk::ceil_div(qk::ceil_div(s.n_groups, pl.gpw), pl.warps_per_block);
    while (n_inst * pl.blocks < (size_t)c->sm_count && (pl.gpw > 1 || pl.warps_per_block > 4)) {
        if (pl.gpw > 1) pl.gpw = qk::ceil_div(pl.gpw, 2);
        else pl.warps_per_block /= 2;
        pl.blocks = qk::ceil_div(qk::ceil_div(s.n_groups, pl.gpw), pl.warps_per_block);
    }
    pl.smem = (pl.smem_digits ? table_bytes : 0) + pl.warps_per_block * kRingPerWarp;
    return pl;
}

bool fed_plan_fits(const qk_ctx *c, const StageShape &s, size_t n_inst, size_t *warps, size_t *smem);
constexpr size_t kSpreadTableSteps = 16;  // k-steps (of 512 inputs) from which the few-instance form gets its table made once

template <bool kFinal>
qk_status launch_bitslice(qk_ctx *c, const StageParams *many, size_t n_inst, const StageShape &s,
                          bool bf16, bool need_few = false) {
    const StagePlan pl = plan_stage(c, s, n_inst);
    // Few instances: the streaming form would leave most SMs idle and make each warp walk
    // its chunks in sequence.  Give every row group a block whose warps split the k-steps.
    size_t sk_warps = s.n_steps < 4 ? 4 : s.n_steps > 16 ? 16 : s.n_steps;
    auto sk_bytes = [&](size_t w) { return s.n_steps * 4096 + w * kRingPerWarp + w * 16 * 32 * 4; };
    while (sk_warps > 4 && sk_bytes(sk_warps) > kSmemBudget) --sk_warps;
    const size_t sk_smem = sk_bytes(sk_warps);
    const bool few = c->gemv_kernel != 3 && n_inst * pl.blocks < (size_t)c->sm_count && s.n_groups <= 65535;
    // A long input vector (the down projection's 14336 entries): every block of the few-instance
    // form would build the whole digit table for itself, about 10 us of the kernel's 16.  The
    // table is built once instead, by a small grid of its own that shares out the records, and
    // the stage's blocks only stream (the form fed plans use).  One more launch, half the time.
    size_t fed_warps, fed_smem;
    if (few && s.n_steps >= kSpreadTableSteps && n_inst <= 65535 && fed_plan_fits(c, s, n_inst, &fed_warps, &fed_smem)) {
        qk_status ts = launch_digit_table<kFinal>(c, many, n_inst, s.n_bits, s.n_steps, bf16);
        if (ts != QK_OK) return ts;
        auto gemv = bf16 ? gemv_bitslice_splitk_kernel<true, kFinal, true>
                         : gemv_bitslice_splitk_kernel<false, kFinal, true>;
        QK_CUDA(cudaFuncSetAttribute(gemv, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
        dim3 grid((unsigned)s.n_groups, (unsigned)n_inst);
        (void)qk::launch_pdl(c->pdl, gemv, grid, dim3((unsigned)fed_warps * 32), fed_smem, c->stream, many);
        QK_CUDA(cudaGetLastError());
        c->launches++;
        return QK_OK;
    }
    if (need_few && !(few && pl.smem_digits && sk_smem <= kSmemBudget && s.n_steps < kSpreadTableSteps))
        return qk::fail(QK_ERR_VALUE, "a plan that pushes its output into an all-reduce must fit the few-instance form");
    if (few && pl.smem_digits && sk_smem <= kSmemBudget) {
        dim3 grid((unsigned)s.n_groups, (unsigned)n_inst);
        auto gemv = bf16 ? gemv_bitslice_splitk_kernel<true, kFinal>
                         : gemv_bitslice_splitk_kernel<false, kFinal>;
        QK_CUDA(cudaFuncSetAttribute(gemv, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)kSmemBudget));
        (void)qk::launch_pdl(c->pdl, gemv, grid, dim3((unsigned)sk_warps * 32), sk_smem, c->stream, many);
        QK_CUDA(cudaGetLastError());
        c->launches++;
        return QK_OK;
    }
    if (!pl.smem_digits) {
        // too wide for shared memory: the table is made in global memory first
        qk_status ts = launch_digit_table<kFinal>(c, many, n_inst, s.n_bits, s.n_steps, bf16);
        if (ts != QK_OK) return ts;
    }
    dim3 grid((unsigned)pl.blocks, (unsigned)n_inst);
    auto gemv = pl.smem_digits ? (bf16 ? gemv_bitslice_kernel<true, kFinal, true>
                                       : gemv_bitslice_kernel<false, kFinal, true>)
                               : (bf16 ? gemv_bitslice_kernel<true, kFinal, false>
                                       : gemv_bitslice_kernel<false, kFinal, false>);
    QK_CUDA(cudaFuncSetAttribute(gemv, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kSmemBudget));
    (void)qk::launch_pdl(c->pdl, gemv, grid, dim3((unsigned)pl.warps_per_block * 32), pl.smem, c->stream,
                         many, (uint32_t)s.n_rows, (uint32_t)s.n_bits, (uint32_t)s.n_groups,
                         (uint32_t)s.n_steps, (uint32_t)pl.gpw);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    return QK_OK;
}

// The fused form applies when there are enough instances to give every SM a block of its
// own and both digit tables, t and the ring fit in shared memory together.
bool fused_plan(const qk_ctx *c, const StageShape &s1, const StageShape &s2, size_t n_inst,
                size_t *warps, size_t *t_bytes, size_t *table_bytes, size_t *smem) {
    if (n_inst < (size_t)c->sm_count) return false;
    const size_t table = (s1.n_steps > s2.n_steps ? s1.n_steps : s2.n_steps) * 4096;
    *t_bytes = qk::ceil_div(s1.n_rows * sizeof(double), 128) * 128;
    *table_bytes = table;
    // two 8-warp blocks per SM overlap one block's serial phases (table builds, the stage
    // boundary) with the other's streaming: measured 3.4 vs 3.1 TB/s for 16-warp blocks
    // (selector 4, for measurement: 4-warp blocks, three of which fit an SM at config 0)
    const size_t w_min = c->gemv_kernel == 4 ? 4 : 8;
    for (size_t w = (c->gemv_kernel == 2 || n_inst < 2 * (size_t)c->sm_count) ? 16 : w_min;
         w >= w_min; w -= 4) {
        if (*t_bytes + table + w * kRingPerWarp <= kSmemBudget) {
            *warps = w;
            *smem = *t_bytes + table + w * kRingPerWarp;
            return true;
        }
    }
    return false;
}

// The persistent streaming form applies when every SM gets at least one instance and the
// two double-buffered tables, the two t buffers and the consumer warps' rings fit in shared
// memory together.
constexpr size_t kPsSmemBudget = 227 * 1024 - 1024;  // (the kernel also holds 768 bytes of static shared memory)
struct PsPlan {
    size_t grid, slots, t_bytes, table1_bytes, table2_bytes, smem;
};
bool stream_plan(const qk_ctx *c, const StageShape &s1, const StageShape &s2, size_t n_inst,
                 PsPlan *pl) {
    if (n_inst < (size_t)c->sm_count) return false;
    pl->grid = (size_t)c->sm_count;
    pl->t_bytes = qk::ceil_div(s1.n_rows * sizeof(double), 128) * 128;
    pl->table1_bytes = s1.n_steps * 4096;
    pl->table2_bytes = s2.n_steps * 4096;
    pl->slots = (size_t)kPsConsumers * kPsDepth;
    pl->smem = pl->slots * kChunkBytes + 2 * (pl->table1_bytes + pl->table2_bytes + pl->t_bytes) +
               4 * sizeof(StageMeta) + (pl->slots + 6) * 8 + kPsBuilders * (8 + 8 + 4) + 16;
    if (pl->smem > kPsSmemBudget) return false;
    return true;
}

// Scratch one instance needs besides its inputs and outputs.
struct InstanceScratch {
    size_t t_bytes, dig1_bytes, dig2_bytes, meta_bytes, total;
};
InstanceScratch scratch_of(const qk_layer *l) {
    InstanceScratch s;
    s.t_bytes = qk::ceil_div(l->r * sizeof(double), 256) * 256;
    s.dig1_bytes = qk::ceil_div(l->din, kStepBits) * kStepBits * 8;
    s.dig2_bytes = qk::ceil_div(l->r, kStepBits) * kStepBits * 8;
    s.meta_bytes = 256;
    s.total = s.t_bytes + s.dig1_bytes + s.dig2_bytes + s.meta_bytes;
    return s;
}

qk_status check_group(qk_ctx *c, const qk_layer *const *layers, size_t n_layers) {
    const qk_layer *l0 = layers[0];
    for (size_t i = 0; i < n_layers; ++i) {
        const qk_layer *l = layers[i];
        if (!l) return qk::fail(QK_ERR_VALUE, "layer %zu is null", i);
        if (l->device != c->device)
            return qk::fail(QK_ERR_VALUE, "layer %zu lives on device %d, context on device %d", i,
                            l->device, c->device);
        if (l->dout != l0->dout || l->din != l0->din || l->r != l0->r || l->serving != l0->serving)
            return qk::fail(QK_ERR_VALUE,
                            "grouped layers must share one shape and serving dtype (layer %zu "
                            "differs from layer 0)",
                            i);
    }
    return QK_OK;
}

// Fills 2*n_inst StageParams (stage 1 entries, then stage 2 entries) for n_layers
// same-shape layers x n_tokens tokens.  Instance k = t*n_layers + i reads
// x + i*x_layer_stride + t*din and writes y + i*y_layer_stride + t*dout; its scratch is
// the k-th slice of `scratch`.
void fill_params(StageParams *h, const qk_layer *const *layers, size_t n_layers, size_t n_tokens,
                 const float *x_dev, float *y_dev, uint8_t *scratch, size_t x_layer_stride,
                 size_t y_layer_stride, const float *gate_up = nullptr, size_t scratch_stride = 0) {
    const size_t n_inst = n_layers * n_tokens;
    InstanceScratch sc = scratch_of(layers[0]);
    if (scratch_stride) sc.total = scratch_stride;
    for (size_t t = 0; t < n_tokens; ++t)
        for (size_t i = 0; i < n_layers; ++i) {
            const qk_layer *l = layers[i];
            size_t k = t * n_layers + i;
            uint8_t *base = scratch + k * sc.total;
            const InstanceScratch own = scratch_of(l);  // the slice's inner layout follows the layer
            void *t_buf = base;
            uint2 *dig1 = (uint2 *)(base + own.t_bytes);
            uint2 *dig2 = (uint2 *)(base + own.t_bytes + own.dig1_bytes);
            StageMeta *meta = (StageMeta *)(base + own.t_bytes + own.dig1_bytes + own.dig2_bytes);
            const float *x = x_dev + i * x_layer_stride + t * l->din;
            float *y = y_dev + i * y_layer_stride + t * l->dout;
            h[k] = StageParams{l->vbt, l->vbt_tiles, x, l->s2, t_buf, nullptr, nullptr, dig1, meta,
                               gate_up, (uint32_t)l->r, (uint32_t)l->din, dig2, meta + 1, nullptr};
            h[n_inst + k] = StageParams{l->ub, l->ub_tiles, t_buf, nullptr, y, l->s1, l->bias, dig2,
                                        meta + 1, nullptr, (uint32_t)l->dout, (uint32_t)l->r,
                                        nullptr, nullptr, nullptr};
        }
}

// A plan whose instances differ in shape runs in the few-instance (split-k) form only; `widest`
// carries the largest dimensions over the instances (din, r, dout separately).
bool mixed_plan_fits(const qk_ctx *c, const StageShape &s, size_t n_inst, size_t *warps, size_t *smem) {
    size_t sk_warps = s.n_steps < 4 ? 4 : s.n_steps > 16 ? 16 : s.n_steps;
    auto sk_bytes = [&](size_t w) { return s.n_steps * 4096 + w * kRingPerWarp + w * 16 * 32 * 4; };
    while (sk_warps > 4 && sk_bytes(sk_warps) > kSmemBudget) --sk_warps;
    *warps = sk_warps;
    *smem = sk_bytes(sk_warps);
    return *smem <= kSmemBudget && s.n_groups <= 65535 && n_inst <= 65535 &&
           n_inst * s.n_groups <= 8 * (size_t)c->sm_count;
}

template <bool kFinal>
qk_status launch_mixed_stage(qk_ctx *c, const StageParams *many, size_t n_inst, const StageShape &s,
                             bool bf16) {
    size_t warps, smem;
    if (!mixed_plan_fits(c, s, n_inst, &warps, &smem))
        return qk::fail(QK_ERR_VALUE, "a plan of mixed shapes must fit the few-instance form");
    auto gemv = bf16 ? gemv_bitslice_splitk_kernel<true, kFinal> : gemv_bitslice_splitk_kernel<false, kFinal>;
    QK_CUDA(cudaFuncSetAttribute(gemv, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
    dim3 grid((unsigned)s.n_groups, (unsigned)n_inst);
    (void)qk::launch_pdl(c->pdl, gemv, grid, dim3((unsigned)warps * 32), smem, c->stream, many);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    return QK_OK;
}

// Fed plans: both stages in the few-instance form without a table of their own.
bool fed_plan_fits(const qk_ctx *c, const StageShape &s, size_t n_inst, size_t *warps, size_t *smem) {
    size_t sk_warps = s.n_steps < 4 ? 4 : s.n_steps > 16 ? 16 : s.n_steps;
    *warps = sk_warps;
    *smem = sk_warps * kRingPerWarp + sk_warps * 16 * 32 * 4;
    return s.n_groups <= 65535 && n_inst <= 65535 && n_inst * s.n_groups <= 16 * (size_t)c->sm_count;
}

template <bool kFinal>
qk_status launch_fed_stage(qk_ctx *c, const StageParams *many, size_t n_inst, const StageShape &s,
                           bool bf16) {
    size_t warps, smem;
    if (!fed_plan_fits(c, s, n_inst, &warps, &smem))
        return qk::fail(QK_ERR_VALUE, "a fed plan must fit the few-instance form");
    auto gemv = bf16 ? gemv_bitslice_splitk_kernel<true, kFinal, true>
                     : gemv_bitslice_splitk_kernel<false, kFinal, true>;
    QK_CUDA(cudaFuncSetAttribute(gemv, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
    dim3 grid((unsigned)s.n_groups, (unsigned)n_inst);
    (void)qk::launch_pdl(c->pdl, gemv, grid, dim3((unsigned)warps * 32), smem, c->stream, many);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    return QK_OK;
}

// Stage 1 of a normed plan: the few-instance form with the norm kernel's 512 threads.
bool normed_plan_fits(const qk_ctx *c, const StageShape &s, size_t n_inst, size_t *smem) {
    constexpr size_t kWarps = 16;
    *smem = s.n_steps * 4096 + kWarps * kRingPerWarp + kWarps * 16 * 32 * 4;
    return *smem <= kSmemBudget && s.n_bits <= 16 * 512 && s.n_groups <= 65535 && n_inst <= 65535 &&
           n_inst * s.n_groups <= 8 * (size_t)c->sm_count;
}
qk_status launch_normed_stage1(qk_ctx *c, const StageParams *many, size_t n_inst, const StageShape &s, bool bf16) {
    size_t smem;
    if (!normed_plan_fits(c, s, n_inst, &smem))
        return qk::fail(QK_ERR_VALUE, "a normed plan must fit the few-instance form");
    auto gemv = bf16 ? gemv_bitslice_splitk_kernel<true, false> : gemv_bitslice_splitk_kernel<false, false>;
    QK_CUDA(cudaFuncSetAttribute(gemv, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBudget));
    dim3 grid((unsigned)s.n_groups, (unsigned)n_inst);
    (void)qk::launch_pdl(c->pdl, gemv, grid, dim3(512), smem, c->stream, many);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    return QK_OK;
}

qk_status launch_both(qk_ctx *c, const qk_layer *l0, const StageParams *d, size_t n_inst,
                      int kernel, bool mixed = false, bool fed = false, bool normed = false, bool pushed = false) {
    if (pushed && !normed && !fed) {
        // (the last stage pushes into the all-reduce inboxes: only the few-instance kernel does)
        const bool bf16 = l0->serving == QK_BF16;
        qk_status e = mixed ? launch_mixed_stage<false>(c, d, n_inst, stage1_shape(l0), bf16)
                            : launch_bitslice<false>(c, d, n_inst, stage1_shape(l0), bf16);
        if (e != QK_OK) return e;
        if (mixed) return launch_mixed_stage<true>(c, d + n_inst, n_inst, stage2_shape(l0), bf16);
        return launch_bitslice<true>(c, d + n_inst, n_inst, stage2_shape(l0), bf16, true);
    }
    if (pushed) return qk::fail(QK_ERR_VALUE, "a normed or fed plan cannot push into an all-reduce");
    if (normed) {
        const bool bf16 = l0->serving == QK_BF16;
        qk_status e = launch_normed_stage1(c, d, n_inst, stage1_shape(l0), bf16);
        if (e != QK_OK) return e;
        if (mixed) return launch_mixed_stage<true>(c, d + n_inst, n_inst, stage2_shape(l0), bf16);
        return launch_bitslice<true>(c, d + n_inst, n_inst, stage2_shape(l0), bf16);
    }
    if (fed) {
        qk_status e = launch_fed_stage<false>(c, d, n_inst, stage1_shape(l0), l0->serving == QK_BF16);
        if (e != QK_OK) return e;
        return launch_fed_stage<true>(c, d + n_inst, n_inst, stage2_shape(l0), l0->serving == QK_BF16);
    }
    if (mixed) {
        // l0 holds the largest din, r and dout over the instances
        qk_status e = launch_mixed_stage<false>(c, d, n_inst, stage1_shape(l0), l0->serving == QK_BF16);
        if (e != QK_OK) return e;
        return launch_mixed_stage<true>(c, d + n_inst, n_inst, stage2_shape(l0), l0->serving == QK_BF16);
    }
    const bool bf16 = l0->serving == QK_BF16;
    const StageShape s1 = stage1_shape(l0), s2 = stage2_shape(l0);
    qk_status st;
    if (kernel == 0) {
        if (signselect_smem(l0->din) > 200 * 1024 || signselect_smem(l0->r) > 200 * 1024)
            return qk::fail(QK_ERR_VALUE,
                            "input width %zu exceeds the sign-select kernel's staging limit",
                            l0->din > l0->r ? l0->din : l0->r);
        if ((st = launch_signselect(c, d, n_inst, s1, bf16)) != QK_OK) return st;
        return launch_signselect(c, d + n_inst, n_inst, s2, bf16);
    }
    // Many instances: one block per instance (below), or - selector 6, a measurement variant
    // that did not beat it - the persistent streaming form.
    if (kernel == 6) {
        PsPlan ps;
        if (stream_plan(c, s1, s2, n_inst, &ps)) {
            qk_status e = qk::error_word(c);
            if (e != QK_OK) return e;
            PsArgs a{d, d + n_inst, (uint32_t)n_inst, (uint32_t)l0->r, (uint32_t)l0->din,
                     (uint32_t)l0->dout,
                     c->wait_limit ? c->wait_limit : kPsWaitLimitDefault, (int *)c->d_err.ptr};
            auto kern = bf16 ? layer_stream_kernel<true> : layer_stream_kernel<false>;
            QK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kPsSmemBudget));
            (void)qk::launch_pdl(c->pdl, kern, dim3((unsigned)ps.grid), dim3(kPsThreads), ps.smem, c->stream,
                                 a, (uint32_t)ps.t_bytes, (uint32_t)ps.table1_bytes,
                                 (uint32_t)ps.table2_bytes);
            QK_CUDA(cudaGetLastError());
            c->launches++;
            c->err_armed = true;
            return QK_OK;
        }
    }
    size_t warps, t_bytes, table_bytes, smem;
    if (fused_plan(c, s1, s2, n_inst, &warps, &t_bytes, &table_bytes, &smem)) {
        auto fused = bf16 ? layer_bitslice_fused_kernel<true> : layer_bitslice_fused_kernel<false>;
        QK_CUDA(cudaFuncSetAttribute(fused, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)kSmemBudget));
        (void)qk::launch_pdl(c->pdl, fused, dim3((unsigned)n_inst), dim3((unsigned)warps * 32), smem,
                             c->stream, d, d + n_inst, (uint32_t)l0->r, (uint32_t)l0->din,
                             (uint32_t)l0->dout, (uint32_t)t_bytes, (uint32_t)table_bytes,
                             (uint32_t)qk::ceil_div(s1.n_groups, warps),
                             (uint32_t)qk::ceil_div(s2.n_groups, warps));
        QK_CUDA(cudaGetLastError());
        c->launches++;
        return QK_OK;
    }
    if ((st = launch_bitslice<false>(c, d, n_inst, s1, bf16)) != QK_OK) return st;
    return launch_bitslice<true>(c, d + n_inst, n_inst, s2, bf16);
}

// Both stages for n_layers same-shape layers x n_tokens tokens, parameters built and
// uploaded on the fly.
qk_status apply_group(qk_ctx *c, const qk_layer *const *layers, size_t n_layers, const float *x_dev,
                      float *y_dev, size_t n_tokens, size_t x_layer_stride, size_t y_layer_stride) {
    qk_status st = check_group(c, layers, n_layers);
    if (st != QK_OK) return st;
    const qk_layer *l0 = layers[0];
    const size_t n_inst = n_layers * n_tokens;
    if (n_inst > 65535)
        return qk::fail(QK_ERR_VALUE, "%zu layer-token instances exceed one launch (65535)", n_inst);
    const InstanceScratch sc = scratch_of(l0);
    if ((st = c->d_t.reserve(n_inst * sc.total)) != QK_OK) return st;
    if ((st = c->d_ptrs.reserve(2 * n_inst * sizeof(StageParams))) != QK_OK) return st;
    void *hp;
    int slot;
    // (no host-side wait here: the pinned blocks form a ring guarded by events, and the device
    // buffers below are reused in stream order)
    if ((st = c->pinned(2 * n_inst * sizeof(StageParams), &hp, &slot)) != QK_OK) return st;
    fill_params((StageParams *)hp, layers, n_layers, n_tokens, x_dev, y_dev, (uint8_t *)c->d_t.ptr,
                x_layer_stride, y_layer_stride);
    StageParams *d = (StageParams *)c->d_ptrs.ptr;
    QK_CUDA(cudaMemcpyAsync(d, hp, 2 * n_inst * sizeof(StageParams), cudaMemcpyHostToDevice,
                            c->stream));
    if ((st = c->pinned_done(slot)) != QK_OK) return st;
    return launch_both(c, l0, d, n_inst, c->gemv_kernel);
}

// What the host hands over for one factor: its rows already separated (row_words bytes each),
// or the container's bit stream of the factor / of its transpose.
enum FactorForm { kFormRows, kFormStream, kFormStreamTransposed };

qk_status upload_factor(qk_ctx *c, const uint8_t *host, size_t len, size_t n_rows, size_t n_bits,
                        uint8_t **rows_out, size_t *stride_out, uint8_t **tiles_out,
                        FactorForm form = kFormRows) {
    size_t row_words = qk::ceil_div(n_bits, 8);
    size_t stride = qk::ceil_div(row_words, 16) * 16;
    size_t n_groups = qk::ceil_div(n_rows, kGroupRows), n_steps = qk::ceil_div(n_bits, kStepBits);
    qk_status st;
    if ((st = c->d_packed.reserve(len)) != QK_OK) return st;
    uint8_t *rows = nullptr, *tiles = nullptr;
    cudaError_t e = cudaMalloc(&rows, n_rows * stride);
    if (e == cudaSuccess) e = cudaMalloc(&tiles, n_groups * n_steps * kChunkBytes);
    if (e != cudaSuccess) {
        if (rows) cudaFree(rows);
        return qk::fail(QK_ERR_ALLOC, "device allocation of %zu bytes failed: %s",
                        n_rows * stride + n_groups * n_steps * kChunkBytes, cudaGetErrorString(e));
    }
    *rows_out = rows;
    *tiles_out = tiles;
    *stride_out = stride;
    QK_CUDA(cudaMemcpyAsync(c->d_packed.ptr, host, len, cudaMemcpyHostToDevice, c->stream));
    size_t total = n_rows * stride;
    if (form == kFormRows)
        pad_rows_kernel<<<(unsigned)qk::ceil_div(total, 256), 256, 0, c->stream>>>(
            (const uint8_t *)c->d_packed.ptr, rows, (uint32_t)n_rows, (uint32_t)n_bits,
            (uint32_t)row_words, (uint32_t)stride);
    else if (form == kFormStream)
        stream_rows_kernel<<<(unsigned)qk::ceil_div(total / 16, 256), 256, 0, c->stream>>>(
            (const uint8_t *)c->d_packed.ptr, len, rows, (uint32_t)n_rows, (uint32_t)n_bits,
            (uint32_t)stride);
    else
        stream_rows_transposed_kernel<<<(unsigned)qk::ceil_div(total / 16, 256), 256, 0,
                                        c->stream>>>((const uint8_t *)c->d_packed.ptr, rows,
                                                     (uint32_t)n_bits, (uint32_t)n_rows,
                                                     (uint32_t)stride);
    QK_CUDA(cudaGetLastError());
    size_t pieces = n_groups * n_steps * 256;
    tile_rows_kernel<<<(unsigned)qk::ceil_div(pieces, 256), 256, 0, c->stream>>>(
        rows, tiles, (uint32_t)n_rows, (uint32_t)stride, (uint32_t)n_groups, (uint32_t)n_steps);
    QK_CUDA(cudaGetLastError());
    c->launches += 2;
    QK_CUDA(cudaStreamSynchronize(c->stream));
    return QK_OK;
}

qk_status upload_f32(qk_ctx *c, const float *host, size_t n, float **out) {
    float *d = nullptr;
    cudaError_t e = cudaMalloc(&d, n * sizeof(float));
    if (e != cudaSuccess)
        return qk::fail(QK_ERR_ALLOC, "device allocation of %zu bytes failed: %s",
                        n * sizeof(float), cudaGetErrorString(e));
    *out = d;
    QK_CUDA(cudaMemcpyAsync(d, host, n * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    QK_CUDA(cudaStreamSynchronize(c->stream));
    return QK_OK;
}

}  // namespace

extern "C" {

static qk_status layer_create(qk_ctx *ctx, bool streams, const uint8_t *ub_rows, size_t ub_len,
                              const uint8_t *vb_t_rows, size_t vb_t_len, size_t dout, size_t din,
                              size_t r, const float *s1, const float *s2, const float *bias,
                              int32_t serving_dtype, qk_layer **out) {
    if (!out) return qk::fail(QK_ERR_VALUE, "qk_layer_create: out is null");
    *out = nullptr;
    if (serving_dtype != QK_F32 && serving_dtype != QK_BF16)
        return qk::fail(QK_ERR_VALUE, "serving dtype must be float32 or bfloat16, got tag %d",
                        serving_dtype);
    if (dout == 0 || din == 0 || r == 0)
        return qk::fail(QK_ERR_VALUE, "layer dimensions must be positive: dout=%zu din=%zu r=%zu",
                        dout, din, r);
    if (streams) {
        // engine/mod.rs:258-289: a container stream holds exactly its matrix's bits
        if (ub_len != qk::ceil_div(dout * r, 8))
            return qk::fail(QK_ERR_VALUE, "container stream holds %zu bytes; %zux%zu bits need %zu",
                            ub_len, dout, r, qk::ceil_div(dout * r, 8));
        if (vb_t_len != qk::ceil_div(din * r, 8))
            return qk::fail(QK_ERR_VALUE, "container stream holds %zu bytes; %zux%zu bits need %zu",
                            vb_t_len, din, r, qk::ceil_div(din * r, 8));
    } else if (ub_len != dout * qk::ceil_div(r, 8) || vb_t_len != r * qk::ceil_div(din, 8)) {
        // engine/mod.rs:343-356: both bitplanes must have the per-row layout's exact length
        return qk::fail(QK_ERR_VALUE, "bitplane length mismatch after repack");
    }
    if ((uint64_t)dout * qk::ceil_div(r, 8) > qk::kIndexCeiling ||
        (uint64_t)r * qk::ceil_div(din, 8) > qk::kIndexCeiling)
        return qk::fail(QK_ERR_VALUE, "layer exceeds the device u32 index ceiling (%llu)",
                        (unsigned long long)qk::kIndexCeiling);
    if (din > (1u << 16) || r > (1u << 16))
        return qk::fail(QK_ERR_VALUE,
                        "reduction width %zu exceeds the int32 digit accumulator's 65536-term "
                        "bound",
                        din > r ? din : r);
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    qk_layer *l = new qk_layer();
    l->device = c->device;
    l->dout = dout;
    l->din = din;
    l->r = r;
    l->serving = serving_dtype;
    st = upload_factor(c, ub_rows, ub_len, dout, r, &l->ub, &l->ub_stride, &l->ub_tiles,
                       streams ? kFormStream : kFormRows);
    if (st == QK_OK)
        st = upload_factor(c, vb_t_rows, vb_t_len, r, din, &l->vbt, &l->vbt_stride, &l->vbt_tiles,
                           streams ? kFormStreamTransposed : kFormRows);
    if (st == QK_OK) st = upload_f32(c, s1, dout, &l->s1);
    if (st == QK_OK) st = upload_f32(c, s2, din, &l->s2);
    if (st == QK_OK && bias) st = upload_f32(c, bias, dout, &l->bias);
    if (st != QK_OK) {
        qk_layer_free(l);
        return st;
    }
    *out = l;
    return QK_OK;
}

qk_status qk_layer_create(qk_ctx *ctx, const uint8_t *ub_rows, size_t ub_len,
                          const uint8_t *vb_t_rows, size_t vb_t_len, size_t dout, size_t din,
                          size_t r, const float *s1, const float *s2, const float *bias,
                          int32_t serving_dtype, qk_layer **out) {
    return layer_create(ctx, false, ub_rows, ub_len, vb_t_rows, vb_t_len, dout, din, r, s1, s2, bias,
                        serving_dtype, out);
}

qk_status qk_layer_create_from_streams(qk_ctx *ctx, const uint8_t *ub_stream, size_t ub_len,
                                       const uint8_t *vb_stream, size_t vb_len, size_t dout,
                                       size_t din, size_t r, const float *s1, const float *s2,
                                       const float *bias, int32_t serving_dtype, qk_layer **out) {
    return layer_create(ctx, true, ub_stream, ub_len, vb_stream, vb_len, dout, din, r, s1, s2, bias,
                        serving_dtype, out);
}

qk_status qk_gpu_container_to_rows(qk_ctx *ctx, const uint8_t *stream, size_t stream_len,
                                   size_t n_rows, size_t r, int32_t transposed, uint8_t *out,
                                   size_t out_len) {
    // the stream holds n_rows x r bits; the result has n_rows rows of r bits, or (transposed)
    // r rows of n_rows bits
    const size_t res_rows = transposed ? r : n_rows, res_bits = transposed ? n_rows : r;
    const size_t row_words = qk::ceil_div(res_bits, 8);
    if (stream_len != qk::ceil_div(n_rows * r, 8))
        return qk::fail(QK_ERR_VALUE, "container stream holds %zu bytes; %zux%zu bits need %zu",
                        stream_len, n_rows, r, qk::ceil_div(n_rows * r, 8));
    if (out_len != res_rows * row_words)
        return qk::fail(QK_ERR_VALUE, "output length %zu does not match %zu rows x %zu bitplanes",
                        out_len, res_rows, row_words);
    if (out_len == 0) return QK_OK;
    if ((uint64_t)res_rows * row_words > qk::kIndexCeiling)
        return qk::fail(QK_ERR_VALUE, "layer exceeds the device u32 index ceiling (%llu)",
                        (unsigned long long)qk::kIndexCeiling);
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    uint8_t *rows = nullptr, *tiles = nullptr;
    size_t stride = 0;
    st = upload_factor(c, stream, stream_len, res_rows, res_bits, &rows, &stride, &tiles,
                       transposed ? kFormStreamTransposed : kFormStream);
    if (st == QK_OK) {
        cudaError_t e = cudaMemcpy2D(out, row_words, rows, stride, row_words, res_rows,
                                     cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) st = qk::fail(QK_ERR_CUDA, "cudaMemcpy2D: %s", cudaGetErrorString(e));
    }
    if (rows) cudaFree(rows);
    if (tiles) cudaFree(tiles);
    return st;
}

void qk_layer_free(qk_layer *l) {
    if (!l) return;
    cudaSetDevice(l->device);
    if (l->ub) cudaFree(l->ub);
    if (l->vbt) cudaFree(l->vbt);
    if (l->ub_tiles) cudaFree(l->ub_tiles);
    if (l->vbt_tiles) cudaFree(l->vbt_tiles);
    if (l->s1) cudaFree(l->s1);
    if (l->s2) cudaFree(l->s2);
    if (l->bias) cudaFree(l->bias);
    delete l;
}

qk_status qk_layer_apply(qk_ctx *ctx, const qk_layer *layer, const float *x_dev, size_t n_tokens,
                         float *y_dev) {
    if (!layer) return qk::fail(QK_ERR_VALUE, "qk_layer_apply: layer is null");
    if (n_tokens == 0) return QK_OK;
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    return apply_group(c, &layer, 1, x_dev, y_dev, n_tokens, 0, 0);
}

qk_status qk_layer_apply_host(qk_ctx *ctx, const qk_layer *layer, const float *x, size_t x_len,
                              float *y, size_t y_len) {
    if (!layer) return qk::fail(QK_ERR_VALUE, "qk_layer_apply_host: layer is null");
    // engine/mod.rs:399-406
    if (x_len != layer->din)
        return qk::fail(QK_ERR_VALUE, "layer expects input dim %zu, got %zu", layer->din, x_len);
    if (y_len != layer->dout)
        return qk::fail(QK_ERR_VALUE, "layer produces output dim %zu, got a buffer of %zu",
                        layer->dout, y_len);
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    if ((st = c->d_in.reserve(x_len * sizeof(float))) != QK_OK) return st;
    if ((st = c->d_out.reserve(y_len * sizeof(float))) != QK_OK) return st;
    QK_CUDA(cudaMemcpyAsync(c->d_in.ptr, x, x_len * sizeof(float), cudaMemcpyHostToDevice,
                            c->stream));
    st = apply_group(c, &layer, 1, (const float *)c->d_in.ptr, (float *)c->d_out.ptr, 1, 0, 0);
    if (st != QK_OK) return st;
    QK_CUDA(cudaMemcpyAsync(y, c->d_out.ptr, y_len * sizeof(float), cudaMemcpyDeviceToHost,
                            c->stream));
    QK_CUDA(cudaStreamSynchronize(c->stream));
    return QK_OK;
}

qk_status qk_layers_apply_group(qk_ctx *ctx, const qk_layer *const *layers, size_t n_layers,
                                const float *x_dev, float *y_dev) {
    if (n_layers == 0) return QK_OK;
    if (!layers || !layers[0])
        return qk::fail(QK_ERR_VALUE, "qk_layers_apply_group: layers is null");
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    return apply_group(c, layers, n_layers, x_dev, y_dev, 1, layers[0]->din, layers[0]->dout);
}

qk_status qk_group_create(qk_ctx *ctx, const qk_layer *const *layers, size_t n_layers,
                          const float *x_dev, float *y_dev, qk_group **out) {
    if (!out) return qk::fail(QK_ERR_VALUE, "qk_group_create: out is null");
    *out = nullptr;
    if (n_layers == 0 || !layers || !layers[0])
        return qk::fail(QK_ERR_VALUE, "qk_group_create: no layers");
    if (n_layers > 65535)
        return qk::fail(QK_ERR_VALUE, "%zu layers exceed one launch (65535)", n_layers);
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    if ((st = check_group(c, layers, n_layers)) != QK_OK) return st;
    const qk_layer *l0 = layers[0];
    qk_group *g = new qk_group();
    g->device = c->device;
    g->n_inst = n_layers;
    g->shape = *l0;  // dimensions and strides only; the pointers are not used
    const InstanceScratch sc = scratch_of(l0);
    cudaError_t e = cudaMalloc(&g->scratch, n_layers * sc.total);
    if (e == cudaSuccess) e = cudaMalloc(&g->params, 2 * n_layers * sizeof(StageParams));
    if (e != cudaSuccess) {
        qk_group_free(g);
        return qk::fail(QK_ERR_ALLOC, "device allocation for a layer group failed: %s",
                        cudaGetErrorString(e));
    }
    std::vector<StageParams> h(2 * n_layers);
    fill_params(h.data(), layers, n_layers, 1, x_dev, y_dev, (uint8_t *)g->scratch, l0->din,
                l0->dout);
    QK_CUDA(cudaMemcpyAsync(g->params, h.data(), h.size() * sizeof(StageParams),
                            cudaMemcpyHostToDevice, c->stream));
    QK_CUDA(cudaStreamSynchronize(c->stream));
    *out = g;
    return QK_OK;
}

static qk_status plan_create(qk_ctx *ctx, const qk_layer *const *layers, const float *const *x_ptrs,
                             const float *const *x2_ptrs, float *const *y_ptrs, size_t n_inst,
                             qk_group **out) {
    if (!out) return qk::fail(QK_ERR_VALUE, "qk_plan_create: out is null");
    *out = nullptr;
    if (n_inst == 0 || !layers || !x_ptrs || !y_ptrs || !layers[0])
        return qk::fail(QK_ERR_VALUE, "qk_plan_create: no instances");
    if (n_inst > 65535)
        return qk::fail(QK_ERR_VALUE, "%zu instances exceed one launch (65535)", n_inst);
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    const qk_layer *l0 = layers[0];
    // instances may differ in shape (q beside k and v) as long as they share the serving dtype
    // and the whole plan fits the few-instance form
    qk_layer widest = *l0;
    bool mixed = false;
    size_t slice = 0;
    for (size_t i = 0; i < n_inst; ++i) {
        const qk_layer *l = layers[i];
        if (!l) return qk::fail(QK_ERR_VALUE, "layer %zu is null", i);
        if (l->device != c->device)
            return qk::fail(QK_ERR_VALUE, "layer %zu lives on device %d, context on device %d", i,
                            l->device, c->device);
        if (l->serving != l0->serving)
            return qk::fail(QK_ERR_VALUE, "planned layers must share one serving dtype (layer %zu "
                            "differs from layer 0)", i);
        if (l->dout != l0->dout || l->din != l0->din || l->r != l0->r) mixed = true;
        if (l->dout > widest.dout) widest.dout = l->dout;
        if (l->din > widest.din) widest.din = l->din;
        if (l->r > widest.r) widest.r = l->r;
        const size_t need = scratch_of(l).total;
        if (need > slice) slice = need;
    }
    if (mixed) {
        size_t warps, smem;
        if (!mixed_plan_fits(c, stage1_shape(&widest), n_inst, &warps, &smem) ||
            !mixed_plan_fits(c, stage2_shape(&widest), n_inst, &warps, &smem))
            return qk::fail(QK_ERR_VALUE,
                            "planned layers of different shapes must fit the few-instance form "
                            "(%zu instances, up to %zu x %zu rank %zu)",
                            n_inst, widest.dout, widest.din, widest.r);
    }
    qk_group *g = new qk_group();
    g->device = c->device;
    g->n_inst = n_inst;
    g->shape = widest;  // dimensions only (the largest over the instances); the pointers are not used
    g->mixed = mixed;
    cudaError_t e = cudaMalloc(&g->scratch, n_inst * slice);
    if (e == cudaSuccess) e = cudaMalloc(&g->params, 2 * n_inst * sizeof(StageParams));
    if (e != cudaSuccess) {
        qk_group_free(g);
        return qk::fail(QK_ERR_ALLOC, "device allocation for a layer plan failed: %s",
                        cudaGetErrorString(e));
    }
    std::vector<StageParams> h(2 * n_inst);
    // fill_params writes {stage 1, stage 2} adjacently for n_inst == 1; regroup so that all
    // stage-1 records come first
    for (size_t k = 0; k < n_inst; ++k) {
        StageParams pair[2];
        const qk_layer *one = layers[k];
        fill_params(pair, &one, 1, 1, x_ptrs[k], y_ptrs[k], (uint8_t *)g->scratch + k * slice, 0, 0,
                    x2_ptrs ? x2_ptrs[k] : nullptr, slice);
        h[k] = pair[0];
        h[n_inst + k] = pair[1];
    }
    QK_CUDA(cudaMemcpyAsync(g->params, h.data(), h.size() * sizeof(StageParams),
                            cudaMemcpyHostToDevice, c->stream));
    QK_CUDA(cudaStreamSynchronize(c->stream));
    *out = g;
    return QK_OK;
}

qk_status qk_plan_create(qk_ctx *ctx, const qk_layer *const *layers, const float *const *x_ptrs,
                         float *const *y_ptrs, size_t n_inst, qk_group **out) {
    return plan_create(ctx, layers, x_ptrs, nullptr, y_ptrs, n_inst, out);
}

qk_status qk_plan_create_gated(qk_ctx *ctx, const qk_layer *const *layers,
                               const float *const *gate_ptrs, const float *const *up_ptrs,
                               float *const *y_ptrs, size_t n_inst, qk_group **out) {
    if (!up_ptrs) return qk::fail(QK_ERR_VALUE, "qk_plan_create_gated: up_ptrs is null");
    return plan_create(ctx, layers, gate_ptrs, up_ptrs, y_ptrs, n_inst, out);
}

qk_status qk_plan_set_norm(qk_ctx *ctx, qk_group *plan, const float *const *residual_ptrs,
                           const float *norm_weight, float eps, float *const *x_out_ptrs) {
    if (!plan || !norm_weight) return qk::fail(QK_ERR_VALUE, "qk_plan_set_norm: plan and norm_weight must be given");
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    if (plan->device != c->device)
        return qk::fail(QK_ERR_VALUE, "plan lives on device %d, context on device %d", plan->device, c->device);
    if (plan->fed) return qk::fail(QK_ERR_VALUE, "a fed plan takes its input from a producer: it cannot be normed");
    if (plan->shape.serving != QK_F32 && plan->shape.serving != QK_BF16)
        return qk::fail(QK_ERR_VALUE, "normed plans exist for float32 and bfloat16 serving");
    const size_t n = plan->n_inst;
    size_t smem;
    if (!normed_plan_fits(c, stage1_shape(&plan->shape), n, &smem))
        return qk::fail(QK_ERR_VALUE,
                        "a plan of %zu instances over %zu inputs does not fit the normed form (the few-instance "
                        "kernel with 512 threads, at most 8192 inputs)", n, plan->shape.din);
    std::vector<StageParams> h(n);
    QK_CUDA(cudaMemcpy(h.data(), plan->params, n * sizeof(StageParams), cudaMemcpyDeviceToHost));
    for (size_t k = 0; k < n; ++k) {
        if (h[k].in_gate_up) return qk::fail(QK_ERR_VALUE, "a gated plan cannot be normed");
        h[k].norm_w = norm_weight;
        h[k].in_residual = residual_ptrs ? residual_ptrs[k] : nullptr;
        h[k].x_out = x_out_ptrs ? x_out_ptrs[k] : nullptr;
        h[k].norm_eps = eps;
        if (h[k].x_out && h[k].x_out == h[k].in)
            return qk::fail(QK_ERR_VALUE, "a normed plan cannot update the residual stream in place (every "
                            "block reads it): x_out must be another buffer than the input");
    }
    QK_CUDA(cudaMemcpy(plan->params, h.data(), n * sizeof(StageParams), cudaMemcpyHostToDevice));
    plan->normed = true;
    return QK_OK;
}

qk_status qk_plan_set_allreduce(qk_ctx *ctx, qk_group *plan, int32_t gather, const uint64_t *inbox_bases,
                                int32_t rank, int32_t world, size_t total_words, const uint32_t *token_of_instance,
                                size_t d, uint32_t *state_dev) {
    if (!plan || !inbox_bases || !token_of_instance || !state_dev)
        return qk::fail(QK_ERR_VALUE, "qk_plan_set_allreduce: plan, inboxes, tokens and state must be given");
    if (world < 2 || world > 8 || rank < 0 || rank >= world)
        return qk::fail(QK_ERR_VALUE, "qk_plan_set_allreduce: rank %d of %d (2 to 8 ranks)", rank, world);
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    if (plan->device != c->device)
        return qk::fail(QK_ERR_VALUE, "plan lives on device %d, context on device %d", plan->device, c->device);
    if ((st = qk::error_word(c)) != QK_OK) return st;
    const size_t n = plan->n_inst;
    if (total_words == 0 || d == 0 || total_words % d != 0 || (uint64_t)world * total_words >= (1ull << 32))
        return qk::fail(QK_ERR_VALUE, "qk_plan_set_allreduce: %zu inbox words per rank for rows of %zu", total_words, d);
    if (gather && (!plan->normed || d > 4096 || plan->shape.din != d))
        return qk::fail(QK_ERR_VALUE, "a plan gathers an all-reduce as the residual of its norm: it must be a normed "
                        "plan over the %zu-entry stream (at most 4096 entries)", d);
    if (!gather && (plan->normed || plan->fed))
        return qk::fail(QK_ERR_VALUE, "a normed or fed plan cannot push into an all-reduce");
    std::vector<StageParams> h(2 * n);
    QK_CUDA(cudaMemcpy(h.data(), plan->params, h.size() * sizeof(StageParams), cudaMemcpyDeviceToHost));
    for (size_t k = 0; k < n; ++k) {
        if ((size_t)token_of_instance[k] * d >= total_words)
            return qk::fail(QK_ERR_VALUE, "instance %zu: token %u is outside the inbox", k, token_of_instance[k]);
        StageParams &p = gather ? h[k] : h[n + k];
        if (!gather && p.n_rows != d)
            return qk::fail(QK_ERR_VALUE, "instance %zu writes %u outputs, the all-reduced stream has %zu", k, p.n_rows, d);
        if (gather) {
            p.ar_inbox = reinterpret_cast<const unsigned long long *>(inbox_bases[0]);
        } else {
            for (int r = 0; r < world; ++r) p.ar_push[r] = reinterpret_cast<unsigned long long *>(inbox_bases[r]);
        }
        p.ar_state = state_dev;
        p.ar_error = (int *)c->d_err.ptr;
        p.ar_rank = (uint32_t)rank;
        p.ar_world = (uint32_t)world;
        p.ar_total = (uint32_t)total_words;
        p.ar_offset = (uint32_t)(token_of_instance[k] * d);
        p.ar_poll_limit = c->wait_limit ? c->wait_limit : (1u << 22);
    }
    QK_CUDA(cudaMemcpy(plan->params, h.data(), h.size() * sizeof(StageParams), cudaMemcpyHostToDevice));
    (gather ? plan->gathered : plan->pushed) = true;
    if (gather) plan->ar_poll_limit = c->wait_limit ? c->wait_limit : (1u << 22);
    return QK_OK;
}

qk_status qk_plan_feed_targets(qk_ctx *ctx, qk_group *plan, const void **targets_dev,
                               size_t *n_targets) {
    if (!plan || !targets_dev || !n_targets)
        return qk::fail(QK_ERR_VALUE, "qk_plan_feed_targets: null argument");
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    if (plan->device != c->device)
        return qk::fail(QK_ERR_VALUE, "plan lives on device %d, context on device %d", plan->device,
                        c->device);
    const size_t n = plan->n_inst;
    if (!plan->feed) {
        size_t warps, smem;
        if (!fed_plan_fits(c, stage1_shape(&plan->shape), n, &warps, &smem) ||
            !fed_plan_fits(c, stage2_shape(&plan->shape), n, &warps, &smem))
            return qk::fail(QK_ERR_VALUE, "a plan of %zu instances is too large to be fed: its "
                            "stages must fit the few-instance form", n);
        std::vector<StageParams> h(2 * n);
        QK_CUDA(cudaMemcpy(h.data(), plan->params, h.size() * sizeof(StageParams), cudaMemcpyDeviceToHost));
        cudaError_t e = cudaMalloc(&plan->feed, n * sizeof(FeedTarget));
        if (e == cudaSuccess) e = cudaMalloc(&plan->tickets, n * sizeof(uint32_t));
        if (e != cudaSuccess)
            return qk::fail(QK_ERR_ALLOC, "device allocation for a fed plan failed: %s", cudaGetErrorString(e));
        QK_CUDA(cudaMemset(plan->tickets, 0, n * sizeof(uint32_t)));
        std::vector<FeedTarget> targets(n);
        for (size_t k = 0; k < n; ++k) {
            targets[k] = FeedTarget{h[k].in_scale, h[k].digits, h[k].meta, h[k].n_bits,
                                    (uint32_t)qk::ceil_div(h[k].n_bits, kStepBits)};
            h[k].ticket = (uint32_t *)plan->tickets + k;
        }
        QK_CUDA(cudaMemcpy(plan->feed, targets.data(), n * sizeof(FeedTarget), cudaMemcpyHostToDevice));
        QK_CUDA(cudaMemcpy(plan->params, h.data(), h.size() * sizeof(StageParams), cudaMemcpyHostToDevice));
        plan->fed = true;
    }
    *targets_dev = plan->feed;
    *n_targets = n;
    return QK_OK;
}

qk_status qk_group_apply(qk_ctx *ctx, const qk_group *group) {
    if (!group) return qk::fail(QK_ERR_VALUE, "qk_group_apply: group is null");
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    if (group->device != c->device)
        return qk::fail(QK_ERR_VALUE, "group lives on device %d, context on device %d",
                        group->device, c->device);
    if ((group->pushed || group->gathered) && (c->gemv_kernel == 0 || c->gemv_kernel == 3))
        return qk::fail(QK_ERR_VALUE, "plans that take part in an all-reduce need the bit-sliced few-instance kernels");
    if (group->pushed || group->gathered) {
        qk_status e = qk::error_word(c);
        if (e != QK_OK) return e;
        c->err_armed = true;
    }
    if (group->gathered) {
        // the polls' limit lives in the plan's parameter records: follow qk_set_wait_limit
        const uint32_t want = c->wait_limit ? c->wait_limit : (1u << 22);
        if (group->ar_poll_limit != want) {
            std::vector<StageParams> h(group->n_inst);
            QK_CUDA(cudaMemcpy(h.data(), group->params, h.size() * sizeof(StageParams), cudaMemcpyDeviceToHost));
            for (auto &p : h) p.ar_poll_limit = want;
            QK_CUDA(cudaMemcpy(group->params, h.data(), h.size() * sizeof(StageParams), cudaMemcpyHostToDevice));
            const_cast<qk_group *>(group)->ar_poll_limit = want;
        }
    }
    return launch_both(c, &group->shape, (const StageParams *)group->params, group->n_inst,
                       c->gemv_kernel, group->mixed, group->fed, group->normed, group->pushed);
}

qk_status qk_groups_apply_host(qk_ctx *ctx, const qk_group *const *groups, const size_t *first_row,
                               size_t n_groups, const float *x_host, float *y_host, float *x_dev,
                               float *y_dev, size_t din, size_t dout) {
    if (!groups || !first_row || !x_host || !y_host || !x_dev || !y_dev || n_groups == 0)
        return qk::fail(QK_ERR_VALUE, "qk_groups_apply_host: groups, rows and buffers must be given");
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    for (size_t p = 0; p < n_groups; ++p) {
        if (!groups[p]) return qk::fail(QK_ERR_VALUE, "qk_groups_apply_host: group %zu is null", p);
        if (groups[p]->device != c->device)
            return qk::fail(QK_ERR_VALUE, "group lives on device %d, context on device %d",
                            groups[p]->device, c->device);
        if (first_row[p + 1] - first_row[p] != groups[p]->n_inst)
            return qk::fail(QK_ERR_VALUE, "group %zu holds %zu instances, its rows say %zu", p,
                            groups[p]->n_inst, first_row[p + 1] - first_row[p]);
    }
    if (!c->up_stream) QK_CUDA(cudaStreamCreateWithFlags(&c->up_stream, cudaStreamNonBlocking));
    if (!c->down_stream) QK_CUDA(cudaStreamCreateWithFlags(&c->down_stream, cudaStreamNonBlocking));
    while (c->pipe_events.size() < 2 * n_groups + 1) {
        cudaEvent_t e;
        QK_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        c->pipe_events.push_back(e);
    }
    // what is on the launch stream already (a previous step's kernels) no longer reads x_dev or
    // writes y_dev once this event has passed
    cudaEvent_t before = c->pipe_events[2 * n_groups];
    QK_CUDA(cudaEventRecord(before, c->stream));
    QK_CUDA(cudaStreamWaitEvent(c->up_stream, before, 0));
    QK_CUDA(cudaStreamWaitEvent(c->down_stream, before, 0));
    for (size_t p = 0; p < n_groups; ++p) {
        const size_t lo = first_row[p], n = first_row[p + 1] - lo;
        cudaEvent_t uploaded = c->pipe_events[2 * p], computed = c->pipe_events[2 * p + 1];
        QK_CUDA(cudaMemcpyAsync(x_dev + lo * din, x_host + lo * din, n * din * sizeof(float),
                                cudaMemcpyHostToDevice, c->up_stream));
        QK_CUDA(cudaEventRecord(uploaded, c->up_stream));
        QK_CUDA(cudaStreamWaitEvent(c->stream, uploaded, 0));
        st = launch_both(c, &groups[p]->shape, (const StageParams *)groups[p]->params, groups[p]->n_inst,
                         c->gemv_kernel, groups[p]->mixed, groups[p]->fed);
        if (st != QK_OK) return st;
        QK_CUDA(cudaEventRecord(computed, c->stream));
        QK_CUDA(cudaStreamWaitEvent(c->down_stream, computed, 0));
        QK_CUDA(cudaMemcpyAsync(y_host + lo * dout, y_dev + lo * dout, n * dout * sizeof(float),
                                cudaMemcpyDeviceToHost, c->down_stream));
    }
    QK_CUDA(cudaStreamSynchronize(c->down_stream));
    return QK_OK;
}

void qk_group_free(qk_group *g) {
    if (!g) return;
    cudaSetDevice(g->device);
    if (g->scratch) cudaFree(g->scratch);
    if (g->params) cudaFree(g->params);
    if (g->feed) cudaFree(g->feed);
    if (g->tickets) cudaFree(g->tickets);
    delete g;
}

}  // extern "C"

namespace {

// ------------------------------------------------------------------ allocation-free apply
// A server that hands every remaining byte of device memory to its KV cache at start-up,
// or a request thread that must never run into cudaMalloc's implicit device-wide
// synchronisation, cannot let this library allocate on its behalf.  For those callers the
// scratch of one single-token layer apply (the float64 intermediate t and the two stage
// records) lives in a fixed array inside the library image instead of in a buffer the
// context grows on demand.  Every GPU that loads the library carries the array until the
// process exits.
constexpr size_t kNoAllocMaxRank = 8192;     // r: t is r doubles
constexpr size_t kNoAllocMaxWidth = 16384;   // din and r must also fit the shared-memory table
constexpr size_t kNoAllocScratchBytes = kNoAllocMaxRank * sizeof(double) + 512;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// One stage of one instance with its parameters passed by value: nothing to stage through
// device memory first.
template <bool kRoundBf16, bool kFinal>
__global__ void __launch_bounds__(512, 1)
gemv_bitslice_value_kernel(const StageParams p, uint32_t n_rows, uint32_t n_bits, uint32_t n_groups,
                           uint32_t n_steps, uint32_t groups_per_warp) {
    qk::pdl_launch();
    extern __shared__ __align__(128) uint8_t smem_dyn[];
    bitslice_stage<kRoundBf16, kFinal, true, false, false>(
        p, smem_dyn, smem_dyn + (size_t)n_steps * 4096, nullptr, nullptr, n_rows, n_bits, n_groups,
        n_steps, blockIdx.x, groups_per_warp, false);
}

constexpr int kMaxDevices = 64;
std::mutex g_noalloc_mu;
unsigned char *g_noalloc_ptr[kMaxDevices] = {};  // device address of the array, per device

// The array's name is only a host-side handle; kernels need its device address, which is
// looked up once per device with that device current.
qk_status noalloc_scratch(int device, unsigned char **out) {
    if (device < 0 || device >= kMaxDevices)
        return qk::fail(QK_ERR_VALUE, "device index %d is outside the supported range", device);
    std::lock_guard<std::mutex> lock(g_noalloc_mu);
    if (!g_noalloc_ptr[device]) {
        void *ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || !ptr)
            return qk::fail(QK_ERR_CUDA, "cudaGetSymbolAddress for the built-in scratch failed: %s",
                            cudaGetErrorString(e));
        g_noalloc_ptr[device] = static_cast<unsigned char *>(ptr);
    }
    *out = g_noalloc_ptr[device];
    return QK_OK;
}

template <bool kFinal>
qk_status launch_value_stage(qk_ctx *c, const StageParams &p, const StageShape &s, bool bf16) {
    const StagePlan pl = plan_stage(c, s, 1);
    dim3 grid((unsigned)pl.blocks);
    auto gemv = bf16 ? gemv_bitslice_value_kernel<true, kFinal>
                     : gemv_bitslice_value_kernel<false, kFinal>;
    QK_CUDA(cudaFuncSetAttribute(gemv, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kSmemBudget));
    (void)qk::launch_pdl(c->pdl, gemv, grid, dim3((unsigned)pl.warps_per_block * 32), pl.smem, c->stream, p,
                         (uint32_t)s.n_rows, (uint32_t)s.n_bits, (uint32_t)s.n_groups,
                         (uint32_t)s.n_steps, (uint32_t)pl.gpw);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    return QK_OK;
}

}  // namespace

extern "C" {

qk_status qk_layer_apply_noalloc(qk_ctx *ctx, const qk_layer *layer, const float *x_dev,
                                 float *y_dev) {
    if (!layer) return qk::fail(QK_ERR_VALUE, "qk_layer_apply_noalloc: layer is null");
    if (!ctx)
        return qk::fail(QK_ERR_VALUE,
                        "qk_layer_apply_noalloc needs an existing context: creating the default "
                        "one would allocate");
    if (layer->r > kNoAllocMaxRank || layer->din > kNoAllocMaxWidth ||
        layer->r > kNoAllocMaxWidth)
        return qk::fail(QK_ERR_VALUE,
                        "layer (din=%zu, r=%zu) exceeds the built-in scratch: the allocation-free "
                        "apply supports r <= %zu and din <= %zu; use qk_layer_apply",
                        layer->din, layer->r, kNoAllocMaxRank, kNoAllocMaxWidth);
    if (!x_dev || !y_dev)
        return qk::fail(QK_ERR_VALUE, "qk_layer_apply_noalloc: x_dev and y_dev must not be null");
    qk_ctx *c = ctx;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    if (layer->device != c->device)
        return qk::fail(QK_ERR_VALUE, "layer lives on device %d, context on device %d",
                        layer->device, c->device);
    unsigned char *scratch = nullptr;
    qk_status st = noalloc_scratch(c->device, &scratch);
    if (st != QK_OK) return st;
    const StageShape s1 = stage1_shape(layer), s2 = stage2_shape(layer);
    if (!plan_stage(c, s1, 1).smem_digits || !plan_stage(c, s2, 1).smem_digits)
        return qk::fail(QK_ERR_VALUE, "layer is too wide for the allocation-free apply");
    // Layout of the array: [t: r doubles][two stage records].  Both are fully rewritten by
    // every call before they are read, so nothing has to be cleared between calls.
    void *t_buf = scratch;
    StageMeta *meta = reinterpret_cast<StageMeta *>(scratch + kNoAllocMaxRank * sizeof(double));
    const bool bf16 = layer->serving == QK_BF16;
    StageParams a{layer->vbt, layer->vbt_tiles, x_dev, layer->s2, t_buf, nullptr, nullptr, nullptr,
                  meta, nullptr, (uint32_t)layer->r, (uint32_t)layer->din, nullptr, nullptr, nullptr};
    StageParams b{layer->ub, layer->ub_tiles, t_buf, nullptr, y_dev, layer->s1, layer->bias, nullptr,
                  meta + 1, nullptr, (uint32_t)layer->dout, (uint32_t)layer->r, nullptr, nullptr, nullptr};
    if ((st = launch_value_stage<false>(c, a, s1, bf16)) != QK_OK) return st;
    return launch_value_stage<true>(c, b, s2, bf16);
}

}  // extern "C"
