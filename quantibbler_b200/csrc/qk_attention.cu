// Exact tiled attention and Sage INT8 attention: host buffers in, host buffers out.
//
// Replaces crates/quantibbler-kernels/src/gpu_attention.rs:451-570 (GpuContext::attention,
// which wraps the third-party cubek-attention 0.3.0 kernel and expands GQA heads on the
// host) and :589-756 + :67-397 (GpuContext::attention_sage and sage_int8_tile_kernel).
// Layouts are the reference's: q [B, H, Sq, d], k [B, KV, Skv, d], v [B, KV, Skv, dv],
// out [B, H, Sq, dv], packed row-major float32; head h reads kv head h / (H / KV);
// causal masks key j for query i when j + Sq > i + Skv.
//
// Exact face: FlashAttention-style online softmax in float32, GQA handled by indexing
// (no host-side head expansion).  Four lanes share one query row, each owning a quarter
// of the head dimension; K and V tiles of 32 keys are staged in shared memory.
//
// Sage face: the arithmetic of the reference's device kernel, stage for stage, in
// float32: Q/sqrt(d) per-token INT8, per-key-block channel mean removed from K then
// per-token INT8, integer QK^T, scores = dQ*dK*dot + (dQ*Qhat).mean, online softmax in
// full precision, P quantised at the static 1/127 scale, V per-channel INT8 per key block,
// integer PV, O = alpha*O + pv*(1/127)*dV, O/l at the end.  Unlike the reference (one thread
// per query row re-quantising every K/V tile into global scratch), the K, V and Q codes are
// produced once per call by three small kernels.  Two main kernels share them:
//   * attention_sage_tc_kernel: both integer products on the INT8 tensor cores (mma.sync
//     m16n8k32), for head_dim = val_dim in {64, 128} and key blocks of 32, 64 or 128;
//   * attention_sage_kernel: integer dots with dp4a, any shape.  A key block's P codes all
//     depend on the block's row maximum, so each block is swept twice there: once for the
//     maximum, once for P and the PV product.
#include <cmath>
#include <cstring>
#include <string>

#include "qk_common.h"
#include "qk_umma.cuh"

namespace {

struct AttnDims {
    uint32_t B, H, KV, Sq, Skv, d, dv, group;
};

constexpr int kQT = 64;  // queries per block (4 lanes each)
constexpr int kTK = 32;  // keys per shared-memory tile

// ------------------------------------------------------------------ exact attention
template <int DPL>
__global__ void __launch_bounds__(256)
attention_exact_kernel(const float *__restrict__ q, const float *__restrict__ k,
                       const float *__restrict__ v, float *__restrict__ out, AttnDims dm,
                       int causal) {
    constexpr int PITCH = DPL + 4;  // +4 floats: the four parts of a key land in distinct banks
    extern __shared__ float sm[];
    float *Ks = sm, *Vs = sm + kTK * 4 * PITCH;
    const int qi = threadIdx.x >> 2, part = threadIdx.x & 3;
    const int i = blockIdx.x * kQT + qi;
    const bool valid = i < (int)dm.Sq;
    const int h = blockIdx.y, b = blockIdx.z, kvh = h / dm.group;
    const float scale = 1.0f / sqrtf((float)dm.d);

    float qr[DPL], o[DPL];
#pragma unroll
    for (int e = 0; e < DPL; ++e) {
        int c = part * DPL + e;
        qr[e] = (valid && c < (int)dm.d)
                    ? q[(((size_t)b * dm.H + h) * dm.Sq + i) * dm.d + c] : 0.f;
        o[e] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    const int skew = (int)dm.Skv - (int)dm.Sq;
    const int last_key = !valid ? -1 : causal ? i + skew : (int)dm.Skv - 1;
    const int i_max = min((int)dm.Sq - 1, (int)blockIdx.x * kQT + kQT - 1);
    const int j_hi = causal ? min((int)dm.Skv, i_max + skew + 1) : (int)dm.Skv;
    const float *kb = k + ((size_t)b * dm.KV + kvh) * dm.Skv * dm.d;
    const float *vb = v + ((size_t)b * dm.KV + kvh) * dm.Skv * dm.dv;

    for (int j0 = 0; j0 < j_hi; j0 += kTK) {
        __syncthreads();
        for (int idx = threadIdx.x; idx < kTK * 4 * DPL; idx += 256) {
            int key = idx / (4 * DPL), c = idx % (4 * DPL);
            int p2 = c / DPL, e = c % DPL;
            bool in = j0 + key < (int)dm.Skv;
            Ks[(key * 4 + p2) * PITCH + e] =
                (in && c < (int)dm.d) ? kb[(size_t)(j0 + key) * dm.d + c] : 0.f;
            Vs[(key * 4 + p2) * PITCH + e] =
                (in && c < (int)dm.dv) ? vb[(size_t)(j0 + key) * dm.dv + c] : 0.f;
        }
        __syncthreads();
        float s[kTK];
        float tmax = -INFINITY;
#pragma unroll
        for (int kk = 0; kk < kTK; ++kk) {
            const float *kr = Ks + (kk * 4 + part) * PITCH;
            float dot = 0.f;
#pragma unroll
            for (int e = 0; e < DPL; ++e) dot = fmaf(qr[e], kr[e], dot);
            dot += __shfl_xor_sync(0xffffffffu, dot, 1);
            dot += __shfl_xor_sync(0xffffffffu, dot, 2);
            float sc = dot * scale;
            if (j0 + kk > last_key) sc = -INFINITY;
            s[kk] = sc;
            tmax = fmaxf(tmax, sc);
        }
        const float m_new = fmaxf(m, tmax);
        if (m_new == -INFINITY) continue;  // nothing admissible yet (barriers sit at the loop top)
        const float alpha = expf(m - m_new);
        l *= alpha;
#pragma unroll
        for (int e = 0; e < DPL; ++e) o[e] *= alpha;
#pragma unroll
        for (int kk = 0; kk < kTK; ++kk) {
            const float p = expf(s[kk] - m_new);
            l += p;
            const float *vr = Vs + (kk * 4 + part) * PITCH;
#pragma unroll
            for (int e = 0; e < DPL; ++e) o[e] = fmaf(p, vr[e], o[e]);
        }
        m = m_new;
    }
    if (valid) {
        float *orow = out + (((size_t)b * dm.H + h) * dm.Sq + i) * dm.dv;
#pragma unroll
        for (int e = 0; e < DPL; ++e) {
            int c = part * DPL + e;
            if (c < (int)dm.dv) orow[c] = o[e] / l;  // a row with no admissible key is 0/0 = NaN
        }
    }
}

// ------------------------------------------------------------------ Sage quantisers
// The tcgen05 kernel (head_dim = val_dim = 128, key block 64) takes its operands as RECORDS: one
// per (plane, pair of key blocks), laid out in global memory byte for byte as the kernel wants
// them in shared memory, so that an iteration's operands arrive by one bulk copy:
//   [K tile: 144 rows of 128 bytes: the 128 keys' codes, then 2 x 8 mean-digit rows]
//   [V tile: 128 channel rows of 128 bytes: the codes of block a's 64 keys, then block b's]
//   [scales: 128 key scales, 2 x 128 channel scales of V, 2 mean units (16 floats reserved)]
// Tile rows are 128-byte-swizzled: the 16-byte piece p of row r sits at piece p ^ (r & 7).
// What a ragged sequence leaves unwritten (keys past the end, a missing second block) is never
// used: those scores are masked before the softmax and the second product is not folded in.
constexpr uint32_t kURecKBytes = 144 * 128, kURecVBytes = 128 * 128;
constexpr uint32_t kURecScaleOff = kURecKBytes + kURecVBytes, kURecScaleFloats = 128 + 2 * 128 + 16;
constexpr uint32_t kURecBytes = kURecScaleOff + kURecScaleFloats * 4;  // what one bulk copy moves
constexpr uint32_t kURecStride = (kURecBytes + 1023) / 1024 * 1024;
// Records of the block-scale variant (attention_sage_block_kernel): the same K tile, a
// bfloat16 V tile per key block ([128 channels][64 keys], 16 KB each, block a then block b),
// 128 key scales (one value per 64-key block, repeated) and the two mean units.
constexpr uint32_t kBRecKBytes = 144 * 128, kBRecVBytes = 2 * 128 * 128;
constexpr uint32_t kBRecScaleOff = kBRecKBytes + kBRecVBytes, kBRecScaleFloats = 128 + 16;
constexpr uint32_t kBRecBytes = kBRecScaleOff + kBRecScaleFloats * 4;
constexpr uint32_t kBRecStride = (kBRecBytes + 1023) / 1024 * 1024;
__host__ __device__ inline uint32_t rec_tile_offset(uint32_t row, uint32_t byte) {
    return row * 128 + (((byte >> 4) ^ (row & 7)) << 4) + (byte & 15);
}

// float32 -> nearest bfloat16 value (ties to even), as a float32
__device__ __forceinline__ float round_bf16_value(float v) {
    uint32_t u = __float_as_uint(v);
    if ((u & 0x7fffffffu) > 0x7f800000u) return __uint_as_float((u | 0x00400000u) & 0xffff0000u);
    u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;
    return __uint_as_float(u);
}
__device__ __forceinline__ int quant_code(float x, float delta) {
    // rint half-to-even of x/delta, clamped to +-127 (gpu_attention.rs:132-155)
    float r = rintf(x / delta);
    r = fminf(fmaxf(r, -127.f), 127.f);
    return (int)r;
}

// psi_Q: one warp per query row.  codes [rows][dpad] int8 (zero padded), scale [rows].
__global__ void sage_quant_q_kernel(const float *__restrict__ q, int8_t *__restrict__ codes,
                                    float *__restrict__ scale, uint32_t rows, uint32_t d,
                                    uint32_t dpad, float inv_sqrt_d) {
    uint32_t row = blockIdx.x * (blockDim.x / 32) + threadIdx.x / 32, lane = threadIdx.x % 32;
    if (row >= rows) return;
    const float *qr = q + (size_t)row * d;
    if (d % 4 == 0 && dpad <= 128) {
        // a lane owns four consecutive channels: one 16-byte load, one 4-byte store of codes
        const uint32_t c = 4 * lane;
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
        if (c < d) x = *reinterpret_cast<const float4 *>(qr + c);
        x.x *= inv_sqrt_d, x.y *= inv_sqrt_d, x.z *= inv_sqrt_d, x.w *= inv_sqrt_d;
        float peak = fmaxf(fmaxf(fabsf(x.x), fabsf(x.y)), fmaxf(fabsf(x.z), fabsf(x.w)));
        for (int off = 16; off > 0; off >>= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, off));
        const float delta = peak > 0.f ? peak / 127.f : 1.f;
        if (c < dpad) {
            const uint32_t w = (uint32_t)(quant_code(x.x, delta) & 0xff) | ((uint32_t)(quant_code(x.y, delta) & 0xff) << 8) |
                               ((uint32_t)(quant_code(x.z, delta) & 0xff) << 16) |
                               ((uint32_t)(quant_code(x.w, delta) & 0xff) << 24);
            *reinterpret_cast<uint32_t *>(codes + (size_t)row * dpad + c) = c < d ? w : 0u;
        }
        if (lane == 0) scale[row] = delta;
        return;
    }
    float peak = 0.f;
    for (uint32_t c = lane; c < d; c += 32) peak = fmaxf(peak, fabsf(qr[c] * inv_sqrt_d));
    for (int off = 16; off > 0; off >>= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, off));
    const float delta = peak > 0.f ? peak / 127.f : 1.f;
    for (uint32_t c = lane; c < dpad; c += 32)
        codes[(size_t)row * dpad + c] = c < d ? (int8_t)quant_code(qr[c] * inv_sqrt_d, delta) : 0;
    if (lane == 0) scale[row] = delta;
}

// gamma + psi_K: one block per (b, kv head, key block).  mean [blk][d] float32 (sequential
// float32 sum over the block's tokens, then one division, as the reference kernel does),
// codes [token][dpad], scale [token].
// mean_digits (may be null) [blk][8][dpad] int8 + mean_scale [blk]: the mean as a 24-bit fixed
// point number in three balanced base-256 digits, mean[c] = mean_scale * (65536 d0 + 256 d1
// + d2); rows 3..7 are zero.  The tensor-core kernel appends these rows to the block's K codes,
// so that (Qhat . mean) falls out of the same integer MMA as the scores.
__global__ void sage_quant_k_kernel(const float *__restrict__ k, int8_t *__restrict__ codes,
                                    float *__restrict__ scale, float *__restrict__ mean,
                                    uint32_t S, uint32_t d, uint32_t dpad, uint32_t block,
                                    uint32_t n_blocks, int8_t *__restrict__ mean_digits,
                                    float *__restrict__ mean_scale, uint8_t *__restrict__ rec,
                                    uint32_t rec_stride = kURecStride, uint32_t rec_scale_off = kURecScaleOff,
                                    uint32_t rec_mscale_at = 128 + 2 * 128, int block_scale = 0) {
    extern __shared__ float mu[];  // d floats
    const uint32_t plane = blockIdx.y, jb = blockIdx.x;
    const uint32_t j0 = jb * block, j1 = min(S, j0 + block), kj = j1 - j0;
    const float *kp = k + (size_t)plane * S * d;
    for (uint32_t c = threadIdx.x; c < d; c += blockDim.x) {
        float ssum = 0.f;
        for (uint32_t j = j0; j < j1; ++j) ssum += kp[(size_t)j * d + c];
        float mval = ssum / (float)kj;
        mu[c] = mval;
        mean[((size_t)plane * n_blocks + jb) * d + c] = mval;
    }
    __syncthreads();
    if (rec) {
        // record form (d = dpad = 128, block = 64, 128 threads): thread c owns channel c of the
        // digit rows, lane l of a warp owns channels 4 l .. 4 l + 3 of a key
        __shared__ float peak_rec[4];
        uint8_t *rc = rec + ((size_t)plane * ((n_blocks + 1) / 2) + jb / 2) * rec_stride;
        const uint32_t half = jb % 2, c = threadIdx.x;
        float peak = fabsf(mu[c]);
        for (int off = 16; off > 0; off >>= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, off));
        if (threadIdx.x % 32 == 0) peak_rec[threadIdx.x / 32] = peak;
        __syncthreads();
        peak = fmaxf(fmaxf(peak_rec[0], peak_rec[1]), fmaxf(peak_rec[2], peak_rec[3]));
        const float unit = peak > 0.f ? peak / 8000000.f : 1.f;   // |fixed| <= 8e6 < 127 * 65536
        int v = (int)rintf(mu[c] / unit);
        const int d2 = ((v + 128) & 255) - 128;
        v = (v - d2) >> 8;
        const int d1 = ((v + 128) & 255) - 128;
        v = (v - d1) >> 8;
        const uint32_t row0 = 128 + 8 * half;
        rc[rec_tile_offset(row0, c)] = (uint8_t)(int8_t)v;
        rc[rec_tile_offset(row0 + 1, c)] = (uint8_t)(int8_t)d1;
        rc[rec_tile_offset(row0 + 2, c)] = (uint8_t)(int8_t)d2;
#pragma unroll
        for (uint32_t dr = 3; dr < 8; ++dr) rc[rec_tile_offset(row0 + dr, c)] = 0;
        float *scales = reinterpret_cast<float *>(rc + rec_scale_off);
        if (threadIdx.x == 0) scales[rec_mscale_at + half] = unit;
        const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
        float block_delta = 0.f;
        if (block_scale) {
            // one scale for the whole 64-key block (the benchmark specification's granularity)
            __shared__ float block_peak[4];
            float pk = 0.f;
            for (uint32_t j = j0 + warp; j < j1; j += 4) {
                const float4 x = *reinterpret_cast<const float4 *>(kp + (size_t)j * d + 4 * lane);
                const float4 mm = *reinterpret_cast<const float4 *>(mu + 4 * lane);
                pk = fmaxf(pk, fmaxf(fmaxf(fabsf(x.x - mm.x), fabsf(x.y - mm.y)), fmaxf(fabsf(x.z - mm.z), fabsf(x.w - mm.w))));
            }
            for (int off = 16; off > 0; off >>= 1) pk = fmaxf(pk, __shfl_xor_sync(0xffffffffu, pk, off));
            if (lane == 0) block_peak[warp] = pk;
            __syncthreads();
            pk = fmaxf(fmaxf(block_peak[0], block_peak[1]), fmaxf(block_peak[2], block_peak[3]));
            block_delta = pk > 0.f ? pk / 127.f : 1.f;
        }
        for (uint32_t j = j0 + warp; j < j1; j += 4) {
            const float4 x = *reinterpret_cast<const float4 *>(kp + (size_t)j * d + 4 * lane);
            const float4 mm = *reinterpret_cast<const float4 *>(mu + 4 * lane);
            const float e0 = x.x - mm.x, e1 = x.y - mm.y, e2 = x.z - mm.z, e3 = x.w - mm.w;
            float pk = fmaxf(fmaxf(fabsf(e0), fabsf(e1)), fmaxf(fabsf(e2), fabsf(e3)));
            for (int off = 16; off > 0; off >>= 1) pk = fmaxf(pk, __shfl_xor_sync(0xffffffffu, pk, off));
            const float delta = block_scale ? block_delta : pk > 0.f ? pk / 127.f : 1.f;
            const uint32_t w = (uint32_t)(quant_code(e0, delta) & 0xff) | ((uint32_t)(quant_code(e1, delta) & 0xff) << 8) |
                               ((uint32_t)(quant_code(e2, delta) & 0xff) << 16) |
                               ((uint32_t)(quant_code(e3, delta) & 0xff) << 24);
            const uint32_t row = 64 * half + (j - j0);
            *reinterpret_cast<uint32_t *>(rc + rec_tile_offset(row, 4 * lane)) = w;
            if (lane == 0) scales[row] = delta;
        }
        return;
    }
    if (mean_digits) {
        __shared__ float peak_sh[4];
        float peak = 0.f;
        for (uint32_t c = threadIdx.x; c < d; c += blockDim.x) peak = fmaxf(peak, fabsf(mu[c]));
        for (int off = 16; off > 0; off >>= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, off));
        if (threadIdx.x % 32 == 0) peak_sh[threadIdx.x / 32] = peak;
        __syncthreads();
        peak = fmaxf(fmaxf(peak_sh[0], peak_sh[1]), fmaxf(peak_sh[2], peak_sh[3]));
        const float unit = peak > 0.f ? peak / 8000000.f : 1.f;   // |fixed| <= 8e6 < 127 * 65536
        int8_t *rows = mean_digits + ((size_t)plane * n_blocks + jb) * 8 * dpad;
        for (uint32_t c = threadIdx.x; c < 8 * dpad; c += blockDim.x) rows[c] = 0;
        __syncthreads();
        for (uint32_t c = threadIdx.x; c < d; c += blockDim.x) {
            int v = (int)rintf(mu[c] / unit);
            const int d2 = ((v + 128) & 255) - 128;
            v = (v - d2) >> 8;
            const int d1 = ((v + 128) & 255) - 128;
            v = (v - d1) >> 8;
            rows[c] = (int8_t)v;
            rows[dpad + c] = (int8_t)d1;
            rows[2 * dpad + c] = (int8_t)d2;
        }
        if (threadIdx.x == 0) mean_scale[(size_t)plane * n_blocks + jb] = unit;
    }
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32, n_warps = blockDim.x / 32;
    for (uint32_t j = j0 + warp; j < j1; j += n_warps) {
        const float *kr = kp + (size_t)j * d;
        float peak = 0.f;
        for (uint32_t c = lane; c < d; c += 32) peak = fmaxf(peak, fabsf(kr[c] - mu[c]));
        for (int off = 16; off > 0; off >>= 1)
            peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, off));
        const float delta = peak > 0.f ? peak / 127.f : 1.f;
        int8_t *cr = codes + ((size_t)plane * S + j) * dpad;
        for (uint32_t c = lane; c < dpad; c += 32)
            cr[c] = c < d ? (int8_t)quant_code(kr[c] - mu[c], delta) : 0;
        if (lane == 0) scale[(size_t)plane * S + j] = delta;
    }
}

// psi_Q with one scale per 64-query block (block-scale variant): a block of 256 threads per
// (head, 64-row block), a warp takes eight rows, a lane four channels (d = dpad = 128).
__global__ void __launch_bounds__(256)
sage_quant_q_block_kernel(const float *__restrict__ q, int8_t *__restrict__ codes, float *__restrict__ scale,
                          uint32_t Sq, float inv_sqrt_d) {
    __shared__ float peaks[8];
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const size_t head_row0 = (size_t)blockIdx.y * Sq;
    const uint32_t r0 = blockIdx.x * 64;
    float4 x[8];
    float peak = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t r = r0 + warp + 8 * i;
        x[i] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < Sq) x[i] = *reinterpret_cast<const float4 *>(q + (head_row0 + r) * 128 + 4 * lane);
        x[i].x *= inv_sqrt_d, x[i].y *= inv_sqrt_d, x[i].z *= inv_sqrt_d, x[i].w *= inv_sqrt_d;
        peak = fmaxf(peak, fmaxf(fmaxf(fabsf(x[i].x), fabsf(x[i].y)), fmaxf(fabsf(x[i].z), fabsf(x[i].w))));
    }
    for (int off = 16; off > 0; off >>= 1) peak = fmaxf(peak, __shfl_xor_sync(0xffffffffu, peak, off));
    if (lane == 0) peaks[warp] = peak;
    __syncthreads();
    peak = peaks[0];
#pragma unroll
    for (int w = 1; w < 8; ++w) peak = fmaxf(peak, peaks[w]);
    const float delta = peak > 0.f ? peak / 127.f : 1.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t r = r0 + warp + 8 * i;
        if (r >= Sq) continue;
        const uint32_t w = (uint32_t)(quant_code(x[i].x, delta) & 0xff) | ((uint32_t)(quant_code(x[i].y, delta) & 0xff) << 8) |
                           ((uint32_t)(quant_code(x[i].z, delta) & 0xff) << 16) |
                           ((uint32_t)(quant_code(x[i].w, delta) & 0xff) << 24);
        *reinterpret_cast<uint32_t *>(codes + (head_row0 + r) * 128 + 4 * lane) = w;
        if (lane == 0) scale[head_row0 + r] = delta;
    }
}

// V of a key block as a bfloat16 tile of the block-scale variant's record: thread c writes
// channel row c (64 keys = 128 bytes, eight swizzled 16-byte pieces); keys past the end are 0.
__global__ void __launch_bounds__(128)
sage_v_bf16_record_kernel(const float *__restrict__ v, uint8_t *__restrict__ rec, uint32_t S, uint32_t n_blocks) {
    const uint32_t plane = blockIdx.y, jb = blockIdx.x, c = threadIdx.x;
    const uint32_t j0 = jb * 64, j1 = min(S, j0 + 64);
    const float *vp = v + (size_t)plane * S * 128;
    uint8_t *tile = rec + ((size_t)plane * ((n_blocks + 1) / 2) + jb / 2) * kBRecStride + kBRecKBytes + (jb % 2) * 16384;
#pragma unroll
    for (int piece = 0; piece < 8; ++piece) {
        uint32_t w[4];
#pragma unroll
        for (int qd = 0; qd < 4; ++qd) {
            const uint32_t ja = j0 + 8 * piece + 2 * qd, jbb = ja + 1;
            const float a = ja < j1 ? vp[(size_t)ja * 128 + c] : 0.f, b = jbb < j1 ? vp[(size_t)jbb * 128 + c] : 0.f;
            w[qd] = (__float_as_uint(round_bf16_value(a)) >> 16) | (__float_as_uint(round_bf16_value(b)) & 0xffff0000u);
        }
        *reinterpret_cast<uint4 *>(tile + rec_tile_offset(c, 16 * piece)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// Where key kk of a block sits in the tensor-core kernel's V tile.  That kernel feeds its P
// codes to the PV MMA straight from the accumulator fragment of QK^T, in which a thread holds
// columns 2t, 2t+1 of each 8-key tile; the MMA's A operand wants four consecutive k per
// register.  Summation order over keys is free, so the keys of every 32-key slab are simply
// renamed: tile j, column c of the slab becomes k index 16*(j/2) + 4*(c/2) + 2*(j%2) + c%2.
__host__ __device__ inline uint32_t sage_tc_key_slot(uint32_t kk) {
    const uint32_t slab = kk / 32, r = kk % 32, j = r / 8, c = r % 8;
    return slab * 32 + (j / 2) * 16 + (c / 2) * 4 + (j % 2) * 2 + (c % 2);
}

// psi_V: one block per (b, kv head, key block): per-channel scale over the block's tokens,
// codes stored channel-major with the block's keys contiguous: [blk][dv][bpad] int8
// (permute: in the tensor-core kernel's key order).
__global__ void sage_quant_v_kernel(const float *__restrict__ v, int8_t *__restrict__ codes,
                                    float *__restrict__ scale, uint32_t S, uint32_t dv,
                                    uint32_t block, uint32_t bpad, uint32_t n_blocks,
                                    int permute, uint8_t *__restrict__ rec) {
    const uint32_t plane = blockIdx.y, jb = blockIdx.x;
    const uint32_t j0 = jb * block, j1 = min(S, j0 + block);
    const float *vp = v + (size_t)plane * S * dv;
    for (uint32_t c = threadIdx.x; c < dv; c += blockDim.x) {
        int8_t *cr = codes + (((size_t)plane * n_blocks + jb) * dv + c) * bpad;
        if (bpad == 64 && !permute) {
            // the block's 64 values of the channel stay in registers between the two passes,
            // and the codes leave as four 16-byte stores
            float x[64];
            float peak = 0.f;
#pragma unroll
            for (int j = 0; j < 64; ++j) {
                x[j] = j0 + j < j1 ? vp[(size_t)(j0 + j) * dv + c] : 0.f;
                peak = fmaxf(peak, fabsf(x[j]));
            }
            const float delta = peak > 0.f ? peak / 127.f : 1.f;
#pragma unroll
            for (int piece = 0; piece < 4; ++piece) {
                uint32_t w[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    w[q] = 0;
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = 16 * piece + 4 * q + e;
                        const int code = j0 + j < j1 ? quant_code(x[j], delta) : 0;
                        w[q] |= (uint32_t)(code & 0xff) << (8 * e);
                    }
                }
                if (rec) {  // record form (dv = 128): row c of the pair's V tile, the block's half of it
                    uint8_t *rc = rec + ((size_t)plane * ((n_blocks + 1) / 2) + jb / 2) * kURecStride + kURecKBytes;
                    *reinterpret_cast<uint4 *>(rc + rec_tile_offset(c, 64 * (jb % 2) + 16 * piece)) =
                        make_uint4(w[0], w[1], w[2], w[3]);
                } else {
                    *reinterpret_cast<uint4 *>(cr + 16 * piece) = make_uint4(w[0], w[1], w[2], w[3]);
                }
            }
            if (rec) {
                uint8_t *rc = rec + ((size_t)plane * ((n_blocks + 1) / 2) + jb / 2) * kURecStride;
                reinterpret_cast<float *>(rc + kURecScaleOff)[128 + 128 * (jb % 2) + c] = delta;
            } else {
                scale[((size_t)plane * n_blocks + jb) * dv + c] = delta;
            }
            continue;
        }
        float peak = 0.f;
        for (uint32_t j = j0; j < j1; ++j) peak = fmaxf(peak, fabsf(vp[(size_t)j * dv + c]));
        const float delta = peak > 0.f ? peak / 127.f : 1.f;
        for (uint32_t j = j0; j < j0 + bpad; ++j)
            cr[permute ? sage_tc_key_slot(j - j0) : j - j0] =
                j < j1 ? (int8_t)quant_code(vp[(size_t)j * dv + c], delta) : 0;
        scale[((size_t)plane * n_blocks + jb) * dv + c] = delta;
    }
}

struct SageArgs {
    const int8_t *qc;
    const float *qs;
    const int8_t *kc;
    const float *ks;
    const float *kmean;
    const int8_t *kmean_digits;  // tensor-core kernel: [blk][8][dpad]
    const float *kmean_scale;    // [blk]
    const int8_t *vc;
    const float *vs;
    float *out;
    uint32_t dpad, bpad, block, n_blocks;
    const uint8_t *rec;  // tcgen05 kernel: the records, [plane][pair of blocks][kURecStride]
};

// Main Sage kernel.  Lane (query, part) owns DPL = dpad/4 (resp. dvpad/4) channels; WPL
// is that count in 32-bit words of four int8 codes.
template <int WPL>
__global__ void __launch_bounds__(256)
attention_sage_kernel(SageArgs a, AttnDims dm, int causal) {
    constexpr int DPL = WPL * 4;
    extern __shared__ int smi[];
    int *Kt = smi;                     // [kTK][4][WPL+1] words of K codes
    float *Kscale = (float *)(Kt + kTK * 4 * (WPL + 1));  // [kTK]
    int *Vt = (int *)(Kscale + kTK);   // [4*DPL channels][kTK/4 + 1] words of V codes (keys packed)
    const int qi = threadIdx.x >> 2, part = threadIdx.x & 3;
    const int i = blockIdx.x * kQT + qi;
    const bool valid = i < (int)dm.Sq;
    const int h = blockIdx.y, b = blockIdx.z, kvh = h / dm.group;
    const size_t qrow = ((size_t)b * dm.H + h) * dm.Sq + (valid ? i : 0);
    const size_t plane = (size_t)b * dm.KV + kvh;

    int qw[WPL];
    float qdq[DPL];  // dequantised query, for the mean shift
    const float qdelta = a.qs[qrow];
#pragma unroll
    for (int w = 0; w < WPL; ++w) {
        int word = valid ? reinterpret_cast<const int *>(a.qc + qrow * a.dpad)[part * WPL + w] : 0;
        qw[w] = word;
#pragma unroll
        for (int e = 0; e < 4; ++e) qdq[w * 4 + e] = (float)(int8_t)(word >> (8 * e)) * qdelta;
    }
    float o[DPL];
#pragma unroll
    for (int e = 0; e < DPL; ++e) o[e] = 0.f;
    float m = -INFINITY, l = 0.f;

    const int block = (int)a.block;
    const int i_max = min((int)dm.Sq - 1, (int)blockIdx.x * kQT + kQT - 1);
    const int jb_hi = causal ? i_max / block + 1 : (int)a.n_blocks;  // key blocks this tile visits
    const int my_jb_hi = !valid ? 0 : causal ? i / block + 1 : (int)a.n_blocks;

    for (int jb = 0; jb < jb_hi; ++jb) {
        const int j0 = jb * block, kj = min(block, (int)dm.Skv - j0);
        const bool mine = jb < my_jb_hi;
        // shift = (dQ * Qhat) . mean of this block
        float shift = 0.f;
        {
            const float *mu = a.kmean + (plane * a.n_blocks + jb) * dm.d;
#pragma unroll
            for (int e = 0; e < DPL; ++e) {
                int c = part * DPL + e;
                if (c < (int)dm.d) shift = fmaf(qdq[e], mu[c], shift);
            }
            shift += __shfl_xor_sync(0xffffffffu, shift, 1);
            shift += __shfl_xor_sync(0xffffffffu, shift, 2);
        }
        float m_new = m;
        int pv[DPL];
        float esum = 0.f, alpha = 0.f;
        for (int pass = 0; pass < 2; ++pass) {
            if (pass == 1) {
                alpha = (m_new == -INFINITY) ? 0.f : expf(m - m_new);
#pragma unroll
                for (int e = 0; e < DPL; ++e) pv[e] = 0;
            }
            for (int t0 = 0; t0 < kj; t0 += kTK) {
                const int tk = min(kTK, kj - t0);
                __syncthreads();
                for (int idx = threadIdx.x; idx < kTK * 4 * WPL; idx += 256) {
                    int key = idx / (4 * WPL), w = idx % (4 * WPL);
                    int word = 0;
                    if (key < tk)
                        word = reinterpret_cast<const int *>(
                            a.kc + (plane * dm.Skv + j0 + t0 + key) * a.dpad)[w];
                    Kt[(key * 4 + w / WPL) * (WPL + 1) + w % WPL] = word;
                }
                if (threadIdx.x < kTK)
                    Kscale[threadIdx.x] =
                        (int)threadIdx.x < tk ? a.ks[plane * dm.Skv + j0 + t0 + threadIdx.x] : 1.f;
                if (pass == 1) {
                    for (int idx = threadIdx.x; idx < 4 * DPL * (kTK / 4); idx += 256) {
                        int c = idx / (kTK / 4), w = idx % (kTK / 4);
                        int word = 0;
                        if (c < (int)dm.dv && t0 + w * 4 < (int)a.bpad)
                            word = reinterpret_cast<const int *>(
                                a.vc + ((plane * a.n_blocks + jb) * dm.dv + c) * a.bpad + t0)[w];
                        Vt[c * (kTK / 4 + 1) + w] = word;
                    }
                }
                __syncthreads();
                float s[kTK];
#pragma unroll
                for (int kk = 0; kk < kTK; ++kk) {
                    const int *kr = Kt + (kk * 4 + part) * (WPL + 1);
                    int dot = 0;
#pragma unroll
                    for (int w = 0; w < WPL; ++w) dot = __dp4a(qw[w], kr[w], dot);
                    dot += __shfl_xor_sync(0xffffffffu, dot, 1);
                    dot += __shfl_xor_sync(0xffffffffu, dot, 2);
                    float sc = (float)dot * qdelta * Kscale[kk] + shift;
                    const int j = j0 + t0 + kk;
                    if (kk >= tk || !mine || (causal && j > i)) sc = -INFINITY;
                    s[kk] = sc;
                }
                if (pass == 0) {
#pragma unroll
                    for (int kk = 0; kk < kTK; ++kk) m_new = fmaxf(m_new, s[kk]);
                } else {
                    // P codes of this 32-key slice, four keys per word, then the integer PV
                    int pw[kTK / 4];
#pragma unroll
                    for (int w = 0; w < kTK / 4; ++w) {
                        int word = 0;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            float p = (m_new == -INFINITY) ? 0.f : expf(s[w * 4 + e] - m_new);
                            esum += p;
                            float r = fminf(fmaxf(rintf(p * 127.f), 0.f), 127.f);
                            word |= ((int)r) << (8 * e);
                        }
                        pw[w] = word;
                    }
#pragma unroll
                    for (int e = 0; e < DPL; ++e) {
                        const int *vr = Vt + (part * DPL + e) * (kTK / 4 + 1);
                        int acc = pv[e];
#pragma unroll
                        for (int w = 0; w < kTK / 4; ++w) acc = __dp4a(pw[w], vr[w], acc);
                        pv[e] = acc;
                    }
                }
            }
        }
        if (mine && m_new != -INFINITY) {
            const float *vsc = a.vs + (plane * a.n_blocks + jb) * dm.dv;
            l = alpha * l + esum;
#pragma unroll
            for (int e = 0; e < DPL; ++e) {
                int c = part * DPL + e;
                float vd = c < (int)dm.dv ? vsc[c] : 1.f;
                o[e] = alpha * o[e] + (float)pv[e] * (1.0f / 127.0f) * vd;
            }
            m = m_new;
        }
    }
    if (valid) {
        float *orow = a.out + qrow * dm.dv;
#pragma unroll
        for (int e = 0; e < DPL; ++e) {
            int c = part * DPL + e;
            if (c < (int)dm.dv) orow[c] = o[e] / l;
        }
    }
}

// ------------------------------------------------------------------ Sage on the tensor cores
__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                     (uint32_t)__cvta_generic_to_shared(smem)),
                 "l"(gmem)
                 : "memory");
}

// Four (two) 8-row x 16-byte matrices from shared memory: lane l supplies the address of row
// l % 8 of matrix l / 8; afterwards every thread (g, t) holds bytes 4t..4t+3 of row g of each
// matrix, which is exactly the B fragment of the 8-bit m16n8k32 MMA.
__device__ __forceinline__ void ldsm_x4(const void *row, int &r0, int &r1, int &r2, int &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"((uint32_t)__cvta_generic_to_shared(row)));
}
__device__ __forceinline__ void ldsm_x2(const void *row, int &r0, int &r1) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];"
                 : "=r"(r0), "=r"(r1)
                 : "r"((uint32_t)__cvta_generic_to_shared(row)));
}

// four codes (each already in [0, 127]) -> one register, code j in byte j
__device__ __forceinline__ int pack_codes(const int (&c)[4]) {
    int hi, w;
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(c[3]), "r"(c[2]), "r"(0));
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(w) : "r"(c[1]), "r"(c[0]), "r"(hi));
    return w;
}

__device__ __forceinline__ void mma_s8(int (&c)[4], const int (&a)[4], int b0, int b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The same arithmetic as attention_sage_kernel with both integer products on the INT8
// tensor cores (mma.sync m16n8k32).  A block of four warps takes 64 queries, 16 per warp;
// one key block (BLK = 32, 64 or 128 keys, the Sage block) is staged in shared memory at a
// time: K codes [BLK][D + 16] and V codes [DV][BLK + 16] (the 16-byte pads make the
// fragment loads bank-conflict free), the key scales, the channel scales and the mean.
//   S = Qhat Khat^T: A = the warp's Q codes (kept in registers for the whole kernel),
//       B = K codes; the int32 accumulator fragment holds rows g, g+8 and columns 2t, 2t+1
//       of each 8-key tile;
//   scores, row maximum (two shuffles within the quad), P = exp(s - m), l, P codes: all on
//       the fragment, then the codes are packed four to a register in the key order of
//       sage_tc_key_slot and are the A operand of
//   PV = Phat Vhat: B = V codes in that same key order; one 8-channel tile at a time is
//       folded into the float32 output fragment with alpha and dV / 127.
// Because the whole block's scores are in registers the block is swept once, not twice.
template <int D32, int DV8, int BLK32>
__global__ void __launch_bounds__(128, 3)
attention_sage_tc_kernel(SageArgs a, AttnDims dm, int causal) {
    constexpr int D = 32 * D32, DV = 8 * DV8, BLK = 32 * BLK32, NT = BLK / 8;
    constexpr int KP = D + 16, VP = BLK + 16;
    // two buffers: the next key block is copied in (cp.async) while this one is used
    // K tile: the block's keys, then eight rows of mean digits (three used)
    constexpr int kBufBytes = (BLK + 8) * KP + DV * VP + (BLK + DV + 4) * (int)sizeof(float);
    extern __shared__ __align__(16) uint8_t sm_tc[];
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane >> 2, t = lane & 3;
    const int h = blockIdx.y, b = blockIdx.z, kvh = h / dm.group;
    const size_t plane = (size_t)b * dm.KV + kvh;
    // under causal masking the last query tiles have the most key blocks: start them first
    const int q_tile = causal ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x;
    const int q0 = q_tile * 64 + warp * 16;
    const int i0 = q0 + g, i1 = i0 + 8;
    const bool v0 = i0 < (int)dm.Sq, v1 = i1 < (int)dm.Sq;
    const size_t row_base = ((size_t)b * dm.H + h) * dm.Sq;

    int qa[D32][4];
    {
        const int *r0 = reinterpret_cast<const int *>(a.qc + (row_base + (v0 ? i0 : 0)) * a.dpad);
        const int *r1 = reinterpret_cast<const int *>(a.qc + (row_base + (v1 ? i1 : 0)) * a.dpad);
#pragma unroll
        for (int ks = 0; ks < D32; ++ks) {
            qa[ks][0] = v0 ? r0[8 * ks + t] : 0;
            qa[ks][1] = v1 ? r1[8 * ks + t] : 0;
            qa[ks][2] = v0 ? r0[8 * ks + 4 + t] : 0;
            qa[ks][3] = v1 ? r1[8 * ks + 4 + t] : 0;
        }
    }
    const float dq0 = v0 ? a.qs[row_base + i0] : 1.f, dq1 = v1 ? a.qs[row_base + i1] : 1.f;

    float o[DV8][4];
#pragma unroll
    for (int nv = 0; nv < DV8; ++nv) o[nv][0] = o[nv][1] = o[nv][2] = o[nv][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    const int i_blk_max = min((int)dm.Sq - 1, q_tile * 64 + 63);
    const int i_warp_max = min((int)dm.Sq - 1, q0 + 15);
    const int jb_hi = causal ? i_blk_max / BLK + 1 : (int)a.n_blocks;

    // A key block comes in by cp.async.  Keys past the end of the sequence re-read the last
    // valid key (their scores are masked before use).
    auto stage = [&](int jb, int buf) {
        uint8_t *Ks = sm_tc + buf * kBufBytes, *Vs = Ks + (BLK + 8) * KP;
        float *kscale = reinterpret_cast<float *>(Vs + DV * VP), *vscale = kscale + BLK, *mscale = vscale + DV;
        const int j0 = jb * BLK, last = min(BLK, (int)dm.Skv - j0) - 1;
        const int8_t *ksrc = a.kc + (plane * dm.Skv + j0) * a.dpad;
        for (int idx = threadIdx.x; idx < BLK * (D / 16); idx += 128) {
            const int key = idx / (D / 16), piece = idx % (D / 16);
            cp_async16(Ks + key * KP + piece * 16, ksrc + (size_t)min(key, last) * a.dpad + piece * 16);
        }
        const int8_t *msrc = a.kmean_digits + (plane * a.n_blocks + jb) * (size_t)8 * a.dpad;
        for (int idx = threadIdx.x; idx < 8 * (D / 16); idx += 128) {
            const int row = idx / (D / 16), piece = idx % (D / 16);
            cp_async16(Ks + (BLK + row) * KP + piece * 16, msrc + (size_t)row * a.dpad + piece * 16);
        }
        if (threadIdx.x == 0)
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(
                             (uint32_t)__cvta_generic_to_shared(mscale)),
                         "l"(a.kmean_scale + plane * a.n_blocks + jb)
                         : "memory");
        const int8_t *vsrc = a.vc + (plane * a.n_blocks + jb) * (size_t)DV * a.bpad;
        for (int idx = threadIdx.x; idx < DV * (BLK / 16); idx += 128) {
            const int c = idx / (BLK / 16), piece = idx % (BLK / 16);
            cp_async16(Vs + c * VP + piece * 16, vsrc + (size_t)c * a.bpad + piece * 16);
        }
        for (int idx = threadIdx.x; idx < BLK; idx += 128)  // 4-byte copies: the offset need not be 16-byte aligned
            asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(
                             (uint32_t)__cvta_generic_to_shared(kscale + idx)),
                         "l"(a.ks + plane * dm.Skv + j0 + min(idx, last))
                         : "memory");
        for (int idx = threadIdx.x; idx < DV / 4; idx += 128)
            cp_async16(vscale + idx * 4, a.vs + (plane * a.n_blocks + jb) * DV + idx * 4);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    if (jb_hi > 0) stage(0, 0);
    for (int jb = 0; jb < jb_hi; ++jb) {
        const int j0 = jb * BLK, kj = min(BLK, (int)dm.Skv - j0);
        if (jb + 1 < jb_hi) {
            stage(jb + 1, (jb + 1) & 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();  // block jb has landed for every thread
        const uint8_t *Ks = sm_tc + (jb & 1) * kBufBytes, *Vs = Ks + (BLK + 8) * KP;
        const float *kscale = reinterpret_cast<const float *>(Vs + DV * VP), *vscale = kscale + BLK,
                    *mscale = vscale + DV;
        // every key of the block may be masked for this warp: it still meets the barriers
        const bool skip = causal && j0 > i_warp_max;
        if (!skip) {

        // shift = (dQ * Qhat) . mean, per query row, from the mean's three digit rows: columns 0,
        // 1 (lane t = 0) and 2 (t = 1) of one more 8-column MMA tile
        float sh0, sh1;
        {
            int accm[4] = {0, 0, 0, 0};
            const uint8_t *mr = Ks + (BLK + lane % 8) * KP + 16 * (lane / 8);
#pragma unroll
            for (int kp = 0; kp < D32 / 2; ++kp) {
                int b[4];
                ldsm_x4(mr + 64 * kp, b[0], b[1], b[2], b[3]);
                mma_s8(accm, qa[2 * kp], b[0], b[1]);
                mma_s8(accm, qa[2 * kp + 1], b[2], b[3]);
            }
            float p0 = t == 0 ? (float)accm[0] * 65536.f + (float)accm[1] * 256.f : t == 1 ? (float)accm[0] : 0.f;
            float p1 = t == 0 ? (float)accm[2] * 65536.f + (float)accm[3] * 256.f : t == 1 ? (float)accm[2] : 0.f;
            p0 += __shfl_xor_sync(0xffffffffu, p0, 1);
            p0 += __shfl_xor_sync(0xffffffffu, p0, 2);
            p1 += __shfl_xor_sync(0xffffffffu, p1, 1);
            p1 += __shfl_xor_sync(0xffffffffu, p1, 2);
            const float unit = mscale[0];
            sh0 = p0 * unit * dq0;
            sh1 = p1 * unit * dq1;
        }

        // S = Qhat Khat^T
        int acc[NT][4];
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0;
            const uint8_t *kr = Ks + (8 * nt + lane % 8) * KP + 16 * (lane / 8);
#pragma unroll
            for (int kp = 0; kp < D32 / 2; ++kp) {
                int b[4];  // B fragments of k-steps 2 kp and 2 kp + 1
                ldsm_x4(kr + 64 * kp, b[0], b[1], b[2], b[3]);
                mma_s8(acc[nt], qa[2 * kp], b[0], b[1]);
                mma_s8(acc[nt], qa[2 * kp + 1], b[2], b[3]);
            }
        }
        // scores and the new row maxima.  Only the block on the diagonal, the last block of a
        // ragged sequence and a warp with rows past the end need the per-element mask.
        float mn0 = m0, mn1 = m1;
        const bool masked = kj < BLK || !v0 || !v1 || (causal && j0 + BLK - 1 > q0);
        if (masked) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int kk = 8 * nt + 2 * t + e, j = j0 + kk;
                    const float ksc = kscale[kk];
                    float s0 = fmaf((float)acc[nt][e] * dq0, ksc, sh0);
                    float s1 = fmaf((float)acc[nt][2 + e] * dq1, ksc, sh1);
                    if (kk >= kj || !v0 || (causal && j > i0)) s0 = -INFINITY;
                    if (kk >= kj || !v1 || (causal && j > i1)) s1 = -INFINITY;
                    acc[nt][e] = __float_as_int(s0);
                    acc[nt][2 + e] = __float_as_int(s1);
                    mn0 = fmaxf(mn0, s0);
                    mn1 = fmaxf(mn1, s1);
                }
        } else {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const float2 ksc = *reinterpret_cast<const float2 *>(kscale + 8 * nt + 2 * t);
                const float s00 = fmaf((float)acc[nt][0] * dq0, ksc.x, sh0);
                const float s01 = fmaf((float)acc[nt][1] * dq0, ksc.y, sh0);
                const float s10 = fmaf((float)acc[nt][2] * dq1, ksc.x, sh1);
                const float s11 = fmaf((float)acc[nt][3] * dq1, ksc.y, sh1);
                acc[nt][0] = __float_as_int(s00);
                acc[nt][1] = __float_as_int(s01);
                acc[nt][2] = __float_as_int(s10);
                acc[nt][3] = __float_as_int(s11);
                mn0 = fmaxf(mn0, fmaxf(s00, s01));
                mn1 = fmaxf(mn1, fmaxf(s10, s11));
            }
        }
        mn0 = fmaxf(mn0, __shfl_xor_sync(0xffffffffu, mn0, 1));
        mn0 = fmaxf(mn0, __shfl_xor_sync(0xffffffffu, mn0, 2));
        mn1 = fmaxf(mn1, __shfl_xor_sync(0xffffffffu, mn1, 1));
        mn1 = fmaxf(mn1, __shfl_xor_sync(0xffffffffu, mn1, 2));
        const float alpha0 = (mn0 == -INFINITY) ? 0.f : expf(m0 - mn0);
        const float alpha1 = (mn1 == -INFINITY) ? 0.f : expf(m1 - mn1);
        // P scaled by 127 (the static P scale): 127 exp(s - m) = exp2(s log2e - m log2e + log2 127),
        // one FMA and one ex2 per score.  Its sum is 127 l and the output below is accumulated
        // as 127 o, so the two factors cancel in o / l and no multiply by 1/127 is needed.
        // pa[slab] is the A fragment of the slab's 32 keys.
        constexpr float kLog2e = 1.4426950408889634f, kLog2_127 = 6.988684686772166f;
        const float off0 = (mn0 == -INFINITY) ? -INFINITY : kLog2_127 - mn0 * kLog2e;
        const float off1 = (mn1 == -INFINITY) ? -INFINITY : kLog2_127 - mn1 * kLog2e;
        int pa[BLK32][4];
        float es0 = 0.f, es1 = 0.f;
#pragma unroll
        for (int sl = 0; sl < BLK32; ++sl)
#pragma unroll
            for (int pair = 0; pair < 2; ++pair) {
                int c0[4], c1[4];
#pragma unroll
                for (int jj = 0; jj < 2; ++jj)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int nt = 4 * sl + 2 * pair + jj;
                        // a masked score is -inf: exp2 gives 0; a fully masked row has off = -inf
                        // and s = -inf, whose sum would be NaN, hence the guard in off
                        const float s0 = __int_as_float(acc[nt][e]), s1 = __int_as_float(acc[nt][2 + e]);
                        const float p0 = (mn0 == -INFINITY) ? 0.f : exp2f(fmaf(s0, kLog2e, off0));
                        const float p1 = (mn1 == -INFINITY) ? 0.f : exp2f(fmaf(s1, kLog2e, off1));
                        es0 += p0;
                        es1 += p1;
                        // p is in [0, 127]: the conversion rounds to nearest even like rint
                        c0[2 * jj + e] = __float2int_rn(p0);
                        c1[2 * jj + e] = __float2int_rn(p1);
                    }
                pa[sl][2 * pair] = pack_codes(c0);
                pa[sl][2 * pair + 1] = pack_codes(c1);
            }
        // PV, one 8-channel tile at a time
#pragma unroll
        for (int nv = 0; nv < DV8; ++nv) {
            int pv[4] = {0, 0, 0, 0};
            if (BLK32 == 1) {
                int b[2];
                ldsm_x2(Vs + (8 * nv + lane % 8) * VP + 16 * ((lane / 8) & 1), b[0], b[1]);
                mma_s8(pv, pa[0], b[0], b[1]);
            } else {
                const uint8_t *vr = Vs + (8 * nv + lane % 8) * VP + 16 * (lane / 8);
#pragma unroll
                for (int sp = 0; sp < BLK32 / 2; ++sp) {
                    int b[4];  // B fragments of slabs 2 sp and 2 sp + 1
                    ldsm_x4(vr + 64 * sp, b[0], b[1], b[2], b[3]);
                    mma_s8(pv, pa[2 * sp], b[0], b[1]);
                    mma_s8(pv, pa[2 * sp + 1], b[2], b[3]);
                }
            }
            const float vd0 = vscale[8 * nv + 2 * t], vd1 = vscale[8 * nv + 2 * t + 1];
            o[nv][0] = fmaf(alpha0, o[nv][0], (float)pv[0] * vd0);
            o[nv][1] = fmaf(alpha0, o[nv][1], (float)pv[1] * vd1);
            o[nv][2] = fmaf(alpha1, o[nv][2], (float)pv[2] * vd0);
            o[nv][3] = fmaf(alpha1, o[nv][3], (float)pv[3] * vd1);
        }
        l0 = alpha0 * l0 + es0;
        l1 = alpha1 * l1 + es1;
        if (mn0 != -INFINITY) m0 = mn0;
        if (mn1 != -INFINITY) m1 = mn1;
        }
        __syncthreads();  // the buffer may be refilled
    }
    // each lane summed P over its own columns only
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
#pragma unroll
    for (int nv = 0; nv < DV8; ++nv) {
        const int c = 8 * nv + 2 * t;
        if (v0)
            *reinterpret_cast<float2 *>(a.out + (row_base + i0) * DV + c) =
                make_float2(o[nv][0] / l0, o[nv][1] / l0);
        if (v1)
            *reinterpret_cast<float2 *>(a.out + (row_base + i1) * DV + c) =
                make_float2(o[nv][2] / l1, o[nv][3] / l1);
    }
}

// ------------------------------------------------------------------ Sage on tcgen05 (kind::i8)
// The same arithmetic once more, with both integer products on the 5th-generation tensor
// cores: tcgen05.mma kind::i8 (s8 x s8 -> s32) with the accumulators in tensor memory.  Built
// for head_dim = val_dim = 128 and the Sage key block of 64 (benchmark configuration 2).
//   * A CTA owns 128 queries; query row r is tensor-memory lane r.  Its 512 threads are four
//     groups of 128: thread (g, r) works on row r's score columns 32 g .. 32 g + 31 of the
//     iteration (groups 0, 1: the first Sage block; 2, 3: the second) and on output channels
//     32 g .. 32 g + 31.  What a row's four threads have to agree on (the blocks' maxima and
//     sums of P) goes through shared memory; every thread then derives the same running
//     maximum, alphas and l.
//   * One iteration covers TWO Sage blocks (128 keys): S = Qhat [Khat_a; Khat_b; mean digits]^T
//     is one 128 x 144 x 128 product (the sixteen extra B rows are the digit rows of the two
//     blocks' channel means, which give the per-row shift), then the online softmax runs block
//     by block exactly as in the other kernels - block b's codes use the maximum after block a -
//     and the two PV products (128 x 128 x 64 each, because V has one scale set per block) go
//     to two accumulators that alias S, which has been read out by then.
//   * Operands are staged by cp.async into 128-byte-swizzled K-major tiles (rows of 128 bytes:
//     Q and K rows are 128 channels, P and V rows are the iteration's 128 keys, V_a and V_b
//     side by side), two iterations ahead.  The P codes go from registers to shared memory and
//     are the A operand of PV.
//   * The products run beside the arithmetic: tensor memory holds two accumulator regions, S of
//     iteration it + 1 is issued as soon as S of iteration it has been read out and runs while
//     the threads exponentiate; PV of iteration it is issued at the end of the iteration and is
//     folded into the output in the middle of the next one, after that one's scores.
// All waits on the MMA barriers are bounded (bit 1 of the context's error word on expiry).
constexpr int kUQ = 128, kUBlk = 64, kUKeys = 2 * kUBlk, kUD = 128;
constexpr int kUThreads = 512, kUGroups = kUThreads / kUQ;
// The warps whose lane 0 issues the S products, the record copies and the PV products.  Each of
// these instructions (tcgen05.mma, tcgen05.commit, the mbarrier operations, the bulk copy) takes
// its thread a hundred cycles and more to issue, one after the other: spread over three warps
// on three schedulers they overlap, and no warp falls far behind the others at the CTA barriers.
constexpr uint32_t kUWarpS = 0, kUWarpRec = 5, kUWarpPV = 10;
constexpr int kUSRows = kUKeys + 16;  // keys + 2 x 8 mean-digit rows: N of the S product
constexpr uint32_t kUQBytes = kUQ * 128, kUPBytes = kUQ * 128;
constexpr int kUBufs = 3;  // record buffers: an iteration's record is fetched two iterations ahead
static_assert(kURecKBytes == kUSRows * 128 && kURecVBytes == kUD * 128, "the record holds the kernel's tiles");
constexpr uint32_t kUSmemBytes = kUQBytes + kUBufs * kURecStride + kUPBytes + 2 * kUGroups * kUQ * 4 + 64;
constexpr uint32_t kUTmemCols = 512, kUPVCol = 256;  // S (144 columns) at column 0, the two PV accumulators from column 256
constexpr uint32_t kUWaitLimitDefault = 1u << 22;

// s8 x s8 -> s32, both operands K-major, M = 128, N = n
__device__ __forceinline__ uint32_t umma_idesc_i8(uint32_t n) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((uint32_t)(kUQ >> 4) << 24);
}
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(kUThreads, 1)
attention_sage_umma_kernel(SageArgs a, AttnDims dm, int causal, uint32_t wait_limit, int *error) {
    extern __shared__ __align__(1024) uint8_t sm_u_raw[];
    // (the swizzled tiles want 1024-byte alignment; the launch asks for 1 KB more than kUSmemBytes)
    uint8_t *sm_u = sm_u_raw + ((1024 - (smem_u32(sm_u_raw) & 1023)) & 1023);
    uint8_t *Qs = sm_u, *Rb = Qs + kUQBytes, *Ps = Rb + kUBufs * kURecStride;  // Q tile, record buffers, P tile
    float *xm = reinterpret_cast<float *>(Ps + kUPBytes), *xe = xm + kUGroups * kUQ;  // [group][row]: block maxima, sums of P
    uint64_t *bar_s = reinterpret_cast<uint64_t *>(xe + kUGroups * kUQ), *bar_pv = bar_s + 1, *bar_drain = bar_s + 2;
    uint64_t *bar_rec = bar_s + 3;  // [kUBufs]: a record has landed in its buffer
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar_rec + kUBufs);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t tid = threadIdx.x, warp = tid / 32;
    const uint32_t g = tid / kUQ, r = tid % kUQ;  // column group, query row
    const int my_blk = g / 2;
    const int h = blockIdx.y, b = blockIdx.z, kvh = h / dm.group;
    const size_t plane = (size_t)b * dm.KV + kvh;
    // under causal masking the last query tiles have the most key blocks: start them first
    const int q_tile = causal ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x;
    const int q0 = q_tile * kUQ, i = q0 + (int)r;
    const bool valid = i < (int)dm.Sq;
    const size_t row_base = ((size_t)b * dm.H + h) * dm.Sq;
    const int S = (int)dm.Skv, n_blocks = (int)a.n_blocks;

    if (tid == 0) {
        mbar_init(bar_s, 1);
        mbar_init(bar_pv, 1);
        mbar_init(bar_drain, 2);
        for (int bi = 0; bi < kUBufs; ++bi) mbar_init(bar_rec + bi, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kUTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // a warp reaches the 32 lanes (rows) 32 (warp % 4) ..; the groups differ in their columns
    const uint32_t tmem_base = *tmem_slot, my_tmem = tmem_base + (((warp % 4) * 32) << 16);

    // 16-byte piece `piece` of row `row` of a swizzled tile
    auto swz = [](uint8_t *tile, int row, int piece) { return tile + row * 128 + ((piece ^ (row & 7)) << 4); };
    // The record of iteration `it` (keys 128 it .., the key blocks 2 it and 2 it + 1) into its
    // buffer: one bulk copy, started by one thread, which completes on the buffer's barrier.
    const uint8_t *rec_src = a.rec + plane * (size_t)((n_blocks + 1) / 2) * kURecStride;
    auto stage = [&](int it) {
        const uint32_t bar = smem_u32(bar_rec + it % kUBufs);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kURecBytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         smem_u32(Rb + (it % kUBufs) * kURecStride)),
                     "l"(rec_src + (size_t)it * kURecStride), "r"(kURecBytes), "r"(bar)
                     : "memory");
    };

    const int i_blk_max = min((int)dm.Sq - 1, q0 + kUQ - 1);
    const int jb_hi = causal ? i_blk_max / kUBlk + 1 : n_blocks;
    const int n_it = (jb_hi + 1) / 2;
    for (int idx = tid; idx < kUQ * 8; idx += kUThreads) {
        const int row = idx / 8, piece = idx % 8;
        cp_async16(swz(Qs, row, piece), a.qc + (row_base + min(q0 + row, (int)dm.Sq - 1)) * a.dpad + piece * 16);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    const float dq = valid ? a.qs[row_base + i] : 1.f;

    // channels 32 g .. 32 g + 31 of row r, in pairs: the per-element arithmetic of this kernel
    // runs on the packed float32 instructions (two IEEE operations per issue slot: the same
    // results, half the instructions)
    float2 o[16];
#pragma unroll
    for (int c = 0; c < 16; ++c) o[c] = make_float2(0.f, 0.f);
    float m = -INFINITY, l = 0.f;
    float prev_alpha_a = 0.f, prev_alpha_b = 0.f;  // of the iteration whose PV is still to be folded in
    const uint32_t idesc_s = umma_idesc_i8(kUSRows), idesc_pv = umma_idesc_i8(kUD);
    const uint32_t limit = wait_limit ? wait_limit : kUWaitLimitDefault;
    bool dead = false;
    int dead_it = n_it;  // the iteration that gave up
    uint32_t v[32];
    auto issue_s = [&](int it) {  // S of iteration `it` (one thread)
        const uint32_t kt = smem_u32(Rb + (it % kUBufs) * kURecStride);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int k = 0; k < kUD / 32; ++k)
            umma_i8(tmem_base, umma_desc(smem_u32(Qs) + k * 32), umma_desc(kt + k * 32), idesc_s, k != 0);
        umma_commit(bar_s);
    };
    // o = alpha * o + PV * dV for one key block: `v` holds the block's 32 integer sums of this
    // thread's channels, `vd` points at their scales
    auto fold_block = [&](float al, const float *vd) {
        const float2 al2 = make_float2(al, al);
        const float4 *vd4 = reinterpret_cast<const float4 *>(vd);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float4 d = vd4[e];
            o[2 * e] = __ffma2_rn(al2, o[2 * e],
                                  __fmul2_rn(make_float2((float)(int)v[4 * e], (float)(int)v[4 * e + 1]), make_float2(d.x, d.y)));
            o[2 * e + 1] = __ffma2_rn(al2, o[2 * e + 1],
                                      __fmul2_rn(make_float2((float)(int)v[4 * e + 2], (float)(int)v[4 * e + 3]),
                                                 make_float2(d.z, d.w)));
        }
    };
    // the channel scales of V of iteration `it`, this thread's 32 channels of block a (block b: + kUD)
    auto vscale_of = [&](int it) {
        return reinterpret_cast<const float *>(Rb + (it % kUBufs) * kURecStride + kURecScaleOff) + kUKeys + 32 * g;
    };
    const bool lane0 = tid % 32 == 0;
    if (warp == kUWarpRec && lane0) {
        stage(0);
        if (n_it > 1) stage(1);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");  // (the Q tile)
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    // (if this wait gives up, no product is issued and every wait below gives up in turn)
    const bool first_landed = warp != kUWarpRec || mbar_wait(bar_rec, 0, abort_flag, limit);
    if (__syncthreads_and(first_landed) && warp == kUWarpS && lane0) issue_s(0);
    __syncwarp();
    for (int it = 0; it < n_it; ++it) {
        const int buf = it % kUBufs;
        const float *kscale = reinterpret_cast<const float *>(Rb + buf * kURecStride + kURecScaleOff);
        const float *mscale = kscale + kUKeys + 2 * kUD;
        // A warp whose wait gives up skips what needs the products and votes at the next CTA
        // barrier: the verdict is taken by the whole CTA, nobody goes on to a barrier the others
        // have left.
        // (one warp saw this iteration's record land before a CTA barrier that lies behind us,
        // which makes the record's scales visible to this thread)
        bool ok = mbar_wait(bar_s, it & 1, abort_flag, limit);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

        // ---- this thread's 32 scores of its Sage block
        const int jb = 2 * it + my_blk, j0 = jb * kUBlk, kj = min(kUBlk, S - j0);
        const bool live = jb < jb_hi;
        float shift = 0.f;
        if (ok) {
            uint32_t c0, c1, c2, c3;
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(c0), "=r"(c1), "=r"(c2), "=r"(c3)
                         : "r"(my_tmem + kUKeys + 8 * my_blk)
                         : "memory");
            tmem_ld32(my_tmem + 32 * g, v);
            tmem_ld_wait();
            (void)c3;
            shift = (((float)(int)c0 * 65536.f + (float)(int)c1 * 256.f) + (float)(int)c2) * mscale[my_blk] * dq;
        }
        // only the iteration on the diagonal, the last one of a ragged sequence, a tile with rows
        // past the end and a missing second block need the per-element mask
        const int it_j0 = it * kUKeys;
        const bool masked = it_j0 + kUKeys > S || q0 + kUQ > (int)dm.Sq || !live || 2 * it + 1 >= jb_hi ||
                            (causal && it_j0 + kUKeys - 1 > q0);
        float s[32];
        float bm = -INFINITY;
        const float *ksc = kscale + 32 * g;
        if (masked) {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                const int kk = 32 * (int)(g % 2) + e, j = j0 + kk;
                float sc = fmaf((float)(int)v[e] * dq, ksc[e], shift);
                if (!live || kk >= kj || !valid || (causal && j > i)) sc = -INFINITY;
                s[e] = sc;
                bm = fmaxf(bm, sc);
            }
        } else {
            const float2 dq2 = make_float2(dq, dq), shift2 = make_float2(shift, shift);
            const float4 *ksc4 = reinterpret_cast<const float4 *>(ksc);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float4 d = ksc4[e];
                const float2 sa = __ffma2_rn(__fmul2_rn(make_float2((float)(int)v[4 * e], (float)(int)v[4 * e + 1]), dq2),
                                             make_float2(d.x, d.y), shift2);
                const float2 sb = __ffma2_rn(__fmul2_rn(make_float2((float)(int)v[4 * e + 2], (float)(int)v[4 * e + 3]), dq2),
                                             make_float2(d.z, d.w), shift2);
                s[4 * e] = sa.x, s[4 * e + 1] = sa.y, s[4 * e + 2] = sb.x, s[4 * e + 3] = sb.y;
                bm = fmaxf(fmaxf(bm, fmaxf(sa.x, sa.y)), fmaxf(sb.x, sb.y));
            }
        }
        xm[g * kUQ + r] = bm;
        // the record of the next iteration was asked for an iteration ago
        if (warp == kUWarpRec && it + 1 < n_it && ok)
            ok = mbar_wait(bar_rec + (it + 1) % kUBufs, ((it + 1) / kUBufs) & 1, abort_flag, limit);
        // after the barrier every thread has read S of this iteration out of tensor memory
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        if (!__syncthreads_and(ok)) {
            dead = true;
            dead_it = it;
            break;
        }
        if (warp == kUWarpS && lane0 && it + 1 < n_it) issue_s(it + 1);  // runs while the threads exponentiate
        __syncwarp();
        // ---- the row's maxima after block a and after block b (the same in its four threads)
        const float bm_a = fmaxf(xm[r], xm[kUQ + r]), bm_b = fmaxf(xm[2 * kUQ + r], xm[3 * kUQ + r]);
        const float mn_a = fmaxf(m, bm_a);
        const float alpha_a = (mn_a == -INFINITY) ? 0.f : expf(m - mn_a);
        const float m_a = (mn_a == -INFINITY) ? m : mn_a;
        const float mn_b = fmaxf(m_a, bm_b);
        const float alpha_b = (mn_b == -INFINITY) ? 0.f : expf(m_a - mn_b);
        const float m_b = (mn_b == -INFINITY) ? m_a : mn_b;
        const float mn = my_blk ? mn_b : mn_a;
        // P scaled by 127 (the static P scale): 127 exp(s - m) = exp2(s log2e - m log2e + log2 127).
        // A masked score is -inf and so is `off` of a row without any key so far: their sum is
        // -inf (never NaN), of which ex2 gives 0.
        constexpr float kLog2e = 1.4426950408889634f, kLog2_127 = 6.988684686772166f;
        const float off = (mn == -INFINITY) ? -INFINITY : kLog2_127 - mn * kLog2e;
        const float2 log2e2 = make_float2(kLog2e, kLog2e), off2 = make_float2(off, off);
        float2 es2 = make_float2(0.f, 0.f);  // the sums over the even and the odd columns
        auto exp_piece = [&](int piece) {  // 16 of the thread's 32 columns: exponentiate, round, store the codes
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                int c[4];
#pragma unroll
                for (int e = 0; e < 4; e += 2) {
                    const int at = 16 * piece + 4 * q + e;
                    const float2 arg = __ffma2_rn(make_float2(s[at], s[at + 1]), log2e2, off2);
                    const float2 pe = make_float2(ex2_approx(arg.x), ex2_approx(arg.y));
                    es2 = __fadd2_rn(es2, pe);
                    c[e] = __float2int_rn(pe.x);  // in [0, 127]: rounds to nearest even like rint
                    c[e + 1] = __float2int_rn(pe.y);
                }
                w[q] = pack_codes(c);
            }
            *reinterpret_cast<uint4 *>(swz(Ps, (int)r, 2 * g + piece)) = make_uint4(w[0], w[1], w[2], w[3]);
        };
        // ---- the exponentials of this iteration (bound by the special-function unit) and, between
        // them, the products of the iteration before folded into the output (bound by issue slots):
        // with the warps of a scheduler at different places of this stretch the two overlap.  The
        // PV accumulators have a tensor-memory region of their own, so they may stay there until
        // the next PV product is issued after the second barrier.  (Both blocks of the iteration
        // before exist: only the last iteration can lack its second block.)
        bool pv_ok = true;
        if (it > 0) {
            pv_ok = mbar_wait(bar_pv, (it - 1) & 1, abort_flag, limit);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        const bool fold = it > 0 && pv_ok;
        const float *vd_prev = vscale_of(it + kUBufs - 1);
        if (fold) tmem_ld32(my_tmem + kUPVCol + 32 * g, v);
        exp_piece(0);
        if (fold) {
            tmem_ld_wait();
            fold_block(prev_alpha_a, vd_prev);
            tmem_ld32(my_tmem + kUPVCol + kUD + 32 * g, v);
        }
        exp_piece(1);
        if (fold) {
            tmem_ld_wait();
            fold_block(prev_alpha_b, vd_prev + kUD);
        }
        xe[g * kUQ + r] = es2.x + es2.y;
        // ---- PV of this iteration: the P codes are in shared memory, the accumulators of the
        // iteration before have been read out, and nobody reads that iteration's record any more
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        if (!__syncthreads_and(pv_ok)) {
            dead = true;
            dead_it = it;
            break;
        }
        if (lane0) {
            if (warp == kUWarpPV) {
                const uint32_t vt = smem_u32(Rb + buf * kURecStride + kURecKBytes);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (int blk = 0; blk < 2; ++blk)
#pragma unroll
                    for (int k = 0; k < 2; ++k)
                        umma_i8(tmem_base + kUPVCol + kUD * blk, umma_desc(smem_u32(Ps) + (2 * blk + k) * 32),
                                umma_desc(vt + (2 * blk + k) * 32), idesc_pv, k != 0);
                umma_commit(bar_pv);
            }
            if (warp == kUWarpRec && it + 2 < n_it) stage(it + 2);  // into the buffer of the iteration before
        }
        __syncwarp();
        l = alpha_a * l + (xe[r] + xe[kUQ + r]);
        l = alpha_b * l + (xe[2 * kUQ + r] + xe[3 * kUQ + r]);
        m = m_b;
        prev_alpha_a = alpha_a;
        prev_alpha_b = alpha_b;
    }
    if (!dead) {
        if (!__syncthreads_and(mbar_wait(bar_pv, (n_it - 1) & 1, abort_flag, limit))) {
            dead = true;
        } else {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float *vd_last = vscale_of(n_it - 1);
            tmem_ld32(my_tmem + kUPVCol + 32 * g, v);
            tmem_ld_wait();
            fold_block(prev_alpha_a, vd_last);
            if (2 * (n_it - 1) + 1 < jb_hi) {  // (the same for the whole CTA)
                tmem_ld32(my_tmem + kUPVCol + kUD + 32 * g, v);
                tmem_ld_wait();
                fold_block(prev_alpha_b, vd_last + kUD);
            }
        }
    }
    if (dead) {
        // Given up: before tensor memory is handed back, the products that were issued must have
        // finished.  A commit on a barrier of its own arrives when everything issued so far is
        // done; it is waited for with the default (long) limit, not the one that just expired.
        // The same for the records still on their way into shared memory: the one of the
        // iteration that gave up and the one after it (later ones have not been asked for).
        __syncthreads();
        // (a commit covers the products its own thread has issued: both issuing threads commit)
        if ((warp == kUWarpS || warp == kUWarpPV) && lane0) umma_commit(bar_drain);
        __syncwarp();
        if (warp == 0) {
            volatile int never = 0;
            (void)mbar_wait(bar_drain, 0, &never, kUWaitLimitDefault);
            for (int k = dead_it; k < min(n_it, dead_it + 2); ++k)
                (void)mbar_wait(bar_rec + k % kUBufs, (k / kUBufs) & 1, &never, kUWaitLimitDefault);
        }
    }
    if (dead) *abort_flag = 1;
    if (valid && !dead) {
        float *dst = a.out + (row_base + i) * kUD + 32 * g;
#pragma unroll
        for (int c = 0; c < 16; c += 2)
            *reinterpret_cast<float4 *>(dst + 2 * c) =
                make_float4(o[c].x / l, o[c].y / l, o[c + 1].x / l, o[c + 1].y / l);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kUTmemCols)
                     : "memory");
    if (tid == 0 && *abort_flag) atomicOr(error, 1);
}

// ------------------------------------------------------------------ the block-scale variant
// The benchmark specification's wording of Sage, which is NOT the reference's arithmetic: Q and
// K quantised to INT8 with ONE scale per 64-token block (K after its block's channel mean has
// been removed, the mean's contribution added back through the digit rows as above), the
// scores' product on tcgen05 kind::i8 exactly as in attention_sage_umma_kernel, and then P and
// V in bfloat16: the PV product is tcgen05 kind::f16 with the output accumulator STAYING in
// tensor memory over the whole key loop.  Nothing is folded per iteration; when a row's maximum
// has grown by more than a factor 2^kBLazy since the accumulator's reference maximum was set, the row's
// threads rescale their columns of the accumulator in place (tcgen05.ld, multiply, tcgen05.st)
// and move the reference; otherwise the exponentials keep the old reference (they may exceed
// 1 by a factor of up to 2^kBLazy, which bfloat16 and the float32 sums hold without loss of
// anything that matters).  Same thread layout, records, barriers and bounded waits as the
// kernel above.  No reference implementation of this variant exists: its parity is against a
// NumPy restatement of the wording only.
constexpr uint32_t kBOCol = 256;  // the output accumulator: tensor-memory columns 256 .. 383
constexpr uint32_t kBPBytes = 2 * kUQ * 128;  // P as two bfloat16 tiles (keys of block a, of block b)
constexpr uint32_t kBSmemBytes = kUQBytes + kUBufs * kBRecStride + kBPBytes + 2 * kUGroups * kUQ * 4 + 64;
constexpr float kBLazy = 8.0f;  // in the log2 domain the kernel keeps its scores in: a factor of 256
static_assert(kBSmemBytes + 1024 <= 227 * 1024, "the block-scale kernel's shared memory");

__device__ __forceinline__ uint32_t umma_idesc_bf16(uint32_t n) {  // bf16 x bf16 -> f32, K-major, M = 128
    return (1u << 4) | (1u << 7) | (1u << 10) | ((n >> 3) << 17) | ((uint32_t)(kUQ >> 4) << 24);
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, %22, "
        "%23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
        "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
        "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
}

__global__ void __launch_bounds__(kUThreads, 1)
attention_sage_block_kernel(SageArgs a, AttnDims dm, int causal, uint32_t wait_limit, int *error) {
    extern __shared__ __align__(1024) uint8_t sm_b_raw[];
    uint8_t *sm_b = sm_b_raw + ((1024 - (smem_u32(sm_b_raw) & 1023)) & 1023);
    uint8_t *Qs = sm_b, *Rb = Qs + kUQBytes, *Ps = Rb + kUBufs * kBRecStride;  // Q tile, record buffers, two P tiles
    float *xm = reinterpret_cast<float *>(Ps + kBPBytes), *xe = xm + kUGroups * kUQ;
    uint64_t *bar_s = reinterpret_cast<uint64_t *>(xe + kUGroups * kUQ), *bar_pv = bar_s + 1, *bar_drain = bar_s + 2;
    uint64_t *bar_rec = bar_s + 3;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar_rec + kUBufs);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t tid = threadIdx.x, warp = tid / 32;
    const uint32_t g = tid / kUQ, r = tid % kUQ;  // column group (32 keys of the iteration), query row
    const int my_blk = g / 2;
    const int h = blockIdx.y, b = blockIdx.z, kvh = h / dm.group;
    const size_t plane = (size_t)b * dm.KV + kvh;
    const int q_tile = causal ? (int)gridDim.x - 1 - (int)blockIdx.x : (int)blockIdx.x;
    const int q0 = q_tile * kUQ, i = q0 + (int)r;
    const bool valid = i < (int)dm.Sq;
    const size_t row_base = ((size_t)b * dm.H + h) * dm.Sq;
    const int S = (int)dm.Skv, n_blocks = (int)a.n_blocks;

    if (tid == 0) {
        mbar_init(bar_s, 1);
        mbar_init(bar_pv, 1);
        mbar_init(bar_drain, 2);
        for (int bi = 0; bi < kUBufs; ++bi) mbar_init(bar_rec + bi, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(kUTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot, my_tmem = tmem_base + (((warp % 4) * 32) << 16);

    auto swz = [](uint8_t *tile, int row, int piece) { return tile + row * 128 + ((piece ^ (row & 7)) << 4); };
    const uint8_t *rec_src = a.rec + plane * (size_t)((n_blocks + 1) / 2) * kBRecStride;
    auto stage = [&](int it) {
        const uint32_t bar = smem_u32(bar_rec + it % kUBufs);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kBRecBytes) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                         smem_u32(Rb + (it % kUBufs) * kBRecStride)),
                     "l"(rec_src + (size_t)it * kBRecStride), "r"(kBRecBytes), "r"(bar)
                     : "memory");
    };

    const int i_blk_max = min((int)dm.Sq - 1, q0 + kUQ - 1);
    const int jb_hi = causal ? i_blk_max / kUBlk + 1 : n_blocks;
    const int n_it = (jb_hi + 1) / 2;
    for (int idx = tid; idx < kUQ * 8; idx += kUThreads) {
        const int row = idx / 8, piece = idx % 8;
        cp_async16(swz(Qs, row, piece), a.qc + (row_base + min(q0 + row, (int)dm.Sq - 1)) * a.dpad + piece * 16);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    const float dq = valid ? a.qs[row_base + i] : 1.f;

    float m = -INFINITY, mref = -INFINITY, l = 0.f;  // running maximum, the accumulator's reference, sum of P
    const uint32_t idesc_s = umma_idesc_i8(kUSRows), idesc_o = umma_idesc_bf16(kUD);
    const uint32_t limit = wait_limit ? wait_limit : kUWaitLimitDefault;
    bool dead = false;
    int dead_it = n_it;
    uint32_t v[32];
    auto issue_s = [&](int it) {
        const uint32_t kt = smem_u32(Rb + (it % kUBufs) * kBRecStride);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int k = 0; k < kUD / 32; ++k)
            umma_i8(tmem_base, umma_desc(smem_u32(Qs) + k * 32), umma_desc(kt + k * 32), idesc_s, k != 0);
        umma_commit(bar_s);
    };
    const bool lane0 = tid % 32 == 0;
    if (warp == kUWarpRec && lane0) {
        stage(0);
        if (n_it > 1) stage(1);
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    const bool first_landed = warp != kUWarpRec || mbar_wait(bar_rec, 0, abort_flag, limit);
    if (__syncthreads_and(first_landed) && warp == kUWarpS && lane0) issue_s(0);
    __syncwarp();
    constexpr float kLog2e = 1.4426950408889634f;
    for (int it = 0; it < n_it; ++it) {
        const int buf = it % kUBufs;
        const float *kscale = reinterpret_cast<const float *>(Rb + buf * kBRecStride + kBRecScaleOff);
        const float *mscale = kscale + kUKeys;
        bool ok = mbar_wait(bar_s, it & 1, abort_flag, limit);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

        // ---- this thread's 32 scores
        const int jb = 2 * it + my_blk, j0 = jb * kUBlk, kj = min(kUBlk, S - j0);
        const bool live = jb < jb_hi;
        float shift = 0.f;
        if (ok) {
            uint32_t c0, c1, c2, c3;
            asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(c0), "=r"(c1), "=r"(c2), "=r"(c3)
                         : "r"(my_tmem + kUKeys + 8 * my_blk)
                         : "memory");
            tmem_ld32(my_tmem + 32 * g, v);
            tmem_ld_wait();
            (void)c3;
            shift = (((float)(int)c0 * 65536.f + (float)(int)c1 * 256.f) + (float)(int)c2) * mscale[my_blk] * dq;
        }
        // Scores in the log2 domain: one scale per (query block, key block), so a thread's 32
        // scores are one fused multiply-add each: t = dot * (dQ dK log2 e) + shift log2 e.
        // Only the iteration on the diagonal, the last one of a ragged sequence, a tile with
        // rows past the end and a missing second block need the per-element mask.
        const float kk2 = dq * kscale[32 * g] * kLog2e, shift2 = shift * kLog2e;
        const int it_j0 = it * kUKeys;
        const bool masked = it_j0 + kUKeys > S || q0 + kUQ > (int)dm.Sq || !live || 2 * it + 1 >= jb_hi ||
                            (causal && it_j0 + kUKeys - 1 > q0);
        float s[32];
        float bm = -INFINITY;
        if (masked) {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
                const int kk = 32 * (int)(g % 2) + e, j = j0 + kk;
                float sc = fmaf((float)(int)v[e], kk2, shift2);
                if (!live || kk >= kj || !valid || (causal && j > i)) sc = -INFINITY;
                s[e] = sc;
                bm = fmaxf(bm, sc);
            }
        } else {
            const float2 k2 = make_float2(kk2, kk2), sh2 = make_float2(shift2, shift2);
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                const float2 sc = __ffma2_rn(make_float2((float)(int)v[2 * e], (float)(int)v[2 * e + 1]), k2, sh2);
                s[2 * e] = sc.x, s[2 * e + 1] = sc.y;
                bm = fmaxf(bm, fmaxf(sc.x, sc.y));
            }
        }
        xm[g * kUQ + r] = bm;
        if (warp == kUWarpRec && it + 1 < n_it && ok)
            ok = mbar_wait(bar_rec + (it + 1) % kUBufs, ((it + 1) / kUBufs) & 1, abort_flag, limit);
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        if (!__syncthreads_and(ok)) {
            dead = true;
            dead_it = it;
            break;
        }
        if (warp == kUWarpS && lane0 && it + 1 < n_it) issue_s(it + 1);
        __syncwarp();
        // ---- the row's maximum, and whether the accumulator's reference has to move
        const float mn = fmaxf(m, fmaxf(fmaxf(xm[r], xm[kUQ + r]), fmaxf(xm[2 * kUQ + r], xm[3 * kUQ + r])));
        float alpha = 1.f;
        if (mn > mref + kBLazy) {  // (also the first finite maximum: mref is -inf until then)
            alpha = mref == -INFINITY ? 0.f : ex2_approx(mref - mn);
            mref = mn;
        }
        m = mn;
        const float off = mref == -INFINITY ? 0.f : -mref;  // (a row without a key yet: every score is -inf)
        // the product of the iteration before has read the P tiles and written the accumulator
        bool pv_ok = true;
        if (it > 0) {
            pv_ok = mbar_wait(bar_pv, (it - 1) & 1, abort_flag, limit);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        }
        // ---- P in bfloat16 into this thread's four 16-byte pieces of its block's tile
        float es = 0.f;
        uint8_t *ptile = Ps + my_blk * (kUQ * 128);
#pragma unroll
        for (int piece = 0; piece < 4; ++piece) {
            uint32_t w[4];
#pragma unroll
            for (int qd = 0; qd < 4; ++qd) {
                const int at = 8 * piece + 2 * qd;
                const float2 arg = __fadd2_rn(make_float2(s[at], s[at + 1]), make_float2(off, off));
                const float p0 = ex2_approx(arg.x), p1 = ex2_approx(arg.y);
                es += p0 + p1;
                asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(w[qd]) : "f"(p1), "f"(p0));
            }
            *reinterpret_cast<uint4 *>(swz(ptile, (int)r, 4 * (int)(g % 2) + piece)) = make_uint4(w[0], w[1], w[2], w[3]);
        }
        xe[g * kUQ + r] = es;
        // ---- the accumulator moves to the new reference where a row of this warp needs it
        if (it > 0 && pv_ok && __any_sync(0xffffffffu, alpha != 1.f)) {
            tmem_ld32(my_tmem + kBOCol + 32 * g, v);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) * alpha);
            tmem_st32(my_tmem + kBOCol + 32 * g, v);
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        if (!__syncthreads_and(pv_ok)) {
            dead = true;
            dead_it = it;
            break;
        }
        if (lane0) {
            if (warp == kUWarpPV) {
                const uint32_t vt = smem_u32(Rb + buf * kBRecStride + kBRecKBytes);
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t acc = it > 0;
#pragma unroll
                for (int blk = 0; blk < 2; ++blk) {
                    if (2 * it + blk >= jb_hi) break;  // (a block that does not exist: its V tile is not defined)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        umma_bf16(tmem_base + kBOCol, umma_desc(smem_u32(Ps) + blk * (kUQ * 128) + k * 32),
                                  umma_desc(vt + blk * (kUD * 128) + k * 32), idesc_o, acc);
                        acc = 1;
                    }
                }
                umma_commit(bar_pv);
            }
            if (warp == kUWarpRec && it + 2 < n_it) stage(it + 2);
        }
        __syncwarp();
        l = alpha * l + ((xe[r] + xe[kUQ + r]) + (xe[2 * kUQ + r] + xe[3 * kUQ + r]));
    }
    if (!dead) {
        if (!__syncthreads_and(mbar_wait(bar_pv, (n_it - 1) & 1, abort_flag, limit))) {
            dead = true;
        } else {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            tmem_ld32(my_tmem + kBOCol + 32 * g, v);
            tmem_ld_wait();
        }
    }
    if (dead) {
        __syncthreads();
        if ((warp == kUWarpS || warp == kUWarpPV) && lane0) umma_commit(bar_drain);
        __syncwarp();
        if (warp == 0) {
            volatile int never = 0;
            (void)mbar_wait(bar_drain, 0, &never, kUWaitLimitDefault);
            for (int k = dead_it; k < min(n_it, dead_it + 2); ++k)
                (void)mbar_wait(bar_rec + k % kUBufs, (k / kUBufs) & 1, &never, kUWaitLimitDefault);
        }
        *abort_flag = 1;
    }
    if (valid && !dead) {
        float *dst = a.out + (row_base + i) * kUD + 32 * g;
#pragma unroll
        for (int c = 0; c < 32; c += 4)
            *reinterpret_cast<float4 *>(dst + c) =
                make_float4(__uint_as_float(v[c]) / l, __uint_as_float(v[c + 1]) / l, __uint_as_float(v[c + 2]) / l,
                            __uint_as_float(v[c + 3]) / l);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kUTmemCols)
                     : "memory");
    if (tid == 0 && *abort_flag) atomicOr(error, 1);
}

// ------------------------------------------------------------------ host side
std::string shape_debug(const qk_attention_shape *s) {
    // Rust's `{:?}` of AttentionShape (gpu_attention.rs:402-411)
    char buf[256];
    snprintf(buf, sizeof buf,
             "AttentionShape { batch: %zu, n_heads: %zu, n_kv_heads: %zu, seq_q: %zu, seq_kv: %zu, "
             "head_dim: %zu, val_dim: %zu }",
             s->batch, s->n_heads, s->n_kv_heads, s->seq_q, s->seq_kv, s->head_dim, s->val_dim);
    return buf;
}

// gpu_attention.rs:468-508 / :604-655: the checks shared by both faces, in the
// reference's order and with its texts.
qk_status validate_attention(const qk_attention_shape *s, size_t q_len, size_t k_len, size_t v_len,
                             bool sage, size_t block_size, size_t out_len) {
    if (!s) return qk::fail(QK_ERR_VALUE, "attention shape is null");
    if (s->batch == 0 || s->n_heads == 0 || s->n_kv_heads == 0)
        return qk::fail(QK_ERR_VALUE, "attention requires non-empty batch and head dimensions");
    if (s->n_heads % s->n_kv_heads != 0)
        return qk::fail(QK_ERR_VALUE, "n_kv_heads must divide n_heads: n_heads=%zu, n_kv_heads=%zu",
                        s->n_heads, s->n_kv_heads);
    if (s->seq_q == 0 || s->seq_kv == 0 || s->head_dim == 0 || s->val_dim == 0)
        return qk::fail(QK_ERR_VALUE, "attention requires non-empty sequence and head dimensions");
    if (sage) {
        if (s->seq_q != s->seq_kv)
            return qk::fail(QK_ERR_VALUE,
                            "sage attention is self-attention over one cache: seq_q=%zu, seq_kv=%zu",
                            s->seq_q, s->seq_kv);
        if (block_size == 0)
            return qk::fail(QK_ERR_VALUE,
                            "sage attention requires a positive block_size ([SA] \xC2\xA7"
                            "4's tile width)");
    }
    size_t eq = s->batch * s->n_heads * s->seq_q * s->head_dim;
    size_t ek = s->batch * s->n_kv_heads * s->seq_kv * s->head_dim;
    size_t ev = s->batch * s->n_kv_heads * s->seq_kv * s->val_dim;
    if (q_len != eq)
        return qk::fail(QK_ERR_VALUE, "query must hold %zu values for %s, got %zu", eq,
                        shape_debug(s).c_str(), q_len);
    if (k_len != ek)
        return qk::fail(QK_ERR_VALUE, "key must hold %zu values for %s, got %zu", ek,
                        shape_debug(s).c_str(), k_len);
    if (v_len != ev)
        return qk::fail(QK_ERR_VALUE, "value must hold %zu values for %s, got %zu", ev,
                        shape_debug(s).c_str(), v_len);
    uint64_t largest = eq > ek ? eq : ek;
    if (ev > largest) largest = ev;
    if (largest > qk::kIndexCeiling)
        return qk::fail(QK_ERR_VALUE,
                        sage ? "sage attention inputs exceed the device u32 index ceiling (%llu); "
                               "use the reference face"
                             : "attention inputs exceed the device u32 index ceiling (%llu); use "
                               "the CPU reference face",
                        (unsigned long long)qk::kIndexCeiling);
    size_t eo = s->batch * s->n_heads * s->seq_q * s->val_dim;
    if (out_len != eo)
        return qk::fail(QK_ERR_VALUE, "output must hold %zu values for %s, got %zu", eo,
                        shape_debug(s).c_str(), out_len);
    if (s->head_dim > 256 || s->val_dim > 256)
        return qk::fail(QK_ERR_VALUE, "head_dim/val_dim above 256 are not supported: %s",
                        shape_debug(s).c_str());
    return QK_OK;
}

AttnDims dims_of(const qk_attention_shape *s) {
    return {(uint32_t)s->batch,   (uint32_t)s->n_heads,  (uint32_t)s->n_kv_heads,
            (uint32_t)s->seq_q,   (uint32_t)s->seq_kv,   (uint32_t)s->head_dim,
            (uint32_t)s->val_dim, (uint32_t)(s->n_heads / s->n_kv_heads)};
}

template <int DPL>
qk_status launch_exact(qk_ctx *c, const float *q, const float *k, const float *v, float *out,
                       const AttnDims &dm, int causal) {
    size_t smem = 2 * kTK * 4 * (DPL + 4) * sizeof(float);
    if (smem > 48 * 1024)
        QK_CUDA(cudaFuncSetAttribute(attention_exact_kernel<DPL>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)qk::ceil_div(dm.Sq, kQT), dm.H, dm.B);
    attention_exact_kernel<DPL><<<grid, 256, smem, c->stream>>>(q, k, v, out, dm, causal);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    return QK_OK;
}

template <int WPL>
qk_status launch_sage(qk_ctx *c, const SageArgs &a, const AttnDims &dm, int causal) {
    size_t smem = (kTK * 4 * (WPL + 1) + kTK + 16 * WPL * (kTK / 4 + 1)) * sizeof(int);
    if (smem > 48 * 1024)
        QK_CUDA(cudaFuncSetAttribute(attention_sage_kernel<WPL>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)qk::ceil_div(dm.Sq, kQT), dm.H, dm.B);
    attention_sage_kernel<WPL><<<grid, 256, smem, c->stream>>>(a, dm, causal);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    return QK_OK;
}

template <int D32, int DV8, int BLK32>
qk_status launch_sage_tc(qk_ctx *c, const SageArgs &a, const AttnDims &dm, int causal) {
    constexpr int D = 32 * D32, DV = 8 * DV8, BLK = 32 * BLK32;
    const size_t smem = 2 * ((BLK + 8) * (D + 16) + DV * (BLK + 16) + (BLK + DV + 4) * sizeof(float));
    if (smem > 48 * 1024)
        QK_CUDA(cudaFuncSetAttribute(attention_sage_tc_kernel<D32, DV8, BLK32>,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)qk::ceil_div(dm.Sq, 64), dm.H, dm.B);
    attention_sage_tc_kernel<D32, DV8, BLK32><<<grid, 128, smem, c->stream>>>(a, dm, causal);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    return QK_OK;
}

// The tensor-core kernel is instantiated for the head sizes and Sage blocks that occur in
// practice; anything else takes the dp4a kernel.
bool sage_tc_eligible(const AttnDims &dm, size_t block) {
    return (dm.d == 64 || dm.d == 128) && dm.dv == dm.d && (block == 32 || block == 64 || block == 128);
}

template <int D32>
qk_status launch_sage_tc_block(qk_ctx *c, const SageArgs &a, const AttnDims &dm, int causal) {
    if (a.block == 32) return launch_sage_tc<D32, 4 * D32, 1>(c, a, dm, causal);
    if (a.block == 64) return launch_sage_tc<D32, 4 * D32, 2>(c, a, dm, causal);
    return launch_sage_tc<D32, 4 * D32, 4>(c, a, dm, causal);
}

}  // namespace

namespace qk {

// Device-buffer form of the Sage face: quantisers, then the main kernel.  `scratch` holds the
// codes and scales (sage_scratch_bytes of it).
size_t sage_scratch_bytes(const qk_attention_shape *s, size_t block_size) {
    const AttnDims dm = dims_of(s);
    const size_t S = dm.Skv;
    if (block_size > S) block_size = S;
    const size_t n_blocks = qk::ceil_div(S, block_size);
    const size_t widest = dm.d > dm.dv ? dm.d : dm.dv;
    const size_t wpl = widest <= 16 ? 1 : widest <= 64 ? 4 : widest <= 128 ? 8 : 16;
    const size_t dpad = wpl * 16, bpad = qk::ceil_div(block_size, kTK) * kTK;
    const size_t planes = (size_t)dm.B * dm.KV, qrows = (size_t)dm.B * dm.H * dm.Sq;
    auto up = [](size_t n) { return (n + 255) / 256 * 256; };
    return up(qrows * dpad) + up(qrows * 4) + up(planes * S * dpad) + up(planes * S * 4) +
           up(planes * n_blocks * dm.d * 4) + up(planes * n_blocks * dm.dv * bpad) +
           up(planes * n_blocks * dm.dv * 4) + up(planes * n_blocks * 8 * dpad) +
           up(planes * n_blocks * 4) + up(planes * ((n_blocks + 1) / 2) * kURecStride) + 1024;
}

// Where each piece of the Sage scratch lies, and the padded sizes the kernels use.
struct SageLayout {
    size_t block, n_blocks, wpl, dpad, bpad, planes, qrows;
    size_t o_qc, o_qs, o_kc, o_ks, o_km, o_vc, o_vs, o_md, o_ms, o_rec;
    bool tc;    // a tensor-core kernel runs: the mean digit rows are produced
    bool umma;  // ... the tcgen05 one, whose K and V operands are written as records (o_rec) only
};
SageLayout sage_layout(const qk_ctx *c, const AttnDims &dm, size_t block_size) {
    SageLayout L{};
    const size_t S = dm.Skv;
    if (block_size > S) block_size = S;  // one block covers the whole sequence either way
    L.block = block_size;
    L.n_blocks = qk::ceil_div(S, block_size);
    const size_t widest = dm.d > dm.dv ? dm.d : dm.dv;
    L.wpl = widest <= 16 ? 1 : widest <= 64 ? 4 : widest <= 128 ? 8 : 16;
    L.dpad = L.wpl * 16;                                   // four lanes x WPL words x four codes
    L.bpad = qk::ceil_div(block_size, kTK) * kTK;          // keys of a block, padded to the tile
    L.planes = (size_t)dm.B * dm.KV;
    L.qrows = (size_t)dm.B * dm.H * dm.Sq;
    auto up = [](size_t n) { return (n + 255) / 256 * 256; };
    size_t off = 0;
    auto take = [&](size_t bytes) { size_t o2 = off; off += up(bytes); return o2; };
    L.o_qc = take(L.qrows * L.dpad), L.o_qs = take(L.qrows * 4);
    L.o_kc = take(L.planes * S * L.dpad), L.o_ks = take(L.planes * S * 4);
    L.o_km = take(L.planes * L.n_blocks * dm.d * 4);
    L.o_vc = take(L.planes * L.n_blocks * dm.dv * L.bpad), L.o_vs = take(L.planes * L.n_blocks * dm.dv * 4);
    L.o_md = take(L.planes * L.n_blocks * 8 * L.dpad), L.o_ms = take(L.planes * L.n_blocks * 4);
    L.o_rec = take(L.planes * ((L.n_blocks + 1) / 2) * kURecStride);  // (+ up to 1023 bytes to align it)
    L.tc = c->sage_kernel != 0 && sage_tc_eligible(dm, block_size);
    L.umma = L.tc && c->sage_kernel == 2 && dm.d == kUD && dm.dv == kUD && block_size == kUBlk;
    return L;
}

// The three quantisers (psi_Q, gamma + psi_K, psi_V) into `scratch`.
uint8_t *sage_records(uint8_t *base, const SageLayout &L) {
    // bulk copies want 16-byte alignment; 1 KB keeps the records on the tiles' own boundary
    uint8_t *p = base + L.o_rec;
    return p + ((1024 - (reinterpret_cast<uintptr_t>(p) & 1023)) & 1023);
}

qk_status sage_quantize_dev(qk_ctx *c, const float *dq, const float *dk, const float *dv,
                            uint8_t *base, const AttnDims &dm, const SageLayout &L) {
    const size_t S = dm.Skv;
    uint8_t *rec = L.umma ? sage_records(base, L) : nullptr;
    const float inv_sqrt_d = 1.0f / sqrtf((float)dm.d);  // gpu_attention.rs:720
    sage_quant_q_kernel<<<(unsigned)qk::ceil_div(L.qrows, 8), 256, 0, c->stream>>>(
        dq, (int8_t *)(base + L.o_qc), (float *)(base + L.o_qs), (uint32_t)L.qrows, dm.d,
        (uint32_t)L.dpad, inv_sqrt_d);
    QK_CUDA(cudaGetLastError());
    dim3 kgrid((unsigned)L.n_blocks, (unsigned)L.planes);
    sage_quant_k_kernel<<<kgrid, 128, dm.d * sizeof(float), c->stream>>>(
        dk, (int8_t *)(base + L.o_kc), (float *)(base + L.o_ks), (float *)(base + L.o_km), (uint32_t)S,
        dm.d, (uint32_t)L.dpad, (uint32_t)L.block, (uint32_t)L.n_blocks,
        L.tc ? (int8_t *)(base + L.o_md) : nullptr, (float *)(base + L.o_ms), rec);
    QK_CUDA(cudaGetLastError());
    sage_quant_v_kernel<<<kgrid, 128, 0, c->stream>>>(
        dv, (int8_t *)(base + L.o_vc), (float *)(base + L.o_vs), (uint32_t)S, dm.dv,
        (uint32_t)L.block, (uint32_t)L.bpad, (uint32_t)L.n_blocks, L.tc && !L.umma ? 1 : 0, rec);
    QK_CUDA(cudaGetLastError());
    c->launches += 3;
    return QK_OK;
}

qk_status attention_sage_dev(qk_ctx *c, const float *dq, const float *dk, const float *dv,
                             float *out, uint8_t *scratch, const qk_attention_shape *shape,
                             int causal, size_t block_size) {
    const AttnDims dm = dims_of(shape);
    const SageLayout L = sage_layout(c, dm, block_size);
    uint8_t *base = scratch;
    qk_status st = sage_quantize_dev(c, dq, dk, dv, base, dm, L);
    if (st != QK_OK) return st;
    SageArgs a{(const int8_t *)(base + L.o_qc), (const float *)(base + L.o_qs),
               (const int8_t *)(base + L.o_kc), (const float *)(base + L.o_ks),
               (const float *)(base + L.o_km),  (const int8_t *)(base + L.o_md),
               (const float *)(base + L.o_ms),  (const int8_t *)(base + L.o_vc),
               (const float *)(base + L.o_vs),  out,
               (uint32_t)L.dpad, (uint32_t)L.bpad, (uint32_t)L.block, (uint32_t)L.n_blocks,
               L.umma ? sage_records(base, L) : nullptr};
    if (L.umma) {
        if ((st = qk::error_word(c)) != QK_OK) return st;
        c->err_armed = true;
        QK_CUDA(cudaFuncSetAttribute(attention_sage_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)(kUSmemBytes + 1024)));
        dim3 grid((unsigned)qk::ceil_div(dm.Sq, kUQ), dm.H, dm.B);
        attention_sage_umma_kernel<<<grid, kUThreads, kUSmemBytes + 1024, c->stream>>>(a, dm, causal, c->wait_limit,
                                                                                 (int *)c->d_err.ptr);
        QK_CUDA(cudaGetLastError());
        c->launches++;
        return QK_OK;
    }
    if (L.tc)
        return dm.d == 64 ? launch_sage_tc_block<2>(c, a, dm, causal) : launch_sage_tc_block<4>(c, a, dm, causal);
    if (L.wpl == 1) return launch_sage<1>(c, a, dm, causal);
    if (L.wpl == 4) return launch_sage<4>(c, a, dm, causal);
    if (L.wpl == 8) return launch_sage<8>(c, a, dm, causal);
    return launch_sage<16>(c, a, dm, causal);
}

// The block-scale variant on device buffers: its three preparation kernels and the main kernel.
// scratch: sage_block_scratch_bytes of it.
size_t sage_block_scratch_bytes(const qk_attention_shape *s) {
    const AttnDims dm = dims_of(s);
    const size_t n_blocks = qk::ceil_div((size_t)dm.Skv, (size_t)kUBlk), planes = (size_t)dm.B * dm.KV;
    const size_t qrows = (size_t)dm.B * dm.H * dm.Sq;
    auto up = [](size_t n) { return (n + 255) / 256 * 256; };
    return up(qrows * 128) + up(qrows * 4) + up(planes * n_blocks * 128 * 4) +
           up(planes * ((n_blocks + 1) / 2) * kBRecStride) + 1024;
}
qk_status attention_sage_block_dev(qk_ctx *c, const float *dq, const float *dk, const float *dv, float *out,
                                   uint8_t *scratch, const qk_attention_shape *shape, int causal) {
    const AttnDims dm = dims_of(shape);
    if (dm.d != (uint32_t)kUD || dm.dv != (uint32_t)kUD || dm.Sq != dm.Skv)
        return qk::fail(QK_ERR_VALUE, "the block-scale Sage variant is built for self-attention with head_dim = "
                        "val_dim = 128 (got head_dim %u, val_dim %u, seq_q %u, seq_kv %u)", dm.d, dm.dv, dm.Sq, dm.Skv);
    const size_t S = dm.Skv, n_blocks = qk::ceil_div(S, (size_t)kUBlk), planes = (size_t)dm.B * dm.KV;
    const size_t qrows = (size_t)dm.B * dm.H * dm.Sq;
    auto up = [](size_t n) { return (n + 255) / 256 * 256; };
    uint8_t *qc = scratch, *qs = qc + up(qrows * 128), *km = qs + up(qrows * 4);
    uint8_t *rec = km + up(planes * n_blocks * 128 * 4);
    rec += (1024 - (reinterpret_cast<uintptr_t>(rec) & 1023)) & 1023;
    qk_status st = qk::error_word(c);
    if (st != QK_OK) return st;
    const float inv_sqrt_d = 1.0f / sqrtf((float)dm.d);
    sage_quant_q_block_kernel<<<dim3((unsigned)qk::ceil_div((size_t)dm.Sq, (size_t)64), dm.B * dm.H), 256, 0, c->stream>>>(
        dq, (int8_t *)qc, (float *)qs, dm.Sq, inv_sqrt_d);
    QK_CUDA(cudaGetLastError());
    dim3 kgrid((unsigned)n_blocks, (unsigned)planes);
    sage_quant_k_kernel<<<kgrid, 128, dm.d * sizeof(float), c->stream>>>(
        dk, nullptr, nullptr, (float *)km, (uint32_t)S, dm.d, 128u, (uint32_t)kUBlk, (uint32_t)n_blocks, nullptr, nullptr,
        rec, kBRecStride, kBRecScaleOff, (uint32_t)kUKeys, 1);
    QK_CUDA(cudaGetLastError());
    sage_v_bf16_record_kernel<<<kgrid, 128, 0, c->stream>>>(dv, rec, (uint32_t)S, (uint32_t)n_blocks);
    QK_CUDA(cudaGetLastError());
    SageArgs a{};
    a.qc = (const int8_t *)qc;
    a.qs = (const float *)qs;
    a.out = out;
    a.dpad = 128, a.bpad = 64, a.block = kUBlk, a.n_blocks = (uint32_t)n_blocks;
    a.rec = rec;
    c->err_armed = true;
    QK_CUDA(cudaFuncSetAttribute(attention_sage_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)(kBSmemBytes + 1024)));
    dim3 grid((unsigned)qk::ceil_div((size_t)dm.Sq, (size_t)kUQ), dm.H, dm.B);
    attention_sage_block_kernel<<<grid, kUThreads, kBSmemBytes + 1024, c->stream>>>(a, dm, causal, c->wait_limit,
                                                                                  (int *)c->d_err.ptr);
    QK_CUDA(cudaGetLastError());
    c->launches += 4;
    return QK_OK;
}

// Device-buffer form of the exact face (also used by the decoder path).
qk_status attention_exact_dev(qk_ctx *c, const float *q, const float *k, const float *v,
                              float *out, const qk_attention_shape *s, int causal) {
    AttnDims dm = dims_of(s);
    size_t widest = s->head_dim > s->val_dim ? s->head_dim : s->val_dim;
    if (widest <= 16) return launch_exact<4>(c, q, k, v, out, dm, causal);
    if (widest <= 64) return launch_exact<16>(c, q, k, v, out, dm, causal);
    if (widest <= 128) return launch_exact<32>(c, q, k, v, out, dm, causal);
    return launch_exact<64>(c, q, k, v, out, dm, causal);
}

}  // namespace qk

extern "C" {

qk_status qk_gpu_attention(qk_ctx *ctx, const qk_attention_shape *shape, const float *query,
                           size_t q_len, const float *key, size_t k_len, const float *value,
                           size_t v_len, int32_t causal, float *out, size_t out_len) {
    qk_status st = validate_attention(shape, q_len, k_len, v_len, false, 0, out_len);
    if (st != QK_OK) return st;
    qk_ctx *c;
    if ((st = qk::resolve_ctx(ctx, &c)) != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    const size_t qb = q_len * 4, kb = k_len * 4, vb = v_len * 4, ob = out_len * 4;
    auto up = [](size_t n) { return (n + 255) / 256 * 256; };
    if ((st = c->d_in.reserve(up(qb) + up(kb) + up(vb))) != QK_OK) return st;
    if ((st = c->d_out.reserve(ob)) != QK_OK) return st;
    uint8_t *base = (uint8_t *)c->d_in.ptr;
    float *dq = (float *)base, *dk = (float *)(base + up(qb)), *dv = (float *)(base + up(qb) + up(kb));
    QK_CUDA(cudaMemcpyAsync(dq, query, qb, cudaMemcpyHostToDevice, c->stream));
    QK_CUDA(cudaMemcpyAsync(dk, key, kb, cudaMemcpyHostToDevice, c->stream));
    QK_CUDA(cudaMemcpyAsync(dv, value, vb, cudaMemcpyHostToDevice, c->stream));
    if ((st = qk::attention_exact_dev(c, dq, dk, dv, (float *)c->d_out.ptr, shape, causal != 0)) !=
        QK_OK)
        return st;
    QK_CUDA(cudaMemcpyAsync(out, c->d_out.ptr, ob, cudaMemcpyDeviceToHost, c->stream));
    QK_CUDA(cudaStreamSynchronize(c->stream));
    return QK_OK;
}

qk_status qk_gpu_attention_sage(qk_ctx *ctx, const qk_attention_shape *shape, const float *query,
                                size_t q_len, const float *key, size_t k_len, const float *value,
                                size_t v_len, int32_t causal, size_t block_size, float *out,
                                size_t out_len) {
    qk_status st = validate_attention(shape, q_len, k_len, v_len, true, block_size, out_len);
    if (st != QK_OK) return st;
    qk_ctx *c;
    if ((st = qk::resolve_ctx(ctx, &c)) != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    auto up = [](size_t n) { return (n + 255) / 256 * 256; };
    const size_t qb = q_len * 4, kb = k_len * 4, vb = v_len * 4, ob = out_len * 4;
    const size_t o_q = 0, o_k = up(qb), o_v = o_k + up(kb), o_scratch = o_v + up(vb);
    if ((st = c->d_in.reserve(o_scratch + qk::sage_scratch_bytes(shape, block_size))) != QK_OK) return st;
    if ((st = c->d_out.reserve(ob)) != QK_OK) return st;
    uint8_t *base = (uint8_t *)c->d_in.ptr;
    float *dq = (float *)(base + o_q), *dk = (float *)(base + o_k), *dv = (float *)(base + o_v);
    QK_CUDA(cudaMemcpyAsync(dq, query, qb, cudaMemcpyHostToDevice, c->stream));
    QK_CUDA(cudaMemcpyAsync(dk, key, kb, cudaMemcpyHostToDevice, c->stream));
    QK_CUDA(cudaMemcpyAsync(dv, value, vb, cudaMemcpyHostToDevice, c->stream));
    if ((st = qk::attention_sage_dev(c, dq, dk, dv, (float *)c->d_out.ptr, base + o_scratch, shape,
                                     causal != 0, block_size)) != QK_OK)
        return st;
    QK_CUDA(cudaMemcpyAsync(out, c->d_out.ptr, ob, cudaMemcpyDeviceToHost, c->stream));
    QK_CUDA(cudaStreamSynchronize(c->stream));
    return QK_OK;
}

qk_status qk_gpu_attention_dev(qk_ctx *ctx, const qk_attention_shape *shape, const float *q_dev,
                               const float *k_dev, const float *v_dev, int32_t causal,
                               float *out_dev) {
    if (!shape) return qk::fail(QK_ERR_VALUE, "attention shape is null");
    const size_t q_len = shape->batch * shape->n_heads * shape->seq_q * shape->head_dim;
    const size_t k_len = shape->batch * shape->n_kv_heads * shape->seq_kv * shape->head_dim;
    const size_t v_len = shape->batch * shape->n_kv_heads * shape->seq_kv * shape->val_dim;
    const size_t o_len = shape->batch * shape->n_heads * shape->seq_q * shape->val_dim;
    qk_status st = validate_attention(shape, q_len, k_len, v_len, false, 0, o_len);
    if (st != QK_OK) return st;
    qk_ctx *c;
    if ((st = qk::resolve_ctx(ctx, &c)) != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    return qk::attention_exact_dev(c, q_dev, k_dev, v_dev, out_dev, shape, causal != 0);
}

qk_status qk_gpu_attention_sage_dev(qk_ctx *ctx, const qk_attention_shape *shape,
                                    const float *q_dev, const float *k_dev, const float *v_dev,
                                    int32_t causal, size_t block_size, float *out_dev) {
    if (!shape) return qk::fail(QK_ERR_VALUE, "attention shape is null");
    const size_t q_len = shape->batch * shape->n_heads * shape->seq_q * shape->head_dim;
    const size_t k_len = shape->batch * shape->n_kv_heads * shape->seq_kv * shape->head_dim;
    const size_t v_len = shape->batch * shape->n_kv_heads * shape->seq_kv * shape->val_dim;
    const size_t o_len = shape->batch * shape->n_heads * shape->seq_q * shape->val_dim;
    qk_status st = validate_attention(shape, q_len, k_len, v_len, true, block_size, o_len);
    if (st != QK_OK) return st;
    qk_ctx *c;
    if ((st = qk::resolve_ctx(ctx, &c)) != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    if ((st = c->d_in.reserve(qk::sage_scratch_bytes(shape, block_size))) != QK_OK) return st;
    return qk::attention_sage_dev(c, q_dev, k_dev, v_dev, out_dev, (uint8_t *)c->d_in.ptr, shape,
                                  causal != 0, block_size);
}

qk_status qk_gpu_attention_sage_block_dev(qk_ctx *ctx, const qk_attention_shape *shape, const float *q_dev,
                                          const float *k_dev, const float *v_dev, int32_t causal, float *out_dev) {
    if (!shape) return qk::fail(QK_ERR_VALUE, "attention shape is null");
    const size_t q_len = shape->batch * shape->n_heads * shape->seq_q * shape->head_dim;
    const size_t k_len = shape->batch * shape->n_kv_heads * shape->seq_kv * shape->head_dim;
    const size_t v_len = shape->batch * shape->n_kv_heads * shape->seq_kv * shape->val_dim;
    const size_t o_len = shape->batch * shape->n_heads * shape->seq_q * shape->val_dim;
    qk_status st = validate_attention(shape, q_len, k_len, v_len, true, 64, o_len);
    if (st != QK_OK) return st;
    if (!q_dev || !k_dev || !v_dev || !out_dev) return qk::fail(QK_ERR_VALUE, "qk_gpu_attention_sage_block_dev: null buffer");
    qk_ctx *c;
    if ((st = qk::resolve_ctx(ctx, &c)) != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    if ((st = c->d_in.reserve(qk::sage_block_scratch_bytes(shape))) != QK_OK) return st;
    return qk::attention_sage_block_dev(c, q_dev, k_dev, v_dev, out_dev, (uint8_t *)c->d_in.ptr, shape, causal != 0);
}

qk_status qk_gpu_sage_quantize(qk_ctx *ctx, const qk_attention_shape *shape, const float *query,
                               size_t q_len, const float *key, size_t k_len, const float *value,
                               size_t v_len, size_t block_size, int8_t *q_codes, float *q_scale,
                               int8_t *k_codes, float *k_scale, float *k_mean, int8_t *v_codes,
                               float *v_scale) {
    if (!shape) return qk::fail(QK_ERR_VALUE, "attention shape is null");
    const size_t o_len = shape->batch * shape->n_heads * shape->seq_q * shape->val_dim;
    qk_status st = validate_attention(shape, q_len, k_len, v_len, true, block_size, o_len);
    if (st != QK_OK) return st;
    if (!q_codes || !q_scale || !k_codes || !k_scale || !k_mean || !v_codes || !v_scale)
        return qk::fail(QK_ERR_VALUE, "qk_gpu_sage_quantize: null output");
    qk_ctx *c;
    if ((st = qk::resolve_ctx(ctx, &c)) != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    auto up = [](size_t n) { return (n + 255) / 256 * 256; };
    const size_t qb = q_len * 4, kb = k_len * 4, vb = v_len * 4;
    const size_t o_k = up(qb), o_v = o_k + up(kb), o_scratch = o_v + up(vb);
    const size_t scratch_bytes = qk::sage_scratch_bytes(shape, block_size);
    if ((st = c->d_in.reserve(o_scratch + scratch_bytes)) != QK_OK) return st;
    uint8_t *base = (uint8_t *)c->d_in.ptr;
    float *dq = (float *)base, *dk = (float *)(base + o_k), *dv = (float *)(base + o_v);
    QK_CUDA(cudaMemcpyAsync(dq, query, qb, cudaMemcpyHostToDevice, c->stream));
    QK_CUDA(cudaMemcpyAsync(dk, key, kb, cudaMemcpyHostToDevice, c->stream));
    QK_CUDA(cudaMemcpyAsync(dv, value, vb, cudaMemcpyHostToDevice, c->stream));
    const AttnDims dm = dims_of(shape);
    const qk::SageLayout L = qk::sage_layout(c, dm, block_size);
    if ((st = qk::sage_quantize_dev(c, dq, dk, dv, base + o_scratch, dm, L)) != QK_OK) return st;
    std::vector<uint8_t> host(scratch_bytes);
    QK_CUDA(cudaMemcpyAsync(host.data(), base + o_scratch, scratch_bytes, cudaMemcpyDeviceToHost,
                            c->stream));
    QK_CUDA(cudaStreamSynchronize(c->stream));
    // un-pad and un-permute into the plain layouts of the reference's quantisers
    const size_t S = dm.Skv, d = dm.d, dv_ = dm.dv;
    const int8_t *qc = (const int8_t *)(host.data() + L.o_qc), *kc = (const int8_t *)(host.data() + L.o_kc);
    const int8_t *vc = (const int8_t *)(host.data() + L.o_vc);
    for (size_t r = 0; r < L.qrows; ++r) std::memcpy(q_codes + r * d, qc + r * L.dpad, d);
    std::memcpy(q_scale, host.data() + L.o_qs, L.qrows * 4);
    std::memcpy(k_mean, host.data() + L.o_km, L.planes * L.n_blocks * d * 4);
    if (L.umma) {
        // the tcgen05 kernel's records: undo the row swizzle
        const uint8_t *rec = host.data() + (qk::sage_records(base + o_scratch, L) - (base + o_scratch));
        const size_t n_rec = (L.n_blocks + 1) / 2;
        for (size_t p = 0; p < L.planes; ++p) {
            for (size_t j = 0; j < S; ++j) {
                const uint8_t *rc = rec + (p * n_rec + j / 128) * kURecStride;
                for (size_t ch = 0; ch < d; ++ch)
                    k_codes[(p * S + j) * d + ch] = (int8_t)rc[rec_tile_offset((uint32_t)(j % 128), (uint32_t)ch)];
                std::memcpy(k_scale + p * S + j, rc + kURecScaleOff + 4 * (j % 128), 4);
            }
            for (size_t jb = 0; jb < L.n_blocks; ++jb) {
                const uint8_t *rc = rec + (p * n_rec + jb / 2) * kURecStride;
                std::memcpy(v_scale + (p * L.n_blocks + jb) * dv_, rc + kURecScaleOff + 4 * (128 + 128 * (jb % 2)),
                            dv_ * 4);
                for (size_t ch = 0; ch < dv_; ++ch)
                    for (size_t kk = 0; kk < L.block && jb * L.block + kk < S; ++kk)
                        v_codes[(p * S + jb * L.block + kk) * dv_ + ch] =
                            (int8_t)rc[kURecKBytes + rec_tile_offset((uint32_t)ch, (uint32_t)(64 * (jb % 2) + kk))];
            }
        }
        return QK_OK;
    }
    for (size_t r = 0; r < L.planes * S; ++r) std::memcpy(k_codes + r * d, kc + r * L.dpad, d);
    std::memcpy(k_scale, host.data() + L.o_ks, L.planes * S * 4);
    std::memcpy(v_scale, host.data() + L.o_vs, L.planes * L.n_blocks * dv_ * 4);
    for (size_t p = 0; p < L.planes; ++p)
        for (size_t jb = 0; jb < L.n_blocks; ++jb)
            for (size_t ch = 0; ch < dv_; ++ch) {
                const int8_t *row = vc + ((p * L.n_blocks + jb) * dv_ + ch) * L.bpad;
                for (size_t kk = 0; kk < L.block && jb * L.block + kk < S; ++kk)
                    v_codes[(p * S + jb * L.block + kk) * dv_ + ch] =
                        row[L.tc && !L.umma ? sage_tc_key_slot((uint32_t)kk) : kk];
            }
    return QK_OK;
}

int32_t qk_set_sage_kernel(qk_ctx *ctx, int32_t which) {
    qk_ctx *c;
    if (qk::resolve_ctx(ctx, &c) != QK_OK) return -1;
    std::lock_guard<std::mutex> lock(c->mu);
    const int32_t before = c->sage_kernel;
    if (which >= 0 && which <= 2) c->sage_kernel = which;
    return before;
}

}  // extern "C"
