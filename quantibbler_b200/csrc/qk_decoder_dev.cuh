// Device code of the decoder-side kernels that is shared between the stand-alone kernels
// (qk_decoder.cu) and the whole-step decode kernel (qk_decode_step.cu): the same functions in
// both places, so that both produce the same bits.
#pragma once

#include <cstdint>

namespace {

__device__ __forceinline__ float round_bf16f(float v) {
    uint32_t u = __float_as_uint(v);
    if ((u & 0x7fffffffu) > 0x7f800000u) return __uint_as_float((u | 0x00400000u) & 0xffff0000u);
    u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;
    return __uint_as_float(u);
}
__device__ __forceinline__ float bf16_bits_to_float(uint16_t b) {
    return __uint_as_float((uint32_t)b << 16);
}
__device__ __forceinline__ uint16_t float_to_bf16_bits(float v) {
    return (uint16_t)(__float_as_uint(round_bf16f(v)) >> 16);
}

template <typename T> __device__ __forceinline__ float load_as_float(const T *p, size_t i);
template <> __device__ __forceinline__ float load_as_float<float>(const float *p, size_t i) {
    return p[i];
}
template <> __device__ __forceinline__ float load_as_float<uint16_t>(const uint16_t *p, size_t i) {
    return bf16_bits_to_float(p[i]);
}
template <typename T> __device__ __forceinline__ void store_from_float(T *p, size_t i, float v);
template <> __device__ __forceinline__ void store_from_float<float>(float *p, size_t i, float v) {
    p[i] = v;
}
template <> __device__ __forceinline__ void store_from_float<uint16_t>(uint16_t *p, size_t i,
                                                                       float v) {
    p[i] = float_to_bf16_bits(v);
}

__device__ __forceinline__ float block_sum(float v, float *red) {
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32, nw = blockDim.x / 32;
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < nw; ++w) total += red[w];
    __syncthreads();
    return total;
}

// RoPE of the pair (a, b) = (x[i], x[i + d/2]) (engine/mod.rs:1169-1184), with the roundings
// spelled out so that every caller gets the same bits.
__device__ __forceinline__ float rope_first(float a, float b, float c, float s) {
    return __fmaf_rn(a, c, -__fmul_rn(b, s));
}
__device__ __forceinline__ float rope_second(float a, float b, float c, float s) {
    return __fmaf_rn(b, c, __fmul_rn(a, s));
}

// A group of 128 threads with a barrier of its own: a whole block (bar_id 0, __syncthreads) or a
// quarter of a larger one (a named barrier).
struct SubBlock {
    uint32_t tid;     // 0..127 within the group
    uint32_t bar_id;  // 0: the block's barrier
    __device__ __forceinline__ void sync() const {
        if (bar_id == 0) __syncthreads();
        else asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
    }
};

__device__ __forceinline__ void mma_bf16_top(float (&c)[4], uint32_t a0, uint32_t a2, uint32_t b0,
                                             uint32_t b1) {
    // rows 8..15 of A are zero
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(0u), "r"(a2), "r"(0u), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_bf16_full(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// x = hi + mid + lo with each term a bfloat16 (to 2^-25 of x)
__device__ __forceinline__ void split3(float x, uint32_t &hi, uint32_t &mid, uint32_t &lo) {
    hi = float_to_bf16_bits(x);
    const float r1 = x - bf16_bits_to_float((uint16_t)hi);
    mid = float_to_bf16_bits(r1);
    lo = float_to_bf16_bits(r1 - bf16_bits_to_float((uint16_t)mid));
}

constexpr int kMmaDecWarps = 4;
constexpr int kMmaDecKPitch = 320, kMmaDecVPitch = 272;  // bytes per staged key row (256 + pad)
constexpr int kMmaDecBufBytes = 16 * (kMmaDecKPitch + kMmaDecVPitch);
// Shared memory of one group: every warp's private ring of staging buffers.  The cross-warp
// combine arrays of a warp ({o[8][128], m[8], l[8]}, 4160 bytes) lie at the start of that
// warp's own ring, which is idle by the time it writes them (its loop has ended, nothing of
// its is in flight).  The stand-alone kernels run a ring of three buffers (two 16-key steps
// in flight per warp: the kernel is bound by the bytes it keeps in flight, and two groups of
// 111 KB fit an SM); the whole-step kernel, whose shared memory is shared out otherwise,
// runs two.
constexpr int kMmaDecBufs = 3;
constexpr int dec_attn_smem_bytes(int bufs) { return kMmaDecWarps * bufs * kMmaDecBufBytes; }
constexpr int kMmaDecSmemBytes = dec_attn_smem_bytes(kMmaDecBufs);
static_assert((8 * 128 + 16) * 4 <= 2 * kMmaDecBufBytes, "a warp's combine arrays must fit its own buffers");
struct DecAttnSmem {
    uint8_t *stage;       // [warp][bufs][kMmaDecBufBytes]
    uint32_t warp_bytes;  // bufs * kMmaDecBufBytes
    __device__ __forceinline__ float *o(uint32_t warp) const {  // [8][128]
        return reinterpret_cast<float *>(stage + warp * warp_bytes);
    }
    __device__ __forceinline__ float *m(uint32_t warp) const { return o(warp) + 8 * 128; }  // [8]
    __device__ __forceinline__ float *l(uint32_t warp) const { return m(warp) + 8; }        // [8]
};
__device__ __forceinline__ DecAttnSmem carve_dec_attn(uint8_t *base, int bufs = kMmaDecBufs) {
    DecAttnSmem s;
    s.stage = base;
    s.warp_bytes = (uint32_t)(bufs * kMmaDecBufBytes);
    return s;
}
// The position a decode step appends (whole-step kernel only): the projections' k and v rows of
// this step, where they go in the cache, and the cos/sin row of the position.
struct FreshKey {
    const float *k, *v;        // [batch][n_kv][128] float32, unrotated
    uint16_t *cache_k, *cache_v;
    const float *cos_sin;      // [64][2] of this position
    int pos, seq;
    bool valid;                // position and sequence lie inside the cache
};


// `sb` is the group of 128 threads (four warps) that works on one (split, kv-head block,
// sequence); `sm` its shared memory; (split, ky, b) what the stand-alone kernel takes from its
// block index.  With kRope the rotation of q (and of the new key) happens here instead of in a
// kernel before: `fresh` describes the position being appended (see FreshKey).
// kPacked (at most four query heads per block): the legacy bf16 MMA issues at about half
// the rate of the INT8 one on this part and the 96 MMAs of a 16-key step, not the cache
// bytes, bound the kernel.  Only 4 of the MMA's 16 A rows were in use, so two of the three
// terms share one MMA: rows 0-3 carry the hi terms of heads 0-3, rows 4-7 their mid terms,
// and the lo terms ride in rows 8-11 of the same MMA for the scores (whose accumulator is
// a temporary) and in rows 0-3 of a second MMA for the outputs (whose accumulators stay in
// registers over the whole loop: two per tile, not four): 48 MMAs per step.  Lane groups g
// and g + 4 then hold the parts of a head's sums; one shuffle per value adds them.
template <bool kRope, int kBufs = kMmaDecBufs, bool kPacked = false>
__device__ __forceinline__ void decode_attention_mma_body(
    const SubBlock sb, const DecAttnSmem sm, const float *__restrict__ q,
    const uint16_t *__restrict__ cache_k, const uint16_t *__restrict__ cache_v, int kv_len_b,
    float *__restrict__ partial, uint32_t n_heads, uint32_t n_kv, uint32_t gq, uint32_t s_max,
    uint32_t chunk, uint32_t n_splits, uint32_t split, uint32_t ky, uint32_t b, const FreshKey fresh) {
    constexpr uint32_t d = 128;
    const uint32_t group = n_heads / n_kv, subs = (group + gq - 1) / gq;
    const uint32_t kvh = ky / subs, hsub = ky % subs;
    const uint32_t h0 = kvh * group + hsub * gq;
    const uint32_t rows = min(gq, group - hsub * gq);  // query heads of this block
    const int len = min(max(kv_len_b, 0), (int)s_max);  // never past the cache's rows
    const int j_begin = split * chunk, j_end = min(len, (int)((split + 1) * chunk));
    const uint32_t warp = sb.tid / 32, lane = sb.tid % 32, g = lane >> 2, t = lane & 3;
    const float scale = 1.0f / sqrtf((float)d);

    // A fragments of q: MMA m (0..7) contracts channels 32 (m/2) + 8 t + 4 (m%2) + {0,1 | 2,3}
    constexpr int kTerms = kPacked ? 2 : 3;
    uint32_t qa[kTerms][8][2];
    const uint32_t qrow = kPacked ? (g & 3u) : g;  // the query head this lane's A rows stand for
    const bool upper = kPacked && g >= 4;           // (packed) this lane's rows carry the mid terms
    {
        // (read through L2: inside the whole-step kernel another block wrote q moments ago)
        const float *qr = q + ((size_t)b * n_heads + h0 + min(qrow, rows - 1)) * d;
        float qv[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float4 lo4 = __ldcg(reinterpret_cast<const float4 *>(qr + 32 * i + 8 * t));
            const float4 hi4 = __ldcg(reinterpret_cast<const float4 *>(qr + 32 * i + 8 * t + 4));
            qv[i][0] = lo4.x, qv[i][1] = lo4.y, qv[i][2] = lo4.z, qv[i][3] = lo4.w;
            qv[i][4] = hi4.x, qv[i][5] = hi4.y, qv[i][6] = hi4.z, qv[i][7] = hi4.w;
        }
        if (kRope) {
            // channel c = 32 i + 8 t + e pairs with c +- 64, i.e. with block i ^ 2 of this lane
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                    const float4 cs = *reinterpret_cast<const float4 *>(fresh.cos_sin + 2 * (32 * i + 8 * t + e));
                    const float a0 = qv[i][e], b0 = qv[i + 2][e], a1 = qv[i][e + 1], b1 = qv[i + 2][e + 1];
                    qv[i][e] = rope_first(a0, b0, cs.x, cs.y);
                    qv[i + 2][e] = rope_second(a0, b0, cs.x, cs.y);
                    qv[i][e + 1] = rope_first(a1, b1, cs.z, cs.w);
                    qv[i + 2][e + 1] = rope_second(a1, b1, cs.z, cs.w);
                }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float (&v)[8] = qv[i];
#pragma unroll
            for (int half = 0; half < 2; ++half)
#pragma unroll
                for (int pr = 0; pr < 2; ++pr) {
                    uint32_t e0[3], e1[3];
                    const float x0 = qrow < rows ? v[4 * half + 2 * pr] * scale : 0.f;
                    const float x1 = qrow < rows ? v[4 * half + 2 * pr + 1] * scale : 0.f;
                    split3(x0, e0[0], e0[1], e0[2]);
                    split3(x1, e1[0], e1[1], e1[2]);
                    if (kPacked) {
                        qa[0][2 * i + half][pr] = upper ? (e0[1] | (e1[1] << 16)) : (e0[0] | (e1[0] << 16));
                        qa[1][2 * i + half][pr] = upper ? 0u : (e0[2] | (e1[2] << 16));
                    } else {
#pragma unroll
                        for (int term = 0; term < kTerms; ++term)
                            qa[term][2 * i + half][pr] = e0[term] | (e1[term] << 16);
                    }
                }
        }
    }
    float o[16][2];
#pragma unroll
    for (int nt = 0; nt < 16; ++nt) o[nt][0] = o[nt][1] = 0.f;
    float m = -INFINITY, l = 0.f;  // row g; l is this lane's share (its own key columns)

    const uint16_t *kb = cache_k + ((size_t)b * n_kv + kvh) * s_max * d;
    const uint16_t *vb = cache_v + ((size_t)b * n_kv + kvh) * s_max * d;
    // Each warp streams its 16-key steps through a private ring of kBufs shared-memory buffers
    // with cp.async, so the next kBufs - 1 steps' 8 KB of K and V each are in flight while this
    // one is multiplied.  Row pitches 320 B (K) and 272 B (V) keep the 16-byte fragment reads
    // conflict-free.
    uint8_t *my_smem = sm.stage + warp * sm.warp_bytes;
    auto fetch = [&](int j, int buf) {
        uint8_t *kt = my_smem + buf * kMmaDecBufBytes, *vt = kt + 16 * kMmaDecKPitch;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int idx = (int)lane + 32 * q, key = idx / 16, piece = idx % 16;
            const int src_key = min(j + key, j_end - 1);      // a valid address even when unused
            const uint32_t bytes = j + key < j_end ? 16u : 0u;  // 0: the 16 bytes are zero-filled
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(
                             (uint32_t)__cvta_generic_to_shared(kt + key * kMmaDecKPitch + piece * 16)),
                         "l"(kb + (size_t)src_key * d + piece * 8), "r"(bytes)
                         : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(
                             (uint32_t)__cvta_generic_to_shared(vt + key * kMmaDecVPitch + piece * 16)),
                         "l"(vb + (size_t)src_key * d + piece * 8), "r"(bytes)
                         : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (kRope && fresh.pos >= j_begin && fresh.pos < (int)((split + 1) * chunk)) {
        // this block's keys include the position being appended: rotate k, write k and v into
        // the cache (every block of the kv head that covers the position writes the same bits)
        if (fresh.valid) {
            const float *kt = fresh.k + ((size_t)b * n_kv + kvh) * d, *vt = fresh.v + ((size_t)b * n_kv + kvh) * d;
            const size_t row = (((size_t)fresh.seq * n_kv + kvh) * s_max + fresh.pos) * d;
            if (sb.tid < d / 2) {
                const uint32_t i = sb.tid;
                const float c = fresh.cos_sin[2 * i], s = fresh.cos_sin[2 * i + 1];
                const float a = __ldcg(kt + i), bb = __ldcg(kt + d / 2 + i);
                fresh.cache_k[row + i] = float_to_bf16_bits(rope_first(a, bb, c, s));
                fresh.cache_k[row + d / 2 + i] = float_to_bf16_bits(rope_second(a, bb, c, s));
            } else {
                const uint32_t i = sb.tid - d / 2;
                fresh.cache_v[row + i] = float_to_bf16_bits(__ldcg(vt + i));
                fresh.cache_v[row + d / 2 + i] = float_to_bf16_bits(__ldcg(vt + d / 2 + i));
            }
            __threadfence();
        }
        sb.sync();
    }
    int buf = 0;
    constexpr int kStride = 16 * kMmaDecWarps;  // keys between a warp's steps
    const int j_first = j_begin + 16 * (int)warp;
#pragma unroll
    for (int ahead = 0; ahead < kBufs - 1; ++ahead)
        if (j_first + ahead * kStride < j_end) fetch(j_first + ahead * kStride, ahead);
    for (int j = j_first; j < j_end; j += kStride, buf = buf + 1 == kBufs ? 0 : buf + 1) {
        // (groups still allowed in flight = the steps after this one that have been started)
        if (j + (kBufs - 1) * kStride < j_end) {
            fetch(j + (kBufs - 1) * kStride, (buf + kBufs - 1) % kBufs);
            asm volatile("cp.async.wait_group %0;" ::"n"(kBufs - 1) : "memory");
        } else if (kBufs > 2 && j + kStride < j_end) {
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncwarp();  // every lane's pieces of this step have landed
        const uint8_t *kt = my_smem + buf * kMmaDecBufBytes, *vt = kt + 16 * kMmaDecKPitch;
        // ---- S for 16 keys: two 8-key tiles
        float s[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            uint4 kw[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                kw[i] = *reinterpret_cast<const uint4 *>(kt + (8 * nt + g) * kMmaDecKPitch + 64 * i + 16 * t);
            s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i)
                if (kPacked) {
                    // (qa[1], the lo terms of lanes g < 4 and zero elsewhere, as rows g + 8)
                    mma_bf16_full(s[nt], qa[0][2 * i][0], qa[1][2 * i][0], qa[0][2 * i][1], qa[1][2 * i][1], kw[i].x,
                                  kw[i].y);
                    mma_bf16_full(s[nt], qa[0][2 * i + 1][0], qa[1][2 * i + 1][0], qa[0][2 * i + 1][1],
                                  qa[1][2 * i + 1][1], kw[i].z, kw[i].w);
                } else {
#pragma unroll
                    for (int term = 0; term < kTerms; ++term) {
                        mma_bf16_top(s[nt], qa[term][2 * i][0], qa[term][2 * i][1], kw[i].x, kw[i].y);
                        mma_bf16_top(s[nt], qa[term][2 * i + 1][0], qa[term][2 * i + 1][1], kw[i].z, kw[i].w);
                    }
                }
            if (kPacked) {  // hi sums (rows 0-3), lo sums (rows 8-11) and mid sums (rows 4-7) of the same head
                const float part0 = s[nt][0] + s[nt][2], part1 = s[nt][1] + s[nt][3];
                s[nt][0] = part0 + __shfl_xor_sync(0xffffffffu, part0, 16);
                s[nt][1] = part1 + __shfl_xor_sync(0xffffffffu, part1, 16);
            }
        }
        // ---- online softmax over the 16 keys (row g holds columns 2t, 2t+1 of each tile)
        float mx = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                if (j + 8 * nt + 2 * (int)t + e >= j_end) s[nt][e] = -INFINITY;
                mx = fmaxf(mx, s[nt][e]);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m, mx);  // finite: the step has at least one valid key
        const float alpha = expf(m - m_new);
        float p[2][2];
        float psum = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                p[nt][e] = expf(s[nt][e] - m_new);
                psum += p[nt][e];
            }
        l = l * alpha + psum;
        m = m_new;
        uint32_t pa[kTerms][2];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            uint32_t e0[3], e1[3];
            split3(p[nt][0], e0[0], e0[1], e0[2]);
            split3(p[nt][1], e1[0], e1[1], e1[2]);
            if (kPacked) {
                pa[0][nt] = upper ? (e0[1] | (e1[1] << 16)) : (e0[0] | (e1[0] << 16));
                pa[1][nt] = upper ? 0u : (e0[2] | (e1[2] << 16));
            } else {
#pragma unroll
                for (int term = 0; term < kTerms; ++term) pa[term][nt] = e0[term] | (e1[term] << 16);
            }
        }
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
            o[nt][0] *= alpha;
            o[nt][1] *= alpha;
        }
        // ---- O += P V: keys 2t, 2t+1 (first k half) and 8+2t, 8+2t+1 (second)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint4 vw[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int key = 8 * (r >> 1) + 2 * (int)t + (r & 1);  // within the step; rows past the end are zero
                vw[r] = *reinterpret_cast<const uint4 *>(vt + key * kMmaDecVPitch + 128 * h + 16 * g);
            }
#pragma unroll
            for (int jj = 0; jj < 8; ++jj) {
                const uint32_t w0 = jj / 2 == 0 ? vw[0].x : jj / 2 == 1 ? vw[0].y : jj / 2 == 2 ? vw[0].z : vw[0].w;
                const uint32_t w1 = jj / 2 == 0 ? vw[1].x : jj / 2 == 1 ? vw[1].y : jj / 2 == 2 ? vw[1].z : vw[1].w;
                const uint32_t w2 = jj / 2 == 0 ? vw[2].x : jj / 2 == 1 ? vw[2].y : jj / 2 == 2 ? vw[2].z : vw[2].w;
                const uint32_t w3 = jj / 2 == 0 ? vw[3].x : jj / 2 == 1 ? vw[3].y : jj / 2 == 2 ? vw[3].z : vw[3].w;
                const uint32_t sel = jj % 2 ? 0x7632u : 0x5410u;
                const uint32_t b0 = __byte_perm(w0, w1, sel), b1 = __byte_perm(w2, w3, sel);
                float acc[4] = {o[8 * h + jj][0], o[8 * h + jj][1], 0.f, 0.f};
#pragma unroll
                for (int term = 0; term < kTerms; ++term) mma_bf16_top(acc, pa[term][0], pa[term][1], b0, b1);
                o[8 * h + jj][0] = acc[0];
                o[8 * h + jj][1] = acc[1];
            }
        }
        __syncwarp();  // the buffer may be refilled by the next iteration's fetch
    }
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    if (kPacked) {  // a head's output: its hi + lo share (rows 0-3) plus its mid share (rows 4-7)
#pragma unroll
        for (int nt = 0; nt < 16; ++nt) {
            o[nt][0] += __shfl_xor_sync(0xffffffffu, o[nt][0], 16);
            o[nt][1] += __shfl_xor_sync(0xffffffffu, o[nt][1], 16);
        }
    }

    // ---- combine the warps of the block (each warp's arrays lie in its own, now idle, ring)
    if (t == 0 && !upper) {
        sm.m(warp)[g] = m;
        sm.l(warp)[g] = l;
    }
    if (!upper) {
        float *mine = sm.o(warp) + g * d;
#pragma unroll
        for (int nt = 0; nt < 16; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) mine[64 * (nt / 8) + 8 * (2 * t + e) + nt % 8] = o[nt][e];
    }
    sb.sync();
    for (uint32_t idx = sb.tid; idx < rows * d; idx += 128) {
        const uint32_t r = idx / d, c = idx % d;
        float mm = -INFINITY;
        for (int w = 0; w < kMmaDecWarps; ++w) mm = fmaxf(mm, sm.m(w)[r]);
        float ll = 0.f, oo = 0.f;
        for (int w = 0; w < kMmaDecWarps; ++w) {
            const float wt = sm.m(w)[r] == -INFINITY ? 0.f : expf(sm.m(w)[r] - mm);
            ll += sm.l(w)[r] * wt;
            oo += sm.o(w)[r * d + c] * wt;
        }
        float *out = partial + (((size_t)b * n_heads + h0 + r) * n_splits + split) * (d + 2);
        out[2 + c] = oo;
        if (c == 0) {
            out[0] = mm;
            out[1] = ll;
        }
    }
}

// out[c] = sum_s o_s[c] * exp(m_s - m) / sum_s l_s * exp(m_s - m) for one (sequence, head), by
// ONE warp: p = that head's n_splits <= 128 partials {m, l, o[d]}; the warp produces the
// channels c0 + lane + i * c_stride, i < kCh (those below d).  The loads of kBatch splits are
// issued together, the products are added in split order, so the result does not depend on
// kCh or kBatch.  No shared memory, no block barrier.
template <int kCh, int kBatch>
__device__ __forceinline__ void decode_combine_warp(uint32_t lane, const float *__restrict__ p,
                                                    float *__restrict__ out, uint32_t d, uint32_t n_splits,
                                                    uint32_t c0, uint32_t c_stride) {
    float ms[4], ls[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t s = lane + 32 * i;
        ms[i] = s < n_splits ? __ldcg(p + (size_t)s * (d + 2)) : -INFINITY;
        ls[i] = s < n_splits ? __ldcg(p + (size_t)s * (d + 2) + 1) : 0.f;
    }
    float mm = fmaxf(fmaxf(ms[0], ms[1]), fmaxf(ms[2], ms[3]));
    for (int off = 16; off > 0; off >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, off));
    float wv[4], ll = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        wv[i] = ms[i] == -INFINITY ? 0.f : expf(ms[i] - mm);
        float part = ls[i] * wv[i];
        for (int off = 16; off > 0; off >>= 1) part += __shfl_xor_sync(0xffffffffu, part, off);
        ll = i == 0 ? part : ll + part;
    }
    float oo[kCh];
#pragma unroll
    for (int i = 0; i < kCh; ++i) oo[i] = 0.f;
    for (uint32_t s0 = 0; s0 < n_splits; s0 += kBatch) {
        float x[kBatch][kCh];
#pragma unroll
        for (int e = 0; e < kBatch; ++e)
#pragma unroll
            for (int i = 0; i < kCh; ++i) {
                const uint32_t c = c0 + lane + i * c_stride;
                x[e][i] = (s0 + e < n_splits && c < d) ? __ldcg(p + (size_t)(s0 + e) * (d + 2) + 2 + c) : 0.f;
            }
#pragma unroll
        for (int e = 0; e < kBatch; ++e) {
            const uint32_t s = s0 + e;
            if (s < n_splits) {  // (the same for every lane)
                const uint32_t q = s / 32;
                const float mine = q == 0 ? wv[0] : q == 1 ? wv[1] : q == 2 ? wv[2] : wv[3];
                const float w = __shfl_sync(0xffffffffu, mine, s % 32);
#pragma unroll
                for (int i = 0; i < kCh; ++i) oo[i] += x[e][i] * w;
            }
        }
    }
#pragma unroll
    for (int i = 0; i < kCh; ++i) {
        const uint32_t c = c0 + lane + i * c_stride;
        if (c < d) out[c] = oo[i] / ll;
    }
}

}  // namespace
