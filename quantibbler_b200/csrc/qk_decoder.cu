// Decoder-side kernels around the factorized linear: what one transformer block needs
// besides its seven linears, on device buffers, launch-only (safe inside CUDA graph
// capture: no allocation, no synchronisation, no host copies).
//
// Semantics follow crates/quantibbler-server/src/engine/mod.rs:
//   RMSNorm        :1154-1160 (rms_norm_into) and :837-851 (norm_apply: bf16 serving rounds
//                  the operand and the result to bfloat16)
//   RoPE           :1169-1184 (rope_rotate: HF rotate_half, pairs (i, i + d/2), the angle
//                  pos * theta^(-2i/d) evaluated in float64 and cast to float32)
//   KV cache       :1189-1209 (append one row per position), kept head-major
//                  [B, KV, S_max, d] as the device contract of gpu_attention.rs wants
//   attention      :1074-1121 (gqa_attention_scalar: one query position against the cache)
//   SwiGLU         :931-935   g * u / (1 + exp(-g))
//   residual       :921-924, :937-940
//   embedding      :768-777, logits :788-800 (float32 accumulation over d_model),
//   greedy         crates/quantibbler-server/src/sampler.rs:5-16 (first maximum wins)
#include <cuda_bf16.h>

#include <cmath>

#include "qk_common.h"
#include "qk_digits.cuh"
#include "qk_decoder_dev.cuh"

namespace {


// Feeding the linears that consume a vector: the kernel that has the whole vector of a token
// in front of it (norm, SwiGLU, attention combine) also writes the digit tables its consumers'
// GEMV blocks multiply with - one table per consumer, because each has its own input scale s2
// (z = s2 * v in float32, rounded to bfloat16 under bfloat16 serving, exactly what the GEMV's
// own table build forms).  vals: the token's vector in shared memory.
struct FeedArgs {
    const FeedTarget *arr[4];   // arrays of targets, token-major: token t owns [t*per_token, (t+1)*per_token)
    uint32_t per_token[4];
    uint32_t n;
};
constexpr unsigned kFeedParts = 8;  // blocks that share the table building of one token
__device__ __forceinline__ void feed_consumers(const FeedArgs &feed, uint32_t token, const float *vals,
                                               bool bf16, uint32_t part = 0, uint32_t n_parts = 1) {
    __shared__ double feed_max[32];
    __shared__ long long feed_sum[32];
    __shared__ int feed_bad;
    for (uint32_t a = 0; a < feed.n; ++a)
        for (uint32_t i = 0; i < feed.per_token[a]; ++i) {
            const FeedTarget tg = feed.arr[a][(size_t)token * feed.per_token[a] + i];
            block_build_table(
                [&](uint32_t k) -> double {
                    if (k >= tg.n_bits) return 0.0;
                    float v = vals[k];
                    if (tg.in_scale) v = tg.in_scale[k] * v;
                    if (bf16) v = round_bf16f(v);
                    return (double)v;
                },
                tg.n_steps, reinterpret_cast<uint4 *>(tg.digits), tg.meta, feed_max, feed_sum, &feed_bad, part,
                n_parts);
        }
}

// h = x (+ residual); x_out = h; y = h * rsqrt(mean(h^2) + eps) * w.  One block per token.
// The row stays in registers between the two passes (up to kRmsPerThread elements per thread;
// wider rows re-read the overflow), so the kernel is one round of loads, one block-wide sum
// and one round of stores: at batch 1 its duration is pure latency.
constexpr int kRmsThreads = 512, kRmsPerThread = 16;
__global__ void __launch_bounds__(kRmsThreads)
rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ residual,
               const float *__restrict__ w, float *__restrict__ x_out, float *__restrict__ y,
               uint32_t d, float eps, int bf16, FeedArgs feed) {
    qk::pdl_launch();  // the next kernel may begin its prologue
    qk::pdl_wait();    // everything before this kernel on the stream is complete and visible
    extern __shared__ float norm_row[];  // the token's y (only when consumers are fed)
    __shared__ float red[kRmsThreads / 32];
    const size_t base = (size_t)blockIdx.x * d;
    // gridDim.y > 1: several blocks per token share the table building; each computes the whole
    // norm (x_out must then be another buffer than x), block 0 alone writes x_out and y
    const bool writer = blockIdx.y == 0;
    float keep[kRmsPerThread];
    float ss = 0.f;
#pragma unroll
    for (int r = 0; r < kRmsPerThread; ++r) {
        const uint32_t i = threadIdx.x + r * kRmsThreads;
        float h = 0.f;
        if (i < d) {
            h = x[base + i];
            if (residual) h += residual[base + i];
            if (x_out && writer) x_out[base + i] = h;
            if (bf16) h = round_bf16f(h);
        }
        keep[r] = h;
        ss += h * h;
    }
    for (uint32_t i = threadIdx.x + kRmsPerThread * kRmsThreads; i < d; i += kRmsThreads) {
        float h = x[base + i];
        if (residual) h += residual[base + i];
        if (x_out && writer) x_out[base + i] = h;
        if (bf16) h = round_bf16f(h);
        ss += h * h;
    }
    const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
#pragma unroll
    for (int r = 0; r < kRmsPerThread; ++r) {
        const uint32_t i = threadIdx.x + r * kRmsThreads;
        if (i < d) {
            float o = keep[r] * inv * w[i];
            if (bf16) o = round_bf16f(o);
            if (writer) y[base + i] = o;
            if (feed.n) norm_row[i] = o;
        }
    }
    for (uint32_t i = threadIdx.x + kRmsPerThread * kRmsThreads; i < d; i += kRmsThreads) {
        // in place (x_out == x, one block per token) x already holds h; otherwise x is untouched
        float h = x_out == x ? x[base + i] : x[base + i] + (residual ? residual[base + i] : 0.f);
        if (bf16) h = round_bf16f(h);
        float o = h * inv * w[i];
        if (bf16) o = round_bf16f(o);
        if (writer) y[base + i] = o;
        if (feed.n) norm_row[i] = o;
    }
    if (feed.n) {
        __syncthreads();
        feed_consumers(feed, blockIdx.x, norm_row, bf16 != 0, blockIdx.y, gridDim.y);
    }
}

// ---- RMSNorm fused with the tensor-parallel all-reduce of its residual input
// Row-parallel linears (o, down) leave one partial `delta` per rank.  Instead of an NCCL
// all-reduce followed by the norm, every rank PUSHES its partial into an inbox in each peer's
// memory (NVLink peer stores) and then adds what has arrived in its own inbox, in rank order -
// the same order on every rank, so all ranks get the same bits - while it forms h = x + sum
// and the norm.  Every 8-byte inbox word carries {value, number of this all-reduce}: a word
// is valid exactly when its tag is the current number, so there are no separate flags and no
// fences: value and tag travel in ONE 64-bit scalar store and are read back by ONE 64-bit
// scalar load (relaxed, system scope), which the PTX memory model makes single-copy atomic for
// an aligned 8-byte access - a vector access of two 32-bit halves would not be.  This is what
// makes a small all-reduce cheap: one posted store per element and peer, then local polling.
//   inbox.at[r] : rank r's inbox for this buffer, [source rank][n_tokens * d] words
//   counter     : this rank's count of all-reduces done (device memory, so that a replayed
//                 CUDA graph keeps counting); the last block to finish advances it.
// The caller alternates between two inboxes (attention block, MLP block): a peer can only
// write all-reduce s + 2 into the inbox being read here after this rank has sent its part of
// s + 1, i.e. after it is done reading s.  The polling is bounded (`poll_limit` rounds per
// peer): on expiry bit 1 of the error word is set, y is left unwritten, and the call is still
// counted (ticket and counter advance as usual), so this rank's tags stay in step with its own
// later calls; the peers' counts may then differ from it, which is why the caller has to
// re-zero inboxes and state on every rank before it uses the all-reduce again.
struct InboxArgs {
    unsigned long long *at[8];
};

__global__ void __launch_bounds__(kRmsThreads)
allreduce_rmsnorm_kernel(InboxArgs inbox, const float *__restrict__ partial,
                         uint32_t *__restrict__ counter, uint32_t *__restrict__ done, int rank,
                         int world, const float *__restrict__ x, const float *__restrict__ w,
                         float *__restrict__ x_out, float *__restrict__ y, uint32_t d, float eps,
                         int bf16, int *__restrict__ error, uint32_t poll_limit, FeedArgs feed) {
    qk::pdl_launch();  // the next kernel may begin its prologue
    qk::pdl_wait();    // everything before this kernel on the stream is complete and visible
    extern __shared__ float norm_row[];  // the token's y (only when consumers are fed)
    __shared__ float red[kRmsThreads / 32];
    __shared__ int gave_up;
    // gridDim.y > 1: several blocks per token share the table building; block 0 alone sends and
    // writes x_out and y, all of them receive (the inbox is local memory) and compute the norm
    const bool writer = blockIdx.y == 0;
    const uint32_t step = *counter + 1;
    if (threadIdx.x == 0) gave_up = 0;
    __syncthreads();
    const size_t base = (size_t)blockIdx.x * d, total = (size_t)gridDim.x * d;
    constexpr int kSlots = 8;  // elements per thread handled with peers (d <= 8 * 512 per pass)
    float keep[kRmsPerThread];
    float ss = 0.f;
    for (uint32_t pass = 0; pass * kSlots * kRmsThreads < d; ++pass) {
        float own[kSlots], xv[kSlots];
        // (the residual stream's elements are asked for now: they arrive while the peers' do)
#pragma unroll
        for (int sl = 0; sl < kSlots; ++sl)
            xv[sl] = x[base + min(threadIdx.x + (pass * kSlots + sl) * kRmsThreads, d - 1)];
        // ---- send: my partial, tagged, into every peer's inbox
#pragma unroll
        for (int sl = 0; sl < kSlots; ++sl) {
            const uint32_t i = threadIdx.x + (pass * kSlots + sl) * kRmsThreads;
            own[sl] = i < d ? partial[base + i] : 0.f;
            if (i < d && writer) {
                const unsigned long long word =
                    (unsigned long long)__float_as_uint(own[sl]) | ((unsigned long long)step << 32);
#pragma unroll
                for (int p = 0; p < 8; ++p)
                    if (p < world && p != rank)
                        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(
                                         inbox.at[p] + (size_t)rank * total + base + i),
                                     "l"(word)
                                     : "memory");
            }
        }
        // ---- receive and add in rank order: for each peer, poll my inbox until the thread's
        // words of this pass all carry the tag (by the time the first peer's have arrived the
        // others' usually have too)
        float sum[kSlots];
#pragma unroll
        for (int sl = 0; sl < kSlots; ++sl) sum[sl] = 0.f;
        for (int r = 0; r < world; ++r) {
            if (r == rank) {
#pragma unroll
                for (int sl = 0; sl < kSlots; ++sl) sum[sl] += own[sl];
                continue;
            }
            const unsigned long long *src = inbox.at[rank] + (size_t)r * total + base;
            float got[kSlots];
            bool ready = false;
            for (uint32_t tries = 0; tries < poll_limit && !ready; ++tries) {
                ready = true;
#pragma unroll
                for (int sl = 0; sl < kSlots; ++sl) {
                    const uint32_t i = threadIdx.x + (pass * kSlots + sl) * kRmsThreads;
                    unsigned long long word = (unsigned long long)step << 32;
                    if (i < d)
                        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];"
                                     : "=l"(word)
                                     : "l"(src + i)
                                     : "memory");
                    got[sl] = __uint_as_float((uint32_t)word);
                    if ((uint32_t)(word >> 32) != step) ready = false;
                }
            }
            if (!ready) gave_up = 1;
#pragma unroll
            for (int sl = 0; sl < kSlots; ++sl) sum[sl] += got[sl];
        }
        // ---- residual add
#pragma unroll
        for (int sl = 0; sl < kSlots; ++sl) {
            const uint32_t i = threadIdx.x + (pass * kSlots + sl) * kRmsThreads;
            if (i < d) {
                float h = xv[sl] + sum[sl];
                if (writer) x_out[base + i] = h;
                if (bf16) h = round_bf16f(h);
                if (pass * kSlots + sl < (uint32_t)kRmsPerThread) keep[pass * kSlots + sl] = h;
                ss += h * h;
            }
        }
    }
    __syncthreads();
    const bool dead = gave_up != 0;  // the same in every thread of the block
    if (dead && threadIdx.x == 0) atomicOr(error, 2);
    if (!dead) {
        const float inv = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
        // (eight of a thread's sixteen elements at a time, the weight's loads issued together:
        // one memory latency per eight instead of one per element)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            if ((uint32_t)half * (kRmsPerThread / 2) * kRmsThreads >= d) break;
            float wv[kRmsPerThread / 2];
#pragma unroll
            for (int r = 0; r < kRmsPerThread / 2; ++r)
                wv[r] = w[min(threadIdx.x + (half * (kRmsPerThread / 2) + r) * kRmsThreads, d - 1)];
#pragma unroll
            for (int r = 0; r < kRmsPerThread / 2; ++r) {
                const uint32_t i = threadIdx.x + (half * (kRmsPerThread / 2) + r) * kRmsThreads;
                if (i < d) {
                    float o = keep[half * (kRmsPerThread / 2) + r] * inv * wv[r];
                    if (bf16) o = round_bf16f(o);
                    if (writer) y[base + i] = o;
                    if (feed.n) norm_row[i] = o;
                }
            }
        }
        for (uint32_t i = threadIdx.x + kRmsPerThread * kRmsThreads; i < d; i += kRmsThreads) {
            float h = x_out[base + i];   // (rows wider than the register cache: one block per token only)
            if (bf16) h = round_bf16f(h);
            float o = h * inv * w[i];
            if (bf16) o = round_bf16f(o);
            if (writer) y[base + i] = o;
            if (feed.n) norm_row[i] = o;
        }
        if (feed.n) {
            __syncthreads();
            feed_consumers(feed, blockIdx.x, norm_row, bf16 != 0, blockIdx.y, gridDim.y);
        }
    }
    // the last block to finish records that this all-reduce is done (every block has read the
    // counter by then); a single block needs no ticket
    if (gridDim.x * gridDim.y == 1) {
        if (threadIdx.x == 0) *counter = step;
    } else {
        __syncthreads();
        if (threadIdx.x == 0) {
            __threadfence();
            if (atomicAdd(done, 1u) == gridDim.x * gridDim.y - 1) {
                *done = 0;
                *counter = step;
            }
        }
    }
}

// Rotates q in place and writes rotated k and v into the cache row of (seq, pos).
// cos_sin: [max_pos][d/2][2] float32.  One block per token; threads cover (head, i).
template <typename KV>
__global__ void __launch_bounds__(256)
rope_cache_kernel(float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                  const float *__restrict__ cos_sin, const int32_t *__restrict__ positions,
                  const int32_t *__restrict__ seq_index, KV *__restrict__ cache_k,
                  KV *__restrict__ cache_v, uint32_t n_heads, uint32_t n_kv, uint32_t d,
                  uint32_t s_max, uint32_t n_seq, int *__restrict__ error) {
    qk::pdl_launch();  // the next kernel may begin its prologue
    qk::pdl_wait();    // everything before this kernel on the stream is complete and visible
    const uint32_t tok = blockIdx.x, half = d / 2;
    const int pos = positions[tok], seq = seq_index[tok];
    // The cache and the cos/sin table hold s_max positions and n_seq sequences.  A token
    // outside them (a graph replayed past the end of the cache) is skipped and reported
    // through the context's error word (bit 2) instead of writing over a neighbour's rows.
    if (pos < 0 || (uint32_t)pos >= s_max || seq < 0 || (uint32_t)seq >= n_seq) {
        if (threadIdx.x == 0 && error) atomicOr(error, 4);
        return;
    }
    const float *cs = cos_sin + (size_t)pos * half * 2;
    float *qt = q + (size_t)tok * n_heads * d;
    for (uint32_t idx = threadIdx.x; idx < n_heads * half; idx += blockDim.x) {
        uint32_t h = idx / half, i = idx % half;
        float c = cs[2 * i], s = cs[2 * i + 1];
        float a = qt[h * d + i], b = qt[h * d + half + i];
        qt[h * d + i] = rope_first(a, b, c, s);
        qt[h * d + half + i] = rope_second(a, b, c, s);
    }
    const float *kt = k + (size_t)tok * n_kv * d, *vt = v + (size_t)tok * n_kv * d;
    for (uint32_t idx = threadIdx.x; idx < n_kv * half; idx += blockDim.x) {
        uint32_t h = idx / half, i = idx % half;
        float c = cs[2 * i], s = cs[2 * i + 1];
        float a = kt[h * d + i], b = kt[h * d + half + i];
        size_t row = (((size_t)seq * n_kv + h) * s_max + pos) * d;
        store_from_float<KV>(cache_k, row + i, rope_first(a, b, c, s));
        store_from_float<KV>(cache_k, row + half + i, rope_second(a, b, c, s));
        store_from_float<KV>(cache_v, row + i, vt[h * d + i]);
        store_from_float<KV>(cache_v, row + half + i, vt[h * d + half + i]);
    }
}

// A lane's DPL consecutive channels of one cache row.  When the slice is a whole number of
// 16-byte pieces (head_dim 128: two pieces in bfloat16, four in float32) it is fetched with
// 16-byte loads into `raw` and unpacked later, so that the next key's slice can be in
// flight while this one is used; the cache rows are 16-byte aligned because
// head_dim * sizeof(KV) is.  Otherwise element by element.
template <typename KV, int DPL>
struct RowSlice {
    static constexpr int kPer = 16 / sizeof(KV);  // elements per 16-byte piece
    static constexpr bool kVec = DPL % kPer == 0;
    static constexpr int kPieces = kVec ? DPL / kPer : 1;
    uint4 raw[kPieces];
    float scalar[kVec ? 1 : DPL];

    __device__ __forceinline__ void load(const KV *__restrict__ row, uint32_t sub, uint32_t d, bool vec) {
        if (kVec && vec) {
            const uint4 *src = reinterpret_cast<const uint4 *>(row + sub * DPL);
#pragma unroll
            for (int piece = 0; piece < kPieces; ++piece) raw[piece] = src[piece];
        } else if (!kVec) {
#pragma unroll
            for (int e = 0; e < DPL; ++e) {
                const uint32_t c = sub * DPL + e;
                scalar[e] = c < d ? load_as_float<KV>(row, c) : 0.f;
            }
        }
    }
    __device__ __forceinline__ void unpack(const KV *__restrict__ row, uint32_t sub, uint32_t d, bool vec,
                                           float (&out)[DPL]) const {
        if (kVec && vec) {
#pragma unroll
            for (int piece = 0; piece < kPieces; ++piece) {
                const uint32_t words[4] = {raw[piece].x, raw[piece].y, raw[piece].z, raw[piece].w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (sizeof(KV) == 2) {
                        out[piece * 8 + 2 * i] = __uint_as_float(words[i] << 16);
                        out[piece * 8 + 2 * i + 1] = __uint_as_float(words[i] & 0xffff0000u);
                    } else {
                        out[piece * 4 + i] = __uint_as_float(words[i]);
                    }
                }
            }
        } else if (kVec) {  // vector-capable type, but this head_dim is not 8 * DPL
#pragma unroll
            for (int e = 0; e < DPL; ++e) {
                const uint32_t c = sub * DPL + e;
                out[e] = c < d ? load_as_float<KV>(row, c) : 0.f;
            }
        } else {
#pragma unroll
            for (int e = 0; e < DPL; ++e) out[e] = scalar[e];
        }
    }
};

// Split-KV decode attention: one query position per sequence against the cache.
// grid (split, kv head, sequence); a block of 128 threads covers the keys
// [split*chunk, min(len, (split+1)*chunk)) for all G = H/KV query heads of the kv head, so
// each K/V row is read once per group.  Eight lanes share a key (d/8 channels each).
// partial[(b, h, split)] = {m, l, o[d]}.
constexpr int kDecThreads = 128;

template <typename KV, int DPL, int GQ>  // DPL = channels per lane (8 lanes per key), GQ = query heads per block
__global__ void __launch_bounds__(kDecThreads)
decode_attention_kernel(const float *__restrict__ q, const KV *__restrict__ cache_k,
                        const KV *__restrict__ cache_v, const int32_t *__restrict__ kv_len,
                        float *__restrict__ partial, uint32_t n_heads, uint32_t n_kv, uint32_t d,
                        uint32_t s_max, uint32_t chunk, uint32_t n_splits) {
    qk::pdl_launch();  // the next kernel may begin its prologue
    qk::pdl_wait();    // everything before this kernel on the stream is complete and visible
    const uint32_t group = n_heads / n_kv, subs = group / GQ;  // blocks per kv head
    const uint32_t split = blockIdx.x, kvh = blockIdx.y / subs, hsub = blockIdx.y % subs;
    const uint32_t b = blockIdx.z, h0 = kvh * group + hsub * GQ;
    const int len = min(max(kv_len[b], 0), (int)s_max);  // never past the cache's rows
    const int j_begin = split * chunk, j_end = min(len, (int)((split + 1) * chunk));
    const uint32_t tid = threadIdx.x, sub = tid % 8, slot = tid / 8;  // 16 key slots per block
    const unsigned gmask = 0xffu << ((tid % 32) / 8 * 8);  // the eight lanes sharing a key
    const float scale = 1.0f / sqrtf((float)d);

    float qr[GQ][DPL], m[GQ], l[GQ], o[GQ][DPL];
#pragma unroll
    for (int gq = 0; gq < GQ; ++gq) {
        m[gq] = -INFINITY;
        l[gq] = 0.f;
#pragma unroll
        for (int e = 0; e < DPL; ++e) {
            uint32_t c = sub * DPL + e;
            qr[gq][e] = c < d ? q[((size_t)b * n_heads + h0 + gq) * d + c] : 0.f;
            o[gq][e] = 0.f;
        }
    }
    const KV *kb = cache_k + ((size_t)b * n_kv + kvh) * s_max * d;
    const KV *vb = cache_v + ((size_t)b * n_kv + kvh) * s_max * d;
    const bool vec = d == 8u * DPL;
    RowSlice<KV, DPL> k_next, v_next;
    if (j_begin + (int)slot < j_end) {
        k_next.load(kb + (size_t)(j_begin + slot) * d, sub, d, vec);
        v_next.load(vb + (size_t)(j_begin + slot) * d, sub, d, vec);
    }
    for (int j = j_begin + slot; j < j_end; j += kDecThreads / 8) {
        float kk[DPL], vv[DPL];
        k_next.unpack(kb + (size_t)j * d, sub, d, vec, kk);
        v_next.unpack(vb + (size_t)j * d, sub, d, vec, vv);
        const int jn = j + kDecThreads / 8;
        if (jn < j_end) {  // the next key's slice is in flight during this key's arithmetic
            k_next.load(kb + (size_t)jn * d, sub, d, vec);
            v_next.load(vb + (size_t)jn * d, sub, d, vec);
        }
#pragma unroll
        for (int gq = 0; gq < GQ; ++gq) {
            float dot = 0.f;
#pragma unroll
            for (int e = 0; e < DPL; ++e) dot = fmaf(qr[gq][e], kk[e], dot);
            dot += __shfl_xor_sync(gmask, dot, 1);
            dot += __shfl_xor_sync(gmask, dot, 2);
            dot += __shfl_xor_sync(gmask, dot, 4);
            const float s = dot * scale;
            const float m_new = fmaxf(m[gq], s);
            const float alpha = expf(m[gq] - m_new), p = expf(s - m_new);
            l[gq] = l[gq] * alpha + p;
#pragma unroll
            for (int e = 0; e < DPL; ++e) o[gq][e] = o[gq][e] * alpha + p * vv[e];
            m[gq] = m_new;
        }
    }
    // combine the 16 key slots of the block through shared memory
    __shared__ float sm_m[kDecThreads / 8][GQ], sm_l[kDecThreads / 8][GQ];
    extern __shared__ float sm_o[];  // [16 slots][GQ][d]
#pragma unroll
    for (int gq = 0; gq < GQ; ++gq) {
        if (sub == 0) {
            sm_m[slot][gq] = m[gq];
            sm_l[slot][gq] = l[gq];
        }
#pragma unroll
        for (int e = 0; e < DPL; ++e) {
            uint32_t c = sub * DPL + e;
            if (c < d) sm_o[((size_t)slot * GQ + gq) * d + c] = o[gq][e];
        }
    }
    __syncthreads();
    for (uint32_t idx = tid; idx < GQ * d; idx += kDecThreads) {
        uint32_t gq = idx / d, c = idx % d;
        float mm = -INFINITY;
        for (int s2 = 0; s2 < kDecThreads / 8; ++s2) mm = fmaxf(mm, sm_m[s2][gq]);
        float ll = 0.f, oo = 0.f;
        for (int s2 = 0; s2 < kDecThreads / 8; ++s2) {
            float w = mm == -INFINITY ? 0.f : expf(sm_m[s2][gq] - mm);
            ll += sm_l[s2][gq] * w;
            oo += sm_o[((size_t)s2 * GQ + gq) * d + c] * w;
        }
        float *out = partial + (((size_t)b * n_heads + h0 + gq) * n_splits + split) * (d + 2);
        out[2 + c] = oo;
        if (c == 0) {
            out[0] = mm;
            out[1] = ll;
        }
    }
}

// ------------------------------------------------------------------ decode attention, tensor cores
// The same split-KV decode attention for a bfloat16 cache and head_dim 128, with both
// products on the bf16 tensor cores (mma.sync m16n8k16), so that the kernel is bound by the
// cache reads instead of by per-key scalar arithmetic.  A warp takes 16 keys per step.
//   S = (q / sqrt(d)) K^T: the M side is the GQ <= 8 query heads of the kv head (rows 8..15 of
//       the MMA are zero), the keys are the N side.  q is float32: it is split into three
//       bfloat16 terms (hi + mid + lo reproduces it to 2^-25), one MMA per term.  The order of
//       the channels inside the contraction is free, so it is chosen such that the four
//       16-byte loads a thread makes from its key row feed eight MMAs directly.
//   O += P V: P (float32) is split into three bfloat16 terms the same way; the accumulator
//       fragment of S already has the A-operand layout.  The contraction runs over keys, which
//       are strided in memory: a thread loads the same eight channels of four key rows and
//       pairs them up with byte permutes; the channel an output column stands for is
//       64 h + 8 (column) + tile (tile = 0..7 within half h).
// Partials {m, l, o[128]} per (sequence, head, split) as in decode_attention_kernel, so the
// same combine kernel finishes.

__global__ void __launch_bounds__(kMmaDecWarps * 32)
decode_attention_mma_kernel(const float *__restrict__ q, const uint16_t *__restrict__ cache_k,
                            const uint16_t *__restrict__ cache_v, const int32_t *__restrict__ kv_len,
                            float *__restrict__ partial, uint32_t n_heads, uint32_t n_kv,
                            uint32_t gq, uint32_t s_max, uint32_t chunk, uint32_t n_splits) {
    qk::pdl_launch();  // the next kernel may begin its prologue
    qk::pdl_wait();    // everything before this kernel on the stream is complete and visible
    extern __shared__ __align__(16) uint8_t dec_smem[];
    if (gq <= 4)
        decode_attention_mma_body<false, kMmaDecBufs, true>(
            SubBlock{threadIdx.x, 0}, carve_dec_attn(dec_smem), q, cache_k, cache_v, kv_len[blockIdx.z], partial,
            n_heads, n_kv, gq, s_max, chunk, n_splits, blockIdx.x, blockIdx.y, blockIdx.z, FreshKey{});
    else
        decode_attention_mma_body<false, kMmaDecBufs, false>(
            SubBlock{threadIdx.x, 0}, carve_dec_attn(dec_smem), q, cache_k, cache_v, kv_len[blockIdx.z], partial,
            n_heads, n_kv, gq, s_max, chunk, n_splits, blockIdx.x, blockIdx.y, blockIdx.z, FreshKey{});
}


// RoPE + cache append + split-KV attention + combine in ONE launch (bfloat16 cache, head_dim 128):
// what rope_cache_kernel, decode_attention_mma_kernel and decode_combine_kernel do in three.
// The rotation of q happens in the fragment loader; the block whose keys include the position
// being appended rotates k and writes k, v into the cache before it streams its keys; the last
// split of a (sequence, kv-head block) to finish - found by a ticket, nobody waits - combines
// the splits, a warp per head.  Same device functions, same bits.  q is left unrotated.
// tickets: one zero-initialised counter per (sequence, kv-head block); the last block resets it.
__global__ void __launch_bounds__(kMmaDecWarps * 32)
decode_attention_rope_kernel(const float *__restrict__ q, const float *__restrict__ k,
                             const float *__restrict__ v, const float *__restrict__ cos_sin,
                             const int32_t *__restrict__ positions, const int32_t *__restrict__ seq_index,
                             uint16_t *__restrict__ cache_k, uint16_t *__restrict__ cache_v,
                             const int32_t *__restrict__ kv_len, float *__restrict__ partial,
                             uint32_t *__restrict__ tickets, float *__restrict__ out, uint32_t n_heads,
                             uint32_t n_kv, uint32_t gq, uint32_t s_max, uint32_t n_seq, uint32_t chunk,
                             uint32_t n_splits, int *__restrict__ error) {
    qk::pdl_launch();  // the next kernel may begin its prologue
    const uint32_t split = blockIdx.x, ky = blockIdx.y, b = blockIdx.z;
    {
        // What this block streams - its split of the cache rows and the rotation's table row -
        // was written by earlier steps, not by the kernel before this one (which makes q, k, v):
        // ask for it before waiting for that kernel, so that the first touch (cold in L2 and in
        // the TLB) overlaps its tail.
        const uint32_t grp = n_heads / n_kv, sub_n = (grp + gq - 1) / gq, kvh = ky / sub_n;
        const int len = min(kv_len[b], (int)s_max);
        const int jb = (int)(split * chunk), je = min(len, (int)((split + 1) * chunk));
        const uint16_t *kb = cache_k + (((size_t)b * n_kv + kvh) * s_max + jb) * 128;
        const uint16_t *vb = cache_v + (((size_t)b * n_kv + kvh) * s_max + jb) * 128;
        for (int line = threadIdx.x; line < 2 * (je - jb); line += blockDim.x) {  // (a row is two 128-byte lines)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(kb + (size_t)line * 64));
            asm volatile("prefetch.global.L2 [%0];" ::"l"(vb + (size_t)line * 64));
        }
        const int p_in = min(max(positions[b], 0), (int)s_max - 1);
        if (threadIdx.x < 4)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(cos_sin + (size_t)p_in * 128 + threadIdx.x * 32));
    }
    qk::pdl_wait();    // everything before this kernel on the stream is complete and visible
    extern __shared__ __align__(16) uint8_t dec_smem[];
    __shared__ int is_last;
    const int pos = positions[b], seq = seq_index[b];
    const bool valid = pos >= 0 && (uint32_t)pos < s_max && seq >= 0 && (uint32_t)seq < n_seq;
    if (!valid && threadIdx.x == 0 && error) atomicOr(error, 4);  // skipped and reported, as rope_cache_kernel does
    const int pos_in = min(max(pos, 0), (int)s_max - 1);
    const FreshKey fresh{k, v, cache_k, cache_v, cos_sin + (size_t)pos_in * 128, pos, seq, valid};
    const SubBlock sb{threadIdx.x, 0};
    if (gq <= 4)
        decode_attention_mma_body<true, kMmaDecBufs, true>(sb, carve_dec_attn(dec_smem), q, cache_k, cache_v, kv_len[b],
                                                           partial, n_heads, n_kv, gq, s_max, chunk, n_splits, split,
                                                           ky, b, fresh);
    else
        decode_attention_mma_body<true, kMmaDecBufs, false>(sb, carve_dec_attn(dec_smem), q, cache_k, cache_v, kv_len[b],
                                                            partial, n_heads, n_kv, gq, s_max, chunk, n_splits, split,
                                                            ky, b, fresh);
    __threadfence();
    __syncthreads();
    const uint32_t group = n_heads / n_kv, subs = (group + gq - 1) / gq;
    if (threadIdx.x == 0) {
        uint32_t *ticket = tickets + (size_t)b * n_kv * subs + ky;
        const uint32_t old = atomicAdd(ticket, 1u);
        is_last = old == n_splits - 1;
        if (is_last) *ticket = 0;
    }
    __syncthreads();
    if (is_last) {
        __threadfence();
        const uint32_t kvh = ky / subs, hsub = ky % subs, h0 = kvh * group + hsub * gq;
        const uint32_t rows = min(gq, group - hsub * gq);
        for (uint32_t r = threadIdx.x / 32; r < rows; r += kMmaDecWarps) {
            const size_t head = (size_t)b * n_heads + h0 + r;
            decode_combine_warp<4, 32>(threadIdx.x % 32, partial + head * n_splits * 130, out + head * 128, 128,
                                       n_splits, 0, 32);
        }
    }
}

// ------------------------------------------------------------------ prefill attention, tensor cores
// Causal attention of T new positions of ONE sequence against the cache (which already holds
// their own keys and values): the attention of a batched prompt prefill.  Same contract as the
// decode kernels - exact softmax(q k^T / sqrt(d)) v in float32 accuracy, engine/mod.rs:1074-1121
// applied at every position - with both products on the bf16 tensor cores (mma.sync m16n8k16):
// the cache is bfloat16, so K and V are exact operands; q and P are float32 and are split
// into three bfloat16 terms each (hi + mid + lo reproduces the value to 2^-25), one MMA per
// term, which keeps the 1e-5 gate against the float64 oracle.
//   q, out : float32, token-major [T][n_heads][128] (the decoder's activation layout)
//   cache  : bfloat16 [n_seq][n_kv][s_max][128]; the queries are positions p0 .. p0+T-1 of
//            sequence `seq`, query i sees keys 0 .. p0+i.
// A CTA of four warps owns 64 query rows that share one kv head: `hw` = min(group, 4) query
// heads times 4/hw blocks of 16 positions, one (head, position block) per warp, so that a K/V
// tile staged in shared memory serves the whole GQA group.  Q is split once into its three
// terms in shared memory; K/V tiles of 32 keys are double-buffered with cp.async; all
// fragments come from ldmatrix (row pitch 272 bytes: conflict-free).
constexpr int kPfKeys = 32, kPfPitch = 136;  // keys per tile; bf16 elements per staged row
constexpr int kPfQBytes = 3 * 64 * kPfPitch * 2, kPfTileBytes = kPfKeys * kPfPitch * 2;
constexpr int kPfSmem = kPfQBytes + 4 * kPfTileBytes;

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_full(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(128)
prefill_attention_mma_kernel(const float *__restrict__ q, const uint16_t *__restrict__ cache_k,
                             const uint16_t *__restrict__ cache_v, float *__restrict__ out,
                             uint32_t n_tokens, uint32_t p0, uint32_t seq, uint32_t n_heads, uint32_t n_kv,
                             uint32_t hw, uint32_t s_max) {
    qk::pdl_launch();
    qk::pdl_wait();
    constexpr uint32_t d = 128;
    extern __shared__ __align__(16) uint8_t pf_smem[];
    uint16_t *Qs = reinterpret_cast<uint16_t *>(pf_smem);                 // [3][64][pitch]
    uint8_t *tiles = pf_smem + kPfQBytes;                                 // [2 buffers][K, V][32][pitch]
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane >> 2, t = lane & 3;
    const uint32_t group = n_heads / n_kv, subs = group / hw;             // CTAs per kv head and position range
    const uint32_t kvh = blockIdx.y / subs, hsub = blockIdx.y % subs;
    const uint32_t pbs = 4 / hw;                                          // 16-position blocks per CTA
    const uint32_t head = kvh * group + hsub * hw + warp % hw;
    const uint32_t tok0 = (blockIdx.x * pbs + warp / hw) * 16;            // this warp's first token
    const uint32_t cta_tok_end = min(n_tokens, (blockIdx.x + 1) * pbs * 16);
    const uint32_t n_tiles = (p0 + cta_tok_end + kPfKeys - 1) / kPfKeys;  // keys 0 .. p0 + last token
    const float scale = 1.0f / sqrtf((float)d);

    const uint16_t *kb = cache_k + ((size_t)seq * n_kv + kvh) * s_max * d;
    const uint16_t *vb = cache_v + ((size_t)seq * n_kv + kvh) * s_max * d;
    auto fetch = [&](uint32_t jt, uint32_t buf) {
        uint8_t *kt = tiles + buf * 2 * kPfTileBytes, *vt = kt + kPfTileBytes;
        // 32 keys x 16 pieces of 16 bytes, for K and for V: 8 of each per thread
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t idx = threadIdx.x + 128 * i, key = idx / 16, piece = idx % 16;
            const uint32_t j = jt * kPfKeys + key;
            const uint32_t src_j = min(j, s_max - 1);              // a valid address even when unused
            const uint32_t bytes = j < p0 + cta_tok_end ? 16u : 0u;  // 0: zero-filled
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(
                             (uint32_t)__cvta_generic_to_shared(kt + (key * kPfPitch + piece * 8) * 2)),
                         "l"(kb + (size_t)src_j * d + piece * 8), "r"(bytes)
                         : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(
                             (uint32_t)__cvta_generic_to_shared(vt + (key * kPfPitch + piece * 8) * 2)),
                         "l"(vb + (size_t)src_j * d + piece * 8), "r"(bytes)
                         : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    fetch(0, 0);

    // ---- this warp's 16 query rows, scaled and split into three bfloat16 terms
    for (uint32_t idx = lane; idx < 16 * (d / 4); idx += 32) {
        const uint32_t r = idx / (d / 4), c4 = idx % (d / 4);
        const uint32_t tok = min(tok0 + r, n_tokens - 1);
        const float4 v = *reinterpret_cast<const float4 *>(q + ((size_t)tok * n_heads + head) * d + c4 * 4);
        const float x[4] = {v.x * scale, v.y * scale, v.z * scale, v.w * scale};
        uint32_t e[4][3];
#pragma unroll
        for (int i = 0; i < 4; ++i) split3(x[i], e[i][0], e[i][1], e[i][2]);
#pragma unroll
        for (int term = 0; term < 3; ++term) {
            uint2 packed = make_uint2(e[0][term] | (e[1][term] << 16), e[2][term] | (e[3][term] << 16));
            *reinterpret_cast<uint2 *>(Qs + ((size_t)term * 64 + warp * 16 + r) * kPfPitch + c4 * 4) = packed;
        }
    }
    __syncwarp();

    float o[16][4];
#pragma unroll
    for (int nd = 0; nd < 16; ++nd) o[nd][0] = o[nd][1] = o[nd][2] = o[nd][3] = 0.f;
    float m_row[2] = {-INFINITY, -INFINITY}, l_row[2] = {0.f, 0.f};
    const int pos_g = (int)(p0 + tok0 + g), pos_h = pos_g + 8;   // positions of rows g and g + 8
    const uint32_t warp_last = p0 + min(tok0 + 15, n_tokens - 1);  // last key any row of this warp sees
    const uint32_t q_addr0 = (uint32_t)__cvta_generic_to_shared(
        Qs + ((size_t)warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * kPfPitch + (lane >> 4) * 8);

    for (uint32_t jt = 0; jt < n_tiles; ++jt) {
        const uint32_t buf = jt & 1;
        if (jt + 1 < n_tiles) {
            fetch(jt + 1, buf ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();  // tile jt has landed for every thread
        const uint32_t j0 = jt * kPfKeys;
        if (tok0 < n_tokens && j0 <= warp_last) {  // warp-uniform: the tile holds keys this warp sees
            const uint32_t kt_addr = (uint32_t)__cvta_generic_to_shared(tiles + buf * 2 * kPfTileBytes);
            const uint32_t vt_addr = kt_addr + kPfTileBytes;
            // ---- S = q k^T for 32 keys: four 8-key tiles
            float sacc[4][4];
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                uint32_t kf[2][4];  // B fragments of key tiles (0,1) and (2,3) for this k-step
#pragma unroll
                for (int pair = 0; pair < 2; ++pair)
                    ldsm_x4(kf[pair], kt_addr + (((2 * pair + (lane >> 4)) * 8 + (lane & 7)) * kPfPitch +
                                                 ks * 16 + ((lane >> 3) & 1) * 8) * 2);
#pragma unroll
                for (int term = 0; term < 3; ++term) {
                    uint32_t a[4];
                    ldsm_x4(a, q_addr0 + (term * 64 * kPfPitch + ks * 16) * 2);
#pragma unroll
                    for (int nt = 0; nt < 4; ++nt)
                        mma_bf16_full(sacc[nt], a, kf[nt / 2][(nt % 2) * 2], kf[nt / 2][(nt % 2) * 2 + 1]);
                }
            }
            // ---- causal mask and online softmax (rows g and g + 8; columns 2t, 2t+1 of each tile)
            float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
            for (int nt = 0; nt < 4; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = (int)j0 + 8 * nt + 2 * (int)t + (e & 1);
                    const int pos = e < 2 ? pos_g : pos_h;
                    if (j > pos) sacc[nt][e] = -INFINITY;
                    mx[e >> 1] = fmaxf(mx[e >> 1], sacc[nt][e]);
                }
            float alpha[2];
#pragma unroll
            for (int r = 0; r < 2; ++r) {
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
                mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
                const float m_new = fmaxf(m_row[r], mx[r]);
                // a row that has seen no admissible key yet keeps m = -inf; exp(-inf - finite) = 0
                alpha[r] = m_new == -INFINITY ? 1.f : expf(m_row[r] - m_new);
                m_row[r] = m_new;
            }
            uint32_t pa[3][2][4];  // [term][16-key step][A fragment]
            float psum[2] = {0.f, 0.f};
#pragma unroll
            for (int nt = 0; nt < 4; ++nt) {
                float p[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float mr = m_row[e >> 1];
                    p[e] = mr == -INFINITY ? 0.f : expf(sacc[nt][e] - mr);
                    psum[e >> 1] += p[e];
                }
                uint32_t e0[3], e1[3], e2[3], e3[3];
                split3(p[0], e0[0], e0[1], e0[2]);
                split3(p[1], e1[0], e1[1], e1[2]);
                split3(p[2], e2[0], e2[1], e2[2]);
                split3(p[3], e3[0], e3[1], e3[2]);
#pragma unroll
                for (int term = 0; term < 3; ++term) {
                    pa[term][nt / 2][(nt % 2) * 2] = e0[term] | (e1[term] << 16);      // row g
                    pa[term][nt / 2][(nt % 2) * 2 + 1] = e2[term] | (e3[term] << 16);  // row g + 8
                }
            }
#pragma unroll
            for (int r = 0; r < 2; ++r) l_row[r] = l_row[r] * alpha[r] + psum[r];
#pragma unroll
            for (int nd = 0; nd < 16; ++nd) {
                o[nd][0] *= alpha[0];
                o[nd][1] *= alpha[0];
                o[nd][2] *= alpha[1];
                o[nd][3] *= alpha[1];
            }
            // ---- O += P V: two 16-key steps, sixteen 8-channel tiles
#pragma unroll
            for (int kk = 0; kk < 2; ++kk)
#pragma unroll
                for (int nd = 0; nd < 16; nd += 2) {
                    uint32_t vf[4];  // B fragments of channel tiles nd and nd + 1
                    ldsm_x4_trans(vf, vt_addr + ((kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * kPfPitch +
                                                 (nd + (lane >> 4)) * 8) * 2);
#pragma unroll
                    for (int term = 0; term < 3; ++term) {
                        mma_bf16_full(o[nd], pa[term][kk], vf[0], vf[1]);
                        mma_bf16_full(o[nd + 1], pa[term][kk], vf[2], vf[3]);
                    }
                }
        }
        __syncthreads();  // the buffer may be refilled by the next iteration's fetch
    }
    // ---- normalise and store (token-major)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 1);
        l_row[r] += __shfl_xor_sync(0xffffffffu, l_row[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const uint32_t tok = tok0 + g + 8 * r;
        if (tok >= n_tokens) continue;
        float *orow = out + ((size_t)tok * n_heads + head) * d;
        const float inv = 1.0f / l_row[r];
#pragma unroll
        for (int nd = 0; nd < 16; ++nd)
            *reinterpret_cast<float2 *>(orow + nd * 8 + 2 * t) =
                make_float2(o[nd][2 * r] * inv, o[nd][2 * r + 1] * inv);
    }
}

// The same attention for any head size and cache dtype: one warp per (token, head), the
// lanes share the channels, online softmax in float32.  The fallback of the tensor-core
// kernel above (small models, float32 caches); not meant to be fast.
template <typename KV>
__global__ void __launch_bounds__(128)
prefill_attention_simple_kernel(const float *__restrict__ q, const KV *__restrict__ cache_k,
                                const KV *__restrict__ cache_v, float *__restrict__ out,
                                uint32_t n_tokens, uint32_t p0, uint32_t seq, uint32_t n_heads,
                                uint32_t n_kv, uint32_t d, uint32_t s_max) {
    qk::pdl_launch();
    qk::pdl_wait();
    const uint32_t row = blockIdx.x * 4 + threadIdx.x / 32, lane = threadIdx.x % 32;
    if (row >= n_tokens * n_heads) return;
    const uint32_t tok = row / n_heads, head = row % n_heads, kvh = head / (n_heads / n_kv);
    const float *qr = q + (size_t)row * d;
    const KV *kb = cache_k + ((size_t)seq * n_kv + kvh) * s_max * d;
    const KV *vb = cache_v + ((size_t)seq * n_kv + kvh) * s_max * d;
    const float scale = 1.0f / sqrtf((float)d);
    float qv[8], o[8];  // channels lane, lane + 32, ... (head_dim <= 256)
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const uint32_t c = lane + 32 * e;
        qv[e] = c < d ? qr[c] : 0.f;
        o[e] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (uint32_t j = 0; j <= p0 + tok; ++j) {
        float dot = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const uint32_t c = lane + 32 * e;
            if (c < d) dot = fmaf(qv[e], load_as_float<KV>(kb, (size_t)j * d + c), dot);
        }
        for (int off = 16; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
        const float sc = dot * scale, m_new = fmaxf(m, sc);
        const float alpha = expf(m - m_new), pj = expf(sc - m_new);
        l = l * alpha + pj;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const uint32_t c = lane + 32 * e;
            if (c < d) o[e] = o[e] * alpha + pj * load_as_float<KV>(vb, (size_t)j * d + c);
        }
        m = m_new;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const uint32_t c = lane + 32 * e;
        if (c < d) out[(size_t)row * d + c] = o[e] / l;
    }
}

// out[b, h, :] = sum_s o_s * exp(m_s - m) / sum_s l_s * exp(m_s - m).  One block per (b, h).
__global__ void __launch_bounds__(128)
decode_combine_kernel(const float *__restrict__ partial, float *__restrict__ out, uint32_t d,
                      uint32_t n_splits) {
    qk::pdl_launch();  // the next kernel may begin its prologue
    qk::pdl_wait();    // everything before this kernel on the stream is complete and visible
    // warp w: channels 32 w + lane, + 128, ...
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    for (uint32_t c0 = 32 * warp; c0 < d; c0 += 128)
        decode_combine_warp<1, 16>(lane, partial + (size_t)blockIdx.x * n_splits * (d + 2),
                                   out + (size_t)blockIdx.x * d, d, n_splits, c0, 0);
}

__global__ void swiglu_kernel(const float *__restrict__ g, const float *__restrict__ u,
                              float *__restrict__ out, size_t n) {
    qk::pdl_launch();  // the next kernel may begin its prologue
    qk::pdl_wait();    // everything before this kernel on the stream is complete and visible
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) {
        float gv = g[i];
        out[i] = gv * u[i] / (1.0f + expf(-gv));
    }
}

// SwiGLU of one token's gate and up vectors, kept in shared memory, and the digit tables of
// the linears that consume it (the down projection): no activation vector goes to memory.
__global__ void __launch_bounds__(512)
swiglu_feed_kernel(const float *__restrict__ g, const float *__restrict__ u, uint32_t n, int bf16,
                   FeedArgs feed) {
    qk::pdl_launch();
    qk::pdl_wait();
    extern __shared__ float act_row[];
    const size_t base = (size_t)blockIdx.x * n;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float gv = g[base + i];
        act_row[i] = gv * u[base + i] / (1.0f + expf(-gv));
    }
    __syncthreads();
    feed_consumers(feed, blockIdx.x, act_row, bf16 != 0, blockIdx.y, gridDim.y);
}

// The combine of the split-KV decode attention for ALL heads of one sequence in one block
// (a warp per head at a time), followed by the digit tables of the linears that consume the
// attention output (the o projection).
__global__ void __launch_bounds__(512)
decode_combine_feed_kernel(const float *__restrict__ partial, float *__restrict__ out, uint32_t n_heads,
                           uint32_t d, uint32_t n_splits, int bf16, FeedArgs feed) {
    qk::pdl_launch();
    qk::pdl_wait();
    extern __shared__ float attn_row[];  // [n_heads * d]
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32, n_warps = blockDim.x / 32;
    for (uint32_t h = warp; h < n_heads; h += n_warps) {
        const float *p = partial + ((size_t)blockIdx.x * n_heads + h) * n_splits * (d + 2);
        float mm = -INFINITY;
        for (uint32_t s2 = lane; s2 < n_splits; s2 += 32) mm = fmaxf(mm, p[s2 * (d + 2)]);
        for (int off = 16; off > 0; off >>= 1) mm = fmaxf(mm, __shfl_xor_sync(0xffffffffu, mm, off));
        float ll = 0.f;
        for (uint32_t s2 = lane; s2 < n_splits; s2 += 32) {
            const float ms = p[s2 * (d + 2)];
            ll += p[s2 * (d + 2) + 1] * (ms == -INFINITY ? 0.f : expf(ms - mm));
        }
        for (int off = 16; off > 0; off >>= 1) ll += __shfl_xor_sync(0xffffffffu, ll, off);
        for (uint32_t c = lane; c < d; c += 32) {
            float oo = 0.f;
            for (uint32_t s2 = 0; s2 < n_splits; ++s2) {
                const float ms = p[s2 * (d + 2)];
                oo += p[s2 * (d + 2) + 2 + c] * (ms == -INFINITY ? 0.f : expf(ms - mm));
            }
            const float o = oo / ll;
            if (blockIdx.y == 0) out[((size_t)blockIdx.x * n_heads + h) * d + c] = o;
            attn_row[h * d + c] = o;
        }
    }
    __syncthreads();
    feed_consumers(feed, blockIdx.x, attn_row, bf16 != 0, blockIdx.y, gridDim.y);
}

__global__ void add_kernel(const float *__restrict__ a, const float *__restrict__ b,
                           float *__restrict__ out, size_t n) {
    qk::pdl_launch();  // the next kernel may begin its prologue
    qk::pdl_wait();    // everything before this kernel on the stream is complete and visible
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = a[i] + b[i];
}

template <typename W>
__global__ void embed_kernel(const W *__restrict__ table, const int32_t *__restrict__ ids,
                             float *__restrict__ out, uint32_t d, uint32_t vocab) {
    qk::pdl_launch();  // the next kernel may begin its prologue
    qk::pdl_wait();    // everything before this kernel on the stream is complete and visible
    const int id = ids[blockIdx.x];
    for (uint32_t i = threadIdx.x; i < d; i += blockDim.x)
        out[(size_t)blockIdx.x * d + i] =
            (id >= 0 && (uint32_t)id < vocab) ? load_as_float<W>(table, (size_t)id * d + i) : 0.f;
}

// logits[t][v] = sum_i hidden[t][i] * W[v][i], float32 accumulation.  One warp per vocab row,
// 16-byte loads of the row (8 bfloat16 or 4 float32 per lane); the row is streamed once per
// tile of TT tokens (it stays in L2 between tiles).  HBM-bound: the head is vocab*d values.
template <typename W> struct HeadVec;
template <> struct HeadVec<uint16_t> {
    static constexpr int kN = 8;
    __device__ static void load(const uint16_t *p, float (&w)[8]) {
        const uint4 v = *reinterpret_cast<const uint4 *>(p);
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            w[2 * i] = __uint_as_float(u[i] << 16);
            w[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
        }
    }
};
template <> struct HeadVec<float> {
    static constexpr int kN = 4;
    __device__ static void load(const float *p, float (&w)[4]) {
        const float4 v = *reinterpret_cast<const float4 *>(p);
        w[0] = v.x; w[1] = v.y; w[2] = v.z; w[3] = v.w;
    }
};

template <typename W, int TT>
__global__ void __launch_bounds__(256)
lm_head_kernel(const float *__restrict__ hidden, const W *__restrict__ weight,
               float *__restrict__ logits, uint32_t n_tokens, uint32_t vocab, uint32_t d,
               uint32_t vocab_stride) {
    qk::pdl_launch();  // the next kernel may begin its prologue
    qk::pdl_wait();    // everything before this kernel on the stream is complete and visible
    constexpr int N = HeadVec<W>::kN;
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t v = blockIdx.x * 8 + warp;
    if (v >= vocab) return;
    const W *row = weight + (size_t)v * d;
    for (uint32_t t0 = 0; t0 < n_tokens; t0 += TT) {
        float acc[TT];
#pragma unroll
        for (int t = 0; t < TT; ++t) acc[t] = 0.f;
        for (uint32_t i = lane * N; i < d; i += 32 * N) {
            float w[N];
            HeadVec<W>::load(row + i, w);
#pragma unroll
            for (int t = 0; t < TT; ++t) {
                if (t0 + t < n_tokens) {
                    const float *h = hidden + (size_t)(t0 + t) * d + i;
#pragma unroll
                    for (int e = 0; e < N; e += 4) {
                        const float4 hv = *reinterpret_cast<const float4 *>(h + e);
                        acc[t] = fmaf(hv.x, w[e], fmaf(hv.y, w[e + 1],
                                 fmaf(hv.z, w[e + 2], fmaf(hv.w, w[e + 3], acc[t]))));
                    }
                }
            }
        }
#pragma unroll
        for (int t = 0; t < TT; ++t) {
            float a = acc[t];
            for (int off = 16; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
            if (lane == 0 && t0 + t < n_tokens) logits[(size_t)(t0 + t) * vocab_stride + v] = a;
        }
    }
}

// First maximum of each row (sampler.rs:5-16: a later equal value does not win), in two
// steps: grid (parts, tokens) blocks each reduce a slice to a (value, index) pair, then one
// block per token reduces the pairs.  idx is offset by `index_base` (vocabulary shards).
__device__ __forceinline__ void argmax_block_reduce(float best, int bi, float *out_val,
                                                    int32_t *out_idx, int32_t offset) {
    __shared__ float sv[256];
    __shared__ int si[256];
    sv[threadIdx.x] = best;
    si[threadIdx.x] = bi;
    __syncthreads();
    for (int off = 128; off > 0; off >>= 1) {
        if ((int)threadIdx.x < off) {
            float ov = sv[threadIdx.x + off];
            int oi = si[threadIdx.x + off];
            if (ov > sv[threadIdx.x] || (ov == sv[threadIdx.x] && oi < si[threadIdx.x])) {
                sv[threadIdx.x] = ov;
                si[threadIdx.x] = oi;
            }
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        *out_val = sv[0];
        *out_idx = (si[0] == 0x7fffffff ? 0 : si[0]) + offset;  // nothing finite: index 0
    }
}

__global__ void __launch_bounds__(256)
argmax_partial_kernel(const float *__restrict__ logits, uint32_t vocab, uint32_t stride,
                      uint32_t slice, float *__restrict__ part_val, int32_t *__restrict__ part_idx) {
    qk::pdl_launch();  // the next kernel may begin its prologue
    qk::pdl_wait();    // everything before this kernel on the stream is complete and visible
    const float *row = logits + (size_t)blockIdx.y * stride;
    const uint32_t lo = blockIdx.x * slice, hi = min(vocab, lo + slice);
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (uint32_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        float v = row[i];
        if (v > best || (v == best && (int)i < bi)) {
            best = v;
            bi = (int)i;
        }
    }
    const size_t o = (size_t)blockIdx.y * gridDim.x + blockIdx.x;
    argmax_block_reduce(best, bi, part_val + o, part_idx + o, 0);
}

__global__ void __launch_bounds__(256)
argmax_final_kernel(const float *__restrict__ part_val, const int32_t *__restrict__ part_idx,
                    uint32_t parts, int32_t index_base, float *__restrict__ out_val,
                    int32_t *__restrict__ out_idx) {
    qk::pdl_launch();  // the next kernel may begin its prologue
    qk::pdl_wait();    // everything before this kernel on the stream is complete and visible
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (uint32_t i = threadIdx.x; i < parts; i += blockDim.x) {
        float v = part_val[(size_t)blockIdx.x * parts + i];
        int idx = part_idx[(size_t)blockIdx.x * parts + i];
        if (v > best || (v == best && idx < bi)) {
            best = v;
            bi = idx;
        }
    }
    argmax_block_reduce(best, bi, out_val + blockIdx.x, out_idx + blockIdx.x, index_base);
}

qk_status enter(qk_ctx *ctx, qk_ctx **c) {
    qk_status st = qk::resolve_ctx(ctx, c);
    if (st != QK_OK) return st;
    QK_CUDA(cudaSetDevice((*c)->device));
    return QK_OK;
}

// Launch on the context's stream as a programmatic dependent launch (the kernels above all
// begin with pdl_launch / pdl_wait).  Variadic so that template arguments with commas pass.
#define QK_PDL(c, kernel, grid, block, smem, ...) \
    (void)qk::launch_pdl((c)->pdl, kernel, grid, block, smem, (c)->stream, __VA_ARGS__)

// The C ABI's qk_feed -> the kernels' FeedArgs (null: nothing is fed).
qk_status feed_args(const qk_feed *feed, FeedArgs *out) {
    *out = FeedArgs{};
    if (!feed) return QK_OK;
    if (feed->n_arrays > 4) return qk::fail(QK_ERR_VALUE, "at most 4 target arrays can be fed, got %zu", feed->n_arrays);
    for (size_t i = 0; i < feed->n_arrays; ++i) {
        if (!feed->targets[i]) return qk::fail(QK_ERR_VALUE, "feed target array %zu is null", i);
        out->arr[i] = static_cast<const FeedTarget *>(feed->targets[i]);
        out->per_token[i] = (uint32_t)feed->per_token[i];
    }
    out->n = (uint32_t)feed->n_arrays;
    return QK_OK;
}

#define QK_LAUNCHED(c)            \
    QK_CUDA(cudaGetLastError()); \
    (c)->launches++;             \
    return QK_OK

}  // namespace

// ------------------------------------------------------------------ LM head for a batch
// logits[token][v] = sum_k h[token][k] * W[v][k] for up to 64 tokens per pass, W bfloat16:
// the head is read ONCE for all tokens (the warp-per-row kernel above re-reads it for
// every eight).  bf16 tensor cores (mma.sync m16n8k16): a warp owns 16 vocabulary rows (the
// M side, streamed straight from global memory in 16-byte loads), the tokens are the N side,
// staged chunk by chunk in shared memory.  The float32 hidden state is split into two
// bfloat16 terms (hi = bf16(h), lo = bf16(h - hi)), so the products are exact to 2^-17 even
// when h is not bfloat16-valued (for bfloat16 serving lo is zero).  The k order inside a
// 32-wide group is renamed (slot 2t, 2t+1 <- k 8t, 8t+1; slot 8+2t <- 8t+2; second MMA
// 8t+4..7) so that one 16-byte load feeds two MMAs on either operand.
__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

constexpr int kHeadPitch = 96;  // bfloat16 elements per staged token row: 64 k + 32 pad (192 B)

// hidden [tokens][d] float32 -> hi, lo [tokens][d] bfloat16 (hi = bf16(h), lo = bf16(h - hi));
// *any_lo is set when some lo is not zero, i.e. when the hidden state is not bfloat16-valued.
__global__ void split_hidden_kernel(const float *__restrict__ hidden, uint16_t *__restrict__ hi,
                                    uint16_t *__restrict__ lo, uint32_t *__restrict__ any_lo,
                                    size_t n) {
    qk::pdl_launch();  // the next kernel may begin its prologue
    qk::pdl_wait();    // everything before this kernel on the stream is complete and visible
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float x = hidden[i];
    const uint16_t h = float_to_bf16_bits(x);
    const uint16_t l = float_to_bf16_bits(x - bf16_bits_to_float(h));
    hi[i] = h;
    lo[i] = l;
    if (l & 0x7fffu) *any_lo = 1u;
}

__device__ __forceinline__ void cp_async_16(void *smem, const void *gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                     (uint32_t)__cvta_generic_to_shared(smem)),
                 "l"(gmem)
                 : "memory");
}

template <int NT>  // token tiles of eight
__global__ void __launch_bounds__(128)
lm_head_mma_kernel(const uint16_t *__restrict__ hid_hi, const uint16_t *__restrict__ hid_lo,
                   const uint32_t *__restrict__ any_lo, const uint16_t *__restrict__ weight,
                   float *__restrict__ logits, uint32_t n_tokens, uint32_t vocab, uint32_t d,
                   uint32_t vocab_stride) {
    qk::pdl_launch();  // the next kernel may begin its prologue
    qk::pdl_wait();    // everything before this kernel on the stream is complete and visible
    extern __shared__ __align__(16) uint16_t sm_head[];  // [2 buffers][hi, lo][8 NT][kHeadPitch]
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32, g = lane >> 2, t = lane & 3;
    const uint32_t tok0 = blockIdx.y * (8 * NT);
    const uint32_t v_lo = min(blockIdx.x * 64 + warp * 16 + g, vocab - 1);
    const uint32_t v_hi = min(blockIdx.x * 64 + warp * 16 + g + 8, vocab - 1);
    const uint4 *row_lo = reinterpret_cast<const uint4 *>(weight + (size_t)v_lo * d) + t;
    const uint4 *row_hi = reinterpret_cast<const uint4 *>(weight + (size_t)v_hi * d) + t;
    const uint32_t n_chunks = d / 64;
    constexpr uint32_t kBuf = 2 * 8 * NT * kHeadPitch;  // elements per buffer (hi and lo)
    const bool with_lo = *any_lo != 0;  // bfloat16-valued hidden states need no second term

    // chunk `chunk` of the tokens' hidden rows: 8 pieces of 16 bytes per token and term
    auto stage = [&](uint32_t chunk, uint32_t buf) {
        uint16_t *hi = sm_head + buf * kBuf, *lo = hi + 8 * NT * kHeadPitch;
        for (uint32_t idx = threadIdx.x; idx < 8 * NT * 8; idx += 128) {
            const uint32_t tok = idx / 8, piece = idx % 8;
            const uint32_t src_tok = min(tok0 + tok, n_tokens - 1);  // rows past the batch are never stored
            const size_t src = (size_t)src_tok * d + chunk * 64 + piece * 8;
            cp_async_16(hi + tok * kHeadPitch + piece * 8, hid_hi + src);
            if (with_lo) cp_async_16(lo + tok * kHeadPitch + piece * 8, hid_lo + src);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float acc[NT][4];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;
    // the weights of the next chunk are in flight while this one is multiplied
    uint4 wl[2], wh[2];
    wl[0] = row_lo[0]; wl[1] = row_lo[4];
    wh[0] = row_hi[0]; wh[1] = row_hi[4];
    stage(0, 0);
    for (uint32_t c = 0; c < n_chunks; ++c) {
        const uint4 cl[2] = {wl[0], wl[1]}, ch[2] = {wh[0], wh[1]};
        if (c + 1 < n_chunks) {
            wl[0] = row_lo[(c + 1) * 8]; wl[1] = row_lo[(c + 1) * 8 + 4];
            wh[0] = row_hi[(c + 1) * 8]; wh[1] = row_hi[(c + 1) * 8 + 4];
            stage(c + 1, (c + 1) & 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();  // chunk c has landed for every thread
        const uint16_t *hi = sm_head + (c & 1) * kBuf, *lo = hi + 8 * NT * kHeadPitch;
#pragma unroll
        for (int gi = 0; gi < 2; ++gi) {
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const uint32_t off = (8 * nt + g) * kHeadPitch + gi * 32 + 8 * t;
                const uint4 bh = *reinterpret_cast<const uint4 *>(hi + off);
                mma_bf16(acc[nt], cl[gi].x, ch[gi].x, cl[gi].y, ch[gi].y, bh.x, bh.y);
                mma_bf16(acc[nt], cl[gi].z, ch[gi].z, cl[gi].w, ch[gi].w, bh.z, bh.w);
                if (with_lo) {
                    const uint4 bl = *reinterpret_cast<const uint4 *>(lo + off);
                    mma_bf16(acc[nt], cl[gi].x, ch[gi].x, cl[gi].y, ch[gi].y, bl.x, bl.y);
                    mma_bf16(acc[nt], cl[gi].z, ch[gi].z, cl[gi].w, ch[gi].w, bl.z, bl.w);
                }
            }
        }
        __syncthreads();  // the buffer may be refilled
    }
    const uint32_t v0 = blockIdx.x * 64 + warp * 16 + g;
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const uint32_t tok = tok0 + 8 * nt + 2 * t + (e & 1), v = v0 + (e >> 1) * 8;
            if (tok < n_tokens && v < vocab) logits[(size_t)tok * vocab_stride + v] = acc[nt][e];
        }
}

template <int NT>
void launch_lm_head_mma(qk_ctx *c, const uint16_t *hi, const uint16_t *lo, const uint32_t *any_lo,
                        const uint16_t *weight, float *logits, size_t n_tokens, size_t vocab, size_t d,
                        size_t stride) {
    const size_t smem = 2 * 2 * 8 * NT * kHeadPitch * sizeof(uint16_t);
    if (smem > 48 * 1024)
        cudaFuncSetAttribute(lm_head_mma_kernel<NT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    dim3 grid((unsigned)qk::ceil_div(vocab, 64), (unsigned)qk::ceil_div(n_tokens, 8 * NT));
    QK_PDL(c, (lm_head_mma_kernel<NT>), dim3(grid), dim3(128), smem, hi, lo, any_lo, weight, logits,
                                                          (uint32_t)n_tokens, (uint32_t)vocab,
                                                          (uint32_t)d, (uint32_t)stride);
}

extern "C" {

qk_status qk_rmsnorm_feed(qk_ctx *ctx, const float *x, const float *residual, const float *weight,
                          size_t n_tokens, size_t d, float eps, int32_t serving_dtype, float *x_out,
                          float *y, const qk_feed *feed) {
    qk_ctx *c;
    qk_status st = enter(ctx, &c);
    if (st != QK_OK) return st;
    FeedArgs fa;
    if ((st = feed_args(feed, &fa)) != QK_OK) return st;
    if (n_tokens == 0) return QK_OK;
    const size_t smem = fa.n ? d * sizeof(float) : 0;
    if (smem > 48 * 1024)
        QK_CUDA(cudaFuncSetAttribute(rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    // several blocks per token share the table building when x_out is not x itself (every block
    // re-reads x) and the row fits the kernel's register cache
    const unsigned parts = (fa.n && x_out != x && d <= (size_t)kRmsThreads * kRmsPerThread) ? kFeedParts : 1;
    QK_PDL(c, rmsnorm_kernel, dim3((unsigned)n_tokens, parts), dim3(kRmsThreads), smem, x, residual, weight,
           x_out, y, (uint32_t)d, eps, serving_dtype == QK_BF16, fa);
    QK_LAUNCHED(c);
}

qk_status qk_rmsnorm(qk_ctx *ctx, const float *x, const float *residual, const float *weight,
                     size_t n_tokens, size_t d, float eps, int32_t serving_dtype, float *x_out,
                     float *y) {
    return qk_rmsnorm_feed(ctx, x, residual, weight, n_tokens, d, eps, serving_dtype, x_out, y, nullptr);
}

qk_status qk_rope_cache(qk_ctx *ctx, float *q, const float *k, const float *v,
                        const float *cos_sin, const int32_t *positions, const int32_t *seq_index,
                        void *cache_k, void *cache_v, int32_t kv_dtype, size_t n_tokens,
                        size_t n_heads, size_t n_kv_heads, size_t head_dim, size_t s_max,
                        size_t n_seq) {
    qk_ctx *c;
    qk_status st = enter(ctx, &c);
    if (st != QK_OK) return st;
    if (head_dim % 2)
        return qk::fail(QK_ERR_VALUE, "RoPE needs an even head_dim, got %zu", head_dim);
    if (kv_dtype != QK_F32 && kv_dtype != QK_BF16)
        return qk::fail(QK_ERR_VALUE, "KV cache dtype must be float32 or bfloat16, got tag %d",
                        kv_dtype);
    if (n_tokens == 0) return QK_OK;
    // out-of-range positions are reported through the error word; it is created on the first
    // call, so make that call before any stream capture
    if ((st = qk::error_word(c)) != QK_OK) return st;
    int *err = (int *)c->d_err.ptr;
    if (kv_dtype == QK_F32)
        QK_PDL(c, (rope_cache_kernel<float>), dim3((unsigned)n_tokens), dim3(256), 0, 
            q, k, v, cos_sin, positions, seq_index, (float *)cache_k, (float *)cache_v,
            (uint32_t)n_heads, (uint32_t)n_kv_heads, (uint32_t)head_dim, (uint32_t)s_max,
            (uint32_t)n_seq, err);
    else
        QK_PDL(c, (rope_cache_kernel<uint16_t>), dim3((unsigned)n_tokens), dim3(256), 0, 
            q, k, v, cos_sin, positions, seq_index, (uint16_t *)cache_k, (uint16_t *)cache_v,
            (uint32_t)n_heads, (uint32_t)n_kv_heads, (uint32_t)head_dim, (uint32_t)s_max,
            (uint32_t)n_seq, err);
    c->err_armed = true;
    QK_LAUNCHED(c);
}

size_t qk_decode_attention_scratch(size_t batch, size_t n_heads, size_t head_dim,
                                   size_t n_splits) {
    return batch * n_heads * n_splits * (head_dim + 2) * sizeof(float);
}

qk_status qk_decode_attention_feed(qk_ctx *ctx, const float *q, const void *cache_k,
                                   const void *cache_v, int32_t kv_dtype, const int32_t *kv_len,
                                   size_t batch, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                                   size_t s_max, size_t n_splits, float *scratch, float *out,
                                   int32_t serving_dtype, const qk_feed *feed) {
    qk_ctx *c;
    qk_status st = enter(ctx, &c);
    if (st != QK_OK) return st;
    FeedArgs fa;
    if ((st = feed_args(feed, &fa)) != QK_OK) return st;
    // the combine step: per (sequence, head), or - when the consumers of the attention output
    // are fed - one block per sequence that also writes their digit tables
    auto combine = [&]() -> qk_status {
        if (fa.n) {
            const size_t smem = n_heads * head_dim * sizeof(float);
            if (smem > 200 * 1024)
                return qk::fail(QK_ERR_VALUE, "%zu attention outputs do not fit shared memory", n_heads * head_dim);
            QK_CUDA(cudaFuncSetAttribute(decode_combine_feed_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)smem));
            QK_PDL(c, decode_combine_feed_kernel, dim3((unsigned)batch, kFeedParts), dim3(512), smem, (const float *)scratch, out,
                   (uint32_t)n_heads, (uint32_t)head_dim, (uint32_t)n_splits, serving_dtype == QK_BF16, fa);
        } else {
            QK_PDL(c, decode_combine_kernel, dim3((unsigned)(batch * n_heads)), dim3(128), 0, (const float *)scratch,
                   out, (uint32_t)head_dim, (uint32_t)n_splits);
        }
        return QK_OK;
    };
    if (n_kv_heads == 0 || n_heads % n_kv_heads != 0)
        return qk::fail(QK_ERR_VALUE, "n_kv_heads must divide n_heads: n_heads=%zu, n_kv_heads=%zu",
                        n_heads, n_kv_heads);
    const size_t group = n_heads / n_kv_heads;
    if (head_dim > 256)
        return qk::fail(QK_ERR_VALUE, "head_dim above 256 is not supported, got %zu", head_dim);
    if (n_splits == 0 || batch == 0) return qk::fail(QK_ERR_VALUE, "empty decode attention");
    if (n_splits > 128)
        return qk::fail(QK_ERR_VALUE, "at most 128 key splits are supported, got %zu", n_splits);
    if (kv_dtype != QK_F32 && kv_dtype != QK_BF16)
        return qk::fail(QK_ERR_VALUE, "KV cache dtype must be float32 or bfloat16, got tag %d",
                        kv_dtype);
    if (kv_dtype == QK_BF16 && head_dim == 128 && c->decode_attention_kernel != 0) {
        // bfloat16 cache, head_dim 128: both products on the tensor cores.  (Even with one
        // query head per kv head, where 15 of the MMA's 16 rows are padding, it measured a
        // little faster than the scalar kernel: 0.471 against 0.480 ms per step on the
        // Llama-2-7B block.)
        const size_t gq8 = group < 8 ? group : 8, subs = qk::ceil_div(group, gq8);
        const size_t chunk8 = qk::ceil_div(s_max, n_splits);
        dim3 grid8((unsigned)n_splits, (unsigned)(n_kv_heads * subs), (unsigned)batch);
        const size_t smem8 = kMmaDecSmemBytes;
        QK_CUDA(cudaFuncSetAttribute(decode_attention_mma_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem8));
        QK_PDL(c, decode_attention_mma_kernel, dim3(grid8), dim3(kMmaDecWarps * 32), smem8, 
            q, (const uint16_t *)cache_k, (const uint16_t *)cache_v, kv_len, scratch,
            (uint32_t)n_heads, (uint32_t)n_kv_heads, (uint32_t)gq8, (uint32_t)s_max,
            (uint32_t)chunk8, (uint32_t)n_splits);
        QK_CUDA(cudaGetLastError());
        c->launches++;
        if ((st = combine()) != QK_OK) return st;
        QK_LAUNCHED(c);
    }
    const int gq = group % 4 == 0 ? 4 : group % 2 == 0 ? 2 : 1;  // query heads per block
    const size_t chunk = qk::ceil_div(s_max, n_splits);
    dim3 grid((unsigned)n_splits, (unsigned)(n_kv_heads * (group / gq)), (unsigned)batch);
    const size_t smem = (kDecThreads / 8) * gq * head_dim * sizeof(float);
    const int dpl = head_dim <= 64 ? 8 : head_dim <= 128 ? 16 : 32;
#define QK_DEC(KV, DPL, GQ)                                                                      \
    do {                                                                                         \
        if (smem > 48 * 1024)                                                                    \
            QK_CUDA(cudaFuncSetAttribute(decode_attention_kernel<KV, DPL, GQ>,                   \
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        QK_PDL(c, (decode_attention_kernel<KV, DPL, GQ>), dim3(grid), dim3(kDecThreads), smem,             \
            q, (const KV *)cache_k, (const KV *)cache_v, kv_len, scratch, (uint32_t)n_heads,     \
            (uint32_t)n_kv_heads, (uint32_t)head_dim, (uint32_t)s_max, (uint32_t)chunk,          \
            (uint32_t)n_splits);                                                                 \
    } while (0)
#define QK_DEC_G(KV, DPL)                                                  \
    do {                                                                   \
        if (gq == 4) QK_DEC(KV, DPL, 4);                                   \
        else if (gq == 2) QK_DEC(KV, DPL, 2);                              \
        else QK_DEC(KV, DPL, 1);                                           \
    } while (0)
    if (kv_dtype == QK_F32) {
        if (dpl == 8) QK_DEC_G(float, 8); else if (dpl == 16) QK_DEC_G(float, 16); else QK_DEC_G(float, 32);
    } else {
        if (dpl == 8) QK_DEC_G(uint16_t, 8); else if (dpl == 16) QK_DEC_G(uint16_t, 16); else QK_DEC_G(uint16_t, 32);
    }
#undef QK_DEC_G
#undef QK_DEC
    QK_CUDA(cudaGetLastError());
    c->launches++;
    if ((st = combine()) != QK_OK) return st;
    QK_LAUNCHED(c);
}

qk_status qk_decode_attention(qk_ctx *ctx, const float *q, const void *cache_k,
                              const void *cache_v, int32_t kv_dtype, const int32_t *kv_len,
                              size_t batch, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                              size_t s_max, size_t n_splits, float *scratch, float *out) {
    return qk_decode_attention_feed(ctx, q, cache_k, cache_v, kv_dtype, kv_len, batch, n_heads, n_kv_heads,
                                    head_dim, s_max, n_splits, scratch, out, QK_F32, nullptr);
}

size_t qk_decode_attention_rope_scratch(size_t batch, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                                        size_t n_splits) {
    // the partials, then one ticket per (sequence, kv-head block) - at most one per head
    return qk_decode_attention_scratch(batch, n_heads, head_dim, n_splits) +
           batch * (n_heads > n_kv_heads ? n_heads : n_kv_heads) * sizeof(uint32_t);
}

qk_status qk_decode_attention_rope(qk_ctx *ctx, const float *q, const float *k, const float *v,
                                   const float *cos_sin, const int32_t *positions, const int32_t *seq_index,
                                   void *cache_k, void *cache_v, int32_t kv_dtype, const int32_t *kv_len,
                                   size_t batch, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                                   size_t s_max, size_t n_seq, size_t n_splits, float *scratch, float *out) {
    qk_ctx *c;
    qk_status st = enter(ctx, &c);
    if (st != QK_OK) return st;
    if (kv_dtype != QK_BF16 || head_dim != 128)
        return qk::fail(QK_ERR_VALUE, "the one-launch decode attention needs a bfloat16 cache and head_dim 128, "
                        "got cache tag %d and head_dim %zu", kv_dtype, head_dim);
    if (n_kv_heads == 0 || n_heads % n_kv_heads != 0)
        return qk::fail(QK_ERR_VALUE, "n_kv_heads must divide n_heads: n_heads=%zu, n_kv_heads=%zu",
                        n_heads, n_kv_heads);
    if (n_splits == 0 || batch == 0) return qk::fail(QK_ERR_VALUE, "empty decode attention");
    if (n_splits > 128)
        return qk::fail(QK_ERR_VALUE, "at most 128 key splits are supported, got %zu", n_splits);
    if ((st = qk::error_word(c)) != QK_OK) return st;
    const size_t group = n_heads / n_kv_heads, gq8 = group < 8 ? group : 8, subs = qk::ceil_div(group, gq8);
    const size_t chunk8 = qk::ceil_div(s_max, n_splits);
    uint32_t *tickets = reinterpret_cast<uint32_t *>(
        reinterpret_cast<uint8_t *>(scratch) + qk_decode_attention_scratch(batch, n_heads, head_dim, n_splits));
    dim3 grid((unsigned)n_splits, (unsigned)(n_kv_heads * subs), (unsigned)batch);
    QK_CUDA(cudaFuncSetAttribute(decode_attention_rope_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kMmaDecSmemBytes));
    QK_PDL(c, decode_attention_rope_kernel, dim3(grid), dim3(kMmaDecWarps * 32), (size_t)kMmaDecSmemBytes, q, k, v,
           cos_sin, positions, seq_index, (uint16_t *)cache_k, (uint16_t *)cache_v, kv_len, scratch, tickets, out,
           (uint32_t)n_heads, (uint32_t)n_kv_heads, (uint32_t)gq8, (uint32_t)s_max, (uint32_t)n_seq,
           (uint32_t)chunk8, (uint32_t)n_splits, (int *)c->d_err.ptr);
    c->err_armed = true;
    QK_LAUNCHED(c);
}

qk_status qk_prefill_attention(qk_ctx *ctx, const float *q, const void *cache_k, const void *cache_v,
                               int32_t kv_dtype, size_t seq, size_t first_position, size_t n_tokens,
                               size_t n_heads, size_t n_kv_heads, size_t head_dim, size_t s_max,
                               float *out) {
    qk_ctx *c;
    qk_status st = enter(ctx, &c);
    if (st != QK_OK) return st;
    if (n_kv_heads == 0 || n_heads % n_kv_heads != 0)
        return qk::fail(QK_ERR_VALUE, "n_kv_heads must divide n_heads: n_heads=%zu, n_kv_heads=%zu",
                        n_heads, n_kv_heads);
    const size_t group = n_heads / n_kv_heads;
    if (kv_dtype != QK_F32 && kv_dtype != QK_BF16)
        return qk::fail(QK_ERR_VALUE, "KV cache dtype must be float32 or bfloat16, got tag %d", kv_dtype);
    if (head_dim > 256)
        return qk::fail(QK_ERR_VALUE, "head_dim above 256 is not supported, got %zu", head_dim);
    if (n_tokens == 0) return QK_OK;
    if (first_position + n_tokens > s_max)
        return qk::fail(QK_ERR_VALUE, "positions %zu..%zu do not fit the KV cache of %zu positions",
                        first_position, first_position + n_tokens - 1, s_max);
    if (kv_dtype != QK_BF16 || head_dim != 128 || (group != 1 && group != 2 && group % 4 != 0) ||
        c->decode_attention_kernel == 0) {
        // any other shape: the plain kernel
        const unsigned blocks = (unsigned)qk::ceil_div(n_tokens * n_heads, 4);
        if (kv_dtype == QK_F32)
            QK_PDL(c, prefill_attention_simple_kernel<float>, dim3(blocks), dim3(128), 0, q,
                   (const float *)cache_k, (const float *)cache_v, out, (uint32_t)n_tokens,
                   (uint32_t)first_position, (uint32_t)seq, (uint32_t)n_heads, (uint32_t)n_kv_heads,
                   (uint32_t)head_dim, (uint32_t)s_max);
        else
            QK_PDL(c, prefill_attention_simple_kernel<uint16_t>, dim3(blocks), dim3(128), 0, q,
                   (const uint16_t *)cache_k, (const uint16_t *)cache_v, out, (uint32_t)n_tokens,
                   (uint32_t)first_position, (uint32_t)seq, (uint32_t)n_heads, (uint32_t)n_kv_heads,
                   (uint32_t)head_dim, (uint32_t)s_max);
        QK_LAUNCHED(c);
    }
    const size_t hw = group < 4 ? group : 4, pbs = 4 / hw;
    dim3 grid((unsigned)qk::ceil_div(n_tokens, 16 * pbs), (unsigned)(n_kv_heads * (group / hw)));
    QK_CUDA(cudaFuncSetAttribute(prefill_attention_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kPfSmem));
    QK_PDL(c, prefill_attention_mma_kernel, grid, dim3(128), (size_t)kPfSmem, q, (const uint16_t *)cache_k,
           (const uint16_t *)cache_v, out, (uint32_t)n_tokens, (uint32_t)first_position, (uint32_t)seq,
           (uint32_t)n_heads, (uint32_t)n_kv_heads, (uint32_t)hw, (uint32_t)s_max);
    QK_LAUNCHED(c);
}

qk_status qk_swiglu_feed(qk_ctx *ctx, const float *gate, const float *up, size_t n_tokens, size_t n,
                         int32_t serving_dtype, const qk_feed *feed) {
    qk_ctx *c;
    qk_status st = enter(ctx, &c);
    if (st != QK_OK) return st;
    FeedArgs fa;
    if ((st = feed_args(feed, &fa)) != QK_OK) return st;
    if (!fa.n) return qk::fail(QK_ERR_VALUE, "qk_swiglu_feed: nothing to feed");
    if (n_tokens == 0 || n == 0) return QK_OK;
    const size_t smem = n * sizeof(float);
    if (smem > 200 * 1024)
        return qk::fail(QK_ERR_VALUE, "a row of %zu activations does not fit shared memory", n);
    QK_CUDA(cudaFuncSetAttribute(swiglu_feed_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    QK_PDL(c, swiglu_feed_kernel, dim3((unsigned)n_tokens, kFeedParts), dim3(512), smem, gate, up, (uint32_t)n,
           serving_dtype == QK_BF16, fa);
    QK_LAUNCHED(c);
}

qk_status qk_swiglu(qk_ctx *ctx, const float *gate, const float *up, size_t n, float *out) {
    qk_ctx *c;
    qk_status st = enter(ctx, &c);
    if (st != QK_OK) return st;
    if (n == 0) return QK_OK;
    QK_PDL(c, swiglu_kernel, dim3((unsigned)qk::ceil_div(n, 256)), dim3(256), 0, gate, up, out, n);
    QK_LAUNCHED(c);
}

qk_status qk_add(qk_ctx *ctx, const float *a, const float *b, size_t n, float *out) {
    qk_ctx *c;
    qk_status st = enter(ctx, &c);
    if (st != QK_OK) return st;
    if (n == 0) return QK_OK;
    QK_PDL(c, add_kernel, dim3((unsigned)qk::ceil_div(n, 256)), dim3(256), 0, a, b, out, n);
    QK_LAUNCHED(c);
}

qk_status qk_embed(qk_ctx *ctx, const void *table, int32_t table_dtype, const int32_t *ids,
                   size_t n_tokens, size_t d, size_t vocab, float *out) {
    qk_ctx *c;
    qk_status st = enter(ctx, &c);
    if (st != QK_OK) return st;
    if (n_tokens == 0) return QK_OK;
    if (table_dtype == QK_F32)
        QK_PDL(c, (embed_kernel<float>), dim3((unsigned)n_tokens), dim3(256), 0, 
            (const float *)table, ids, out, (uint32_t)d, (uint32_t)vocab);
    else if (table_dtype == QK_BF16)
        QK_PDL(c, (embed_kernel<uint16_t>), dim3((unsigned)n_tokens), dim3(256), 0, 
            (const uint16_t *)table, ids, out, (uint32_t)d, (uint32_t)vocab);
    else
        return qk::fail(QK_ERR_VALUE, "embedding dtype must be float32 or bfloat16, got tag %d",
                        table_dtype);
    QK_LAUNCHED(c);
}

qk_status qk_lm_head(qk_ctx *ctx, const float *hidden, const void *weight, int32_t weight_dtype,
                     size_t n_tokens, size_t vocab, size_t d, size_t logits_stride,
                     float *logits) {
    qk_ctx *c;
    qk_status st = enter(ctx, &c);
    if (st != QK_OK) return st;
    if (d % 8) return qk::fail(QK_ERR_VALUE, "d_model must be a multiple of 8, got %zu", d);
    if (n_tokens == 0 || vocab == 0) return QK_OK;
    const unsigned blocks = (unsigned)qk::ceil_div(vocab, 8);
    if (weight_dtype == QK_F32) {
        if (n_tokens == 1)
            QK_PDL(c, (lm_head_kernel<float, 1>), dim3(blocks), dim3(256), 0, 
                hidden, (const float *)weight, logits, 1, (uint32_t)vocab, (uint32_t)d,
                (uint32_t)logits_stride);
        else
            QK_PDL(c, (lm_head_kernel<float, 8>), dim3(blocks), dim3(256), 0, 
                hidden, (const float *)weight, logits, (uint32_t)n_tokens, (uint32_t)vocab,
                (uint32_t)d, (uint32_t)logits_stride);
    } else if (weight_dtype == QK_BF16 && n_tokens >= 8 && d % 64 == 0) {
        // a batch: one pass over the head on the bf16 tensor cores
        const uint16_t *w = (const uint16_t *)weight;
        const size_t n = n_tokens * d, term = qk::ceil_div(n * 2, 256) * 256;
        if ((st = c->d_head.reserve(2 * term + 256)) != QK_OK) return st;
        uint16_t *hi = (uint16_t *)c->d_head.ptr, *lo = (uint16_t *)((uint8_t *)c->d_head.ptr + term);
        uint32_t *any_lo = (uint32_t *)((uint8_t *)c->d_head.ptr + 2 * term);
        QK_CUDA(cudaMemsetAsync(any_lo, 0, sizeof(uint32_t), c->stream));
        QK_PDL(c, split_hidden_kernel, dim3((unsigned)qk::ceil_div(n, 256)), dim3(256), 0, hidden, hi, lo, any_lo, n);
        QK_CUDA(cudaGetLastError());
        c->launches++;
        if (n_tokens <= 8) launch_lm_head_mma<1>(c, hi, lo, any_lo, w, logits, n_tokens, vocab, d, logits_stride);
        else if (n_tokens <= 16) launch_lm_head_mma<2>(c, hi, lo, any_lo, w, logits, n_tokens, vocab, d, logits_stride);
        else if (n_tokens <= 32) launch_lm_head_mma<4>(c, hi, lo, any_lo, w, logits, n_tokens, vocab, d, logits_stride);
        else launch_lm_head_mma<8>(c, hi, lo, any_lo, w, logits, n_tokens, vocab, d, logits_stride);
    } else if (weight_dtype == QK_BF16) {
        if (n_tokens == 1)
            QK_PDL(c, (lm_head_kernel<uint16_t, 1>), dim3(blocks), dim3(256), 0, 
                hidden, (const uint16_t *)weight, logits, 1, (uint32_t)vocab, (uint32_t)d,
                (uint32_t)logits_stride);
        else
            QK_PDL(c, (lm_head_kernel<uint16_t, 8>), dim3(blocks), dim3(256), 0, 
                hidden, (const uint16_t *)weight, logits, (uint32_t)n_tokens, (uint32_t)vocab,
                (uint32_t)d, (uint32_t)logits_stride);
    } else {
        return qk::fail(QK_ERR_VALUE, "head dtype must be float32 or bfloat16, got tag %d",
                        weight_dtype);
    }
    QK_LAUNCHED(c);
}

qk_status qk_argmax_first(qk_ctx *ctx, const float *logits, size_t n_tokens, size_t vocab,
                          size_t logits_stride, int32_t index_base, float *out_val,
                          int32_t *out_idx) {
    qk_ctx *c;
    qk_status st = enter(ctx, &c);
    if (st != QK_OK) return st;
    if (n_tokens == 0) return QK_OK;
    // partial results live in the context's scratch; it is sized on the first call, so make
    // that call before any stream capture
    const size_t parts = vocab >= 65536 ? 64 : vocab >= 4096 ? 16 : 1;
    const size_t slice = qk::ceil_div(vocab, parts);
    if ((st = c->d_z.reserve(n_tokens * parts * 8)) != QK_OK) return st;
    float *part_val = (float *)c->d_z.ptr;
    int32_t *part_idx = (int32_t *)(part_val + n_tokens * parts);
    dim3 grid((unsigned)parts, (unsigned)n_tokens);
    QK_PDL(c, argmax_partial_kernel, dim3(grid), dim3(256), 0, logits, (uint32_t)vocab,
                                                       (uint32_t)logits_stride, (uint32_t)slice,
                                                       part_val, part_idx);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    QK_PDL(c, argmax_final_kernel, dim3((unsigned)n_tokens), dim3(256), 0, 
        part_val, part_idx, (uint32_t)parts, index_base, out_val, out_idx);
    QK_LAUNCHED(c);
}

qk_status qk_allreduce_rmsnorm(qk_ctx *ctx, const float *partial, const uint64_t *peer_inbox,
                               uint32_t *state_dev, int32_t rank, int32_t world, const float *x,
                               const float *weight, size_t n_tokens, size_t d, float eps,
                               int32_t serving_dtype, float *x_out, float *y) {
    return qk_allreduce_rmsnorm_feed(ctx, partial, peer_inbox, state_dev, rank, world, x, weight, n_tokens, d,
                                     eps, serving_dtype, x_out, y, nullptr);
}

qk_status qk_allreduce_rmsnorm_feed(qk_ctx *ctx, const float *partial, const uint64_t *peer_inbox,
                                    uint32_t *state_dev, int32_t rank, int32_t world, const float *x,
                                    const float *weight, size_t n_tokens, size_t d, float eps,
                                    int32_t serving_dtype, float *x_out, float *y, const qk_feed *feed) {
    qk_ctx *c;
    qk_status st = enter(ctx, &c);
    if (st != QK_OK) return st;
    FeedArgs fa;
    if ((st = feed_args(feed, &fa)) != QK_OK) return st;
    if (world < 1 || world > 8 || rank < 0 || rank >= world)
        return qk::fail(QK_ERR_VALUE, "qk_allreduce_rmsnorm: rank %d of %d (1..8 ranks)", rank, world);
    if (!partial || !peer_inbox || !state_dev || !x_out)
        return qk::fail(QK_ERR_VALUE, "qk_allreduce_rmsnorm: null argument");
    if (n_tokens == 0) return QK_OK;
    if ((st = qk::error_word(c)) != QK_OK) return st;
    InboxArgs inbox{};
    for (int r = 0; r < world; ++r) inbox.at[r] = reinterpret_cast<unsigned long long *>(peer_inbox[r]);
    const size_t smem = fa.n ? d * sizeof(float) : 0;
    if (smem > 48 * 1024)
        QK_CUDA(cudaFuncSetAttribute(allreduce_rmsnorm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)smem));
    const unsigned parts = (fa.n && x_out != x && d <= (size_t)kRmsThreads * 8) ? kFeedParts : 1;
    QK_PDL(c, allreduce_rmsnorm_kernel, dim3((unsigned)n_tokens, parts), dim3(kRmsThreads), smem,
        inbox, partial, state_dev, state_dev + 1, rank, world, x, weight, x_out, y, (uint32_t)d, eps,
        serving_dtype == QK_BF16, (int *)c->d_err.ptr, c->wait_limit ? c->wait_limit : (1u << 22), fa);
    c->err_armed = true;
    QK_LAUNCHED(c);
}

int32_t qk_set_decode_attention_kernel(qk_ctx *ctx, int32_t which) {
    qk_ctx *c;
    if (qk::resolve_ctx(ctx, &c) != QK_OK) return -1;
    std::lock_guard<std::mutex> lock(c->mu);
    const int32_t before = c->decode_attention_kernel;
    if (which == 0 || which == 1) c->decode_attention_kernel = which;
    return before;
}

}  // extern "C"
