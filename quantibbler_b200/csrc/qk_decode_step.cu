// One decode step's transformer blocks as ONE cooperative kernel.
//
// A single-token step of the reference's transformer_forward (engine/mod.rs:878-945) is, per
// block: norm, q/k/v, RoPE + cache append, attention, o, norm, gate/up, SwiGLU, down - about
// fourteen dependent kernels when each is a launch of its own, and at batch 1 every one of them
// lasts as long as its chain of dependent memory round trips (5 to 10 us), not as long as its
// bytes.  Here the whole sequence of blocks runs in one persistent kernel, one CTA per SM, with
// a grid-wide barrier between phases (about 1.3 us) instead of a kernel boundary, and with the
// small operations folded into the phases that consume them:
//   phase 1  q, k, v stage 1 (t = Vb^T (s2 * h))      the RMSNorm (and residual add) is redone by
//                                                      every block that needs h: one vector read
//                                                      and one block-wide sum
//   phase 2  q, k, v stage 2 (s1 * (Ub t) + bias)
//   phase 3  attention over the cache                  RoPE of q in the fragment loader; the block
//                                                      whose keys include the new position rotates
//                                                      k and appends k, v to the cache; the last
//                                                      split of a head group to finish (a ticket)
//                                                      combines the splits
//   phase 4, 5  o stages 1, 2
//   phase 6, 7  gate, up stages 1 (norm redone as in phase 1), 2
//   phase 8, 9  down stages 1 (SwiGLU in the loader), 2
// Every block prefetches the weight tiles of its first work item of the next phase BEFORE it
// waits at the barrier, so the DRAM latency of the weights hides behind the barrier.
//
// The linears run in the table-free direct form (qk_direct.cuh), the attention and the combine
// are the device functions of the stand-alone kernels (qk_decoder_dev.cuh), and norm, RoPE and
// SwiGLU repeat those kernels' arithmetic in the same order, so a step through this kernel
// gives the bits of the same step made of stand-alone launches with direct plans.
//
// Waiting is bounded: a barrier that does not complete within `wait_limit` polls sets bit 16 of
// the context's error word; the block then stops waiting at every later barrier (it still
// arrives, so the barrier count stays whole) and the kernel runs to its end with meaningless
// results; the next qk_gpu_synchronize reports QK_ERR_TIMEOUT.
#include <cmath>
#include <new>

#include "qk_common.h"
#include "qk_decoder_dev.cuh"
#include "qk_direct.cuh"

namespace {

constexpr int kStepThreads = qk_direct::kThreads;  // 512
constexpr int kSubBlocks = 2;                      // attention groups of 128 threads per CTA
constexpr int kSubSmemBytes = kMmaDecSmemBytes + (128 + 4 + 4) * 4;
constexpr uint32_t kStepWaitLimitDefault = 4u << 20;  // polls of ~0.5 us: seconds

struct StepLinear {
    const uint8_t *vbt_tiles, *ub_tiles;
    const float *s1, *s2, *bias;
    uint32_t r, din, dout;
};
enum { LIN_Q, LIN_K, LIN_V, LIN_O, LIN_GATE, LIN_UP, LIN_DOWN, LIN_COUNT };
struct StepLayer {
    StepLinear lin[LIN_COUNT];
    const float *in_norm, *post_norm;
    uint16_t *cache_k, *cache_v;
};

struct StepArgs {
    const StepLayer *layers;
    uint32_t n_layers, n_tok, d_model, n_heads, n_kv, d_ff, s_max, n_seq, n_splits, chunk, gq;
    float eps;
    float *x_a, *x_b;   // the residual stream alternates between the two
    float *t[3];        // intermediates of up to three linears, [n_tok][t_stride] each
    uint32_t t_stride;
    float *q, *k, *v, *attn, *delta_attn, *delta_mlp, *g, *u, *partial;
    const float *cos_sin;
    const int32_t *positions, *seq_index, *kv_len;
    unsigned long long *barrier;
    uint32_t *tickets;
    int *error;
    uint32_t wait_limit;
    uint32_t n_steps_max;  // widest linear input, in k-steps
};

// ---- grid barrier ---------------------------------------------------------------------
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long *p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
struct GridBarrier {
    unsigned long long *counter;
    unsigned long long target;  // the count that completes the next barrier
    uint32_t limit;
    int *error;
    int *gave_up;  // shared memory: this block no longer waits
};
// Every block arrives exactly once per barrier (also after it gave up waiting), so the counter
// is a whole multiple of the grid size between launches.
__device__ __forceinline__ void grid_sync(GridBarrier &gb) {
    __syncthreads();
    gb.target += gridDim.x;
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(gb.counter, 1ull);
        if (!*gb.gave_up) {
            uint32_t polls = 0;
            while (ld_acquire_u64(gb.counter) < gb.target) {
                if (++polls > gb.limit) {
                    atomicOr(gb.error, 16);
                    *gb.gave_up = 1;
                    break;
                }
            }
        }
    }
    __syncthreads();
}

// ---- the linears ------------------------------------------------------------------------
// One stage of one linear for all tokens.
struct LinJob {
    const uint8_t *tiles;
    uint32_t n_rows, n_bits;
    const float *in_scale;  // s2 of stage 1, null in stage 2
    const float *src;       // PLAIN: [n_tok][src_stride]
    uint32_t src_stride;
    float *out;             // [n_tok][out_stride]
    uint32_t out_stride;
    const float *out_scale, *out_bias;  // stage 2: s1 and bias
    bool final;
};
enum Loader { LOAD_PLAIN, LOAD_NORM, LOAD_SWIGLU };
struct NormSource {
    const float *x_in, *residual, *weight;  // residual may be null
    float *x_out;
};
struct StepSmem {
    float *y;        // [n_tok][d_model]: the normalised rows of the current phase
    float *norm_red; // [16]
    qk_direct::Smem direct;
    uint8_t *attn;   // [kSubBlocks][kSubSmemBytes], aliases everything above
};

// The RMSNorm of rmsnorm_kernel (qk_decoder.cu) for every token, by this block alone, into
// sm.y; `writer` also stores h = x + residual to x_out.  Same element-to-thread assignment and
// the same reductions as the stand-alone kernel, hence the same bits.
template <bool kBf16>
__device__ __forceinline__ void norm_rows(const StepArgs &a, const StepSmem &sm, const NormSource &ns, bool writer) {
    constexpr int kPer = 16;
    const uint32_t d = a.d_model;
    for (uint32_t tok = 0; tok < a.n_tok; ++tok) {
        const size_t base = (size_t)tok * d;
        float keep[kPer];
        float ss = 0.f;
#pragma unroll
        for (int r = 0; r < kPer; ++r) {
            const uint32_t i = threadIdx.x + r * kStepThreads;
            float h = 0.f;
            if (i < d) {
                h = __ldcg(ns.x_in + base + i);
                if (ns.residual) h += __ldcg(ns.residual + base + i);
                if (writer) ns.x_out[base + i] = h;
                if (kBf16) h = round_bf16f(h);
            }
            keep[r] = h;
            ss += h * h;
        }
        const float inv = 1.0f / sqrtf(block_sum(ss, sm.norm_red) / (float)d + a.eps);
#pragma unroll
        for (int r = 0; r < kPer; ++r) {
            const uint32_t i = threadIdx.x + r * kStepThreads;
            if (i < d) {
                float o = keep[r] * inv * ns.weight[i];
                if (kBf16) o = round_bf16f(o);
                sm.y[base + i] = o;
            }
        }
    }
    __syncthreads();
}

// A phase of up to three jobs that share a loader.  `gb`: the barrier that separates this
// phase from the one before (null for the very first phase of the kernel).
template <bool kBf16>
__device__ __forceinline__ void linear_phase(const StepArgs &a, const StepSmem &sm, const LinJob *jobs, int n_jobs,
                                             Loader loader, const NormSource &ns, const float *gate,
                                             const float *up, uint32_t gu_stride, GridBarrier *gb) {
    constexpr int kN = qk_direct::Terms<kBf16>::kN;
    uint32_t first[4] = {0, 0, 0, 0};
    for (int j = 0; j < n_jobs; ++j)
        first[j + 1] = first[j] + (jobs[j].n_rows + qk_direct::kGroupRows - 1) / qk_direct::kGroupRows;
    const uint32_t total = first[n_jobs];
    // a balanced contiguous share of the items: a block's items mostly belong to one job
    const uint32_t begin = (uint32_t)((uint64_t)blockIdx.x * total / gridDim.x);
    const uint32_t end = (uint32_t)((uint64_t)(blockIdx.x + 1) * total / gridDim.x);
    auto job_of = [&](uint32_t item) {
        int j = 0;
        while (j + 1 < n_jobs && item >= first[j + 1]) ++j;
        return j;
    };
    auto work_of = [&](uint32_t item, int j) {
        return qk_direct::Work{jobs[j].tiles, (jobs[j].n_bits + qk_direct::kStepBits - 1) / qk_direct::kStepBits,
                               item - first[j]};
    };
    if (begin < end) qk_direct::prefetch(sm.direct, work_of(begin, job_of(begin)));
    if (gb) grid_sync(*gb);
    if (begin >= end) return;
    if (loader == LOAD_NORM) norm_rows<kBf16>(a, sm, ns, begin == 0);
    int staged = -1;
    for (uint32_t item = begin; item < end; ++item) {
        const int j = job_of(item);
        const LinJob &job = jobs[j];
        const qk_direct::Work work = work_of(item, j);
        if (item != begin) qk_direct::prefetch(sm.direct, work);
        if (j != staged) {
            const uint32_t padded = work.n_steps * qk_direct::kStepBits;
            for (uint32_t tok = 0; tok < a.n_tok; ++tok)
                for (uint32_t k = threadIdx.x; k < padded; k += kStepThreads) {
                    float v = 0.f;
                    if (k < job.n_bits) {
                        if (loader == LOAD_NORM) {
                            v = sm.y[(size_t)tok * a.d_model + k];
                        } else if (loader == LOAD_SWIGLU) {
                            const float gv = __ldcg(gate + (size_t)tok * gu_stride + k);
                            v = gv * __ldcg(up + (size_t)tok * gu_stride + k) / (1.0f + expf(-gv));
                        } else {
                            v = __ldcg(job.src + (size_t)tok * job.src_stride + k);
                        }
                        if (job.in_scale) v = job.in_scale[k] * v;
                    }
                    qk_direct::stage_value<kBf16>(sm.direct, tok, k, v);
                }
            __syncthreads();
            staged = j;
        }
        qk_direct::multiply(sm.direct, work, a.n_tok * kN);
        if (threadIdx.x < qk_direct::kGroupRows * a.n_tok) {
            const uint32_t r64 = threadIdx.x % qk_direct::kGroupRows, tok = threadIdx.x / qk_direct::kGroupRows;
            float sum = qk_direct::gather<kBf16>(sm.direct, r64, tok);
            const uint32_t row = work.group * qk_direct::kGroupRows + r64;
            if (row < job.n_rows) {
                if (kBf16) sum = round_bf16f(sum);
                if (job.final) {
                    if (job.out_scale) sum = sum * job.out_scale[row];
                    if (job.out_bias) sum = sum + job.out_bias[row];
                }
                job.out[(size_t)tok * job.out_stride + row] = sum;
            }
        }
        __syncthreads();  // the partial sums and the columns may be overwritten
    }
}

__device__ __forceinline__ LinJob stage1_job(const StepLinear &l, const float *src, uint32_t src_stride, float *t,
                                             uint32_t t_stride) {
    return LinJob{l.vbt_tiles, l.r, l.din, l.s2, src, src_stride, t, t_stride, nullptr, nullptr, false};
}
__device__ __forceinline__ LinJob stage2_job(const StepLinear &l, const float *t, uint32_t t_stride, float *out,
                                             uint32_t out_stride) {
    return LinJob{l.ub_tiles, l.dout, l.r, nullptr, t, t_stride, out, out_stride, l.s1, l.bias, true};
}

// ---- the attention phase ---------------------------------------------------------------
__device__ __forceinline__ void attention_groups(const StepArgs &a, const StepSmem &sm, const StepLayer &L,
                                                 uint32_t sub) {
    const SubBlock sb{threadIdx.x % 128, 1 + sub};
    uint8_t *mine = sm.attn + (size_t)sub * kSubSmemBytes;
    const DecAttnSmem asm_ = carve_dec_attn(mine);
    float *wgt = reinterpret_cast<float *>(mine + kMmaDecSmemBytes), *red = wgt + 128;
    int *is_last = reinterpret_cast<int *>(red + 4);
    const uint32_t group = a.n_heads / a.n_kv, subs = (group + a.gq - 1) / a.gq;
    const uint32_t per_seq = a.n_splits * a.n_kv * subs, total = per_seq * a.n_tok;
    for (uint32_t vb = sub * gridDim.x + blockIdx.x; vb < total; vb += kSubBlocks * gridDim.x) {
        const uint32_t split = vb % a.n_splits, ky = (vb / a.n_splits) % (a.n_kv * subs), b = vb / per_seq;
        const int pos = a.positions[b], seq = a.seq_index[b];
        const bool valid = pos >= 0 && (uint32_t)pos < a.s_max && seq >= 0 && (uint32_t)seq < a.n_seq;
        if (!valid && sb.tid == 0) atomicOr(a.error, 4);  // reported like rope_cache_kernel does
        const int pos_in = min(max(pos, 0), (int)a.s_max - 1);
        const FreshKey fresh{a.k, a.v, L.cache_k, L.cache_v, a.cos_sin + (size_t)pos_in * 128, pos, seq, valid};
        decode_attention_mma_body<true>(sb, asm_, a.q, L.cache_k, L.cache_v, a.kv_len[b], a.partial, a.n_heads,
                                        a.n_kv, a.gq, a.s_max, a.chunk, a.n_splits, split, ky, b, fresh);
        // the last split of this (sequence, kv-head block) to finish combines them
        __threadfence();
        sb.sync();
        if (sb.tid == 0) {
            uint32_t *ticket = a.tickets + (size_t)b * a.n_kv * subs + ky;
            const uint32_t old = atomicAdd(ticket, 1u);
            *is_last = old == a.n_splits - 1;
            if (*is_last) *ticket = 0;
        }
        sb.sync();
        if (*is_last) {
            __threadfence();
            const uint32_t kvh = ky / subs, hsub = ky % subs, h0 = kvh * group + hsub * a.gq;
            const uint32_t rows = min(a.gq, group - hsub * a.gq);
            for (uint32_t r = 0; r < rows; ++r) {
                const size_t head = (size_t)b * a.n_heads + h0 + r;
                decode_combine_body(sb, wgt, red, a.partial + head * a.n_splits * 130, a.attn + head * 128, 128,
                                    a.n_splits);
            }
        }
        sb.sync();  // is_last and the staging buffers are free again
    }
}

__device__ __forceinline__ void attention_phase(const StepArgs &a, const StepSmem &sm, const StepLayer &L,
                                                GridBarrier &gb) {
    grid_sync(gb);
    const uint32_t sub = threadIdx.x / 128;
    if (sub < kSubBlocks) attention_groups(a, sm, L, sub);
    // the other warps go on to the next phase, whose weight prefetch lands in shared memory the
    // groups are using: hold them here
    __syncthreads();
}

// ---- the kernel --------------------------------------------------------------------------
template <bool kBf16>
__global__ void __launch_bounds__(kStepThreads, 1)
decode_blocks_kernel(const StepArgs a) {
    extern __shared__ __align__(128) uint8_t step_smem[];
    __shared__ int gave_up;
    constexpr int kN = qk_direct::Terms<kBf16>::kN;
    StepSmem sm;
    sm.y = reinterpret_cast<float *>(step_smem);
    sm.norm_red = sm.y + (size_t)a.n_tok * a.d_model;
    sm.direct = qk_direct::carve(reinterpret_cast<uint8_t *>(sm.norm_red + 32), a.n_steps_max, a.n_tok * kN);
    sm.attn = step_smem;
    if (threadIdx.x == 0) gave_up = 0;
    GridBarrier gb{a.barrier, 0, a.wait_limit, a.error, &gave_up};
    // (the counter is a whole multiple of the grid size between launches; a block that reads it
    // after others have arrived at the first barrier still rounds down to the same base)
    gb.target = ld_acquire_u64(a.barrier) / gridDim.x * gridDim.x;
    __syncthreads();

    float *x_in = a.x_a, *x_out = a.x_b;
    const NormSource none{};
    for (uint32_t li = 0; li < a.n_layers; ++li) {
        const StepLayer &L = a.layers[li];
        const uint32_t dq = a.n_heads * 128, dkv = a.n_kv * 128;
        {   // q, k, v: stage 1 behind the input norm, stage 2
            const NormSource ns{x_in, li ? a.delta_mlp : nullptr, L.in_norm, x_out};
            const LinJob s1[3] = {stage1_job(L.lin[LIN_Q], nullptr, 0, a.t[0], a.t_stride),
                                  stage1_job(L.lin[LIN_K], nullptr, 0, a.t[1], a.t_stride),
                                  stage1_job(L.lin[LIN_V], nullptr, 0, a.t[2], a.t_stride)};
            linear_phase<kBf16>(a, sm, s1, 3, LOAD_NORM, ns, nullptr, nullptr, 0, li ? &gb : nullptr);
            const LinJob s2[3] = {stage2_job(L.lin[LIN_Q], a.t[0], a.t_stride, a.q, dq),
                                  stage2_job(L.lin[LIN_K], a.t[1], a.t_stride, a.k, dkv),
                                  stage2_job(L.lin[LIN_V], a.t[2], a.t_stride, a.v, dkv)};
            linear_phase<kBf16>(a, sm, s2, 3, LOAD_PLAIN, none, nullptr, nullptr, 0, &gb);
            float *tmp = x_in; x_in = x_out; x_out = tmp;
        }
        attention_phase(a, sm, L, gb);
        {   // o
            const LinJob s1[1] = {stage1_job(L.lin[LIN_O], a.attn, dq, a.t[0], a.t_stride)};
            linear_phase<kBf16>(a, sm, s1, 1, LOAD_PLAIN, none, nullptr, nullptr, 0, &gb);
            const LinJob s2[1] = {stage2_job(L.lin[LIN_O], a.t[0], a.t_stride, a.delta_attn, a.d_model)};
            linear_phase<kBf16>(a, sm, s2, 1, LOAD_PLAIN, none, nullptr, nullptr, 0, &gb);
        }
        {   // gate, up behind the post-attention norm
            const NormSource ns{x_in, a.delta_attn, L.post_norm, x_out};
            const LinJob s1[2] = {stage1_job(L.lin[LIN_GATE], nullptr, 0, a.t[0], a.t_stride),
                                  stage1_job(L.lin[LIN_UP], nullptr, 0, a.t[1], a.t_stride)};
            linear_phase<kBf16>(a, sm, s1, 2, LOAD_NORM, ns, nullptr, nullptr, 0, &gb);
            const LinJob s2[2] = {stage2_job(L.lin[LIN_GATE], a.t[0], a.t_stride, a.g, a.d_ff),
                                  stage2_job(L.lin[LIN_UP], a.t[1], a.t_stride, a.u, a.d_ff)};
            linear_phase<kBf16>(a, sm, s2, 2, LOAD_PLAIN, none, nullptr, nullptr, 0, &gb);
            float *tmp = x_in; x_in = x_out; x_out = tmp;
        }
        {   // down behind the SwiGLU
            const LinJob s1[1] = {stage1_job(L.lin[LIN_DOWN], nullptr, 0, a.t[0], a.t_stride)};
            linear_phase<kBf16>(a, sm, s1, 1, LOAD_SWIGLU, none, a.g, a.u, a.d_ff, &gb);
            const LinJob s2[1] = {stage2_job(L.lin[LIN_DOWN], a.t[0], a.t_stride, a.delta_mlp, a.d_model)};
            linear_phase<kBf16>(a, sm, s2, 1, LOAD_PLAIN, none, nullptr, nullptr, 0, &gb);
        }
    }
}

size_t step_smem_bytes(const StepArgs &a, bool bf16) {
    const size_t linear = ((size_t)a.n_tok * a.d_model + 32) * sizeof(float) +
                          qk_direct::smem_bytes(a.n_steps_max, a.n_tok * (bf16 ? 1 : 3));
    const size_t attention = (size_t)kSubBlocks * kSubSmemBytes;
    return linear > attention ? linear : attention;
}

}  // namespace

struct qk_decode_step {
    int device = 0;
    bool bf16 = false;
    StepArgs args{};
    size_t smem = 0;
    int grid = 0;
    void *d_layers = nullptr, *d_t = nullptr, *d_sync = nullptr;
};

extern "C" {

qk_status qk_decode_step_create(qk_ctx *ctx, const qk_step_desc *desc, qk_decode_step **out) {
    if (!desc || !out) return qk::fail(QK_ERR_VALUE, "qk_decode_step_create: desc and out must not be null");
    *out = nullptr;
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    if (desc->n_blocks == 0 || desc->n_tokens == 0 || !desc->blocks)
        return qk::fail(QK_ERR_VALUE, "a decode step needs at least one block and one token");
    if (desc->head_dim != 128 || desc->kv_dtype != QK_BF16)
        return qk::fail(QK_ERR_VALUE, "the whole-step kernel needs head_dim 128 and a bfloat16 KV cache, got "
                        "head_dim %zu, cache tag %d", desc->head_dim, desc->kv_dtype);
    if (desc->serving_dtype != QK_F32 && desc->serving_dtype != QK_BF16)
        return qk::fail(QK_ERR_VALUE, "serving dtype must be float32 or bfloat16, got tag %d", desc->serving_dtype);
    const bool bf16 = desc->serving_dtype == QK_BF16;
    if (desc->n_tokens * (bf16 ? 1 : 3) > (size_t)qk_direct::kMaxCols)
        return qk::fail(QK_ERR_VALUE, "the whole-step kernel takes at most %d tokens under %s serving, got %zu",
                        qk_direct::kMaxCols / (bf16 ? 1 : 3), bf16 ? "bfloat16" : "float32", desc->n_tokens);
    if (desc->n_kv_heads == 0 || desc->n_heads % desc->n_kv_heads != 0)
        return qk::fail(QK_ERR_VALUE, "n_kv_heads must divide n_heads: n_heads=%zu, n_kv_heads=%zu",
                        desc->n_heads, desc->n_kv_heads);
    if (desc->n_splits == 0 || desc->n_splits > 128)
        return qk::fail(QK_ERR_VALUE, "between 1 and 128 key splits are supported, got %zu", desc->n_splits);
    if (desc->d_model > 16 * (size_t)kStepThreads || desc->d_model % 8 != 0)
        return qk::fail(QK_ERR_VALUE, "d_model must be a multiple of 8 and at most %d, got %zu", 16 * kStepThreads,
                        desc->d_model);
    const qk_step_buffers &b = desc->buf;
    if (!b.x || !b.x2 || !b.q || !b.k || !b.v || !b.attn || !b.delta_attn || !b.delta_mlp || !b.gate || !b.up ||
        !b.att_scratch || !b.cos_sin || !b.positions || !b.seq_index || !b.kv_len)
        return qk::fail(QK_ERR_VALUE, "qk_decode_step_create: every buffer of the step must be given");
    const size_t dq = desc->n_heads * 128, dkv = desc->n_kv_heads * 128;
    std::vector<StepLayer> layers(desc->n_blocks);
    size_t r_max = 0, steps_max = 0;
    for (size_t i = 0; i < desc->n_blocks; ++i) {
        const qk_step_block &blk = desc->blocks[i];
        const qk_layer *lin[LIN_COUNT] = {blk.q, blk.k, blk.v, blk.o, blk.gate, blk.up, blk.down};
        const size_t want_out[LIN_COUNT] = {dq, dkv, dkv, desc->d_model, desc->d_ff, desc->d_ff, desc->d_model};
        const size_t want_in[LIN_COUNT] = {desc->d_model, desc->d_model, desc->d_model, dq, desc->d_model,
                                           desc->d_model, desc->d_ff};
        for (int j = 0; j < LIN_COUNT; ++j) {
            const qk_layer *l = lin[j];
            if (!l) return qk::fail(QK_ERR_VALUE, "block %zu: linear %d is null", i, j);
            if (l->device != c->device)
                return qk::fail(QK_ERR_VALUE, "block %zu: a layer lives on device %d, the context on %d", i,
                                l->device, c->device);
            if (l->serving != desc->serving_dtype)
                return qk::fail(QK_ERR_VALUE, "block %zu: the layers must share the step's serving dtype", i);
            if (l->dout != want_out[j] || l->din != want_in[j])
                return qk::fail(QK_ERR_VALUE, "block %zu: linear %d is %zu x %zu, the step expects %zu x %zu", i, j,
                                l->dout, l->din, want_out[j], want_in[j]);
            layers[i].lin[j] = StepLinear{l->vbt_tiles, l->ub_tiles, l->s1, l->s2, l->bias, (uint32_t)l->r,
                                          (uint32_t)l->din, (uint32_t)l->dout};
            r_max = l->r > r_max ? l->r : r_max;
            const size_t steps = qk::ceil_div(l->din > l->r ? l->din : l->r, qk_direct::kStepBits);
            steps_max = steps > steps_max ? steps : steps_max;
        }
        if (!blk.input_norm || !blk.post_norm || !blk.cache_k || !blk.cache_v)
            return qk::fail(QK_ERR_VALUE, "block %zu: norm weights and caches must be given", i);
        layers[i].in_norm = blk.input_norm;
        layers[i].post_norm = blk.post_norm;
        layers[i].cache_k = (uint16_t *)blk.cache_k;
        layers[i].cache_v = (uint16_t *)blk.cache_v;
    }
    qk_decode_step *s = new (std::nothrow) qk_decode_step();
    if (!s) return qk::fail(QK_ERR_CUDA, "out of host memory");
    s->device = c->device;
    s->bf16 = bf16;
    auto bail = [&](qk_status code) {
        cudaFree(s->d_layers);
        cudaFree(s->d_t);
        cudaFree(s->d_sync);
        delete s;
        return code;
    };
    StepArgs &a = s->args;
    const size_t group = desc->n_heads / desc->n_kv_heads, gq = group < 8 ? group : 8, subs = qk::ceil_div(group, gq);
    const size_t t_stride = qk::ceil_div(r_max, 64) * 64;
    const size_t n_tickets = desc->n_tokens * desc->n_kv_heads * subs;
    if (cudaMalloc(&s->d_layers, layers.size() * sizeof(StepLayer)) != cudaSuccess ||
        cudaMalloc(&s->d_t, 3 * desc->n_tokens * t_stride * sizeof(float)) != cudaSuccess ||
        cudaMalloc(&s->d_sync, 256 + n_tickets * sizeof(uint32_t)) != cudaSuccess)
        return bail(qk::fail(QK_ERR_CUDA, "qk_decode_step_create: device allocation failed: %s",
                             cudaGetErrorString(cudaGetLastError())));
    if (cudaMemcpyAsync(s->d_layers, layers.data(), layers.size() * sizeof(StepLayer), cudaMemcpyHostToDevice,
                        c->stream) != cudaSuccess ||
        cudaMemsetAsync(s->d_sync, 0, 256 + n_tickets * sizeof(uint32_t), c->stream) != cudaSuccess ||
        cudaMemsetAsync(s->d_t, 0, 3 * desc->n_tokens * t_stride * sizeof(float), c->stream) != cudaSuccess ||
        cudaStreamSynchronize(c->stream) != cudaSuccess)
        return bail(qk::fail(QK_ERR_CUDA, "qk_decode_step_create: upload failed: %s",
                             cudaGetErrorString(cudaGetLastError())));
    a.layers = (const StepLayer *)s->d_layers;
    a.n_layers = (uint32_t)desc->n_blocks;
    a.n_tok = (uint32_t)desc->n_tokens;
    a.d_model = (uint32_t)desc->d_model;
    a.n_heads = (uint32_t)desc->n_heads;
    a.n_kv = (uint32_t)desc->n_kv_heads;
    a.d_ff = (uint32_t)desc->d_ff;
    a.s_max = (uint32_t)desc->s_max;
    a.n_seq = (uint32_t)desc->n_seq;
    a.n_splits = (uint32_t)desc->n_splits;
    a.chunk = (uint32_t)qk::ceil_div(desc->s_max, desc->n_splits);
    a.gq = (uint32_t)gq;
    a.eps = desc->rms_eps;
    a.x_a = b.x;
    a.x_b = b.x2;
    for (int j = 0; j < 3; ++j) a.t[j] = (float *)s->d_t + (size_t)j * desc->n_tokens * t_stride;
    a.t_stride = (uint32_t)t_stride;
    a.q = b.q, a.k = b.k, a.v = b.v, a.attn = b.attn;
    a.delta_attn = b.delta_attn, a.delta_mlp = b.delta_mlp, a.g = b.gate, a.u = b.up, a.partial = b.att_scratch;
    a.cos_sin = b.cos_sin;
    a.positions = b.positions, a.seq_index = b.seq_index, a.kv_len = b.kv_len;
    a.barrier = (unsigned long long *)s->d_sync;
    a.tickets = (uint32_t *)((uint8_t *)s->d_sync + 256);
    a.n_steps_max = (uint32_t)steps_max;
    s->smem = step_smem_bytes(a, bf16);
    if (s->smem > 227 * 1024)
        return bail(qk::fail(QK_ERR_VALUE, "the step needs %zu bytes of shared memory per block, more than the "
                             "227 KB a block can have (widest linear input: %zu k-steps)", s->smem, steps_max));
    auto kern = bf16 ? decode_blocks_kernel<true> : decode_blocks_kernel<false>;
    int per_sm = 0;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)s->smem) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kStepThreads, s->smem) != cudaSuccess ||
        per_sm < 1)
        return bail(qk::fail(QK_ERR_CUDA, "the whole-step kernel cannot be made resident: %s",
                             cudaGetErrorString(cudaGetLastError())));
    s->grid = c->sm_count;
    *out = s;
    return QK_OK;
}

qk_status qk_decode_step_run(qk_ctx *ctx, const qk_decode_step *step) {
    if (!step) return qk::fail(QK_ERR_VALUE, "qk_decode_step_run: step is null");
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    if (step->device != c->device)
        return qk::fail(QK_ERR_VALUE, "the step lives on device %d, the context on %d", step->device, c->device);
    if ((st = qk::error_word(c)) != QK_OK) return st;
    StepArgs a = step->args;
    a.error = (int *)c->d_err.ptr;
    a.wait_limit = c->wait_limit ? c->wait_limit : kStepWaitLimitDefault;
    auto kern = step->bf16 ? decode_blocks_kernel<true> : decode_blocks_kernel<false>;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)step->grid);
    cfg.blockDim = dim3(kStepThreads);
    cfg.dynamicSmemBytes = step->smem;
    cfg.stream = c->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // all blocks resident at once: they wait on one another
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    QK_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
    c->launches++;
    return QK_OK;
}

void qk_decode_step_free(qk_decode_step *step) {
    if (!step) return;
    cudaFree(step->d_layers);
    cudaFree(step->d_t);
    cudaFree(step->d_sync);
    delete step;
}

}  // extern "C"
