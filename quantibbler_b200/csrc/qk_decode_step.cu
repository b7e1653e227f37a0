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
// The linears are the bit-sliced INT8 tensor-core form of qk_gemv.cu (exact integer sums; the
// block builds the digit table of its input vector in shared memory), the attention and the
// combine are the device functions of the stand-alone kernels (qk_decoder_dev.cuh), and norm,
// RoPE and SwiGLU repeat those kernels' arithmetic in the same order, so a step through this
// kernel gives the bits of the same step made of stand-alone launches.
//
// Waiting is bounded: a barrier that does not complete within `wait_limit` polls sets bit 16 of
// the context's error word; the block then stops waiting at every later barrier (it still
// arrives, so the barrier count stays whole) and the kernel runs to its end with meaningless
// results; the next qk_gpu_synchronize reports QK_ERR_TIMEOUT.
#include <cmath>
#include <initializer_list>
#include <new>
#include <utility>

#include "qk_common.h"
#include "qk_decoder_dev.cuh"
#include "qk_digits.cuh"

namespace {

constexpr int kStepThreads = 256;                  // 8 warps = 2 k-lanes x 4 row tiles (and two attention
                                                   // groups); 255 registers per thread, so nothing spills
constexpr int kKLanes = 2, kGroupTiles = 4;
constexpr int kNormThreads = 512, kNormPer = 16;   // the stand-alone norm kernel's geometry, reproduced here
constexpr int kRingStages = 3;                     // tiles in flight per warp
constexpr int kTileBytes = 1024, kChunkBytes = kGroupTiles * kTileBytes, kGroupRows = 64;
constexpr int kSubBlocks = 2;                      // attention groups of 128 threads per CTA
constexpr int kSubAttnBufs = 2;                    // staging buffers per warp of an attention group
constexpr int kSubAttnBytes = dec_attn_smem_bytes(kSubAttnBufs);
constexpr int kSubSmemBytes = kSubAttnBytes + 16;
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

struct PhaseDesc;
struct StepArgs {
    const PhaseDesc *phases;
    uint32_t n_phases, n_tok, d_model, n_heads, n_kv, d_ff, s_max, n_seq, n_splits, chunk, gq;
    float eps;
    float *q, *k, *v, *attn, *partial;
    const float *cos_sin;
    const int32_t *positions, *seq_index, *kv_len;
    unsigned long long *barrier;
    uint32_t *tickets;
    int *error;
    uint32_t wait_limit;
    uint32_t n_steps_max;  // widest linear input, in k-steps
    uint32_t vec_bytes;    // widest staged input vector
    unsigned long long *stamps;  // trace: %globaltimer of block 0 at kernel start and after every barrier
    uint32_t stamps_cap;
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
    unsigned long long *stamps;
    uint32_t stamps_cap, n_stamps;
};
__device__ __forceinline__ void stamp(GridBarrier &gb) {
    if (gb.stamps && blockIdx.x == 0 && threadIdx.x == 0 && gb.n_stamps < gb.stamps_cap) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        gb.stamps[gb.n_stamps++] = t;
    }
}
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
    stamp(gb);
    __syncthreads();
}

// Trace of the inside of a phase: entry `slot` of phase `phase` in the upper half of the stamp buffer.
__device__ __forceinline__ void sub_stamp(const StepArgs &a, uint32_t phase, int slot, bool who) {
    if (a.stamps && who && threadIdx.x % 128 == 0) {
        const uint32_t at = a.stamps_cap / 2 + phase * 8 + slot;
        if (at < a.stamps_cap) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            a.stamps[at] = t;
        }
    }
}

// ---- the linears ------------------------------------------------------------------------
// One stage of one linear for all tokens.
struct LinJob {
    const uint8_t *tiles;
    uint32_t n_rows, n_bits;
    const float *in_scale;  // s2 of stage 1, null in stage 2
    const void *src;        // PLAIN: float32 (stage 1) or float64 t (stage 2), [n_tok][src_stride]
    uint32_t src_stride;
    void *out;              // float64 t (stage 1) or float32 (stage 2), [n_tok][out_stride]
    uint32_t out_stride;
    const float *out_scale, *out_bias;  // stage 2: s1 and bias
    bool final;
};
enum Loader { LOAD_PLAIN, LOAD_NORM, LOAD_SWIGLU };
struct NormSource {
    const float *x_in, *residual, *weight;  // residual may be null
    float *x_out;
};
// One phase of the step, prepared by the host: up to three jobs behind one loader, or the
// attention of one block of the model.
enum { PHASE_LINEAR, PHASE_ATTENTION };
struct PhaseDesc {
    int kind, n_jobs, loader;
    LinJob jobs[3];
    NormSource ns;
    const float *gate, *up;  // LOAD_SWIGLU: [n_tok][gu_stride]
    uint32_t gu_stride;
    uint16_t *cache_k, *cache_v;  // PHASE_ATTENTION
};
struct StepSmem {
    uint8_t *vec;      // the staged input vector: float32[n_bits] (stage 1) or float64[n_bits] (stage 2)
    uint8_t *table;    // its digit table, 4 KB per k-step
    uint8_t *ring;     // [warp][kRingStages][kTileBytes]
    int *red;          // [k-lane][tile][4][32]: the warps' accumulator fragments
    double *red_max;   // [32]
    long long *red_sum;  // [32]
    int *red_bad;
    StageMeta *meta;
    float *norm_red;   // [16]
    uint8_t *attn;     // [kSubBlocks][kSubSmemBytes], aliases everything above
};
__host__ __device__ inline size_t round128(size_t n) { return (n + 127) / 128 * 128; }
// vec_bytes: the widest staged vector (4 bytes per stage-1 input element, 8 per rank element)
__device__ __forceinline__ StepSmem carve_step(uint8_t *base, uint32_t vec_bytes, uint32_t n_steps_max) {
    StepSmem sm;
    sm.attn = base;
    sm.vec = base;
    sm.table = sm.vec + round128(vec_bytes);
    sm.ring = sm.table + (size_t)n_steps_max * 4096;
    sm.red = reinterpret_cast<int *>(sm.ring + (size_t)(kStepThreads / 32) * kRingStages * kTileBytes);
    sm.red_max = reinterpret_cast<double *>(sm.red + kKLanes * kGroupTiles * 4 * 32);
    sm.red_sum = reinterpret_cast<long long *>(sm.red_max + 32);
    sm.meta = reinterpret_cast<StageMeta *>(sm.red_sum + 32);
    sm.norm_red = reinterpret_cast<float *>(sm.meta + 1);
    sm.red_bad = reinterpret_cast<int *>(sm.norm_red + kNormThreads / 32);
    return sm;
}
size_t linear_smem_bytes(uint32_t vec_bytes, uint32_t n_steps_max) {
    return round128(vec_bytes) + (size_t)n_steps_max * 4096 + (size_t)(kStepThreads / 32) * kRingStages * kTileBytes +
           kKLanes * kGroupTiles * 4 * 32 * 4 + 32 * 8 + 32 * 8 + sizeof(StageMeta) + 16 * 4 + 16;
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
__device__ __forceinline__ void prefetch_l2(const void *p) {
    asm volatile("prefetch.global.L2 [%0];" ::"l"(p));
}
// Asks for n floats at p to be brought into L2 (one request per 128 bytes).
__device__ __forceinline__ void prefetch_floats(const float *p, uint32_t n) {
    if (p)
        for (uint32_t k = 32 * threadIdx.x; k < n; k += 32 * kStepThreads) prefetch_l2(p + k);
}
__device__ __forceinline__ void mma_u8s8(int (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm("mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};\n"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// One row group (64 rows) of one packed factor: tiles of 16 rows x 512 bits, four per 4 KB
// chunk, chunks ordered [group][k-step].  Warp w owns tile w % 4 of the group and the k-steps
// w / 4, w / 4 + 4, ... and streams its 1 KB tiles through a private ring.
struct Work {
    const uint8_t *tiles;
    uint32_t n_steps, group;
};
__device__ __forceinline__ uint32_t warp_items(uint32_t n_steps) {
    const uint32_t kl = (threadIdx.x / 32) / kGroupTiles;
    return kl < n_steps ? (n_steps - kl + kKLanes - 1) / kKLanes : 0;
}
__device__ __forceinline__ void issue_tile(const StepSmem &sm, const Work &w, uint32_t i, uint32_t n_items) {
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t m = warp % kGroupTiles, kl = warp / kGroupTiles;
    if (i < n_items) {
        uint4 *dst = reinterpret_cast<uint4 *>(sm.ring + ((size_t)warp * kRingStages + i % kRingStages) * kTileBytes) + lane;
        const uint4 *from = reinterpret_cast<const uint4 *>(w.tiles) +
                            ((size_t)w.group * w.n_steps + kl + (size_t)i * kKLanes) * (kChunkBytes / 16) +
                            m * (kTileBytes / 16) + lane;
        cp16(dst, from);            // row g:     bits 128 t .. 128 t + 127 of the k-step
        cp16(dst + 32, from + 32);  // row g + 8
    }
    cp_commit();  // (an empty group keeps the group count in step with i)
}
__device__ __forceinline__ void prefetch_tiles(const StepSmem &sm, const Work &w) {
    const uint32_t n_items = warp_items(w.n_steps);
#pragma unroll
    for (int st = 0; st < kRingStages - 1; ++st) issue_tile(sm, w, st, n_items);
}

// The row group against the digit table in sm.table (gemv_bitslice's inner loop, one tile per
// warp), the k-lanes' integer partial sums added through shared memory, and the exact
// recombination of bitslice_stage: with X = sum_n c_n 256^n = 128 S and T = sum q_k the row's
// value is (X - 64 T) / 64 * 2^-shift, X - 64 T formed exactly in int64.
// row_scale, row_bias: s1 and bias of the row this lane finishes (warps 0..3, lanes t < 2).
template <bool kBf16>
__device__ __forceinline__ void multiply_and_finish(const StepSmem &sm, const Work &w, const LinJob &job,
                                                    uint32_t tok, float row_scale, float row_bias) {
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const uint32_t m = warp % kGroupTiles, kl = warp / kGroupTiles;
    const uint32_t g = lane / 4, t = lane % 4;
    const uint32_t n_items = warp_items(w.n_steps);
    // two accumulator chains: consecutive MMAs do not wait for one another (integer sums: any order)
    int acc[4] = {0, 0, 0, 0}, acc2[4] = {0, 0, 0, 0};
    const uint2 *dig = reinterpret_cast<const uint2 *>(sm.table) + t * 8 + g;
    const uint4 *ring = reinterpret_cast<const uint4 *>(sm.ring + (size_t)warp * kRingStages * kTileBytes) + lane;
    for (uint32_t i = 0; i < n_items; ++i) {
        issue_tile(sm, w, i + kRingStages - 1, n_items);
        cp_wait<kRingStages - 1>();
        const uint4 *stage = ring + (size_t)(i % kRingStages) * (kTileBytes / 16);
        const uint4 lo = stage[0], hi = stage[32];
        const uint2 *dk = dig + (size_t)(kl + i * kKLanes) * 512;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const uint32_t wg = q == 0 ? lo.x : q == 1 ? lo.y : q == 2 ? lo.z : lo.w;
            const uint32_t wh = q == 0 ? hi.x : q == 1 ? hi.y : q == 2 ? hi.z : hi.w;
#pragma unroll
            for (int ip = 0; ip < 4; ++ip) {
                const uint2 b = dk[(q * 4 + ip) * 32];
                const uint32_t m0 = 0x01010101u << (2 * ip), m1 = m0 << 1;
                if (ip % 2) mma_u8s8(acc2, wg & m0, wh & m0, wg & m1, wh & m1, b.x, b.y);
                else mma_u8s8(acc, wg & m0, wh & m0, wg & m1, wh & m1, b.x, b.y);
            }
        }
    }
    cp_wait<0>();
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[e] += acc2[e];
#pragma unroll
    for (int e = 0; e < 4; ++e) sm.red[((kl * kGroupTiles + m) * 4 + e) * 32 + lane] = acc[e];
    __syncthreads();
    if (warp < kGroupTiles) {  // warp `warp` finishes tile `warp`
        int a[4] = {0, 0, 0, 0};
#pragma unroll
        for (int k2 = 0; k2 < kKLanes; ++k2)
#pragma unroll
            for (int e = 0; e < 4; ++e) a[e] += sm.red[((k2 * kGroupTiles + warp) * 4 + e) * 32 + lane];
        const StageMeta meta = *sm.meta;
        const long long th = meta.total >> 26, tl = (meta.total & ((1ll << 26) - 1)) << 6;
        const int sh0 = 16 * (t & 1);
        const int oexp = -meta.shift - 6;
        const bool odirect = oexp > -1000 && oexp < 1000;
        const double oscale = odirect ? __hiloint2double((1023 + oexp) << 20, 0) : 0.0;
        long long pg = ((long long)a[0] << sh0) + ((long long)a[1] << (sh0 + 8));
        long long ph = ((long long)a[2] << sh0) + ((long long)a[3] << (sh0 + 8));
        pg += __shfl_xor_sync(0xffffffffu, pg, 1);  // t=0,1: low half; t=2,3: high half
        ph += __shfl_xor_sync(0xffffffffu, ph, 1);
        const long long og = __shfl_xor_sync(0xffffffffu, pg, 2);
        const long long oh = __shfl_xor_sync(0xffffffffu, ph, 2);
        const uint32_t row = w.group * kGroupRows + warp * 16 + g + 8 * t;
        if (t < 2 && row < job.n_rows) {
            const long long lo = t == 0 ? pg : ph, hi = t == 0 ? og : oh;
            double val = (double)(hi - th) * 4294967296.0 + (double)(lo - tl);
            val = odirect ? val * oscale : ldexp(val, oexp);
            if (meta.nonfinite) val = nan("");
            if (kBf16) val = (double)round_bf16((float)val);
            if (job.final) {
                float y = (float)val;
                if (job.out_scale) y = y * row_scale;
                if (job.out_bias) y = y + row_bias;
                static_cast<float *>(job.out)[(size_t)tok * job.out_stride + row] = y;
            } else {
                static_cast<double *>(job.out)[(size_t)tok * job.out_stride + row] = val;
            }
        }
    }
    __syncthreads();  // the partial sums may be overwritten, the ring is free
}

// `bytes` (rounded up to 16) from global to shared memory, 16 bytes per request, asynchronously:
// the whole vector is in flight at once and costs a handful of instructions.
__device__ __forceinline__ void copy_in(void *dst, const void *src, uint32_t bytes) {
    for (uint32_t o = 16 * threadIdx.x; o < bytes; o += 16 * kStepThreads)
        cp16(static_cast<uint8_t *>(dst) + o, static_cast<const uint8_t *>(src) + o);
}

// A phase of up to three jobs that share a loader.  `gb`: the barrier that separates this
// phase from the one before (null for the very first phase of the kernel).  What a block needs
// that the previous phase does not produce - the weight tiles of its first item, the input
// scale s2, the norm weights, the output scale and bias of its rows - is requested BEFORE the
// barrier; after it only the activation vector is fetched, as one asynchronous copy.
template <bool kBf16>
__device__ __noinline__ void linear_phase(const StepArgs &a, const StepSmem &sm, const PhaseDesc &ph,
                                          GridBarrier *gb, uint32_t phase) {
    const LinJob *jobs = ph.jobs;
    const int n_jobs = ph.n_jobs;
    const Loader loader = (Loader)ph.loader;
    const NormSource ns = ph.ns;
    const float *gate = ph.gate, *up = ph.up;
    const uint32_t gu_stride = ph.gu_stride;
    uint32_t first[4] = {0, 0, 0, 0};
    for (int j = 0; j < n_jobs; ++j) first[j + 1] = first[j] + (jobs[j].n_rows + kGroupRows - 1) / kGroupRows;
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
        return Work{jobs[j].tiles, (jobs[j].n_bits + kStepBits - 1) / kStepBits, item - first[j]};
    };
    // s1 and bias of the row a finishing lane (warps 0..3, t < 2) stores
    const uint32_t warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    auto row_constants = [&](uint32_t item, int j, float &scale, float &bias) {
        scale = 1.f, bias = 0.f;
        const uint32_t row = (item - first[j]) * kGroupRows + warp * 16 + lane / 4 + 8 * (lane % 4);
        if (jobs[j].final && warp < kGroupTiles && lane % 4 < 2 && row < jobs[j].n_rows) {
            if (jobs[j].out_scale) scale = jobs[j].out_scale[row];
            if (jobs[j].out_bias) bias = jobs[j].out_bias[row];
        }
    };
    float row_scale = 1.f, row_bias = 0.f;
    const bool traced = begin == 0 && begin < end && threadIdx.x == 0;
    sub_stamp(a, phase, 0, traced);
    // Shared memory while a vector is being staged: the vector area holds s2 (then, in place,
    // z = s2 * v), the normalised row and the norm weights; the table area, not yet in use,
    // holds the raw inputs.  All of it arrives by asynchronous copies and is then worked on
    // by short loops over shared memory: little code (this kernel runs every phase once per
    // block of the model, so its size decides whether it stays in the instruction cache).
    float *vec = reinterpret_cast<float *>(sm.vec), *y = vec + a.d_model, *norm_w = vec + 2 * a.d_model;
    float *raw0 = reinterpret_cast<float *>(sm.table);
    if (begin < end) {
        const int j0 = job_of(begin);
        if (jobs[j0].in_scale) copy_in(vec, jobs[j0].in_scale, jobs[j0].n_bits * 4);
        if (loader == LOAD_NORM) copy_in(norm_w, ns.weight, a.d_model * 4);
        cp_commit();
        prefetch_tiles(sm, work_of(begin, j0));
        row_constants(begin, j0, row_scale, row_bias);
    }
    if (gb) grid_sync(*gb);
    if (begin >= end) return;
    sub_stamp(a, phase, 1, traced);
    bool scale_staged = true;  // s2 of the block's first job is on its way since before the barrier
    for (uint32_t tok = 0; tok < a.n_tok; ++tok) {
        if (loader == LOAD_NORM) {
            // ---- the norm of this token.  rmsnorm_kernel runs 512 threads with 16 elements each
            // (element i belongs to thread i % 512); a thread here plays two of them (v = tid and
            // tid + 256), a warp two of its warps (w and w + 8), with its order of additions.
            const size_t base = (size_t)tok * a.d_model;
            float *raw1 = raw0 + a.d_model;
            copy_in(raw0, ns.x_in + base, a.d_model * 4);
            if (ns.residual) copy_in(raw1, ns.residual + base, a.d_model * 4);
            cp_commit();
            cp_wait<0>();
            __syncthreads();
            for (uint32_t pv = 0; pv < kNormThreads / kStepThreads; ++pv) {
                float ss = 0.f;
                for (uint32_t i = threadIdx.x + pv * kStepThreads; i < a.d_model; i += kNormThreads) {
                    float h = raw0[i];
                    if (ns.residual) h += raw1[i];
                    if (begin == 0) ns.x_out[base + i] = h;  // the block that owns item 0 writes the stream
                    if (kBf16) h = round_bf16f(h);
                    raw0[i] = h;
                    ss += h * h;
                }
                for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
                if (lane == 0) sm.norm_red[warp + pv * (kStepThreads / 32)] = ss;
            }
            __syncthreads();
            float total = 0.f;
            for (int w = 0; w < kNormThreads / 32; ++w) total += sm.norm_red[w];
            const float inv = 1.0f / sqrtf(total / (float)a.d_model + a.eps);
            for (uint32_t i = threadIdx.x; i < a.d_model; i += kStepThreads) {
                float o = raw0[i] * inv * norm_w[i];
                if (kBf16) o = round_bf16f(o);
                y[i] = o;
            }
            __syncthreads();
        }
        sub_stamp(a, phase, 2, traced);
        int staged = -1;
        for (uint32_t item = begin; item < end; ++item) {
            const int j = job_of(item);
            const LinJob job = jobs[j];
            const Work work = work_of(item, j);
            if (item != begin || tok != 0) {
                prefetch_tiles(sm, work);
                row_constants(item, j, row_scale, row_bias);
            }
            if (j != staged) {
                // ---- z = s2 * v (float32, rounded to bfloat16 under bfloat16 serving) or t, then its table
                const bool in_double = job.final;  // stage 2 reads the float64 t
                const uint32_t n = job.n_bits;
                if (job.in_scale && !scale_staged) copy_in(vec, job.in_scale, n * 4);
                scale_staged = false;
                if (loader == LOAD_SWIGLU) {
                    copy_in(raw0, gate + (size_t)tok * gu_stride, n * 4);
                    copy_in(raw0 + n, up + (size_t)tok * gu_stride, n * 4);
                } else if (in_double) {
                    copy_in(sm.vec, static_cast<const double *>(job.src) + (size_t)tok * job.src_stride, n * 8);
                } else if (loader == LOAD_PLAIN) {
                    copy_in(raw0, static_cast<const float *>(job.src) + (size_t)tok * job.src_stride, n * 4);
                }
                cp_commit();
                cp_wait<0>();
                __syncthreads();
                if (!in_double) {
                    const float *in = loader == LOAD_NORM ? y : raw0;
                    for (uint32_t k = threadIdx.x; k < n; k += kStepThreads) {
                        float v = in[k];
                        if (loader == LOAD_SWIGLU) v = v * raw0[n + k] / (1.0f + expf(-v));
                        if (job.in_scale) v = vec[k] * v;
                        if (kBf16) v = round_bf16f(v);
                        vec[k] = v;
                    }
                    __syncthreads();
                }
                sub_stamp(a, phase, 3, traced && item == begin);
                if (in_double)
                    block_build_table_bits(reinterpret_cast<const double *>(sm.vec), n, work.n_steps,
                                           reinterpret_cast<uint4 *>(sm.table), sm.meta,
                                           reinterpret_cast<unsigned long long *>(sm.red_max), sm.red_sum, sm.red_bad);
                else
                    block_build_table_bits(reinterpret_cast<const float *>(sm.vec), n, work.n_steps,
                                           reinterpret_cast<uint4 *>(sm.table), sm.meta,
                                           reinterpret_cast<unsigned long long *>(sm.red_max), sm.red_sum, sm.red_bad);
                staged = j;
                sub_stamp(a, phase, 4, traced && item == begin);
            }
            multiply_and_finish<kBf16>(sm, work, job, tok, row_scale, row_bias);
            sub_stamp(a, phase, 5, traced && item == begin);
        }
    }
    sub_stamp(a, phase, 6, traced);
}

LinJob stage1_job(const StepLinear &l, const float *src, uint32_t src_stride, double *t,
                                             uint32_t t_stride) {
    return LinJob{l.vbt_tiles, l.r, l.din, l.s2, src, src_stride, t, t_stride, nullptr, nullptr, false};
}
LinJob stage2_job(const StepLinear &l, const double *t, uint32_t t_stride, float *out,
                                             uint32_t out_stride) {
    return LinJob{l.ub_tiles, l.dout, l.r, nullptr, t, t_stride, out, out_stride, l.s1, l.bias, true};
}

// ---- the attention phase ---------------------------------------------------------------
__device__ __noinline__ void attention_groups(const StepArgs &a, const StepSmem &sm, const PhaseDesc &L,
                                              uint32_t sub, uint32_t phase) {
    const SubBlock sb{threadIdx.x % 128, 1 + sub};
    uint8_t *mine = sm.attn + (size_t)sub * kSubSmemBytes;
    const DecAttnSmem asm_ = carve_dec_attn(mine, kSubAttnBufs);
    int *is_last = reinterpret_cast<int *>(mine + kSubAttnBytes);
    const uint32_t group = a.n_heads / a.n_kv, subs = (group + a.gq - 1) / a.gq;
    const uint32_t per_seq = a.n_splits * a.n_kv * subs, total = per_seq * a.n_tok;
    for (uint32_t vb = sub * gridDim.x + blockIdx.x; vb < total; vb += kSubBlocks * gridDim.x) {
        const uint32_t split = vb % a.n_splits, ky = (vb / a.n_splits) % (a.n_kv * subs), b = vb / per_seq;
        const bool traced = vb == 0;
        sub_stamp(a, phase, 0, traced);
        const int pos = a.positions[b], seq = a.seq_index[b];
        const bool valid = pos >= 0 && (uint32_t)pos < a.s_max && seq >= 0 && (uint32_t)seq < a.n_seq;
        if (!valid && sb.tid == 0) atomicOr(a.error, 4);  // reported like rope_cache_kernel does
        const int pos_in = min(max(pos, 0), (int)a.s_max - 1);
        const FreshKey fresh{a.k, a.v, L.cache_k, L.cache_v, a.cos_sin + (size_t)pos_in * 128, pos, seq, valid};
        if (a.gq <= 4)
            decode_attention_mma_body<true, kSubAttnBufs, true>(sb, asm_, a.q, L.cache_k, L.cache_v, a.kv_len[b],
                                                                a.partial, a.n_heads, a.n_kv, a.gq, a.s_max, a.chunk,
                                                                a.n_splits, split, ky, b, fresh);
        else
            decode_attention_mma_body<true, kSubAttnBufs, false>(sb, asm_, a.q, L.cache_k, L.cache_v, a.kv_len[b],
                                                                 a.partial, a.n_heads, a.n_kv, a.gq, a.s_max, a.chunk,
                                                                 a.n_splits, split, ky, b, fresh);
        sub_stamp(a, phase, 1, traced);
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
        sub_stamp(a, phase, 2, traced);
        if (*is_last) {
            __threadfence();
            const uint32_t kvh = ky / subs, hsub = ky % subs, h0 = kvh * group + hsub * a.gq;
            const uint32_t rows = min(a.gq, group - hsub * a.gq);
            for (uint32_t r = sb.tid / 32; r < rows; r += 4) {  // a warp per head
                const size_t head = (size_t)b * a.n_heads + h0 + r;
                decode_combine_warp<4, 32>(sb.tid % 32, a.partial + head * a.n_splits * 130, a.attn + head * 128,
                                          128, a.n_splits, 0, 32);
            }
        }
        sub_stamp(a, phase, 3, traced || *is_last);
        sb.sync();  // is_last and the staging buffers are free again
    }
}

__device__ __forceinline__ void attention_phase(const StepArgs &a, const StepSmem &sm, const PhaseDesc &L,
                                                GridBarrier &gb, uint32_t phase) {
    grid_sync(gb);
    const uint32_t sub = threadIdx.x / 128;
    if (sub < kSubBlocks) attention_groups(a, sm, L, sub, phase);
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
    const StepSmem sm = carve_step(step_smem, a.vec_bytes, a.n_steps_max);
    if (threadIdx.x == 0) gave_up = 0;
    GridBarrier gb{a.barrier, 0, a.wait_limit, a.error, &gave_up, a.stamps, a.stamps_cap, 0};
    stamp(gb);
    // (the counter is a whole multiple of the grid size between launches; a block that reads it
    // after others have arrived at the first barrier still rounds down to the same base)
    gb.target = ld_acquire_u64(a.barrier) / gridDim.x * gridDim.x;
    __syncthreads();

    for (uint32_t p = 0; p < a.n_phases; ++p) {
        const PhaseDesc &ph = a.phases[p];
        if (ph.kind == PHASE_ATTENTION) attention_phase(a, sm, ph, gb, p);
        else linear_phase<kBf16>(a, sm, ph, p ? &gb : nullptr, p);
    }
    stamp(gb);
}

size_t step_smem_bytes(const StepArgs &a) {
    const size_t linear = linear_smem_bytes(a.vec_bytes, a.n_steps_max);
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
    void *d_phases = nullptr, *d_t = nullptr, *d_sync = nullptr;
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
    if (desc->n_tokens > 8)
        return qk::fail(QK_ERR_VALUE, "the whole-step kernel is for small batches (at most 8 tokens), got %zu",
                        desc->n_tokens);
    if (desc->n_kv_heads == 0 || desc->n_heads % desc->n_kv_heads != 0)
        return qk::fail(QK_ERR_VALUE, "n_kv_heads must divide n_heads: n_heads=%zu, n_kv_heads=%zu",
                        desc->n_heads, desc->n_kv_heads);
    if (desc->n_splits == 0 || desc->n_splits > 128)
        return qk::fail(QK_ERR_VALUE, "between 1 and 128 key splits are supported, got %zu", desc->n_splits);
    if (desc->d_model > (size_t)kNormPer * kNormThreads || desc->d_model % 8 != 0 || desc->d_ff % 4 != 0)
        return qk::fail(QK_ERR_VALUE, "d_model must be a multiple of 8 and at most %d, d_ff a multiple of 4; got "
                        "%zu and %zu", kNormPer * kNormThreads, desc->d_model, desc->d_ff);
    const qk_step_buffers &b = desc->buf;
    if (!b.x || !b.x2 || !b.q || !b.k || !b.v || !b.attn || !b.delta_attn || !b.delta_mlp || !b.gate || !b.up ||
        !b.att_scratch || !b.cos_sin || !b.positions || !b.seq_index || !b.kv_len)
        return qk::fail(QK_ERR_VALUE, "qk_decode_step_create: every buffer of the step must be given");
    const size_t dq = desc->n_heads * 128, dkv = desc->n_kv_heads * 128;
    std::vector<StepLayer> layers(desc->n_blocks);
    size_t r_max = 0, steps_max = 0, din_max = 0;
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
            din_max = l->din > din_max ? l->din : din_max;
            const size_t steps = qk::ceil_div(l->din > l->r ? l->din : l->r, (size_t)kStepBits);
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
        cudaFree(s->d_phases);
        cudaFree(s->d_t);
        cudaFree(s->d_sync);
        delete s;
        return code;
    };
    StepArgs &a = s->args;
    const size_t group = desc->n_heads / desc->n_kv_heads, gq = group < 8 ? group : 8, subs = qk::ceil_div(group, gq);
    const size_t t_stride = qk::ceil_div(r_max, 64) * 64;
    const size_t n_tickets = desc->n_tokens * desc->n_kv_heads * subs;
    const size_t n_phases = 9 * desc->n_blocks;
    if (cudaMalloc(&s->d_phases, n_phases * sizeof(PhaseDesc)) != cudaSuccess ||
        cudaMalloc(&s->d_t, 3 * desc->n_tokens * t_stride * sizeof(double)) != cudaSuccess ||
        cudaMalloc(&s->d_sync, 256 + n_tickets * sizeof(uint32_t)) != cudaSuccess)
        return bail(qk::fail(QK_ERR_CUDA, "qk_decode_step_create: device allocation failed: %s",
                             cudaGetErrorString(cudaGetLastError())));
    // ---- the phases: nine per block, the residual stream alternating between x and x2
    double *t[3];
    for (int j = 0; j < 3; ++j) t[j] = (double *)s->d_t + (size_t)j * desc->n_tokens * t_stride;
    const uint32_t ts = (uint32_t)t_stride, dm = (uint32_t)desc->d_model, dff = (uint32_t)desc->d_ff;
    std::vector<PhaseDesc> phases;
    phases.reserve(n_phases);
    float *x_in = b.x, *x_out = b.x2;
    auto linear = [&](Loader loader, std::initializer_list<LinJob> jobs) {
        PhaseDesc ph{};
        ph.kind = PHASE_LINEAR;
        ph.loader = loader;
        for (const LinJob &j : jobs) ph.jobs[ph.n_jobs++] = j;
        return ph;
    };
    for (size_t i = 0; i < desc->n_blocks; ++i) {
        const StepLayer &L = layers[i];
        PhaseDesc ph = linear(LOAD_NORM, {stage1_job(L.lin[LIN_Q], nullptr, 0, t[0], ts),
                                          stage1_job(L.lin[LIN_K], nullptr, 0, t[1], ts),
                                          stage1_job(L.lin[LIN_V], nullptr, 0, t[2], ts)});
        ph.ns = NormSource{x_in, i ? b.delta_mlp : nullptr, L.in_norm, x_out};
        phases.push_back(ph);
        std::swap(x_in, x_out);
        phases.push_back(linear(LOAD_PLAIN, {stage2_job(L.lin[LIN_Q], t[0], ts, b.q, (uint32_t)dq),
                                             stage2_job(L.lin[LIN_K], t[1], ts, b.k, (uint32_t)dkv),
                                             stage2_job(L.lin[LIN_V], t[2], ts, b.v, (uint32_t)dkv)}));
        PhaseDesc at{};
        at.kind = PHASE_ATTENTION;
        at.cache_k = L.cache_k;
        at.cache_v = L.cache_v;
        phases.push_back(at);
        phases.push_back(linear(LOAD_PLAIN, {stage1_job(L.lin[LIN_O], b.attn, (uint32_t)dq, t[0], ts)}));
        phases.push_back(linear(LOAD_PLAIN, {stage2_job(L.lin[LIN_O], t[0], ts, b.delta_attn, dm)}));
        ph = linear(LOAD_NORM, {stage1_job(L.lin[LIN_GATE], nullptr, 0, t[0], ts),
                                stage1_job(L.lin[LIN_UP], nullptr, 0, t[1], ts)});
        ph.ns = NormSource{x_in, b.delta_attn, L.post_norm, x_out};
        phases.push_back(ph);
        std::swap(x_in, x_out);
        phases.push_back(linear(LOAD_PLAIN, {stage2_job(L.lin[LIN_GATE], t[0], ts, b.gate, dff),
                                             stage2_job(L.lin[LIN_UP], t[1], ts, b.up, dff)}));
        ph = linear(LOAD_SWIGLU, {stage1_job(L.lin[LIN_DOWN], nullptr, 0, t[0], ts)});
        ph.gate = b.gate, ph.up = b.up, ph.gu_stride = dff;
        phases.push_back(ph);
        phases.push_back(linear(LOAD_PLAIN, {stage2_job(L.lin[LIN_DOWN], t[0], ts, b.delta_mlp, dm)}));
    }
    if (cudaMemcpyAsync(s->d_phases, phases.data(), phases.size() * sizeof(PhaseDesc), cudaMemcpyHostToDevice,
                        c->stream) != cudaSuccess ||
        cudaMemsetAsync(s->d_sync, 0, 256 + n_tickets * sizeof(uint32_t), c->stream) != cudaSuccess ||
        cudaMemsetAsync(s->d_t, 0, 3 * desc->n_tokens * t_stride * sizeof(double), c->stream) != cudaSuccess ||
        cudaStreamSynchronize(c->stream) != cudaSuccess)
        return bail(qk::fail(QK_ERR_CUDA, "qk_decode_step_create: upload failed: %s",
                             cudaGetErrorString(cudaGetLastError())));
    a.phases = (const PhaseDesc *)s->d_phases;
    a.n_phases = (uint32_t)phases.size();
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
    a.q = b.q, a.k = b.k, a.v = b.v, a.attn = b.attn, a.partial = b.att_scratch;
    a.cos_sin = b.cos_sin;
    a.positions = b.positions, a.seq_index = b.seq_index, a.kv_len = b.kv_len;
    a.barrier = (unsigned long long *)s->d_sync;
    a.tickets = (uint32_t *)((uint8_t *)s->d_sync + 256);
    a.n_steps_max = (uint32_t)steps_max;
    a.vec_bytes = (uint32_t)(din_max * 4 > r_max * 8 ? din_max * 4 : r_max * 8);
    if (a.vec_bytes < 12 * desc->d_model) a.vec_bytes = (uint32_t)(12 * desc->d_model);  // z, normalised row, norm weights
    s->smem = step_smem_bytes(a);
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
    c->err_armed = true;
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

qk_status qk_decode_step_trace(qk_decode_step *step, uint64_t *stamps_dev, size_t capacity) {
    if (!step) return qk::fail(QK_ERR_VALUE, "qk_decode_step_trace: step is null");
    step->args.stamps = (unsigned long long *)stamps_dev;
    step->args.stamps_cap = stamps_dev ? (uint32_t)capacity : 0;
    return QK_OK;
}

void qk_decode_step_free(qk_decode_step *step) {
    if (!step) return;
    cudaFree(step->d_phases);
    cudaFree(step->d_t);
    cudaFree(step->d_sync);
    delete step;
}

}  // extern "C"
