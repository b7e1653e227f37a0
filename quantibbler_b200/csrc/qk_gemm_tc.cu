// Prefill GEMM of the factorized linear on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// For T tokens at once the two stages of y = s1 * (Ub (Vb^T (s2 * x))) + bias are dense
// contractions: stage 1 is [T x din] . [r x din]^T, stage 2 is [T x r] . [dout x r]^T.  This
// is the column-batched product of crates/quantibbler-kernels/src/core.rs:288-317
// (packed_matmul) under the bfloat16 serving contract of
// crates/quantibbler-server/src/engine/mod.rs:449-460 (apply_bf16): operands bfloat16,
// float32 accumulation, z, t and u each rounded once to bfloat16.
//
// tcgen05 has no 1-bit x bf16 mode, so the +-1 weights are expanded to bfloat16 on the fly.
// The weights take the M side of the MMA (128 weight rows per tile) and the tokens the N
// side (up to 256 tokens), so that the costly operand - the one that has to be expanded -
// is the narrow one.  One persistent CTA per SM walks over its tiles with these roles:
//   * warps 0..15, producers, in four groups of 128 threads; group g owns pipeline stage g
//     and fills it for every fourth 64-wide k-chunk.  Thread i of a group owns weight row
//     i of the tile: it reads the row's 64 bits of the chunk (two such loads ahead) and
//     turns them into 64 bfloat16 +-1 values in registers (a multiply that spreads four
//     bits to the tops of four bytes, one LOP3, two byte permutes per four weights: no
//     table, because shared-memory bandwidth is what bounds this kernel), stored as eight
//     16-byte pieces in the 128-byte-swizzled K-major layout
//     the UMMA descriptors expect.  The group's first thread also starts the TMA copy
//     (cp.async.bulk.tensor, one CTA per copy) of the chunk's activation tile, up to 256
//     tokens x 64 k; rows beyond the token count are zero-filled by the copy;
//   * warp 16 issues tcgen05.mma (M = 128, N = tokens, K = 16 per instruction, four per
//     stage) with the float32 accumulator in tensor memory; tcgen05.commit hands the stage
//     back to its group.  The wait-issue-commit loop costs about 530 cycles per chunk
//     whatever N is, which is why the token tile is as wide as it can be (N = 256 is 512
//     cycles of tensor-core work per chunk);
//   * warps 17..20, epilogue: tensor memory holds two accumulators, so the epilogue of one
//     tile (tcgen05.ld, one weight row per thread so that a warp's stores to the
//     token-major output are contiguous; rounding, scale, bias) overlaps the main loop of
//     the next.
// All hand-offs go through mbarriers.  Every wait is bounded: on expiry the kernel records an
// error code, frees its tensor memory and returns, and the host reports QK_ERR_TIMEOUT.
#include <cuda.h>  // CUtensorMap types only; the encoder is fetched through the runtime

#include <algorithm>
#include <cstring>
#include <type_traits>

#include "qk_common.h"
#include "qk_umma.cuh"

namespace {

constexpr int kBM = 128;        // weight rows per tile (UMMA M)
constexpr int kBNMax = 256;     // tokens per tile (UMMA N), a multiple of 16
constexpr int kBK = 64;         // k per stage: one 128-byte swizzle row of bfloat16
constexpr int kStages = 4;
constexpr int kGroups = kStages;            // producer groups; group g fills stage g
constexpr int kGroupThreads = 128;          // one thread per weight row of the tile
constexpr int kProducerWarps = kGroups * kGroupThreads / 32;  // warps 0..15
constexpr int kMmaWarp = kProducerWarps;                      // warp 16
constexpr int kEpilogueWarp0 = kMmaWarp + 1;                  // warps 17..20
constexpr int kEpilogueWarps = 4;
constexpr int kThreads = (kEpilogueWarp0 + kEpilogueWarps) * 32;
constexpr uint32_t kABytes = kBM * kBK * 2, kBBytes = kBNMax * kBK * 2;  // A: weights, B: tokens
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kTmemCols = 2 * kBNMax;    // two accumulators
constexpr uint32_t kWaitLimitDefault = 1u << 22;  // polls; qk_set_wait_limit overrides it

// The four epilogue warps agree on a verdict (named barrier 1 with an AND reduction): either
// all of them go on, or all of them leave, so that none is left waiting at one of the
// epilogue's own barriers for a warp that has gone.
__device__ __forceinline__ bool epilogue_vote(bool ok, uint32_t n_threads) {
    uint32_t all;
    asm volatile(
        "{\n .reg .pred p, q;\n setp.ne.b32 p, %1, 0;\n"
        " barrier.cta.red.and.pred q, 1, %2, p;\n selp.u32 %0, 1, 0, q;\n}"
        : "=r"(all)
        : "r"((uint32_t)ok), "r"(n_threads)
        : "memory");
    return all != 0;
}
// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M = 128, N = bn.
__device__ __forceinline__ uint32_t umma_idesc(uint32_t bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((bn >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}
// round-to-nearest-even float32 -> bfloat16, kept in the high half (NaN stays NaN)
__device__ __forceinline__ uint32_t round_bf16_hi(uint32_t u) {
    return (u & 0x7fffffffu) > 0x7f800000u ? ((u | 0x00400000u) & 0xffff0000u)
                                           : ((u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u);
}

// Four weight bits (bit i of n = element i; 1 means +1) -> the four high bytes of their
// bfloat16 values: 0x3F for +1.0, 0xBF for -1.0.  The multiply puts bit i at the top of byte
// i (the four shifted copies of n do not overlap, so nothing carries); the rest is one LOP3.
__device__ __forceinline__ uint32_t expand_nibble(uint32_t n) {
    return ((n * 0x10204080u) & 0x80808080u) ^ 0xBFBFBFBFu;
}

// One launch can serve up to four factors that share the token count (the q, k, v or the
// gate, up projections of a block): problem p owns the units [unit_begin, next unit_begin).
constexpr int kMaxProblems = 4;
struct Problem {
    const uint8_t *w_rows; // weight bits, rows padded to w_stride bytes
    void *out;             // bf16 [tokens][out_pitch] (stage 1) or float [tokens][n_rows]
    const float *out_scale, *out_bias;
    uint32_t n_rows, k_chunks, w_stride, out_pitch;
    uint32_t row_tiles;    // tile t of the problem covers row tile t % row_tiles, token tile t / row_tiles
    uint32_t unit_begin;   // the problem's first unit; a tile is k_chunks consecutive units
};
constexpr int kMaxCtas = 192;
struct GemmArgs {
    Problem p[kMaxProblems];
    uint32_t n_problems;
    int *error;
    uint32_t tokens;
    uint32_t bn;           // tokens per tile
    uint32_t units;        // all tiles x their k_chunks: the work that is dealt out evenly to the CTAs
    float *partials;       // [CTAs][256][128] float32 accumulators of split tiles
    uint32_t *flags;       // [CTAs] flags[i] != 0: CTA i's partial is in place (its one reader clears it)
    uint32_t wait_limit;   // polls before a wait gives up
    // CTA i works on units [cta_begin[i], cta_begin[i + 1]) (plan_ctas, on the host)
    uint32_t cta_begin[kMaxCtas + 1];
};


// Where unit u lies: which problem, which of its tiles, which k-chunk of the tile.
struct UnitPos {
    uint32_t problem, tile, kc, tile_begin;  // tile_begin: the unit number of the tile's chunk 0
};
__device__ __forceinline__ UnitPos locate(const GemmArgs &g, uint32_t u) {
    uint32_t pi = 0;
#pragma unroll
    for (int i = 1; i < kMaxProblems; ++i)
        if ((uint32_t)i < g.n_problems && u >= g.p[i].unit_begin) pi = i;
    const uint32_t local = u - g.p[pi].unit_begin, k = g.p[pi].k_chunks;
    const uint32_t tile = local / k;
    return {pi, tile, local - tile * k, g.p[pi].unit_begin + tile * k};
}

// The epilogue of one output element: kFinal = false: out = bf16(acc) as the next stage's
// activation (zero in the padding columns);  true: y = bf16(acc) * s1 + bias.
template <bool kFinal>
__device__ __forceinline__ void store_output(const Problem &g, uint32_t tok, uint32_t n, uint32_t acc_bits,
                                             float scale, float bias) {
    // one rounding to bfloat16, as packed_matmul's bf16 instantiation does
    const uint32_t rb = round_bf16_hi(acc_bits);
    if (kFinal) {
        static_cast<float *>(g.out)[(size_t)tok * g.n_rows + n] = __uint_as_float(rb) * scale + bias;
    } else {
        static_cast<uint16_t *>(g.out)[(size_t)tok * g.out_pitch + n] =
            n < g.n_rows ? (uint16_t)(rb >> 16) : (uint16_t)0;
    }
}

template <bool kFinal>
__global__ void __launch_bounds__(kThreads, 1)
factorized_gemm_tc_kernel(const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                          const __grid_constant__ CUtensorMap map2, const __grid_constant__ CUtensorMap map3,
                          GemmArgs g) {
    qk::pdl_launch();  // the kernel after this one may begin its prologue
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment of the tiles is what the swizzle pattern assumes
    uint8_t *tiles = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t *full = reinterpret_cast<uint64_t *>(tiles + kStages * kStageBytes);
    uint64_t *empty = full + kStages;
    uint64_t *acc_full = empty + kStages;   // [2]
    uint64_t *acc_empty = acc_full + 2;     // [2]
    uint64_t *staged_bar = acc_empty + 2;   // a neighbour's partial accumulator has landed
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(staged_bar + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t kBN = g.bn;
    // This CTA's share of the work.  It is a run of consecutive units, so it is cut into
    // segments at tile borders: the rest of a tile another CTA began, whole tiles, the head of
    // a tile.  Only the first segment can start inside a tile; its accumulator goes to
    // partials[this CTA] and flags[this CTA] is raised (its reader clears it again).  A segment that starts a tile is
    // finished here: if it stops short of the tile's end, the CTAs after this one hold the
    // rest as THEIR first segments, which they computed at the very start of the kernel, so
    // by now those partials are in place; they are added in CTA order (a fixed order, so the
    // sum is reproducible) before the epilogue.  The wait on the flags is bounded all the same.
    const uint32_t u_begin = g.cta_begin[blockIdx.x];
    const uint32_t u_end = g.cta_begin[blockIdx.x + 1];
    const uint32_t total_chunks = u_end - u_begin;
    // What depends on no other kernel is fetched before the dependency wait: the weight bits
    // of each producer's first two chunks (a first touch of those rows: one DRAM latency that
    // would otherwise open the main loop), the lines of its later chunks and the tensor maps
    // into L2 / the descriptor cache, the first segment's scales and biases.
    // The ring of stages runs on across tiles: chunk number gc (counted from the CTA's first
    // unit) uses stage gc % 4 and belongs to group gc % 4.  Rows past the end of the factor
    // re-read the last row: their accumulator lanes are never stored.
    const uint32_t group = tid / kGroupThreads, row = tid % kGroupThreads;
    auto bits_at = [&](uint32_t gc) -> const uint2 * {
        const UnitPos at = locate(g, u_begin + gc);
        const Problem &pr = g.p[at.problem];
        const uint32_t n_src = min((at.tile % pr.row_tiles) * kBM + row, pr.n_rows - 1);
        return reinterpret_cast<const uint2 *>(pr.w_rows + (size_t)n_src * pr.w_stride) + at.kc;
    };
    auto load_bits = [&](uint32_t gc) -> uint2 {
        return gc < total_chunks ? *bits_at(gc) : make_uint2(0, 0);
    };
    uint2 q0 = make_uint2(0, 0), q1 = q0;
    if (warp < kProducerWarps) {
        q0 = load_bits(group);
        q1 = load_bits(group + kGroups);
        // (a 128-byte line of a row holds sixteen chunks)
        for (uint32_t gc = group + 16; gc < total_chunks && gc < group + 16 * 8; gc += 16)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(bits_at(gc)));
    } else if (warp == kMmaWarp) {
        if (lane < g.n_problems) {
            const CUtensorMap *m = lane == 0 ? &map0 : lane == 1 ? &map1 : lane == 2 ? &map2 : &map3;
            asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
        }
    } else if (kFinal && total_chunks) {
        const UnitPos at = locate(g, u_begin);
        const Problem &pr = g.p[at.problem];
        const uint32_t n = min((at.tile % pr.row_tiles) * kBM + (warp % 4) * 32 + lane, pr.n_rows - 1);
        if (pr.out_scale) asm volatile("prefetch.global.L2 [%0];" ::"l"(pr.out_scale + n));
        if (pr.out_bias) asm volatile("prefetch.global.L2 [%0];" ::"l"(pr.out_bias + n));
    }

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], kGroupThreads / 32 + 1);  // the group's warps + the expect_tx
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], kEpilogueWarps);
        }
        mbar_init(staged_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // Barriers and tensor memory are set up; from here on the kernel reads what the kernel
    // before it wrote (the activations, the partial-sum workspace and its flags).  Every thread
    // waits, so that this kernel's completion implies the completion of everything before it.
    qk::pdl_wait();
    const uint32_t tmem_base = *tmem_slot;

    if (warp < kProducerWarps) {
        // ------------------------------------------------------------ producers
        uint8_t *a_tile = tiles + group * kStageBytes, *b_tile = a_tile + kABytes;
        uint64_t *my_full = &full[group], *my_empty = &empty[group];
        const uint32_t dst_base = smem_u32(a_tile) + row * 128, swz = (row & 7) << 4;
        uint32_t it = 0;
        for (uint32_t gc = group; gc < total_chunks; gc += kGroups, ++it) {
            const uint2 cur = q0;
            q0 = q1;
            q1 = load_bits(gc + 2 * kGroups);
            if (!mbar_wait(my_empty, (it & 1) ^ 1, abort_flag, g.wait_limit)) {
                *abort_flag = 1;
                break;
            }
            if (row == 0) {
                // tokens: one TMA box of 64 k x bn tokens, completing on the full barrier
                const UnitPos at = locate(g, u_begin + gc);
                const uint32_t kc = at.kc, t0 = (at.tile / g.p[at.problem].row_tiles) * kBN;
                const CUtensorMap *b_map = at.problem == 0 ? &map0 : at.problem == 1 ? &map1
                                         : at.problem == 2 ? &map2 : &map3;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                                 smem_u32(my_full)),
                             "r"(kBN * kBK * 2)
                             : "memory");
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
                    "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(b_tile)),
                    "l"(b_map), "r"(kc * kBK), "r"(t0), "r"(smem_u32(my_full))
                    : "memory");
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                // byte c of the chunk -> eight bfloat16 +-1 values, in registers: shared memory
                // is the contended resource of this kernel (TMA writes, tensor-core operand
                // reads and these stores all go through its 128 bytes per clock)
                const uint32_t byte = __byte_perm(c < 4 ? cur.x : cur.y, 0, 0x4440 + (c & 3));
                const uint32_t h0 = expand_nibble(byte & 15u), h1 = expand_nibble(byte >> 4);
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(dst_base + ((c << 4) ^ swz)),
                             "r"(__byte_perm(h0, 0x80808080u, 0x1404)),
                             "r"(__byte_perm(h0, 0x80808080u, 0x3424)),
                             "r"(__byte_perm(h1, 0x80808080u, 0x1404)),
                             "r"(__byte_perm(h1, 0x80808080u, 0x3424))
                             : "memory");
            }
            // generic-proxy writes must be visible to the tensor core's async proxy
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(my_full);
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------ MMA issue
        // The whole warp runs the loop and waits on the barriers; lane 0 alone issues.  (A
        // lone diverged lane beside 31 lanes parked at the block barrier issues several
        // times slower.)
        const uint32_t idesc = umma_idesc(kBN);
        uint32_t gc = 0;
        bool dead = false;
        for (uint32_t u = u_begin, seg = 0; u < u_end && !dead; ++seg) {
            const UnitPos at = locate(g, u);
            const uint32_t kc0 = at.kc, kc1 = min(g.p[at.problem].k_chunks, kc0 + (u_end - u));
            const uint32_t acc = seg & 1;
            // the epilogue must have drained this accumulator (segment seg - 2)
            if (!mbar_wait(&acc_empty[acc], ((seg >> 1) & 1) ^ 1, abort_flag, g.wait_limit)) {
                dead = true;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t d_tmem = tmem_base + acc * kBNMax;
            for (uint32_t kc = kc0; kc < kc1; ++kc, ++gc) {
                const uint32_t s = gc % kStages;
                if (!mbar_wait(&full[s], (gc / kStages) & 1, abort_flag, g.wait_limit)) {
                    dead = true;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (lane == 0) {
                    const uint32_t a_addr = smem_u32(tiles + s * kStageBytes), b_addr = a_addr + kABytes;
#pragma unroll
                    for (int k = 0; k < kBK / 16; ++k) {
                        const uint64_t ad = umma_desc(a_addr + k * 32), bd = umma_desc(b_addr + k * 32);
                        const uint32_t accumulate = (kc != kc0 || k != 0) ? 1u : 0u;
                        asm volatile(
                            "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                            " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(d_tmem),
                            "l"(ad), "l"(bd), "r"(idesc), "r"(accumulate)
                            : "memory");
                    }
                    umma_commit(&empty[s]);  // the stage may be refilled once these MMAs have read it
                }
                __syncwarp();
            }
            if (!dead && lane == 0) umma_commit(&acc_full[acc]);
            __syncwarp();
            u += kc1 - kc0;
        }
        if (dead) *abort_flag = 1;
    } else {
        // ------------------------------------------------------------ epilogue
        // thread = weight row n (tensor-memory lane; a warp reaches the 32 lanes of its number
        // modulo 4), columns = tokens
        const uint32_t quarter = warp % 4;
        const size_t slot_elems = (size_t)kBNMax * kBM;
        bool dead = false;
        for (uint32_t u = u_begin, seg = 0; u < u_end && !dead; ++seg) {
            const UnitPos at = locate(g, u);
            const Problem &pr = g.p[at.problem];
            const uint32_t tile = at.tile, kc0 = at.kc;
            const uint32_t len = min(pr.k_chunks - kc0, u_end - u);
            const uint32_t acc = seg & 1;
            const uint32_t n_local = quarter * 32 + lane;
            const uint32_t n = (tile % pr.row_tiles) * kBM + n_local;
            const uint32_t t0 = (tile / pr.row_tiles) * kBN;
            // CTAs [blockIdx.x + 1, last) hold the rest of this tile
            uint32_t last = blockIdx.x + 1;
            if (kc0 == 0 && len < pr.k_chunks) {
                const uint32_t hi = at.tile_begin + pr.k_chunks;
                while (last < gridDim.x && g.cta_begin[last] < hi) ++last;
            }
            // this CTA's own share of the tile first: once its accumulator is complete, every
            // MMA of the CTA so far has read its operands
            dead = !mbar_wait(&acc_full[acc], (seg >> 1) & 1, abort_flag, g.wait_limit);
            // When this is the CTA's last segment the pipeline has drained and the stages are
            // free: as many of the following CTAs' partials as fit there (each is contiguous,
            // bn x 128 floats) come in by bulk copies instead of latency-bound loads, each one
            // started the moment its flag is seen, so that the copies run while the later CTAs
            // are still being waited for.  Any further partials are read directly.
            const uint32_t part_bytes = kBN * kBM * 4;
            uint32_t n_staged = 0;
            if (last > blockIdx.x + 1 && u + len == u_end)
                n_staged = min(last - blockIdx.x - 1, (uint32_t)(kStages * kStageBytes) / part_bytes);
            const bool staged = n_staged > 0, issuer = warp == kEpilogueWarp0 && lane == 0;
            for (uint32_t j = blockIdx.x + 1; j < last && !dead; ++j) {
                uint32_t seen = 0;
                for (uint32_t i = 0; i < g.wait_limit; ++i) {
                    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(seen) : "l"(g.flags + j) : "memory");
                    if (seen) break;
                    if ((i & 255u) == 255u && *abort_flag) break;
                    __nanosleep(64);
                }
                // every lane made its own acquire load; the warp goes on only if all saw it
                dead = __all_sync(0xffffffffu, seen != 0) == 0;
                const uint32_t slot = j - blockIdx.x - 1;
                if (!dead && issuer && slot < n_staged) {
                    // (the partial was written through the generic proxy and is read by the
                    // asynchronous one)
                    asm volatile("fence.proxy.async.global;" ::: "memory");
                    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(
                                     smem_u32(staged_bar)),
                                 "r"(part_bytes)
                                 : "memory");
                    asm volatile(
                        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
                            "r"(smem_u32(tiles) + slot * part_bytes),
                        "l"(g.partials + (size_t)j * slot_elems), "r"(part_bytes), "r"(smem_u32(staged_bar))
                        : "memory");
                }
            }
            // (the barrier's one pending arrival keeps its phase open until every copy that was
            // started has been accounted for; the issuer arrives whether or not its warp gave
            // up, and every warp waits for the copies that are in flight before it votes)
            if (issuer && staged) mbar_arrive(staged_bar);
            if (staged && !mbar_wait(staged_bar, 0, abort_flag, g.wait_limit)) dead = true;
            // one verdict for the four epilogue warps before any of them touches tensor memory
            // or one of the epilogue's barriers
            if (!epilogue_vote(!dead, kEpilogueWarps * 32)) {
                *abort_flag = 1;
                dead = true;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool n_live = kFinal ? n < pr.n_rows : n < pr.out_pitch;
            const float scale = (kFinal && pr.out_scale && n < pr.n_rows) ? pr.out_scale[n] : 1.f;
            const float bias = (kFinal && pr.out_bias && n < pr.n_rows) ? pr.out_bias[n] : 0.f;
            float *part = g.partials + (size_t)blockIdx.x * slot_elems;
            const float *staged_part = reinterpret_cast<const float *>(tiles);
            // kW token columns at a time: tensor memory -> registers, the other CTAs' shares
            // added in CTA order, then the partial or the finished outputs stored
            auto columns = [&](uint32_t c0, auto width) {
                constexpr int kW = decltype(width)::value;
                uint32_t v[kW];
                const uint32_t taddr = tmem_base + ((quarter * 32) << 16) + acc * kBNMax + c0;
                if constexpr (kW == 32) {
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]),
                          "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]),
                          "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]),
                          "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]),
                          "=r"(v[30]), "=r"(v[31])
                        : "r"(taddr)
                        : "memory");
                } else {
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
                        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]),
                          "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]),
                          "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
                        : "r"(taddr)
                        : "memory");
                }
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (kc0 != 0) {
                    // the rest of a tile another CTA began: the raw accumulator,
                    // [token column][weight row]
#pragma unroll
                    for (int j = 0; j < kW; ++j)
                        part[(size_t)(c0 + j) * kBM + n_local] = __uint_as_float(v[j]);
                    return;
                }
                for (uint32_t i = 0; i < n_staged; ++i) {  // in CTA order
                    const float *sp = staged_part + (size_t)i * (kBN * kBM) + c0 * kBM + n_local;
#pragma unroll
                    for (int j = 0; j < kW; ++j)
                        v[j] = __float_as_uint(__uint_as_float(v[j]) + sp[j * kBM]);
                }
                for (uint32_t p = blockIdx.x + 1 + n_staged; p < last; ++p) {
                    const float *src = g.partials + (size_t)p * slot_elems + (size_t)c0 * kBM + n_local;
                    float got[kW];
#pragma unroll
                    for (int j = 0; j < kW; ++j) got[j] = __ldcg(src + j * kBM);
#pragma unroll
                    for (int j = 0; j < kW; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + got[j]);
                }
                if (n_live) {
#pragma unroll
                    for (int j = 0; j < kW; ++j) {
                        const uint32_t tok = t0 + c0 + j;
                        if (tok >= g.tokens) break;
                        store_output<kFinal>(pr, tok, n, v[j], scale, bias);
                    }
                }
            };
            for (uint32_t c0 = 0; c0 < kBN;) {
                if (t0 + c0 >= g.tokens) break;  // warp-uniform
                if (kBN - c0 >= 32) {
                    columns(c0, std::integral_constant<int, 32>{});
                    c0 += 32;
                } else {
                    columns(c0, std::integral_constant<int, 16>{});
                    c0 += 16;
                }
            }
            // the accumulator may be overwritten once every epilogue warp has read it
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[acc]);
            if (last > blockIdx.x + 1) {
                // every partial of this tile has been read: hand the flags back, cleared, for
                // the next launch (this CTA is their only reader)
                asm volatile("bar.sync 1, %0;" ::"r"(kEpilogueWarps * 32) : "memory");
                if (warp == kEpilogueWarp0 && lane == 0)
                    for (uint32_t j = blockIdx.x + 1; j < last; ++j) g.flags[j] = 0;
            }
            if (kc0 != 0) {
                // publish the partial: the four warps meet (which orders their stores before
                // the one thread that goes on), and that thread raises the flag with a release
                // at device scope, which is cumulative over what it has synchronised with
                asm volatile("bar.sync 1, %0;" ::"r"(kEpilogueWarps * 32) : "memory");
                if (warp == kEpilogueWarp0 && lane == 0)
                    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(g.flags + blockIdx.x), "r"(1u) : "memory");
            }
            u += len;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"(kTmemCols)
                     : "memory");
    }
    if (tid == 0 && *abort_flag) atomicOr(g.error, 1);
}

// z_p = bf16(s2_p * x) (float32 product, one rounding), zero padded to the pitch, for each of
// the problems of a launch (grid.y).  One thread makes eight consecutive outputs (one
// 16-byte store).  With `up` given, x is the SwiGLU of the two inputs, silu(x) * up, formed
// here with swiglu_kernel's expression instead of being written and read back as an
// activation (engine/mod.rs:931-935).
struct ScaleArgs {
    const float *s2[kMaxProblems];
    uint16_t *z[kMaxProblems];
};
__device__ __forceinline__ float gated_value(float g, float u) { return g * u / (1.0f + expf(-g)); }
__global__ void scale_to_bf16_kernel(const float *__restrict__ x, const float *__restrict__ up, ScaleArgs a,
                                     uint32_t n_tokens, uint32_t din, uint32_t pitch, int vec) {
    qk::pdl_launch();  // the kernel after this one may begin its prologue
    const float *__restrict__ s2 = a.s2[blockIdx.y];
    uint16_t *__restrict__ z = a.z[blockIdx.y];
    const uint32_t per_row = pitch / 8;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = idx < (size_t)n_tokens * per_row;
    const uint32_t t = (uint32_t)(idx / per_row), k = (uint32_t)(idx % per_row) * 8;
    const bool wide = vec && k + 8 <= din;
    // (the scale is a constant of the layer: it is read before the dependency wait)
    float4 c0 = make_float4(0.f, 0.f, 0.f, 0.f), d0 = c0;
    if (live && wide) {
        c0 = *reinterpret_cast<const float4 *>(s2 + k);
        d0 = *reinterpret_cast<const float4 *>(s2 + k + 4);
    }
    qk::pdl_wait();    // everything before this kernel on the stream is complete and visible
    if (!live) return;
    const float *xr = x + (size_t)t * din;
    float v[8];
    if (wide) {
        float4 a0 = *reinterpret_cast<const float4 *>(xr + k);
        float4 b0 = *reinterpret_cast<const float4 *>(xr + k + 4);
        if (up) {
            const float *ur = up + (size_t)t * din;
            const float4 e0 = *reinterpret_cast<const float4 *>(ur + k);
            const float4 f0 = *reinterpret_cast<const float4 *>(ur + k + 4);
            a0 = make_float4(gated_value(a0.x, e0.x), gated_value(a0.y, e0.y), gated_value(a0.z, e0.z),
                             gated_value(a0.w, e0.w));
            b0 = make_float4(gated_value(b0.x, f0.x), gated_value(b0.y, f0.y), gated_value(b0.z, f0.z),
                             gated_value(b0.w, f0.w));
        }
        v[0] = c0.x * a0.x; v[1] = c0.y * a0.y; v[2] = c0.z * a0.z; v[3] = c0.w * a0.w;
        v[4] = d0.x * b0.x; v[5] = d0.y * b0.y; v[6] = d0.z * b0.z; v[7] = d0.w * b0.w;
    } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float xv = k + i < din ? xr[k + i] : 0.f;
            if (up && k + i < din) xv = gated_value(xv, up[(size_t)t * din + k + i]);
            v[i] = k + i < din ? s2[k + i] * xv : 0.f;
        }
    }
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
        w[i] = (round_bf16_hi(__float_as_uint(v[2 * i])) >> 16) |
               round_bf16_hi(__float_as_uint(v[2 * i + 1]));
    *reinterpret_cast<uint4 *>(z + (size_t)t * pitch + k) = make_uint4(w[0], w[1], w[2], w[3]);
}

constexpr size_t kSmemBytes = 1024 + kStages * kStageBytes + (2 * kStages + 5) * 8 + 16;
static_assert(kSmemBytes <= 227 * 1024, "the stages must fit the 227 KB a CTA may have");

// cuTensorMapEncodeTiled, obtained through the runtime so that the library does not link
// against the driver library directly.
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

qk_status encode_activation_map(const uint16_t *base, size_t rows, size_t pitch, uint32_t box_rows,
                                CUtensorMap *out) {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *sym = nullptr;
        cudaDriverEntryPointQueryResult qres;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault,
                                                &qres);
        if (e != cudaSuccess || qres != cudaDriverEntryPointSuccess || !sym)
            return qk::fail(QK_ERR_CUDA, "cuTensorMapEncodeTiled is not available: %s",
                            cudaGetErrorString(e));
        fn = (EncodeTiledFn)sym;
    }
    const cuuint64_t dims[2] = {pitch, rows};             // innermost first
    const cuuint64_t strides[1] = {pitch * 2};            // bytes between rows
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void *)base, dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return qk::fail(QK_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)r);
    return QK_OK;
}

// Tokens per tile.  The MMA warp's wait-issue-commit loop takes about 530 cycles per chunk
// whatever N is, and N = 256 is 512 cycles of tensor-core work, so a narrower tile is never
// faster per tile; it only helps when there are fewer tokens than that.
// Which units each CTA takes.  Many tiles (a prompt): the units are dealt out evenly, a CTA's
// run crossing tile borders wherever it falls.  Few tiles (a decode batch: at most half as
// many tiles as CTAs): every tile goes to a whole number of CTAs in equal parts, so that no
// CTA has to publish the tail of one tile before it can begin the head of the next - that
// serial step was on the critical path of the launch - and a tile's sharers finish at the same
// time.  A tile is shared by at most seven CTAs (the six partials the head CTA can stage)
// unless that would make a CTA's run longer than sixteen k-chunks.  Returns the grid size.
unsigned plan_ctas(GemmArgs &g, size_t units, const size_t *tiles, size_t n_problems, unsigned sm_count) {
    const size_t most = std::min<size_t>(sm_count, kMaxCtas);
    const size_t ctas = std::max<size_t>(1, std::min<size_t>(most, units / 8));
    size_t tiles_total = 0;
    for (size_t p = 0; p < n_problems; ++p) tiles_total += tiles[p];
    size_t n = 0;
    bool aligned = tiles_total * 2 <= ctas;
    if (aligned) {
        for (size_t p = 0; p < n_problems && aligned; ++p) {
            const size_t k = g.p[p].k_chunks;
            size_t share = std::max<size_t>(1, std::min<size_t>(k, k * ctas / units));
            if (share > 7 && qk::ceil_div(k, 7) <= 16) share = 7;
            for (size_t t = 0; t < tiles[p] && aligned; ++t)
                for (size_t j = 0; j < share; ++j) {
                    if (n >= most) {
                        aligned = false;
                        break;
                    }
                    g.cta_begin[n++] = (uint32_t)(g.p[p].unit_begin + t * k + j * k / share);
                }
        }
    }
    if (!aligned) {
        n = ctas;
        for (size_t i = 0; i < n; ++i) g.cta_begin[i] = (uint32_t)((uint64_t)i * units / n);
    }
    g.cta_begin[n] = (uint32_t)units;
    return (unsigned)n;
}

uint32_t pick_bn(size_t tokens) {
    return tokens >= (size_t)kBNMax ? (uint32_t)kBNMax : (uint32_t)(qk::ceil_div(tokens, 16) * 16);
}

}  // namespace

static qk_status apply_prefill(qk_ctx *ctx, const qk_layer *const *layers, size_t n_layers, const float *x_dev,
                               const float *up_dev, size_t n_tokens, float *const *y_devs) {
    if (n_layers == 0 || n_layers > (size_t)kMaxProblems)
        return qk::fail(QK_ERR_VALUE, "between 1 and %d layers per call, got %zu", kMaxProblems, n_layers);
    if (!layers || !y_devs) return qk::fail(QK_ERR_VALUE, "qk_layers_apply_prefill: null array");
    for (size_t i = 0; i < n_layers; ++i) {
        if (!layers[i]) return qk::fail(QK_ERR_VALUE, "qk_layers_apply_prefill: layer %zu is null", i);
        if (layers[i]->serving != QK_BF16)
            return qk::fail(QK_ERR_VALUE,
                            "the tensor-core prefill computes in bfloat16 with float32 accumulation; "
                            "it needs a layer created with the bfloat16 serving dtype");
        if (layers[i]->din != layers[0]->din)
            return qk::fail(QK_ERR_VALUE, "layers of one call share their input: layer %zu has din=%zu, "
                            "layer 0 has din=%zu", i, layers[i]->din, layers[0]->din);
    }
    if (n_tokens == 0) return QK_OK;
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    for (size_t i = 0; i < n_layers; ++i)
        if (layers[i]->device != c->device)
            return qk::fail(QK_ERR_VALUE, "layer lives on device %d, context on device %d",
                            layers[i]->device, c->device);
    const size_t din = layers[0]->din;
    const size_t kp1 = qk::ceil_div(din, kBK) * kBK;
    // scratch: per layer z [T][kp1] and t [T][kp2] in bfloat16; the error word and the CTA
    // flags live for the context's life
    const size_t z_bytes = qk::ceil_div(n_tokens * kp1 * 2, 256) * 256;
    size_t kp2[kMaxProblems], t_off[kMaxProblems], need = n_layers * z_bytes;
    for (size_t i = 0; i < n_layers; ++i) {
        kp2[i] = qk::ceil_div(layers[i]->r, kBK) * kBK;
        t_off[i] = need;
        need += qk::ceil_div(n_tokens * kp2[i] * 2, 256) * 256;
    }
    if ((st = c->d_z.reserve(need)) != QK_OK) return st;
    if ((st = qk::error_word(c)) != QK_OK) return st;  // error word + CTA flags
    uint8_t *base = (uint8_t *)c->d_z.ptr;
    int *err = (int *)c->d_err.ptr;
    ScaleArgs sa{};
    for (size_t i = 0; i < n_layers; ++i) {
        sa.s2[i] = layers[i]->s2;
        sa.z[i] = (uint16_t *)(base + i * z_bytes);
    }
    const int vec = ((uintptr_t)x_dev & 15) == 0 && ((uintptr_t)up_dev & 15) == 0 && (din & 3) == 0;
    const size_t total = n_tokens * (kp1 / 8);
    (void)qk::launch_pdl(c->pdl, scale_to_bf16_kernel,
                         dim3((unsigned)qk::ceil_div(total, 256), (unsigned)n_layers), dim3(256), 0, c->stream, x_dev,
                         up_dev, sa, (uint32_t)n_tokens, (uint32_t)din, (uint32_t)kp1, vec);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    QK_CUDA(cudaFuncSetAttribute(factorized_gemm_tc_kernel<false>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
    QK_CUDA(cudaFuncSetAttribute(factorized_gemm_tc_kernel<true>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
    const uint32_t bn = pick_bn(n_tokens);
    const size_t tok_tiles = qk::ceil_div(n_tokens, bn);
    uint32_t *flags = (uint32_t *)c->d_err.ptr + 64;  // after the error word's 256 bytes
    GemmArgs g1{}, g2{};
    CUtensorMap maps1[kMaxProblems], maps2[kMaxProblems];
    size_t units1 = 0, units2 = 0, tiles1[kMaxProblems] = {}, tiles2[kMaxProblems] = {};
    for (size_t i = 0; i < n_layers; ++i) {
        const qk_layer *L = layers[i];
        uint16_t *z = (uint16_t *)(base + i * z_bytes), *t = (uint16_t *)(base + t_off[i]);
        if ((st = encode_activation_map(z, n_tokens, kp1, bn, &maps1[i])) != QK_OK) return st;
        if ((st = encode_activation_map(t, n_tokens, kp2[i], bn, &maps2[i])) != QK_OK) return st;
        const size_t rows1 = qk::ceil_div(kp2[i], kBM), rows2 = qk::ceil_div(L->dout, kBM);
        g1.p[i] = Problem{L->vbt, t, nullptr, nullptr, (uint32_t)L->r, (uint32_t)(kp1 / kBK),
                          (uint32_t)L->vbt_stride, (uint32_t)kp2[i], (uint32_t)rows1, (uint32_t)units1};
        g2.p[i] = Problem{L->ub, y_devs[i], L->s1, L->bias, (uint32_t)L->dout, (uint32_t)(kp2[i] / kBK),
                          (uint32_t)L->ub_stride, (uint32_t)L->dout, (uint32_t)rows2, (uint32_t)units2};
        tiles1[i] = rows1 * tok_tiles;
        tiles2[i] = rows2 * tok_tiles;
        units1 += rows1 * tok_tiles * (kp1 / kBK);
        units2 += rows2 * tok_tiles * (kp2[i] / kBK);
    }
    for (size_t i = n_layers; i < (size_t)kMaxProblems; ++i) {  // unused slots: valid descriptors
        maps1[i] = maps1[0];
        maps2[i] = maps2[0];
    }
    if (units1 >= (1ull << 32) || units2 >= (1ull << 32))
        return qk::fail(QK_ERR_VALUE, "the work of one call must stay below 2^32 tile-chunks");
    // (tile, k-chunk) units per CTA: about eight or more
    const unsigned grid1 = plan_ctas(g1, units1, tiles1, n_layers, (unsigned)c->sm_count);
    const unsigned grid2 = plan_ctas(g2, units2, tiles2, n_layers, (unsigned)c->sm_count);
    const size_t slot_bytes = (size_t)kBNMax * kBM * sizeof(float);
    if ((st = c->d_t.reserve((size_t)std::max(grid1, grid2) * slot_bytes)) != QK_OK) return st;
    float *partials = (float *)c->d_t.ptr;
    g1.n_problems = g2.n_problems = (uint32_t)n_layers;
    g1.error = g2.error = err;
    g1.tokens = g2.tokens = (uint32_t)n_tokens;
    g1.bn = g2.bn = bn;
    g1.units = (uint32_t)units1;
    g2.units = (uint32_t)units2;
    g1.partials = g2.partials = partials;
    g1.flags = g2.flags = flags;
    g1.wait_limit = g2.wait_limit = c->wait_limit ? c->wait_limit : kWaitLimitDefault;
    (void)qk::launch_pdl(c->pdl, factorized_gemm_tc_kernel<false>, dim3(grid1), dim3(kThreads), kSmemBytes,
                         c->stream, maps1[0], maps1[1], maps1[2], maps1[3], g1);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    (void)qk::launch_pdl(c->pdl, factorized_gemm_tc_kernel<true>, dim3(grid2), dim3(kThreads), kSmemBytes,
                         c->stream, maps2[0], maps2[1], maps2[2], maps2[3], g2);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    c->err_armed = true;
    return QK_OK;
}

extern "C" {

qk_status qk_layers_apply_prefill(qk_ctx *ctx, const qk_layer *const *layers, size_t n_layers,
                                  const float *x_dev, size_t n_tokens, float *const *y_devs) {
    return apply_prefill(ctx, layers, n_layers, x_dev, nullptr, n_tokens, y_devs);
}

qk_status qk_layers_apply_prefill_gated(qk_ctx *ctx, const qk_layer *const *layers, size_t n_layers,
                                        const float *gate_dev, const float *up_dev, size_t n_tokens,
                                        float *const *y_devs) {
    if (!gate_dev || !up_dev)
        return qk::fail(QK_ERR_VALUE, "qk_layers_apply_prefill_gated: gate and up must be given");
    return apply_prefill(ctx, layers, n_layers, gate_dev, up_dev, n_tokens, y_devs);
}

qk_status qk_prefill_work_split(size_t n_problems, const size_t *tiles, const size_t *k_chunks,
                                size_t sm_count, uint32_t *cta_begin, size_t cta_begin_len, size_t *n_ctas) {
    if (n_problems == 0 || n_problems > (size_t)kMaxProblems || !tiles || !k_chunks || !cta_begin || !n_ctas)
        return qk::fail(QK_ERR_VALUE, "qk_prefill_work_split: between 1 and %d problems and all arrays", kMaxProblems);
    if (sm_count == 0) return qk::fail(QK_ERR_VALUE, "qk_prefill_work_split: sm_count must be positive");
    GemmArgs g{};
    size_t units = 0;
    for (size_t p = 0; p < n_problems; ++p) {
        if (tiles[p] == 0 || k_chunks[p] == 0)
            return qk::fail(QK_ERR_VALUE, "qk_prefill_work_split: problem %zu is empty", p);
        g.p[p].k_chunks = (uint32_t)k_chunks[p];
        g.p[p].unit_begin = (uint32_t)units;
        units += tiles[p] * k_chunks[p];
    }
    if (units >= (1ull << 32))
        return qk::fail(QK_ERR_VALUE, "the work of one call must stay below 2^32 tile-chunks");
    const unsigned n = plan_ctas(g, units, tiles, n_problems, (unsigned)std::min<size_t>(sm_count, 1u << 20));
    if (cta_begin_len < (size_t)n + 1)
        return qk::fail(QK_ERR_VALUE, "cta_begin holds %zu entries; %u are needed", cta_begin_len, n + 1);
    for (unsigned i = 0; i <= n; ++i) cta_begin[i] = g.cta_begin[i];
    *n_ctas = n;
    return QK_OK;
}

qk_status qk_layer_apply_prefill(qk_ctx *ctx, const qk_layer *layer, const float *x_dev,
                                 size_t n_tokens, float *y_dev) {
    if (!layer) return qk::fail(QK_ERR_VALUE, "qk_layer_apply_prefill: layer is null");
    return qk_layers_apply_prefill(ctx, &layer, 1, x_dev, n_tokens, &y_dev);
}

}  // extern "C"
