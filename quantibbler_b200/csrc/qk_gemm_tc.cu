// Prefill GEMM of the factorized linear on the 5th-generation tensor cores (tcgen05 + TMEM).
//
// For T tokens at once the two stages of y = s1 * (Ub (Vb^T (s2 * x))) + bias are dense
// contractions: stage 1 is [T x din] . [r x din]^T, stage 2 is [T x r] . [dout x r]^T.  This
// is the column-batched product of crates/quantibbler-kernels/src/core.rs:288-317
// (packed_matmul) under the bfloat16 serving contract of
// crates/quantibbler-server/src/engine/mod.rs:449-460 (apply_bf16): operands bfloat16,
// float32 accumulation, z, t and u each rounded once to bfloat16.
//
// tcgen05 has no 1-bit x bf16 mode, so the +-1 weights are expanded to bfloat16 on the fly:
// The weights take the M side of the MMA (128 weight rows per tile) and the tokens the N
// side (up to 256 tokens), so that the costly operand - the one that has to be expanded -
// is the narrow one:
//   * the activation tile (up to 256 tokens x 64 k) is brought to shared memory by TMA
//     (cp.async.bulk.tensor, 128-byte swizzle, one CTA per copy) in the K-major layout the
//     UMMA descriptors expect; rows beyond the token count are zero-filled by the copy;
//   * each of 128 producer threads owns one weight row: it reads the row's bits sixteen
//     bytes at a time, two such loads ahead, and writes 64 bfloat16 +-1 values per stage
//     (eight 16-byte pieces, each from two lookups in a conflict-free 16-entry nibble table)
//     into the same swizzled layout: 16 KB per stage from 1 KB of bits;
//   * one elected thread issues tcgen05.mma (M = 128, N = tokens, K = 16 per instruction,
//     four per stage) with the float32 accumulator in tensor memory, and tcgen05.commit
//     releases the stage to the producers;
//   * the epilogue reads the accumulator with tcgen05.ld (one weight row per thread, so a
//     warp's stores to the token-major output are contiguous), applies the stage's
//     rounding / scale / bias and stores.
// A four-deep ring of stages is synchronised with mbarriers.  Every wait is bounded: on
// expiry the kernel records an error code, frees its tensor memory and returns, and the
// host reports QK_ERR_TIMEOUT.
#include <cuda.h>  // CUtensorMap types only; the encoder is fetched through the runtime

#include <cstring>

#include "qk_common.h"

namespace {

constexpr int kBM = 128;        // weight rows per tile (UMMA M)
constexpr int kBNMax = 256;     // tokens per tile (UMMA N): 128, 160, 192 or 256
constexpr int kBK = 64;         // k per stage: one 128-byte swizzle row of bfloat16
constexpr int kStages = 4;
constexpr int kProducers = 128; // warps 0..3: producers, then epilogue
constexpr int kThreads = kProducers + 32;  // + warp 4: MMA issue and tensor-memory owner
constexpr uint32_t kABytes = kBM * kBK * 2, kBBytes = kBNMax * kBK * 2;  // A: weights, B: tokens
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kWaitLimit = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait: false if the phase did not complete within the limit.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t i = 0; i < kWaitLimit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            " selp.u32 %0, 1, 0, p;\n}"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
// UMMA shared-memory descriptor for a K-major, 128-byte-swizzled tile whose rows are 128
// bytes and whose 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);   // start address
    d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset: 8 rows
    d |= (uint64_t)1 << 46;                        // descriptor version
    d |= (uint64_t)2 << 61;                        // SWIZZLE_128B
    return d;
}
// Instruction descriptor: bf16 x bf16 -> f32, both operands K-major, M = 128, N = bn.
__device__ __forceinline__ uint32_t umma_idesc(uint32_t bn) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((bn >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
}

struct GemmArgs {
    const uint8_t *w_rows; // weight bits, rows padded to w_stride bytes
    void *out;             // bf16 [tokens][out_pitch] (stage 1) or float [tokens][n_rows]
    const float *out_scale, *out_bias;
    int *error;
    uint32_t tokens, n_rows, k_chunks, w_stride, out_pitch, bn;  // bn: tokens per tile
};

// kFinal = false: out = bf16(acc) as the next stage's activation;  true: y = bf16(acc)*s1 + bias.
template <bool kFinal>
__global__ void __launch_bounds__(kThreads, 1)
factorized_gemm_tc_kernel(const __grid_constant__ CUtensorMap b_map, GemmArgs g) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // 1024-byte alignment of the tiles is what the swizzle pattern assumes
    uint8_t *tiles = reinterpret_cast<uint8_t *>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint2 *lut = reinterpret_cast<uint2 *>(tiles + kStages * kStageBytes);
    uint64_t *full = reinterpret_cast<uint64_t *>(lut + 16);
    uint64_t *empty = full + kStages;
    uint64_t *acc_full = empty + kStages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(acc_full + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const uint32_t tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t kBN = g.bn;
    const uint32_t n0 = blockIdx.x * kBM;   // first weight row of the tile
    const uint32_t t0 = blockIdx.y * kBN;   // first token of the tile

    // nibble -> four bfloat16 +-1 values (bit i of the nibble is element i).  Entry e sits in
    // banks 2e and 2e+1, so lookups of different entries never collide.
    if (tid < 16) {
        uint32_t w[2];
#pragma unroll
        for (int p = 0; p < 2; ++p) {
            uint32_t lo = (tid >> (2 * p)) & 1 ? 0x3F80u : 0xBF80u;
            uint32_t hi = (tid >> (2 * p + 1)) & 1 ? 0x3F80u : 0xBF80u;
            w[p] = lo | (hi << 16);
        }
        lut[tid] = make_uint2(w[0], w[1]);
    }
    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], kProducers + 1);  // every producer + the TMA issuer's expect_tx
            mbar_init(&empty[s], 1);
        }
        mbar_init(acc_full, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                         smem_u32(tmem_slot)),
                     "r"((uint32_t)kBNMax)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 4) {
        // ------------------------------------------------------------ producers
        // thread tid expands weight row n0 + tid.  Its bits arrive 16 bytes (two k-chunks)
        // per load, and the loads run two pairs ahead of the expansion.
        const bool live = n0 + tid < g.n_rows;
        const uint4 *wrow = reinterpret_cast<const uint4 *>(g.w_rows + (size_t)(n0 + tid) * g.w_stride);
        const uint32_t n_pairs = (g.k_chunks + 1) / 2;
        const uint4 zero4 = make_uint4(0, 0, 0, 0);
        uint4 q0 = live && 0 < n_pairs ? wrow[0] : zero4;
        uint4 q1 = live && 1 < n_pairs ? wrow[1] : zero4;
        bool dead = false;
        for (uint32_t pair = 0; pair < n_pairs && !dead; ++pair) {
            const uint4 cur = q0;
            q0 = q1;
            q1 = live && pair + 2 < n_pairs ? wrow[pair + 2] : zero4;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint32_t kc = pair * 2 + h;
                if (kc >= g.k_chunks) break;
                const uint32_t s = kc % kStages, it = kc / kStages;
                if (!mbar_wait(&empty[s], (it & 1) ^ 1) || *abort_flag) {
                    *abort_flag = 1;
                    dead = true;
                    break;
                }
                uint8_t *a_tile = tiles + s * kStageBytes, *b_tile = a_tile + kABytes;
                if (tid == 0) {
                    // tokens: one TMA box of 64 k x bn tokens, completing on the full barrier
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(
                                     smem_u32(&full[s])),
                                 "r"(kBN * kBK * 2)
                                 : "memory");
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes "
                        "[%0], [%1, {%2, %3}], [%4];" ::"r"(smem_u32(b_tile)),
                        "l"(&b_map), "r"(kc * kBK), "r"(t0), "r"(smem_u32(&full[s]))
                        : "memory");
                }
                const uint32_t lo = h ? cur.z : cur.x, hi = h ? cur.w : cur.y;
                uint4 *dst = reinterpret_cast<uint4 *>(a_tile + tid * 128);
#pragma unroll
                for (int c = 0; c < 8; ++c) {
                    const uint32_t byte = ((c < 4 ? lo : hi) >> (8 * (c & 3))) & 0xff;
                    const uint2 e0 = lut[byte & 15], e1 = lut[byte >> 4];
                    dst[c ^ (tid & 7)] = live ? make_uint4(e0.x, e0.y, e1.x, e1.y) : zero4;
                }
                // generic-proxy writes must be visible to the tensor core's async proxy
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(&full[s]);
            }
        }
    } else if (lane == 0) {
        // ------------------------------------------------------------ MMA issue (one thread)
        const uint32_t idesc = umma_idesc(kBN);
        for (uint32_t kc = 0; kc < g.k_chunks; ++kc) {
            const uint32_t s = kc % kStages, it = kc / kStages;
            if (!mbar_wait(&full[s], it & 1)) {
                *abort_flag = 1;
                break;
            }
            if (*abort_flag) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_addr = smem_u32(tiles + s * kStageBytes), b_addr = a_addr + kABytes;
#pragma unroll
            for (int k = 0; k < kBK / 16; ++k) {
                const uint64_t ad = umma_desc(a_addr + k * 32), bd = umma_desc(b_addr + k * 32);
                const uint32_t accumulate = (kc | k) ? 1u : 0u;
                asm volatile(
                    "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
                    " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}" ::"r"(tmem_base),
                    "l"(ad), "l"(bd), "r"(idesc), "r"(accumulate)
                    : "memory");
            }
            // the stage may be refilled once these MMAs have read it
            asm volatile(
                "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                    smem_u32(&empty[s]))
                : "memory");
        }
        asm volatile(
            "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                smem_u32(acc_full))
            : "memory");
    }

    // ---------------------------------------------------------------- epilogue (warps 0..3)
    // thread = weight row n (tensor-memory lane), columns = tokens
    if (warp < 4) {
        bool ok = !*abort_flag && mbar_wait(acc_full, 0);
        ok = __all_sync(0xffffffffu, ok);  // tcgen05.ld below needs the whole warp
        if (!ok) *abort_flag = 1;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t n = n0 + warp * 32 + lane;
        const bool n_live = kFinal ? n < g.n_rows : n < g.out_pitch;
        const float scale = (kFinal && g.out_scale && n < g.n_rows) ? g.out_scale[n] : 1.f;
        const float bias = (kFinal && g.out_bias && n < g.n_rows) ? g.out_bias[n] : 0.f;
        if (ok) {
            for (uint32_t c0 = 0; c0 < kBN; c0 += 32) {
                if (t0 + c0 >= g.tokens) break;  // warp-uniform
                uint32_t v[32];
                const uint32_t taddr = tmem_base + ((warp * 32) << 16) + c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                    "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, "
                    "[%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]),
                      "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]),
                      "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]),
                      "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                      "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]),
                      "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (n_live) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t tok = t0 + c0 + j;
                        if (tok >= g.tokens) break;
                        // one rounding to bfloat16, as packed_matmul's bf16 instantiation does
                        const uint32_t u = v[j];
                        const uint32_t rb = (u & 0x7fffffffu) > 0x7f800000u
                                                ? ((u | 0x00400000u) & 0xffff0000u)
                                                : ((u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u);
                        if (kFinal) {
                            static_cast<float *>(g.out)[(size_t)tok * g.n_rows + n] =
                                __uint_as_float(rb) * scale + bias;
                        } else {
                            static_cast<uint16_t *>(g.out)[(size_t)tok * g.out_pitch + n] =
                                n < g.n_rows ? (uint16_t)(rb >> 16) : (uint16_t)0;
                        }
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 4) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base),
                     "r"((uint32_t)kBNMax)
                     : "memory");
    }
    if (tid == 0 && *abort_flag) atomicExch(g.error, 1);
}

// z = bf16(s2 * x) (float32 product, one rounding), zero padded to the pitch.
__global__ void scale_to_bf16_kernel(const float *__restrict__ x, const float *__restrict__ s2,
                                     uint16_t *__restrict__ z, uint32_t n_tokens, uint32_t din,
                                     uint32_t pitch) {
    size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (size_t)n_tokens * pitch) return;
    uint32_t t = (uint32_t)(idx / pitch), k = (uint32_t)(idx % pitch);
    uint16_t r = 0;
    if (k < din) {
        float v = s2[k] * x[(size_t)t * din + k];
        uint32_t u = __float_as_uint(v);
        r = (u & 0x7fffffffu) > 0x7f800000u ? (uint16_t)((u >> 16) | 0x0040u)
                                            : (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
    }
    z[idx] = r;
}

constexpr size_t kSmemBytes = 1024 + kStages * kStageBytes + 16 * 8 + (2 * kStages + 1) * 8 + 16;

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

// The N tile that wastes the least of the last wave (ties go to the larger tile).
uint32_t pick_bn(size_t row_tiles, size_t tokens, int sms) {
    const uint32_t cands[4] = {256, 192, 160, 128};
    uint32_t best = 256;
    double best_cost = 1e30;
    for (uint32_t bn : cands) {
        size_t tiles = row_tiles * qk::ceil_div(tokens, bn);
        size_t waves = qk::ceil_div(tiles, (size_t)sms);
        // time ~ waves x (per-tile work ~ bn, plus a fixed cost per tile)
        double cost = (double)waves * (bn + 24.0);
        if (cost < best_cost - 1e-9) {
            best_cost = cost;
            best = bn;
        }
    }
    return best;
}

}  // namespace

extern "C" {

qk_status qk_layer_apply_prefill(qk_ctx *ctx, const qk_layer *layer, const float *x_dev,
                                 size_t n_tokens, float *y_dev) {
    if (!layer) return qk::fail(QK_ERR_VALUE, "qk_layer_apply_prefill: layer is null");
    if (layer->serving != QK_BF16)
        return qk::fail(QK_ERR_VALUE,
                        "the tensor-core prefill computes in bfloat16 with float32 accumulation; "
                        "it needs a layer created with the bfloat16 serving dtype");
    if (n_tokens == 0) return QK_OK;
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    if (layer->device != c->device)
        return qk::fail(QK_ERR_VALUE, "layer lives on device %d, context on device %d",
                        layer->device, c->device);
    const size_t din = layer->din, r = layer->r, dout = layer->dout;
    const size_t kp1 = qk::ceil_div(din, kBK) * kBK, kp2 = qk::ceil_div(r, kBK) * kBK;
    // scratch: z [T][kp1] bf16, t [T][kp2] bf16, error word
    const size_t z_bytes = qk::ceil_div(n_tokens * kp1 * 2, 256) * 256;
    const size_t t_bytes = qk::ceil_div(n_tokens * kp2 * 2, 256) * 256;
    if ((st = c->d_z.reserve(z_bytes + t_bytes + 256)) != QK_OK) return st;
    uint16_t *z = (uint16_t *)c->d_z.ptr;
    uint16_t *t = (uint16_t *)((uint8_t *)c->d_z.ptr + z_bytes);
    int *err = (int *)((uint8_t *)c->d_z.ptr + z_bytes + t_bytes);
    QK_CUDA(cudaMemsetAsync(err, 0, sizeof(int), c->stream));
    const size_t total = n_tokens * kp1;
    scale_to_bf16_kernel<<<(unsigned)qk::ceil_div(total, 256), 256, 0, c->stream>>>(
        x_dev, layer->s2, z, (uint32_t)n_tokens, (uint32_t)din, (uint32_t)kp1);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    QK_CUDA(cudaFuncSetAttribute(factorized_gemm_tc_kernel<false>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
    QK_CUDA(cudaFuncSetAttribute(factorized_gemm_tc_kernel<true>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes));
    const size_t rows1 = qk::ceil_div(kp2, kBM), rows2 = qk::ceil_div(dout, kBM);
    const uint32_t bn1 = pick_bn(rows1, n_tokens, c->sm_count);
    const uint32_t bn2 = pick_bn(rows2, n_tokens, c->sm_count);
    CUtensorMap map1, map2;
    if ((st = encode_activation_map(z, n_tokens, kp1, bn1, &map1)) != QK_OK) return st;
    if ((st = encode_activation_map(t, n_tokens, kp2, bn2, &map2)) != QK_OK) return st;
    GemmArgs g1{layer->vbt, t, nullptr, nullptr, err, (uint32_t)n_tokens, (uint32_t)r,
                (uint32_t)(kp1 / kBK), (uint32_t)layer->vbt_stride, (uint32_t)kp2, bn1};
    dim3 grid1((unsigned)rows1, (unsigned)qk::ceil_div(n_tokens, bn1));
    factorized_gemm_tc_kernel<false><<<grid1, kThreads, kSmemBytes, c->stream>>>(map1, g1);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    GemmArgs g2{layer->ub, y_dev, layer->s1, layer->bias, err, (uint32_t)n_tokens, (uint32_t)dout,
                (uint32_t)(kp2 / kBK), (uint32_t)layer->ub_stride, (uint32_t)dout, bn2};
    dim3 grid2((unsigned)rows2, (unsigned)qk::ceil_div(n_tokens, bn2));
    factorized_gemm_tc_kernel<true><<<grid2, kThreads, kSmemBytes, c->stream>>>(map2, g2);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    int h_err = 0;
    QK_CUDA(cudaMemcpyAsync(&h_err, err, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
    QK_CUDA(cudaStreamSynchronize(c->stream));
    if (h_err)
        return qk::fail(QK_ERR_TIMEOUT,
                        "the tensor-core prefill gave up waiting on a pipeline barrier");
    return QK_OK;
}

}  // extern "C"
