// Decode GEMV over packed +-1 factors and the device-resident factorized linear
//   y = s1 * (Ub (Vb^T (s2 * x))) + bias.
//
// Replaces, for device-resident operation, crates/quantibbler-server/src/engine/mod.rs
// :342-381 (PackedLayer::from_layer) and :393-480 (apply / apply_bf16), whose inner
// loop is crates/quantibbler-kernels/src/core.rs:202-221 (accumulate_row).
//
// Data layout in HBM.  Each factor keeps the reference's per-row bitplane order
// (element k of a row at bit k&7 of byte k>>3) but every row is padded with zero bits
// to a multiple of 16 bytes, so that a lane can fetch 128 weights with one aligned
// 128-bit load and a warp fetches 512 contiguous bytes of one row.  Pad bits are
// cleared when the layer is created; the matching vector entries are zero, so they
// add nothing.
//
// Rounding points.  fp32 serving computes z = s2*x in float32 as the reference does;
// the reference then sums in float64, this kernel sums float32 lane partials combined
// by a fixed butterfly (bit-reproducible run to run), inside the reference's declared
// backward bound for reassociating faces (|delta| <= 1e-6 * sum|v_k|,
// crates/quantibbler-kernels/tests/parity.rs:795).  bf16 serving rounds z, t and u to
// bfloat16 exactly where apply_bf16 does.
#include <cstring>

#include "qk_common.h"

namespace {

constexpr int kWarpsPerBlock = 8;
constexpr int kRowsPerWarp = 4;
constexpr int kChunkBits = 4096;  // 32 lanes x 128 bits

struct StageParams {
    const uint8_t *w;       // rows x stride bytes
    const float *in;        // n_bits values
    const float *in_scale;  // n_bits values or null (s2)
    float *out;             // n_rows values
    const float *out_scale; // n_rows values or null (s1)
    const float *out_bias;  // n_rows values or null
};

__device__ __forceinline__ float round_bf16(float v) {
    uint32_t u = __float_as_uint(v);
    if ((u & 0x7fffffffu) > 0x7f800000u) return __uint_as_float((u | 0x00400000u) & 0xffff0000u);
    u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;
    return __uint_as_float(u);
}

// (bit b of w) ? v : -v: the weight bit is moved onto the sign position and flips
// the sign of v when it is 0.  Compiles to one shift and one three-input logic op.
__device__ __forceinline__ float signed_term(uint32_t w, int b, float v) {
    uint32_t t = w << (31 - b);
    return __uint_as_float(__float_as_uint(v) ^ (~t & 0x80000000u));
}

// One stage of the factorized linear: out[i] = epilogue(sum_k sign(i,k) * prologue(in[k])).
// grid.x tiles the rows, grid.y indexes the layer of a group.
template <bool kRoundBf16>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
gemv_signselect_kernel(const StageParams single, const StageParams *__restrict__ many,
                       uint32_t n_rows, uint32_t n_bits, uint32_t stride) {
    extern __shared__ float vs[];  // permuted copy of the input vector, zero padded
    const StageParams p = many ? many[blockIdx.y] : single;
    const uint32_t n_chunks = (n_bits + kChunkBits - 1) / kChunkBits;
    // stage the vector: element k of chunk c held by lane l = (k/128)%32 at slot e = k%128
    for (uint32_t k = threadIdx.x; k < n_chunks * kChunkBits; k += blockDim.x) {
        float v = 0.f;
        if (k < n_bits) {
            v = p.in[k];
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
        uint4 w[kRowsPerWarp];
#pragma unroll
        for (int r = 0; r < kRowsPerWarp; ++r) {
            w[r] = make_uint4(0, 0, 0, 0);
            if (row0 + r < n_rows && byte_off < stride)
                w[r] = *reinterpret_cast<const uint4 *>(p.w + (size_t)(row0 + r) * stride + byte_off);
        }
        if (byte_off >= stride) continue;  // vector entries there are zero as well
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
            p.out[row0 + r] = a;
        }
    }
}

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

size_t smem_bytes(size_t n_bits) {
    return qk::ceil_div(n_bits, kChunkBits) * kChunkBits * sizeof(float);
}

// `many` (device array, one entry per grid.y index) or, when null, `single` by value.
qk_status launch_stage(qk_ctx *c, const StageParams &single, const StageParams *many,
                       size_t n_layers, size_t n_rows, size_t n_bits, size_t stride, bool bf16) {
    size_t smem = smem_bytes(n_bits);
    dim3 grid((unsigned)qk::ceil_div(n_rows, kWarpsPerBlock * kRowsPerWarp), (unsigned)n_layers);
    auto kern = bf16 ? gemv_signselect_kernel<true> : gemv_signselect_kernel<false>;
    if (smem > 48 * 1024)
        QK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, kWarpsPerBlock * 32, smem, c->stream>>>(single, many, (uint32_t)n_rows,
                                                         (uint32_t)n_bits, (uint32_t)stride);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    return QK_OK;
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
    if (smem_bytes(l0->din) > 200 * 1024 || smem_bytes(l0->r) > 200 * 1024)
        return qk::fail(QK_ERR_VALUE, "input width %zu exceeds the GEMV kernel's staging limit",
                        l0->din > l0->r ? l0->din : l0->r);
    return QK_OK;
}

// Fills 2*n_inst StageParams (stage 1 entries, then stage 2 entries) for n_layers
// same-shape layers x n_tokens tokens.  Instance k = t*n_layers + i reads
// x + i*x_layer_stride + t*din and writes y + i*y_layer_stride + t*dout.
void fill_params(StageParams *h, const qk_layer *const *layers, size_t n_layers, size_t n_tokens,
                 const float *x_dev, float *y_dev, float *t_dev, size_t x_layer_stride,
                 size_t y_layer_stride) {
    const size_t n_inst = n_layers * n_tokens;
    for (size_t t = 0; t < n_tokens; ++t)
        for (size_t i = 0; i < n_layers; ++i) {
            const qk_layer *l = layers[i];
            size_t k = t * n_layers + i;
            const float *x = x_dev + i * x_layer_stride + t * l->din;
            float *y = y_dev + i * y_layer_stride + t * l->dout;
            h[k] = StageParams{l->vbt, x, l->s2, t_dev + k * l->r, nullptr, nullptr};
            h[n_inst + k] = StageParams{l->ub, t_dev + k * l->r, nullptr, y, l->s1, l->bias};
        }
}

qk_status launch_both(qk_ctx *c, const qk_layer *l0, const StageParams *d, size_t n_inst) {
    const bool bf16 = l0->serving == QK_BF16;
    StageParams none{};
    qk_status st = launch_stage(c, none, d, n_inst, l0->r, l0->din, l0->vbt_stride, bf16);
    if (st != QK_OK) return st;
    return launch_stage(c, none, d + n_inst, n_inst, l0->dout, l0->r, l0->ub_stride, bf16);
}

// Both stages for n_layers same-shape layers x n_tokens tokens, parameters built and
// uploaded on the fly.
qk_status apply_group(qk_ctx *c, const qk_layer *const *layers, size_t n_layers, const float *x_dev,
                      float *y_dev, size_t n_tokens, size_t x_layer_stride, size_t y_layer_stride) {
    qk_status st = check_group(c, layers, n_layers);
    if (st != QK_OK) return st;
    const qk_layer *l0 = layers[0];
    const size_t n_inst = n_layers * n_tokens;
    if ((st = c->d_t.reserve(n_inst * l0->r * sizeof(float))) != QK_OK) return st;
    const bool bf16 = l0->serving == QK_BF16;
    if (n_inst == 1) {
        // one layer, one token: parameters travel as kernel arguments, no staging copy
        float *t1 = (float *)c->d_t.ptr;
        StageParams a{l0->vbt, x_dev, l0->s2, t1, nullptr, nullptr};
        StageParams b{l0->ub, t1, nullptr, y_dev, l0->s1, l0->bias};
        if ((st = launch_stage(c, a, nullptr, 1, l0->r, l0->din, l0->vbt_stride, bf16)) != QK_OK)
            return st;
        return launch_stage(c, b, nullptr, 1, l0->dout, l0->r, l0->ub_stride, bf16);
    }
    if ((st = c->d_ptrs.reserve(2 * n_inst * sizeof(StageParams))) != QK_OK) return st;
    void *hp;
    if ((st = c->pinned(2 * n_inst * sizeof(StageParams), &hp)) != QK_OK) return st;
    // the pinned block is reused by the next call: wait for the previous copy out of it
    QK_CUDA(cudaStreamSynchronize(c->stream));
    fill_params((StageParams *)hp, layers, n_layers, n_tokens, x_dev, y_dev, (float *)c->d_t.ptr,
                x_layer_stride, y_layer_stride);
    StageParams *d = (StageParams *)c->d_ptrs.ptr;
    QK_CUDA(cudaMemcpyAsync(d, hp, 2 * n_inst * sizeof(StageParams), cudaMemcpyHostToDevice,
                            c->stream));
    return launch_both(c, l0, d, n_inst);
}

qk_status upload_padded(qk_ctx *c, const uint8_t *host, size_t len, size_t n_rows, size_t n_bits,
                        uint8_t **out, size_t *stride_out) {
    size_t row_words = qk::ceil_div(n_bits, 8);
    size_t stride = qk::ceil_div(row_words, 16) * 16;
    qk_status st;
    if ((st = c->d_packed.reserve(len)) != QK_OK) return st;
    uint8_t *dst = nullptr;
    cudaError_t e = cudaMalloc(&dst, n_rows * stride);
    if (e != cudaSuccess)
        return qk::fail(QK_ERR_ALLOC, "device allocation of %zu bytes failed: %s", n_rows * stride,
                        cudaGetErrorString(e));
    QK_CUDA(cudaMemcpyAsync(c->d_packed.ptr, host, len, cudaMemcpyHostToDevice, c->stream));
    size_t total = n_rows * stride;
    pad_rows_kernel<<<(unsigned)qk::ceil_div(total, 256), 256, 0, c->stream>>>(
        (const uint8_t *)c->d_packed.ptr, dst, (uint32_t)n_rows, (uint32_t)n_bits,
        (uint32_t)row_words, (uint32_t)stride);
    QK_CUDA(cudaGetLastError());
    c->launches++;
    QK_CUDA(cudaStreamSynchronize(c->stream));
    *out = dst;
    *stride_out = stride;
    return QK_OK;
}

qk_status upload_f32(qk_ctx *c, const float *host, size_t n, float **out) {
    float *d = nullptr;
    cudaError_t e = cudaMalloc(&d, n * sizeof(float));
    if (e != cudaSuccess)
        return qk::fail(QK_ERR_ALLOC, "device allocation of %zu bytes failed: %s",
                        n * sizeof(float), cudaGetErrorString(e));
    QK_CUDA(cudaMemcpyAsync(d, host, n * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    QK_CUDA(cudaStreamSynchronize(c->stream));
    *out = d;
    return QK_OK;
}

}  // namespace

extern "C" {

qk_status qk_layer_create(qk_ctx *ctx, const uint8_t *ub_rows, size_t ub_len,
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
    // engine/mod.rs:343-356: both bitplanes must have the per-row layout's exact length
    if (ub_len != dout * qk::ceil_div(r, 8) || vb_t_len != r * qk::ceil_div(din, 8))
        return qk::fail(QK_ERR_VALUE, "bitplane length mismatch after repack");
    if ((uint64_t)dout * qk::ceil_div(r, 8) > qk::kIndexCeiling ||
        (uint64_t)r * qk::ceil_div(din, 8) > qk::kIndexCeiling)
        return qk::fail(QK_ERR_VALUE, "layer exceeds the device u32 index ceiling (%llu)",
                        (unsigned long long)qk::kIndexCeiling);
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
    st = upload_padded(c, ub_rows, ub_len, dout, r, &l->ub, &l->ub_stride);
    if (st == QK_OK) st = upload_padded(c, vb_t_rows, vb_t_len, r, din, &l->vbt, &l->vbt_stride);
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

void qk_layer_free(qk_layer *l) {
    if (!l) return;
    cudaSetDevice(l->device);
    if (l->ub) cudaFree(l->ub);
    if (l->vbt) cudaFree(l->vbt);
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
    if (!layers) return qk::fail(QK_ERR_VALUE, "qk_layers_apply_group: layers is null");
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
    if (n_layers == 0 || !layers) return qk::fail(QK_ERR_VALUE, "qk_group_create: no layers");
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
    cudaError_t e = cudaMalloc(&g->t_dev, n_layers * l0->r * sizeof(float));
    if (e == cudaSuccess) e = cudaMalloc(&g->params, 2 * n_layers * sizeof(StageParams));
    if (e != cudaSuccess) {
        qk_group_free(g);
        return qk::fail(QK_ERR_ALLOC, "device allocation for a layer group failed: %s",
                        cudaGetErrorString(e));
    }
    std::vector<StageParams> h(2 * n_layers);
    fill_params(h.data(), layers, n_layers, 1, x_dev, y_dev, g->t_dev, l0->din, l0->dout);
    QK_CUDA(cudaMemcpyAsync(g->params, h.data(), h.size() * sizeof(StageParams),
                            cudaMemcpyHostToDevice, c->stream));
    QK_CUDA(cudaStreamSynchronize(c->stream));
    *out = g;
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
    return launch_both(c, &group->shape, (const StageParams *)group->params, group->n_inst);
}

void qk_group_free(qk_group *g) {
    if (!g) return;
    cudaSetDevice(g->device);
    if (g->t_dev) cudaFree(g->t_dev);
    if (g->params) cudaFree(g->params);
    delete g;
}

}  // extern "C"
