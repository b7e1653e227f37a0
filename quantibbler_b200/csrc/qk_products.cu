// Parity faces of the packed products: host buffers in, host buffers out, results
// bit-identical to the reference.
//
// Replaces crates/quantibbler-kernels/src/gpu.rs:47-73 (packed_matvec_kernel) and the
// device route for core.rs:247-260 / :288-317.  Like the reference's device kernel,
// each output element is produced by one thread that walks its row's bits in element
// order and accumulates left to right in the dtype's accumulator (f64 -> f64,
// f32 -> f32, bf16 -> f32 with one rounding at the end; dtype.rs:45-92).  Every term is
// exactly +-v, so the sum is the same sequence of roundings as the CPU faces and the
// NumPy reference perform: the outputs match them bit for bit, which the tests check.
// These kernels are the correctness lane; the bandwidth-bound path is qk_gemv.cu.
#include <cstring>

#include "qk_common.h"

namespace {

template <typename T>
struct Acc;
template <>
struct Acc<double> {
    using type = double;
    __device__ static double load(const double *p, size_t i) { return p[i]; }
    __device__ static double add(double a, double b) { return __dadd_rn(a, b); }
    __device__ static void store(double *p, size_t i, double a) { p[i] = a; }
};
template <>
struct Acc<float> {
    using type = float;
    __device__ static float load(const float *p, size_t i) { return p[i]; }
    __device__ static float add(float a, float b) { return __fadd_rn(a, b); }
    __device__ static void store(float *p, size_t i, float a) { p[i] = a; }
};
// bf16 travels as uint16 bit patterns
template <>
struct Acc<uint16_t> {
    using type = float;
    __device__ static float load(const uint16_t *p, size_t i) {
        return __uint_as_float((uint32_t)p[i] << 16);
    }
    __device__ static float add(float a, float b) { return __fadd_rn(a, b); }
    __device__ static void store(uint16_t *p, size_t i, float a) {
        uint32_t u = __float_as_uint(a);
        uint16_t r;
        if ((u & 0x7fffffffu) > 0x7f800000u)
            r = (uint16_t)((u >> 16) | 0x0040u);
        else
            r = (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
        p[i] = r;
    }
};

// out[i*kc + j] = sum_t sign(i,t) * mat[t*n_cols + j], t ascending.  One thread per
// output element, j fastest so that a warp's loads of mat are contiguous.
template <typename T>
__global__ void __launch_bounds__(128)
sequential_product_kernel(const uint8_t *__restrict__ packed, const T *__restrict__ mat,
                          T *__restrict__ out, uint32_t n_rows, uint32_t n_bits,
                          uint32_t row_words, uint32_t kc, uint32_t n_cols) {
    uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (gid >= (uint64_t)n_rows * kc) return;
    uint32_t i = (uint32_t)(gid / kc);
    uint32_t j = (uint32_t)(gid % kc);
    const uint8_t *row = packed + (size_t)i * row_words;
    typename Acc<T>::type acc = 0;
    for (uint32_t base = 0; base < n_bits; base += 8) {
        uint32_t byte = row[base >> 3];
        uint32_t lim = n_bits - base < 8 ? n_bits - base : 8;
        for (uint32_t k = 0; k < lim; ++k) {
            typename Acc<T>::type v = Acc<T>::load(mat, (size_t)(base + k) * n_cols + j);
            acc = Acc<T>::add(acc, ((byte >> k) & 1u) ? v : -v);
        }
    }
    Acc<T>::store(out, gid, acc);
}

size_t dtype_size(int32_t dtype) { return dtype == QK_F64 ? 8 : dtype == QK_F32 ? 4 : 2; }

// Upload, launch, download; shared by every host-buffer product.
qk_status run_product(qk_ctx *c, const uint8_t *packed, size_t packed_len, size_t n_rows,
                      size_t n_bits, size_t n_words, int32_t dtype, const void *mat,
                      size_t mat_len, size_t n_cols, size_t kc, void *out) {
    size_t es = dtype_size(dtype);
    size_t out_elems = n_rows * kc;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    qk_status st;
    if ((st = c->d_packed.reserve(packed_len)) != QK_OK) return st;
    if ((st = c->d_in.reserve(mat_len * es)) != QK_OK) return st;
    if ((st = c->d_out.reserve(out_elems * es)) != QK_OK) return st;
    QK_CUDA(cudaMemcpyAsync(c->d_packed.ptr, packed, packed_len, cudaMemcpyHostToDevice,
                            c->stream));
    QK_CUDA(cudaMemcpyAsync(c->d_in.ptr, mat, mat_len * es, cudaMemcpyHostToDevice, c->stream));
    uint32_t threads = 128;
    uint32_t blocks = (uint32_t)qk::ceil_div(out_elems, threads);
    const uint8_t *p = (const uint8_t *)c->d_packed.ptr;
    switch (dtype) {
        case QK_F64:
            sequential_product_kernel<double><<<blocks, threads, 0, c->stream>>>(
                p, (const double *)c->d_in.ptr, (double *)c->d_out.ptr, (uint32_t)n_rows,
                (uint32_t)n_bits, (uint32_t)n_words, (uint32_t)kc, (uint32_t)n_cols);
            break;
        case QK_F32:
            sequential_product_kernel<float><<<blocks, threads, 0, c->stream>>>(
                p, (const float *)c->d_in.ptr, (float *)c->d_out.ptr, (uint32_t)n_rows,
                (uint32_t)n_bits, (uint32_t)n_words, (uint32_t)kc, (uint32_t)n_cols);
            break;
        default:
            sequential_product_kernel<uint16_t><<<blocks, threads, 0, c->stream>>>(
                p, (const uint16_t *)c->d_in.ptr, (uint16_t *)c->d_out.ptr, (uint32_t)n_rows,
                (uint32_t)n_bits, (uint32_t)n_words, (uint32_t)kc, (uint32_t)n_cols);
            break;
    }
    QK_CUDA(cudaGetLastError());
    c->launches++;
    QK_CUDA(cudaMemcpyAsync(out, c->d_out.ptr, out_elems * es, cudaMemcpyDeviceToHost,
                            c->stream));
    QK_CUDA(cudaStreamSynchronize(c->stream));
    return QK_OK;
}

// gpu.rs:130-137: the device index arithmetic is 32-bit; larger shapes are refused.
qk_status check_ceiling(size_t n_rows, size_t n_words) {
    uint64_t lin = (uint64_t)n_rows * (uint64_t)n_words;
    if (lin > qk::kIndexCeiling || (uint64_t)n_rows > qk::kIndexCeiling)
        return qk::fail(QK_ERR_VALUE,
                        "packed shape %zu x %zu words exceeds the device u32 index ceiling "
                        "(%llu); use the CPU rlib face",
                        n_rows, n_words, (unsigned long long)qk::kIndexCeiling);
    return QK_OK;
}

}  // namespace

extern "C" {

qk_status qk_packed_matvec(qk_ctx *ctx, const uint8_t *packed, size_t packed_len, size_t n_rows,
                           size_t n_bits, int32_t dtype, const void *vec, size_t vec_len,
                           void *out) {
    if (dtype < QK_F64 || dtype > QK_BF16)
        return qk::fail(QK_ERR_VALUE, "unknown kernel dtype tag %d", dtype);
    size_t n_words = 0;
    qk_status st = qk::validate_packed(packed_len, n_rows, n_bits, &n_words);
    if (st != QK_OK) return st;
    if (vec_len != n_bits)
        return qk::fail(QK_ERR_VALUE, "vec must have length %zu, got %zu", n_bits, vec_len);
    if ((st = check_ceiling(n_rows, n_words)) != QK_OK) return st;
    if (n_rows * n_words == 0) {
        // gpu.rs:139-143: degenerate shapes return zeros without a launch
        memset(out, 0, n_rows * dtype_size(dtype));
        return QK_OK;
    }
    qk_ctx *c;
    if ((st = qk::resolve_ctx(ctx, &c)) != QK_OK) return st;
    return run_product(c, packed, packed_len, n_rows, n_bits, n_words, dtype, vec, vec_len, 1, 1,
                       out);
}

qk_status qk_gpu_packed_matvec(qk_ctx *ctx, const uint8_t *packed, size_t packed_len,
                               size_t n_rows, size_t n_bits, const double *vec, size_t vec_len,
                               double *out) {
    return qk_packed_matvec(ctx, packed, packed_len, n_rows, n_bits, QK_F64, vec, vec_len, out);
}

qk_status qk_packed_matmul(qk_ctx *ctx, const uint8_t *packed, size_t packed_len, size_t n_rows,
                           size_t n_bits, int32_t dtype, const void *mat, size_t mat_len,
                           size_t n_cols, void *out, size_t out_len) {
    if (dtype < QK_F64 || dtype > QK_BF16)
        return qk::fail(QK_ERR_VALUE, "unknown kernel dtype tag %d", dtype);
    size_t n_words = 0;
    qk_status st = qk::validate_packed(packed_len, n_rows, n_bits, &n_words);
    if (st != QK_OK) return st;
    if (n_bits != 0 && mat_len % n_bits != 0)
        return qk::fail(QK_ERR_VALUE, "mat length %zu is not a multiple of n_bits %zu", mat_len,
                        n_bits);
    size_t kc = n_bits ? mat_len / n_bits : mat_len;  // core.rs:302
    if (out_len != n_rows * kc)
        return qk::fail(QK_ERR_VALUE, "output length %zu does not match %zux%zu", out_len, n_rows,
                        kc);
    if ((st = check_ceiling(n_rows, n_words)) != QK_OK) return st;
    if (n_rows * kc == 0) return QK_OK;
    if (n_bits == 0) {
        memset(out, 0, out_len * dtype_size(dtype));
        return QK_OK;
    }
    // The kernel reads mat[t*n_cols + j] for t < n_bits, j < kc; an off-nominal n_cols
    // must still stay inside the operand (the reference would panic on the slice).
    if ((n_bits - 1) * n_cols + (kc - 1) >= mat_len)
        return qk::fail(QK_ERR_VALUE,
                        "n_cols %zu addresses beyond the operand: mat length %zu, n_bits %zu",
                        n_cols, mat_len, n_bits);
    if ((uint64_t)mat_len > qk::kIndexCeiling || (uint64_t)out_len > qk::kIndexCeiling)
        return qk::fail(QK_ERR_VALUE,
                        "operand of %zu values exceeds the device u32 index ceiling (%llu); use "
                        "the CPU rlib face",
                        mat_len, (unsigned long long)qk::kIndexCeiling);
    qk_ctx *c;
    if ((st = qk::resolve_ctx(ctx, &c)) != QK_OK) return st;
    return run_product(c, packed, packed_len, n_rows, n_bits, n_words, dtype, mat, mat_len, n_cols,
                       kc, out);
}

}  // extern "C"
