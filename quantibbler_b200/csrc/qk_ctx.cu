// Device context: the CUDA equivalent of the reference's GpuContext
// (crates/quantibbler-kernels/src/gpu.rs:76-113).  One context owns one stream on one
// device plus reusable staging buffers; every failure to obtain a device is a typed
// QK_ERR_INIT carrying qk_gpu_init_hint(), never a silent fallback.
#include "qk_common.h"

qk_status qk_scratch::reserve(size_t bytes) {
    if (bytes <= cap) return QK_OK;
    if (ptr) cudaFree(ptr);
    ptr = nullptr;
    cap = 0;
    size_t want = bytes < 4096 ? 4096 : bytes;
    cudaError_t e = cudaMalloc(&ptr, want);
    if (e != cudaSuccess) {
        ptr = nullptr;
        return qk::fail(QK_ERR_ALLOC, "device allocation of %zu bytes failed: %s", want,
                        cudaGetErrorString(e));
    }
    cap = want;
    return QK_OK;
}

void qk_scratch::release() {
    if (ptr) cudaFree(ptr);
    ptr = nullptr;
    cap = 0;
}

qk_status qk_ctx::pinned(size_t bytes, void **out, int *slot) {
    PinnedSlot &ps = h_pinned[h_pinned_next];
    *slot = h_pinned_next;
    h_pinned_next = (h_pinned_next + 1) % kPinnedSlots;
    if (ps.in_flight) {
        // only when the ring has come round to a block whose copy has not finished
        QK_CUDA(cudaEventSynchronize(ps.copied));
        ps.in_flight = false;
    }
    if (bytes > ps.cap) {
        if (ps.ptr) cudaFreeHost(ps.ptr);
        ps.ptr = nullptr;
        ps.cap = 0;
        size_t want = bytes < 65536 ? 65536 : bytes;
        cudaError_t e = cudaMallocHost(&ps.ptr, want);
        if (e != cudaSuccess) {
            ps.ptr = nullptr;
            return qk::fail(QK_ERR_ALLOC, "pinned host allocation of %zu bytes failed: %s", want,
                            cudaGetErrorString(e));
        }
        ps.cap = want;
    }
    if (!ps.copied) QK_CUDA(cudaEventCreateWithFlags(&ps.copied, cudaEventDisableTiming));
    *out = ps.ptr;
    return QK_OK;
}

qk_status qk_ctx::pinned_done(int slot) {
    PinnedSlot &ps = h_pinned[slot];
    QK_CUDA(cudaEventRecord(ps.copied, stream));
    ps.in_flight = true;
    return QK_OK;
}

namespace qk {

static std::mutex g_default_mu;
static qk_ctx *g_default_ctx = nullptr;

qk_status resolve_ctx(qk_ctx *ctx, qk_ctx **out) {
    if (ctx) {
        *out = ctx;
        return QK_OK;
    }
    std::lock_guard<std::mutex> lock(g_default_mu);
    if (!g_default_ctx) {
        qk_status st = qk_gpu_init_at(0, &g_default_ctx);
        if (st != QK_OK) return st;
    }
    *out = g_default_ctx;
    return QK_OK;
}

qk_status error_word(qk_ctx *c) {
    if (c->d_err.ptr) return QK_OK;
    qk_status st = c->d_err.reserve(256 + 4096);
    if (st != QK_OK) return st;
    QK_CUDA(cudaMemsetAsync(c->d_err.ptr, 0, 256 + 4096, c->stream));
    return QK_OK;
}

}  // namespace qk

extern "C" {

qk_status qk_gpu_init_at(size_t device_index, qk_ctx **out) {
    if (!out) return qk::fail(QK_ERR_VALUE, "qk_gpu_init_at: out is null");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return qk::fail(QK_ERR_INIT, "%s; device probe failed at index %zu: %s",
                        qk_gpu_init_hint(), device_index, cudaGetErrorString(e));
    }
    if (device_index >= (size_t)count)
        return qk::fail(QK_ERR_INIT,
                        "%s; device probe failed at index %zu: only %d device(s) visible",
                        qk_gpu_init_hint(), device_index, count);
    int dev = (int)device_index;
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, dev);
    if (e != cudaSuccess)
        return qk::fail(QK_ERR_INIT, "%s; device probe failed at index %zu: %s",
                        qk_gpu_init_hint(), device_index, cudaGetErrorString(e));
    if (prop.major != 10)
        return qk::fail(QK_ERR_INIT,
                        "%s; device probe failed at index %zu: %s has compute capability %d.%d",
                        qk_gpu_init_hint(), device_index, prop.name, prop.major, prop.minor);
    e = cudaSetDevice(dev);
    if (e != cudaSuccess)
        return qk::fail(QK_ERR_INIT, "%s; device probe failed at index %zu: %s",
                        qk_gpu_init_hint(), device_index, cudaGetErrorString(e));
    qk_ctx *ctx = new qk_ctx();
    ctx->device = dev;
    ctx->sm_count = prop.multiProcessorCount;
    e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e != cudaSuccess) {
        delete ctx;
        return qk::fail(QK_ERR_INIT, "%s; stream creation failed at index %zu: %s",
                        qk_gpu_init_hint(), device_index, cudaGetErrorString(e));
    }
    ctx->own_stream = ctx->stream;
    *out = ctx;
    return QK_OK;
}

qk_status qk_gpu_set_stream(qk_ctx *ctx, void *stream) {
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    std::lock_guard<std::mutex> lock(c->mu);
    QK_CUDA(cudaSetDevice(c->device));
    QK_CUDA(cudaStreamSynchronize(c->stream));
    c->stream = stream ? (cudaStream_t)stream : c->own_stream;
    return QK_OK;
}

qk_status qk_gpu_init(qk_ctx **out) { return qk_gpu_init_at(0, out); }

int32_t qk_gpu_available(void) {
    qk_ctx *c = nullptr;
    if (qk_gpu_init_at(0, &c) != QK_OK) return 0;
    qk_gpu_free(c);
    return 1;
}

void qk_gpu_free(qk_ctx *ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    if (ctx->own_stream) cudaStreamDestroy(ctx->own_stream);
    if (ctx->up_stream) cudaStreamDestroy(ctx->up_stream);
    if (ctx->down_stream) cudaStreamDestroy(ctx->down_stream);
    for (cudaEvent_t e : ctx->pipe_events) cudaEventDestroy(e);
    ctx->d_packed.release();
    ctx->d_in.release();
    ctx->d_out.release();
    ctx->d_z.release();
    ctx->d_t.release();
    ctx->d_ptrs.release();
    ctx->d_err.release();
    ctx->d_head.release();
    for (auto &ps : ctx->h_pinned) {
        if (ps.copied) cudaEventDestroy(ps.copied);
        if (ps.ptr) cudaFreeHost(ps.ptr);
    }
    delete ctx;
}

qk_status qk_gpu_synchronize(qk_ctx *ctx) {
    qk_ctx *c;
    qk_status st = qk::resolve_ctx(ctx, &c);
    if (st != QK_OK) return st;
    QK_CUDA(cudaSetDevice(c->device));
    QK_CUDA(cudaStreamSynchronize(c->stream));
    std::lock_guard<std::mutex> lock(c->mu);
    if (c->err_armed) {
        // Kernels that can raise the error word have been launched on this context (or captured
        // into a graph that may be replayed at any time, which is why the check stays armed).
        int h_err = 0;
        QK_CUDA(cudaMemcpyAsync(&h_err, c->d_err.ptr, sizeof(int), cudaMemcpyDeviceToHost, c->stream));
        QK_CUDA(cudaStreamSynchronize(c->stream));
        if (h_err) {
            QK_CUDA(cudaMemsetAsync(c->d_err.ptr, 0, sizeof(int), c->stream));
            if (h_err & 4)
                return qk::fail(QK_ERR_VALUE,
                                "a token's position or sequence index lies outside the KV cache; "
                                "the token was skipped");
            return qk::fail(QK_ERR_TIMEOUT, "a bounded device-side wait gave up:%s%s%s%s",
                            (h_err & 1) ? " a pipeline barrier of a tcgen05 kernel (prefill GEMM, Sage attention);" : "",
                            (h_err & 2) ? " the inbox of a fused all-reduce (a peer did not send);"
                                        : "",
                            (h_err & 8) ? " a ring or table barrier of the streaming GEMV;" : "",
                            (h_err & 16) ? " a grid barrier of the whole-step decode kernel;" : "");
        }
    }
    return QK_OK;
}

void *qk_gpu_stream(qk_ctx *ctx) {
    qk_ctx *c;
    if (qk::resolve_ctx(ctx, &c) != QK_OK) return nullptr;
    return (void *)c->stream;
}

int32_t qk_set_gemv_kernel(qk_ctx *ctx, int32_t which) {
    qk_ctx *c;
    if (qk::resolve_ctx(ctx, &c) != QK_OK) return -1;
    int prev = c->gemv_kernel;
    if (which >= 0 && which <= 6) c->gemv_kernel = which;
    return prev;
}

int32_t qk_set_dependent_launch(qk_ctx *ctx, int32_t on) {
    qk_ctx *c;
    if (qk::resolve_ctx(ctx, &c) != QK_OK) return -1;
    std::lock_guard<std::mutex> lock(c->mu);
    const int32_t prev = c->pdl ? 1 : 0;
    if (on == 0 || on == 1) c->pdl = on != 0;
    return prev;
}

uint32_t qk_set_wait_limit(qk_ctx *ctx, uint32_t polls) {
    qk_ctx *c;
    if (qk::resolve_ctx(ctx, &c) != QK_OK) return 0;
    std::lock_guard<std::mutex> lock(c->mu);
    const uint32_t prev = c->wait_limit;
    c->wait_limit = polls;
    return prev;
}

uint64_t qk_gpu_launch_count(qk_ctx *ctx) {
    qk_ctx *c;
    if (qk::resolve_ctx(ctx, &c) != QK_OK) return 0;
    return c->launches.load();
}

}  // extern "C"
