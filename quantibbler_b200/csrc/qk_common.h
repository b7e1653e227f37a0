// Internal declarations shared by the translation units of libqk_kernels.so.
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/qk_kernels.h"

namespace qk {

// Thread-local error text behind qk_last_error().
void set_error(const char *fmt, ...) __attribute__((format(printf, 1, 2)));
qk_status fail(qk_status code, const char *fmt, ...) __attribute__((format(printf, 2, 3)));

// Index ceiling of the device kernels' 32-bit address arithmetic
// (crates/quantibbler-kernels/src/gpu.rs:42-45, GPU_INDEX_CEILING).
constexpr uint64_t kIndexCeiling = 0xFFFFFFFFull;

inline size_t ceil_div(size_t a, size_t b) { return (a + b - 1) / b; }

// Shared validation of a packed operand (core.rs:223-240); sets the error text.
qk_status validate_packed(size_t packed_len, size_t n_rows, size_t n_bits, size_t *n_words);

#define QK_CUDA(call)                                                                   \
    do {                                                                                \
        cudaError_t e__ = (call);                                                       \
        if (e__ != cudaSuccess)                                                         \
            return qk::fail(QK_ERR_CUDA, "CUDA call %s failed: %s", #call,              \
                            cudaGetErrorString(e__));                                   \
    } while (0)

}  // namespace qk

// A device buffer that grows on demand and is reused between calls.
struct qk_scratch {
    void *ptr = nullptr;
    size_t cap = 0;
    qk_status reserve(size_t bytes);
    void release();
};

struct qk_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;      // the stream calls launch on
    cudaStream_t own_stream = nullptr;  // created with the context
    std::mutex mu;  // serialises calls from several host threads
    int sm_count = 0;
    int gemv_kernel = 1;  // 0 sign-select, 1 bit-sliced INT8 tensor core
    int sage_kernel = 2;  // 0 dp4a, 1 INT8 tensor core (mma.sync), 2 tcgen05 kind::i8 where the shape allows, else 1
    int decode_attention_kernel = 1;  // 0 scalar, 1 bf16 tensor core where the cache allows
    std::atomic<uint64_t> launches{0};
    // staging for the host-buffer entry points
    qk_scratch d_packed, d_in, d_out;
    // intermediates of the factorized linear (z and t) and of grouped applies
    qk_scratch d_z, d_t, d_ptrs;
    // error word of the asynchronous tensor-core kernels, read back by qk_gpu_synchronize
    qk_scratch d_err;
    qk_scratch d_head;  // the LM head's bfloat16 split of the hidden state
    bool err_armed = false;  // sticky: set by the first launch that can raise the error word
    uint32_t wait_limit = 0;  // polls before a device-side wait gives up (0: the default)
    bool pdl = true;          // decoder-path kernels may overlap their prologue with the kernel before
    // Pinned staging for launch parameters: a small ring of blocks, each guarded by an event
    // that is recorded after the copy out of it, so that a call only waits (on the host) when
    // it comes back to a block whose copy is still in flight - not on every call.
    static constexpr int kPinnedSlots = 4;
    struct PinnedSlot {
        void *ptr = nullptr;
        size_t cap = 0;
        cudaEvent_t copied = nullptr;
        bool in_flight = false;
    } h_pinned[kPinnedSlots];
    int h_pinned_next = 0;
    // the copy streams and events of the host-buffer pipeline (qk_groups_apply_host), made on first use
    cudaStream_t up_stream = nullptr, down_stream = nullptr;
    std::vector<cudaEvent_t> pipe_events;
    // A block of at least `bytes`, free to be overwritten; *slot names it for pinned_done().
    qk_status pinned(size_t bytes, void **out, int *slot);
    // Call after the asynchronous copy out of the block has been issued on `stream`.
    qk_status pinned_done(int slot);
};

struct qk_layer {
    int device = 0;
    size_t dout = 0, din = 0, r = 0;
    int serving = QK_F32;
    // per-row bitplanes, rows padded to a multiple of 16 bytes (zero pad bits)
    uint8_t *ub = nullptr;    // dout rows x ub_stride bytes
    uint8_t *vbt = nullptr;   // r rows x vbt_stride bytes
    // the same factors as 16-row x 512-bit tiles for the tensor-core GEMV
    uint8_t *ub_tiles = nullptr, *vbt_tiles = nullptr;
    size_t ub_stride = 0, vbt_stride = 0;
    float *s1 = nullptr, *s2 = nullptr, *bias = nullptr;  // bias may be null
};

// A fixed set of same-shape layers bound to input/output buffers: the launch parameters
// live on the device, so applying the group is two kernel launches and nothing else.
struct qk_group {
    int device = 0;
    size_t n_inst = 0;
    qk_layer shape;          // dimensions/strides of the member layers (the largest, if they differ)
    bool mixed = false;      // the members differ in shape: few-instance form only
    bool fed = false;        // the stage-1 tables are written by the kernels that produce the inputs
    bool normed = false;     // stage 1 applies an RMSNorm to its input itself (qk_plan_set_norm)
    bool pushed = false;     // the last stage pushes its outputs into all-reduce inboxes (qk_plan_set_allreduce)
    bool gathered = false;   // the norm's residual is what an all-reduce left in this rank's inbox
    uint32_t ar_poll_limit = 0;  // ... and the poll limit its parameter records hold
    void *feed = nullptr;    // device array of per-instance feed targets (fed plans)
    void *tickets = nullptr; // device array of per-instance block counters (fed plans)
    void *scratch = nullptr; // per member: intermediate t, digit tables, stage metadata
    void *params = nullptr;  // device array of 2*n_inst stage parameter records
};

namespace qk {
// Programmatic dependent launch.  A kernel launched through launch_pdl may start while the
// kernel before it on the stream is still running; it reads nothing that kernel wrote, and
// writes nothing at all, before it has executed pdl_wait() (griddepcontrol.wait returns when
// the preceding kernel has completed and its writes are visible).  What comes before the wait
// is work that depends on no other kernel: fetching weight bits, setting up shared memory.
// Every such kernel calls pdl_wait() in every thread (so that its own completion implies the
// completion of everything before it) and pdl_launch() as early as it can, which lets the
// kernel after it begin its own prologue.  Inside a captured CUDA graph the same launches
// become programmatic edges.
#ifdef __CUDACC__
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
cudaError_t launch_pdl(bool allow_overlap, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                       cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = allow_overlap ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

// Returns the context to use for a call: `ctx` itself, or the process-wide default on
// device 0 (created on first use) when `ctx` is null.
qk_status resolve_ctx(qk_ctx *ctx, qk_ctx **out);
// Makes sure the context's error word (an int, bits: 1 a prefill pipeline wait, 2 an all-reduce
// inbox wait, 4 a token outside the KV cache, 8 a wait of the streaming GEMV, 16 a grid barrier of the
// whole-step decode kernel) and the prefill's CTA flags after it exist.
qk_status error_word(qk_ctx *c);
}  // namespace qk
