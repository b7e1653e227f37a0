/*
 * qk_kernels.h - C ABI of libqk_kernels.so, the sm_100a implementation of the
 * quantibbler-kernels hot path.
 *
 * Every entry point is what a Rust `extern "C"` block (or ctypes / cffi) binds in
 * place of one item of the reference crate's API; the comment above each one names
 * the reference item it replaces as file:line inside the reference project.
 *
 * Conventions
 *  - Every function returns a qk_status; QK_OK is 0.  On failure the message is
 *    readable through qk_last_error() on the calling thread until that thread's
 *    next failing call.  No exception crosses the ABI.
 *  - QK_ERR_VALUE carries the reference's KernelError text verbatim
 *    (crates/quantibbler-kernels/src/core.rs:31-44); a Python binding raises
 *    ValueError with it (crates/quantibbler-kernels/src/lib.rs:34-36).
 *  - Inputs are borrowed for the duration of the call and never retained, except by
 *    qk_layer_create / qk_layer_create_from_streams / qk_layer_from_qpk1, which copy them to the device.  Outputs are
 *    caller-allocated.
 *  - "host" pointers are ordinary process memory; "dev" pointers are CUDA device
 *    memory on the context's device.  bfloat16 travels as uint16_t bit patterns
 *    (crates/quantibbler-kernels/src/lib.rs:245-261).
 *  - Products run on the GPU.  There is no CPU fallback: without a usable device the
 *    product entry points fail with QK_ERR_INIT and the text of QK_GPU_INIT_HINT.
 *  - A qk_ctx may be used from several host threads; calls on one context are
 *    serialised on its stream.
 */
#ifndef QK_KERNELS_H
#define QK_KERNELS_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int32_t qk_status;
enum {
    QK_OK = 0,
    QK_ERR_VALUE = 1,   /* validation failure: the reference's KernelError */
    QK_ERR_INIT = 2,    /* no usable CUDA device / context creation failed */
    QK_ERR_CUDA = 3,    /* a CUDA runtime call failed after start-up */
    QK_ERR_TIMEOUT = 4, /* a bounded device-side wait gave up */
    QK_ERR_ALLOC = 5
};

/* dtype tags: crates/quantibbler-kernels/src/dtype.rs:99-129 (Dtype, NAMES). */
enum { QK_F64 = 0, QK_F32 = 1, QK_BF16 = 2 };

typedef struct qk_ctx qk_ctx;
typedef struct qk_layer qk_layer;
typedef struct qk_group qk_group;

/* Thread-local text of the last failure on this thread ("" if none). */
const char *qk_last_error(void);

/* crates/quantibbler-kernels/src/lib.rs:86-89 (backend_version). */
const char *qk_backend_version(void);

/* crates/quantibbler-kernels/src/gpu.rs:36-40 (GPU_INIT_HINT): the actionable text
 * embedded in every initialisation failure, here naming the CUDA requirements. */
const char *qk_gpu_init_hint(void);

/* ---- integer bitplane core (host) ------------------------------------------ */

/* core.rs:129-162 (pack_bits).  factor is row-major n_rows x n_cols of +-1; out
 * holds n_rows * ceil(n_cols/8) bytes. */
qk_status qk_pack_bits(const int8_t *factor, size_t factor_len, size_t n_rows, size_t n_cols,
                       uint8_t *out, size_t out_len);
/* lib.rs:93-116 (the PyO3 pack_bits): float64 values, anything but exactly +-1.0 is
 * rejected before packing. */
qk_status qk_pack_bits_f64(const double *factor, size_t factor_len, size_t n_rows,
                           size_t n_cols, uint8_t *out, size_t out_len);
/* core.rs:166-189 (unpack_bits). */
qk_status qk_unpack_bits(const uint8_t *packed, size_t packed_len, size_t n_rows, size_t n_bits,
                         int8_t *out, size_t out_len);
/* core.rs:193-197 (sign_estimate). */
qk_status qk_sign_estimate(const double *x, size_t n, int8_t *out);
/* core.rs:327-424 (joint_itq) with its helpers :47-126; NumPy face
 * src/quantibbler/kernels/__init__.py:345-512.  Alternating Procrustes over
 * Z = [u_hat; v_hat] (row-major dout x rank and din x rank float64): R0 from splitmix64(seed)
 * + modified Gram-Schmidt, then B <- sign(Z R), R <- Psi Phi^T from the SVD of B^T Z, until
 * ||R_new - R_old||_F <= tol (only when tol > 0) or max_iter.  Writes the +-1 factors
 * sign(Z R) to u_t (dout x rank) and v_t (din x rank), the iteration count and the
 * convergence flag.  Host code, as in the reference; errors: "joint_itq expects non-empty
 * factors", "joint_itq shape mismatch: ...", "joint_itq produced a degenerate zero column
 * building R0". */
qk_status qk_joint_itq(const double *u_hat, size_t u_len, const double *v_hat, size_t v_len,
                       size_t dout, size_t din, size_t rank, size_t max_iter, double tol,
                       uint64_t seed, int8_t *u_t, int8_t *v_t, size_t *n_iter,
                       int32_t *converged);
/* core.rs:223-240 (validate_packed). */
qk_status qk_validate_packed(size_t packed_len, size_t n_rows, size_t n_bits, size_t *n_words);
/* dtype.rs:106-119 (Dtype::from_name) and :121-128 (Dtype::name). */
qk_status qk_dtype_from_name(const char *name, int32_t *dtype);
const char *qk_dtype_name(int32_t dtype);
/* crates/quantibbler-server/src/engine/mod.rs:258-273 (container_to_rows) and
 * :277-289 (container_to_rows_transposed): container bit stream -> per-row planes. */
qk_status qk_container_to_rows(const uint8_t *packed, size_t packed_len, size_t n_rows, size_t r,
                               uint8_t *out, size_t out_len);
qk_status qk_container_to_rows_transposed(const uint8_t *packed, size_t packed_len, size_t din,
                                          size_t r, uint8_t *out, size_t out_len);

/* ---- device context --------------------------------------------------------- */

/* gpu.rs:187-189 (gpu_available): 1 if a context can be created on device 0. */
int32_t qk_gpu_available(void);
/* gpu.rs:85-101 (GpuContext::init_at, ::init).  *out receives an owned context. */
qk_status qk_gpu_init_at(size_t device_index, qk_ctx **out);
qk_status qk_gpu_init(qk_ctx **out);
void qk_gpu_free(qk_ctx *ctx);
/* Blocks until every call issued on the context has finished on the device. */
qk_status qk_gpu_synchronize(qk_ctx *ctx);
/* The CUDA stream (cudaStream_t) the context launches on, for event timing. */
void *qk_gpu_stream(qk_ctx *ctx);
/* Make the context launch on a caller-owned stream (cudaStream_t; NULL restores the
 * context's own stream).  Lets a host framework order these kernels with its own work
 * without a device-wide synchronisation. */
qk_status qk_gpu_set_stream(qk_ctx *ctx, void *stream);

/* ---- packed products, host buffers in and out -------------------------------- */

/* gpu.rs:116-183 (GpuContext::packed_matvec): float64, strictly sequential
 * accumulation per row, bit-identical to the CPU faces.  Validation happens before
 * any device work; zero-size work returns zeros without a launch. */
qk_status qk_gpu_packed_matvec(qk_ctx *ctx, const uint8_t *packed, size_t packed_len,
                               size_t n_rows, size_t n_bits, const double *vec, size_t vec_len,
                               double *out);
/* core.rs:247-260 (packed_matvec::<T>) / dispatch.rs:81-93 (packed_matvec_dyn) /
 * lib.rs:292-321 (packed_matvec_dtype).  vec and out have the tagged dtype; the
 * accumulation is sequential in the dtype's accumulator (f64, f32, f32) and the
 * result is bit-identical to the reference's.  ctx may be NULL: a process-wide
 * context on device 0 is created on first use. */
qk_status qk_packed_matvec(qk_ctx *ctx, const uint8_t *packed, size_t packed_len, size_t n_rows,
                           size_t n_bits, int32_t dtype, const void *vec, size_t vec_len,
                           void *out);
/* core.rs:288-317 (packed_matmul::<T>) / dispatch.rs:96-109 / lib.rs:326-381.
 * mat is addressed mat[t*n_cols + j]; the output is n_rows x (mat_len / n_bits). */
qk_status qk_packed_matmul(qk_ctx *ctx, const uint8_t *packed, size_t packed_len, size_t n_rows,
                           size_t n_bits, int32_t dtype, const void *mat, size_t mat_len,
                           size_t n_cols, void *out, size_t out_len);

/* ---- attention, host buffers in and out --------------------------------------- */

/* gpu_attention.rs:402-411 (AttentionShape). */
typedef struct qk_attention_shape {
    size_t batch, n_heads, n_kv_heads, seq_q, seq_kv, head_dim, val_dim;
} qk_attention_shape;

/* gpu_attention.rs:451-570 (GpuContext::attention): exact softmax(QK^T/sqrt(d))V in
 * float32.  query [B,H,Sq,d], key [B,KV,Skv,d], value [B,KV,Skv,dv], out [B,H,Sq,dv],
 * packed row-major; head h reads kv head h/(H/KV); causal masks key j for query i when
 * j + Sq > i + Skv.  GQA is native: no head expansion on the host. */
qk_status qk_gpu_attention(qk_ctx *ctx, const qk_attention_shape *shape, const float *query,
                           size_t q_len, const float *key, size_t k_len, const float *value,
                           size_t v_len, int32_t causal, float *out, size_t out_len);
/* gpu_attention.rs:589-756 (GpuContext::attention_sage) with the arithmetic of
 * sage_int8_tile_kernel (:67-397): per-token INT8 Q/sqrt(d), per-key-block mean-smoothed
 * per-token INT8 K, static-scale INT8 P, per-channel-per-block INT8 V, int32 dots.
 * Requires seq_q == seq_kv; block_size is the key-block width. */
qk_status qk_gpu_attention_sage(qk_ctx *ctx, const qk_attention_shape *shape, const float *query,
                                size_t q_len, const float *key, size_t k_len, const float *value,
                                size_t v_len, int32_t causal, size_t block_size, float *out,
                                size_t out_len);
/* The quantisers of the Sage face on their own: src/quantibbler/kernels/attention_sage.py
 * :164-198 (quantize_per_token, quantize_per_channel, smooth_k_block) as the device path
 * applies them (gpu_attention.rs:132-155, :197-260).  Runs exactly the kernels
 * qk_gpu_attention_sage runs before its integer products and returns their INT8 codes and
 * scales in plain layouts, so that a caller can compare them bit for bit with the reference's:
 * q_codes [B,H,S,d] and q_scale [B,H,S] (of Q/sqrt(d), per token); k_codes [B,KV,S,d],
 * k_scale [B,KV,S] (of K minus its key block's mean, per token), k_mean [B,KV,blocks,d];
 * v_codes [B,KV,S,dv], v_scale [B,KV,blocks,dv] (per channel over the key block's tokens). */
qk_status qk_gpu_sage_quantize(qk_ctx *ctx, const qk_attention_shape *shape, const float *query,
                               size_t q_len, const float *key, size_t k_len, const float *value,
                               size_t v_len, size_t block_size, int8_t *q_codes, float *q_scale,
                               int8_t *k_codes, float *k_scale, float *k_mean, int8_t *v_codes,
                               float *v_scale);
/* The two attention faces on device buffers (same layouts, float32), asynchronous on the
 * context's stream: for callers whose q, k, v already live on the GPU (a resident prefill).
 * Additive; the reference's API has only the host-slice forms above. */
qk_status qk_gpu_attention_dev(qk_ctx *ctx, const qk_attention_shape *shape, const float *q_dev,
                               const float *k_dev, const float *v_dev, int32_t causal,
                               float *out_dev);
qk_status qk_gpu_attention_sage_dev(qk_ctx *ctx, const qk_attention_shape *shape,
                                    const float *q_dev, const float *k_dev, const float *v_dev,
                                    int32_t causal, size_t block_size, float *out_dev);
/* NOT the reference's arithmetic: the benchmark specification's wording of Sage on device
 * buffers (self-attention, head_dim == val_dim == 128).  Q / sqrt(d) and K (after its 64-key
 * block's channel mean has been removed; the mean's share of the scores is added back) are
 * quantised to INT8 with ONE symmetric scale per 64-token block, the scores' product runs on
 * tcgen05 kind::i8, the softmax in float32, and P and V go into the second product as
 * bfloat16 (tcgen05 kind::f16, float32 accumulation in tensor memory).  The reference quantises
 * per token, P and V to INT8 (gpu_attention.rs:67-397); this entry exists so that the
 * specification's variant can be measured beside it.  Asynchronous on the context's stream;
 * an expired in-kernel wait is reported by the next qk_gpu_synchronize as QK_ERR_TIMEOUT. */
qk_status qk_gpu_attention_sage_block_dev(qk_ctx *ctx, const qk_attention_shape *shape, const float *q_dev,
                                          const float *k_dev, const float *v_dev, int32_t causal, float *out_dev);
/* Which kernel the Sage face runs: 2 (default) the tcgen05 kernel (kind::i8 products with
 * the accumulators in tensor memory) where the shape allows (head_dim == val_dim == 128,
 * block_size 64), else as 1; 1 the mma.sync INT8 tensor-core kernel where the shape allows
 * (head_dim == val_dim in {64, 128}, block_size in {32, 64, 128}), else as 0; 0 always the
 * dp4a kernel.  All three do the same arithmetic.  A bounded wait of the tcgen05 kernel that
 * expires is reported by the next qk_gpu_synchronize as QK_ERR_TIMEOUT.  Returns the
 * previous choice. */
int32_t qk_set_sage_kernel(qk_ctx *ctx, int32_t which);
/* Which kernel qk_decode_attention runs for a bfloat16 cache with head_dim 128: 1 (default)
 * the bf16 tensor-core kernel, 0 the scalar kernel.  Returns the previous choice. */
int32_t qk_set_decode_attention_kernel(qk_ctx *ctx, int32_t which);

/* ---- the factorized linear with device-resident factors ----------------------
 * Replaces crates/quantibbler-server/src/engine/mod.rs:313-381 (PackedLayer,
 * PackedLayer::from_layer) and :393-480 (apply, apply_bf16, kernel_matvec).  The
 * reference re-reads its factors from host memory on every call; here they are
 * uploaded once and re-tiled for the GEMV kernels. */

/* ub_rows: dout x ceil(r/8) bytes; vb_t_rows: r x ceil(din/8) bytes (per-row
 * bitplanes, as PackedLayer holds them); s1[dout], s2[din] float32; bias[dout]
 * float32 or NULL (the all-zero bias of a version-1 stream).  serving_dtype is QK_F32
 * (ServingDtype::Fp32) or QK_BF16 (ServingDtype::Bf16). */
qk_status qk_layer_create(qk_ctx *ctx, const uint8_t *ub_rows, size_t ub_len,
                          const uint8_t *vb_t_rows, size_t vb_t_len, size_t dout, size_t din,
                          size_t r, const float *s1, const float *s2, const float *bias,
                          int32_t serving_dtype, qk_layer **out);
/* engine/mod.rs:342-381 (PackedLayer::from_layer) with the repack of :258-289 done on the
 * device: ub_stream and vb_stream are the container's bit streams of Ub (dout x r) and Vb
 * (din x r), ceil(rows * r / 8) bytes each, uploaded as they are; kernels separate the rows
 * of Ub and of Vb^T, pad and tile them.  Same layer, bit for bit, as qk_layer_create on the
 * output of qk_container_to_rows / qk_container_to_rows_transposed; a wrong stream length is
 * refused with the same text. */
qk_status qk_layer_create_from_streams(qk_ctx *ctx, const uint8_t *ub_stream, size_t ub_len,
                                       const uint8_t *vb_stream, size_t vb_len, size_t dout,
                                       size_t din, size_t r, const float *s1, const float *s2,
                                       const float *bias, int32_t serving_dtype, qk_layer **out);
/* The device's repack alone, result back in host memory in the layout of
 * qk_container_to_rows (transposed == 0: n_rows rows of ceil(r/8) bytes) or of
 * qk_container_to_rows_transposed (transposed != 0: r rows of ceil(n_rows/8) bytes). */
qk_status qk_gpu_container_to_rows(qk_ctx *ctx, const uint8_t *stream, size_t stream_len,
                                   size_t n_rows, size_t r, int32_t transposed, uint8_t *out,
                                   size_t out_len);
void qk_layer_free(qk_layer *layer);
/* ---- qpk1 layer stream ----------------------------------------------------------
 * crates/quantibbler-qpk1/src/lib.rs:229-320 (parse) / src/quantibbler/qpk1.py:211-258
 * (deserialize): header "QPK1", version (1: no bias, 2: bias), dtype tag (1 float16, 2
 * float32), dout, din, r as u32 little-endian; s1, s2, bias; the Ub and Vb container bit
 * streams.  The reader is fail-closed and keeps the reference's messages. */
typedef struct qk_qpk1_info {
    uint32_t version, dtype_tag;
    size_t dout, din, r;
    size_t s1_offset, s2_offset, bias_offset; /* bias_offset 0: a version-1 stream */
    size_t ub_offset, ub_len, vb_offset, vb_len;
} qk_qpk1_info;
qk_status qk_qpk1_parse(const uint8_t *bytes, size_t len, qk_qpk1_info *info);
/* s1[dout], s2[din], bias[dout] (may be NULL; zeros for a version-1 stream) as float32. */
qk_status qk_qpk1_scales(const uint8_t *bytes, size_t len, float *s1, float *s2, float *bias);
/* engine/mod.rs:342-381 (PackedLayer::from_layer) straight from the stream: parse, the
 * loader's rank gate r <= min(dout, din), upload, repack on the device. */
qk_status qk_layer_from_qpk1(qk_ctx *ctx, const uint8_t *bytes, size_t len, int32_t serving_dtype,
                             qk_layer **out);
/* y[n_tokens x dout] = layer(x[n_tokens x din]), float32 row-major device buffers.
 * Asynchronous on the context's stream. */
qk_status qk_layer_apply(qk_ctx *ctx, const qk_layer *layer, const float *x_dev, size_t n_tokens,
                         float *y_dev);
/* Prefill: n_tokens at once through one bfloat16-serving layer on the tcgen05 tensor
 * cores (core.rs:288-317 packed_matmul under the contract of engine/mod.rs:449-460: z, t
 * and u each rounded once to bfloat16, float32 accumulation).  x_dev [n_tokens, din] and
 * y_dev [n_tokens, dout] are float32 device buffers.  Asynchronous on the context's stream,
 * like qk_layer_apply.  Every wait inside the kernels is bounded; if one expires the result
 * is incomplete and the next qk_gpu_synchronize returns QK_ERR_TIMEOUT. */
qk_status qk_layer_apply_prefill(qk_ctx *ctx, const qk_layer *layer, const float *x_dev,
                                 size_t n_tokens, float *y_dev);
/* The same for up to four layers that read the same x_dev (the q, k, v or the gate, up
 * projections of a block): one scaling launch and one launch per stage serve them all,
 * y_devs[i] [n_tokens, layers[i]->dout].  The layers must have the same din. */
qk_status qk_layers_apply_prefill(qk_ctx *ctx, const qk_layer *const *layers, size_t n_layers,
                                  const float *x_dev, size_t n_tokens, float *const *y_devs);
/* The same with the input formed on the way in: x = silu(gate) * up (engine/mod.rs:931-935,
 * the SwiGLU in front of the down projection), gate_dev and up_dev float32 [n_tokens x din].
 * Same values as qk_swiglu followed by qk_layers_apply_prefill, without the activation being
 * written and read back. */
qk_status qk_layers_apply_prefill_gated(qk_ctx *ctx, const qk_layer *const *layers, size_t n_layers,
                                        const float *gate_dev, const float *up_dev, size_t n_tokens,
                                        float *const *y_devs);
/* How the prefill calls above deal their work out (host arithmetic only; no device is touched):
 * problem p has tiles[p] output tiles of k_chunks[p] 64-wide k-chunks each, the units of
 * work are (tile, k-chunk) pairs in problem-major, tile-major order, and CTA i of *n_ctas
 * takes units [cta_begin[i], cta_begin[i + 1]).  With many tiles the units are dealt out
 * evenly; with at most half as many tiles as CTAs every tile goes to a whole number of CTAs
 * in equal parts.  cta_begin needs *n_ctas + 1 <= min(sm_count, 192) + 1 entries. */
qk_status qk_prefill_work_split(size_t n_problems, const size_t *tiles, const size_t *k_chunks,
                                size_t sm_count, uint32_t *cta_begin, size_t cta_begin_len, size_t *n_ctas);
/* One token through one layer without any allocation by the library.  It has no
 * counterpart in the reference.  For callers that cannot let a library allocate device
 * memory on their behalf: a server that gave all remaining device memory to its KV cache
 * at start-up, or a request thread that must not run into cudaMalloc's device-wide
 * synchronisation.  The intermediates live in a fixed array inside the library image
 * (64.5 KB, held by every GPU that loads the library until the process exits), so the
 * layer must have r <= 8192 and din <= 16384; larger layers are refused with
 * QK_ERR_VALUE.  ctx must be an existing context (NULL is refused).  x_dev holds din and
 * y_dev dout float32 values on the context's device; the call is asynchronous on the
 * context's stream and gives the same values as qk_layer_apply with the default kernel
 * selector (it always runs the bit-sliced kernel).  The first call on each
 * device looks up the array's device address (cudaGetSymbolAddress): make that first call
 * before any stream capture begins.  All calls share the one array and it keeps the last
 * call's contents (every call overwrites what it later reads, so nothing needs clearing);
 * two calls that overlap on the GPU, from different streams or contexts, race on it. */
qk_status qk_layer_apply_noalloc(qk_ctx *ctx, const qk_layer *layer, const float *x_dev,
                                 float *y_dev);
/* The same with host buffers: x is copied in, y is copied out, and the call returns
 * when y is complete.  This is the drop-in for PackedLayer::apply. */
qk_status qk_layer_apply_host(qk_ctx *ctx, const qk_layer *layer, const float *x, size_t x_len,
                              float *y, size_t y_len);
/* n_layers independent layers of identical shape, layer i reading x_dev + i*din and
 * writing y_dev + i*dout, in one pair of launches (how q/k/v or gate/up share a
 * launch, and how the bandwidth benchmark streams more bytes than the L2 holds). */
qk_status qk_layers_apply_group(qk_ctx *ctx, const qk_layer *const *layers, size_t n_layers,
                                const float *x_dev, float *y_dev);
/* The same set of layers bound once to its buffers: qk_group_apply is then exactly two
 * kernel launches with no host-side staging, so steps can be queued back to back. */
qk_status qk_group_create(qk_ctx *ctx, const qk_layer *const *layers, size_t n_layers,
                          const float *x_dev, float *y_dev, qk_group **out);
/* The general form: instance k applies layers[k] to x_ptrs[k] (din floats) and writes
 * y_ptrs[k] (dout floats).  This is how a batch of tokens shares q/k/v (same input pointers)
 * or gate/up launches.  The layers share one serving dtype; they may differ in shape (q beside
 * k and v) as long as the plan is small enough for the few-instance kernel form, otherwise
 * QK_ERR_VALUE. */
qk_status qk_plan_create(qk_ctx *ctx, const qk_layer *const *layers, const float *const *x_ptrs,
                         float *const *y_ptrs, size_t n_inst, qk_group **out);
/* The same with the SwiGLU of engine/mod.rs:931-935 as the input transform: instance k reads
 * gate_ptrs[k] and up_ptrs[k] (din floats each) and applies layers[k] to
 * g * u / (1 + exp(-g)), which is how the down projection follows gate and up without a
 * separate activation pass. */
qk_status qk_plan_create_gated(qk_ctx *ctx, const qk_layer *const *layers,
                               const float *const *gate_ptrs, const float *const *up_ptrs,
                               float *const *y_ptrs, size_t n_inst, qk_group **out);
/* Makes a plan apply an RMSNorm to its input itself (engine/mod.rs:900-907 followed by the
 * linears of :908-915 in one launch): instance k then reads x_ptrs[k] as the residual stream,
 * adds residual_ptrs[k] (the array or an entry may be null), and applies its layer to
 * (x + residual) * rsqrt(mean((x + residual)^2) + eps) * norm_weight - the bits of
 * qk_rmsnorm followed by the plain plan.  Where x_out_ptrs[k] is not null the instance also
 * writes x + residual there (give it for ONE instance per token, and not the input buffer:
 * every block of the launch reads the input).  The plan must fit the few-instance kernel
 * form with at most 8192 inputs, otherwise QK_ERR_VALUE and the plan is unchanged. */
qk_status qk_plan_set_norm(qk_ctx *ctx, qk_group *plan, const float *const *residual_ptrs,
                           const float *norm_weight, float eps, float *const *x_out_ptrs);
/* Tensor parallel: the all-reduce of a row-parallel linear's output inside the plans on either
 * side of it (the reference has no parallelism; the partition is the benchmark's).  With
 * gather = 0 the plan's last stage pushes every output it finishes, tagged with the number of
 * the all-reduce, into the inbox of every rank (inbox_bases[0 .. world), peer memory, this
 * rank's own included) instead of storing it.  With gather = 1 the plan - a normed plan over the
 * stream of d <= 4096 entries - takes as the residual of its norm the sum, in rank order, of what
 * has arrived in this rank's inbox (inbox_bases[0]); its blocks poll for the words they need
 * with the context's wait limit (QK_ERR_TIMEOUT at the next qk_gpu_synchronize on expiry).  An
 * inbox holds world x total_words 8-byte words {value, number}; instance k belongs to token
 * token_of_instance[k] (words token * d ..).  state_dev: two zero-initialised uint32 shared by
 * all plans and qk_allreduce_rmsnorm calls of the process group member, in call order: the
 * number of all-reduces completed and a block ticket.  Same bits as qk_allreduce_rmsnorm
 * between the plain plans.  Successive all-reduces must alternate between two inboxes. */
qk_status qk_plan_set_allreduce(qk_ctx *ctx, qk_group *plan, int32_t gather, const uint64_t *inbox_bases,
                                int32_t rank, int32_t world, size_t total_words, const uint32_t *token_of_instance,
                                size_t d, uint32_t *state_dev);
qk_status qk_group_apply(qk_ctx *ctx, const qk_group *group);
/* Many independent applies with HOST buffers as a pipeline: groups[p] (made by qk_group_create
 * over rows first_row[p] .. first_row[p+1] of x_dev / y_dev) has its inputs copied up from
 * x_host, runs, and has its outputs copied down to y_host, on three streams, so that the upload
 * of one group, the kernels of the previous one and the download of the one before overlap (the
 * link is full duplex).  x_host [rows][din] and y_host [rows][dout] should be pinned memory;
 * returns when y_host is complete.  This is what a caller with all same-shape layers of a
 * step, or one layer for many requests, uses instead of one qk_layer_apply_host per layer
 * (PackedLayer::apply, engine/mod.rs:416-431). */
qk_status qk_groups_apply_host(qk_ctx *ctx, const qk_group *const *groups, const size_t *first_row,
                               size_t n_groups, const float *x_host, float *y_host, float *x_dev,
                               float *y_dev, size_t din, size_t dout);
void qk_group_free(qk_group *group);
/* ---- the blocks of a decode step as one kernel ---------------------------------------
 * transformer_forward (engine/mod.rs:878-945) runs, per block, norm -> q/k/v -> RoPE + cache
 * append -> attention -> o -> norm -> gate/up -> SwiGLU -> down.  As separate launches that is
 * about fourteen dependent kernels per block, each as long as its chain of memory round trips;
 * qk_decode_step_run does ALL blocks of a step in one cooperative kernel (one CTA per SM, a
 * bounded grid barrier between phases, the small operations folded into the phases that
 * consume them, every block prefetching its next weight tiles before it waits).  The linears
 * are the exact bit-sliced form, so a step equals, bit for bit, the same step made of
 * qk_rmsnorm / plans / qk_rope_cache / qk_decode_attention / qk_swiglu calls.  Measured on a
 * Llama-3-8B-shaped stack it is SLOWER than those launches (5.1 against 4.4 ms per one-token
 * step: with one CTA of eight warps per SM, the per-vector work that every block repeats -
 * norm, SwiGLU, digit table - is not hidden), so callers opt in.
 * Limits: head_dim 128, bfloat16 cache, at most 8 tokens, no per-head q/k norms, a model
 * narrow enough for the kernel's shared memory; anything else is refused with QK_ERR_VALUE and
 * the caller keeps the separate launches.
 * Buffers (all float32 unless said, token-major): x holds the embedded tokens on entry and
 * the residual stream before the last block's down output on exit (delta_mlp holds that
 * output: the caller's final norm adds it); x2 is the stream's second buffer; q/k/v/attn/
 * gate/up are [tokens][width] work buffers; att_scratch is qk_decode_attention_scratch bytes;
 * cos_sin is [s_max][64][2]; positions, seq_index, kv_len as for qk_rope_cache and
 * qk_decode_attention.  A token outside the cache is skipped and reported like there.
 * A grid barrier that does not complete within the context's wait limit sets the error word
 * (QK_ERR_TIMEOUT from the next qk_gpu_synchronize); the kernel still runs to its end. */
typedef struct qk_step_block {
    const qk_layer *q, *k, *v, *o, *gate, *up, *down;
    const float *input_norm, *post_norm; /* d_model weights each */
    void *cache_k, *cache_v;             /* bfloat16 [n_seq][n_kv_heads][s_max][128] */
} qk_step_block;
typedef struct qk_step_buffers {
    float *x, *x2, *q, *k, *v, *attn, *delta_attn, *delta_mlp, *gate, *up, *att_scratch;
    const float *cos_sin;
    const int32_t *positions, *seq_index, *kv_len;
} qk_step_buffers;
typedef struct qk_step_desc {
    size_t n_blocks, n_tokens, d_model, n_heads, n_kv_heads, head_dim, d_ff, s_max, n_seq, n_splits;
    float rms_eps;
    int32_t serving_dtype, kv_dtype;
    const qk_step_block *blocks;
    qk_step_buffers buf;
} qk_step_desc;
typedef struct qk_decode_step qk_decode_step;
qk_status qk_decode_step_create(qk_ctx *ctx, const qk_step_desc *desc, qk_decode_step **out);
qk_status qk_decode_step_run(qk_ctx *ctx, const qk_decode_step *step);
/* Diagnostic: later runs of the step write the device's nanosecond timer, as block 0 sees it,
 * at kernel start, after every grid barrier and at the end into stamps_dev (capacity entries;
 * 9 barriers per block of the model); NULL switches the trace off.  The differences are the
 * durations of the phases. */
qk_status qk_decode_step_trace(qk_decode_step *step, uint64_t *stamps_dev, size_t capacity);
void qk_decode_step_free(qk_decode_step *step);

/* ---- fed plans ------------------------------------------------------------------
 * At a small batch the cost of a GEMV launch is not its weight bits but what every one of
 * its blocks does first: scan the input vector, put it on a fixed-point grid, build the
 * digit table it multiplies with.  A fed plan moves that work to where the vector is
 * produced, once per vector: qk_plan_feed_targets turns a plan into a fed plan and returns a
 * device array with one target per instance (in instance order); the *_feed forms of the
 * norm, SwiGLU and decode-attention calls below take such arrays and write the tables of
 * the plan's stage-1 inputs along with their own output; stage 1 hands over to stage 2 the
 * same way (its last block to finish builds the table of the intermediate).  A fed plan's
 * stage kernels never read the x pointers the plan was created with.  Every apply of a fed
 * plan must be preceded, on the same stream, by a *_feed call that names its targets.  Plans
 * too large for the few-instance kernel form are refused with QK_ERR_VALUE.  No reference
 * counterpart (the reference recomputes nothing because it has no device). */
typedef struct qk_feed {
    const void *targets[4]; /* arrays returned by qk_plan_feed_targets */
    size_t per_token[4];    /* consecutive targets of array i that read token t: [t*per_token, ...) */
    size_t n_arrays;
} qk_feed;
qk_status qk_plan_feed_targets(qk_ctx *ctx, qk_group *plan, const void **targets_dev,
                               size_t *n_targets);

/* ---- decoder-side kernels on device buffers -----------------------------------
 * What one transformer block needs around its linears.  All are launch-only on the
 * context's stream (no allocation, no synchronisation), so a whole decode step can be
 * captured in a CUDA graph.  Activations are float32 row-major [tokens, width]. */

/* engine/mod.rs:1154-1160 (rms_norm_into) + :837-851 (norm_apply).  h = x + residual
 * (residual may be NULL); if x_out is not NULL it receives h; y = h*rsqrt(mean(h^2)+eps)*w.
 * bfloat16 serving rounds h and y to bfloat16 as the reference does. */
qk_status qk_rmsnorm(qk_ctx *ctx, const float *x, const float *residual, const float *weight,
                     size_t n_tokens, size_t d, float eps, int32_t serving_dtype, float *x_out,
                     float *y);
/* qk_rmsnorm that also writes the digit tables of the linears that read y (fed plans). */
qk_status qk_rmsnorm_feed(qk_ctx *ctx, const float *x, const float *residual, const float *weight,
                          size_t n_tokens, size_t d, float eps, int32_t serving_dtype, float *x_out,
                          float *y, const qk_feed *feed);
/* Tensor parallel: RMSNorm whose residual input is the SUM over ranks of the row-parallel
 * linears' partial outputs - the all-reduce after the o and down projections fused into the
 * norm that follows it.  Every rank pushes its partial into an inbox in each peer's memory
 * (NVLink peer stores; every 8-byte word carries the value and the number of the all-reduce,
 * so no flags and no fences are needed) and adds what arrives in its own inbox in rank order:
 * every rank gets the same bits.  No reference counterpart (the reference has no parallelism).
 * partial: this rank's [n_tokens, d] float32.  peer_inbox[r]: device address, valid on this
 * GPU, of rank r's inbox for this call, world x n_tokens x d 8-byte words, zero at start.
 * state_dev: two zero-initialised words of this rank (call count, block ticket).  Consecutive
 * calls must alternate between two inboxes.  x_out = x + sum, y = norm(x_out) * weight.
 * The polling is bounded (qk_set_wait_limit); on expiry y is not written and the next
 * qk_gpu_synchronize returns QK_ERR_TIMEOUT.  The call that timed out still counts on this
 * rank, but the ranks' counts may now differ: before the all-reduce is used again, every rank
 * must (after a host-side barrier) zero its inboxes and its two state words. */
qk_status qk_allreduce_rmsnorm(qk_ctx *ctx, const float *partial, const uint64_t *peer_inbox,
                               uint32_t *state_dev, int32_t rank, int32_t world, const float *x,
                               const float *weight, size_t n_tokens, size_t d, float eps,
                               int32_t serving_dtype, float *x_out, float *y);
qk_status qk_allreduce_rmsnorm_feed(qk_ctx *ctx, const float *partial, const uint64_t *peer_inbox,
                                    uint32_t *state_dev, int32_t rank, int32_t world, const float *x,
                                    const float *weight, size_t n_tokens, size_t d, float eps,
                                    int32_t serving_dtype, float *x_out, float *y, const qk_feed *feed);
/* engine/mod.rs:1169-1184 (rope_rotate) and :1204-1209 (KvCache::push).  Rotates q
 * [tokens, n_heads*d] in place and writes the rotated k and v [tokens, n_kv*d] into the
 * head-major cache [n_seq, n_kv, s_max, d] (float32 or bfloat16) at row positions[t] of
 * sequence seq_index[t].  cos_sin is [s_max, d/2, 2] float32.  The reference's cache is a
 * growable Vec; this one is a fixed allocation, so a token whose position is not in
 * [0, s_max) or whose sequence is not in [0, n_seq) is skipped on the device and the next
 * qk_gpu_synchronize fails with QK_ERR_VALUE.  The first call on a context creates the
 * context's error word: make it before any stream capture. */
qk_status qk_rope_cache(qk_ctx *ctx, float *q, const float *k, const float *v,
                        const float *cos_sin, const int32_t *positions, const int32_t *seq_index,
                        void *cache_k, void *cache_v, int32_t kv_dtype, size_t n_tokens,
                        size_t n_heads, size_t n_kv_heads, size_t head_dim, size_t s_max,
                        size_t n_seq);
/* engine/mod.rs:1074-1121 (gqa_attention_scalar): one query per sequence, q [batch,
 * n_heads, d], against kv_len[b] cached positions; out [batch, n_heads, d].  The keys are
 * split n_splits ways across blocks; scratch must hold qk_decode_attention_scratch bytes. */
size_t qk_decode_attention_scratch(size_t batch, size_t n_heads, size_t head_dim, size_t n_splits);
qk_status qk_decode_attention(qk_ctx *ctx, const float *q, const void *cache_k,
                              const void *cache_v, int32_t kv_dtype, const int32_t *kv_len,
                              size_t batch, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                              size_t s_max, size_t n_splits, float *scratch, float *out);
/* RoPE + KV-cache append + decode attention + combine in ONE launch, for a bfloat16 cache and
 * head_dim 128: what qk_rope_cache followed by qk_decode_attention does (the same bits in
 * `out` and in the cache), except that q is read unrotated and left so.  k, v: this step's
 * projections [batch][n_kv_heads][128] float32.  scratch: qk_decode_attention_rope_scratch
 * bytes, ZEROED once by the caller before the first call (it holds the split partials and one
 * counter per head group, which the kernel returns to zero).  Other configurations are refused
 * with QK_ERR_VALUE: use the two separate calls. */
size_t qk_decode_attention_rope_scratch(size_t batch, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                                        size_t n_splits);
qk_status qk_decode_attention_rope(qk_ctx *ctx, const float *q, const float *k, const float *v,
                                   const float *cos_sin, const int32_t *positions, const int32_t *seq_index,
                                   void *cache_k, void *cache_v, int32_t kv_dtype, const int32_t *kv_len,
                                   size_t batch, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                                   size_t s_max, size_t n_seq, size_t n_splits, float *scratch, float *out);
/* qk_decode_attention whose combine step also writes the digit tables of the linears that
 * read `out` (the o projection of a fed plan); serving_dtype is that of those linears. */
qk_status qk_decode_attention_feed(qk_ctx *ctx, const float *q, const void *cache_k,
                                   const void *cache_v, int32_t kv_dtype, const int32_t *kv_len,
                                   size_t batch, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                                   size_t s_max, size_t n_splits, float *scratch, float *out,
                                   int32_t serving_dtype, const qk_feed *feed);
/* The attention of a batched prompt prefill: engine/mod.rs:1393-1413 feeds the prompt one
 * position at a time through gqa_attention (:1074-1121); here n_tokens consecutive positions
 * first_position .. first_position+n_tokens-1 of sequence `seq` attend causally, each to the
 * cache rows 0 .. its own position (qk_rope_cache has already appended their keys and values).
 * q and out are float32, token-major [n_tokens, n_heads*head_dim]; the cache is
 * [n_seq, n_kv_heads, s_max, head_dim].  A bfloat16 cache with head_dim 128 runs on the bf16
 * tensor cores (q and the softmax weights split into three bfloat16 terms each, float32
 * accuracy); other shapes take a plain kernel. */
qk_status qk_prefill_attention(qk_ctx *ctx, const float *q, const void *cache_k, const void *cache_v,
                               int32_t kv_dtype, size_t seq, size_t first_position, size_t n_tokens,
                               size_t n_heads, size_t n_kv_heads, size_t head_dim, size_t s_max,
                               float *out);
/* engine/mod.rs:931-935: out = g*u/(1+exp(-g)). */
qk_status qk_swiglu(qk_ctx *ctx, const float *gate, const float *up, size_t n, float *out);
/* The same activation for n_tokens rows of n values, not written to memory but turned
 * straight into the digit tables of the linears that consume it (the down projection of a
 * fed plan). */
qk_status qk_swiglu_feed(qk_ctx *ctx, const float *gate, const float *up, size_t n_tokens, size_t n,
                         int32_t serving_dtype, const qk_feed *feed);
/* engine/mod.rs:921-924: out = a + b. */
qk_status qk_add(qk_ctx *ctx, const float *a, const float *b, size_t n, float *out);
/* engine/mod.rs:768-777 (embed): out[t] = table[ids[t]] (float32 or bfloat16 table). */
qk_status qk_embed(qk_ctx *ctx, const void *table, int32_t table_dtype, const int32_t *ids,
                   size_t n_tokens, size_t d, size_t vocab, float *out);
/* engine/mod.rs:788-800 (logits): logits[t*logits_stride + v] = hidden[t] . weight[v],
 * float32 accumulation; weight [vocab, d] float32 or bfloat16. */
qk_status qk_lm_head(qk_ctx *ctx, const float *hidden, const void *weight, int32_t weight_dtype,
                     size_t n_tokens, size_t vocab, size_t d, size_t logits_stride,
                     float *logits);
/* crates/quantibbler-server/src/sampler.rs:5-16 (greedy): the first maximum of each row;
 * out_idx is offset by index_base (for a vocabulary shard). */
qk_status qk_argmax_first(qk_ctx *ctx, const float *logits, size_t n_tokens, size_t vocab,
                          size_t logits_stride, int32_t index_base, float *out_val,
                          int32_t *out_idx);

/* Which GEMV kernel qk_layer_apply and the group calls use: 0 = sign-select SIMT, 1 = bit-sliced
 * INT8 tensor-core (default; many instances per launch run in the persistent streaming form),
 * 3 = the same without the split-k form, 5 = the same with one block per instance instead of
 * the streaming form, 2 and 4 = as 5 with 16-warp resp. 4-warp blocks (measurement variants).
 * Returns the previous value; values out of range leave it unchanged. */
int32_t qk_set_gemv_kernel(qk_ctx *ctx, int32_t which);
/* Programmatic dependent launch for the decoder-path kernels (norms, GEMV stages, RoPE,
 * decode attention, SwiGLU, head, argmax): 1 (default) lets each kernel begin its prologue -
 * fetching weight bits, which depend on no other kernel - while the kernel before it on the
 * stream finishes; 0 launches them strictly one after the other.  Results are identical.
 * Returns the previous setting.  No reference counterpart. */
int32_t qk_set_dependent_launch(qk_ctx *ctx, int32_t on);
/* How many polls a device-side wait of this context's kernels (the prefill GEMM's pipeline
 * barriers and split-tile flags, the fused all-reduce's inbox) makes before it gives up and
 * the next qk_gpu_synchronize returns QK_ERR_TIMEOUT.  0 restores the default (2^22, seconds).
 * Returns the previous value.  No reference counterpart. */
uint32_t qk_set_wait_limit(qk_ctx *ctx, uint32_t polls);
/* Number of kernels launched on this context since creation (for benchmarks). */
uint64_t qk_gpu_launch_count(qk_ctx *ctx);

#ifdef __cplusplus
}
#endif
#endif /* QK_KERNELS_H */
