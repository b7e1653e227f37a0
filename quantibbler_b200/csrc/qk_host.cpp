// Host side of libqk_kernels.so: error plumbing and the integer bitplane core.
//
// These functions are exact integer work that the reference also does on the host
// at load/compress time (crates/quantibbler-kernels/src/core.rs:129-240,
// crates/quantibbler-server/src/engine/mod.rs:258-289).  The floating-point products
// are not here: they run on the device (qk_products.cu, qk_gemv.cu).
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "qk_common.h"

namespace qk {

static thread_local std::string g_last_error;

void set_error(const char *fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
}

qk_status fail(qk_status code, const char *fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

qk_status validate_packed(size_t packed_len, size_t n_rows, size_t n_bits, size_t *n_words) {
    // core.rs:223-240
    if (n_bits == 0 && packed_len != 0 && n_rows != 0)
        return fail(QK_ERR_VALUE, "n_bits=0 with non-empty packed rows");
    size_t w = ceil_div(n_bits, 8);
    if (n_rows * w != packed_len)
        return fail(QK_ERR_VALUE, "packed length %zu does not match %zu rows x %zu bitplanes",
                    packed_len, n_rows, w);
    if (n_words) *n_words = w;
    return QK_OK;
}

// Shortest decimal text that round-trips, in the style of Rust's `{:?}` for f64
// ("1.0001", "2.0", "NaN", "inf").
static std::string debug_f64(double v) {
    if (std::isnan(v)) return "NaN";
    if (std::isinf(v)) return v > 0 ? "inf" : "-inf";
    char buf[64];
    for (int prec = 1; prec <= 17; ++prec) {
        snprintf(buf, sizeof buf, "%.*g", prec, v);
        if (strtod(buf, nullptr) == v) break;
    }
    std::string s(buf);
    if (s.find_first_of(".eEn") == std::string::npos) s += ".0";
    return s;
}

}  // namespace qk

using namespace qk;

extern "C" {

const char *qk_last_error(void) { return g_last_error.c_str(); }

const char *qk_backend_version(void) { return "0.1.0+b200"; }

const char *qk_gpu_init_hint(void) {
    return "no usable CUDA device; this library needs an NVIDIA B200-class GPU (compute "
           "capability 10.0, built for sm_100a), a driver new enough for CUDA 12.9 (libcuda.so "
           "on the loader path, /dev/nvidia* visible in the container) and, if "
           "CUDA_VISIBLE_DEVICES is set, the requested index inside it; there is no CPU "
           "fallback";
}

qk_status qk_pack_bits(const int8_t *factor, size_t factor_len, size_t n_rows, size_t n_cols,
                       uint8_t *out, size_t out_len) {
    if (n_rows * n_cols != factor_len)
        return fail(QK_ERR_VALUE, "factor length %zu does not match %zux%zu", factor_len, n_rows,
                    n_cols);
    size_t n_words = ceil_div(n_cols, 8);
    if (out_len != n_rows * n_words)
        return fail(QK_ERR_VALUE, "output length %zu does not match %zu rows x %zu bitplanes",
                    out_len, n_rows, n_words);
    for (size_t i = 0; i < n_rows; ++i) {
        const int8_t *row = factor + i * n_cols;
        for (size_t j = 0; j < n_words; ++j) {
            unsigned byte = 0;
            size_t lim = n_cols - j * 8 < 8 ? n_cols - j * 8 : 8;
            for (size_t k = 0; k < lim; ++k) {
                int v = row[j * 8 + k];
                if (v == 1)
                    byte |= 1u << k;
                else if (v != -1)
                    return fail(QK_ERR_VALUE,
                                "pack_bits expects values in {-1, +1}; got %d at row %zu, "
                                "column %zu",
                                v, i, j * 8 + k);
            }
            out[i * n_words + j] = (uint8_t)byte;
        }
    }
    return QK_OK;
}

qk_status qk_pack_bits_f64(const double *factor, size_t factor_len, size_t n_rows, size_t n_cols,
                           uint8_t *out, size_t out_len) {
    std::vector<int8_t> as_i8(factor_len);
    for (size_t i = 0; i < factor_len; ++i) {
        double v = factor[i];
        if (v == 1.0)
            as_i8[i] = 1;
        else if (v == -1.0)
            as_i8[i] = -1;
        else
            return fail(QK_ERR_VALUE, "pack_bits expects values in {-1, +1}; got %s",
                        debug_f64(v).c_str());
    }
    return qk_pack_bits(as_i8.data(), factor_len, n_rows, n_cols, out, out_len);
}

qk_status qk_unpack_bits(const uint8_t *packed, size_t packed_len, size_t n_rows, size_t n_bits,
                         int8_t *out, size_t out_len) {
    size_t n_words = ceil_div(n_bits, 8);
    if (n_rows * n_words != packed_len)
        return fail(QK_ERR_VALUE, "packed length %zu does not match %zu rows x %zu bitplanes",
                    packed_len, n_rows, n_words);
    if (out_len != n_rows * n_bits)
        return fail(QK_ERR_VALUE, "output length %zu does not match %zux%zu", out_len, n_rows,
                    n_bits);
    for (size_t i = 0; i < n_rows; ++i) {
        const uint8_t *row = packed + i * n_words;
        int8_t *o = out + i * n_bits;
        for (size_t k = 0; k < n_bits; ++k) o[k] = ((row[k >> 3] >> (k & 7)) & 1) ? 1 : -1;
    }
    return QK_OK;
}

qk_status qk_sign_estimate(const double *x, size_t n, int8_t *out) {
    for (size_t i = 0; i < n; ++i) out[i] = x[i] >= 0.0 ? 1 : -1;
    return QK_OK;
}

qk_status qk_validate_packed(size_t packed_len, size_t n_rows, size_t n_bits, size_t *n_words) {
    return validate_packed(packed_len, n_rows, n_bits, n_words);
}

qk_status qk_dtype_from_name(const char *name, int32_t *dtype) {
    static const char *names[3] = {"float64", "float32", "bfloat16"};
    for (int i = 0; i < 3; ++i)
        if (name && strcmp(name, names[i]) == 0) {
            *dtype = i;
            return QK_OK;
        }
    // dtype.rs:115-117; `{:?}` of a str is the quoted, escaped text
    std::string quoted = "\"";
    for (const char *p = name ? name : ""; *p; ++p) {
        if (*p == '"' || *p == '\\') quoted += '\\';
        quoted += *p;
    }
    quoted += "\"";
    return fail(QK_ERR_VALUE,
                "unknown kernel dtype %s; expected one of \"float64\", \"float32\", \"bfloat16\"",
                quoted.c_str());
}

const char *qk_dtype_name(int32_t dtype) {
    switch (dtype) {
        case QK_F64: return "float64";
        case QK_F32: return "float32";
        case QK_BF16: return "bfloat16";
        default: return "";
    }
}

qk_status qk_container_to_rows(const uint8_t *packed, size_t packed_len, size_t n_rows, size_t r,
                               uint8_t *out, size_t out_len) {
    size_t rw = ceil_div(r, 8);
    if (packed_len != ceil_div(n_rows * r, 8))
        return fail(QK_ERR_VALUE, "container stream holds %zu bytes; %zux%zu bits need %zu",
                    packed_len, n_rows, r, ceil_div(n_rows * r, 8));
    if (out_len != n_rows * rw)
        return fail(QK_ERR_VALUE, "output length %zu does not match %zu rows x %zu bitplanes",
                    out_len, n_rows, rw);
    if (r % 8 == 0) {
        memcpy(out, packed, out_len);
        return QK_OK;
    }
    memset(out, 0, out_len);
    for (size_t i = 0; i < n_rows; ++i)
        for (size_t j = 0; j < r; ++j) {
            size_t b = i * r + j;
            if ((packed[b >> 3] >> (b & 7)) & 1) out[i * rw + (j >> 3)] |= (uint8_t)(1u << (j & 7));
        }
    return QK_OK;
}

qk_status qk_container_to_rows_transposed(const uint8_t *packed, size_t packed_len, size_t din,
                                          size_t r, uint8_t *out, size_t out_len) {
    size_t rw = ceil_div(din, 8);
    if (packed_len != ceil_div(din * r, 8))
        return fail(QK_ERR_VALUE, "container stream holds %zu bytes; %zux%zu bits need %zu",
                    packed_len, din, r, ceil_div(din * r, 8));
    if (out_len != r * rw)
        return fail(QK_ERR_VALUE, "output length %zu does not match %zu rows x %zu bitplanes",
                    out_len, r, rw);
    memset(out, 0, out_len);
    for (size_t j = 0; j < din; ++j)
        for (size_t k = 0; k < r; ++k) {
            size_t b = j * r + k;
            if ((packed[b >> 3] >> (b & 7)) & 1) out[k * rw + (j >> 3)] |= (uint8_t)(1u << (j & 7));
        }
    return QK_OK;
}

}  // extern "C"

// ---- qpk1 layer stream (crates/quantibbler-qpk1/src/lib.rs:229-320, parse; the format is
// src/quantibbler/qpk1.py:59,150-258): 24-byte header "QPK1", version, dtype tag, dout, din,
// r (u32 little-endian), then s1[dout], s2[din], bias[dout] (version 2 only) in float16 or
// float32, then the Ub and Vb container bit streams.  Fail-closed, with the reader's texts.
namespace {

uint32_t u32le(const uint8_t *p) {
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}

float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else {  // subnormal: renormalise
            int e = -1;
            uint32_t m = man;
            do {
                ++e;
                m <<= 1;
            } while (!(m & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((m & 0x3ffu) << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

void decode_scales(const uint8_t *src, size_t n, uint32_t tag, float *dst) {
    for (size_t i = 0; i < n; ++i) {
        if (tag == 1) {
            dst[i] = half_to_float((uint16_t)(src[2 * i] | (src[2 * i + 1] << 8)));
        } else {
            const uint32_t bits = u32le(src + 4 * i);
            memcpy(dst + i, &bits, 4);
        }
    }
}

}  // namespace

extern "C" {

qk_status qk_qpk1_parse(const uint8_t *bytes, size_t len, qk_qpk1_info *info) {
    using qk::fail;
    if (!info) return fail(QK_ERR_VALUE, "qk_qpk1_parse: info is null");
    if (len < 24)
        return fail(QK_ERR_VALUE, "stream is %zu bytes; shorter than the 24-byte header", len);
    if (memcmp(bytes, "QPK1", 4) != 0)
        return fail(QK_ERR_VALUE, "bad magic [%u, %u, %u, %u]; expected [81, 80, 75, 49]", bytes[0],
                    bytes[1], bytes[2], bytes[3]);
    const uint32_t version = u32le(bytes + 4), tag = u32le(bytes + 8);
    if (version != 1 && version != 2)
        return fail(QK_ERR_VALUE,
                    "unsupported representation version %u; this reader implements version 1 "
                    "(pre-bias legacy) and version 2 (current, with bias)",
                    version);
    if (tag != 1 && tag != 2)
        return fail(QK_ERR_VALUE, "unknown dtype tag %u; expected 1 (float16) or 2 (float32)", tag);
    const size_t dout = u32le(bytes + 12), din = u32le(bytes + 16), r = u32le(bytes + 20);
    if (dout == 0 || din == 0 || r == 0)
        return fail(QK_ERR_VALUE, "dout, din and r must all be >= 1, got (%zu, %zu, %zu)", dout, din, r);
    const size_t item = tag == 1 ? 2 : 4;
    const bool has_bias = version >= 2;
    const size_t ub_len = qk::ceil_div(dout * r, 8), vb_len = qk::ceil_div(din * r, 8);
    const size_t expected = 24 + ((has_bias ? 2 : 1) * dout + din) * item + ub_len + vb_len;
    if (len < expected)
        return fail(QK_ERR_VALUE, "truncated stream: %zu bytes; header declares %zu", len, expected);
    if (len > expected)
        return fail(QK_ERR_VALUE, "trailing garbage: %zu bytes; one layer at this header is %zu", len,
                    expected);
    info->version = version;
    info->dtype_tag = tag;
    info->dout = dout;
    info->din = din;
    info->r = r;
    info->s1_offset = 24;
    info->s2_offset = info->s1_offset + dout * item;
    info->bias_offset = has_bias ? info->s2_offset + din * item : 0;
    info->ub_offset = info->s2_offset + din * item + (has_bias ? dout * item : 0);
    info->ub_len = ub_len;
    info->vb_offset = info->ub_offset + ub_len;
    info->vb_len = vb_len;
    return QK_OK;
}

qk_status qk_qpk1_scales(const uint8_t *bytes, size_t len, float *s1, float *s2, float *bias) {
    qk_qpk1_info info;
    qk_status st = qk_qpk1_parse(bytes, len, &info);
    if (st != QK_OK) return st;
    decode_scales(bytes + info.s1_offset, info.dout, info.dtype_tag, s1);
    decode_scales(bytes + info.s2_offset, info.din, info.dtype_tag, s2);
    if (bias) {
        if (info.bias_offset)
            decode_scales(bytes + info.bias_offset, info.dout, info.dtype_tag, bias);
        else
            memset(bias, 0, info.dout * sizeof(float));  // a version-1 stream: the zero bias
    }
    return QK_OK;
}

qk_status qk_layer_from_qpk1(qk_ctx *ctx, const uint8_t *bytes, size_t len, int32_t serving_dtype,
                             qk_layer **out) {
    qk_qpk1_info info;
    qk_status st = qk_qpk1_parse(bytes, len, &info);
    if (st != QK_OK) return st;
    // the model loader's rank gate (src/quantibbler/qpk1.py:129-138)
    if (info.r > (info.dout < info.din ? info.dout : info.din))
        return qk::fail(QK_ERR_VALUE, "r=%zu exceeds min(dout, din)=%zu", info.r,
                        info.dout < info.din ? info.dout : info.din);
    std::vector<float> s1(info.dout), s2(info.din), bias(info.dout);
    if ((st = qk_qpk1_scales(bytes, len, s1.data(), s2.data(), bias.data())) != QK_OK) return st;
    // the two container streams go to the device as they are; the rows are separated there
    return qk_layer_create_from_streams(ctx, bytes + info.ub_offset, info.ub_len,
                                        bytes + info.vb_offset, info.vb_len, info.dout, info.din,
                                        info.r, s1.data(), s2.data(),
                                        info.bias_offset ? bias.data() : nullptr, serving_dtype,
                                        out);
}

}  // extern "C"
