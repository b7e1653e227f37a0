// Joint-ITQ (alternating Procrustes over Z = [u_hat; v_hat]) on the host.
//
// Compress-time code: the reference runs it on the host in both of its faces
// (crates/quantibbler-kernels/src/core.rs:47-124,327-424 and
// src/quantibbler/kernels/__init__.py:345-512) and pins the int8 sign outputs by golden
// vectors.  Everything that decides a sign follows the reference's order of operations:
// the splitmix64 fill, the modified Gram-Schmidt and every matrix product accumulate left
// to right in float64.  The r x r SVD is the one step the reference delegates to a library
// (nalgebra there, LAPACK in NumPy); only the product Psi * Phi^T of its factors is used,
// which is the orthogonal polar factor of (B^T Z)^T and does not depend on the SVD
// algorithm, so a one-sided Jacobi SVD is used here.
#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdint>
#include <thread>
#include <vector>

#include "qk_common.h"

// keep a*b+c as two roundings: the reference's loops round the product first
#if defined(__GNUC__) && !defined(__clang__)
#pragma GCC optimize("fp-contract=off")
#endif

namespace {

using qk::fail;

constexpr uint64_t kGolden = 0x9E3779B97F4A7C15ull;
constexpr uint64_t kMix1 = 0xBF58476D1CE4E5B9ull;
constexpr uint64_t kMix2 = 0x94D049BB133111EBull;

// core.rs:47-66: rank x rank values in [-1, 1), row-major, from splitmix64.
void splitmix_matrix(uint64_t seed, size_t rank, std::vector<double> &out) {
    uint64_t state = seed;
    out.resize(rank * rank);
    for (size_t i = 0; i < rank * rank; ++i) {
        state += kGolden;
        uint64_t z = state;
        z = (z ^ (z >> 30)) * kMix1;
        z = (z ^ (z >> 27)) * kMix2;
        z ^= z >> 31;
        double u01 = static_cast<double>(z >> 11) / 9007199254740992.0;  // 2^53
        out[i] = u01 * 2.0 - 1.0;
    }
}

// core.rs:72-95: modified Gram-Schmidt, column by column, in place.
bool gram_schmidt(std::vector<double> &a, size_t rank) {
    std::vector<double> v(rank);
    for (size_t j = 0; j < rank; ++j) {
        for (size_t t = 0; t < rank; ++t) v[t] = a[t * rank + j];
        for (size_t i = 0; i < j; ++i) {
            double d = 0.0;
            for (size_t t = 0; t < rank; ++t) d += a[t * rank + i] * v[t];
            for (size_t t = 0; t < rank; ++t) v[t] -= d * a[t * rank + i];
        }
        double s = 0.0;
        for (size_t t = 0; t < rank; ++t) s += v[t] * v[t];
        double nrm = std::sqrt(s);
        if (nrm == 0.0) return false;
        for (size_t t = 0; t < rank; ++t) a[t * rank + j] = v[t] / nrm;
    }
    return true;
}

// Rows [0, n) of a job split over the host's threads; each output element is still
// produced by one thread in the reference's order.
template <class F>
void parallel_rows(size_t n, size_t work_per_row, F &&body) {
    size_t hw = std::max<size_t>(1, std::thread::hardware_concurrency());
    size_t want = std::min(hw, std::max<size_t>(1, n * work_per_row / (1u << 16)));
    want = std::min(want, n);
    if (want <= 1) {
        body(size_t(0), n);
        return;
    }
    std::vector<std::thread> pool;
    size_t per = (n + want - 1) / want;
    for (size_t b = 0; b < n; b += per) pool.emplace_back(body, b, std::min(n, b + per));
    for (auto &t : pool) t.join();
}

// core.rs:98-107: zr = z (n x r) * rr (r x r); element (i, j) sums t = 0..r-1 in order.
void matmul_lr(const double *z, size_t n, size_t r, const double *rr, double *zr) {
    parallel_rows(n, r * r, [&](size_t b, size_t e) {
        std::vector<double> acc(r);
        for (size_t i = b; i < e; ++i) {
            std::fill(acc.begin(), acc.end(), 0.0);
            for (size_t t = 0; t < r; ++t) {
                double x = z[i * r + t];
                const double *row = rr + t * r;
                for (size_t j = 0; j < r; ++j) acc[j] += x * row[j];
            }
            std::copy(acc.begin(), acc.end(), zr + i * r);
        }
    });
}

// core.rs:110-126: out (r x r) = sign(zr)^T * z; element (i, j) sums the n rows in order.
void matmul_signt_z(const double *zr, const double *z, size_t n, size_t r, double *out) {
    parallel_rows(r, n * r, [&](size_t b, size_t e) {
        for (size_t i = b; i < e; ++i) std::fill(out + i * r, out + (i + 1) * r, 0.0);
        for (size_t t = 0; t < n; ++t) {
            const double *zt = z + t * r;
            for (size_t i = b; i < e; ++i) {
                double s = zr[t * r + i] >= 0.0 ? 1.0 : -1.0;
                double *o = out + i * r;
                for (size_t j = 0; j < r; ++j) o[j] += s * zt[j];
            }
        }
    });
}

// One-sided Jacobi (Hestenes) SVD of the r x r matrix a (row-major): on return the columns
// of `u` and `v` hold the left and right singular vectors (a = u * diag(s) * v^T).  Columns
// of u that belong to a zero singular value are completed to an orthonormal basis.
void jacobi_svd(const std::vector<double> &a, size_t r, std::vector<double> &u,
                std::vector<double> &v) {
    // work on columns: store w = a^T so that column p of a is the contiguous row p of w
    std::vector<double> w(r * r), vt(r * r, 0.0);
    for (size_t i = 0; i < r; ++i)
        for (size_t j = 0; j < r; ++j) w[j * r + i] = a[i * r + j];
    for (size_t i = 0; i < r; ++i) vt[i * r + i] = 1.0;
    const double eps = 1e-15;
    // One rotation: make rows p and q of w orthogonal, carry it to vt.  Returns false when the
    // pair is already orthogonal to rounding.
    auto rotate = [&](size_t p, size_t q) -> bool {
        double *wp = &w[p * r], *wq = &w[q * r];
        double alpha = 0.0, beta = 0.0, gamma = 0.0;
        for (size_t t = 0; t < r; ++t) {
            alpha += wp[t] * wp[t];
            beta += wq[t] * wq[t];
            gamma += wp[t] * wq[t];
        }
        if (gamma == 0.0 || std::fabs(gamma) <= eps * std::sqrt(alpha * beta)) return false;
        double zeta = (beta - alpha) / (2.0 * gamma);
        double tn = (zeta >= 0.0 ? 1.0 : -1.0) / (std::fabs(zeta) + std::sqrt(1.0 + zeta * zeta));
        double c = 1.0 / std::sqrt(1.0 + tn * tn), sn = c * tn;
        double *vp = &vt[p * r], *vq = &vt[q * r];
        for (size_t t = 0; t < r; ++t) {
            double x = wp[t], y = wq[t];
            wp[t] = c * x - sn * y;
            wq[t] = sn * x + c * y;
            x = vp[t];
            y = vq[t];
            vp[t] = c * x - sn * y;
            vq[t] = sn * x + c * y;
        }
        return true;
    };
    // Round-robin ordering: a sweep is m - 1 rounds of m / 2 disjoint pairs (m = r rounded up
    // to even; the extra player sits out), so the pairs of a round can be rotated by different
    // threads.  A pair's rotation depends only on its two rows: the result does not depend on
    // the number of threads.
    const size_t m = r + (r & 1), half = m / 2;
    auto pair_of = [&](size_t round, size_t i, size_t *p, size_t *q) {
        size_t a = i == 0 ? m - 1 : (round + i) % (m - 1);
        size_t b = i == 0 ? round : (round + (m - 1) - i) % (m - 1);
        *p = a < b ? a : b;
        *q = a < b ? b : a;
    };
    size_t n_threads = 1;
    if (r >= 128) {
        size_t hw = std::max<size_t>(1, std::thread::hardware_concurrency());
        n_threads = std::min(hw, half / 8);
    }
    std::atomic<int> rotated{0};
    std::atomic<size_t> arrived{0}, generation{0};
    auto barrier = [&]() {
        if (n_threads == 1) return;
        size_t gen = generation.load(std::memory_order_acquire);
        if (arrived.fetch_add(1, std::memory_order_acq_rel) + 1 == n_threads) {
            arrived.store(0, std::memory_order_relaxed);
            generation.fetch_add(1, std::memory_order_acq_rel);
        } else {
            while (generation.load(std::memory_order_acquire) == gen) std::this_thread::yield();
        }
    };
    auto worker = [&](size_t tid) {
        const size_t per = (half + n_threads - 1) / n_threads;
        const size_t lo = std::min(half, tid * per), hi = std::min(half, lo + per);
        for (int sweep = 0; sweep < 60; ++sweep) {
            for (size_t round = 0; round + 1 < m; ++round) {
                bool any = false;
                for (size_t i = lo; i < hi; ++i) {
                    size_t p, q;
                    pair_of(round, i, &p, &q);
                    if (q < r) any |= rotate(p, q);
                }
                if (any) rotated.store(1, std::memory_order_relaxed);
                barrier();
            }
            const bool again = rotated.load(std::memory_order_relaxed) != 0;
            barrier();
            if (tid == 0) rotated.store(0, std::memory_order_relaxed);
            barrier();
            if (!again) break;
        }
    };
    if (m >= 2) {
        std::vector<std::thread> pool;
        for (size_t t = 1; t < n_threads; ++t) pool.emplace_back(worker, t);
        worker(0);
        for (auto &t : pool) t.join();
    }
    // singular values = column norms; normalise, then complete the null columns
    std::vector<double> sigma(r);
    double smax = 0.0;
    for (size_t p = 0; p < r; ++p) {
        double s = 0.0;
        for (size_t t = 0; t < r; ++t) s += w[p * r + t] * w[p * r + t];
        sigma[p] = std::sqrt(s);
        smax = std::max(smax, sigma[p]);
    }
    std::vector<size_t> null_cols;
    for (size_t p = 0; p < r; ++p) {
        if (sigma[p] > smax * 1e-14 && sigma[p] > 0.0) {
            for (size_t t = 0; t < r; ++t) w[p * r + t] /= sigma[p];
        } else {
            null_cols.push_back(p);
            std::fill(&w[p * r], &w[(p + 1) * r], 0.0);
        }
    }
    for (size_t p : null_cols) {
        // the unit vector that is least represented so far, made orthogonal to the rest
        for (size_t cand = 0; cand < r; ++cand) {
            std::vector<double> x(r, 0.0);
            x[cand] = 1.0;
            for (int pass = 0; pass < 2; ++pass)
                for (size_t o = 0; o < r; ++o) {
                    if (o == p) continue;
                    double d = 0.0;
                    for (size_t t = 0; t < r; ++t) d += w[o * r + t] * x[t];
                    for (size_t t = 0; t < r; ++t) x[t] -= d * w[o * r + t];
                }
            double s = 0.0;
            for (size_t t = 0; t < r; ++t) s += x[t] * x[t];
            if (s > 1e-4) {
                s = std::sqrt(s);
                for (size_t t = 0; t < r; ++t) w[p * r + t] = x[t] / s;
                break;
            }
        }
    }
    u.resize(r * r);
    v.resize(r * r);
    for (size_t i = 0; i < r; ++i)
        for (size_t j = 0; j < r; ++j) {
            u[i * r + j] = w[j * r + i];
            v[i * r + j] = vt[j * r + i];
        }
}

}  // namespace

extern "C" qk_status qk_joint_itq(const double *u_hat, size_t u_len, const double *v_hat,
                                  size_t v_len, size_t dout, size_t din, size_t rank,
                                  size_t max_iter, double tol, uint64_t seed, int8_t *u_t,
                                  int8_t *v_t, size_t *n_iter, int32_t *converged) {
    // core.rs:337-346
    if (rank == 0 || dout + din == 0)
        return fail(QK_ERR_VALUE, "joint_itq expects non-empty factors");
    if (u_len != dout * rank || v_len != din * rank)
        return fail(QK_ERR_VALUE, "joint_itq shape mismatch: u_hat %zux%zu, v_hat %zux%zu", dout,
                    u_len / std::max<size_t>(dout, 1), din, rank);
    if ((u_len && !u_hat) || (v_len && !v_hat) || (u_len && !u_t) || (v_len && !v_t))
        return fail(QK_ERR_VALUE, "joint_itq: null buffer");
    const size_t n = dout + din, r = rank;
    std::vector<double> z(n * r);
    std::copy(u_hat, u_hat + u_len, z.begin());
    std::copy(v_hat, v_hat + v_len, z.begin() + u_len);
    std::vector<double> rr;
    splitmix_matrix(seed, r, rr);
    if (!gram_schmidt(rr, r))
        return fail(QK_ERR_VALUE, "joint_itq produced a degenerate zero column building R0");
    std::vector<double> zr(n * r), btz(r * r), phi, psi, r_new(r * r);
    size_t iters = 0;
    bool conv = false;
    for (size_t it = 1; it <= max_iter; ++it) {
        matmul_lr(z.data(), n, r, rr.data(), zr.data());             // B <- sign(Z R)
        matmul_signt_z(zr.data(), z.data(), n, r, btz.data());        // B^T Z
        jacobi_svd(btz, r, phi, psi);                                 // = Phi S Psi^T
        for (size_t i = 0; i < r; ++i)                                // R <- Psi Phi^T
            for (size_t j = 0; j < r; ++j) {
                double acc = 0.0;
                for (size_t t = 0; t < r; ++t) acc += psi[i * r + t] * phi[j * r + t];
                r_new[i * r + j] = acc;
            }
        double delta_sq = 0.0;
        for (size_t i = 0; i < r * r; ++i) {
            double d = r_new[i] - rr[i];
            delta_sq += d * d;
        }
        rr = r_new;
        iters = it;
        if (tol > 0.0 && std::sqrt(delta_sq) <= tol) {
            conv = true;
            break;
        }
    }
    matmul_lr(z.data(), n, r, rr.data(), zr.data());
    for (size_t i = 0; i < u_len; ++i) u_t[i] = zr[i] >= 0.0 ? 1 : -1;
    for (size_t i = 0; i < v_len; ++i) v_t[i] = zr[u_len + i] >= 0.0 ? 1 : -1;
    if (n_iter) *n_iter = iters;
    if (converged) *converged = conv ? 1 : 0;
    return QK_OK;
}
