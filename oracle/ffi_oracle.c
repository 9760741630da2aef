/*
 * TEST INFRASTRUCTURE ONLY.  CPU restatement of the reference's fixed-fan-in (FFI)
 * sparse layer, used as the parity oracle by tests/, by the smoke check and as the
 * timed CPU baseline of the benchmark.  Nothing in the product path may call it.
 *
 * Pinned against: the reference's own known-answer forward case (testing/test.cpp:13-47),
 * its eight size fixtures (testing/test.cpp:50-59) and outputs of the reference's own
 * CPU kernels compiled from their sources (see build_oracle.py / ref_adapter.cpp);
 * the committed fixtures under tests/golden/ hold those outputs.
 * Adam and sigmoid-BCE follow third-party (Keras / TensorFlow) formulas that the
 * reference only calls; no reference test pins them: parity unpinned for those two.
 *
 * Layouts (tfsparse/cc/kernels/kernel_data.cu.h:197-225): features [B,N] row-major, or
 * [N,B] when `transposed`; lookup and weights [L,K]; output and out_grad [B,L].
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static int clamp_threads(int threads) {
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_max_threads();
    return threads;
#else
    (void)threads;
    return 1;
#endif
}

int oracle_max_threads(void) { return clamp_threads(0); }

#define X_AT(b, i) (transposed ? x[(size_t)(i) * (size_t)B + (size_t)(b)] : x[(size_t)(b) * (size_t)N + (size_t)(i)])

/* Forward, fp32, same summation order as tfsparse/cc/kernels/forward.cpp:27-43:
 * four partial sums by k mod 4 over the multiple-of-4 prefix, the tail into lane 0,
 * then v0+v1+v2+v3.  Work is split over units as forward.cpp:61-64 does.
 * `bias` (may be NULL) is added afterwards, as sparse/layer.py:245-247 does. */
void oracle_forward_f32(const float* x, const int32_t* idx, const float* W, const float* bias,
                        float* y, int64_t B, int64_t N, int64_t L, int64_t K, int transposed,
                        int threads) {
    threads = clamp_threads(threads);
    (void)threads;
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t o = 0; o < L; ++o) {
        const int32_t* io = idx + (size_t)o * (size_t)K;
        const float* wo = W + (size_t)o * (size_t)K;
        for (int64_t b = 0; b < B; ++b) {
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            int64_t k = 0;
            for (; k + 4 <= K; k += 4)
                for (int j = 0; j < 4; ++j) v[j] += X_AT(b, io[k + j]) * wo[k + j];
            for (; k < K; ++k) v[0] += X_AT(b, io[k]) * wo[k];
            float r = v[0] + v[1] + v[2] + v[3];
            if (bias) r = r + bias[o];
            y[(size_t)b * (size_t)L + (size_t)o] = r;
        }
    }
}

/* Forward with fp64 accumulation (tolerance reference). */
void oracle_forward_f64(const float* x, const int32_t* idx, const float* W, const float* bias,
                        double* y, int64_t B, int64_t N, int64_t L, int64_t K, int transposed,
                        int threads) {
    threads = clamp_threads(threads);
    (void)threads;
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t o = 0; o < L; ++o) {
        const int32_t* io = idx + (size_t)o * (size_t)K;
        const float* wo = W + (size_t)o * (size_t)K;
        for (int64_t b = 0; b < B; ++b) {
            double r = bias ? (double)bias[o] : 0.0;
            for (int64_t k = 0; k < K; ++k) r += (double)X_AT(b, io[k]) * (double)wo[k];
            y[(size_t)b * (size_t)L + (size_t)o] = r;
        }
    }
}

/* grad_W, fp32, batch ascending: tfsparse/cc/kernels/backward.cpp:26-35. */
void oracle_grad_w_f32(const float* x, const int32_t* idx, const float* g, float* gW, int64_t B,
                       int64_t N, int64_t L, int64_t K, int transposed, int threads) {
    threads = clamp_threads(threads);
    (void)threads;
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t o = 0; o < L; ++o) {
        for (int64_t k = 0; k < K; ++k) {
            int32_t src = idx[(size_t)o * (size_t)K + (size_t)k];
            float r = 0.f;
            for (int64_t b = 0; b < B; ++b) r += X_AT(b, src) * g[(size_t)b * (size_t)L + (size_t)o];
            gW[(size_t)o * (size_t)K + (size_t)k] = r;
        }
    }
}

void oracle_grad_w_f64(const float* x, const int32_t* idx, const float* g, double* gW, int64_t B,
                       int64_t N, int64_t L, int64_t K, int transposed, int threads) {
    threads = clamp_threads(threads);
    (void)threads;
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t o = 0; o < L; ++o) {
        for (int64_t k = 0; k < K; ++k) {
            int32_t src = idx[(size_t)o * (size_t)K + (size_t)k];
            double r = 0.0;
            for (int64_t b = 0; b < B; ++b)
                r += (double)X_AT(b, src) * (double)g[(size_t)b * (size_t)L + (size_t)o];
            gW[(size_t)o * (size_t)K + (size_t)k] = r;
        }
    }
}

/* grad_x, fp32: zero the rows, then unit ascending, k ascending
 * (tfsparse/cc/kernels/backward.cpp:52-72).  Work is split over the batch as
 * backward.cpp:103-107 does, so at most B threads are busy. */
void oracle_grad_x_f32(const int32_t* idx, const float* W, const float* g, float* gx, int64_t B,
                       int64_t N, int64_t L, int64_t K, int transposed, int threads) {
    threads = clamp_threads(threads);
    (void)threads;
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t b = 0; b < B; ++b) {
        for (int64_t i = 0; i < N; ++i) {
            if (transposed) gx[(size_t)i * (size_t)B + (size_t)b] = 0.f;
            else gx[(size_t)b * (size_t)N + (size_t)i] = 0.f;
        }
        for (int64_t o = 0; o < L; ++o) {
            float out = g[(size_t)b * (size_t)L + (size_t)o];
            for (int64_t k = 0; k < K; ++k) {
                int32_t src = idx[(size_t)o * (size_t)K + (size_t)k];
                float inc = W[(size_t)o * (size_t)K + (size_t)k] * out;
                if (transposed) gx[(size_t)src * (size_t)B + (size_t)b] += inc;
                else gx[(size_t)b * (size_t)N + (size_t)src] += inc;
            }
        }
    }
}

void oracle_grad_x_f64(const int32_t* idx, const float* W, const float* g, double* gx, int64_t B,
                       int64_t N, int64_t L, int64_t K, int transposed, int threads) {
    threads = clamp_threads(threads);
    (void)threads;
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t b = 0; b < B; ++b) {
        for (int64_t i = 0; i < N; ++i) {
            if (transposed) gx[(size_t)i * (size_t)B + (size_t)b] = 0.0;
            else gx[(size_t)b * (size_t)N + (size_t)i] = 0.0;
        }
        for (int64_t o = 0; o < L; ++o) {
            double out = (double)g[(size_t)b * (size_t)L + (size_t)o];
            for (int64_t k = 0; k < K; ++k) {
                int32_t src = idx[(size_t)o * (size_t)K + (size_t)k];
                double inc = (double)W[(size_t)o * (size_t)K + (size_t)k] * out;
                if (transposed) gx[(size_t)src * (size_t)B + (size_t)b] += inc;
                else gx[(size_t)b * (size_t)N + (size_t)src] += inc;
            }
        }
    }
}

/* grad_bias[o] = sum_b g[b,o]: what TensorFlow's BiasAddGrad computes for the
 * bias_add at sparse/layer.py:247. */
void oracle_grad_bias_f64(const float* g, double* gbias, int64_t B, int64_t L) {
    for (int64_t o = 0; o < L; ++o) gbias[o] = 0.0;
    for (int64_t b = 0; b < B; ++b)
        for (int64_t o = 0; o < L; ++o) gbias[o] += (double)g[(size_t)b * (size_t)L + (size_t)o];
}

/* Transposed (CSR-by-input) index.  The reference has none (its grad_x uses atomics,
 * tfsparse/cc/kernels/backward.cu.h:119-182); this is the normative definition the CUDA
 * build must reproduce bit for bit: flat position p = o*K+k, `perm` lists positions by
 * key idx[p] ascending, ties by p ascending; rowptr[i] = number of entries with key < i.
 * Returns 0, or -1 when an index lies outside [0,N). */
int oracle_transpose_index(const int32_t* idx, int64_t L, int64_t K, int64_t N, int32_t* rowptr,
                           int32_t* perm) {
    int64_t total = L * K;
    int64_t* cursor = (int64_t*)calloc((size_t)N + 1, sizeof(int64_t));
    if (!cursor) return -2;
    for (int64_t p = 0; p < total; ++p) {
        int32_t key = idx[p];
        if (key < 0 || key >= N) {
            free(cursor);
            return -1;
        }
        cursor[key + 1]++;
    }
    for (int64_t i = 0; i < N; ++i) cursor[i + 1] += cursor[i];
    for (int64_t i = 0; i <= N; ++i) rowptr[i] = (int32_t)cursor[i];
    for (int64_t p = 0; p < total; ++p) perm[cursor[idx[p]]++] = (int32_t)p;
    free(cursor);
    return 0;
}

/* Sigmoid binary cross-entropy with sparse multi-hot targets, fp64.
 * Loss value follows sparse/metrics.py:136-139,173 with sparse/utils.py:15-21 and the
 * Keras batch mean: per element max(z,0) - z*t + log1p(exp(-|z|)), mean over the L
 * labels, then mean over the B samples.  Gradient g[b,o] = (sigmoid(z) - t) / (B*L).
 * Targets are CSR: row_ptr[B+1], labels[nnz] (labels within a row are distinct). */
double oracle_bce_f64(const float* z, const int32_t* row_ptr, const int32_t* labels, double* g,
                      int64_t B, int64_t L) {
    double scale = 1.0 / ((double)B * (double)L);
    double total = 0.0;
    for (int64_t b = 0; b < B; ++b) {
        const float* zb = z + (size_t)b * (size_t)L;
        double* gb = g ? g + (size_t)b * (size_t)L : NULL;
        double row = 0.0;
        for (int64_t o = 0; o < L; ++o) {
            double v = (double)zb[o];
            row += (v > 0 ? v : 0.0) + log1p(exp(-fabs(v)));
            if (gb) gb[o] = scale / (1.0 + exp(-v));
        }
        for (int32_t e = row_ptr[b]; e < row_ptr[b + 1]; ++e) {
            int32_t o = labels[e];
            row -= (double)zb[o];
            if (gb) gb[o] -= scale;
        }
        total += row;
    }
    return total * scale;
}

/* Hinge (squared = 0) and squared hinge (squared = 1) losses with sparse multi-hot targets, fp64.
 * Follows SparseHingeLoss / SparseSquaredHingeLoss (sparse/metrics.py:146-164) evaluated the way
 * SparseLossBase.call does (sparse/metrics.py:136-139: every element with target 0, then the
 * positives overwritten, sparse/utils.py:15-21), with the Keras batch mean:
 * margin = (2t-1)*z, h = max(0, 1 - margin), element = h or h^2, mean over L then over B.
 * Gradient g[b,o] = -(2t-1) * (h > 0 ? 1 : 0) / (B*L) (hinge; relu'(0) = 0 as in TensorFlow) or
 * -(2t-1) * 2h / (B*L) (squared). */
double oracle_hinge_f64(const float* z, const int32_t* row_ptr, const int32_t* labels, double* g,
                        int64_t B, int64_t L, int squared) {
    double scale = 1.0 / ((double)B * (double)L);
    double total = 0.0;
    for (int64_t b = 0; b < B; ++b) {
        const float* zb = z + (size_t)b * (size_t)L;
        double* gb = g ? g + (size_t)b * (size_t)L : NULL;
        double row = 0.0;
        for (int64_t o = 0; o < L; ++o) {
            double h = 1.0 + (double)zb[o];
            if (h < 0) h = 0;
            row += squared ? h * h : h;
            if (gb) gb[o] = squared ? 2.0 * h * scale : (h > 0 ? scale : 0.0);
        }
        for (int32_t e = row_ptr[b]; e < row_ptr[b + 1]; ++e) {
            int32_t o = labels[e];
            double hn = 1.0 + (double)zb[o], hp = 1.0 - (double)zb[o];
            if (hn < 0) hn = 0;
            if (hp < 0) hp = 0;
            row += squared ? hp * hp - hn * hn : hp - hn;
            if (gb) gb[o] = squared ? -2.0 * hp * scale : (hp > 0 ? -scale : 0.0);
        }
        total += row;
    }
    return total * scale;
}

/* One Adam step as Keras' Adam.update_step does (the optimizer sparse/optimizer.py:9-12
 * derives from): t = step (1-based), alpha = lr*sqrt(1-b2^t)/(1-b1^t),
 * m += (g-m)(1-b1), v += (g*g-v)(1-b2), w -= alpha*m/(sqrt(v)+eps).  fp64 state. */
void oracle_adam_f64(double* w, double* m, double* v, const double* grad, int64_t n, double lr,
                     double beta1, double beta2, double eps, int64_t step) {
    double alpha = lr * sqrt(1.0 - pow(beta2, (double)step)) / (1.0 - pow(beta1, (double)step));
    for (int64_t j = 0; j < n; ++j) {
        m[j] += (grad[j] - m[j]) * (1.0 - beta1);
        v[j] += (grad[j] * grad[j] - v[j]) * (1.0 - beta2);
        w[j] -= alpha * m[j] / (sqrt(v[j]) + eps);
    }
}
