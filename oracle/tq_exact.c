/*
 * Exact-order CPU restatement of TurboQuant quantize (test infrastructure).
 *
 * Follows leankv/turboquant/quantizer.py:119-129 — norm, normalise by (norm + 1e-10),
 * rotate by Pi, count decision boundaries strictly below each rotated coordinate
 * (torch.searchsorted, right=False) — with the summation order the reference leaves to its
 * BLAS fixed as follows, so that the CUDA kernels can be compared bit for bit:
 *   norm = (float) sqrt( S_lo + S_hi ), S_* = fp64 fma sums of squares over coordinates
 *          0..63 and 64..127, ascending
 *   u_k  = x_k / (norm + 1e-10f)                    fp32 division
 *   y_j  = fmaf(Pi[j][k], u_k, y_j), k ascending     fp32
 * margin[j] = min_i |y_j - b_i| lets a caller tell a genuine mismatch from a coordinate
 * that sits within rounding distance of a boundary.
 */
#include <math.h>
#include <stdint.h>
#include <stddef.h>

#define DIM 128

void tq_exact_quantize(const float* x, long n_vec, const float* Pi, const float* bounds,
                       int n_bounds, uint8_t* codes, float* norms, float* y_out, float* margin) {
#pragma omp parallel for schedule(static)
    for (long v = 0; v < n_vec; ++v) {
        const float* xv = x + (size_t)v * DIM;
        double s_lo = 0.0, s_hi = 0.0;
        for (int k = 0; k < 64; ++k) s_lo = fma((double)xv[k], (double)xv[k], s_lo);
        for (int k = 64; k < DIM; ++k) s_hi = fma((double)xv[k], (double)xv[k], s_hi);
        const float norm = (float)sqrt(s_lo + s_hi);
        const float denom = norm + 1e-10f;
        float u[DIM];
        for (int k = 0; k < DIM; ++k) u[k] = xv[k] / denom;
        norms[v] = norm;
        for (int j = 0; j < DIM; ++j) {
            const float* row = Pi + (size_t)j * DIM;
            float y = 0.0f;
            for (int k = 0; k < DIM; ++k) y = fmaf(row[k], u[k], y);
            int c = 0;
            float m = INFINITY;
            for (int i = 0; i < n_bounds; ++i) {
                c += (bounds[i] < y) ? 1 : 0;
                const float dist = fabsf(y - bounds[i]);
                if (dist < m) m = dist;
            }
            codes[(size_t)v * DIM + j] = (uint8_t)c;
            if (y_out) y_out[(size_t)v * DIM + j] = y;
            if (margin) margin[(size_t)v * DIM + j] = m;
        }
    }
}

/* x_hat = norm * (centroids[codes] @ Pi), k ascending fp32 fma; leankv/turboquant/quantizer.py:131-137 */
void tq_exact_dequantize(const uint8_t* codes, const float* norms, long n_vec, const float* Pi,
                         const float* centroids, float* x_hat) {
#pragma omp parallel for schedule(static)
    for (long v = 0; v < n_vec; ++v) {
        float acc[DIM];
        for (int j = 0; j < DIM; ++j) acc[j] = 0.0f;
        for (int k = 0; k < DIM; ++k) {
            const float c = centroids[codes[(size_t)v * DIM + k]];
            const float* row = Pi + (size_t)k * DIM;
            for (int j = 0; j < DIM; ++j) acc[j] = fmaf(c, row[j], acc[j]);
        }
        for (int j = 0; j < DIM; ++j) x_hat[(size_t)v * DIM + j] = acc[j] * norms[v];
    }
}
