/*
 * CPU oracle for the oriented 1D depthwise convolution.  TEST INFRASTRUCTURE ONLY:
 * it is the checker the CUDA path is compared against, never the product path.
 * Nothing in the package imports, links or executes this file.
 *
 * Plain-C restatement of the reference operator's CPU loops
 * (models/dwoconv1d_reference/kernels/kernels.cpp):
 *   - index helper            kernels.cpp:16-18
 *   - fprop loops             kernels.cpp:36-52
 *   - dgrad loops             kernels.cpp:71-90
 *   - wgrad loops             kernels.cpp:111-126
 * The tap rasterisation is the expression at kernels.cpp:37,43-44:
 *   float sin_ = sin(theta[c]), cos_ = cos(theta[c]);   (float overloads -> sinf/cosf)
 *   dh = int(-sin_ * (k - pad));  dw = int(cos_ * (k - pad));   (float product, truncation)
 *
 * Layout of every tensor here is NCHW contiguous fp32, as in the reference loops.
 * The *_f64 variants accumulate in double; they anchor the wgrad tolerance, whose
 * single fp32 accumulator in the reference carries ~1e-5 relative error of its own.
 *
 * Parity status: pinned.  tests/golden/ holds outputs of the reference's own
 * kernels.cpp (compiled by oracle/build.py) and tests/test_oracle.py checks this
 * file against them bit for bit.
 */
#include <math.h>
#include <stdint.h>
#include <stddef.h>

/* kernels.cpp:16-18 */
static inline size_t at4(int n, int c, int h, int w, int C, int H, int W) {
    return (((size_t)n * C + c) * H + h) * W + w;
}

/* kernels.cpp:37,43-44 — tap k of channel c moves by (dh, dw). */
void o1d_oracle_offsets(const float *theta, int C, int K, int32_t *dh, int32_t *dw) {
    const int pad = K / 2;
    for (int c = 0; c < C; c++) {
        float sin_ = sinf(theta[c]), cos_ = cosf(theta[c]);
        for (int k = 0; k < K; k++) {
            dh[(size_t)c * K + k] = (int)(-sin_ * (k - pad));
            dw[(size_t)c * K + k] = (int)(cos_ * (k - pad));
        }
    }
}

/* kernels.cpp:36-52 */
void o1d_oracle_fprop(const float *x, const float *w, const float *theta, float *y,
                      int N, int C, int H, int W, int K, int stride) {
    const int pad = K / 2, P = H / stride, Q = W / stride;
    for (int c = 0; c < C; c++) {
        float sin_ = sinf(theta[c]), cos_ = cosf(theta[c]);
        for (int n = 0; n < N; n++)
            for (int p = 0; p < P; p++)
                for (int q = 0; q < Q; q++) {
                    float sum = 0;
                    for (int s = 0; s < K; s++) {
                        int h = p * stride + (int)(-sin_ * (s - pad));
                        int ww = q * stride + (int)(cos_ * (s - pad));
                        if (h >= 0 && h < H && ww >= 0 && ww < W)
                            sum += x[at4(n, c, h, ww, C, H, W)] * w[(size_t)c * K + s];
                    }
                    y[at4(n, c, p, q, C, P, Q)] = sum;
                }
    }
}

/* kernels.cpp:71-90.  C's % and / truncate toward zero exactly as in the reference,
 * so a negative pp passes the divisibility test only when it is a multiple of stride
 * and is then rejected by p >= 0. */
void o1d_oracle_dgrad(const float *dy, const float *w, const float *theta, float *dx,
                      int N, int C, int P, int Q, int K, int stride) {
    const int pad = K / 2, H = P * stride, W = Q * stride;
    for (int c = 0; c < C; c++) {
        float sin_ = sinf(theta[c]), cos_ = cosf(theta[c]);
        for (int n = 0; n < N; n++)
            for (int h = 0; h < H; h++)
                for (int ww = 0; ww < W; ww++) {
                    float sum = 0;
                    for (int s = 0; s < K; s++) {
                        int pp = h - (int)(-sin_ * (s - pad));
                        int qq = ww - (int)(cos_ * (s - pad));
                        if (pp % stride != 0 || qq % stride != 0) continue;
                        int p = pp / stride, q = qq / stride;
                        if (p >= 0 && p < P && q >= 0 && q < Q)
                            sum += dy[at4(n, c, p, q, C, P, Q)] * w[(size_t)c * K + s];
                    }
                    dx[at4(n, c, h, ww, C, H, W)] = sum;
                }
    }
}

/* kernels.cpp:111-126 (loop order c, s, p, q, n — kept, it fixes the fp32 rounding). */
void o1d_oracle_wgrad(const float *dy, const float *x, const float *theta, float *dwt,
                      int N, int C, int H, int W, int K, int stride) {
    const int pad = K / 2, P = H / stride, Q = W / stride;
    for (int c = 0; c < C; c++) {
        float sin_ = sinf(theta[c]), cos_ = cosf(theta[c]);
        for (int s = 0; s < K; s++) {
            float sum = 0;
            for (int p = 0; p < P; p++)
                for (int q = 0; q < Q; q++) {
                    int h = p * stride + (int)(-sin_ * (s - pad));
                    int ww = q * stride + (int)(cos_ * (s - pad));
                    if (h >= 0 && h < H && ww >= 0 && ww < W)
                        for (int n = 0; n < N; n++)
                            sum += x[at4(n, c, h, ww, C, H, W)] * dy[at4(n, c, p, q, C, P, Q)];
                }
            dwt[(size_t)c * K + s] = sum;
        }
    }
}

/* ---- double-accumulator variants of the same three loops (tolerance anchors) ---- */

void o1d_oracle_fprop_f64(const float *x, const float *w, const float *theta, double *y,
                          int N, int C, int H, int W, int K, int stride) {
    const int pad = K / 2, P = H / stride, Q = W / stride;
    for (int c = 0; c < C; c++) {
        float sin_ = sinf(theta[c]), cos_ = cosf(theta[c]);
        for (int n = 0; n < N; n++)
            for (int p = 0; p < P; p++)
                for (int q = 0; q < Q; q++) {
                    double sum = 0;
                    for (int s = 0; s < K; s++) {
                        int h = p * stride + (int)(-sin_ * (s - pad));
                        int ww = q * stride + (int)(cos_ * (s - pad));
                        if (h >= 0 && h < H && ww >= 0 && ww < W)
                            sum += (double)x[at4(n, c, h, ww, C, H, W)] * (double)w[(size_t)c * K + s];
                    }
                    y[at4(n, c, p, q, C, P, Q)] = sum;
                }
    }
}

void o1d_oracle_dgrad_f64(const float *dy, const float *w, const float *theta, double *dx,
                          int N, int C, int P, int Q, int K, int stride) {
    const int pad = K / 2, H = P * stride, W = Q * stride;
    for (int c = 0; c < C; c++) {
        float sin_ = sinf(theta[c]), cos_ = cosf(theta[c]);
        for (int n = 0; n < N; n++)
            for (int h = 0; h < H; h++)
                for (int ww = 0; ww < W; ww++) {
                    double sum = 0;
                    for (int s = 0; s < K; s++) {
                        int pp = h - (int)(-sin_ * (s - pad));
                        int qq = ww - (int)(cos_ * (s - pad));
                        if (pp % stride != 0 || qq % stride != 0) continue;
                        int p = pp / stride, q = qq / stride;
                        if (p >= 0 && p < P && q >= 0 && q < Q)
                            sum += (double)dy[at4(n, c, p, q, C, P, Q)] * (double)w[(size_t)c * K + s];
                    }
                    dx[at4(n, c, h, ww, C, H, W)] = sum;
                }
    }
}

void o1d_oracle_wgrad_f64(const float *dy, const float *x, const float *theta, double *dwt,
                          int N, int C, int H, int W, int K, int stride) {
    const int pad = K / 2, P = H / stride, Q = W / stride;
    for (int c = 0; c < C; c++) {
        float sin_ = sinf(theta[c]), cos_ = cosf(theta[c]);
        for (int s = 0; s < K; s++) {
            double sum = 0;
            for (int p = 0; p < P; p++)
                for (int q = 0; q < Q; q++) {
                    int h = p * stride + (int)(-sin_ * (s - pad));
                    int ww = q * stride + (int)(cos_ * (s - pad));
                    if (h >= 0 && h < H && ww >= 0 && ww < W)
                        for (int n = 0; n < N; n++)
                            sum += (double)x[at4(n, c, h, ww, C, H, W)] *
                                   (double)dy[at4(n, c, p, q, C, P, Q)];
                }
            dwt[(size_t)c * K + s] = sum;
        }
    }
}
