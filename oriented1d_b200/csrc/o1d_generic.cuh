// General kernels: any stride, any odd K, any per-channel angle, both layouts, both
// dtypes.  They read through L1/L2 with per-tap bounds tests and are the route for
// every request the tiled kernels (o1d_tiled.cuh) do not take.  Semantics follow the
// reference loops (models/dwoconv1d_reference/kernels/kernels.cpp:36-52, :71-90,
// :111-126); unlike the reference's GPU kernels the tap offsets come from the plan's
// table instead of a per-tap sincosf/float->int conversion (kernels.h:239-240,285).
#pragma once

#include "o1d_common.cuh"

namespace o1d {

constexpr int kGenericThreads = 256;
constexpr int kTapSmemBudget = 32 * 1024;   // class tables are staged in smem up to this size

// Stage the class tap tables into shared memory when they fit; returns the pointer to use.
__device__ __forceinline__ const int8_t *stage_taps(const int8_t *taps_gmem, int ncls, int K,
                                                    int8_t *smem, bool staged) {
    if (!staged) return taps_gmem;
    const int bytes = ncls * K * 2;
    for (int i = threadIdx.x; i < bytes; i += blockDim.x) smem[i] = taps_gmem[i];
    __syncthreads();
    return smem;
}

// Decode a flat output index.  NHWC: c fastest; NCHW: w fastest.
template <int LAYOUT>
__device__ __forceinline__ void decode(int64_t idx, int C, int P, int Q, int &n, int &c, int &p, int &q) {
    if (LAYOUT == O1D_NHWC) {
        c = (int)(idx % C); idx /= C;
        q = (int)(idx % Q); idx /= Q;
        p = (int)(idx % P); n = (int)(idx / P);
    } else {
        q = (int)(idx % Q); idx /= Q;
        p = (int)(idx % P); idx /= P;
        c = (int)(idx % C); n = (int)(idx / C);
    }
}

// y[n,c,p,q] = bias[c] + sum_k w'[c,k] x[n,c,p*s+dh_k,q*s+dw_k]      (kernels.cpp:36-52)
template <typename T, int LAYOUT>
__global__ void __launch_bounds__(kGenericThreads)
generic_fprop_kernel(const T *__restrict__ x, const float *__restrict__ w,
                     const float *__restrict__ bias, const uint16_t *__restrict__ cls,
                     const int8_t *__restrict__ taps_gmem, int ncls, int staged,
                     T *__restrict__ y, int N, int H, int W, int C, int K, int stride,
                     int P, int Q, int add_identity) {
    extern __shared__ int8_t s_taps[];
    const int8_t *taps = stage_taps(taps_gmem, ncls, K, s_taps, staged != 0);
    const int pad = K / 2;
    const int64_t total = (int64_t)N * P * Q * C;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        int n, c, p, q;
        decode<LAYOUT>(idx, C, P, Q, n, c, p, q);
        const int8_t *t = taps + (size_t)cls[c] * K * 2;
        const float *wc = w + (size_t)c * K;
        float acc = bias ? __ldg(bias + c) : 0.f;
        for (int k = 0; k < K; k++) {
            const int h = p * stride + t[2 * k], ww = q * stride + t[2 * k + 1];
            if ((unsigned)h < (unsigned)H && (unsigned)ww < (unsigned)W) {
                float wk = __ldg(wc + k);
                if (add_identity && k == pad) wk += 1.f;
                acc = fmaf(ld(x + at<LAYOUT>(n, c, h, ww, C, H, W)), wk, acc);
            }
        }
        st(y + idx, acc);
    }
}

// dx[n,c,h,w] = sum_k w'[c,k] dy[n,c,(h-dh_k)/s,(w-dw_k)/s], taken only where both
// differences are non-negative multiples of s inside [0,P)x[0,Q)     (kernels.cpp:71-90)
template <typename T, int LAYOUT>
__global__ void __launch_bounds__(kGenericThreads)
generic_dgrad_kernel(const T *__restrict__ dy, const float *__restrict__ w,
                     const uint16_t *__restrict__ cls, const int8_t *__restrict__ taps_gmem,
                     int ncls, int staged, T *__restrict__ dx, int N, int H, int W, int C, int K,
                     int stride, int P, int Q, int add_identity) {
    extern __shared__ int8_t s_taps[];
    const int8_t *taps = stage_taps(taps_gmem, ncls, K, s_taps, staged != 0);
    const int pad = K / 2;
    const int64_t total = (int64_t)N * H * W * C;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        int n, c, h, ww;
        decode<LAYOUT>(idx, C, H, W, n, c, h, ww);
        const int8_t *t = taps + (size_t)cls[c] * K * 2;
        const float *wc = w + (size_t)c * K;
        float acc = 0.f;
        for (int k = 0; k < K; k++) {
            const int pp = h - t[2 * k], qq = ww - t[2 * k + 1];
            if (pp < 0 || qq < 0 || pp % stride != 0 || qq % stride != 0) continue;
            const int p = pp / stride, q = qq / stride;
            if (p < P && q < Q) {
                float wk = __ldg(wc + k);
                if (add_identity && k == pad) wk += 1.f;
                acc = fmaf(ld(dy + at<LAYOUT>(n, c, p, q, C, P, Q)), wk, acc);
            }
        }
        st(dx + idx, acc);
    }
}

// ---------------------------------------------------------------------------------
// Weight gradient, two deterministic levels                         (kernels.cpp:111-126)
//   level 1: block (chunk of channels, slice s of the N*P*Q outputs) -> partial[s][c][0..K]
//            (slot K holds the bias-gradient partial)
//   level 2: dw[c][k] = sum_s partial[s][c][k] in slice order
// Block shape: CL channel lanes x PG pixel groups.  NHWC: 32 x 8 (lanes along C, the
// contiguous axis); NCHW: 1 x 256 (threads along W).  Taps are processed in chunks of
// kWgradTapChunk register accumulators so that any K is handled.
// ---------------------------------------------------------------------------------
constexpr int kWgradTapChunk = 32;

template <int LAYOUT> struct WgradShape {
    static constexpr int CL = (LAYOUT == O1D_NHWC) ? 32 : 1;
    static constexpr int PG = kGenericThreads / CL;
};

template <typename T, int LAYOUT>
__global__ void __launch_bounds__(kGenericThreads)
generic_wgrad_partial_kernel(const T *__restrict__ dy, const T *__restrict__ x,
                             const uint16_t *__restrict__ cls, const int8_t *__restrict__ taps,
                             float *__restrict__ partial, int N, int H, int W, int C, int K,
                             int stride, int P, int Q, int slices) {
    constexpr int CL = WgradShape<LAYOUT>::CL, PG = WgradShape<LAYOUT>::PG;
    __shared__ float red[kGenericThreads];
    const int lane = threadIdx.x % CL, grp = threadIdx.x / CL;
    const int c = blockIdx.x * CL + lane;
    const int s = blockIdx.y;
    const int64_t npq = (int64_t)N * P * Q;
    const int64_t per = (npq + slices - 1) / slices;
    const int64_t lo = (int64_t)s * per, hi = (lo + per < npq) ? lo + per : npq;
    const bool live = c < C;
    const int8_t *t = taps + (live ? (size_t)cls[c] * K * 2 : 0);
    float *out = partial + ((size_t)s * C + (live ? c : 0)) * (K + 1);

    for (int k0 = 0; k0 < K + 1; k0 += kWgradTapChunk) {   // slot K is the db accumulator
        float acc[kWgradTapChunk];
#pragma unroll
        for (int i = 0; i < kWgradTapChunk; i++) acc[i] = 0.f;
        if (live) {
            for (int64_t pix = lo + grp; pix < hi; pix += PG) {
                const int q = (int)(pix % Q);
                const int p = (int)((pix / Q) % P);
                const int n = (int)(pix / ((int64_t)P * Q));
                const float g = ld(dy + at<LAYOUT>(n, c, p, q, C, P, Q));
#pragma unroll
                for (int i = 0; i < kWgradTapChunk; i++) {
                    const int k = k0 + i;
                    if (k < K) {
                        const int h = p * stride + t[2 * k], ww = q * stride + t[2 * k + 1];
                        if ((unsigned)h < (unsigned)H && (unsigned)ww < (unsigned)W)
                            acc[i] = fmaf(ld(x + at<LAYOUT>(n, c, h, ww, C, H, W)), g, acc[i]);
                    } else if (k == K) {
                        acc[i] += g;
                    }
                }
            }
        }
        // Fixed-order reduction over the PG pixel groups, one tap at a time.
#pragma unroll 1
        for (int i = 0; i < kWgradTapChunk; i++) {
            if (k0 + i > K) break;
            __syncthreads();
            red[threadIdx.x] = acc[i];
            __syncthreads();
            if (CL == 1) {      // 256 values of one channel: tree over a fixed pairing
                for (int off = kGenericThreads / 2; off > 0; off >>= 1) {
                    if (threadIdx.x < off) red[threadIdx.x] += red[threadIdx.x + off];
                    __syncthreads();
                }
                if (threadIdx.x == 0 && live) out[k0 + i] = red[0];
            } else if (grp == 0 && live) {
                float sum = 0.f;
                for (int g2 = 0; g2 < PG; g2++) sum += red[g2 * CL + lane];
                out[k0 + i] = sum;
            }
        }
    }
}

// Level 2: fixed-order sum over slices.  One thread per (c, k); k == K is db.
__global__ void wgrad_final_kernel(const float *__restrict__ partial, float *__restrict__ dw,
                                   float *__restrict__ db, int C, int K, int slices) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= C * (K + 1)) return;
    const int c = idx / (K + 1), k = idx % (K + 1);
    if (k == K && db == nullptr) return;
    float sum = 0.f;
    for (int s = 0; s < slices; s++) sum += partial[((size_t)s * C + c) * (K + 1) + k];
    if (k == K) db[c] = sum; else dw[(size_t)c * K + k] = sum;
}

}  // namespace o1d
