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
                     int P, int Q, int add_identity, int act) {
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
                float xv = ld(x + at<LAYOUT>(n, c, h, ww, C, H, W));
                if (act) xv = gelu_exact(xv);
                acc = fmaf(xv, wk, acc);
            }
        }
        st(y + idx, acc);
    }
}

// Forward, NHWC, 16-byte channel vectors: a thread owns VE = 16/sizeof(T) consecutive channels
// of one output pixel.  Requires that every aligned group of VE channels shares one
// orientation class (true for the models' block assignment, models/convnext.py:60-65), so the
// group moves along one line and each tap is one 128-bit load.  Weights are staged in shared
// memory transposed ([k][C]) when they fit.  Used for what the tiled kernels do not take
// (stride 2 stems, large images).
template <typename T> struct GVec;
template <> struct GVec<float> {
    static constexpr int N = 4;
    __device__ static void unpack(const uint4 &v, float (&f)[4]) {
        f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
    }
    __device__ static uint4 pack(const float (&f)[4]) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    }
};
template <> struct GVec<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void unpack(const uint4 &v, float (&f)[8]) {
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; i++) { f[2 * i] = __uint_as_float(u[i] << 16); f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u); }
    }
    __device__ static uint4 pack(const float (&f)[8]) {
        uint32_t u[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            u[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(u[0], u[1], u[2], u[3]);
    }
};

template <typename T>
__global__ void __launch_bounds__(kGenericThreads)
generic_fprop_nhwc_vec_kernel(const T *__restrict__ x, const float *__restrict__ w,
                              const float *__restrict__ bias, const uint16_t *__restrict__ cls,
                              const int8_t *__restrict__ taps_gmem, int ncls, int w_staged,
                              T *__restrict__ y, int N, int H, int W, int C, int K, int stride,
                              int P, int Q, int add_identity, int act) {
    constexpr int VE = GVec<T>::N;
    extern __shared__ __align__(16) unsigned char s_raw[];
    // [taps: ncls*K*2 bytes, padded to 16] [weights: K*C floats, if staged]
    int8_t *s_taps = reinterpret_cast<int8_t *>(s_raw);
    const int tap_bytes = (ncls * K * 2 + 15) & ~15;
    float *s_w = reinterpret_cast<float *>(s_raw + tap_bytes);
    for (int i = threadIdx.x; i < ncls * K * 2; i += blockDim.x) s_taps[i] = taps_gmem[i];
    const int pad = K / 2;
    if (w_staged)
        for (int i = threadIdx.x; i < C * K; i += blockDim.x) {
            const int c = i / K, k = i - c * K;
            s_w[k * C + c] = __ldg(w + i) + ((add_identity && k == pad) ? 1.f : 0.f);
        }
    __syncthreads();
    const int G = C / VE;
    const int64_t total = (int64_t)N * P * Q * G;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = idx;
        const int g = (int)(r % G); r /= G;
        const int q = (int)(r % Q); r /= Q;
        const int p = (int)(r % P);
        const int n = (int)(r / P);
        const int c0 = g * VE;
        const int8_t *t = s_taps + (size_t)cls[c0] * K * 2;
        float acc[VE];
#pragma unroll
        for (int j = 0; j < VE; j++) acc[j] = bias ? __ldg(bias + c0 + j) : 0.f;
        for (int k = 0; k < K; k++) {
            const int h = p * stride + t[2 * k], ww = q * stride + t[2 * k + 1];
            if ((unsigned)h < (unsigned)H && (unsigned)ww < (unsigned)W) {
                float xv[VE], wv[VE];
                GVec<T>::unpack(__ldg(reinterpret_cast<const uint4 *>(x + (((int64_t)n * H + h) * W + ww) * C + c0)), xv);
                if (act) {
#pragma unroll
                    for (int j = 0; j < VE; j++) xv[j] = gelu_exact(xv[j]);
                }
                if (w_staged) {
#pragma unroll
                    for (int j = 0; j < VE; j += 4) {
                        const float4 f = *reinterpret_cast<const float4 *>(s_w + k * C + c0 + j);
                        wv[j] = f.x; wv[j + 1] = f.y; wv[j + 2] = f.z; wv[j + 3] = f.w;
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < VE; j++)
                        wv[j] = __ldg(w + (size_t)(c0 + j) * K + k) + ((add_identity && k == pad) ? 1.f : 0.f);
                }
#pragma unroll
                for (int j = 0; j < VE; j++) acc[j] = fmaf(xv[j], wv[j], acc[j]);
            }
        }
        *reinterpret_cast<uint4 *>(y + idx * VE) = GVec<T>::pack(acc);
    }
}

// dx[n,c,h,w] = sum_k w'[c,k] dy[n,c,(h-dh_k)/s,(w-dw_k)/s], taken only where both
// differences are non-negative multiples of s inside [0,P)x[0,Q)     (kernels.cpp:71-90)
template <typename T, int LAYOUT>
__global__ void __launch_bounds__(kGenericThreads)
generic_dgrad_kernel(const T *__restrict__ dy, const float *__restrict__ w,
                     const uint16_t *__restrict__ cls, const int8_t *__restrict__ taps_gmem,
                     int ncls, int staged, T *__restrict__ dx, int N, int H, int W, int C, int K,
                     int stride, int P, int Q, int add_identity, const T *__restrict__ pre) {
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
        if (pre) acc *= gelu_exact_grad(ld(pre + idx));     // the input was GELU(pre): chain rule
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
                             int stride, int P, int Q, int slices, int act) {
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
                        if ((unsigned)h < (unsigned)H && (unsigned)ww < (unsigned)W) {
                            float xv = ld(x + at<LAYOUT>(n, c, h, ww, C, H, W));
                            if (act) xv = gelu_exact(xv);
                            acc[i] = fmaf(xv, g, acc[i]);
                        }
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
