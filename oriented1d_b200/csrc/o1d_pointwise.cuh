// Stem input projection: y[n,h,w,o] = b[o] + sum_c w[o,c] * x[n,c,h,w] for a handful of input
// channels (images: 3), reading the NCHW image and writing the channels-last tensor the first
// oriented convolution wants.  Replaces `x.permute(0,2,3,1)` + `nn.Linear(3, 64)`
// (models/convnext.py:143,170-176), which as a library GEMM with K = 3 plus a separate bias
// pass costs several times the 1.6 GB this moves at batch 256.  Memory-bound: each thread
// produces 8 consecutive output channels of a pixel (one or two 16-byte stores); the CIN input
// values of a pixel are read by the lanes of its channel groups together (one broadcast load).
#pragma once

#include "o1d_common.cuh"

namespace o1d {

constexpr int kPointwiseThreads = 256;
constexpr int kPointwisePasses = 8;      // pixels per thread

// Thread = (group of 8 output channels, pixel lane); its 8 x CIN weights and 8 biases stay in
// registers while it walks kPointwisePasses pixels.
template <typename T, int CIN>
__global__ void __launch_bounds__(kPointwiseThreads)
pointwise_in_kernel(const T *__restrict__ x, const float *__restrict__ w, const float *__restrict__ b,
                    T *__restrict__ y, long long npix, int HW, int Cout) {
    const int groups = Cout / 8;
    const int ppp = kPointwiseThreads / groups;            // pixels per pass of the block
    const int g = threadIdx.x % groups, lp = threadIdx.x / groups;
    if (lp >= ppp) return;
    float wr[8][CIN], br[8];
#pragma unroll
    for (int j = 0; j < 8; j++) {
        br[j] = b ? __ldg(b + g * 8 + j) : 0.f;
#pragma unroll
        for (int c = 0; c < CIN; c++) wr[j][c] = __ldg(w + (g * 8 + j) * CIN + c);
    }
    const long long first = (long long)blockIdx.x * ppp * kPointwisePasses + lp;
#pragma unroll 2
    for (int i = 0; i < kPointwisePasses; i++) {
        const long long pix = first + (long long)i * ppp;
        if (pix >= npix) return;
        const long long n = pix / HW;
        const int hw = (int)(pix - n * HW);
        float xin[CIN];
#pragma unroll
        for (int c = 0; c < CIN; c++) xin[c] = ld(x + (n * CIN + c) * HW + hw);
        float out[8];
#pragma unroll
        for (int j = 0; j < 8; j++) {
            float acc = br[j];
#pragma unroll
            for (int c = 0; c < CIN; c++) acc = fmaf(wr[j][c], xin[c], acc);
            out[j] = acc;
        }
        T *dst = y + pix * Cout + g * 8;
        if constexpr (sizeof(T) == 4) {
            reinterpret_cast<float4 *>(dst)[0] = make_float4(out[0], out[1], out[2], out[3]);
            reinterpret_cast<float4 *>(dst)[1] = make_float4(out[4], out[5], out[6], out[7]);
        } else {
            uint32_t u[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                __nv_bfloat162 h = __floats2bfloat162_rn(out[2 * j], out[2 * j + 1]);
                u[j] = *reinterpret_cast<uint32_t *>(&h);
            }
            *reinterpret_cast<uint4 *>(dst) = make_uint4(u[0], u[1], u[2], u[3]);
        }
    }
}

}  // namespace o1d
