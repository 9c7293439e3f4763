// Stem input projection: y[n,h,w,o] = b[o] + sum_c w[o,c] * x[n,c,h,w] for a handful of input
// channels (images: 3), reading the NCHW image and writing the channels-last tensor the first
// oriented convolution wants.  Replaces `x.permute(0,2,3,1)` + `nn.Linear(3, 64)`
// (models/convnext.py:143,170-176), which as a library GEMM with K = 3 plus a separate bias
// pass costs several times the 1.6 GB this moves at batch 256.  Memory-bound: each thread
// produces 8 consecutive output channels of a pixel (one or two 16-byte stores); the CIN input
// values of a pixel are read by the lanes of its channel groups together (one broadcast load).
#pragma once

#include "o1d_common.cuh"
#include "o1d_generic.cuh"   // GVec

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


// Column sums of a channels-last matrix: out[c] = sum over rows of x[r, c].  This is the bias gradient of
// the Linear layers around the convolution in a block (models/convnext.py:298-300,310,312 through
// autograd, which sums grad_output over its rows).  CTA (bx, by): columns [bx*256*VE, ...) as one 16-byte
// vector per thread, rows by, by + gridDim.y, ...; fp32 partial per (by, column); a second kernel
// (layernorm_cl_bwd_final_kernel's pattern, here colsum_final_kernel) adds the row slices in a fixed
// order.  Every load is a full 16-byte vector of a contiguous 4 KB row segment.
constexpr int kColsumThreads = 256;
// RL = rows a CTA reads per pass = 256 / (vectors per row rounded up to a power of two), so that narrow
// matrices still use every lane; the RL row lanes of a column are added in lane order through shared memory.
template <typename T, int RL>
__global__ void __launch_bounds__(kColsumThreads)
colsum_partial_kernel(const T *__restrict__ x, float *__restrict__ partial, int64_t rows, int C) {
    constexpr int VE = 16 / (int)sizeof(T), VPB = kColsumThreads / RL;       // vectors of a row per CTA
    __shared__ float red[RL > 1 ? kColsumThreads * VE : 1];
    const int vl = threadIdx.x % VPB, rl = threadIdx.x / VPB;
    const int vec = blockIdx.x * VPB + vl, nvec = C / VE;
    const bool act = vec < nvec;
    float acc[VE];
#pragma unroll
    for (int j = 0; j < VE; j++) acc[j] = 0.f;
    if (act) {
        const T *col = x + (size_t)vec * VE;
        const int64_t step = (int64_t)gridDim.y * RL;
        int64_t r = (int64_t)blockIdx.y * RL + rl;
        for (; r + 3 * step < rows; r += 4 * step) {         // four rows in flight per thread
            uint4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) v[u] = __ldg(reinterpret_cast<const uint4 *>(col + (r + u * step) * C));
#pragma unroll
            for (int u = 0; u < 4; u++) {
                float f[VE];
                GVec<T>::unpack(v[u], f);
#pragma unroll
                for (int j = 0; j < VE; j++) acc[j] += f[j];
            }
        }
        for (; r < rows; r += step) {
            float f[VE];
            GVec<T>::unpack(__ldg(reinterpret_cast<const uint4 *>(col + r * C)), f);
#pragma unroll
            for (int j = 0; j < VE; j++) acc[j] += f[j];
        }
    }
    if (RL > 1) {
#pragma unroll
        for (int j = 0; j < VE; j++) red[(rl * VE + j) * VPB + vl] = acc[j];
        __syncthreads();
        if (rl == 0 && act) {
#pragma unroll
            for (int j = 0; j < VE; j++) {
                float s = 0.f;
                for (int q = 0; q < RL; q++) s += red[(q * VE + j) * VPB + vl];
                acc[j] = s;
            }
        }
    }
    if (rl == 0 && act) {
        float *dst = partial + (size_t)blockIdx.y * C + (size_t)vec * VE;
#pragma unroll
        for (int j = 0; j < VE; j++) dst[j] = acc[j];
    }
}

// out[c] = sum over slices (in a fixed order) of partial[slice][c].  Block (32, 8) as in the LayerNorm backward.
__global__ void colsum_final_kernel(const float *__restrict__ partial, float *__restrict__ out, int slices, int C) {
    __shared__ float part[8][33];
    const int c = blockIdx.x * 32 + threadIdx.x;
    float s = 0.f;
    if (c < C)
        for (int b = threadIdx.y; b < slices; b += 8) s += partial[(size_t)b * C + c];
    part[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && c < C) {
        float t = 0.f;
#pragma unroll
        for (int y = 0; y < 8; y++) t += part[y][threadIdx.x];
        out[c] = t;
    }
}

}  // namespace o1d
