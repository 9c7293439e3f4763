// Channels-last LayerNorm (optionally followed by exact GELU) for the step right after the
// oriented convolution in ConvNeXt-1D blocks and stems (reference: models/convnext.py:28-56,
// :183-189, :309; the reference uses F.layer_norm).  Rows are pixels, the normalised axis is
// the contiguous channel axis (64..1024 channels).  A row is handled by a group of G lanes
// (8, 16 or 32) so that short rows still fill the warp; every lane moves 16-byte vectors,
// keeps its part of the row in registers, and the statistics are two-pass (mean, then
// centred sum of squares) with shuffle reductions inside the group.  One read and one write
// of the tensor: HBM-bound.
#pragma once

#include "o1d_common.cuh"
#include "o1d_generic.cuh"   // GVec

namespace o1d {

constexpr int kLnThreads = 256;

__device__ __forceinline__ float gelu_erf(float v) { return 0.5f * v * (1.f + erff(v * 0.70710678118654752f)); }

// G lanes per row, VPL vectors per lane (row length C <= G * VPL * VE, C % VE == 0)
template <typename T, int G, int VPL>
__global__ void __launch_bounds__(kLnThreads)
layernorm_cl_kernel(const T *__restrict__ x, const float *__restrict__ gamma, const float *__restrict__ beta,
                    T *__restrict__ y, int64_t rows, int C, float eps, int gelu) {
    constexpr int VE = GVec<T>::N;
    const int lane_in_group = threadIdx.x % G;
    const int64_t group = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
    const int64_t ngroups = ((int64_t)gridDim.x * blockDim.x) / G;
    const int nvec = C / VE;
    // this lane's columns: vectors lane_in_group, lane_in_group + G, ...
    float g[VPL][VE], b[VPL][VE];
#pragma unroll
    for (int v = 0; v < VPL; v++) {
        const int vi = lane_in_group + v * G;
#pragma unroll
        for (int j = 0; j < VE; j++) {
            g[v][j] = (vi < nvec) ? __ldg(gamma + vi * VE + j) : 0.f;
            b[v][j] = (vi < nvec) ? __ldg(beta + vi * VE + j) : 0.f;
        }
    }
    const float inv_c = 1.f / (float)C;
    for (int64_t r = group; r < rows; r += ngroups) {
        const T *xr = x + r * C;
        float f[VPL][VE];
        float sum = 0.f;
#pragma unroll
        for (int v = 0; v < VPL; v++) {
            const int vi = lane_in_group + v * G;
            if (vi < nvec) {
                GVec<T>::unpack(__ldg(reinterpret_cast<const uint4 *>(xr + vi * VE)), f[v]);
#pragma unroll
                for (int j = 0; j < VE; j++) sum += f[v][j];
            } else {
#pragma unroll
                for (int j = 0; j < VE; j++) f[v][j] = 0.f;
            }
        }
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float mean = sum * inv_c;
        float sq = 0.f;
#pragma unroll
        for (int v = 0; v < VPL; v++) {
            const int vi = lane_in_group + v * G;
            if (vi < nvec) {
#pragma unroll
                for (int j = 0; j < VE; j++) { const float d = f[v][j] - mean; sq += d * d; }
            }
        }
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        const float rstd = rsqrtf(sq * inv_c + eps);
        T *yr = y + r * C;
#pragma unroll
        for (int v = 0; v < VPL; v++) {
            const int vi = lane_in_group + v * G;
            if (vi < nvec) {
                float o[VE];
#pragma unroll
                for (int j = 0; j < VE; j++) {
                    float t = (f[v][j] - mean) * rstd * g[v][j] + b[v][j];
                    o[j] = gelu ? gelu_erf(t) : t;
                }
                *reinterpret_cast<uint4 *>(yr + vi * VE) = GVec<T>::pack(o);
            }
        }
    }
}


// Backward of the same LayerNorm (no GELU): dx, and per-CTA partial sums of dgamma / dbeta that a
// second kernel adds in CTA order (no atomics: bit-reproducible).  The row statistics are
// recomputed from x (the row sits in registers anyway), so the forward pass keeps nothing but x.
//   xhat = (x - mean) * rstd,  g = dy * gamma,
//   dx = rstd * (g - mean_C(g) - xhat * mean_C(g * xhat)),  dgamma = sum_rows dy * xhat,  dbeta = sum_rows dy.
// F.layer_norm's backward in the reference's training step (models/convnext.py:28-56 through autograd).
// partial: [gridDim.x][2][C] floats.  Dynamic shared memory: (kLnThreads / 32) * 2 * C floats.
// GELU: the forward pass was LayerNorm followed by exact GELU (the stems); dy is then the gradient of the
// GELU output and is first multiplied by GELU'(xhat * gamma + beta).
template <typename T, int G, int VPL, bool GELU>
__global__ void __launch_bounds__(kLnThreads)
layernorm_cl_bwd_kernel(const T *__restrict__ x, const T *__restrict__ dy, const float *__restrict__ gamma,
                        const float *__restrict__ beta, T *__restrict__ dx, float *__restrict__ partial, int64_t rows,
                        int C, float eps) {
    extern __shared__ float ln_red[];                 // [warps][2][C]
    constexpr int VE = GVec<T>::N;
    const int lane_in_group = threadIdx.x % G;
    const int64_t group = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) / G;
    const int64_t ngroups = ((int64_t)gridDim.x * blockDim.x) / G;
    const int nvec = C / VE;
    float g[VPL][VE], bt[GELU ? VPL : 1][VE], sg[VPL][VE], sb[VPL][VE];
#pragma unroll
    for (int v = 0; v < VPL; v++) {
        const int vi = lane_in_group + v * G;
#pragma unroll
        for (int j = 0; j < VE; j++) {
            g[v][j] = (vi < nvec) ? __ldg(gamma + vi * VE + j) : 0.f;
            if (GELU) bt[GELU ? v : 0][j] = (vi < nvec) ? __ldg(beta + vi * VE + j) : 0.f;
            sg[v][j] = 0.f; sb[v][j] = 0.f;
        }
    }
    const float inv_c = 1.f / (float)C;
    // The loop count must be the same for every lane of a warp: the column sums are shuffled across the
    // warp's groups after the loop, and a lane that left the loop early would meet the others at a
    // different shuffle.  So a warp walks its groups' rows together; a group past the last row runs on zeros.
    const int group_in_warp = (threadIdx.x & 31) / G;
    for (int64_t rb = group - group_in_warp; rb < rows; rb += ngroups) {
        const int64_t r = rb + group_in_warp;
        const bool act = r < rows;
        const T *xr = x + (act ? r : 0) * C, *dr = dy + (act ? r : 0) * C;
        float f[VPL][VE], d[VPL][VE];
        float sum = 0.f;
#pragma unroll
        for (int v = 0; v < VPL; v++) {
            const int vi = lane_in_group + v * G;
            if (act && vi < nvec) {
                GVec<T>::unpack(__ldg(reinterpret_cast<const uint4 *>(xr + vi * VE)), f[v]);
                GVec<T>::unpack(__ldg(reinterpret_cast<const uint4 *>(dr + vi * VE)), d[v]);
#pragma unroll
                for (int j = 0; j < VE; j++) sum += f[v][j];
            } else {
#pragma unroll
                for (int j = 0; j < VE; j++) { f[v][j] = 0.f; d[v][j] = 0.f; }
            }
        }
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float mean = sum * inv_c;
        float sq = 0.f;
#pragma unroll
        for (int v = 0; v < VPL; v++) {
            const int vi = lane_in_group + v * G;
            if (vi < nvec) {
#pragma unroll
                for (int j = 0; j < VE; j++) { const float c = f[v][j] - mean; sq += c * c; }
            }
        }
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        const float rstd = rsqrtf(sq * inv_c + eps);
        float c1 = 0.f, c2 = 0.f;
#pragma unroll
        for (int v = 0; v < VPL; v++) {
            const int vi = lane_in_group + v * G;
            if (vi < nvec) {
#pragma unroll
                for (int j = 0; j < VE; j++) {
                    const float xh = (f[v][j] - mean) * rstd;
                    f[v][j] = xh;                                 // keep xhat
                    if (GELU) d[v][j] *= gelu_exact_grad(xh * g[v][j] + bt[GELU ? v : 0][j]);
                    const float gg = d[v][j] * g[v][j];
                    c1 += gg; c2 += gg * xh;
                    sg[v][j] += d[v][j] * xh; sb[v][j] += d[v][j];
                }
            }
        }
#pragma unroll
        for (int o = G / 2; o > 0; o >>= 1) {
            c1 += __shfl_xor_sync(0xffffffffu, c1, o);
            c2 += __shfl_xor_sync(0xffffffffu, c2, o);
        }
        c1 *= inv_c; c2 *= inv_c;
        T *xo = dx + (act ? r : 0) * C;
#pragma unroll
        for (int v = 0; v < VPL; v++) {
            const int vi = lane_in_group + v * G;
            if (act && vi < nvec) {
                float o[VE];
#pragma unroll
                for (int j = 0; j < VE; j++) o[j] = rstd * (d[v][j] * g[v][j] - c1 - f[v][j] * c2);
                *reinterpret_cast<uint4 *>(xo + vi * VE) = GVec<T>::pack(o);
            }
        }
    }
    // column sums: groups of one warp (same lane_in_group), then the warps of the CTA in order
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int v = 0; v < VPL; v++)
#pragma unroll
        for (int j = 0; j < VE; j++) {
#pragma unroll
            for (int o = G; o < 32; o <<= 1) {
                sg[v][j] += __shfl_xor_sync(0xffffffffu, sg[v][j], o);
                sb[v][j] += __shfl_xor_sync(0xffffffffu, sb[v][j], o);
            }
        }
    if (lane < G) {
#pragma unroll
        for (int v = 0; v < VPL; v++) {
            const int vi = lane_in_group + v * G;
            if (vi < nvec) {
#pragma unroll
                for (int j = 0; j < VE; j++) {
                    ln_red[(warp * 2 + 0) * C + vi * VE + j] = sg[v][j];
                    ln_red[(warp * 2 + 1) * C + vi * VE + j] = sb[v][j];
                }
            }
        }
    }
    __syncthreads();
    for (int e = threadIdx.x; e < 2 * C; e += blockDim.x) {
        const int which = e / C, c = e - which * C;
        float s = 0.f;
        for (int w = 0; w < nwarps; w++) s += ln_red[(w * 2 + which) * C + c];
        partial[(size_t)blockIdx.x * 2 * C + e] = s;
    }
}

// dgamma[c] = sum over CTAs of partial[cta][0][c], dbeta likewise from partial[cta][1][c].  Block (32, 8):
// thread (x, y) adds the CTAs congruent to y modulo 8 for one column, the eight sums are then added in
// order of y: a fixed order, with an eighth of the dependent loads per thread.
__global__ void layernorm_cl_bwd_final_kernel(const float *__restrict__ partial, float *__restrict__ dgamma,
                                              float *__restrict__ dbeta, int ctas, int C) {
    __shared__ float part[8][33];
    const int e = blockIdx.x * 32 + threadIdx.x;
    float s = 0.f;
    if (e < 2 * C)
        for (int b = threadIdx.y; b < ctas; b += 8) s += partial[(size_t)b * 2 * C + e];
    part[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && e < 2 * C) {
        float t = 0.f;
#pragma unroll
        for (int y = 0; y < 8; y++) t += part[y][threadIdx.x];
        if (e < C) dgamma[e] = t; else dbeta[e - C] = t;
    }
}

}  // namespace o1d
