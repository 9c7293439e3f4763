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

}  // namespace o1d
