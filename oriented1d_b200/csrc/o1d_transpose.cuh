// Batched 2-D transpose [n, a, b] -> [n, b, a] with 128-bit global accesses on both
// sides.  Serves NHWC<->NCHW (reference: nab_to_nba_kernel, a 32x33 tile moved with
// scalar 4-byte accesses, models/dwoconv1d/kernels/nhwc_utils.h:46-110).
//
// One block moves a TILE x TILE patch, TILE = 8 vectors of 16 bytes (32 fp32 / 64 bf16
// elements).  Each thread loads one 16-byte vector per pass along b, scatters it into a
// shared tile whose pitch is an odd number of 32-bit words, then gathers along a and
// stores one 16-byte vector.  Extents that are not a multiple of the vector length use
// element-wise accesses for the affected side.
#pragma once

#include "o1d_common.cuh"

namespace o1d {

constexpr int kTransposeThreads = 256;

template <typename T>
__global__ void __launch_bounds__(kTransposeThreads)
transpose_kernel(const T *__restrict__ in, T *__restrict__ out, int a, int b, int vec_in, int vec_out) {
    constexpr int VEC = 16 / sizeof(T);
    constexpr int TILE = 8 * VEC;
    constexpr int PITCH = TILE + 4 / sizeof(T);     // odd number of 32-bit words
    __shared__ T tile[TILE][PITCH];                 // tile[b_local][a_local]

    const int64_t plane = (int64_t)a * b;
    const T *src = in + (int64_t)blockIdx.z * plane;
    T *dst = out + (int64_t)blockIdx.z * plane;
    const int a0 = blockIdx.y * TILE, b0 = blockIdx.x * TILE;
    const int j = threadIdx.x % 8, r0 = threadIdx.x / 8;

    // load: rows along a, vectors along b
#pragma unroll
    for (int r = r0; r < TILE; r += kTransposeThreads / 8) {
        const int ai = a0 + r, bi = b0 + j * VEC;
        if (ai >= a) continue;
        if (vec_in && bi + VEC <= b) {
            union { uint4 v; T e[VEC]; } u;
            u.v = __ldg(reinterpret_cast<const uint4 *>(src + (int64_t)ai * b + bi));
#pragma unroll
            for (int m = 0; m < VEC; m++) tile[j * VEC + m][r] = u.e[m];
        } else {
#pragma unroll
            for (int m = 0; m < VEC; m++)
                if (bi + m < b) tile[j * VEC + m][r] = src[(int64_t)ai * b + bi + m];
        }
    }
    __syncthreads();
    // store: rows along b, vectors along a
#pragma unroll
    for (int r = r0; r < TILE; r += kTransposeThreads / 8) {
        const int bi = b0 + r, ai = a0 + j * VEC;
        if (bi >= b) continue;
        if (vec_out && ai + VEC <= a) {
            union { uint4 v; T e[VEC]; } u;
#pragma unroll
            for (int m = 0; m < VEC; m++) u.e[m] = tile[r][j * VEC + m];
            *reinterpret_cast<uint4 *>(dst + (int64_t)bi * a + ai) = u.v;
        } else {
#pragma unroll
            for (int m = 0; m < VEC; m++)
                if (ai + m < a) dst[(int64_t)bi * a + ai + m] = tile[r][j * VEC + m];
        }
    }
}

}  // namespace o1d
