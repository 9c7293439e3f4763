// Shared definitions for the o1d kernels: plan blob layout, dtype helpers, error macros.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/o1d.h"

namespace o1d {

// ---------------------------------------------------------------------------------
// Plan blob.  The same bytes live on the host and on the device.
//   [PlanHeader (64 B)] [cls: C x uint16, padded to 16 B] [taps: ncls x K x (dh,dw) int8,
//   padded to 16 B] [canon: ncls x int8, padded to 16 B] [comps: 5 x KindComp]
//   [chan: C x int8, padded to 16 B]
// cls[c]    orientation class of channel c
// taps      rasterised offsets of each class, exactly the reference's
//           (int)(-sinf(theta)*j), (int)(cosf(theta)*j)  (kernels.cpp:43-44)
// canon[i]  0..7 when class i's line equals the built-in table of the i*22.5 degree
//           orientation (those have compile-time specialised kernels), else -1
// chan[c]   canon[cls[c]]: the canonical id of channel c in one lookup
// comps[i]  for chunk width kChunkWidths[i]: the distinct (axis, slant, diagonal) channel
//           counts a chunk of that many consecutive channels can have (tiled kernels size
//           their thread groups from it); n = -1 when C is not a multiple of the width or
//           there are more than kMaxComps distinct triples
// ---------------------------------------------------------------------------------
constexpr int kNumChunkWidths = 5;
constexpr int kChunkWidths[kNumChunkWidths] = {4, 8, 16, 32, 64};
constexpr int kMaxComps = 16;
struct KindComp {
    int32_t n;
    uint8_t tri[kMaxComps][3];
};

constexpr uint32_t kPlanMagic = 0x4f314450u;  // "O1DP"

struct PlanHeader {
    uint32_t magic;
    int32_t C, K, ncls;
    int32_t max_dh, max_dw;   // largest |dh|, |dw| over all classes
    int32_t all_canon;        // 1 when every class has canon >= 0
    uint32_t cls_off, taps_off, canon_off, total_bytes;
    uint32_t comps_off, chan_off;
    int32_t uniform4, uniform8;   // every aligned group of 4 / 8 channels shares one class
    uint32_t reserved[1];
};
static_assert(sizeof(PlanHeader) == 64, "plan header is 64 bytes");

__host__ __device__ inline uint32_t align16(uint32_t v) { return (v + 15u) & ~15u; }

struct PlanView {   // pointers into one blob (host or device)
    const uint16_t *cls;
    const int8_t *taps;   // [ncls][K][2]
    const int8_t *canon;
    const int8_t *chan;   // [C] canonical id per channel
    int ncls;
};

inline PlanView plan_view(const void *blob, const PlanHeader &h) {
    const char *b = static_cast<const char *>(blob);
    return PlanView{reinterpret_cast<const uint16_t *>(b + h.cls_off),
                    reinterpret_cast<const int8_t *>(b + h.taps_off),
                    reinterpret_cast<const int8_t *>(b + h.canon_off),
                    reinterpret_cast<const int8_t *>(b + h.chan_off), h.ncls};
}

// ---------------------------------------------------------------------------------
// Element access: storage type T (float or __nv_bfloat16), arithmetic in float.
// ---------------------------------------------------------------------------------
__device__ __forceinline__ float ld(const float *p) { return __ldg(p); }
__device__ __forceinline__ float ld(const __nv_bfloat16 *p) {
    return __bfloat162float(*p);
}
__device__ __forceinline__ void st(float *p, float v) { *p = v; }
__device__ __forceinline__ void st(__nv_bfloat16 *p, float v) { *p = __float2bfloat16_rn(v); }

// Index of element (n, c, h, w) in an [N,C,H,W] tensor stored NCHW (LAYOUT 0) or NHWC (1).
template <int LAYOUT>
__device__ __forceinline__ int64_t at(int n, int c, int h, int w, int C, int H, int W) {
    if (LAYOUT == O1D_NHWC) return (((int64_t)n * H + h) * W + w) * C + c;
    return (((int64_t)n * C + c) * H + h) * W + w;
}

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Exact (erf) GELU and its derivative, as torch.nn.functional.gelu computes them.  A conv whose
// input is the GELU of a tensor applies it while loading that tensor ("activation on load"), and
// its input gradient is multiplied by the derivative at the same pre-activation values.
__device__ __forceinline__ float gelu_exact(float v) { return 0.5f * v * (1.f + erff(v * 0.70710678118654752f)); }
__device__ __forceinline__ float gelu_exact_grad(float v) {
    return 0.5f * (1.f + erff(v * 0.70710678118654752f)) + v * 0.3989422804014327f * expf(-0.5f * v * v);
}

}  // namespace o1d
