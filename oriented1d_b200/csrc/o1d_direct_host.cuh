// Host side of the direct kernels: applicability, tile selection, TMA descriptor, launch.
#pragma once

#include "o1d_direct.cuh"
#include "o1d_tiled_host.cuh"   // encode_tiled_fn

namespace o1d {

struct DirectConfig {
    DirectParams p;
    int smem_bytes, grid, kt, npx;
    bool whole_image;      // one tile covers a whole image (no halo re-reads)
};

// Tile selection for an H x W map with halo (hh, hw) and `tap_bytes` of per-CTA tap tables.
// wgrad: also reserve room for the dy tiles and the end-of-kernel reduction scratch.
inline bool direct_configure_tiles(int N, int H, int W, int C, int K, int stride, int esize, int smem_limit, int sms,
                                   bool wgrad, int hh, int hw, int kt, int tap_bytes, DirectConfig *out) {
    const int CCs = 32 / esize;
    DirectParams p{};
    p.N = N; p.H = H; p.W = W; p.C = C; p.K = K; p.stride = stride;
    p.P = ceil_div(H, stride); p.Q = ceil_div(W, stride);
    p.CCs = CCs; p.nchunks = C / CCs;
    p.hh = hh; p.hw = hw;
    auto tile_bytes = [&](int th, int tq, int ni) {
        return (long long)((th - 1) * stride + 1 + 2 * p.hh) * ((tq - 1) * stride + 1 + 2 * p.hw) * CCs * esize * ni;
    };
    const long long kSmall = 40 * 1024, kLarge = (wgrad ? 84 : 100) * 1024;
    int Th = p.P, Tq = p.Q, NI = 1;
    bool whole = true;
    if ((Tq - 1) * stride + 1 + 2 * p.hw > 256 || (Th - 1) * stride + 1 + 2 * p.hh > 256 || tile_bytes(Th, Tq, 1) > kLarge) {
        whole = false;
        while ((Tq - 1) * stride + 1 + 2 * p.hw > 256) Tq = (Tq + 1) / 2;
        // rows: as many as fit the large budget (at least as many output rows as halo rows,
        // so that re-read rows stay below ~2x)
        while (Th > 1 && ((Th - 1) * stride + 1 + 2 * p.hh > 256 || tile_bytes(Th, Tq, 1) > kLarge)) Th = (Th + 1) / 2;
        if (tile_bytes(Th, Tq, 1) > kLarge) {          // still too wide: split columns further
            while (Tq > 8 && tile_bytes(Th, Tq, 1) > kLarge) Tq = (Tq + 1) / 2;
            if (tile_bytes(Th, Tq, 1) > kLarge) return false;
        }
    } else {
        NI = (int)(kSmall / tile_bytes(Th, Tq, 1));
    }
    if (NI < 1) NI = 1;
    if (NI > 16) NI = 16;
    if (NI > N) NI = N;
    p.Th = Th; p.Tq = Tq; p.NI = NI;
    p.THp = (Th - 1) * stride + 1 + 2 * p.hh;
    p.TWp = (Tq - 1) * stride + 1 + 2 * p.hw;
    p.tiles_p = ceil_div(p.P, Th); p.tiles_q = ceil_div(p.Q, Tq); p.tiles_n = ceil_div(N, NI);
    p.tiles_per_chunk = p.tiles_p * p.tiles_q * p.tiles_n;
    p.tile_bytes = p.THp * p.TWp * CCs * esize * NI;
    // slack after each buffer: the last row segment of a tile may read up to 16 pixels past it
    p.tile_stride = ((p.tile_bytes + 127) & ~127) + 16 * stride * CCs * esize;
    p.dy_bytes = wgrad ? Th * Tq * CCs * esize * NI : 0;
    p.buf_stride = p.tile_stride + (wgrad ? ((p.dy_bytes + 127) & ~127) + 16 * CCs * esize : 0);
    const int plw = 32 / CCs;
    const int npx = (Tq >= 3 * plw) ? 4 : (Tq > plw ? 2 : 1);
    p.segs_q = ceil_div(Tq, plw * npx);
    p.off_taps_bytes = 2 * p.buf_stride;
    p.off_bar_bytes = p.off_taps_bytes + tap_bytes;
    int smem = p.off_bar_bytes + 16;
    const int red_bytes = (kDirectThreads / 32) * CCs * kDirectPartialStride * 4;   // reuses the tile buffers
    if (wgrad && smem < red_bytes) smem = red_bytes;
    if (smem > smem_limit) return false;
    int ctas = (228 * 1024) / (smem + 1024);
    if (ctas > 2) ctas = 2;
    if (ctas < 1) ctas = 1;
    int groups = (sms * ctas) / p.nchunks;
    if (groups < 1) groups = 1;
    if (groups > p.tiles_per_chunk) groups = p.tiles_per_chunk;
    p.div_sq = FastDiv::make(p.segs_q); p.div_thsq = FastDiv::make(Th * p.segs_q);
    p.div_tiles_q = FastDiv::make(p.tiles_q); p.div_tiles_pq = FastDiv::make(p.tiles_p * p.tiles_q);
    out->p = p;
    out->smem_bytes = smem;
    out->grid = groups * p.nchunks;
    out->kt = kt;
    out->npx = npx;
    out->whole_image = whole;
    return true;
}

// Forward / weight gradient: halo = the lines' reach clipped to the image, KT = longest clipped tap list.
inline bool direct_configure(const PlanHeader &ph, const void *plan_host, int N, int H, int W, int C, int K,
                             int stride, int layout, int esize, int smem_limit, int sms, bool wgrad,
                             DirectConfig *out) {
    if (layout != O1D_NHWC || K > kMaxTaps || (stride != 1 && stride != 2)) return false;
    const int CCs = 32 / esize;
    if (C % CCs != 0) return false;
    const int hh = ph.max_dh < H - 1 ? ph.max_dh : H - 1;
    const int hw = ph.max_dw < W - 1 ? ph.max_dw : W - 1;
    // longest tap list after dropping taps that cannot reach the image
    PlanView pv = plan_view(plan_host, ph);
    int longest = 0;
    for (int i = 0; i < ph.ncls; i++) {
        int n = 0;
        for (int k = 0; k < K; k++) {
            const int dh = pv.taps[((size_t)i * K + k) * 2], dw = pv.taps[((size_t)i * K + k) * 2 + 1];
            if ((dh < 0 ? -dh : dh) <= hh && (dw < 0 ? -dw : dw) <= hw) n++;
        }
        if (n > longest) longest = n;
    }
    const int kt = longest <= 15 ? 15 : longest <= 23 ? 23 : 31;
    return direct_configure_tiles(N, H, W, C, K, stride, esize, smem_limit, sms, wgrad, hh, hw, kt, CCs * kt * 8, out);
}

// Stride-2 input gradient: tiles of the dy grid (P x Q) with a halo of half the lines' reach.
// Not applicable when some class has more than kDgrad2Slots distinct taps of one parity.
inline bool direct_configure_dgrad2(const PlanHeader &ph, const void *plan_host, int N, int H, int W, int C, int K,
                                    int layout, int esize, int smem_limit, int sms, DirectConfig *out) {
    if (layout != O1D_NHWC || K > kMaxTaps) return false;
    const int CCs = 32 / esize;
    if (C % CCs != 0) return false;
    PlanView pv = plan_view(plan_host, ph);
    for (int i = 0; i < ph.ncls; i++) {
        int n[4] = {0, 0, 0, 0};
        int seen[4][kMaxTaps];
        for (int k = 0; k < K; k++) {
            const int dh = pv.taps[((size_t)i * K + k) * 2], dw = pv.taps[((size_t)i * K + k) * 2 + 1];
            const int q = (dh & 1) * 2 + (dw & 1), key = dh * 64 + dw;
            bool dup = false;
            for (int j = 0; j < n[q]; j++) dup = dup || seen[q][j] == key;
            if (!dup) seen[q][n[q]++] = key;
        }
        for (int q = 0; q < 4; q++) if (n[q] > kDgrad2Slots) return false;
    }
    const int P = ceil_div(H, 2), Q = ceil_div(W, 2);
    const int hh = (ph.max_dh + 1) / 2, hw = (ph.max_dw + 1) / 2;
    const int tap_bytes = 4 * CCs * kDgrad2Slots * 8 + 4 * CCs * 4;
    if (!direct_configure_tiles(N, P, Q, C, K, 1, esize, smem_limit, sms, false, hh, hw, kDgrad2Slots, tap_bytes, out))
        return false;
    return true;
}

// 4-D tensor map over an NHWC tensor with a box CCs x TWp x THp x NI.
inline bool make_direct_tensor_map(CUtensorMap *map, const void *base, int N, int H, int W, int C, int esize,
                                   const DirectParams &p) {
    PFN_encodeTiled enc = encode_tiled_fn();
    if (!enc || ((uintptr_t)base & 15) || (C * esize) % 16 != 0) return false;
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
    cuuint64_t strides[3] = {(cuuint64_t)C * esize, (cuuint64_t)W * C * esize, (cuuint64_t)H * W * C * esize};
    cuuint32_t box[4] = {(cuuint32_t)p.CCs, (cuuint32_t)p.TWp, (cuuint32_t)p.THp, (cuuint32_t)p.NI};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return enc(map, esize == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
               const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 4-D tensor map over dy [N][P][Q][C] with a box CCs x Tq x Th x NI.
inline bool make_direct_dy_tensor_map(CUtensorMap *map, const void *base, int N, int P, int Q, int C, int esize,
                                      const DirectParams &p) {
    PFN_encodeTiled enc = encode_tiled_fn();
    if (!enc || ((uintptr_t)base & 15) || (C * esize) % 16 != 0) return false;
    cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)Q, (cuuint64_t)P, (cuuint64_t)N};
    cuuint64_t strides[3] = {(cuuint64_t)C * esize, (cuuint64_t)Q * C * esize, (cuuint64_t)P * Q * C * esize};
    cuuint32_t box[4] = {(cuuint32_t)p.CCs, (cuuint32_t)p.Tq, (cuuint32_t)p.Th, (cuuint32_t)p.NI};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    return enc(map, esize == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
               const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
               CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T, int KT, int NPX, int STRIDE>
cudaError_t launch_direct_wgrad_one(const DirectConfig &cfg, const CUtensorMap &mx, const CUtensorMap &mdy,
                                    const PlanView &pv, float *partial, cudaStream_t st) {
    auto kern = direct_wgrad_nhwc_kernel<T, KT, NPX, STRIDE>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg.smem_bytes);
    if (e != cudaSuccess) return e;
    kern<<<cfg.grid, kDirectThreads, cfg.smem_bytes, st>>>(mx, mdy, pv.cls, pv.taps, partial, cfg.p);
    return cudaGetLastError();
}
template <typename T, int KT, int STRIDE>
cudaError_t launch_direct_wgrad_npx(const DirectConfig &cfg, const CUtensorMap &mx, const CUtensorMap &mdy,
                                    const PlanView &pv, float *partial, cudaStream_t st) {
    switch (cfg.npx) {
        case 4: return launch_direct_wgrad_one<T, KT, 4, STRIDE>(cfg, mx, mdy, pv, partial, st);
        case 2: return launch_direct_wgrad_one<T, KT, 2, STRIDE>(cfg, mx, mdy, pv, partial, st);
        default: return launch_direct_wgrad_one<T, KT, 1, STRIDE>(cfg, mx, mdy, pv, partial, st);
    }
}
template <typename T, int STRIDE>
cudaError_t launch_direct_wgrad_kt(const DirectConfig &cfg, const CUtensorMap &mx, const CUtensorMap &mdy,
                                   const PlanView &pv, float *partial, cudaStream_t st) {
    switch (cfg.kt) {
        case 15: return launch_direct_wgrad_npx<T, 15, STRIDE>(cfg, mx, mdy, pv, partial, st);
        case 23: return launch_direct_wgrad_npx<T, 23, STRIDE>(cfg, mx, mdy, pv, partial, st);
        default: return launch_direct_wgrad_npx<T, 31, STRIDE>(cfg, mx, mdy, pv, partial, st);
    }
}
template <typename T>
cudaError_t launch_direct_wgrad(const DirectConfig &cfg, const CUtensorMap &mx, const CUtensorMap &mdy,
                                const PlanView &pv, float *partial, cudaStream_t st) {
    return cfg.p.stride == 1 ? launch_direct_wgrad_kt<T, 1>(cfg, mx, mdy, pv, partial, st)
                             : launch_direct_wgrad_kt<T, 2>(cfg, mx, mdy, pv, partial, st);
}

template <typename T, int NPX>
cudaError_t launch_direct_dgrad2_one(const DirectConfig &cfg, const CUtensorMap &map, const float *w, const PlanView &pv,
                                     void *dx, int Hx, int Wx, cudaStream_t st) {
    auto kern = direct_dgrad2_nhwc_kernel<T, NPX>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg.smem_bytes);
    if (e != cudaSuccess) return e;
    kern<<<cfg.grid, kDirectThreads, cfg.smem_bytes, st>>>(map, w, pv.cls, pv.taps, (T *)dx, Hx, Wx, cfg.p);
    return cudaGetLastError();
}
template <typename T>
cudaError_t launch_direct_dgrad2(const DirectConfig &cfg, const CUtensorMap &map, const float *w, const PlanView &pv,
                                 void *dx, int Hx, int Wx, cudaStream_t st) {
    switch (cfg.npx) {
        case 4: return launch_direct_dgrad2_one<T, 4>(cfg, map, w, pv, dx, Hx, Wx, st);
        case 2: return launch_direct_dgrad2_one<T, 2>(cfg, map, w, pv, dx, Hx, Wx, st);
        default: return launch_direct_dgrad2_one<T, 1>(cfg, map, w, pv, dx, Hx, Wx, st);
    }
}

template <typename T, int KT, int NPX, int STRIDE>
cudaError_t launch_direct_one(const DirectConfig &cfg, const CUtensorMap &map, const float *w, const float *bias,
                              const PlanView &pv, void *y, cudaStream_t st) {
    auto kern = direct_fprop_nhwc_kernel<T, KT, NPX, STRIDE>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg.smem_bytes);
    if (e != cudaSuccess) return e;
    kern<<<cfg.grid, kDirectThreads, cfg.smem_bytes, st>>>(map, w, bias, pv.cls, pv.taps, (T *)y, cfg.p);
    return cudaGetLastError();
}

template <typename T, int KT, int STRIDE>
cudaError_t launch_direct_npx(const DirectConfig &cfg, const CUtensorMap &map, const float *w, const float *bias,
                              const PlanView &pv, void *y, cudaStream_t st) {
    switch (cfg.npx) {
        case 4: return launch_direct_one<T, KT, 4, STRIDE>(cfg, map, w, bias, pv, y, st);
        case 2: return launch_direct_one<T, KT, 2, STRIDE>(cfg, map, w, bias, pv, y, st);
        default: return launch_direct_one<T, KT, 1, STRIDE>(cfg, map, w, bias, pv, y, st);
    }
}

template <typename T, int STRIDE>
cudaError_t launch_direct_kt(const DirectConfig &cfg, const CUtensorMap &map, const float *w, const float *bias,
                             const PlanView &pv, void *y, cudaStream_t st) {
    switch (cfg.kt) {
        case 15: return launch_direct_npx<T, 15, STRIDE>(cfg, map, w, bias, pv, y, st);
        case 23: return launch_direct_npx<T, 23, STRIDE>(cfg, map, w, bias, pv, y, st);
        default: return launch_direct_npx<T, 31, STRIDE>(cfg, map, w, bias, pv, y, st);
    }
}

template <typename T>
cudaError_t launch_direct(const DirectConfig &cfg, const CUtensorMap &map, const float *w, const float *bias,
                          const PlanView &pv, void *y, cudaStream_t st) {
    return cfg.p.stride == 1 ? launch_direct_kt<T, 1>(cfg, map, w, bias, pv, y, st)
                             : launch_direct_kt<T, 2>(cfg, map, w, bias, pv, y, st);
}

}  // namespace o1d
