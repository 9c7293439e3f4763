// Host side of the direct kernels: applicability, tile selection, TMA descriptor, launch.
#pragma once

#include "o1d_direct.cuh"
#include "o1d_tiled_host.cuh"   // encode_tiled_fn

namespace o1d {

struct ChunkRange { int chunk0, nchunks, reach_h, reach_w; };

struct DirectConfig {
    DirectParams p;
    int smem_bytes, grid, kt, npx;
    bool whole_image;      // one tile covers a whole image (no halo re-reads)
};

// Tile selection for an H x W map with halo (hh, hw) and `tap_bytes` of per-CTA tap tables.
// wgrad: also reserve room for the dy tiles and the end-of-kernel reduction scratch.
inline bool direct_configure_tiles(int N, int H, int W, int C, int K, int stride, int esize, int smem_limit, int sms,
                                   bool wgrad, int hh, int hw, int kt, int tap_bytes, const ChunkRange &rg,
                                   bool pair, DirectConfig *out) {
    const int CCs = 32 / esize;
    DirectParams p{};
    p.N = N; p.H = H; p.W = W; p.C = C; p.K = K; p.stride = stride;
    p.P = ceil_div(H, stride); p.Q = ceil_div(W, stride);
    p.CCs = CCs; p.nchunks = rg.nchunks; p.chunk0 = rg.chunk0;
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
        // the halvings overshoot: take back as many rows as still fit
        while (Th < p.P && (Th * stride + 1 + 2 * p.hh) <= 256 && tile_bytes(Th + 1, Tq, 1) <= kLarge) Th++;
        Th = ceil_div(p.P, ceil_div(p.P, Th));         // equal tiles, same count
        Tq = ceil_div(p.Q, ceil_div(p.Q, Tq));
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
    const int plw = pair ? 4 : 32 / CCs;      // pixel lanes per warp
    const int npx = (Tq >= 3 * plw) ? 4 : (Tq > plw ? 2 : 1);
    p.segs_q = ceil_div(Tq, plw * npx);
    p.off_taps_bytes = 2 * p.buf_stride;
    p.off_bar_bytes = p.off_taps_bytes + tap_bytes;
    int smem = p.off_bar_bytes + 16;
    const int red_bytes = (kDirectThreadsMax / 32) * CCs * kDirectPartialStride * 4;   // reuses the tile buffers
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

// Contiguous runs of channel chunks whose lines reach equally far (max |dh|, max |dw| over the
// chunk's channels).  A layer whose channels all mix orientations is one range; the models'
// block-wise angle assignment gives one range per orientation, and a range of horizontal lines
// needs no halo rows at all, which is what makes row tiles of large maps cheap.  Each range is
// its own launch with its own tile shape.

inline int direct_chunk_ranges(const PlanHeader &ph, const void *plan_host, int C, int K, int CCs, ChunkRange *out) {
    PlanView pv = plan_view(plan_host, ph);
    int8_t cls_h[1024], cls_w[1024];
    const int nchunks = C / CCs;
    if (ph.ncls > 1024) { out[0] = ChunkRange{0, nchunks, ph.max_dh, ph.max_dw}; return 1; }
    for (int i = 0; i < ph.ncls; i++) {
        int mh = 0, mw = 0;
        for (int k = 0; k < K; k++) {
            const int dh = pv.taps[((size_t)i * K + k) * 2], dw = pv.taps[((size_t)i * K + k) * 2 + 1];
            mh = mh > (dh < 0 ? -dh : dh) ? mh : (dh < 0 ? -dh : dh);
            mw = mw > (dw < 0 ? -dw : dw) ? mw : (dw < 0 ? -dw : dw);
        }
        cls_h[i] = (int8_t)mh; cls_w[i] = (int8_t)mw;
    }
    int n = 0;
    for (int ch = 0; ch < nchunks; ch++) {
        int mh = 0, mw = 0;
        for (int i = 0; i < CCs; i++) {
            const int c = pv.cls[ch * CCs + i];
            mh = mh > cls_h[c] ? mh : cls_h[c];
            mw = mw > cls_w[c] ? mw : cls_w[c];
        }
        if (n > 0 && out[n - 1].reach_h == mh && out[n - 1].reach_w == mw) { out[n - 1].nchunks++; continue; }
        if (n == kMaxChunkRanges) { out[0] = ChunkRange{0, nchunks, ph.max_dh, ph.max_dw}; return 1; }
        out[n++] = ChunkRange{ch, 1, mh, mw};
    }
    return n;
}

// Forward / weight gradient: halo = the lines' reach clipped to the image, KT = longest clipped tap list.
inline bool direct_configure(const PlanHeader &ph, const void *plan_host, const ChunkRange &rg, int N, int H, int W,
                             int C, int K, int stride, int layout, int esize, int smem_limit, int sms, bool wgrad,
                             bool pair, DirectConfig *out) {
    if (layout != O1D_NHWC || K > kMaxTaps || (stride != 1 && stride != 2)) return false;
    const int CCs = 32 / esize;
    if (C % CCs != 0) return false;
    const int hh = rg.reach_h < H - 1 ? rg.reach_h : H - 1;
    const int hw = rg.reach_w < W - 1 ? rg.reach_w : W - 1;
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
    return direct_configure_tiles(N, H, W, C, K, stride, esize, smem_limit, sms, wgrad, hh, hw, kt, CCs * kt * 8, rg, pair,
                                  out);
}

// Stride-2 input gradient: tiles of the dy grid (P x Q) with a halo of half the lines' reach.
// Not applicable when some class has more than kDgrad2Slots distinct taps of one parity.
inline bool direct_configure_dgrad2(const PlanHeader &ph, const void *plan_host, const ChunkRange &rg, int N, int H,
                                    int W, int C, int K, int layout, int esize, int smem_limit, int sms,
                                    DirectConfig *out) {
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
    const int hh = (rg.reach_h + 1) / 2, hw = (rg.reach_w + 1) / 2;
    const int tap_bytes = 4 * CCs * kDgrad2Slots * 8 + 4 * CCs * 4;
    if (!direct_configure_tiles(N, P, Q, C, K, 1, esize, smem_limit, sms, false, hh, hw, kDgrad2Slots, tap_bytes, rg, false,
                                out))
        return false;
    return true;
}

// 4-D tensor map over an NHWC tensor with a box CCs x TWp x THp x NI.
inline int make_direct_tensor_map(CUtensorMap *map, const void *base, int N, int H, int W, int C, int esize,
                                  const DirectParams &p) {
    const cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
    const cuuint64_t strides[3] = {(cuuint64_t)C * esize, (cuuint64_t)W * C * esize, (cuuint64_t)H * W * C * esize};
    const cuuint32_t box[4] = {(cuuint32_t)p.CCs, (cuuint32_t)p.TWp, (cuuint32_t)p.THp, (cuuint32_t)p.NI};
    return encode_map4(map, base, esize, dims, strides, box);
}

// 4-D tensor map over dy [N][P][Q][C] with a box CCs x Tq x Th x NI.
inline int make_direct_dy_tensor_map(CUtensorMap *map, const void *base, int N, int P, int Q, int C, int esize,
                                     const DirectParams &p) {
    const cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)Q, (cuuint64_t)P, (cuuint64_t)N};
    const cuuint64_t strides[3] = {(cuuint64_t)C * esize, (cuuint64_t)Q * C * esize, (cuuint64_t)P * Q * C * esize};
    const cuuint32_t box[4] = {(cuuint32_t)p.CCs, (cuuint32_t)p.Tq, (cuuint32_t)p.Th, (cuuint32_t)p.NI};
    return encode_map4(map, base, esize, dims, strides, box);
}

// The launches of one call: a single range over all chunks when one tile then holds a whole image
// (small maps: the halo is mostly cheap zero fill), else one range per run of chunks with equal
// reach.  All ranges run in one launch (DirectMulti), so they share the template parameters:
// the longest tap list, the smallest outputs-per-thread, the largest shared-memory need.
enum : int { DIRECT_FPROP = 0, DIRECT_WGRAD = 1, DIRECT_DGRAD2 = 2 };
struct DirectLaunchSet {
    int n;
    DirectConfig cfg[kMaxChunkRanges];
    int kt, npx, smem_bytes, grid, threads;
    bool whole_image;
    bool pair;                   // forward, 2-byte elements: every even/odd channel pair shares its line
    size_t partial_floats;       // weight gradient: floats of partial sums over all ranges
};
inline bool direct_plan_launches(const PlanHeader &ph, const void *plan_host, int N, int H, int W, int C, int K,
                                 int stride, int layout, int esize, int smem_limit, int sms, int mode,
                                 DirectLaunchSet *out) {
    if (layout != O1D_NHWC || K > kMaxTaps || C % (32 / esize) != 0) return false;
    bool pair = false;
    // measured with block-wise angles, bf16: 7x7 80 vs 88 us, 14x14 142 vs 153, 28x28 233 vs 270 at batch 256;
    // stride 2 loses 6 % (two weight sets leave registers for two outputs per thread only)
    if (mode == DIRECT_FPROP && esize == 2 && stride == 1) {
        PlanView pv = plan_view(plan_host, ph);
        pair = true;
        for (int c = 0; c + 1 < C && pair; c += 2) pair = pv.cls[c] == pv.cls[c + 1];
    }
    out->pair = pair;
    auto configure = [&](const ChunkRange &rg, DirectConfig *cfg) {
        return mode == DIRECT_DGRAD2
                   ? direct_configure_dgrad2(ph, plan_host, rg, N, H, W, C, K, layout, esize, smem_limit, sms, cfg)
                   : direct_configure(ph, plan_host, rg, N, H, W, C, K, stride, layout, esize, smem_limit, sms,
                                      mode == DIRECT_WGRAD, pair, cfg);
    };
    const ChunkRange all{0, C / (32 / esize), ph.max_dh, ph.max_dw};
    DirectConfig whole;
    const bool whole_ok = configure(all, &whole);
    out->n = 0;
    // One range over all chunks unless its tiles would read many times the pixels they produce
    // (long lines force row tiles with tall halos).  Measured: ranges take the 800x1280 stride-2
    // stem from 1706 to 974 us, but cost 30% where the common halo is small (K=15 stems), and the
    // stride-2 input gradient (half-size halo, empty parity classes skipped) never gains.
    if (whole_ok) {
        const DirectParams &wp = whole.p;
        const double amp = (double)wp.THp * wp.TWp / ((double)wp.Th * wp.Tq * stride * stride);
        if (whole.whole_image || mode == DIRECT_DGRAD2 || amp <= 4.0) { out->n = 1; out->cfg[0] = whole; }
    }
    if (!out->n) {
        ChunkRange rg[kMaxChunkRanges];
        const int n = direct_chunk_ranges(ph, plan_host, C, K, 32 / esize, rg);
        bool ok = true;
        for (int i = 0; i < n && ok; i++) ok = configure(rg[i], &out->cfg[i]);
        if (ok) out->n = n;
        else if (whole_ok) { out->n = 1; out->cfg[0] = whole; }
        else return false;
    }
    // common launch parameters; every range gets a share of the SMs in proportion to its chunks
    const int plw = (esize == 4 || pair) ? 4 : 2;
    const int total_chunks = C / (32 / esize);
    out->kt = 0; out->npx = 4; out->smem_bytes = 0; out->grid = 0; out->partial_floats = 0;
    out->whole_image = out->cfg[0].whole_image;
    for (int i = 0; i < out->n; i++) {
        if (out->cfg[i].kt > out->kt) out->kt = out->cfg[i].kt;
        if (out->cfg[i].npx < out->npx) out->npx = out->cfg[i].npx;
    }
    // two weight sets per thread: four outputs per thread would spill with the longest tap lists
    if (pair && out->npx == 4 && out->kt > 15) out->npx = 2;
    for (int i = 0; i < out->n; i++) {
        DirectConfig &c = out->cfg[i];
        if (mode != DIRECT_DGRAD2) {     // the tap tables are sized by the common KT
            c.p.off_bar_bytes = c.p.off_taps_bytes + c.p.CCs * out->kt * 8;
            const int red_bytes = (kDirectThreadsMax / 32) * c.p.CCs * kDirectPartialStride * 4;
            c.smem_bytes = c.p.off_bar_bytes + 16;
            if (mode == DIRECT_WGRAD && c.smem_bytes < red_bytes) c.smem_bytes = red_bytes;
        }
        if (c.smem_bytes > out->smem_bytes) out->smem_bytes = c.smem_bytes;
    }
    if (out->smem_bytes > smem_limit) return false;
    // one CTA per SM (large tiles): give it twice the warps
    // (measured: weight gradient 28x28x192 121 -> 115 us; the stride-2 input gradient loses, 449 -> 541 us)
    out->threads = ((228 * 1024) / (out->smem_bytes + 1024) >= 2 || mode == DIRECT_DGRAD2) ? kDirectThreads
                                                                                          : kDirectThreadsMax;
    for (int i = 0; i < out->n; i++) {
        DirectConfig &c = out->cfg[i];
        DirectParams &p = c.p;
        p.segs_q = ceil_div(p.Tq, plw * out->npx);
        p.div_sq = FastDiv::make(p.segs_q); p.div_thsq = FastDiv::make(p.Th * p.segs_q);
        if (out->n > 1) {      // the ranges run side by side: split the CTAs the device can hold
            int ctas = (228 * 1024) / (out->smem_bytes + 1024);
            if (ctas > 2) ctas = 2;
            if (ctas < 1) ctas = 1;
            int groups = (sms * ctas) / total_chunks;
            if (groups < 1) groups = 1;
            if (groups > p.tiles_per_chunk) groups = p.tiles_per_chunk;
            c.grid = groups * p.nchunks;
        }
        p.partial_off = (int)out->partial_floats;
        out->partial_floats += (size_t)c.grid * p.CCs * kDirectPartialStride;
        out->grid += c.grid;
    }
    return true;
}

// Kernel parameter block of a launch set (tensor maps are filled in by the caller).
inline void direct_fill_multi(const DirectLaunchSet &ls, DirectMulti *mp) {
    mp->n = ls.n;
    int at = 0;
    for (int i = 0; i < ls.n; i++) {
        mp->start[i] = at;
        mp->p[i] = ls.cfg[i].p;
        at += ls.cfg[i].grid;
    }
    for (int i = ls.n; i <= kMaxChunkRanges; i++) mp->start[i] = at;
}

template <typename T, int KT, int NPX, int STRIDE>
cudaError_t launch_direct_one(const DirectLaunchSet &ls, const DirectMulti &mp, const DirectMaps &maps, const float *w, const float *bias,
                              const PlanView &pv, void *y, cudaStream_t st) {
    auto kern = ls.n > 1 ? direct_fprop_nhwc_kernel<T, KT, NPX, STRIDE, true, false>
                         : direct_fprop_nhwc_kernel<T, KT, NPX, STRIDE, false, false>;
    if constexpr (sizeof(T) == 2) {
        if (ls.pair)
            kern = ls.n > 1 ? direct_fprop_nhwc_kernel<T, KT, NPX, STRIDE, true, true>
                            : direct_fprop_nhwc_kernel<T, KT, NPX, STRIDE, false, true>;
    }
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ls.smem_bytes);
    if (e != cudaSuccess) return e;
    kern<<<ls.grid, ls.threads, ls.smem_bytes, st>>>(mp, maps, w, bias, pv.cls, pv.taps, (T *)y);
    return cudaGetLastError();
}
template <typename T, int KT, int NPX, int STRIDE>
cudaError_t launch_direct_wgrad_one(const DirectLaunchSet &ls, const DirectMulti &mp, const DirectMaps &maps, const DirectMaps &dym,
                                    const PlanView &pv, float *partial, cudaStream_t st) {
    auto kern = ls.n > 1 ? direct_wgrad_nhwc_kernel<T, KT, NPX, STRIDE, true>
                         : direct_wgrad_nhwc_kernel<T, KT, NPX, STRIDE, false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ls.smem_bytes);
    if (e != cudaSuccess) return e;
    kern<<<ls.grid, ls.threads, ls.smem_bytes, st>>>(mp, maps, dym, pv.cls, pv.taps, partial);
    return cudaGetLastError();
}

// Dispatch over (taps kept in registers, outputs per thread, stride); F is a generic callable
// taking std::integral_constant<int, KT>, <NPX>, <STRIDE>.
template <typename F>
cudaError_t direct_dispatch(int kt, int npx, int stride, F &&f) {
    auto with_stride = [&](auto KT, auto NPX) {
        return stride == 1 ? f(KT, NPX, std::integral_constant<int, 1>{}) : f(KT, NPX, std::integral_constant<int, 2>{});
    };
    auto with_npx = [&](auto KT) {
        switch (npx) {
            case 4: return with_stride(KT, std::integral_constant<int, 4>{});
            case 2: return with_stride(KT, std::integral_constant<int, 2>{});
            default: return with_stride(KT, std::integral_constant<int, 1>{});
        }
    };
    switch (kt) {
        case 15: return with_npx(std::integral_constant<int, 15>{});
        case 23: return with_npx(std::integral_constant<int, 23>{});
        default: return with_npx(std::integral_constant<int, 31>{});
    }
}

template <typename T>
cudaError_t launch_direct(const DirectLaunchSet &ls, const DirectMulti &mp, const DirectMaps &maps, const float *w, const float *bias,
                          const PlanView &pv, void *y, cudaStream_t st) {
    return direct_dispatch(ls.kt, ls.npx, ls.cfg[0].p.stride, [&](auto KT, auto NPX, auto S) {
        return launch_direct_one<T, decltype(KT)::value, decltype(NPX)::value, decltype(S)::value>(ls, mp, maps, w, bias, pv, y, st);
    });
}
template <typename T>
cudaError_t launch_direct_wgrad(const DirectLaunchSet &ls, const DirectMulti &mp, const DirectMaps &maps, const DirectMaps &dym,
                                const PlanView &pv, float *partial, cudaStream_t st) {
    return direct_dispatch(ls.kt, ls.npx, ls.cfg[0].p.stride, [&](auto KT, auto NPX, auto S) {
        return launch_direct_wgrad_one<T, decltype(KT)::value, decltype(NPX)::value, decltype(S)::value>(ls, mp, maps, dym, pv, partial, st);
    });
}

template <typename T, int NPX>
cudaError_t launch_direct_dgrad2_one(const DirectLaunchSet &ls, const DirectMulti &mp, const DirectMaps &maps, const float *w,
                                     const PlanView &pv, void *dx, int Hx, int Wx, cudaStream_t st) {
    auto kern = ls.n > 1 ? direct_dgrad2_nhwc_kernel<T, NPX, true> : direct_dgrad2_nhwc_kernel<T, NPX, false>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ls.smem_bytes);
    if (e != cudaSuccess) return e;
    kern<<<ls.grid, ls.threads, ls.smem_bytes, st>>>(mp, maps, w, pv.cls, pv.taps, (T *)dx, Hx, Wx);
    return cudaGetLastError();
}
template <typename T>
cudaError_t launch_direct_dgrad2(const DirectLaunchSet &ls, const DirectMulti &mp, const DirectMaps &maps, const float *w, const PlanView &pv,
                                 void *dx, int Hx, int Wx, cudaStream_t st) {
    switch (ls.npx) {
        case 4: return launch_direct_dgrad2_one<T, 4>(ls, mp, maps, w, pv, dx, Hx, Wx, st);
        case 2: return launch_direct_dgrad2_one<T, 2>(ls, mp, maps, w, pv, dx, Hx, Wx, st);
        default: return launch_direct_dgrad2_one<T, 1>(ls, mp, maps, w, pv, dx, Hx, Wx, st);
    }
}

}  // namespace o1d
