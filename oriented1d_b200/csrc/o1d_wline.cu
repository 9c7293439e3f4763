// Host side of the whole-line kernels: applicability, shared-memory layout, launch.
#include "o1d_wline.h"

#include "o1d_wline.cuh"

namespace o1d {

namespace {

template <int L>
bool configure_side(const int8_t *chan, int N, int C, int K, int smem_per_sm, int smem_per_block, int sms,
                    WlConfig *cfg) {
    using G = wl::Geo<L>;
    const int nchunks = C / wl::kCC;
    int off = 0;
    for (int c0 = 0; c0 < C; c0 += wl::kCC) {
        int kind[wl::kCC];
        for (int j = 0; j < wl::kCC; j++) {
            const int o = chan[c0 + j];
            if (o < 0 || o > 7) return false;
            kind[j] = canon_kind(o);
        }
        bool ok = true;
        const int need = wl::chunk_plane_floats<L>(kind, &ok);
        if (!ok) return false;                 // slanted channels are evaluated in pairs
        if (need > off) off = need;
    }
    cfg->plane_floats = off;
    cfg->off_wts = (off + 3) & ~3;
    const int fixed = (((cfg->off_wts + wl::kCC * 32 + wl::kMapInts + wl::kMaxStages) * 4) + 127) & ~127;
    // two CTAs per SM when they fit with at least two stages; the ring grows into what is left
    int ctas = 0, nstg = 0;
    for (int t = 2; t >= 1 && !ctas; t--) {
        int budget = smem_per_sm / t - 1024;
        if (budget > smem_per_block) budget = smem_per_block;
        const int fit = (budget - fixed - 8 * wl::kMaxStages) / G::kStageBytes;
        if (fit >= 2) { ctas = t; nstg = fit < wl::kMaxStages ? fit : wl::kMaxStages; }
    }
    if (!ctas) return false;
    if (nstg > G::NB) nstg = G::NB;
    cfg->L = L; cfg->N = N; cfg->C = C; cfg->K = K; cfg->nchunks = nchunks;
    cfg->off_stage_bytes = fixed;
    cfg->nstg = nstg;
    cfg->off_bar_bytes = fixed + nstg * G::kStageBytes;
    cfg->smem_bytes = cfg->off_bar_bytes + 8 * wl::kMaxStages;
    cfg->ctas_per_sm = ctas;
    const long long items = (long long)N * nchunks;
    cfg->grid = (int)(items < (long long)sms * ctas ? items : (long long)sms * ctas);
    cfg->box_c = wl::kCC;
    cfg->box_rows = wl::kBR;
    return true;
}

template <int L>
cudaError_t launch_side(const WlConfig &cfg, const CUtensorMap &map, const float *w, const float *bias,
                        const int8_t *chan, float *y, int flip, int add_identity, int *err_flag, cudaStream_t st) {
    wl::WlParams p{};
    p.N = cfg.N; p.C = cfg.C; p.K = cfg.K; p.nchunks = cfg.nchunks; p.total_items = cfg.N * cfg.nchunks;
    p.flip = flip; p.add_identity = add_identity;
    p.plane_floats = cfg.plane_floats; p.off_wts = cfg.off_wts;
    p.off_stage_bytes = cfg.off_stage_bytes; p.nstg = cfg.nstg; p.off_bar_bytes = cfg.off_bar_bytes;
    p.step_n = cfg.grid / cfg.nchunks; p.step_chunk = cfg.grid % cfg.nchunks;
    auto kern = wl::wline_fprop_kernel<L, kHalf>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg.smem_bytes);
    if (e != cudaSuccess) return e;
    kern<<<cfg.grid, wl::kThreads, cfg.smem_bytes, st>>>(map, w, bias, chan, y, err_flag, p);
    return cudaGetLastError();
}

}  // namespace

bool wline_configure(const int8_t *chan, int N, int H, int W, int C, int K, int stride, int layout, int esize,
                     int smem_per_sm, int smem_per_block, int sms, WlConfig *cfg) {
    if (!chan || stride != 1 || layout != O1D_NHWC || esize != 4 || K > kMaxTaps || H != W || C % wl::kCC != 0)
        return false;
    switch (H) {
        case 56: return configure_side<56>(chan, N, C, K, smem_per_sm, smem_per_block, sms, cfg);
        default: return false;
    }
}

cudaError_t wline_launch_fprop(const WlConfig &cfg, const CUtensorMap &map, const float *w, const float *bias,
                               const int8_t *chan, float *y, int flip, int add_identity, int *err_flag,
                               cudaStream_t st) {
    switch (cfg.L) {
        case 56: return launch_side<56>(cfg, map, w, bias, chan, y, flip, add_identity, err_flag, st);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace o1d
