// Host side of the walker kernels: applicability, shared-memory layout, launch.
#include "o1d_walk.h"

#include "o1d_walk.cuh"

namespace o1d {

bool walk_configure(const int8_t *chan, int N, int H, int W, int C, int K, int stride, int layout, int esize,
                    int smem_per_block, int sms, WalkConfig *cfg) {
    if (!chan || stride != 1 || layout != O1D_NHWC || esize != 4 || K > kMaxTaps || (K & 1) == 0 || H != W ||
        C % walk::kCC != 0)
        return false;
    const int L = H;
    if (L != 28 && L != 56) return false;      // whole segments of kSeg columns, at most 32 row pairs
    cfg->line_only = 1;
    for (int c = 0; c < C; c++) {
        if (chan[c] < 0 || chan[c] > 7) return false;
        if (chan[c] & 1) cfg->line_only = 0;
    }
    const int P = L | 1;
    const int nbands = (L + walk::kBandRows - 1) / walk::kBandRows;
    if (nbands > walk::kMaxBands) return false;
    cfg->L = L; cfg->N = N; cfg->C = C; cfg->K = K; cfg->nchunks = C / walk::kCC;
    cfg->P = P; cfg->nbands = nbands;
    cfg->band_bytes = walk::kBandRows * P * walk::kCC * 4;
    cfg->tile_bytes = nbands * cfg->band_bytes;
    cfg->plane_words = L == 56 ? walk::Plane<56>::kWords : walk::Plane<28>::kWords;
    cfg->off_plane = 2 * cfg->tile_bytes;
    cfg->off_wts = (cfg->off_plane + cfg->plane_words * 4 + 15) & ~15;
    cfg->off_misc = cfg->off_wts + 2 * walk::kCC * 32 * 4;
    cfg->smem_bytes = cfg->off_misc + 64;
    if (cfg->smem_bytes > smem_per_block) return false;
    const long long items = (long long)N * cfg->nchunks;
    cfg->grid = (int)(items < sms ? items : sms);
    cfg->box_c = walk::kCC; cfg->box_w = P; cfg->box_rows = walk::kBandRows;
    return true;
}

cudaError_t walk_launch_fprop(const WalkConfig &cfg, const CUtensorMap &in_map, const CUtensorMap &out_map,
                              const float *w, const float *bias, const int8_t *chan, int flip, int add_identity,
                              int *err_flag, cudaStream_t st) {
    walk::WalkParams p{};
    p.N = cfg.N; p.L = cfg.L; p.C = cfg.C; p.K = cfg.K; p.nchunks = cfg.nchunks; p.total_items = cfg.N * cfg.nchunks;
    p.P = cfg.P; p.nbands = cfg.nbands; p.band_bytes = cfg.band_bytes; p.tile_bytes = cfg.tile_bytes;
    p.flip = flip; p.add_identity = add_identity;
    p.off_plane = cfg.off_plane; p.off_wts = cfg.off_wts; p.off_misc = cfg.off_misc;
    auto kern = cfg.L == 56 ? walk::walk_fprop_kernel<56, kHalf> : walk::walk_fprop_kernel<28, kHalf>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg.smem_bytes);
    if (e != cudaSuccess) return e;
    kern<<<cfg.grid, walk::kThreads, cfg.smem_bytes, st>>>(in_map, out_map, w, bias, chan, err_flag, p);
    return cudaGetLastError();
}

}  // namespace o1d
