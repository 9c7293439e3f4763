// Host-callable interface of the walker kernels (o1d_walk.cuh), compiled in their own
// translation unit.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace o1d {

struct WalkConfig {
    int L, N, C, K, nchunks;
    int P, nbands, band_bytes, tile_bytes;
    int off_plane, off_wts, off_misc, plane_words;
    int smem_bytes, grid;
    int box_c, box_w, box_rows;     // TMA box: box_c channels x box_w pixels x box_rows rows x 1 image
    int line_only;                  // no slanted channel in the layer (rows, columns and diagonals only)
};

// Does the walker family take this request?  `chan` is the host copy of the plan's table of
// canonical line ids.  Fills *cfg when it does.
bool walk_configure(const int8_t *chan, int N, int H, int W, int C, int K, int stride, int layout, int esize,
                    int smem_per_block, int sms, WalkConfig *cfg);

// y = conv(x) + bias (flip = 1: input gradient of stride 1).  `in_map` / `out_map` are 4-D tensor maps
// of x and y with the box named in cfg; `chan` the device copy of the channel table; `err_flag` the
// device-side failure flag raised when a bounded wait runs out.
cudaError_t walk_launch_fprop(const WalkConfig &cfg, const CUtensorMap &in_map, const CUtensorMap &out_map,
                              const float *w, const float *bias, const int8_t *chan, int flip, int add_identity,
                              int *err_flag, cudaStream_t st);

}  // namespace o1d
