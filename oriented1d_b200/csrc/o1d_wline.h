// Host-callable interface of the whole-line kernels (o1d_wline.cuh), compiled in their own
// translation unit.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace o1d {

struct WlConfig {
    int L;                       // side of the square map
    int N, C, K, nchunks;
    int plane_floats, off_wts, off_stage_bytes, off_bar_bytes, nstg;
    int smem_bytes, grid, ctas_per_sm;
    int box_c, box_rows;         // TMA box: box_c channels x L pixels x box_rows rows x 1 image
};

// Does the whole-line family take this request?  `chan` holds the canonical line id of every
// channel (host copy of the plan's table).  Fills *cfg when it does.
bool wline_configure(const int8_t *chan, int N, int H, int W, int C, int K, int stride, int layout, int esize,
                     int smem_per_sm, int smem_per_block, int sms, WlConfig *cfg);

// y = conv(x) + bias (flip = 1: input gradient of stride 1).  `map` is the 4-D tensor map of x with
// the box named in cfg; `chan` the device copy of the channel table; `err_flag` the device-side
// failure flag raised when a bounded TMA wait runs out.
cudaError_t wline_launch_fprop(const WlConfig &cfg, const CUtensorMap &map, const float *w, const float *bias,
                               const int8_t *chan, float *y, int flip, int add_identity, int *err_flag,
                               cudaStream_t st);

}  // namespace o1d
