// C ABI of libo1d (see include/o1d.h): argument checks, plan building, kernel selection,
// launches.  No allocation, no synchronisation, no global mutable state besides a
// per-device attribute cache and a thread-local error string.
#include <math.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <vector>

#include "o1d_common.cuh"
#include "o1d_generic.cuh"
#include "o1d_tiled_host.cuh"
#include "o1d_direct_host.cuh"
#include "o1d_small.cuh"
#include "o1d_layernorm.cuh"
#include "o1d_transpose.cuh"
#include "o1d_pointwise.cuh"
#include "o1d_wline.h"
#include "o1d_walk.h"

using namespace o1d;

namespace {

thread_local char g_err[256] = "";
thread_local int g_last_route = O1D_ROUTE_NONE;   // kernel family of this thread's last operator call
int g_force_generic = 0;   // o1d_set_route(): 1 = general kernels only (testing aid)
int g_prefer = 0;          // o1d_set_route(): 2 = prefer the tiled kernels, 3 = direct, 4 = whole-line, 5 = walker

int cuda_fail(cudaError_t e, const char *what) {
    snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
    return O1D_ERR_CUDA;
}
// A tensor map the driver refused although the request passed every documented check.
int map_fail(const char *what) {
    snprintf(g_err, sizeof(g_err), "%s: cuTensorMapEncodeTiled failed (CUresult %d)", what, last_encode_result());
    return O1D_ERR_CUDA;
}
// `expr` yields MAP_OK / MAP_NA / MAP_FAIL.
#define O1D_MAP(expr, what)                         \
    do {                                            \
        const int m_ = (expr);                      \
        if (m_ == MAP_NA) return kNotTiled;         \
        if (m_ == MAP_FAIL) return map_fail(what);  \
    } while (0)

#define O1D_CUDA(call)                                              \
    do {                                                            \
        cudaError_t e_ = (call);                                    \
        if (e_ != cudaSuccess) return cuda_fail(e_, #call);         \
    } while (0)

constexpr int kNotTiled = -1;          // "this kernel family does not take the request"

struct DeviceInfo { int sms; int smem_optin; };

// Attributes of the current device, queried once per device.
int device_info(DeviceInfo *out) {
    static std::atomic<uint64_t> cache[64];      // (sms << 32) | smem_optin; 0 = not yet queried
    int dev = 0;
    O1D_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return O1D_ERR_UNSUPPORTED;
    uint64_t v = cache[dev].load(std::memory_order_acquire);
    if (!v) {
        int sms = 0, smem = 0;
        O1D_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        O1D_CUDA(cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        v = ((uint64_t)(uint32_t)sms << 32) | (uint32_t)smem;
        cache[dev].store(v, std::memory_order_release);
    }
    out->sms = (int)(v >> 32);
    out->smem_optin = (int)(v & 0xffffffffu);
    return O1D_OK;
}

bool bad_common(int N, int H, int W, int C, int K, int stride, int layout, int dtype) {
    return N <= 0 || H <= 0 || W <= 0 || C <= 0 || K <= 0 || (K & 1) == 0 || K > 255 || stride <= 0 ||
           (layout != O1D_NCHW && layout != O1D_NHWC) || (dtype != O1D_F32 && dtype != O1D_BF16);
}

int check_plan(const void *plan_host, int C, int K, PlanHeader *h) {
    if (!plan_host) return O1D_ERR_INVALID;
    memcpy(h, plan_host, sizeof(PlanHeader));
    if (h->magic != kPlanMagic || h->C != C || h->K != K || h->ncls <= 0 || h->ncls > C) return O1D_ERR_PLAN;
    return O1D_OK;
}

// The reference's rasterisation, kernels.cpp:37,43-44.
void raster(float theta, int K, int8_t *dh, int8_t *dw) {
    const int pad = K / 2;
    const float sin_ = sinf(theta), cos_ = cosf(theta);
    for (int k = 0; k < K; k++) {
        dh[k] = (int8_t)(int)(-sin_ * (k - pad));
        dw[k] = (int8_t)(int)(cos_ * (k - pad));
    }
}

int grid_for(int64_t total, int threads, const DeviceInfo &d, int waves) {
    int64_t blocks = (total + threads - 1) / threads;
    int64_t cap = (int64_t)d.sms * waves;
    return (int)(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

// ---- generic launches --------------------------------------------------------------

template <typename T, int LAYOUT>
int launch_generic_fprop(const void *x, const float *w, const float *bias, const PlanHeader &ph,
                         const void *plan_dev, void *y, int N, int H, int W, int C, int K, int stride,
                         int add_identity, int act, cudaStream_t st, const DeviceInfo &d) {
    const int P = ceil_div(H, stride), Q = ceil_div(W, stride);
    PlanView pv = plan_view(plan_dev, ph);
    // NHWC with class-uniform channel vectors: 128-bit loads per tap
    constexpr int VE = 16 / (int)sizeof(T);
    const bool uniform = (VE == 4) ? ph.uniform4 != 0 : ph.uniform8 != 0;
    if (LAYOUT == O1D_NHWC && uniform && ((uintptr_t)x & 15) == 0 && ((uintptr_t)y & 15) == 0) {
        const int tapb = (ph.ncls * K * 2 + 15) & ~15;
        const int wb = C * K * 4;
        if (tapb <= kTapSmemBudget) {
            const int w_staged = (tapb + wb <= 96 * 1024);
            const int smem = tapb + (w_staged ? wb : 0);
            auto kern = generic_fprop_nhwc_vec_kernel<T>;
            if (smem > 48 * 1024) O1D_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
            const int grid = grid_for((int64_t)N * P * Q * (C / VE), kGenericThreads, d, 8);
            kern<<<grid, kGenericThreads, smem, st>>>((const T *)x, w, bias, pv.cls, pv.taps, ph.ncls, w_staged,
                                                       (T *)y, N, H, W, C, K, stride, P, Q, add_identity, act);
            O1D_CUDA(cudaGetLastError());
            g_last_route = O1D_ROUTE_GENERAL;
            return O1D_OK;
        }
    }
    const int tap_bytes = ph.ncls * K * 2;
    const int staged = tap_bytes <= kTapSmemBudget;
    const int grid = grid_for((int64_t)N * P * Q * C, kGenericThreads, d, 16);
    generic_fprop_kernel<T, LAYOUT><<<grid, kGenericThreads, staged ? tap_bytes : 0, st>>>(
        (const T *)x, w, bias, pv.cls, pv.taps, ph.ncls, staged, (T *)y, N, H, W, C, K, stride, P, Q,
        add_identity, act);
    O1D_CUDA(cudaGetLastError());
    g_last_route = O1D_ROUTE_GENERAL;
    return O1D_OK;
}

template <typename T, int LAYOUT>
int launch_generic_dgrad(const void *dy, const float *w, const PlanHeader &ph, const void *plan_dev,
                         void *dx, int N, int H, int W, int C, int K, int stride, int add_identity,
                         const void *pre, cudaStream_t st, const DeviceInfo &d) {
    const int P = ceil_div(H, stride), Q = ceil_div(W, stride);
    PlanView pv = plan_view(plan_dev, ph);
    const int tap_bytes = ph.ncls * K * 2;
    const int staged = tap_bytes <= kTapSmemBudget;
    const int grid = grid_for((int64_t)N * H * W * C, kGenericThreads, d, 16);
    generic_dgrad_kernel<T, LAYOUT><<<grid, kGenericThreads, staged ? tap_bytes : 0, st>>>(
        (const T *)dy, w, pv.cls, pv.taps, ph.ncls, staged, (T *)dx, N, H, W, C, K, stride, P, Q,
        add_identity, (const T *)pre);
    O1D_CUDA(cudaGetLastError());
    g_last_route = O1D_ROUTE_GENERAL;
    return O1D_OK;
}

// Number of output slices of the general weight-gradient: enough blocks for ~4 per SM,
// never fewer than 64 outputs per slice.  Depends on the shape only (B200 has 148 SMs),
// so the summation order — and the result, bit for bit — is reproducible.
int generic_wgrad_slices(int N, int P, int Q, int C, int layout) {
    const int cl = layout == O1D_NHWC ? 32 : 1;
    const int chunks = ceil_div(C, cl);
    const int64_t npq = (int64_t)N * P * Q;
    int64_t s = (4 * 148 + chunks - 1) / chunks;
    const int64_t cap = (npq + 63) / 64;
    if (s > cap) s = cap;
    if (s < 1) s = 1;
    return (int)s;
}

template <typename T, int LAYOUT>
int launch_generic_wgrad(const void *dy, const void *x, const PlanHeader &ph, const void *plan_dev,
                         float *dw, float *db, float *partial, int N, int H, int W, int C, int K,
                         int stride, int act, cudaStream_t st) {
    const int P = ceil_div(H, stride), Q = ceil_div(W, stride);
    PlanView pv = plan_view(plan_dev, ph);
    const int slices = generic_wgrad_slices(N, P, Q, C, LAYOUT);
    dim3 grid(ceil_div(C, WgradShape<LAYOUT>::CL), slices);
    generic_wgrad_partial_kernel<T, LAYOUT><<<grid, kGenericThreads, 0, st>>>(
        (const T *)dy, (const T *)x, pv.cls, pv.taps, partial, N, H, W, C, K, stride, P, Q, slices, act);
    O1D_CUDA(cudaGetLastError());
    const int tot = C * (K + 1);
    wgrad_final_kernel<<<ceil_div(tot, 256), 256, 0, st>>>(partial, dw, db, C, K, slices);
    O1D_CUDA(cudaGetLastError());
    g_last_route = O1D_ROUTE_GENERAL;
    return O1D_OK;
}

constexpr int kMaxTiledCtas = 256;   // upper bound on SMs (grid of the persistent kernels)

// Forward / stride-1 input gradient through the tiled kernels; kNotTiled when they do not apply.
int try_tiled(const void *x, const float *w, const float *bias, const PlanHeader &ph, const void *plan_host,
              const void *plan_dev, void *y, int N, int H, int W, int C, int K, int stride, int layout, int dtype,
              int add_identity, int flip, int act, const void *pre, cudaStream_t st, const DeviceInfo &d) {
    if (g_force_generic) return kNotTiled;
    const int esize = dtype == O1D_F32 ? 4 : 2;
    TiledConfig cfg;
    if (!tiled_configure(ph, plan_host, N, H, W, C, K, stride, layout, esize, d.smem_optin, d.sms, OP_FPROP, &cfg))
        return kNotTiled;
    if (((uintptr_t)y & 15) != 0 || ((uintptr_t)pre & 15) != 0) return kNotTiled;
    if ((act || pre) && !tiled_supports_act(cfg)) return kNotTiled;
    CUtensorMap map;
    O1D_MAP(make_nhwc_tensor_map(&map, x, N, H, W, C, esize, cfg.p.CC, cfg.p.BR), "tiled fprop");
    cfg.p.flip = flip;
    cfg.p.add_identity = add_identity;
    cfg.p.act = act;
    PlanView pv = plan_view(plan_dev, ph);
    cudaError_t e = launch_tiled<OP_FPROP>(cfg, dtype, map, w, bias, pv, y, nullptr, pre, st);
    if (e != cudaSuccess) return cuda_fail(e, "tiled fprop launch");
    g_last_route = O1D_ROUTE_TILED;
    return O1D_OK;
}

// Forward / stride-1 input gradient through the direct kernels; kNotTiled when they do not apply.
int try_direct(const void *x, const float *w, const float *bias, const PlanHeader &ph, const void *plan_host,
               const void *plan_dev, void *y, int N, int H, int W, int C, int K, int stride, int layout, int dtype,
               int add_identity, int flip, cudaStream_t st, const DeviceInfo &d, bool whole_image_only) {
    if (g_force_generic) return kNotTiled;
    const int esize = dtype == O1D_F32 ? 4 : 2;
    DirectLaunchSet ls;
    if (!direct_plan_launches(ph, plan_host, N, H, W, C, K, stride, layout, esize, d.smem_optin, d.sms, DIRECT_FPROP, &ls))
        return kNotTiled;
    if (whole_image_only && !ls.whole_image) return kNotTiled;
    // measured against the tiled kernels the direct ones only win while several images share a
    // tile (7x7: 34 vs 37 us fp32, 39 vs 41 bf16; 14x14: 68 vs 63 fp32, 95 vs 63 bf16)
    if (whole_image_only && ls.cfg[0].p.NI < 2) return kNotTiled;
    if (((uintptr_t)y & 3) != 0) return kNotTiled;
    for (int i = 0; i < ls.n; i++) {
        ls.cfg[i].p.flip = flip;
        ls.cfg[i].p.add_identity = add_identity;
    }
    DirectMulti mp;
    DirectMaps maps;
    direct_fill_multi(ls, &mp);
    for (int i = 0; i < ls.n; i++)
        O1D_MAP(make_direct_tensor_map(&maps.map[i], x, N, H, W, C, esize, ls.cfg[i].p), "direct fprop");
    PlanView pv = plan_view(plan_dev, ph);
    const cudaError_t e = dtype == O1D_F32 ? launch_direct<float>(ls, mp, maps, w, bias, pv, y, st)
                                           : launch_direct<__nv_bfloat16>(ls, mp, maps, w, bias, pv, y, st);
    if (e != cudaSuccess) return cuda_fail(e, "direct fprop launch");
    g_last_route = O1D_ROUTE_DIRECT;
    return O1D_OK;
}

// Forward / stride-1 input gradient of 7x7 maps with one channel plane per thread.
int try_small7(const void *x, const float *w, const float *bias, const PlanHeader &ph, const void *plan_dev, void *y,
               int N, int H, int W, int C, int K, int stride, int layout, int dtype, int add_identity, int flip,
               cudaStream_t st, const DeviceInfo &d) {
    if (g_force_generic) return kNotTiled;
    const int esize = dtype == O1D_F32 ? 4 : 2;
    SmallConfig cfg;
    if (!small7_configure(ph, N, H, W, C, K, stride, layout, esize, d.smem_optin, d.sms, &cfg)) return kNotTiled;
    if (((uintptr_t)y & 15) != 0) return kNotTiled;
    CUtensorMap map;
    O1D_MAP(make_small7_tensor_map(&map, x, N, C, esize, cfg.p.CCs), "7x7 plane fprop");
    cfg.p.flip = flip;
    cfg.p.add_identity = add_identity;
    PlanView pv = plan_view(plan_dev, ph);
    const cudaError_t e = dtype == O1D_F32 ? launch_small7<float>(cfg, map, w, bias, pv.chan, y, st)
                                           : launch_small7<__nv_bfloat16>(cfg, map, w, bias, pv.chan, y, st);
    if (e != cudaSuccess) return cuda_fail(e, "7x7 plane kernel launch");
    g_last_route = O1D_ROUTE_PLANE7;
    return O1D_OK;
}

// Weight gradient of 7x7 maps with one channel plane per thread.
int try_small7_wgrad(const void *dy, const void *x, const PlanHeader &ph, const void *plan_dev, float *dw, float *db,
                     void *workspace, size_t workspace_bytes, int N, int H, int W, int C, int K, int stride,
                     int layout, int dtype, cudaStream_t st, const DeviceInfo &d) {
    if (g_force_generic) return kNotTiled;
    const int esize = dtype == O1D_F32 ? 4 : 2;
    SmallConfig cfg;
    if (!small7_wgrad_configure(ph, N, H, W, C, K, stride, layout, esize, d.smem_optin, d.sms, &cfg)) return kNotTiled;
    if (((uintptr_t)workspace & 15) != 0) return kNotTiled;
    if (workspace_bytes < small7_wgrad_partial_bytes(cfg)) return O1D_ERR_WORKSPACE;
    CUtensorMap mx, mdy;
    O1D_MAP(make_small7_tensor_map(&mx, x, N, C, esize, cfg.p.CCs), "7x7 plane wgrad (x)");
    O1D_MAP(make_small7_tensor_map(&mdy, dy, N, C, esize, cfg.p.CCs), "7x7 plane wgrad (dy)");
    PlanView pv = plan_view(plan_dev, ph);
    float *partial = (float *)workspace;
    const cudaError_t e = dtype == O1D_F32 ? launch_small7_wgrad<float>(cfg, mx, mdy, pv.chan, partial, st)
                                           : launch_small7_wgrad<__nv_bfloat16>(cfg, mx, mdy, pv.chan, partial, st);
    if (e != cudaSuccess) return cuda_fail(e, "7x7 plane wgrad launch");
    const int tot = C * (K + 1);
    small7_wgrad_final_kernel<<<ceil_div(tot, 128), 128, 0, st>>>(partial, dw, db, C, K, cfg.p.CCs, cfg.p.nchunks,
                                                                  cfg.p.tiles_n);
    O1D_CUDA(cudaGetLastError());
    g_last_route = O1D_ROUTE_PLANE7;
    return O1D_OK;
}

// Device address of the failure flag on the current device (kernels of other translation units
// receive it as a pointer); resolved on first use.
int device_flag_ptr(int **out) {
    static std::atomic<int *> cache[64];
    int dev = 0;
    O1D_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return O1D_ERR_UNSUPPORTED;
    int *ptr = cache[dev].load(std::memory_order_acquire);
    if (!ptr) {
        O1D_CUDA(cudaGetSymbolAddress((void **)&ptr, g_o1d_device_error));
        if (!ptr) return O1D_ERR_CUDA;
        cache[dev].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return O1D_OK;
}

// Forward / stride-1 input gradient through the whole-line kernels (square stage maps, canonical
// lines, fp32); kNotTiled when they do not apply.
int try_wline(const void *x, const float *w, const float *bias, const PlanHeader &ph, const void *plan_host,
              const void *plan_dev, void *y, int N, int H, int W, int C, int K, int stride, int layout, int dtype,
              int add_identity, int flip, cudaStream_t st, const DeviceInfo &d, bool need_two_ctas) {
    if (g_force_generic || !ph.all_canon || ph.chan_off == 0) return kNotTiled;
    const int esize = dtype == O1D_F32 ? 4 : 2;
    const int8_t *chan_host = reinterpret_cast<const int8_t *>(static_cast<const char *>(plan_host) + ph.chan_off);
    WlConfig cfg;
    if (!wline_configure(chan_host, N, H, W, C, K, stride, layout, esize, 228 * 1024, d.smem_optin, d.sms, &cfg))
        return kNotTiled;
    if (need_two_ctas && cfg.ctas_per_sm < 2) return kNotTiled;
    if (((uintptr_t)y & 15) != 0) return kNotTiled;
    CUtensorMap map;
    O1D_MAP(make_nhwc_tensor_map(&map, x, N, H, W, C, esize, cfg.box_c, cfg.box_rows), "whole-line fprop");
    int *flag = nullptr;
    int rc = device_flag_ptr(&flag);
    if (rc) return rc;
    PlanView pv = plan_view(plan_dev, ph);
    const cudaError_t e = wline_launch_fprop(cfg, map, w, bias, pv.chan, (float *)y, flip, add_identity, flag, st);
    if (e != cudaSuccess) return cuda_fail(e, "whole-line fprop launch");
    g_last_route = O1D_ROUTE_LINES;
    return O1D_OK;
}

// Forward / stride-1 input gradient through the walker kernels (square fp32 NHWC maps, canonical lines).
int try_walk(const void *x, const float *w, const float *bias, const PlanHeader &ph, const void *plan_host,
             const void *plan_dev, void *y, int N, int H, int W, int C, int K, int stride, int layout, int dtype,
             int add_identity, int flip, cudaStream_t st, const DeviceInfo &d, bool faster_only) {
    if (g_force_generic || !ph.all_canon || ph.chan_off == 0) return kNotTiled;
    const int esize = dtype == O1D_F32 ? 4 : 2;
    const int8_t *chan_host = reinterpret_cast<const int8_t *>(static_cast<const char *>(plan_host) + ph.chan_off);
    WalkConfig cfg;
    if (!walk_configure(chan_host, N, H, W, C, K, stride, layout, esize, d.smem_optin, d.sms, &cfg)) return kNotTiled;
    // Automatic route: only where it is the faster family - 56x56 layers without slanted channels
    // (rows, columns, diagonals in any mix: 138-153 us against 161-183 us for the tiled kernels, batch 128).
    if (faster_only && !(cfg.line_only && cfg.L == 56)) return kNotTiled;
    if (((uintptr_t)y & 15) != 0) return kNotTiled;
    const cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
    const cuuint64_t strides[3] = {(cuuint64_t)C * esize, (cuuint64_t)W * C * esize, (cuuint64_t)H * W * C * esize};
    const cuuint32_t box[4] = {(cuuint32_t)cfg.box_c, (cuuint32_t)cfg.box_w, (cuuint32_t)cfg.box_rows, 1};
    CUtensorMap in_map, out_map;
    O1D_MAP(encode_map4(&in_map, x, esize, dims, strides, box), "walker fprop (input)");
    O1D_MAP(encode_map4(&out_map, y, esize, dims, strides, box), "walker fprop (output)");
    int *flag = nullptr;
    int rc = device_flag_ptr(&flag);
    if (rc) return rc;
    PlanView pv = plan_view(plan_dev, ph);
    const cudaError_t e = walk_launch_fprop(cfg, in_map, out_map, w, bias, pv.chan, flip, add_identity, flag, st);
    if (e != cudaSuccess) return cuda_fail(e, "walker fprop launch");
    g_last_route = O1D_ROUTE_WALK;
    return O1D_OK;
}

// Route of a forward-type call (flip = 1: stride-1 input gradient):
//   1. direct kernels when one tile holds a whole image (small maps),
//   2. tiled kernels (canonical lines, stride 1, sizes in multiples of 7/8),
//   3. direct kernels with row/column tiles (stems, large maps, arbitrary angles),
//   4. general kernels (the caller falls through on kNotTiled).
int route_forward(const void *x, const float *w, const float *bias, const PlanHeader &ph, const void *plan_host,
                  const void *plan_dev, void *y, int N, int H, int W, int C, int K, int stride, int layout,
                  int dtype, int add_identity, int flip, int act, const void *pre, cudaStream_t st,
                  const DeviceInfo &d) {
    int rc = kNotTiled;
    if (act || pre)       // activation on load / its derivative on store: tiled kernels, else general
        return try_tiled(x, w, bias, ph, plan_host, plan_dev, y, N, H, W, C, K, stride, layout, dtype, add_identity,
                         flip, act, pre, st, d);
    if (g_prefer == 0 || g_prefer == 5) {   // items computed in place in their NHWC layout
        rc = try_walk(x, w, bias, ph, plan_host, plan_dev, y, N, H, W, C, K, stride, layout, dtype, add_identity, flip,
                      st, d, /*faster_only=*/g_prefer == 0);
        if (rc != kNotTiled) return rc;
    }
    if (g_prefer == 0 || g_prefer == 4) {   // stage maps with whole lines per thread
        rc = try_wline(x, w, bias, ph, plan_host, plan_dev, y, N, H, W, C, K, stride, layout, dtype, add_identity,
                       flip, st, d, /*need_two_ctas=*/g_prefer == 0);
        if (rc != kNotTiled) return rc;
    }
    if (g_prefer == 0) {       // 7x7 maps on canonical lines: a channel plane per thread
        rc = try_small7(x, w, bias, ph, plan_dev, y, N, H, W, C, K, stride, layout, dtype, add_identity, flip, st, d);
        if (rc != kNotTiled) return rc;
    }
    // Layers whose chunks are all of one line kind (the models' block-wise angle assignment) can
    // leave half of a tiled CTA's threads without a segment; the direct kernels then win even
    // with row tiles (28x28x192 fp32, batch 128: 167 vs 250 us).
    bool weak_tiled = false;
    if (g_prefer == 0 && stride == 1) {
        TiledConfig t;
        if (tiled_configure(ph, plan_host, N, H, W, C, K, stride, layout, dtype == O1D_F32 ? 4 : 2, d.smem_optin, d.sms,
                            OP_FPROP, &t))
            weak_tiled = t.util < 0.7;
    }
    if (g_prefer != 2) {
        rc = try_direct(x, w, bias, ph, plan_host, plan_dev, y, N, H, W, C, K, stride, layout, dtype, add_identity,
                        flip, st, d, /*whole_image_only=*/g_prefer != 3 && !weak_tiled);
        if (rc != kNotTiled) return rc;
    }
    rc = try_tiled(x, w, bias, ph, plan_host, plan_dev, y, N, H, W, C, K, stride, layout, dtype, add_identity, flip,
                   0, nullptr, st, d);
    if (rc != kNotTiled) return rc;
    return try_direct(x, w, bias, ph, plan_host, plan_dev, y, N, H, W, C, K, stride, layout, dtype, add_identity,
                      flip, st, d, false);
}

// Weight gradient through the tiled kernels.  `cfg_only`: just report the workspace size.
int try_tiled_wgrad(const void *dy, const void *x, const PlanHeader &ph, const void *plan_host,
                    const void *plan_dev, float *dw, float *db, void *workspace, size_t workspace_bytes, int N,
                    int H, int W, int C, int K, int stride, int layout, int dtype, int act, cudaStream_t st,
                    const DeviceInfo &d, size_t *need_bytes) {
    if (g_force_generic) return kNotTiled;
    const int esize = dtype == O1D_F32 ? 4 : 2;
    TiledConfig cfg;
    if (!tiled_configure(ph, plan_host, N, H, W, C, K, stride, layout, esize, d.smem_optin, d.sms, OP_WGRAD, &cfg))
        return kNotTiled;
    const size_t need = tiled_wgrad_partial_bytes(cfg);
    if (need_bytes) { *need_bytes = need; return O1D_OK; }
    if (((uintptr_t)dy & 15) != 0 || ((uintptr_t)workspace & 15) != 0) return kNotTiled;
    if (workspace_bytes < need) return O1D_ERR_WORKSPACE;
    CUtensorMap map;
    O1D_MAP(make_nhwc_tensor_map(&map, x, N, H, W, C, esize, cfg.p.CC, cfg.p.BR), "tiled wgrad");
    PlanView pv = plan_view(plan_dev, ph);
    float *partial = (float *)workspace;
    if (act && !tiled_supports_act(cfg)) return kNotTiled;
    cfg.p.act = act;
    cudaError_t e = launch_tiled<OP_WGRAD>(cfg, dtype, map, nullptr, nullptr, pv, const_cast<void *>(dy), partial,
                                           nullptr, st);
    if (e != cudaSuccess) return cuda_fail(e, "tiled wgrad launch");
    const MergeTables mt = merge_tables_for(cfg.jh);
    const int tot = C * (K + 1);
    tiled_wgrad_final_kernel<<<ceil_div(tot, 128), 128, 0, st>>>(partial, pv.chan, dw, db, C, K, cfg.p.CC, N,
                                                                 cfg.p.total_items, cfg.grid, cfg.p.max_visits, cfg.p.order, mt);
    O1D_CUDA(cudaGetLastError());
    g_last_route = O1D_ROUTE_TILED;
    return O1D_OK;
}

// Stride-2 input gradient through the direct kernel (tiles of the dy grid, one pass per output parity class).
int try_direct_dgrad2(const void *dy, const float *w, const PlanHeader &ph, const void *plan_host,
                      const void *plan_dev, void *dx, int N, int H, int W, int C, int K, int layout, int dtype,
                      int add_identity, cudaStream_t st, const DeviceInfo &d) {
    if (g_force_generic) return kNotTiled;
    const int esize = dtype == O1D_F32 ? 4 : 2;
    DirectLaunchSet ls;
    if (!direct_plan_launches(ph, plan_host, N, H, W, C, K, 2, layout, esize, d.smem_optin, d.sms, DIRECT_DGRAD2, &ls))
        return kNotTiled;
    if (((uintptr_t)dx & 3) != 0) return kNotTiled;
    for (int i = 0; i < ls.n; i++) ls.cfg[i].p.add_identity = add_identity;
    DirectMulti mp;
    DirectMaps maps;
    direct_fill_multi(ls, &mp);
    for (int i = 0; i < ls.n; i++)
        O1D_MAP(make_direct_tensor_map(&maps.map[i], dy, N, ls.cfg[i].p.H, ls.cfg[i].p.W, C, esize, ls.cfg[i].p),
                "direct stride-2 dgrad");
    PlanView pv = plan_view(plan_dev, ph);
    const cudaError_t e = dtype == O1D_F32 ? launch_direct_dgrad2<float>(ls, mp, maps, w, pv, dx, H, W, st)
                                           : launch_direct_dgrad2<__nv_bfloat16>(ls, mp, maps, w, pv, dx, H, W, st);
    if (e != cudaSuccess) return cuda_fail(e, "direct stride-2 dgrad launch");
    g_last_route = O1D_ROUTE_DIRECT;
    return O1D_OK;
}

// Weight gradient through the direct kernels (any angles, stride 1 or 2); kNotTiled when they do not apply.
int try_direct_wgrad(const void *dy, const void *x, const PlanHeader &ph, const void *plan_host,
                     const void *plan_dev, float *dw, float *db, void *workspace, size_t workspace_bytes, int N,
                     int H, int W, int C, int K, int stride, int layout, int dtype, cudaStream_t st,
                     const DeviceInfo &d, size_t *need_bytes) {
    if (g_force_generic) return kNotTiled;
    const int esize = dtype == O1D_F32 ? 4 : 2;
    DirectLaunchSet ls;
    if (!direct_plan_launches(ph, plan_host, N, H, W, C, K, stride, layout, esize, d.smem_optin, d.sms, DIRECT_WGRAD, &ls))
        return kNotTiled;
    const size_t need = ls.partial_floats * sizeof(float);
    if (need_bytes) { *need_bytes = need; return O1D_OK; }
    if (((uintptr_t)workspace & 15) != 0) return kNotTiled;
    if (workspace_bytes < need) return O1D_ERR_WORKSPACE;
    DirectMulti mp;
    DirectMaps maps, dym;
    direct_fill_multi(ls, &mp);
    for (int i = 0; i < ls.n; i++) {
        const DirectParams &p = ls.cfg[i].p;
        O1D_MAP(make_direct_tensor_map(&maps.map[i], x, N, H, W, C, esize, p), "direct wgrad (x)");
        O1D_MAP(make_direct_dy_tensor_map(&dym.map[i], dy, N, p.P, p.Q, C, esize, p), "direct wgrad (dy)");
    }
    PlanView pv = plan_view(plan_dev, ph);
    float *partial = (float *)workspace;
    const cudaError_t e = dtype == O1D_F32 ? launch_direct_wgrad<float>(ls, mp, maps, dym, pv, partial, st)
                                           : launch_direct_wgrad<__nv_bfloat16>(ls, mp, maps, dym, pv, partial, st);
    if (e != cudaSuccess) return cuda_fail(e, "direct wgrad launch");
    const int tot = C * (K + 1);
    direct_wgrad_final_kernel<<<ceil_div(tot, 128), 128, 0, st>>>(mp, partial, pv.cls, pv.taps, dw, db, C, K);
    O1D_CUDA(cudaGetLastError());
    g_last_route = O1D_ROUTE_DIRECT;
    return O1D_OK;
}

#define O1D_DISPATCH(fn, ...)                                                                    \
    (dtype == O1D_F32                                                                            \
         ? (layout == O1D_NHWC ? fn<float, O1D_NHWC>(__VA_ARGS__) : fn<float, O1D_NCHW>(__VA_ARGS__)) \
         : (layout == O1D_NHWC ? fn<__nv_bfloat16, O1D_NHWC>(__VA_ARGS__)                        \
                               : fn<__nv_bfloat16, O1D_NCHW>(__VA_ARGS__)))

}  // namespace

extern "C" {

int o1d_abi_version(void) { return O1D_ABI_VERSION; }

const char *o1d_strerror(int status) {
    switch (status) {
        case O1D_OK: return "ok";
        case O1D_ERR_INVALID: return "invalid argument";
        case O1D_ERR_UNSUPPORTED: return "unsupported configuration";
        case O1D_ERR_CUDA: return "CUDA error";
        case O1D_ERR_WORKSPACE: return "workspace missing or too small";
        case O1D_ERR_PLAN: return "plan does not match the call";
        default: return "unknown status";
    }
}

const char *o1d_last_error(void) { return g_err; }

int o1d_last_route(void) { return g_last_route; }

int o1d_set_route(int route) {
    if (route < 0 || route > 5) return O1D_ERR_INVALID;
    g_force_generic = (route == 1);
    g_prefer = (route >= 2) ? route : 0;
    return O1D_OK;
}

int o1d_device_status(int *flag_out) {
    if (!flag_out) return O1D_ERR_INVALID;
    O1D_CUDA(cudaMemcpyFromSymbol(flag_out, g_o1d_device_error, sizeof(int)));
    return O1D_OK;
}

int o1d_selftest_wait_timeout(int *scratch_dev, void *stream) {
    if (!scratch_dev) return O1D_ERR_INVALID;
    wait_timeout_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(1u << 10, scratch_dev);
    O1D_CUDA(cudaGetLastError());
    return O1D_OK;
}

int o1d_device_status_clear(int *flag_out) {
    int flag = 0;
    O1D_CUDA(cudaMemcpyFromSymbol(&flag, g_o1d_device_error, sizeof(int)));
    if (flag) {
        const int zero = 0;
        O1D_CUDA(cudaMemcpyToSymbol(g_o1d_device_error, &zero, sizeof(int)));
    }
    if (flag_out) *flag_out = flag;
    return O1D_OK;
}

int o1d_uses_tiled(const void *plan_host, int N, int H, int W, int C, int K, int stride, int layout, int dtype) {
    if (bad_common(N, H, W, C, K, stride, layout, dtype) || g_force_generic) return 0;
    PlanHeader ph;
    if (check_plan(plan_host, C, K, &ph)) return 0;
    // 148 SMs / 227 KB: the B200 values; the answer does not depend on a device being present
    const int esize = dtype == O1D_F32 ? 4 : 2;
    TiledConfig cfg;
    if (tiled_configure(ph, plan_host, N, H, W, C, K, stride, layout, esize, 232448, 148, OP_FPROP, &cfg)) return 1;
    DirectConfig dcfg;
    const ChunkRange all{0, C / (32 / esize), ph.max_dh, ph.max_dw};
    return direct_configure(ph, plan_host, all, N, H, W, C, K, stride, layout, esize, 232448, 148, false, false, &dcfg) ? 1 : 0;
}

int o1d_offsets(const float *theta_host, int C, int K, int8_t *dh, int8_t *dw) {
    if (!theta_host || !dh || !dw || C <= 0 || K <= 0 || (K & 1) == 0 || K > 255) return O1D_ERR_INVALID;
    for (int c = 0; c < C; c++) raster(theta_host[c], K, dh + (size_t)c * K, dw + (size_t)c * K);
    return O1D_OK;
}

// Worst case: every channel its own class.
size_t o1d_plan_bytes(int C, int K) {
    if (C <= 0 || K <= 0) return 0;
    return sizeof(PlanHeader) + align16((uint32_t)C * 2) + align16((uint32_t)C * K * 2) + align16((uint32_t)C) +
           align16(kNumChunkWidths * sizeof(KindComp)) + align16((uint32_t)C);
}

int o1d_plan_build(const float *theta_host, int C, int K, void *plan_host) {
    if (!theta_host || !plan_host || C <= 0 || C > 65535 || K <= 0 || (K & 1) == 0 || K > 255)
        return O1D_ERR_INVALID;
    std::vector<int8_t> line((size_t)2 * K), dh(K), dw(K);
    std::vector<int8_t> tables;   // ncls * K * 2
    std::vector<uint16_t> cls(C);
    int ncls = 0, max_dh = 0, max_dw = 0;
    for (int c = 0; c < C; c++) {
        // channels with bit-identical angles share a class without re-rasterising
        if (c > 0 && memcmp(theta_host + c, theta_host + c - 1, sizeof(float)) == 0) {
            cls[c] = cls[c - 1];
            continue;
        }
        raster(theta_host[c], K, dh.data(), dw.data());
        for (int k = 0; k < K; k++) { line[2 * k] = dh[k]; line[2 * k + 1] = dw[k]; }
        int found = -1;
        for (int i = 0; i < ncls && found < 0; i++)
            if (memcmp(tables.data() + (size_t)i * 2 * K, line.data(), 2 * K) == 0) found = i;
        if (found < 0) {
            found = ncls++;
            tables.insert(tables.end(), line.begin(), line.end());
            for (int k = 0; k < K; k++) {
                if (abs(dh[k]) > max_dh) max_dh = abs(dh[k]);
                if (abs(dw[k]) > max_dw) max_dw = abs(dw[k]);
            }
        }
        cls[c] = (uint16_t)found;
    }
    PlanHeader h;
    memset(&h, 0, sizeof(h));
    h.magic = kPlanMagic; h.C = C; h.K = K; h.ncls = ncls; h.max_dh = max_dh; h.max_dw = max_dw;
    h.cls_off = sizeof(PlanHeader);
    h.taps_off = h.cls_off + align16((uint32_t)C * 2);
    h.canon_off = h.taps_off + align16((uint32_t)ncls * K * 2);
    h.comps_off = h.canon_off + align16((uint32_t)ncls);
    h.chan_off = h.comps_off + align16(kNumChunkWidths * sizeof(KindComp));
    h.total_bytes = h.chan_off + align16((uint32_t)C);
    char *b = static_cast<char *>(plan_host);
    memset(b, 0, o1d_plan_bytes(C, K));
    memcpy(b + h.cls_off, cls.data(), (size_t)C * 2);
    memcpy(b + h.taps_off, tables.data(), tables.size());
    // canonical orientation of each class: its taps equal the centre of a built-in table
    int all_canon = 1;
    std::vector<int8_t> canon_of(ncls, -1);
    for (int i = 0; i < ncls; i++) {
        int8_t canon = -1;
        for (int o = 0; o < 8 && canon < 0 && K <= kMaxTaps; o++) {
            bool same = true;
            for (int k = 0; k < K && same; k++) {
                const int kk = k - K / 2 + kHalf;
                same = tables[(size_t)i * 2 * K + 2 * k] == kCanonDh[o][kk] &&
                       tables[(size_t)i * 2 * K + 2 * k + 1] == kCanonDw[o][kk];
            }
            if (same) canon = (int8_t)o;
        }
        b[h.canon_off + i] = canon;
        canon_of[i] = canon;
        if (canon < 0) all_canon = 0;
    }
    // distinct (axis, slant, diagonal) compositions of aligned chunks of 4/8/16/32/64 channels
    KindComp comps[kNumChunkWidths];
    for (int ci = 0; ci < kNumChunkWidths; ci++) {
        KindComp &kc = comps[ci];
        memset(&kc, 0, sizeof(kc));
        const int CC = kChunkWidths[ci];
        if (!all_canon || C % CC != 0) { kc.n = -1; continue; }
        for (int c0 = 0; c0 < C && kc.n >= 0; c0 += CC) {
            uint8_t tri[3] = {0, 0, 0};
            for (int c = c0; c < c0 + CC; c++) tri[canon_kind(canon_of[cls[c]])]++;
            bool seen = false;
            for (int t = 0; t < kc.n && !seen; t++) seen = memcmp(kc.tri[t], tri, 3) == 0;
            if (seen) continue;
            if (kc.n == kMaxComps) { kc.n = -1; break; }
            memcpy(kc.tri[kc.n++], tri, 3);
        }
    }
    memcpy(b + h.comps_off, comps, sizeof(comps));
    for (int c = 0; c < C; c++) b[h.chan_off + c] = canon_of[cls[c]];
    h.all_canon = all_canon;
    h.uniform4 = (C % 4 == 0);
    h.uniform8 = (C % 8 == 0);
    for (int c = 0; c < C; c++) {
        if (cls[c] != cls[c & ~3]) h.uniform4 = 0;
        if (cls[c] != cls[c & ~7]) h.uniform8 = 0;
    }
    memcpy(b, &h, sizeof(h));
    return O1D_OK;
}

int o1d_plan_num_classes(const void *plan_host) {
    if (!plan_host) return -1;
    PlanHeader h;
    memcpy(&h, plan_host, sizeof(h));
    return h.magic == kPlanMagic ? h.ncls : -1;
}

int o1d_fprop(const void *x, const float *w, const float *bias, const void *plan_host,
              const void *plan_dev, void *y, int N, int H, int W, int C, int K, int stride, int layout,
              int dtype, int add_identity, void *stream) {
    if (!x || !w || !y || !plan_dev || bad_common(N, H, W, C, K, stride, layout, dtype)) return O1D_ERR_INVALID;
    PlanHeader ph;
    int rc = check_plan(plan_host, C, K, &ph);
    if (rc) return rc;
    DeviceInfo d;
    if ((rc = device_info(&d))) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const int identity = add_identity & O1D_FLAG_IDENTITY, act = (add_identity & O1D_FLAG_GELU_INPUT) ? 1 : 0;
    rc = route_forward(x, w, bias, ph, plan_host, plan_dev, y, N, H, W, C, K, stride, layout, dtype, identity,
                       /*flip=*/0, act, nullptr, st, d);
    if (rc != kNotTiled) return rc;
    return O1D_DISPATCH(launch_generic_fprop, x, w, bias, ph, plan_dev, y, N, H, W, C, K, stride,
                        identity, act, st, d);
}

int o1d_dgrad(const void *dy, const float *w, const void *plan_host, const void *plan_dev, void *dx,
              int N, int H, int W, int C, int K, int stride, int layout, int dtype, int add_identity,
              void *stream) {
    return o1d_dgrad_act(dy, w, nullptr, plan_host, plan_dev, dx, N, H, W, C, K, stride, layout, dtype,
                         add_identity, stream);
}

int o1d_dgrad_act(const void *dy, const float *w, const void *pre, const void *plan_host, const void *plan_dev,
                  void *dx, int N, int H, int W, int C, int K, int stride, int layout, int dtype, int add_identity,
                  void *stream) {
    if (!dy || !w || !dx || !plan_dev || bad_common(N, H, W, C, K, stride, layout, dtype)) return O1D_ERR_INVALID;
    PlanHeader ph;
    int rc = check_plan(plan_host, C, K, &ph);
    if (rc) return rc;
    DeviceInfo d;
    if ((rc = device_info(&d))) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    // stride 1: dx = fprop(dy) with the taps mirrored, i.e. (the lines being odd-symmetric)
    // with the weights read in reverse order
    add_identity &= O1D_FLAG_IDENTITY;
    rc = stride == 1 ? route_forward(dy, w, nullptr, ph, plan_host, plan_dev, dx, N, H, W, C, K, stride, layout,
                                     dtype, add_identity, /*flip=*/1, 0, pre, st, d)
         : (stride == 2 && !pre) ? try_direct_dgrad2(dy, w, ph, plan_host, plan_dev, dx, N, H, W, C, K, layout, dtype,
                                                     add_identity, st, d)
                                 : kNotTiled;
    if (rc != kNotTiled) return rc;
    return O1D_DISPATCH(launch_generic_dgrad, dy, w, ph, plan_dev, dx, N, H, W, C, K, stride,
                        add_identity, pre, st, d);
}

size_t o1d_wgrad_workspace_bytes(int N, int H, int W, int C, int K, int stride, int layout, int dtype) {
    if (bad_common(N, H, W, C, K, stride, layout, dtype)) return 0;
    const int P = ceil_div(H, stride), Q = ceil_div(W, stride);
    // Large enough for every kernel family, without needing the plan: the general kernels' slices;
    // one partial per persistent CTA and chunk visit (tiled and direct kernels, an upper bound);
    // one partial per (channel, tile of 32 images) for the 7x7 plane kernels.
    const size_t general = (size_t)generic_wgrad_slices(N, P, Q, C, layout) * C * (K + 1) * sizeof(float);
    const size_t tiled = (size_t)kMaxTiledCtas * 4 * kMaxCC * kPartialStride * sizeof(float);
    const size_t plane7 = (H == 7 && W == 7) ? (size_t)C * ceil_div(N, kSmallImgs) * 32 * sizeof(float) : 0;
    size_t need = general > tiled ? general : tiled;
    if (plane7 > need) need = plane7;
    return need;
}

}  // extern "C"

namespace {
// Weight gradient with `workspace_bytes` of scratch at `workspace`: each kernel family in the order
// of preference, skipping a family whose partial sums do not fit.  Small maps: the direct kernels
// first (measured at batch 128: fp32 28x28 120 vs 142 us, 14x14 75 vs 84, 7x7 33 vs 59; bf16 only at
// 7x7, 40 vs 64, since every 2-byte load needs a widening shift).  Otherwise tiled, then direct
// (stems, dense-prediction maps, arbitrary angles), then general.
int wgrad_dispatch(const void *dy, const void *x, const PlanHeader &ph, const void *plan_host, const void *plan_dev,
                   float *dw, float *db, void *workspace, size_t workspace_bytes, int N, int H, int W, int C, int K,
                   int stride, int layout, int dtype, int act, cudaStream_t st, const DeviceInfo &d) {
    int rc;
    if (act) {                 // x is GELU(pre), applied on load: tiled kernels, else general
        rc = try_tiled_wgrad(dy, x, ph, plan_host, plan_dev, dw, db, workspace, workspace_bytes, N, H, W, C, K, stride,
                             layout, dtype, act, st, d, nullptr);
        if (rc != kNotTiled && rc != O1D_ERR_WORKSPACE) return rc;
    } else
    if (g_prefer == 0) {       // 7x7 maps on canonical lines: a channel plane per thread
        rc = try_small7_wgrad(dy, x, ph, plan_dev, dw, db, workspace, workspace_bytes, N, H, W, C, K, stride, layout,
                              dtype, st, d);
        if (rc != kNotTiled && rc != O1D_ERR_WORKSPACE) return rc;
    }
    const bool small_map = (dtype == O1D_F32) ? (H * W <= 32 * 32) : (H * W <= 10 * 10);
    bool weak_tiled = false;     // see route_forward
    if (g_prefer == 0 && !small_map) {
        TiledConfig t;
        if (tiled_configure(ph, plan_host, N, H, W, C, K, stride, layout, dtype == O1D_F32 ? 4 : 2, d.smem_optin, d.sms,
                            OP_WGRAD, &t))
            weak_tiled = t.util < 0.7;
    }
    const bool direct_first = !act && (g_prefer == 3 || (g_prefer == 0 && (small_map || weak_tiled)));
    if (direct_first) {
        rc = try_direct_wgrad(dy, x, ph, plan_host, plan_dev, dw, db, workspace, workspace_bytes, N, H, W, C, K,
                              stride, layout, dtype, st, d, nullptr);
        if (rc != kNotTiled && rc != O1D_ERR_WORKSPACE) return rc;
    }
    if (!act) {
        rc = try_tiled_wgrad(dy, x, ph, plan_host, plan_dev, dw, db, workspace, workspace_bytes, N, H, W, C, K, stride,
                             layout, dtype, 0, st, d, nullptr);
        if (rc != kNotTiled && rc != O1D_ERR_WORKSPACE) return rc;
    }
    if (!direct_first && !act) {
        rc = try_direct_wgrad(dy, x, ph, plan_host, plan_dev, dw, db, workspace, workspace_bytes, N, H, W, C, K,
                              stride, layout, dtype, st, d, nullptr);
        if (rc != kNotTiled && rc != O1D_ERR_WORKSPACE) return rc;
    }
    const int P = ceil_div(H, stride), Q = ceil_div(W, stride);
    const size_t need = (size_t)generic_wgrad_slices(N, P, Q, C, layout) * C * (K + 1) * sizeof(float);
    if (need > workspace_bytes) {
        snprintf(g_err, sizeof(g_err), "weight gradient needs %zu bytes of scratch, %zu are available", need,
                 workspace_bytes);
        return O1D_ERR_WORKSPACE;
    }
    return O1D_DISPATCH(launch_generic_wgrad, dy, x, ph, plan_dev, dw, db, (float *)workspace, N, H, W,
                        C, K, stride, act, st);
}
}  // namespace

extern "C" {

int o1d_wgrad(const void *dy, const void *x, const void *plan_host, const void *plan_dev, float *dw,
              float *db, void *workspace, size_t workspace_bytes, int N, int H, int W, int C, int K,
              int stride, int layout, int dtype, void *stream) {
    return o1d_wgrad_act(dy, x, plan_host, plan_dev, dw, db, workspace, workspace_bytes, N, H, W, C, K, stride, layout,
                         dtype, 0, stream);
}

int o1d_wgrad_act(const void *dy, const void *x, const void *plan_host, const void *plan_dev, float *dw,
                  float *db, void *workspace, size_t workspace_bytes, int N, int H, int W, int C, int K,
                  int stride, int layout, int dtype, int flags, void *stream) {
    if (!dy || !x || !dw || !plan_dev || bad_common(N, H, W, C, K, stride, layout, dtype)) return O1D_ERR_INVALID;
    PlanHeader ph;
    int rc = check_plan(plan_host, C, K, &ph);
    if (rc) return rc;
    if (!workspace || workspace_bytes < o1d_wgrad_workspace_bytes(N, H, W, C, K, stride, layout, dtype))
        return O1D_ERR_WORKSPACE;
    DeviceInfo d;
    if ((rc = device_info(&d))) return rc;
    return wgrad_dispatch(dy, x, ph, plan_host, plan_dev, dw, db, workspace, workspace_bytes, N, H, W, C, K, stride,
                          layout, dtype, (flags & O1D_FLAG_GELU_INPUT) ? 1 : 0, (cudaStream_t)stream, d);
}

// ---------------------------------------------------------------------------------------
// Weight gradient for callers that cannot allocate.
//
// Some hosts of this library have no way to hand it a workspace: code that runs inside a
// framework hook or a plugin sandbox where device allocation is forbidden, a process whose
// memory pool was sized once at start-up and is fully committed, or a call site reached
// while an allocator lock is held.  For them the per-block partial sums of the weight
// gradient live in the fixed array below instead of a caller buffer.  The array is part
// of the library image: every GPU that loads libo1d holds these bytes until the process
// exits, which is why the size is modest and requests that need more are refused.
//
// The array's name is only a host-side handle.  Its device address is looked up once per
// device with cudaGetSymbolAddress (with that device current) and that address is what the
// kernels receive.
// ---------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_wgrad_static_scratch[O1D_STATIC_SCRATCH_BYTES];

}  // extern "C"

namespace {
// Device address of the static scratch on the current device; resolved on first use.  Threads
// that race on a device's first use each look the address up and publish the same value.
int static_scratch_ptr(void **out) {
    static std::atomic<void *> cache[64];
    int dev = 0;
    O1D_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return O1D_ERR_UNSUPPORTED;
    void *ptr = cache[dev].load(std::memory_order_acquire);
    if (!ptr) {
        O1D_CUDA(cudaGetSymbolAddress(&ptr, g_wgrad_static_scratch));
        if (!ptr) return O1D_ERR_CUDA;
        cache[dev].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return O1D_OK;
}
}  // namespace

extern "C" {

int o1d_wgrad_static(const void *dy, const void *x, const void *plan_host, const void *plan_dev, float *dw,
                     float *db, int N, int H, int W, int C, int K, int stride, int layout, int dtype,
                     void *stream) {
    if (!dy || !x || !dw || !plan_dev || bad_common(N, H, W, C, K, stride, layout, dtype)) return O1D_ERR_INVALID;
    PlanHeader ph;
    int rc = check_plan(plan_host, C, K, &ph);
    if (rc) return rc;
    DeviceInfo d;
    if ((rc = device_info(&d))) return rc;
    void *scratch = nullptr;
    if ((rc = static_scratch_ptr(&scratch))) return rc;
    // Same order of kernel families as o1d_wgrad(); a family whose partial sums exceed the array
    // is skipped, and when even the general kernels' do not fit the request is refused.
    rc = wgrad_dispatch(dy, x, ph, plan_host, plan_dev, dw, db, scratch, O1D_STATIC_SCRATCH_BYTES, N, H, W, C, K,
                        stride, layout, dtype, 0, (cudaStream_t)stream, d);
    if (rc == O1D_ERR_WORKSPACE) {
        snprintf(g_err, sizeof(g_err), "o1d_wgrad_static: the partial sums of this shape do not fit the built-in "
                 "array of %d bytes; use o1d_wgrad() with a workspace", O1D_STATIC_SCRATCH_BYTES);
        return O1D_ERR_UNSUPPORTED;
    }
    return rc;
}

}  // extern "C"

namespace {
template <typename T, int G, int VPL>
int launch_ln(const void *x, const float *gamma, const float *beta, void *y, int64_t rows, int C, float eps, int gelu,
              cudaStream_t st, const DeviceInfo &d) {
    const int64_t groups = (rows * G + kLnThreads - 1) / kLnThreads;
    const int64_t cap = (int64_t)d.sms * 16;
    const int grid = (int)(groups < cap ? (groups > 0 ? groups : 1) : cap);
    layernorm_cl_kernel<T, G, VPL><<<grid, kLnThreads, 0, st>>>((const T *)x, gamma, beta, (T *)y, rows, C, eps, gelu);
    O1D_CUDA(cudaGetLastError());
    return O1D_OK;
}
// Grid of the LayerNorm backward for `rows` rows handled by groups of G lanes.
inline int ln_bwd_grid(int64_t rows, int G, int sms) {
    const int64_t groups = (rows * G + kLnThreads - 1) / kLnThreads;
    const int64_t cap = (int64_t)sms * 4;
    return (int)(groups < cap ? (groups > 0 ? groups : 1) : cap);
}
template <typename T, int G, int VPL>
int launch_ln_bwd(const void *x, const void *dy, const float *gamma, const float *beta, void *dx, float *dgamma,
                  float *dbeta, float *partial, int64_t rows, int C, float eps, int gelu, cudaStream_t st,
                  const DeviceInfo &d) {
    const int grid = ln_bwd_grid(rows, G, d.sms);
    const int smem = (kLnThreads / 32) * 2 * C * (int)sizeof(float);
    if (gelu) {
        auto kern = layernorm_cl_bwd_kernel<T, G, VPL, true>;
        if (smem > 48 * 1024) O1D_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        kern<<<grid, kLnThreads, smem, st>>>((const T *)x, (const T *)dy, gamma, beta, (T *)dx, partial, rows, C, eps);
    } else {
        auto kern = layernorm_cl_bwd_kernel<T, G, VPL, false>;
        if (smem > 48 * 1024) O1D_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        kern<<<grid, kLnThreads, smem, st>>>((const T *)x, (const T *)dy, gamma, beta, (T *)dx, partial, rows, C, eps);
    }
    O1D_CUDA(cudaGetLastError());
    layernorm_cl_bwd_final_kernel<<<ceil_div(2 * C, 32), dim3(32, 8), 0, st>>>(partial, dgamma, dbeta, grid, C);
    O1D_CUDA(cudaGetLastError());
    return O1D_OK;
}
template <typename T>
int dispatch_ln_bwd(const void *x, const void *dy, const float *gamma, const float *beta, void *dx, float *dgamma,
                    float *dbeta, float *partial, int64_t rows, int C, float eps, int gelu, cudaStream_t st,
                    const DeviceInfo &d) {
    const int nvec = C / (16 / (int)sizeof(T));
#define O1D_LNB(G, V) launch_ln_bwd<T, G, V>(x, dy, gamma, beta, dx, dgamma, dbeta, partial, rows, C, eps, gelu, st, d)
    if (nvec <= 8) return O1D_LNB(8, 1);
    if (nvec <= 16) return O1D_LNB(8, 2);
    if (nvec <= 32) return O1D_LNB(16, 2);
    if (nvec <= 64) return O1D_LNB(32, 2);
    if (nvec <= 128) return O1D_LNB(32, 4);
#undef O1D_LNB
    return O1D_ERR_UNSUPPORTED;
}
template <typename T>
int dispatch_ln(const void *x, const float *gamma, const float *beta, void *y, int64_t rows, int C, float eps,
                int gelu, cudaStream_t st, const DeviceInfo &d) {
    const int nvec = C / (16 / (int)sizeof(T));
    if (nvec <= 8) return launch_ln<T, 8, 1>(x, gamma, beta, y, rows, C, eps, gelu, st, d);
    // two vectors per lane: fewer shuffle steps and more rows in flight per warp
    if (nvec <= 16) return launch_ln<T, 8, 2>(x, gamma, beta, y, rows, C, eps, gelu, st, d);
    if (nvec <= 32) return launch_ln<T, 16, 2>(x, gamma, beta, y, rows, C, eps, gelu, st, d);
    if (nvec <= 64) return launch_ln<T, 32, 2>(x, gamma, beta, y, rows, C, eps, gelu, st, d);
    if (nvec <= 128) return launch_ln<T, 32, 4>(x, gamma, beta, y, rows, C, eps, gelu, st, d);
    if (nvec <= 256) return launch_ln<T, 32, 8>(x, gamma, beta, y, rows, C, eps, gelu, st, d);
    return O1D_ERR_UNSUPPORTED;
}
}  // namespace

extern "C" {

int o1d_layernorm_cl(const void *x, const float *gamma, const float *beta, void *y, long long rows, int C,
                     float eps, int dtype, int gelu, void *stream) {
    if (!x || !gamma || !beta || !y || rows <= 0 || C <= 0 || (dtype != O1D_F32 && dtype != O1D_BF16))
        return O1D_ERR_INVALID;
    const int ve = dtype == O1D_F32 ? 4 : 8;
    if (C % ve != 0 || ((uintptr_t)x & 15) || ((uintptr_t)y & 15)) return O1D_ERR_UNSUPPORTED;
    DeviceInfo d;
    int rc = device_info(&d);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    return dtype == O1D_F32 ? dispatch_ln<float>(x, gamma, beta, y, rows, C, eps, gelu, st, d)
                            : dispatch_ln<__nv_bfloat16>(x, gamma, beta, y, rows, C, eps, gelu, st, d);
}

size_t o1d_layernorm_cl_bwd_workspace_bytes(long long rows, int C) {
    if (rows <= 0 || C <= 0) return 0;
    DeviceInfo d;
    if (device_info(&d)) return 0;
    return (size_t)d.sms * 4 * 2 * (size_t)C * sizeof(float);       // one partial per CTA of the largest grid
}

int o1d_layernorm_cl_bwd(const void *x, const void *dy, const float *gamma, const float *beta, void *dx, float *dgamma,
                         float *dbeta, void *workspace, size_t workspace_bytes, long long rows, int C, float eps,
                         int dtype, int gelu, void *stream) {
    if (!x || !dy || !gamma || !dx || !dgamma || !dbeta || (gelu && !beta) || rows <= 0 || C <= 0 ||
        (dtype != O1D_F32 && dtype != O1D_BF16))
        return O1D_ERR_INVALID;
    const int ve = dtype == O1D_F32 ? 4 : 8;
    if (C % ve != 0 || C / ve > 128 || ((uintptr_t)x & 15) || ((uintptr_t)dy & 15) || ((uintptr_t)dx & 15))
        return O1D_ERR_UNSUPPORTED;
    if (!workspace || workspace_bytes < o1d_layernorm_cl_bwd_workspace_bytes(rows, C)) return O1D_ERR_WORKSPACE;
    DeviceInfo d;
    int rc = device_info(&d);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    return dtype == O1D_F32 ? dispatch_ln_bwd<float>(x, dy, gamma, beta, dx, dgamma, dbeta, (float *)workspace, rows, C,
                                                     eps, gelu, st, d)
                            : dispatch_ln_bwd<__nv_bfloat16>(x, dy, gamma, beta, dx, dgamma, dbeta, (float *)workspace,
                                                             rows, C, eps, gelu, st, d);
}

extern "C++" {
namespace {
// rows a CTA reads per pass (1, 2, 4, 8 or 16): narrow matrices give every lane a vector
int colsum_row_lanes(int nvec) {
    int rl = 1;
    while (rl < 16 && nvec * rl * 2 <= kColsumThreads) rl *= 2;
    return rl;
}
int colsum_slices(long long rows, int C, int ve, int sms) {
    const int nvec = C / ve, rl = colsum_row_lanes(nvec);
    const int col_blocks = ceil_div(nvec, kColsumThreads / rl);
    long long s = ((long long)sms * 4 + col_blocks - 1) / col_blocks;      // about four CTAs per SM in all
    const long long most = (rows + 8LL * rl - 1) / (8LL * rl);             // at least eight passes per slice
    if (s > most) s = most;
    if (s > 4096) s = 4096;
    return (int)(s < 1 ? 1 : s);
}
template <typename T>
void launch_colsum(const void *x, float *partial, long long rows, int C, int slices, cudaStream_t st) {
    const int nvec = C / (16 / (int)sizeof(T)), rl = colsum_row_lanes(nvec);
    dim3 grid(ceil_div(nvec, kColsumThreads / rl), slices);
    switch (rl) {
        case 1: colsum_partial_kernel<T, 1><<<grid, kColsumThreads, 0, st>>>((const T *)x, partial, rows, C); break;
        case 2: colsum_partial_kernel<T, 2><<<grid, kColsumThreads, 0, st>>>((const T *)x, partial, rows, C); break;
        case 4: colsum_partial_kernel<T, 4><<<grid, kColsumThreads, 0, st>>>((const T *)x, partial, rows, C); break;
        case 8: colsum_partial_kernel<T, 8><<<grid, kColsumThreads, 0, st>>>((const T *)x, partial, rows, C); break;
        default: colsum_partial_kernel<T, 16><<<grid, kColsumThreads, 0, st>>>((const T *)x, partial, rows, C); break;
    }
}
}  // namespace
}  // extern "C++"

size_t o1d_colsum_workspace_bytes(long long rows, int C, int dtype) {
    if (rows <= 0 || C <= 0) return 0;
    DeviceInfo d;
    if (device_info(&d)) return 0;
    const int ve = dtype == O1D_F32 ? 4 : 8;
    if (C % ve != 0) return 0;
    return (size_t)colsum_slices(rows, C, ve, d.sms) * (size_t)C * sizeof(float);
}

int o1d_colsum(const void *x, float *out, void *workspace, size_t workspace_bytes, long long rows, int C, int dtype,
               void *stream) {
    if (!x || !out || rows <= 0 || C <= 0 || (dtype != O1D_F32 && dtype != O1D_BF16)) return O1D_ERR_INVALID;
    const int ve = dtype == O1D_F32 ? 4 : 8;
    if (C % ve != 0 || ((uintptr_t)x & 15)) return O1D_ERR_UNSUPPORTED;
    DeviceInfo d;
    int rc = device_info(&d);
    if (rc) return rc;
    const int slices = colsum_slices(rows, C, ve, d.sms);
    if (!workspace || workspace_bytes < (size_t)slices * C * sizeof(float)) return O1D_ERR_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == O1D_F32) launch_colsum<float>(x, (float *)workspace, rows, C, slices, st);
    else launch_colsum<__nv_bfloat16>(x, (float *)workspace, rows, C, slices, st);
    O1D_CUDA(cudaGetLastError());
    colsum_final_kernel<<<ceil_div(C, 32), dim3(32, 8), 0, st>>>((const float *)workspace, out, slices, C);
    O1D_CUDA(cudaGetLastError());
    return O1D_OK;
}

int o1d_pointwise_in(const void *x, const float *w, const float *bias, void *y, int N, int Cin, long long HW,
                     int Cout, int dtype, void *stream) {
    if (!x || !w || !y || N <= 0 || HW <= 0 || Cin <= 0 || Cout <= 0 || (dtype != O1D_F32 && dtype != O1D_BF16))
        return O1D_ERR_INVALID;
    if (Cin > 4 || Cout % 8 != 0 || HW > 0x7fffffffLL || ((uintptr_t)y & 15)) return O1D_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    if (Cout / 8 > kPointwiseThreads) return O1D_ERR_UNSUPPORTED;
    const long long npix = (long long)N * HW;
    const long long per_block = (long long)(kPointwiseThreads / (Cout / 8)) * kPointwisePasses;
    const long long blocks = (npix + per_block - 1) / per_block;
    if (blocks > 0x7fffffffLL) return O1D_ERR_UNSUPPORTED;
#define O1D_PW(T, CIN)                                                                                     \
    pointwise_in_kernel<T, CIN><<<(unsigned)blocks, kPointwiseThreads, 0, st>>>((const T *)x, w, bias, (T *)y, npix, \
                                                                                (int)HW, Cout)
    if (dtype == O1D_F32) {
        switch (Cin) { case 1: O1D_PW(float, 1); break; case 2: O1D_PW(float, 2); break;
                       case 3: O1D_PW(float, 3); break; default: O1D_PW(float, 4); break; }
    } else {
        switch (Cin) { case 1: O1D_PW(__nv_bfloat16, 1); break; case 2: O1D_PW(__nv_bfloat16, 2); break;
                       case 3: O1D_PW(__nv_bfloat16, 3); break; default: O1D_PW(__nv_bfloat16, 4); break; }
    }
#undef O1D_PW
    O1D_CUDA(cudaGetLastError());
    return O1D_OK;
}

int o1d_transpose(const void *in, void *out, int n, int a, int b, int dtype, void *stream) {
    if (!in || !out || n <= 0 || a <= 0 || b <= 0 || (dtype != O1D_F32 && dtype != O1D_BF16)) return O1D_ERR_INVALID;
    if (n > 65535) return O1D_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    const bool al_in = ((uintptr_t)in & 15) == 0, al_out = ((uintptr_t)out & 15) == 0;
    if (dtype == O1D_F32) {
        dim3 grid(ceil_div(b, 32), ceil_div(a, 32), n);
        transpose_kernel<uint32_t><<<grid, kTransposeThreads, 0, st>>>(
            (const uint32_t *)in, (uint32_t *)out, a, b, al_in && b % 4 == 0, al_out && a % 4 == 0);
    } else {
        dim3 grid(ceil_div(b, 64), ceil_div(a, 64), n);
        transpose_kernel<uint16_t><<<grid, kTransposeThreads, 0, st>>>(
            (const uint16_t *)in, (uint16_t *)out, a, b, al_in && b % 8 == 0, al_out && a % 8 == 0);
    }
    O1D_CUDA(cudaGetLastError());
    return O1D_OK;
}

}  // extern "C"
