/*
 * o1d — oriented 1D depthwise convolution for NVIDIA B200 (sm_100a).  C ABI.
 *
 * This is the boundary a binding of the reference project would call instead of its
 * JIT-compiled extension modules.  Every entry point
 *   - takes plain pointers and sizes (no torch types),
 *   - works on CALLER-ALLOCATED device buffers, allocates nothing and never
 *     synchronises the device,
 *   - launches on the CUDA stream passed as `stream` (a cudaStream_t; NULL = default),
 *   - returns an int status (O1D_OK or an O1D_ERR_* code; see o1d_strerror()).
 *
 * Operator definition (reference: models/dwoconv1d_reference/kernels/kernels.cpp:20-129).
 * For channel c with angle theta[c], tap k in [0,K), pad = K/2, j = k - pad:
 *     dh[c,k] = (int)(-sinf(theta[c]) * j),   dw[c,k] = (int)(cosf(theta[c]) * j)
 *     y [n,c,p,q] = bias[c] + sum_k w'[c,k] * x[n,c,p*s+dh, q*s+dw]       (zero outside)
 *     dx[n,c,h,w] = sum_k w'[c,k] * dy[n,c,(h-dh)/s,(w-dw)/s]   (divisible, in range)
 *     dw[c,k]     = sum_{n,p,q} x[n,c,p*s+dh, q*s+dw] * dy[n,c,p,q];   db[c] = sum dy
 * with w' = w + (k == pad) when add_identity is set (the reference's `resid`,
 * models/dwoconv1d/dwoconv1d.py:22-23,136-141).  H, W are always the INPUT extents;
 * the output extents are P = ceil(H/s), Q = ceil(W/s) (the reference's forward()
 * requires divisibility, kernels.cu:19-20; its forward_safe() pads and crops to the
 * same ceil sizes, dwoconv1d.py:154-187).
 *
 * Tensors x, y, dy, dx are fp32 or bf16 (`dtype`), NCHW or NHWC contiguous (`layout`).
 * w [C,K], bias [C], dw [C,K], db [C] are always fp32; accumulation is fp32.
 */
#ifndef O1D_H_
#define O1D_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define O1D_ABI_VERSION 2

enum {
    O1D_OK = 0,
    O1D_ERR_INVALID = 1,      /* null pointer, non-positive size, even K, bad enum ...   */
    O1D_ERR_UNSUPPORTED = 2,  /* valid request this build has no kernel for              */
    O1D_ERR_CUDA = 3,         /* a CUDA call or launch failed; see o1d_last_error()      */
    O1D_ERR_WORKSPACE = 4,    /* workspace pointer missing or too small                  */
    O1D_ERR_PLAN = 5          /* plan blob does not match C / K or is corrupt            */
};

enum { O1D_NCHW = 0, O1D_NHWC = 1 };
/* Bits of the `add_identity` / `flags` argument of the operators. */
enum {
    O1D_FLAG_IDENTITY = 1,    /* w' = w + (k == pad): the reference's `resid`                     */
    O1D_FLAG_GELU_INPUT = 2   /* the input tensor is a pre-activation: exact GELU is applied as it is loaded */
};
enum { O1D_F32 = 0, O1D_BF16 = 1 };

/* Library identification.  (No counterpart in the reference: its modules are found by
 * name in the torch extension cache, models/dwoconv1d/dwoconv1d_kernel.py:76-90.) */
int o1d_abi_version(void);
const char *o1d_strerror(int status);
/* Text of the last CUDA failure seen by the calling thread ("" if none). */
const char *o1d_last_error(void);

/* Kernel routing, for tests and A/B timing: 0 = automatic, 1 = general kernels only,
 * 2 = prefer the tiled kernels, 3 = prefer the direct kernels, 4 = prefer the whole-line
 * kernels, 5 = prefer the walker kernels.  Process-wide.  (No counterpart in
 * the reference, which picks general vs specialised kernels with the SPECIALIZED
 * environment variable at import time, models/convnext.py:16-23.) */
int o1d_set_route(int route);

/* Kernel family that served the calling thread's last successful o1d_fprop / o1d_dgrad /
 * o1d_wgrad / o1d_wgrad_static call (O1D_ROUTE_NONE before the first one).  A diagnostic: a
 * request that a fast family declines lands on the general kernels with the same results but
 * several times the run time, and this is how a host or a test notices.  Per thread.  (No
 * counterpart in the reference, whose module either is the specialised one or is not,
 * models/convnext.py:16-23.) */
enum {
    O1D_ROUTE_NONE = -1,
    O1D_ROUTE_GENERAL = 0,   /* gather kernels: any stride, layout, angle                      */
    O1D_ROUTE_TILED = 1,     /* restaged channel planes with register windows                  */
    O1D_ROUTE_DIRECT = 2,    /* TMA halo tiles, one tap list per thread                        */
    O1D_ROUTE_PLANE7 = 3,    /* 7x7 maps, one channel plane per thread                         */
    O1D_ROUTE_LINES = 4,     /* whole lines per thread (round-robin angle assignment)          */
    O1D_ROUTE_WALK = 5       /* items computed in place in their NHWC layout (square fp32 maps) */
};
int o1d_last_route(void);

/* Reads the device-side failure flag of the current device into *flag_out (0 = healthy,
 * 1 = a kernel gave up waiting for a TMA transfer and its output is invalid).  This call
 * SYNCHRONISES the device; it is a diagnostic, not part of the hot path.  (The reference
 * checks no launch or device errors at all, kernels.h:529,542,555.) */
int o1d_device_status(int *flag_out);
/* The same, and resets the flag to 0 afterwards (flag_out may be NULL). */
int o1d_device_status_clear(int *flag_out);
/* Exercises that failure path without a fault: launches one warp that waits, with a limit of
 * about a thousand polls, on a barrier nothing will ever complete.  The wait runs out, the
 * kernel raises the device flag, writes 1 to *scratch_dev (a caller-allocated int in device
 * memory) and returns normally; the context stays usable.  Afterwards o1d_device_status()
 * reads 1 until o1d_device_status_clear() is called.  (No counterpart in the reference.) */
int o1d_selftest_wait_timeout(int *scratch_dev, void *stream);

/* 1 if o1d_fprop would take one of the TMA-staged kernel families (tiled or direct) for this
 * request, 0 if the general kernels.  Lets a host decide whether converting an NCHW tensor
 * to NHWC first pays off (the tiled kernels are NHWC only).  Host-only; no counterpart in
 * the reference. */
int o1d_uses_tiled(const void *plan_host, int N, int H, int W, int C, int K, int stride,
                   int layout, int dtype);

/* Rasterised tap offsets of C channels, computed on the host exactly as the reference's
 * CPU loops do (kernels.cpp:37,43-44).  theta_host: C floats (radians, fp32);
 * dh, dw: C*K int8 each.  Requires K odd, K <= 255. */
int o1d_offsets(const float *theta_host, int C, int K, int8_t *dh, int8_t *dw);

/* A "plan" is the per-layer tap table in the form the kernels consume: channels with
 * identical rasterised lines share one orientation class.  It replaces the per-thread
 * sincosf() + float->int conversion the reference kernels redo for every tap of every
 * output (models/dwoconv1d/kernels/kernels.h:239-240,285).  The caller allocates
 * o1d_plan_bytes() bytes on the host, fills them with o1d_plan_build(), and uploads a
 * byte-for-byte copy to the device; the operators take both pointers (the host copy
 * steers kernel selection, the device copy is read by the kernels). */
size_t o1d_plan_bytes(int C, int K);
int o1d_plan_build(const float *theta_host, int C, int K, void *plan_host);
/* Number of distinct orientation classes in a built plan (negative on a bad blob). */
int o1d_plan_num_classes(const void *plan_host);

/* Forward.  Replaces fprop(x, w, theta) of the reference's extension module
 * (models/dwoconv1d/kernels/kernels.cu:15-27, kernels.h:207-310; specialized:
 * models/dwoconv1d_specialized/kernels/kernels.cu:17-30) together with the separate
 * bias add and w+resid passes of its Python wrapper (dwoconv1d.py:22-23,34-35).
 * bias may be NULL.  `add_identity` is a flag word: O1D_FLAG_IDENTITY, and O1D_FLAG_GELU_INPUT for
 * y = conv(GELU(x)) with x the pre-activation tensor, which removes the separate F.gelu pass in
 * front of the 1D++ / 2D++ blocks' second conv (models/convnext.py:389-391, :463-465). */
int o1d_fprop(const void *x, const float *w, const float *bias,
              const void *plan_host, const void *plan_dev, void *y,
              int N, int H, int W, int C, int K, int stride,
              int layout, int dtype, int add_identity, void *stream);

/* Input gradient.  Replaces dgrad(dy, w, theta) (kernels.cu:29-40, kernels.h:312-399).
 * dy has extents ceil(H/s) x ceil(W/s); dx has extents H x W. */
int o1d_dgrad(const void *dy, const float *w,
              const void *plan_host, const void *plan_dev, void *dx,
              int N, int H, int W, int C, int K, int stride,
              int layout, int dtype, int add_identity, void *stream);

/* Input gradient of y = conv(GELU(pre)) with respect to `pre`: the input gradient above multiplied,
 * as it is stored, by GELU'(pre) (the chain-rule pass the reference leaves to autograd behind
 * models/convnext.py:389-391).  pre has the shape of dx; pre == NULL is o1d_dgrad(). */
int o1d_dgrad_act(const void *dy, const float *w, const void *pre,
                  const void *plan_host, const void *plan_dev, void *dx,
                  int N, int H, int W, int C, int K, int stride,
                  int layout, int dtype, int add_identity, void *stream);

/* Weight gradient (and bias gradient when db != NULL).  Replaces wgrad(dy, x, theta)
 * (kernels.cu:42-54, kernels.h:402-518) and the separate dy.sum([0,2,3]) pass
 * (dwoconv1d.py:66-67).  Deterministic: per-block partial sums go to `workspace`
 * (o1d_wgrad_workspace_bytes() bytes, caller-allocated, contents need no
 * initialisation) and are combined in a fixed order; no atomics. */
size_t o1d_wgrad_workspace_bytes(int N, int H, int W, int C, int K, int stride,
                                 int layout, int dtype);
int o1d_wgrad(const void *dy, const void *x,
              const void *plan_host, const void *plan_dev,
              float *dw, float *db, void *workspace, size_t workspace_bytes,
              int N, int H, int W, int C, int K, int stride,
              int layout, int dtype, void *stream);

/* o1d_wgrad() with a flag word: O1D_FLAG_GELU_INPUT makes `x` a pre-activation tensor to which exact
 * GELU is applied as it is loaded (the weight gradient of y = conv(GELU(x))). */
int o1d_wgrad_act(const void *dy, const void *x,
                  const void *plan_host, const void *plan_dev,
                  float *dw, float *db, void *workspace, size_t workspace_bytes,
                  int N, int H, int W, int C, int K, int stride,
                  int layout, int dtype, int flags, void *stream);

/* Weight gradient without a workspace argument, for callers that are not able to allocate
 * device memory at the call site (plugin sandboxes and framework hooks that forbid it,
 * processes whose memory pool is fixed at start-up, code running under an allocator lock).
 * It has no counterpart in the reference.  The per-block partial sums go to an array of
 * O1D_STATIC_SCRATCH_BYTES that is compiled into the library (each GPU that loads the
 * library keeps that much memory until the process exits).  The call allocates nothing
 * and frees nothing.  It tries the kernel families in the same order as o1d_wgrad() and
 * skips one whose partial sums exceed the array, so the result equals o1d_wgrad()'s bit
 * for bit when both take the same family (o1d_last_route() tells) and otherwise agrees
 * to rounding: the sums are then taken in a different order.
 *   - Shapes whose partial sums fit no family are refused with O1D_ERR_UNSUPPORTED and a
 *     message in o1d_last_error(); use o1d_wgrad() with your own workspace for those.
 *   - The first call on each device looks up the array's device address; make that first
 *     call outside of any CUDA stream capture.
 *   - All calls on a device share the one array, and it still holds the previous call's
 *     partial sums afterwards (nothing in it needs clearing: every slot a call reads it has
 *     written first).  Two calls that may run on the GPU at the same time — different
 *     streams, different threads — would overwrite each other's partial sums: serialise them. */
#define O1D_STATIC_SCRATCH_BYTES (4 * 1024 * 1024)
int o1d_wgrad_static(const void *dy, const void *x,
                     const void *plan_host, const void *plan_dev,
                     float *dw, float *db,
                     int N, int H, int W, int C, int K, int stride,
                     int layout, int dtype, void *stream);

/* LayerNorm over the contiguous channel axis of a channels-last tensor, y = (x - mean) /
 * sqrt(var + eps) * gamma + beta, optionally followed by exact (erf) GELU: the step that
 * follows every oriented convolution in the reference's blocks and stems
 * (models/convnext.py:28-56 LayerNorm, :183-189 stem LayerNorm+GELU, :309 block norm; the
 * reference calls F.layer_norm / F.gelu).  x, y: [rows, C] fp32 or bf16; gamma, beta: [C]
 * fp32; statistics in fp32, biased variance.  C must be a multiple of 4 (fp32) / 8 (bf16)
 * and at most 1024 (fp32) / 2048 (bf16).  Forward only. */
int o1d_layernorm_cl(const void *x, const float *gamma, const float *beta, void *y,
                     long long rows, int C, float eps, int dtype, int gelu, void *stream);

/* Backward of o1d_layernorm_cl (what autograd derives from F.layer_norm, and F.gelu after it when
 * gelu != 0, in the reference's training step, models/convnext.py:28-56,183-189): dx [rows, C] in
 * the element type, dgamma, dbeta [C] fp32.  dy is the gradient of the forward call's output.  The
 * row statistics are recomputed from x, so the forward pass keeps nothing but x.  beta is read only
 * when gelu != 0.  dgamma / dbeta are summed from per-CTA partials in a fixed order (bit-
 * reproducible).  C a multiple of 4 (fp32) / 8 (bf16), at most 512 (fp32) / 1024 (bf16).
 * workspace: o1d_layernorm_cl_bwd_workspace_bytes(rows, C) bytes, no initialisation needed. */
size_t o1d_layernorm_cl_bwd_workspace_bytes(long long rows, int C);
int o1d_layernorm_cl_bwd(const void *x, const void *dy, const float *gamma, const float *beta, void *dx,
                         float *dgamma, float *dbeta, void *workspace, size_t workspace_bytes,
                         long long rows, int C, float eps, int dtype, int gelu, void *stream);

/* Column sums of a channels-last matrix, out[c] = sum_r x[r, c] in fp32: the bias gradient that
 * autograd forms for the Linear layers on either side of the convolution in a block
 * (models/convnext.py:298-300,310,312).  x [rows, C] fp32 or bf16, C a multiple of 4 / 8; summed in
 * a fixed order.  workspace: o1d_colsum_workspace_bytes(rows, C, dtype) bytes, uninitialised. */
size_t o1d_colsum_workspace_bytes(long long rows, int C, int dtype);
int o1d_colsum(const void *x, float *out, void *workspace, size_t workspace_bytes, long long rows, int C,
               int dtype, void *stream);

/* Stem input projection: y[n,hw,o] = bias[o] + sum_c w[o,c] * x[n,c,hw], x an NCHW image
 * tensor with Cin <= 4 channels, y channels-last with Cout (a multiple of 8) channels: the
 * `x.permute(0,2,3,1)` + `nn.Linear(in_chans, 64)` that opens the reference's 1D stem
 * (models/convnext.py:143,170-176), in one pass.  x, y fp32 or bf16; w [Cout,Cin], bias [Cout]
 * (or NULL) fp32.  Forward only. */
int o1d_pointwise_in(const void *x, const float *w, const float *bias, void *y,
                     int N, int Cin, long long HW, int Cout, int dtype, void *stream);

/* Batched 2-D transpose [n, a, b] -> [n, b, a].  Replaces nhwc_to_nchw / nchw_to_nhwc
 * (kernels.cu:56-68, nhwc_utils.h:46-110): NHWC->NCHW is (n=N, a=H*W, b=C),
 * NCHW->NHWC is (n=N, a=C, b=H*W). */
int o1d_transpose(const void *in, void *out, int n, int a, int b, int dtype, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* O1D_H_ */
