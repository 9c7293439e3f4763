// Build shim around the reference's own specialised CUDA kernels.  BENCHMARK / TEST
// INFRASTRUCTURE ONLY: it is the "GPU baseline to beat", never part of the product path.
//
// It textually includes models/dwoconv1d_specialized/kernels/kernels.h and nhwc_utils.h
// from the reference checkout (path given with -I at compile time; no reference source is
// stored in this repository) and exports the launchers of the three kernels
// (kernels.h:511-548) and of the layout transpose (nhwc_utils.h:106-110) through a C ABI for
// the four ConvNeXt-T stage shapes, K=31, stride 1 (the reference compiles one module per
// (H, W, K, stride, pad) tuple, dwoconv1d_specialized_kernel.py:68-83).
#include <cuda_runtime.h>

#include "kernels.h"
#include "nhwc_utils.h"

namespace {
using Elem = float;
using Prm = ProblemParams<Elem>;

template <int HW>
void run_fprop(Elem *y, Elem *w, Elem *x, Elem *theta, int N, int C, cudaStream_t st) {
    SpecializedFpropKernel<Elem, SpecializedFpropProblem<HW, HW, 31, 1, 15>, Prm>::run(y, w, x, Prm(theta, N, C), st);
}
template <int HW>
void run_dgrad(Elem *dx, Elem *w, Elem *dy, Elem *theta, int N, int C, cudaStream_t st) {
    SpecializedDgradKernel<Elem, SpecializedDgradProblem<HW, HW, 31, 1, 15>, Prm>::run(dx, w, dy, Prm(theta, N, C), st);
}
template <int HW>
void run_wgrad(Elem *dw, Elem *dy, Elem *x, Elem *theta, int N, int C, cudaStream_t st) {
    SpecializedWgradKernel<Elem, SpecializedWgradProblem<HW, HW, 31, 1, 15>, Prm>::run(dw, dy, x, Prm(theta, N, C), st);
}
}  // namespace

#define O1D_REF_SWITCH(fn, ...)                 \
    switch (hw) {                               \
        case 56: fn<56>(__VA_ARGS__); break;    \
        case 28: fn<28>(__VA_ARGS__); break;    \
        case 14: fn<14>(__VA_ARGS__); break;    \
        case 7: fn<7>(__VA_ARGS__); break;      \
        default: return 1;                      \
    }                                           \
    return cudaGetLastError() == cudaSuccess ? 0 : 2;

extern "C" {
// NCHW fp32 tensors, H = W = hw in {56, 28, 14, 7}; returns 0, 1 (shape not built) or 2 (launch error)
int o1d_refgpu_fprop(int hw, float *y, float *w, float *x, float *theta, int N, int C, void *stream) {
    O1D_REF_SWITCH(run_fprop, y, w, x, theta, N, C, (cudaStream_t)stream)
}
int o1d_refgpu_dgrad(int hw, float *dx, float *w, float *dy, float *theta, int N, int C, void *stream) {
    O1D_REF_SWITCH(run_dgrad, dx, w, dy, theta, N, C, (cudaStream_t)stream)
}
int o1d_refgpu_wgrad(int hw, float *dw, float *dy, float *x, float *theta, int N, int C, void *stream) {
    O1D_REF_SWITCH(run_wgrad, dw, dy, x, theta, N, C, (cudaStream_t)stream)
}
// [n, a, b] -> [n, b, a]
int o1d_refgpu_transpose(int n, int a, int b, float *out, float *in, void *stream) {
    nab_to_nba<float>(n, a, b, out, in, (cudaStream_t)stream);
    return cudaGetLastError() == cudaSuccess ? 0 : 2;
}
}
