// Build shim around the reference's own CPU operator.  TEST INFRASTRUCTURE ONLY.
//
// It textually includes models/dwoconv1d_reference/kernels/kernels.cpp from the
// reference checkout (path given with -I at compile time; no reference source is
// stored in this repository) and exports its three loops and its autograd function
// through a C ABI, so that Python can call them with numpy arrays via ctypes.
//
// Two things in that file stop it running on host tensors as written:
//   * every entry point begins with CHECK_CUDA(x) (kernels.cpp:12-14, :22-23), a
//     TORCH_CHECK on x.is_cuda();
//   * each loop announces itself with printf (kernels.cpp:29, :66, :103).
// Both are neutralised from the outside: the torch headers are included first (their
// include guards make the reference's own includes no-ops), then TORCH_CHECK and
// printf are redefined to nothing before the reference file is pulled in.  The
// arithmetic is untouched.
#include <torch/extension.h>
#include <cuda.h>
#include <cuda_runtime.h>
#include <ATen/cuda/CUDAContext.h>
#include <torch/torch.h>
#include <cstdio>
#include <cstring>

#undef TORCH_CHECK
#define TORCH_CHECK(...) ((void)0)
#define printf(...) ((void)0)
#include "kernels.cpp"   // resolved through -I<reference>/models/dwoconv1d_reference/kernels
#undef printf

namespace {
torch::Tensor wrap(const float *p, std::initializer_list<int64_t> shape) {
    return torch::from_blob(const_cast<float *>(p), shape, torch::kFloat32).clone();
}
void emit(const torch::Tensor &t, float *out) {
    auto c = t.contiguous();
    std::memcpy(out, c.data_ptr<float>(), sizeof(float) * c.numel());
}
}  // namespace

extern "C" {

// template_fprop<float>: kernels.cpp:20-55
int o1d_ref_fprop(const float *x, const float *w, const float *theta, float *y,
                  int N, int C, int H, int W, int K, int stride) {
    auto out = template_fprop<float>(wrap(x, {N, C, H, W}), wrap(w, {C, 1, 1, K}),
                                     wrap(theta, {C}), K, stride, K / 2);
    emit(out, y);
    return 0;
}

// template_dgrad<float>: kernels.cpp:57-93
int o1d_ref_dgrad(const float *dy, const float *w, const float *theta, float *dx,
                  int N, int C, int P, int Q, int K, int stride) {
    auto out = template_dgrad<float>(wrap(dy, {N, C, P, Q}), wrap(w, {C, 1, 1, K}),
                                     wrap(theta, {C}), K, stride, K / 2);
    emit(out, dx);
    return 0;
}

// template_wgrad<float>: kernels.cpp:95-129
int o1d_ref_wgrad(const float *dy, const float *x, const float *theta, float *dw,
                  int N, int C, int H, int W, int K, int stride) {
    const int P = H / stride, Q = W / stride;
    auto out = template_wgrad<float>(wrap(dy, {N, C, P, Q}), wrap(x, {N, C, H, W}),
                                     wrap(theta, {C}), K, stride, K / 2);
    emit(out, dw);
    return 0;
}

// template_dwoconv1d<float> (the autograd function, kernels.cpp:141-203): forward with
// the reference's resid / bias / nhwc handling, then backward with upstream gradient dy.
// x and dy are in the module's layout (NHWC when nhwc != 0).  db may be null.
int o1d_ref_module(const float *x, const float *w, const float *theta, const float *bias,
                   const float *dy, float *y, float *dx, float *dw, float *db,
                   int N, int C, int H, int W, int K, int stride, int nhwc, int with_bias,
                   int with_resid) {
    const int P = H / stride, Q = W / stride;
    auto xt = nhwc ? wrap(x, {N, H, W, C}) : wrap(x, {N, C, H, W});
    auto dyt = nhwc ? wrap(dy, {N, P, Q, C}) : wrap(dy, {N, C, P, Q});
    auto wt = wrap(w, {C, 1, 1, K});
    auto tt = wrap(theta, {C});
    auto bt = with_bias ? wrap(bias, {C}) : torch::zeros({0});
    auto rt = torch::zeros({0});
    if (with_resid) {   // same delta the Python module builds (dwoconv1d.py:136-141)
        rt = torch::zeros({C, 1, 1, K});
        rt.index_put_({torch::indexing::Slice(), 0, 0, K / 2}, 1.0f);
    }
    xt.requires_grad_(true);
    wt.requires_grad_(true);
    if (with_bias) bt.requires_grad_(true);
    auto yt = template_dwoconv1d<float>(xt, wt, tt, bt, rt, with_bias != 0, with_resid != 0,
                                        nhwc != 0, K, stride, K / 2);
    emit(yt, y);
    yt.backward(dyt);
    emit(xt.grad(), dx);
    emit(wt.grad(), dw);
    if (with_bias && db) emit(bt.grad(), db);
    return 0;
}

}  // extern "C"
