"""The allocation-free weight-gradient entry point, o1d_wgrad_static.

It exists for callers that cannot allocate device memory where they call the library
(sandboxed plugins, framework hooks, processes with a fixed memory pool): its partial sums
live in an array compiled into libo1d.so instead of a caller-provided workspace.  Here it is
called straight through the C ABI, twice in a row per case, and compared with o1d_wgrad on
the same device inputs.  The file name sorts last so that a run stopping at the first failure
has already run every other test."""
import pytest
import torch

import oriented1d_b200 as o1d
from oriented1d_b200 import _lib
from tests.util import TOL_WGRAD, angle_list

pytestmark = pytest.mark.gpu


def _call_static(dy, x, plan, dw, db, N, H, W, C, K, stride, nhwc, code):
    with torch.cuda.device(x.device):
        return _lib.lib.o1d_wgrad_static(dy.data_ptr(), x.data_ptr(), plan.host.data_ptr(),
                                         plan.on(x.device).data_ptr(), dw.data_ptr(), db.data_ptr(), N, H, W, C, K,
                                         stride, int(nhwc), code, torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("N,C,H,W,K,stride,nhwc,dtype,mode", [
    (6, 96, 56, 56, 31, 1, True, torch.float32, "rr"),       # stage shape, round-robin angles
    (4, 192, 28, 28, 31, 1, True, torch.bfloat16, "model"),  # block-wise angles, bf16
    (40, 768, 7, 7, 31, 1, True, torch.float32, "rr"),       # 7x7 plane kernels, two tiles of images
    (2, 64, 32, 48, 15, 2, True, torch.float32, "model+"),   # stem: stride 2
    (2, 24, 25, 40, 13, 1, False, torch.float32, "random"),  # general kernels, NCHW, odd size
])
def test_static_scratch_matches_workspace_entry_point(N, C, H, W, K, stride, nhwc, dtype, mode):
    dev = torch.device("cuda")
    g = torch.Generator(device="cpu").manual_seed(N * C + H)
    P, Q = -(-H // stride), -(-W // stride)
    xs, ys = ((N, H, W, C), (N, P, Q, C)) if nhwc else ((N, C, H, W), (N, C, P, Q))
    plan = o1d.Plan(angle_list(mode, C, seed=C), K)
    code = _lib.F32 if dtype == torch.float32 else _lib.BF16
    # everything the entry point touches is allocated here, before it is called
    dw = torch.empty((C, 1, 1, K), dtype=torch.float32, device=dev)
    db = torch.empty((C,), dtype=torch.float32, device=dev)
    for call in range(2):                       # two calls in a row share the built-in array
        x = torch.randn(xs, generator=g).to(dev).to(dtype)
        dy = torch.randn(ys, generator=g).to(dev).to(dtype)
        ref_dw, ref_db = o1d.wgrad(dy, x, plan, stride, nhwc, with_bias=True)
        ref_route = o1d.ops.last_route()
        dw.fill_(float("nan"))
        db.fill_(float("nan"))
        torch.cuda.synchronize()
        # what "allocates nothing" means, measured: neither the driver's free memory nor torch's
        # allocator moves across the call (after the first call on this device, which loads the
        # kernels and looks the array's address up)
        if call == 0:
            rc = _call_static(dy, x, plan, dw, db, N, H, W, C, K, stride, nhwc, code)
            assert rc == 0, (_lib.lib.o1d_strerror(rc), _lib.lib.o1d_last_error())
            torch.cuda.synchronize()
            dw.fill_(float("nan"))
            db.fill_(float("nan"))
            torch.cuda.synchronize()
        free0, torch0 = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        rc = _call_static(dy, x, plan, dw, db, N, H, W, C, K, stride, nhwc, code)
        assert rc == 0, (_lib.lib.o1d_strerror(rc), _lib.lib.o1d_last_error())
        static_route = o1d.ops.last_route()
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free0 and torch.cuda.memory_allocated() == torch0
        if static_route == ref_route:           # same kernels, same order of summation
            assert torch.equal(dw, ref_dw) and torch.equal(db, ref_db), call
        assert float((dw - ref_dw).abs().max()) <= TOL_WGRAD * float(ref_dw.abs().max()), call
        assert float((db - ref_db).abs().max()) <= TOL_WGRAD * float(ref_db.abs().max()), call
    assert o1d.ops.device_status() == 0


def test_static_scratch_refuses_what_does_not_fit():
    """A general-route shape whose partial sums exceed the built-in array gets a clear error."""
    dev = torch.device("cuda")
    N, C, H, W, K = 64, 256, 9, 9, 63            # general route: 74 slices * 256 ch * 64 floats > 4 MiB
    plan = o1d.Plan(angle_list("random", C, seed=1), K)
    x = torch.zeros((N, H, W, C), device=dev)
    dw = torch.empty((C, 1, 1, K), device=dev)
    db = torch.empty((C,), device=dev)
    rc = _call_static(x, x, plan, dw, db, N, H, W, C, K, 1, True, _lib.F32)
    assert rc == 2
    assert b"built-in array" in _lib.lib.o1d_last_error()
