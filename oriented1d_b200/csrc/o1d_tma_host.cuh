// Host-side construction of TMA tensor maps, shared by every kernel family that stages tiles
// with cp.async.bulk.tensor.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace o1d {

typedef CUresult (*PFN_encodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                    CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                    CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point lookup, so that the
// library does not link against libcuda and loads on machines without a driver.
inline PFN_encodeTiled encode_tiled_fn() {
    static PFN_encodeTiled fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (PFN_encodeTiled)p;
    }
    return fn;
}

// Outcome of building a tensor map: it was built, the request is outside what a tiled copy can
// describe (the caller moves on to the next kernel family), or the driver refused a request that
// should have been valid (reported to the caller as O1D_ERR_CUDA, never as a silent fallback).
enum : int { MAP_OK = 0, MAP_NA = 1, MAP_FAIL = 2 };

// CUresult of the last failed encode on this thread (-1: the driver entry point was not found).
inline int &last_encode_result() {
    thread_local int r = 0;
    return r;
}

static __global__ void context_probe_kernel() {}

// Makes the device's primary context current on the calling thread.  The encode below is a driver
// API call; on a thread that has only ever made runtime calls which need no context (a framework's
// backward worker, for instance) it can run before any context is bound.  Querying a kernel's
// attributes forces the runtime to bind one, is not a stream operation and is legal during capture.
inline void bind_primary_context() {
    cudaFuncAttributes a;
    (void)cudaFuncGetAttributes(&a, context_probe_kernel);
}

// 4-D tiled tensor map, dims/box innermost first, strides in bytes for dims 1..3.
inline int encode_map4(CUtensorMap *map, const void *base, int esize, const cuuint64_t (&dims)[4],
                       const cuuint64_t (&strides)[3], const cuuint32_t (&box)[4]) {
    if ((uintptr_t)base & 15) return MAP_NA;
    for (int i = 0; i < 4; i++)
        if (box[i] == 0 || box[i] > 256 || dims[i] == 0 || dims[i] > 0xffffffffull) return MAP_NA;
    for (int i = 0; i < 3; i++)
        if (strides[i] % 16 != 0 || strides[i] >= (1ull << 40)) return MAP_NA;
    if ((box[0] * (cuuint64_t)esize) % 16 != 0) return MAP_NA;
    thread_local bool bound = false;
    if (!bound) { bind_primary_context(); bound = true; }
    PFN_encodeTiled enc = encode_tiled_fn();
    if (!enc) { last_encode_result() = -1; return MAP_FAIL; }
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = CUDA_SUCCESS;
    for (int attempt = 0; attempt < 2; attempt++) {
        r = enc(map, esize == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r == CUDA_SUCCESS) return MAP_OK;
        bind_primary_context();
    }
    last_encode_result() = (int)r;
    return MAP_FAIL;
}

}  // namespace o1d
