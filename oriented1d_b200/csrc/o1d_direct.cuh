// "Direct" kernels: NHWC forward (any stride) and stride-1 input gradient for the cases where
// a zero-haloed input tile of a 32-byte channel chunk fits shared memory: small feature maps
// as whole images (several images per tile when they are tiny), large or strided ones (stems,
// dense-prediction sizes) as row/column tiles.  Any per-channel angle, any K <= 31.
//
//   * TMA (cp.async.bulk.tensor.4d, no multicast) brings a box CCs x TWp x THp x NI of the NHWC
//     tensor into one of two tile buffers; coordinates outside the image are zero-filled by the
//     hardware, which is the operator's zero padding: no tap needs a bounds test.
//   * a warp is 4 pixels x 8 channels (2 x 16 for 2-byte elements).  With the tile stored
//     [pixel][CCs] the bank of an access is 8*(pixel mod 4) + channel for 4-byte elements, so
//     the 32 lanes hit 32 banks whatever offsets the individual channels use: the per-channel
//     rasterised lines cost no bank conflicts and no divergence.
//   * each thread keeps its channel's taps (weight, tile offset) in registers for the whole
//     launch (a CTA stays on one channel chunk); taps that cannot reach inside the image are
//     dropped when the list is built.  Per output: KT x (address add, LDS, FMA), then one
//     32-byte-sector store per pixel.
//   * one CTA barrier per tile (buffer hand-back), tiles double-buffered.
//
// Compared with the tiled kernels (o1d_tiled.cuh) this spends one shared-memory load per FMA
// instead of one per 3-7, but has no restage / band-buffer passes and almost no barriers,
// which wins on small maps; at 56x56 the halo'd tile no longer fits and the tiled kernels run.
#pragma once

#include "o1d_common.cuh"
#include "o1d_tiled.cuh"   // mbarrier / TMA primitives, FastDiv

namespace o1d {

constexpr int kDirectThreads = 256;

struct DirectParams {
    int N, H, W, C, K, stride, P, Q;
    int CCs, nchunks;
    int Th, Tq, NI;               // output rows / columns / images per tile
    int THp, TWp;                 // input tile extents incl. halo
    int hh, hw;                   // halo rows / columns on each side
    int tiles_p, tiles_q, tiles_n, tiles_per_chunk;
    int tile_bytes, tile_stride;  // bytes of one box / spacing of the two buffers
    int off_taps_bytes, off_bar_bytes;
    int flip, add_identity;
    int segs_q;                   // column segments (of PLW*NPX pixels) per tile row
    FastDiv div_sq, div_thsq, div_tiles_q, div_tiles_pq;
};

// Load one element from a 32-bit shared-memory address plus a compile-time byte offset (the
// offset is an immediate of the load, so a thread's NPX pixels share one address register).
template <typename T, int IMM> __device__ __forceinline__ float ld_smem(uint32_t addr) {
    if constexpr (sizeof(T) == 4) {
        float v;
        asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(addr), "n"(IMM));
        return v;
    } else {
        unsigned short h;
        asm volatile("ld.shared.u16 %0, [%1+%2];" : "=h"(h) : "r"(addr), "n"(IMM));
        return __uint_as_float((uint32_t)h << 16);
    }
}

// KT: taps kept in registers per thread (>= the longest clipped tap list of any channel).
// NPX: outputs per thread and unit.  A warp works on one row segment of PLW*NPX pixels
// (PLW = 32/CCs pixel lanes); a thread's NPX pixels are PLW apart, so their tile addresses
// differ by the compile-time constant 32*sizeof(T)*STRIDE bytes and share one address add per
// tap, while the lanes of every single load still cover 32 different banks.
template <typename T, int KT, int NPX, int STRIDE>
__global__ void __launch_bounds__(kDirectThreads, 2)
direct_fprop_nhwc_kernel(const __grid_constant__ CUtensorMap tmap, const float *__restrict__ wgt,
                         const float *__restrict__ bias, const uint16_t *__restrict__ cls,
                         const int8_t *__restrict__ taps, T *__restrict__ y, const DirectParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw + p.off_bar_bytes);
    // per-channel compressed tap lists, built once: [CCs][KT] (weight, offset)
    float *s_w = reinterpret_cast<float *>(smem_raw + p.off_taps_bytes);
    int *s_off = reinterpret_cast<int *>(s_w + p.CCs * KT);

    const int tid = threadIdx.x;
    const int CCs = p.CCs;
    const int lane = tid & 31, warp = tid >> 5;
    const int cl = lane % CCs;                // channel within the chunk
    const int pl = lane / CCs;                // pixel lane within the warp
    const int PLW = 32 / CCs;                 // pixel lanes per warp
    constexpr int DELTA = 32 * (int)sizeof(T) * STRIDE;   // bytes between a thread's pixels
    const int groups = gridDim.x / p.nchunks; // CTAs per chunk
    const int chunk = blockIdx.x % p.nchunks;
    const int first = blockIdx.x / p.nchunks;
    const int c0 = chunk * CCs;
    const int my_tiles = (p.tiles_per_chunk - first + groups - 1) / groups;

    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // tap lists: thread i < CCs compresses channel c0+i (taps that can land inside the image)
    if (tid < CCs) {
        const int c = c0 + tid;
        const int8_t *t = taps + (size_t)cls[c] * p.K * 2;
        const int pad = p.K / 2;
        int n = 0;
        for (int k = 0; k < p.K; k++) {
            const int dh = t[2 * k], dw = t[2 * k + 1];
            const int adh = dh < 0 ? -dh : dh, adw = dw < 0 ? -dw : dw;
            if (adh > p.hh || adw > p.hw) continue;          // cannot reach the image
            const int kk = p.flip ? p.K - 1 - k : k;         // input gradient: mirrored line
            float wv = __ldg(wgt + (size_t)c * p.K + kk);
            if (p.add_identity && kk == pad) wv += 1.f;
            // tile offsets are kept in BYTES so that a tap is one 32-bit add + one LDS
            if (n < KT) { s_w[tid * KT + n] = wv; s_off[tid * KT + n] = (dh * p.TWp + dw) * CCs * (int)sizeof(T); n++; }
        }
        for (; n < KT; n++) { s_w[tid * KT + n] = 0.f; s_off[tid * KT + n] = 0; }
    }
    __syncthreads();
    float w[KT];
    int off[KT];
#pragma unroll
    for (int k = 0; k < KT; k++) { w[k] = s_w[cl * KT + k]; off[k] = s_off[cl * KT + k]; }
    const float bv = bias ? __ldg(bias + c0 + cl) : 0.f;

    auto tile_coords = [&](int it, int &n0, int &p0, int &q0) {
        const int t = first + it * groups;
        const int tn = p.div_tiles_pq.div(t), r = t - tn * (p.tiles_p * p.tiles_q);
        const int tp = p.div_tiles_q.div(r), tq = r - tp * p.tiles_q;
        n0 = tn * p.NI; p0 = tp * p.Th; q0 = tq * p.Tq;
    };
    auto issue = [&](int it) {
        int n0, p0, q0;
        tile_coords(it, n0, p0, q0);
        const int b = it & 1;
        mbar_expect_tx(&full[b], p.tile_bytes);
        tma_load_4d(smem_raw + (size_t)b * p.tile_stride, &tmap, &full[b], c0, q0 * p.stride - p.hw,
                    p0 * p.stride - p.hh, n0);
    };
    if (tid == 0) {
        if (my_tiles > 0) issue(0);
        if (my_tiles > 1) issue(1);
    }

    const int units = p.NI * p.Th * p.segs_q;           // (image, row, column segment)
    const int img_elems = p.THp * p.TWp * CCs;
    bool failed = false;
    for (int it = 0; it < my_tiles; it++) {
        int n0, p0, q0;
        tile_coords(it, n0, p0, q0);
        const int b = it & 1;
        if (!failed && !mbar_wait(&full[b], (it >> 1) & 1)) failed = true;
        const uint32_t tile_b = smem_u32(smem_raw) + b * p.tile_stride;   // shared address of the buffer
        for (int u = warp; u < units; u += kDirectThreads / 32) {
            const int img = p.div_thsq.div(u), r = u - img * (p.Th * p.segs_q);
            const int pr = p.div_sq.div(r), sq = r - pr * p.segs_q;
            const int pc0 = sq * (PLW * NPX) + pl;
            const int n = n0 + img, pp = p0 + pr;
            if (n >= p.N || pp >= p.P) continue;
            const uint32_t base = tile_b + (img * img_elems + ((pr * STRIDE + p.hh) * p.TWp + pc0 * STRIDE + p.hw) * CCs + cl) * (int)sizeof(T);
            float acc[NPX];
#pragma unroll
            for (int j = 0; j < NPX; j++) acc[j] = bv;
#pragma unroll
            for (int k = 0; k < KT; k++) {
                const uint32_t a = base + off[k];
                static_for<0, NPX>([&](auto j) { acc[j] = fmaf(w[k], ld_smem<T, j * DELTA>(a), acc[j]); });
            }
            T *yrow = y + (((size_t)n * p.P + pp) * p.Q + q0) * p.C + c0 + cl;
#pragma unroll
            for (int j = 0; j < NPX; j++) {
                const int pc = pc0 + PLW * j;
                if (pc < p.Tq && q0 + pc < p.Q) st(yrow + (size_t)pc * p.C, acc[j]);
            }
        }
        __syncthreads();                                   // everyone is done with buffer b
        if (tid == 0 && it + 2 < my_tiles) issue(it + 2);
    }
}

}  // namespace o1d
