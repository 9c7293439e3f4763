// "Direct" kernels: NHWC forward (stride 1 or 2) and stride-1 input gradient, weight gradient
// (stride 1 or 2) and stride-2 input gradient, all on zero-haloed input tiles of a 32-byte
// channel chunk in shared memory: small feature maps as whole images (several images per tile
// when they are tiny), large or strided ones (stems, dense-prediction sizes) as row/column
// tiles.  Any per-channel angle, any K <= 31.
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
// which wins on tiny maps, and they take every shape the tiled kernels do not (strides, sizes
// that are not multiples of 7 or 8, arbitrary angles, layers whose chunks hold a single line kind).
#pragma once

#include "o1d_common.cuh"
#include "o1d_tiled.cuh"   // mbarrier / TMA primitives, FastDiv

namespace o1d {

constexpr int kDirectThreads = 256;      // CTA size when two CTAs share an SM
constexpr int kDirectThreadsMax = 512;   // CTA size when the tiles leave room for one CTA per SM only

struct DirectParams {
    int N, H, W, C, K, stride, P, Q;
    int CCs, nchunks, chunk0;     // this launch covers chunks [chunk0, chunk0 + nchunks)
    int Th, Tq, NI;               // output rows / columns / images per tile
    int THp, TWp;                 // input tile extents incl. halo
    int hh, hw;                   // halo rows / columns on each side
    int tiles_p, tiles_q, tiles_n, tiles_per_chunk;
    int tile_bytes, tile_stride;  // bytes of one input box / of the buffer part that holds it
    int dy_bytes, buf_stride;     // weight gradient: bytes of one dy box; spacing of the two buffers (both ops)
    int off_taps_bytes, off_bar_bytes;
    int flip, add_identity;
    int segs_q;                   // column segments (of PLW*NPX pixels) per tile row
    int partial_off;              // weight gradient: first float of this range's partials
    FastDiv div_sq, div_thsq, div_tiles_q, div_tiles_pq;
};

// One launch covers up to kMaxChunkRanges channel-chunk ranges, each with its own tile shape,
// halo and tensor map (contiguous CTA index ranges): layers whose chunks reach differently far
// (the models' block-wise angle assignment) get small halos where the lines allow it without
// paying one launch per range.
constexpr int kMaxChunkRanges = 8;
struct DirectMulti {
    int n;
    int start[kMaxChunkRanges + 1];          // first CTA of each range; start[n] = grid
    DirectParams p[kMaxChunkRanges];
};
// Tensor maps travel in a parameter of their own: their address is taken (TMA wants a pointer),
// and a parameter whose address is taken is no longer read through constant-bank operands.
struct DirectMaps { CUtensorMap map[kMaxChunkRanges]; };

__device__ __forceinline__ int direct_range_of(const DirectMulti &mp, int cta) {
    int r = 0;
    while (r + 1 < mp.n && cta >= mp.start[r + 1]) r++;
    return r;
}

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
// MULTI: the launch holds several chunk ranges (parameters are then indexed by range at run time).
// PAIR (2-byte elements whose even/odd channel neighbours share their line): a thread owns two
// adjacent channels, loads them as one 32-bit word (half the shared-memory wavefronts of two
// 16-bit loads), widens both halves and runs two FMAs; a warp is then 4 pixels x 8 channel pairs.
// The CTA has 256 threads when two CTAs fit an SM and 512 when the tiles only leave room for one.
template <typename T, int KT, int NPX, int STRIDE, bool MULTI, bool PAIR>
__global__ void __launch_bounds__(kDirectThreadsMax, 1)
direct_fprop_nhwc_kernel(const DirectMulti mp, const __grid_constant__ DirectMaps maps, const float *__restrict__ wgt,
                         const float *__restrict__ bias, const uint16_t *__restrict__ cls,
                         const int8_t *__restrict__ taps, T *__restrict__ y) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int rng = MULTI ? direct_range_of(mp, blockIdx.x) : 0;
    const DirectParams &p = mp.p[rng];
    const CUtensorMap *tmap = &maps.map[rng];
    const int bid = blockIdx.x - mp.start[rng], gsz = mp.start[rng + 1] - mp.start[rng];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw + p.off_bar_bytes);
    // per-channel compressed tap lists, built once: [CCs][KT] (weight, offset)
    float *s_w = reinterpret_cast<float *>(smem_raw + p.off_taps_bytes);
    int *s_off = reinterpret_cast<int *>(s_w + p.CCs * KT);

    const int tid = threadIdx.x;
    const int CCs = p.CCs;
    const int lane = tid & 31, warp = tid >> 5, nwarps = (int)blockDim.x >> 5;
    static_assert(!PAIR || sizeof(T) == 2, "channel pairs are for 2-byte elements");
    constexpr int CPT = PAIR ? 2 : 1;         // channels per thread
    const int CL = CCs / CPT;                 // channel lanes per pixel
    const int cl = (lane % CL) * CPT;         // (first) channel of this thread within the chunk
    const int pl = lane / CL;                 // pixel lane within the warp
    const int PLW = 32 / CL;                  // pixel lanes per warp
    constexpr int DELTA = 32 * (int)sizeof(T) * CPT * STRIDE;   // bytes between a thread's pixels (PLW pixels)
    const int groups = gsz / p.nchunks;        // CTAs per chunk
    const int chunk = p.chunk0 + bid % p.nchunks;
    const int first = bid / p.nchunks;
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
    float w[KT], w2[PAIR ? KT : 1];
    int off[KT];
#pragma unroll
    for (int k = 0; k < KT; k++) {
        w[k] = s_w[cl * KT + k]; off[k] = s_off[cl * KT + k];
        if constexpr (PAIR) w2[k] = s_w[(cl + 1) * KT + k];      // same line, hence the same kept taps and offsets
    }
    const float bv = bias ? __ldg(bias + c0 + cl) : 0.f;
    const float bv2 = (PAIR && bias) ? __ldg(bias + c0 + cl + 1) : 0.f;

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
        tma_load_4d(smem_raw + (size_t)b * p.buf_stride, tmap, &full[b], c0, q0 * p.stride - p.hw,
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
        const uint32_t tile_b = smem_u32(smem_raw) + b * p.buf_stride;    // shared address of the buffer
        for (int u = warp; u < units; u += nwarps) {
            const int img = p.div_thsq.div(u), r = u - img * (p.Th * p.segs_q);
            const int pr = p.div_sq.div(r), sq = r - pr * p.segs_q;
            const int pc0 = sq * (PLW * NPX) + pl;
            const int n = n0 + img, pp = p0 + pr;
            if (n >= p.N || pp >= p.P) continue;
            const uint32_t base = tile_b + (img * img_elems + ((pr * STRIDE + p.hh) * p.TWp + pc0 * STRIDE + p.hw) * CCs + cl) * (int)sizeof(T);
            float acc[NPX], acc2[PAIR ? NPX : 1];
#pragma unroll
            for (int j = 0; j < NPX; j++) { acc[j] = bv; if constexpr (PAIR) acc2[j] = bv2; }
#pragma unroll
            for (int k = 0; k < KT; k++) {
                const uint32_t a = base + off[k];
                static_for<0, NPX>([&](auto j) {
                    if constexpr (PAIR) {
                        uint32_t word;
                        asm volatile("ld.shared.b32 %0, [%1+%2];" : "=r"(word) : "r"(a), "n"(j * DELTA));
                        acc[j] = fmaf(w[k], __uint_as_float(word << 16), acc[j]);
                        acc2[j] = fmaf(w2[k], __uint_as_float(word & 0xffff0000u), acc2[j]);
                    } else {
                        acc[j] = fmaf(w[k], ld_smem<T, j * DELTA>(a), acc[j]);
                    }
                });
            }
            T *yrow = y + (((size_t)n * p.P + pp) * p.Q + q0) * p.C + c0 + cl;
#pragma unroll
            for (int j = 0; j < NPX; j++) {
                const int pc = pc0 + PLW * j;
                if (pc < p.Tq && q0 + pc < p.Q) {
                    if constexpr (PAIR) {
                        __nv_bfloat162 h = __floats2bfloat162_rn(acc[j], acc2[j]);
                        *reinterpret_cast<__nv_bfloat162 *>(yrow + (size_t)pc * p.C) = h;
                    } else {
                        st(yrow + (size_t)pc * p.C, acc[j]);
                    }
                }
            }
        }
        __syncthreads();                                   // everyone is done with buffer b
        if (tid == 0 && it + 2 < my_tiles) issue(it + 2);
    }
}


constexpr int kDirectPartialStride = 32;   // floats per channel in a partial: up to 31 taps + bias-gradient sum

// Weight gradient with the same tiles and the same thread layout as the forward kernel:
//   dw[c][k] = sum over (n, p, q) of x[n, p*s+dh_k, q*s+dw_k, c] * dy[n, p, q, c],  db[c] = sum dy.
// A second TMA box per tile brings dy[NI][Th][Tq][CCs]; out-of-range rows, columns and images of
// both boxes are hardware zero fill, so edge tiles need no masks beyond the segment overrun.
// Each thread keeps one accumulator per kept tap of its channel for the whole launch; at the
// end the accumulators are added across the pixel lanes of a warp (shuffles), across the warps
// (shared memory, warp order) and written as one partial per (CTA, channel);
// direct_wgrad_final_kernel adds the partials of a chunk's CTAs in CTA order.  No atomics:
// bit-reproducible.  (Reference: models/dwoconv1d/kernels/kernels.h:402-518, 31 atomicAdd per block.)
template <typename T, int KT, int NPX, int STRIDE, bool MULTI>
__global__ void __launch_bounds__(kDirectThreadsMax, 1)
direct_wgrad_nhwc_kernel(const DirectMulti mp, const __grid_constant__ DirectMaps maps,
                         const __grid_constant__ DirectMaps dym,
                         const uint16_t *__restrict__ cls, const int8_t *__restrict__ taps,
                         float *__restrict__ partial) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int rng = MULTI ? direct_range_of(mp, blockIdx.x) : 0;
    const DirectParams &p = mp.p[rng];
    const CUtensorMap *tmap_x = &maps.map[rng], *tmap_dy = &dym.map[rng];
    const int bid = blockIdx.x - mp.start[rng], gsz = mp.start[rng + 1] - mp.start[rng];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw + p.off_bar_bytes);
    int *s_off = reinterpret_cast<int *>(smem_raw + p.off_taps_bytes);   // [CCs][KT] byte offsets

    const int tid = threadIdx.x;
    const int CCs = p.CCs;
    const int lane = tid & 31, warp = tid >> 5, nwarps = (int)blockDim.x >> 5;
    const int cl = lane % CCs, pl = lane / CCs;
    const int PLW = 32 / CCs;
    constexpr int DELTA = 32 * (int)sizeof(T) * STRIDE;
    constexpr int DDY = 32 * (int)sizeof(T);              // dy pixels of one thread are PLW apart too
    const int groups = gsz / p.nchunks;
    const int chunk = p.chunk0 + bid % p.nchunks;
    const int first = bid / p.nchunks;
    const int c0 = chunk * CCs;
    const int my_tiles = (p.tiles_per_chunk - first + groups - 1) / groups;

    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (tid < CCs) {       // same compression as the forward kernel: slot n <-> n-th tap that can reach the image
        const int8_t *t = taps + (size_t)cls[c0 + tid] * p.K * 2;
        int n = 0;
        for (int k = 0; k < p.K; k++) {
            const int dh = t[2 * k], dw = t[2 * k + 1];
            const int adh = dh < 0 ? -dh : dh, adw = dw < 0 ? -dw : dw;
            if (adh > p.hh || adw > p.hw) continue;
            if (n < KT) s_off[tid * KT + n++] = (dh * p.TWp + dw) * CCs * (int)sizeof(T);
        }
        for (; n < KT; n++) s_off[tid * KT + n] = 0;
    }
    __syncthreads();
    int off[KT];
    float acc[KT];
#pragma unroll
    for (int k = 0; k < KT; k++) { off[k] = s_off[cl * KT + k]; acc[k] = 0.f; }
    float acc_db = 0.f;
    // The slack behind each input tile is read (times a zero dy) by the overrun pixels of the
    // last row segment: it must hold finite numbers.  TMA never writes there.
    for (int b = 0; b < 2; b++)
        for (int i = p.tile_bytes / 4 + tid; i < p.tile_stride / 4; i += (int)blockDim.x)
            reinterpret_cast<uint32_t *>(smem_raw + (size_t)b * p.buf_stride)[i] = 0u;
    __syncthreads();

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
        unsigned char *buf = smem_raw + (size_t)b * p.buf_stride;
        mbar_expect_tx(&full[b], p.tile_bytes + p.dy_bytes);
        tma_load_4d(buf, tmap_x, &full[b], c0, q0 * p.stride - p.hw, p0 * p.stride - p.hh, n0);
        tma_load_4d(buf + p.tile_stride, tmap_dy, &full[b], c0, q0, p0, n0);
    };
    if (tid == 0) {
        if (my_tiles > 0) issue(0);
        if (my_tiles > 1) issue(1);
    }

    const int units = p.NI * p.Th * p.segs_q;
    const int img_elems = p.THp * p.TWp * CCs;
    bool failed = false;
    for (int it = 0; it < my_tiles; it++) {
        int n0, p0, q0;
        tile_coords(it, n0, p0, q0);
        const int b = it & 1;
        if (!failed && !mbar_wait(&full[b], (it >> 1) & 1)) failed = true;
        const uint32_t tile_b = smem_u32(smem_raw) + b * p.buf_stride;
        const uint32_t dy_b = tile_b + p.tile_stride;
        for (int u = warp; u < units; u += nwarps) {
            const int img = p.div_thsq.div(u), r = u - img * (p.Th * p.segs_q);
            const int pr = p.div_sq.div(r), sq = r - pr * p.segs_q;
            const int pc0 = sq * (PLW * NPX) + pl;
            if (n0 + img >= p.N || p0 + pr >= p.P) continue;      // zero-filled part of an edge tile
            const uint32_t gaddr = dy_b + (((img * p.Th + pr) * p.Tq + pc0) * CCs + cl) * (int)sizeof(T);
            float g[NPX];
            static_for<0, NPX>([&](auto j) {
                // columns past the tile belong to the next row of the box
                g[j] = (pc0 + PLW * j < p.Tq) ? ld_smem<T, j * DDY>(gaddr) : 0.f;
                acc_db += g[j];
            });
            const uint32_t base = tile_b + (img * img_elems + ((pr * STRIDE + p.hh) * p.TWp + pc0 * STRIDE + p.hw) * CCs + cl) * (int)sizeof(T);
#pragma unroll
            for (int k = 0; k < KT; k++) {
                const uint32_t a = base + off[k];
                static_for<0, NPX>([&](auto j) { acc[k] = fmaf(ld_smem<T, j * DELTA>(a), g[j], acc[k]); });
            }
        }
        __syncthreads();
        if (tid == 0 && it + 2 < my_tiles) issue(it + 2);
    }

    // ---- reduction: pixel lanes (shuffles), then warps (shared memory, fixed order) ----------
#pragma unroll
    for (int k = 0; k < KT; k++)
        for (int d = CCs; d < 32; d <<= 1) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], d);
    for (int d = CCs; d < 32; d <<= 1) acc_db += __shfl_xor_sync(0xffffffffu, acc_db, d);
    float *red = reinterpret_cast<float *>(smem_raw);        // [warps][CCs][32]; the tiles are done with
    if (pl == 0) {
        float *r = red + (warp * CCs + cl) * kDirectPartialStride;
#pragma unroll
        for (int k = 0; k < KT; k++) r[k] = acc[k];
        r[kDirectPartialStride - 1] = acc_db;
    }
    __syncthreads();
    for (int e = tid; e < CCs * kDirectPartialStride; e += (int)blockDim.x) {
        const int k = e % kDirectPartialStride;
        float sum = 0.f;
        if (k < KT || k == kDirectPartialStride - 1)
            for (int w = 0; w < nwarps; w++) sum += red[w * CCs * kDirectPartialStride + e];
        partial[p.partial_off + (size_t)bid * CCs * kDirectPartialStride + e] = sum;
    }
}

// dw[c][k] = sum over the CTAs of c's chunk, in CTA order, of their partial for the slot tap k was kept in
// (0 if the tap cannot reach inside an image of this size).
__global__ void direct_wgrad_final_kernel(const DirectMulti mp, const float *__restrict__ partial,
                                          const uint16_t *__restrict__ cls, const int8_t *__restrict__ taps,
                                          float *__restrict__ dw, float *__restrict__ db, int C, int K) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= C * (K + 1)) return;
    const int c = idx / (K + 1), k = idx % (K + 1);
    if (k == K && db == nullptr) return;
    const int CCs = mp.p[0].CCs;
    int r = 0;
    while (r + 1 < mp.n && c / CCs >= mp.p[r + 1].chunk0) r++;
    const DirectParams &p = mp.p[r];
    const int chunk = c / CCs - p.chunk0, cl = c % CCs;
    const int groups = (mp.start[r + 1] - mp.start[r]) / p.nchunks;
    int slot = kDirectPartialStride - 1;
    if (k < K) {
        const int8_t *t = taps + (size_t)cls[c] * K * 2;
        slot = 0;
        bool kept = false;
        for (int i = 0; i <= k; i++) {
            const int dh = t[2 * i], dwv = t[2 * i + 1];
            const bool in = (dh < 0 ? -dh : dh) <= p.hh && (dwv < 0 ? -dwv : dwv) <= p.hw;
            if (i < k) slot += in ? 1 : 0; else kept = in;
        }
        if (!kept) slot = -1;
    }
    float sum = 0.f;
    for (int g = 0; g < groups && slot >= 0; g++)
        sum += partial[p.partial_off + ((size_t)(g * p.nchunks + chunk) * CCs + cl) * kDirectPartialStride + slot];
    if (k == K) db[c] = sum; else dw[(size_t)c * K + k] = sum;
}

constexpr int kDgrad2Slots = 16;   // merged taps per parity class (a line of 31 offsets has at most 16 of one parity)

// Input gradient for stride 2, gathered per output pixel:
//   dx[n,h,w,c] = sum over taps k with (h-dh_k, w-dw_k) both even of w'[c,k] * dy[n,(h-dh_k)/2,(w-dw_k)/2,c].
// Output pixels split into four parity classes (h&1, w&1); class (ph,pw) only sees taps with
// dh_k = ph, dw_k = pw (mod 2), for which (h-dh_k)/2 = a - e_k with h = 2a+ph, e_k = (dh_k-ph)/2.
// So the kernel is the forward kernel's tile machinery run over the dy grid (a, b) with
// stride 1 and a halo of ceil(max|d|/2): a TMA box of dy per tile (zero fill outside is the
// range test), and per class a short tap list (weight, byte offset -(e*TWp+f)*32) in registers.
// The four classes are four passes over the tile; passes whose longest list in this CTA's
// channel chunk is 0 or <= 8 run a shorter unrolled loop.  p.H/p.W are the dy grid extents here;
// Hx, Wx those of dx.  (Reference: models/dwoconv1d/kernels/kernels.h:312-399 tests `%` and `/`
// by the stride for every tap of every pixel.)
template <typename T, int NPX, bool MULTI>
__global__ void __launch_bounds__(kDirectThreadsMax, 1)
direct_dgrad2_nhwc_kernel(const DirectMulti mp, const __grid_constant__ DirectMaps maps, const float *__restrict__ wgt,
                          const uint16_t *__restrict__ cls, const int8_t *__restrict__ taps,
                          T *__restrict__ dx, int Hx, int Wx) {
    constexpr int KS = kDgrad2Slots;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int rng = MULTI ? direct_range_of(mp, blockIdx.x) : 0;
    const DirectParams &p = mp.p[rng];
    const CUtensorMap *tmap = &maps.map[rng];
    const int bid = blockIdx.x - mp.start[rng], gsz = mp.start[rng + 1] - mp.start[rng];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw + p.off_bar_bytes);
    float *s_w = reinterpret_cast<float *>(smem_raw + p.off_taps_bytes);     // [4][CCs][KS]
    int *s_off = reinterpret_cast<int *>(s_w + 4 * p.CCs * KS);               // [4][CCs][KS]
    int *s_len = s_off + 4 * p.CCs * KS;                                      // [4][CCs]

    const int tid = threadIdx.x;
    const int CCs = p.CCs;
    const int lane = tid & 31, warp = tid >> 5, nwarps = (int)blockDim.x >> 5;
    const int cl = lane % CCs, pl = lane / CCs;
    const int PLW = 32 / CCs;
    constexpr int DELTA = 32 * (int)sizeof(T);
    const int groups = gsz / p.nchunks;
    const int chunk = p.chunk0 + bid % p.nchunks;
    const int first = bid / p.nchunks;
    const int c0 = chunk * CCs;
    const int my_tiles = (p.tiles_per_chunk - first + groups - 1) / groups;

    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (tid < CCs) {
        const int c = c0 + tid;
        const int8_t *t = taps + (size_t)cls[c] * p.K * 2;
        const int pad = p.K / 2;
        int n[4] = {0, 0, 0, 0};
        for (int k = 0; k < p.K; k++) {
            const int dh = t[2 * k], dw = t[2 * k + 1];
            const int ph = dh & 1, pw = dw & 1, q = ph * 2 + pw;
            const int e = (dh - ph) >> 1, f = (dw - pw) >> 1;          // exact: dh-ph and dw-pw are even
            float wv = __ldg(wgt + (size_t)c * p.K + k);
            if (p.add_identity && k == pad) wv += 1.f;
            const int off = -(e * p.TWp + f) * CCs * (int)sizeof(T);
            float *lw = s_w + (q * CCs + tid) * KS;
            int *lo = s_off + (q * CCs + tid) * KS;
            int hit = -1;
            for (int i = 0; i < n[q]; i++) if (lo[i] == off) hit = i;   // colliding taps add their weights
            if (hit >= 0) lw[hit] += wv;
            else if (n[q] < KS) { lw[n[q]] = wv; lo[n[q]] = off; n[q]++; }
        }
        for (int q = 0; q < 4; q++) {
            for (int i = n[q]; i < KS; i++) { s_w[(q * CCs + tid) * KS + i] = 0.f; s_off[(q * CCs + tid) * KS + i] = 0; }
            s_len[q * CCs + tid] = n[q];
        }
    }
    __syncthreads();

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
        tma_load_4d(smem_raw + (size_t)b * p.buf_stride, tmap, &full[b], c0, q0 - p.hw, p0 - p.hh, n0);
    };
    if (tid == 0) {
        if (my_tiles > 0) issue(0);
        if (my_tiles > 1) issue(1);
    }

    const int units = p.NI * p.Th * p.segs_q;
    const int img_elems = p.THp * p.TWp * CCs;
    bool failed = false;
    for (int it = 0; it < my_tiles; it++) {
        int n0, p0, q0;
        tile_coords(it, n0, p0, q0);
        const int b = it & 1;
        if (!failed && !mbar_wait(&full[b], (it >> 1) & 1)) failed = true;
        const uint32_t tile_b = smem_u32(smem_raw) + b * p.buf_stride;
        for (int q = 0; q < 4; q++) {
            const int ph = q >> 1, pw = q & 1;
            int lmax = 0;
            for (int i = 0; i < CCs; i++) lmax = max(lmax, s_len[q * CCs + i]);    // uniform over the CTA
            float w[KS];
            int off[KS];
#pragma unroll
            for (int k = 0; k < KS; k++) { w[k] = s_w[(q * CCs + cl) * KS + k]; off[k] = s_off[(q * CCs + cl) * KS + k]; }
            auto pass = [&](auto nslots) {
                constexpr int NS = decltype(nslots)::value;
                for (int u = warp; u < units; u += nwarps) {
                    const int img = p.div_thsq.div(u), r = u - img * (p.Th * p.segs_q);
                    const int pr = p.div_sq.div(r), sq = r - pr * p.segs_q;
                    const int pc0 = sq * (PLW * NPX) + pl;
                    const int n = n0 + img, h = 2 * (p0 + pr) + ph;
                    if (n >= p.N || h >= Hx) continue;
                    const uint32_t base = tile_b + (img * img_elems + ((pr + p.hh) * p.TWp + pc0 + p.hw) * CCs + cl) * (int)sizeof(T);
                    float acc[NPX];
#pragma unroll
                    for (int j = 0; j < NPX; j++) acc[j] = 0.f;
#pragma unroll
                    for (int k = 0; k < NS; k++) {
                        const uint32_t a = base + off[k];
                        static_for<0, NPX>([&](auto j) { acc[j] = fmaf(w[k], ld_smem<T, j * DELTA>(a), acc[j]); });
                    }
                    T *row = dx + (((size_t)n * Hx + h) * Wx) * p.C + c0 + cl;
#pragma unroll
                    for (int j = 0; j < NPX; j++) {
                        const int pc = pc0 + PLW * j, wx = 2 * (q0 + pc) + pw;
                        if (pc < p.Tq && wx < Wx) st(row + (size_t)wx * p.C, acc[j]);
                    }
                }
            };
            if (lmax == 0) pass(std::integral_constant<int, 0>{});
            else if (lmax <= KS / 2) pass(std::integral_constant<int, KS / 2>{});
            else pass(std::integral_constant<int, KS>{});
        }
        __syncthreads();
        if (tid == 0 && it + 2 < my_tiles) issue(it + 2);
    }
}

}  // namespace o1d
