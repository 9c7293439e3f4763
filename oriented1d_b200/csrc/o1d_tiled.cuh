// Tiled kernels for the common case: stride 1, K <= 31, every channel on one of the eight
// canonical lines, NHWC.  One persistent CTA per SM walks work items (image n, chunk of CC
// channels):
//
//   1. TMA (cp.async.bulk.tensor, 4-D box CC x W x BR x 1 over the NHWC tensor) streams the
//      item's row bands into a ring of staging buffers; the producer runs NSTG bands ahead,
//      across item boundaries, so HBM reads overlap the arithmetic of the previous item.
//   2. "restage": each band is re-indexed into one fp32 plane per channel in (line, position)
//      coordinates (o1d_lines.cuh) with zero gaps between lines, so that every canonical
//      line becomes one of three base shapes and no tap needs a bounds test.
//   3. compute: a thread owns a segment of R consecutive outputs along the line direction,
//      loads each needed input once into a register window and reuses it for all taps of
//      that line row (1 shared-memory load per ~3-7 FMAs instead of 1 per FMA).  Warps are
//      uniform in base shape, so there is no divergence and offsets are immediates.
//   4. forward: outputs go through a small planar staging buffer and leave as 128-bit NHWC
//      stores, with bias added on the way.
//      weight gradient: the same staging buffer is filled the other way round (dy band,
//      128-bit NHWC loads), each thread multiplies its register window with its R dy values
//      into one accumulator per tap and keeps accumulating over bands and images; when the
//      CTA moves to another channel chunk the accumulators are reduced across threads in a
//      fixed order and written as one partial per (CTA, chunk); a second kernel adds the
//      partials in CTA order.  No atomics anywhere: results are bit-reproducible.
//
// The reference kernels (models/dwoconv1d_specialized/kernels/kernels.h:201-291, :388-509)
// give each block one (n, c) plane band, re-read the halo rows per band (up to 15x read
// amplification at 56x56), redo sincosf + float->int + four compares per tap, and finish
// the weight gradient with 31 fp32 atomicAdd per block.
#pragma once

#include <cuda.h>

#include <type_traits>

#include "o1d_common.cuh"
#include "o1d_lines.cuh"

namespace o1d {

constexpr int kTiledThreads = 512;
constexpr int kMaxStages = 8;
constexpr int kMaxCC = 64;
constexpr int kZeroFloats = 64;              // block of zeros a missing line is redirected to
constexpr int kHaloLines = 10;               // zero lines around a plane that make every line exist (largest |dl|)
constexpr uint32_t kSpinLimit = 1u << 22;    // mbarrier polls before giving up
constexpr int kPartialStride = 32;           // floats per channel in a weight-gradient partial:
                                             // 31 stored taps + the bias-gradient sum

enum : int { OP_FPROP = 0, OP_WGRAD = 1 };

// Device-side failure flag (a TMA wait that ran out of polls).  Read with o1d_device_status().
__device__ int g_o1d_device_error = 0;

struct FastDiv {   // q = n / d for n*d < 2^32
    uint32_t mul, d;
    __host__ __device__ static FastDiv make(uint32_t d_) { return FastDiv{(uint32_t)(0x100000000ull / d_) + 1u, d_}; }
    __device__ __forceinline__ uint32_t div(uint32_t n) const { return d == 1 ? n : __umulhi(n, mul); }
};

struct TiledParams {
    int N, H, W, C, K;
    int CC, nchunks, total_items;
    int R, BR, NB, NSTG;
    int pitch_n, pitch_t;         // line pitch of non-transposed / transposed planes (floats)
    int plane_stride;             // floats between channel planes
    int plane_base;               // index of (line 0, position 0) of channel 0's plane
    int halo;                     // zero lines before the first and after every plane (0: lines are bounds-checked)
    int grp;                      // restage: bands copied between CTA barriers (stages handed back together)
    int out_pitch_n, out_pitch_t, out_plane_stride;
    int nseg_line, nseg_diag;     // segments per channel per band
    int flip, add_identity;
    int act;                      // 1: the planes hold GELU(x) (applied while restaging)
    int rezero;                   // planes must be cleared per item (H != W)
    int TR;                       // restage/store: rows of a band the movers cover per pass
    int max_visits;               // weight gradient: partial slots per CTA
    int order;                    // 0: image-major items (item = cta + i*grid), 1: chunk-major ranges
    // shared memory layout, in floats from the start of dynamic smem
    int off_planar, off_zero, off_out, off_wts, off_misc;
    int off_stage_bytes, stage_bytes, stage_stride, off_bar_bytes;
    int zero_floats_total;        // floats to clear at kernel start (planar + zero block)
    FastDiv div_gv, div_w, div_nseg_line, div_nseg_diag, div_br, div_wline, div_wdiag, div_chunks, div_nb, div_n;
};

template <int I, int N, typename F>
__device__ __forceinline__ void static_for(F &&f) {
    if constexpr (I < N) {
        f(std::integral_constant<int, I>{});
        static_for<I + 1, N>(f);
    }
}

// ---- mbarrier / TMA primitives ------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: returns false (and raises the device flag) if the data never arrives.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, uint32_t limit = kSpinLimit) {
    for (uint32_t i = 0; i < limit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(&g_o1d_device_error, 1);
    return false;
}

// Self-test of that failure path: one warp waits, with a small poll limit, on an mbarrier that no
// thread and no copy will ever complete.  The wait must run out, raise the device flag and let
// the kernel return normally (no trap, no hang); *gave_up reports that it did.
__global__ void wait_timeout_selftest_kernel(uint32_t limit, int *gave_up) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    const bool ok = mbar_wait(&bar, 0, limit);
    if (threadIdx.x == 0) *gave_up = ok ? 0 : 1;
}
__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

// ---- segment evaluation --------------------------------------------------------------
// AXIS / SLANT: R outputs at (line, pos0 .. pos0+R-1).  `sm` is the float view of shared
// memory, `at0` the index of (line, pos0) in the channel plane.  CHECK = false when every
// line the segment touches is known to exist (no redirect to the zero block).
//   forward:          acc[o]  += w[k] * x(line+dl_k, pos0+o+dp_k)
//   weight gradient:  acc[k]  += sum_o x(line+dl_k, pos0+o+dp_k) * g[o]
template <int OP, int KIND, int JH, int R, bool CHECK>
__device__ __forceinline__ void seg_line(const float *__restrict__ sm, int at0, int pitch, int nlines,
                                         int zero_idx, int line,
                                         const float (&w)[OP == OP_FPROP ? kMaxTaps : R],
                                         float (&acc)[OP == OP_FPROP ? R : kMaxTaps]) {
    using P = LP<KIND, JH>;
    static_for<0, P::p.nrows>([&](auto ri) {
        constexpr int r = decltype(ri)::value;
        constexpr int d = P::p.row_d[r], lo = P::p.row_lo[r], hi = P::p.row_hi[r];
        constexpr int WN = hi - lo + R;
        int src = at0 + d * pitch + lo;
        if (CHECK && d != 0) src = ((unsigned)(line + d) < (unsigned)nlines) ? src : zero_idx;
        float win[WN];
#pragma unroll
        for (int i = 0; i < WN; i++) win[i] = sm[src + i];
        static_for<0, P::p.ntaps>([&](auto ti) {
            constexpr int t = decltype(ti)::value;
            if constexpr (P::p.tap_row[t] == r) {
                constexpr int off = P::p.tap_dp[t] - lo, k = P::p.tap_k[t];
                if constexpr (OP == OP_FPROP) {
#pragma unroll
                    for (int o = 0; o < R; o++) acc[o] = fmaf(w[k], win[off + o], acc[o]);
                } else {
                    float s = acc[k];
#pragma unroll
                    for (int o = 0; o < R; o++) s = fmaf(win[off + o], w[o], s);
                    acc[k] = s;
                }
            }
        });
    });
}

// DIAG: outputs r = 0..R-1 at (ltop - r, pos0 + r); tap m reads (ltop - (r+m), pos0 + (r+m)).
// `origin` is the index of (ltop, pos0).
template <int OP, int JH, int R, bool CHECK>
__device__ __forceinline__ void seg_diag(const float *__restrict__ sm, int origin, int pitch, int nlines,
                                         int zero_idx, int ltop,
                                         const float (&w)[OP == OP_FPROP ? kMaxTaps : R],
                                         float (&acc)[OP == OP_FPROP ? R : kMaxTaps]) {
    using P = LP<KIND_DIAG, JH>;
    constexpr int lo = P::p.row_lo[0], hi = P::p.row_hi[0];
    constexpr int WN = hi - lo + R;
    float win[WN];
    const int step = 1 - pitch;
#pragma unroll
    for (int i = 0; i < WN; i++) {
        const int t = lo + i;
        int src = origin + t * step;
        if (CHECK) src = ((unsigned)(ltop - t) < (unsigned)nlines) ? src : zero_idx;
        win[i] = sm[src];
    }
    static_for<0, P::p.ntaps>([&](auto ti) {
        constexpr int t = decltype(ti)::value;
        constexpr int off = P::p.tap_dp[t] - lo, k = P::p.tap_k[t];
        if constexpr (OP == OP_FPROP) {
#pragma unroll
            for (int o = 0; o < R; o++) acc[o] = fmaf(w[k], win[off + o], acc[o]);
        } else {
            float s = acc[k];
#pragma unroll
            for (int o = 0; o < R; o++) s = fmaf(win[off + o], w[o], s);
            acc[k] = s;
        }
    });
}

// Sum colliding taps into the first of their group (the reference adds the products of
// all taps that land on the same pixel; merging the weights first is the same sum).
template <int KIND, int JH>
__device__ __forceinline__ void merge_weights(float (&w)[kMaxTaps]) {
    using P = LP<KIND, JH>;
    static_for<0, kMaxTaps>([&](auto ki) {
        constexpr int k = decltype(ki)::value;
        constexpr int into = P::p.merge_into[k];
        if constexpr (into >= 0 && into != k) w[into] += w[k];
    });
}

// merge_into tables of the three base lines as kernel-parameter data (second-level reduce).
struct MergeTables { int8_t t[3][32]; };
template <int JH> constexpr MergeTables make_merge_tables() {
    MergeTables m{};
    for (int kind = 0; kind < 3; kind++) {
        LinePlan p = make_line_plan(kind, JH);
        for (int k = 0; k < kMaxTaps; k++) m.t[kind][k] = (int8_t)p.merge_into[k];
        m.t[kind][31] = -1;
    }
    return m;
}

// Elements of T per 16-byte vector, and the unpack / pack helpers.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    __device__ static void unpack(const uint4 &v, float (&f)[4]) {
        f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y); f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
    }
    __device__ static uint4 pack(const float (&f)[4]) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    __device__ static void unpack(const uint4 &v, float (&f)[8]) {
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            f[2 * i] = __uint_as_float(u[i] << 16);
            f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
        }
    }
    __device__ static uint4 pack(const float (&f)[8]) {
        uint32_t u[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            u[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(u[0], u[1], u[2], u[3]);
    }
};

// Item range of a CTA in the weight gradient: contiguous in chunk-major order, so that a
// CTA stays on one channel chunk for many images and seldom flushes its accumulators.
__host__ __device__ inline int wgrad_item_lo(int cta, int ctas, int total) {
    return (int)(((long long)cta * total) / ctas);
}

// ---------------------------------------------------------------------------------
// OP_FPROP: y = conv(x) (+bias); with flip=1 the weights are read in reverse order, which
//           for stride 1 is the input gradient.  `io` is y.
// OP_WGRAD: partial[(cta, visit)][CC][32] = per-chunk sums of x (*) dy; `io` is dy.
// ---------------------------------------------------------------------------------
// ACT: the instantiation that applies GELU while restaging (p.act) and multiplies the stored
// result by GELU'(preact) (preact != nullptr); the plain instantiation carries neither test.
template <typename T, int R, int JH, int OP, bool ACT>
__global__ void __launch_bounds__(kTiledThreads, 1)
tiled_nhwc_kernel(const __grid_constant__ CUtensorMap tmap, const float *__restrict__ wgt,
                  const float *__restrict__ bias, const int8_t *__restrict__ chan,
                  T *__restrict__ io, float *__restrict__ partial, const T *__restrict__ preact,
                  const TiledParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *sm = reinterpret_cast<float *>(smem_raw);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw + p.off_bar_bytes);
    float *wts = sm + p.off_wts;                               // [CC][32]
    int *misc = reinterpret_cast<int *>(sm + p.off_misc);
    // misc layout: [0..2] channels per kind, [3] error flag, [4..4+CC) channels sorted by kind,
    // then per-channel int4 index maps for the planes and for the band buffer, then bias
    int *ch_sorted = misc + 4;
    int4 *map_in = reinterpret_cast<int4 *>(misc + 4 + kMaxCC);
    int4 *map_out = map_in + kMaxCC;
    float *bias_s = reinterpret_cast<float *>(map_out + kMaxCC);
    int2 *ch_range = reinterpret_cast<int2 *>(bias_s + kMaxCC);   // threads [x, x+y) work on channel i
    int *err_s = misc + 3;

    constexpr int VE = Vec16<T>::N;
    // Segments of 7 (maps of 7..49 pixels, where shared memory has room): every plane is
    // surrounded by zero lines, so no line is ever missing and the checked paths are not
    // instantiated.  Segments of 8 (56x56 fills shared memory): lines are bounds-checked.
    constexpr bool HALO = (R == 7);
    const int tid = threadIdx.x, nt = blockDim.x;
    // hot parameters in registers
    const int CC = p.CC, GV = CC / VE, W = p.W, H = p.H, BR = p.BR, NB = p.NB, NSTG = p.NSTG;
    const int C = p.C;

    for (int i = tid; i < p.zero_floats_total; i += nt) sm[p.off_planar + i] = 0.f;
    if (tid == 0) {
        for (int s = 0; s < NSTG; s++) mbar_init(&full[s], 1);
        *err_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    // ---- item sequence of this CTA ------------------------------------------------------
    // Image-major order makes neighbouring CTAs read neighbouring chunks of the same pixels at
    // the same time (every DRAM sector and page is used while it is open); with a grid that is a
    // multiple of the chunk count each CTA also stays on one chunk.  Chunk-major ranges are the
    // weight gradient's fallback when no such grid exists (it must not hop between chunks).
    int my_items, item_base;
    if (p.order == 0) {
        my_items = (p.total_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
        item_base = blockIdx.x;
    } else {
        item_base = wgrad_item_lo(blockIdx.x, gridDim.x, p.total_items);
        my_items = wgrad_item_lo(blockIdx.x + 1, gridDim.x, p.total_items) - item_base;
    }
    auto item_of = [&](int it, int &n, int &chunk) {
        if (p.order == 0) {             // image-major
            const int item = item_base + it * gridDim.x;
            n = p.div_chunks.div(item); chunk = item - n * p.nchunks;
        } else {                        // chunk-major
            const int item = item_base + it;
            chunk = p.div_n.div(item); n = item - chunk * p.N;
        }
    };
    const int total_bands = my_items * NB;

    auto issue = [&](int gb) {   // producer: one elected thread
        const int it = p.div_nb.div(gb), b = gb - it * NB;
        int n, chunk;
        item_of(it, n, chunk);
        const int s = gb % NSTG;
        mbar_expect_tx(&full[s], p.stage_bytes);
        tma_load_4d(smem_raw + p.off_stage_bytes + (size_t)s * p.stage_stride, &tmap, &full[s], chunk * CC, 0,
                    b * BR, n);
    };
    if (tid == 0)
        for (int gb = 0; gb < NSTG && gb < total_bands; gb++) issue(gb);

    // Band <-> NHWC movement (restage, store, dy fetch): thread -> (row, column, 16-byte vector)
    // of the first TR rows of a band, then the same column TR rows further down: no column
    // wrap, so every index advances by a per-thread constant.  Threads past TR rows idle here.
    const int g_vec = tid % GV;
    const int pix_first = tid / GV;
    const int rl_first = p.div_w.div(pix_first), col_first = pix_first - rl_first * W;
    const bool mover = rl_first < p.TR;
    const int pix_step = p.TR * W;          // pixels between a thread's passes
    const int band_pixels = BR * W;
    const int band_floats = CC * p.out_plane_stride;
    float *const outb = sm + p.off_out;

    constexpr int NACC = (OP == OP_WGRAD) ? kMaxTaps : 1;
    float acc_w[NACC];
    float acc_db = 0.f;
#pragma unroll
    for (int k = 0; k < NACC; k++) acc_w[k] = 0.f;

    int cur_chunk = -1, visit = -1;
    bool have_next_band = false;        // weight gradient: dy band 0 of this item is already staged
    int stage = 0;                      // staging slot and mbarrier parity of the next band to consume
    uint32_t parity = 0;
    int gb = 0;                         // bands consumed so far

    // per-thread segment, set when the chunk changes
    int kind = -1, ch = 0, seg = 0, group_n = 0;
    int at_base = 0, at_step = 0;       // plane index of (line, pos0) at band 0, advance per band
    int line0 = 0, line_step = 0;       // storage line of the segment at band 0, advance per band
    int nlines = 0, pitch = 0;
    int oidx = 0;                       // index of the segment's first output in a band buffer
    int diag_pos0 = 0;

    // Cross-thread reduction of the weight-gradient accumulators of the current chunk, in
    // thread order (fixed), a few taps per pass through the idle band buffers.
    auto flush = [&]() {
        float *red = outb;
        const int cap = (2 * band_floats) / nt;   // taps per pass (host ensures >= 1)
        float *dst = partial + ((size_t)blockIdx.x * p.max_visits + visit) * CC * kPartialStride;
        for (int k0 = 0; k0 < kPartialStride; k0 += cap) {
            __syncthreads();
#pragma unroll
            for (int k = 0; k < kPartialStride; k++)
                if (k >= k0 && k < k0 + cap) {
                    float v = 0.f;
                    if (kind >= 0) v = (k < kMaxTaps) ? acc_w[k < NACC ? k : 0] : acc_db;
                    red[(k - k0) * nt + tid] = v;
                }
            __syncthreads();
            const int ntap = (kPartialStride - k0 < cap) ? kPartialStride - k0 : cap;
            for (int e = tid; e < CC * ntap; e += nt) {
                const int i = e / ntap, kk = e - i * ntap;
                const int2 rg = ch_range[i];
                float sum = 0.f;
                for (int t = 0; t < rg.y; t++) sum += red[kk * nt + rg.x + t];
                dst[i * kPartialStride + k0 + kk] = sum;
            }
        }
        __syncthreads();
    };

    for (int it = 0; it < my_items; it++) {
        int n, chunk;
        item_of(it, n, chunk);
        const int c0 = chunk * CC;
        const bool new_chunk = (chunk != cur_chunk);

        if (OP == OP_WGRAD && new_chunk && cur_chunk >= 0) {
            flush();
#pragma unroll
            for (int k = 0; k < NACC; k++) acc_w[k] = 0.f;
            acc_db = 0.f;
        }

        // ---- per-chunk channel tables --------------------------------------------------
        if (new_chunk) {
            if (tid < 32) {
                int cnt_before = 0;
                int counts[3];
#pragma unroll
                for (int kd = 0; kd < 3; kd++) {
                    int cnt = 0;
                    for (int base = 0; base < CC; base += 32) {
                        const int i = base + tid;
                        const int o = (i < CC) ? chan[c0 + i] : -1;
                        const bool mine = o >= 0 && canon_kind(o) == kd;
                        const unsigned m = __ballot_sync(0xffffffffu, mine);
                        if (mine) ch_sorted[cnt_before + cnt + __popc(m & ((1u << tid) - 1))] = i;
                        cnt += __popc(m);
                    }
                    counts[kd] = cnt;
                    cnt_before += cnt;
                }
#pragma unroll
                for (int kd = 0; kd < 3; kd++) if (tid == kd) misc[kd] = counts[kd];
            }
            for (int i = tid; i < CC; i += nt) {
                const int o = chan[c0 + i];
                const int mode = canon_mode(o);
                const int pbase = p.plane_base + i * p.plane_stride;
                const int obase = i * p.out_plane_stride;
                int4 mi, mo;   // storage index = x*h + y*w + z
                if (mode & MODE_T) {
                    mi = make_int4((mode & MODE_FP) ? -1 : 1, p.pitch_t, pbase + ((mode & MODE_FP) ? H - 1 : 0), mode);
                    mo = make_int4((mode & MODE_FP) ? -1 : 1, p.out_pitch_t, obase + ((mode & MODE_FP) ? BR - 1 : 0), mode);
                } else {
                    mi = make_int4(p.pitch_n, (mode & MODE_FP) ? -1 : 1, pbase + ((mode & MODE_FP) ? W - 1 : 0), mode);
                    mo = make_int4(p.out_pitch_n, (mode & MODE_FP) ? -1 : 1, obase + ((mode & MODE_FP) ? W - 1 : 0), mode);
                }
                map_in[i] = mi;
                map_out[i] = mo;
                bias_s[i] = (OP == OP_FPROP && bias) ? __ldg(bias + c0 + i) : 0.f;
            }
            if (OP == OP_FPROP) {
                const int pad = p.K / 2;
                for (int e = tid; e < CC * 32; e += nt) {
                    const int i = e >> 5, k = e & 31;
                    float v = 0.f;
                    if (k < kMaxTaps) {
                        const int o = chan[c0 + i];
                        int kk = k - kHalf + pad;                      // tap of the K-long kernel
                        if (kk >= 0 && kk < p.K) {
                            const bool rev = ((canon_mode(o) & MODE_REV) != 0) != (p.flip != 0);
                            if (rev) kk = p.K - 1 - kk;
                            v = __ldg(wgt + (size_t)(c0 + i) * p.K + kk);
                            if (p.add_identity && kk == pad) v += 1.f;
                        }
                    }
                    wts[e] = v;
                }
            }
        }
        if (p.rezero) {
            for (int i = tid; i < p.off_zero - 32; i += nt) sm[p.off_planar + 32 + i] = 0.f;
        }
        if (new_chunk || p.rezero) __syncthreads();

        // ---- thread -> (kind, channel, segment), channels grouped by kind
        if (new_chunk) {
            const int nA = misc[0], nS = misc[1], nD = misc[2];
            // groups start on warp boundaries: a warp of mixed kinds would run every path in turn
            // and, being the slowest warp, hold up the band barrier
            const int slotsA = (nA * p.nseg_line + 31) & ~31, slotsS = (nS * p.nseg_line + 31) & ~31;
            kind = -1; ch = 0; seg = 0;
            int idx = tid;
            if (idx < slotsA) {
                const int j = p.div_nseg_line.div(idx);
                if (j < nA) { kind = KIND_AXIS; ch = ch_sorted[j]; seg = idx - j * p.nseg_line; group_n = p.nseg_line; }
            } else if ((idx -= slotsA) < slotsS) {
                const int j = p.div_nseg_line.div(idx);
                if (j < nS) { kind = KIND_SLANT; ch = ch_sorted[nA + j]; seg = idx - j * p.nseg_line; group_n = p.nseg_line; }
            } else {
                idx -= slotsS;
                const int j = p.div_nseg_diag.div(idx);
                if (j < nD) { kind = KIND_DIAG; ch = ch_sorted[nA + nS + j]; seg = idx - j * p.nseg_diag; group_n = p.nseg_diag; }
            }
            if (kind >= 0 && seg == 0) ch_range[ch] = make_int2(tid, group_n);
            cur_chunk = chunk; visit++;

            // geometry of the segment, hoisted out of the band loop
            const int mode = map_in[ch].w;
            const bool transposed = (mode & MODE_T) != 0, fp = (mode & MODE_FP) != 0;
            const int pbase = p.plane_base + ch * p.plane_stride;
            const int obase = ch * p.out_plane_stride;
            if (kind == KIND_DIAG) {
                const int wd = W + R - 1;
                const int sub = p.div_wdiag.div(seg), qi = seg - sub * wd;
                diag_pos0 = qi - (R - 1);
                const int ltop_local = sub * R + R - 1;
                pitch = p.pitch_n; nlines = H;
                line0 = ltop_local; line_step = BR;
                at_base = pbase + ltop_local * pitch + diag_pos0; at_step = BR * pitch;
                oidx = obase + ltop_local * p.out_pitch_n + diag_pos0;
            } else if (!transposed) {                    // lines are image rows
                const int sg = p.div_br.div(seg), rl = seg - sg * BR;
                pitch = p.pitch_n; nlines = H;
                line0 = rl; line_step = BR;
                at_base = pbase + rl * pitch + sg * R; at_step = BR * pitch;
                oidx = obase + rl * p.out_pitch_n + sg * R;
            } else {                                     // lines are image columns
                // lines are dealt to threads rotated by 5, so that the first warp of a channel gets
                // lines 5..36, all of whose neighbours within +-5 exist (no-check fast path)
                const int sub = p.div_wline.div(seg);
                int l = seg - sub * W + 5;
                if (l >= W) l -= W;
                pitch = p.pitch_t; nlines = W;
                line0 = l; line_step = 0;
                at_base = pbase + l * pitch + (fp ? H - BR : 0) + sub * R; at_step = fp ? -BR : BR;
                oidx = obase + l * p.out_pitch_t + sub * R;
            }
        }

        // ---- restage: staging bands -> planes -------------------------------------------
        {
            int ia[VE], dstep[VE], dband[VE];
#pragma unroll
            for (int j = 0; j < VE; j++) {
                const int4 m = map_in[g_vec * VE + j];
                ia[j] = m.x * rl_first + m.y * col_first + m.z;
                dstep[j] = m.x * p.TR;
                dband[j] = m.x * BR;
            }
            int pending = 0;
            for (int b = 0; b < NB; b++) {
                if (*err_s == 0 && !mbar_wait(&full[stage], parity)) *err_s = 1;
                const uint4 *stg = reinterpret_cast<const uint4 *>(smem_raw + p.off_stage_bytes + (size_t)stage * p.stage_stride);
                int idx[VE];
#pragma unroll
                for (int j = 0; j < VE; j++) idx[j] = ia[j];
                for (int pix = mover ? pix_first : band_pixels; pix < band_pixels; pix += pix_step) {
                    float f[VE];
                    Vec16<T>::unpack(stg[pix * GV + g_vec], f);
                    if (ACT && p.act) {
#pragma unroll
                        for (int j = 0; j < VE; j++) f[j] = gelu_exact(f[j]);
                    }
#pragma unroll
                    for (int j = 0; j < VE; j++) { sm[idx[j]] = f[j]; idx[j] += dstep[j]; }
                }
#pragma unroll
                for (int j = 0; j < VE; j++) ia[j] += dband[j];
                gb++;
                if (++stage == NSTG) { stage = 0; parity ^= 1; }
                // A stage may be refilled once every thread has read it: one CTA barrier per
                // group of bands (and after the last band, before the planes are read).
                if (++pending == p.grp || b + 1 == NB) {
                    __syncthreads();
                    if (tid == 0)
                        for (int g = gb - pending; g < gb; g++)
                            if (g + NSTG < total_bands) issue(g + NSTG);
                    pending = 0;
                }
            }
        }

        // ---- compute -----------------------------------------------------------------
        float w[kMaxTaps];
        if (OP == OP_FPROP) {
            const float4 *wp = reinterpret_cast<const float4 *>(wts + ch * 32);
#pragma unroll
            for (int q = 0; q < 8; q++) {
                const float4 v = wp[q];
                w[4 * q] = v.x; w[4 * q + 1] = v.y; w[4 * q + 2] = v.z;
                if (4 * q + 3 < kMaxTaps) w[4 * q + 3] = v.w;
            }
            if (kind == KIND_AXIS) merge_weights<KIND_AXIS, JH>(w);
            else if (kind == KIND_SLANT) merge_weights<KIND_SLANT, JH>(w);
            else if (kind == KIND_DIAG) merge_weights<KIND_DIAG, JH>(w);
        }

        // band buffer <-> global: per-thread constants (index walk as in restage)
        int oa[VE], ostep[VE];
        const float bias_v = (OP == OP_FPROP) ? bias_s[ch] : 0.f;      // accumulators start at the bias
#pragma unroll
        for (int j = 0; j < VE; j++) {
            const int4 m = map_out[g_vec * VE + j];
            oa[j] = m.x * rl_first + m.y * col_first + m.z;
            ostep[j] = m.x * p.TR;
        }
        T *gbase = io + ((size_t)n * H * W) * C + c0 + g_vec * VE;

        // Weight gradient: a dy band travels global -> registers (128-bit NHWC loads, issued
        // before the arithmetic of the previous band) -> band buffer (after it).
        constexpr int kPre = 2;                       // vectors per thread kept in registers
        uint4 pre[kPre];
        auto dy_fetch = [&](const T *src_band) {      // first kPre vectors of this thread
#pragma unroll
            for (int u = 0; u < kPre; u++) {
                const int pix = pix_first + u * pix_step;
                if (mover && pix < band_pixels) pre[u] = __ldg(reinterpret_cast<const uint4 *>(src_band + (size_t)pix * C));
            }
        };
        auto dy_commit = [&](const T *src_band, float *dstb) {
            int idx[VE];
#pragma unroll
            for (int j = 0; j < VE; j++) idx[j] = oa[j];
            int u = 0;
            for (int pix = mover ? pix_first : band_pixels; pix < band_pixels; pix += pix_step, u++) {
                uint4 v;
                if (u < kPre) v = (u == 0) ? pre[0] : pre[kPre - 1];
                else v = __ldg(reinterpret_cast<const uint4 *>(src_band + (size_t)pix * C));
                float f[VE];
                Vec16<T>::unpack(v, f);
#pragma unroll
                for (int j = 0; j < VE; j++) { dstb[idx[j]] = f[j]; idx[j] += ostep[j]; }
            }
        };
        if (OP == OP_WGRAD && !have_next_band) {       // first band of the item, not prefetched
            dy_fetch(gbase);
            dy_commit(gbase, outb + ((it * NB) & 1) * band_floats);
            __syncthreads();
        }
        have_next_band = false;

        int at = at_base, line = line0;
        for (int b = 0; b < NB; b++, at += at_step, line += line_step) {
            const int gbi = it * NB + b;               // global band index: selects the buffer
            float *ob = outb + (gbi & 1) * band_floats + oidx;
            const T *next_src = nullptr;
            if (OP == OP_WGRAD) {
                if (b + 1 < NB) {
                    next_src = gbase + (size_t)(b + 1) * band_pixels * C;
                } else if (it + 1 < my_items) {
                    int n2, chunk2;
                    item_of(it + 1, n2, chunk2);
                    if (chunk2 == chunk) next_src = io + ((size_t)n2 * H * W) * C + c0 + g_vec * VE;
                }
                if (next_src) dy_fetch(next_src);
            }
            // Do all lines this warp's segments touch exist?  Voted by every lane (idle lanes
            // included, they agree) so that the answer is warp-uniform.
            bool lane_inside = true;
            if (kind == KIND_SLANT) {
                constexpr int MD = LP<KIND_SLANT, JH>::p.max_d;
                lane_inside = line - MD >= 0 && line + MD < nlines;
            } else if (kind == KIND_DIAG) {
                using PD = LP<KIND_DIAG, JH>;
                constexpr int TLO = PD::p.row_lo[0], THI = PD::p.row_hi[0] + R - 1;   // t range read
                lane_inside = line - THI >= 0 && line - TLO < nlines;
            }
            const bool inside = HALO || __all_sync(0xffffffffu, lane_inside);
            if (kind == KIND_AXIS) {
                // a single line row (d = 0) and the segment's own line always exists: no checks
                if constexpr (OP == OP_FPROP) {
                    float acc[R];
#pragma unroll
                    for (int o = 0; o < R; o++) acc[o] = bias_v;
                    seg_line<OP_FPROP, KIND_AXIS, JH, R, false>(sm, at, pitch, nlines, p.off_zero, line, w, acc);
#pragma unroll
                    for (int o = 0; o < R; o++) ob[o] = acc[o];
                } else {
                    float g[R];
#pragma unroll
                    for (int o = 0; o < R; o++) { g[o] = ob[o]; acc_db += g[o]; }
                    seg_line<OP_WGRAD, KIND_AXIS, JH, R, false>(sm, at, pitch, nlines, p.off_zero, line, g, acc_w);
                }
            } else if (kind == KIND_SLANT) {
                if constexpr (OP == OP_FPROP) {
                    float acc[R];
#pragma unroll
                    for (int o = 0; o < R; o++) acc[o] = bias_v;
                    if (inside) seg_line<OP_FPROP, KIND_SLANT, JH, R, false>(sm, at, pitch, nlines, p.off_zero, line, w, acc);
                    else seg_line<OP_FPROP, KIND_SLANT, JH, R, true>(sm, at, pitch, nlines, p.off_zero, line, w, acc);
#pragma unroll
                    for (int o = 0; o < R; o++) ob[o] = acc[o];
                } else {
                    float g[R];
#pragma unroll
                    for (int o = 0; o < R; o++) { g[o] = ob[o]; acc_db += g[o]; }
                    if (inside) seg_line<OP_WGRAD, KIND_SLANT, JH, R, false>(sm, at, pitch, nlines, p.off_zero, line, g, acc_w);
                    else seg_line<OP_WGRAD, KIND_SLANT, JH, R, true>(sm, at, pitch, nlines, p.off_zero, line, g, acc_w);
                }
            } else if (kind == KIND_DIAG) {
                const int odiag = 1 - p.out_pitch_n;
                if constexpr (OP == OP_FPROP) {
                    float acc[R];
#pragma unroll
                    for (int o = 0; o < R; o++) acc[o] = bias_v;
                    if (inside) seg_diag<OP_FPROP, JH, R, false>(sm, at, pitch, nlines, p.off_zero, line, w, acc);
                    else seg_diag<OP_FPROP, JH, R, true>(sm, at, pitch, nlines, p.off_zero, line, w, acc);
#pragma unroll
                    for (int o = 0; o < R; o++)
                        if ((unsigned)(diag_pos0 + o) < (unsigned)W) ob[o * odiag] = acc[o];
                } else {
                    float g[R];
#pragma unroll
                    for (int o = 0; o < R; o++) {
                        g[o] = ((unsigned)(diag_pos0 + o) < (unsigned)W) ? ob[o * odiag] : 0.f;
                        acc_db += g[o];
                    }
                    if (inside) seg_diag<OP_WGRAD, JH, R, false>(sm, at, pitch, nlines, p.off_zero, line, g, acc_w);
                    else seg_diag<OP_WGRAD, JH, R, true>(sm, at, pitch, nlines, p.off_zero, line, g, acc_w);
                }
            }
            if (OP == OP_WGRAD && next_src) {
                // the other buffer was last read one band ago, before the previous barrier
                dy_commit(next_src, outb + ((gbi + 1) & 1) * band_floats);
                if (b + 1 == NB) have_next_band = true;
            }
            __syncthreads();
            if (OP == OP_FPROP) {
                // ---- store band b: band buffer -> NHWC, 16 bytes per thread ---------------------
                const float *src = outb + (gbi & 1) * band_floats;
                T *gdst = gbase + (size_t)b * band_pixels * C;
                int idx[VE];
#pragma unroll
                for (int j = 0; j < VE; j++) idx[j] = oa[j];
                for (int pix = mover ? pix_first : band_pixels; pix < band_pixels; pix += pix_step) {
                    float f[VE];
#pragma unroll
                    for (int j = 0; j < VE; j++) { f[j] = src[idx[j]]; idx[j] += ostep[j]; }
                    if (ACT && preact) {   // input gradient of a conv over GELU(preact): times GELU'(preact)
                        float g[VE];
                        Vec16<T>::unpack(__ldg(reinterpret_cast<const uint4 *>(preact + (gdst - io) + (size_t)pix * C)), g);
#pragma unroll
                        for (int j = 0; j < VE; j++) f[j] *= gelu_exact_grad(g[j]);
                    }
                    *reinterpret_cast<uint4 *>(gdst + (size_t)pix * C) = Vec16<T>::pack(f);
                }
            }
        }
    }
    if (OP == OP_WGRAD && cur_chunk >= 0) flush();
}

// Second level of the weight gradient: dw[c][k] = sum over the CTAs that visited c's chunk,
// in CTA order, of their partial for the stored tap that original tap k maps to.
__global__ void tiled_wgrad_final_kernel(const float *__restrict__ partial, const int8_t *__restrict__ chan,
                                         float *__restrict__ dw,
                                         float *__restrict__ db, int C, int K, int CC, int N, int total_items,
                                         int ctas, int max_visits, int order, const MergeTables mt) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= C * (K + 1)) return;
    const int c = idx / (K + 1), k = idx % (K + 1);
    if (k == K && db == nullptr) return;
    const int chunk = c / CC, i = c % CC;
    int slot;
    if (k == K) {
        slot = kMaxTaps;                                   // bias-gradient sum
    } else {
        const int o = chan[c];
        const int kk = (canon_mode(o) & MODE_REV) ? K - 1 - k : k;
        slot = mt.t[canon_kind(o)][kk + kHalf - K / 2];
    }
    const int item_lo = chunk * N, item_hi = item_lo + N;
    float sum = 0.f;
    // slot < 0: the tap cannot reach inside an image of this size; its gradient is exactly 0
    if (order == 0) {     // every CTA stayed on chunk (cta % nchunks) and wrote one partial
        const int nchunks = C / CC;
        for (int b = chunk; b < ctas && slot >= 0; b += nchunks)
            if (b < total_items) sum += partial[(((size_t)b * max_visits) * CC + i) * kPartialStride + slot];
    } else
    for (int b = 0; b < ctas && slot >= 0; b++) {
        const int lo = wgrad_item_lo(b, ctas, total_items), hi = wgrad_item_lo(b + 1, ctas, total_items);
        if (hi <= item_lo || lo >= item_hi || hi == lo) continue;
        const int v = chunk - lo / N;
        sum += partial[(((size_t)b * max_visits + v) * CC + i) * kPartialStride + slot];
    }
    if (k == K) db[c] = sum; else dw[(size_t)c * K + k] = sum;
}

}  // namespace o1d
