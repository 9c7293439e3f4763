// Whole-line kernels: stride 1, K <= 31, every channel on one of the eight canonical lines,
// NHWC, square maps whose side L is a compile-time constant (the ConvNeXt stage maps).
//
// A work item is (image n, 4 consecutive channels) = 16 bytes per pixel in fp32.  A CTA of four
// warps owns one item at a time, one warp per channel, and two CTAs share an SM so that one
// CTA's arithmetic overlaps the other's data movement.  Per item:
//
//   1. TMA (cp.async.bulk.tensor, 4-D box 4 x L x 8 x 1) streams the item's row bands into a small
//      ring; the producer runs ahead across item boundaries.
//   2. restage: every band is scattered into one fp32 plane per channel in (line, position)
//      coordinates (o1d_lines.cuh): rows for horizontal lines, columns for vertical ones,
//      anti-diagonals (wrapped, with a gap of zeros between the two pieces that share a storage
//      row) for the 45-degree lines.  After this step every line of an axis or diagonal channel
//      is one contiguous storage row.
//   3. compute: a lane owns whole storage rows.  It loads a row into registers ONCE (one
//      shared-memory load per output instead of one per tap or per window) and evaluates all
//      outputs of the row with compile-time tap offsets; taps that fall off the row do not
//      exist at compile time, so there are no bounds tests and no halo columns.  Axis and
//      diagonal rows are private to their lane and are overwritten in place.  Slanted lines
//      (22.5 degrees: 29 taps spread over 11 rows) are evaluated for two adjacent rows and half
//      a row of outputs at a time, so that each loaded row segment serves both output rows;
//      their results go to a second plane.
//   4. destage: planes are gathered back to NHWC 16-byte vectors, bias added, and stored.
//
// Shared-memory plane layouts are chosen so that every phase is free of bank conflicts:
// a storage row r starts at (r >> 2) * G4 + (r & 3) * Q4 (planes whose rows are image rows) or at
// (r >> 3) * G8 + (r & 7) * Q8 (planes whose rows are image columns), with G = 1 (mod 32) and
// Q chosen so that the 4 (8) rows of a group start 8 (4) banks apart.  The movers work on tiles
// of 8 pixels x 4 rows per warp, which then hit 32 different banks in either plane type, and the
// compute lanes (consecutive rows, or every second row) do too.
//
// The reference kernels (models/dwoconv1d_specialized/kernels/kernels.h:201-291) give each block
// one (n, c) plane band, re-read the halo rows per band and redo sincosf + float->int + four
// compares per tap.
#pragma once

#include <cuda.h>

#include <type_traits>

#include "o1d_common.cuh"
#include "o1d_lines.cuh"

namespace o1d {
namespace wl {

constexpr int kThreads = 128;            // four warps, one per channel of the item
constexpr int kCC = 4;                   // channels per item
constexpr int kBR = 8;                   // rows per TMA band
constexpr int kMaxStages = 4;
constexpr int kGap = 10;                 // zeros between the two diagonal pieces of a storage row (largest |dp|)
constexpr int kHaloRows = 8;             // zero rows above a slanted-line plane (largest |dl| is 5; 8 keeps groups aligned)
constexpr uint32_t kSpinLimit = 1u << 22;

constexpr int next_mod(int v, int m, int r) {
    int x = v;
    while (x % m != r) x++;
    return x;
}

template <int L>
struct Geo {
    static_assert(L % 8 == 0 && L / 2 <= 32 && L >= 16, "side must be a multiple of 8 with L/2 lanes");
    static constexpr int Q4 = next_mod(L, 16, 8), G4 = 4 * Q4 + 1;              // rows are image rows
    static constexpr int Q8 = next_mod(L, 8, 4), G8 = 8 * Q8 + 1;               // rows are image columns
    static constexpr int LD = L + kGap;                                         // wrapped diagonal row
    static constexpr int QD = next_mod(LD, 16, 8), GD = 4 * QD + 1;
    static constexpr int SR = L + 2 * kHaloRows;                                // rows of a slanted-line plane
    static constexpr int cmax(int a, int b) { return a > b ? a : b; }
    static constexpr int kAxisFloats = cmax((L / 4) * G4, (L / 8) * G8);
    static constexpr int kSlantFloats = cmax((SR / 4) * G4, (SR / 8) * G8);
    static constexpr int kDiagFloats = (L / 4) * GD;
    static constexpr int kOutFloats = kAxisFloats;                              // second plane of a slanted channel
    static constexpr int kTilesX = L / 8, kTilesBand = (kBR / 4) * kTilesX, kTilesImage = (L / 4) * kTilesX;
    static constexpr int NB = L / kBR;
    static constexpr int kStageBytes = kBR * L * kCC * 4;
};

struct WlParams {
    int N, C, K, nchunks, total_items;
    int flip, add_identity;
    int in_off[kCC], out_off[kCC];       // plane offsets (floats); out_off == in_off for in-place kinds
    int plane_floats;                    // floats to clear at kernel start
    int off_wts;                         // [kCC][32] floats
    int off_stage_bytes, nstg, off_bar_bytes;
};

// ---- mbarrier / TMA primitives -----------------------------------------------------------------
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
// Bounded wait: gives up (and raises the caller's flag) if the data never arrives.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int *err_flag) {
    for (uint32_t i = 0; i < kSpinLimit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(err_flag, 1);
    return false;
}
__device__ __forceinline__ void tma_load_4d(void *dst, const CUtensorMap *map, uint64_t *bar, int c0, int c1,
                                            int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

template <int I, int N, typename F>
__device__ __forceinline__ void static_for(F &&f) {
    if constexpr (I < N) {
        f(std::integral_constant<int, I>{});
        static_for<I + 1, N>(f);
    }
}

// ---- plane addressing ----------------------------------------------------------------------------
// Start of storage row r of a plane at `off`.
struct RowBase {
    int off, sh, msk, G, Q;
    __device__ __forceinline__ int operator()(int r) const { return off + (r >> sh) * G + (r & msk) * Q; }
};

// Where a mover lane's pixel of a tile lands in a channel plane: addr = a*hb + b*wb + c, with hb, wb
// the tile's row (4 image rows) and column (8 pixels) index, plus `wrapfix` on the second piece of
// a wrapped diagonal (4*hb + tb*wb + tc >= L).
struct ChanMap {
    int a, b, c;
    int tb, tc, wrapfix;
};

template <int L>
__device__ __forceinline__ ChanMap make_map(int o, int off, int halo, int hi, int wi) {
    using G = Geo<L>;
    const int kind = canon_kind(o), mode = canon_mode(o);
    const bool fp = (mode & MODE_FP) != 0;
    ChanMap m;
    m.tb = 0; m.tc = -(1 << 24); m.wrapfix = 0;
    if (kind == KIND_DIAG) {
        const int wi2 = fp ? 7 - wi : wi, s = hi + wi2;
        const int per_wb = 2 * G::GD + 8;
        m.a = G::GD;
        m.b = fp ? -per_wb : per_wb;
        m.c = off + (s >> 2) * G::GD + (s & 3) * G::QD + wi2 + (fp ? (L / 8 - 1) * per_wb : 0);
        m.tb = fp ? -8 : 8;
        m.tc = s + (fp ? 8 * (L / 8 - 1) : 0);
        m.wrapfix = kGap - (L / 4) * G::GD;
    } else if (!(mode & MODE_T)) {
        m.a = G::G4;
        m.b = fp ? -8 : 8;
        m.c = off + (halo / 4) * G::G4 + hi * G::Q4 + (fp ? L - 1 - wi : wi);
    } else {
        m.a = fp ? -4 : 4;
        m.b = G::G8;
        m.c = off + (halo / 8) * G::G8 + wi * G::Q8 + (fp ? L - 1 - hi : hi);
    }
    return m;
}

__device__ __forceinline__ int map_addr(const ChanMap &m, int hb, int wb, int Lside) {
    int a = m.a * hb + m.b * wb + m.c;
    if (m.wrapfix != 0 && 4 * hb + m.tb * wb + m.tc >= Lside) a += m.wrapfix;     // wrapped diagonals only
    return a;
}

template <int L>
__device__ __forceinline__ RowBase row_base_of(int o, int off) {
    using G = Geo<L>;
    const int kind = canon_kind(o), mode = canon_mode(o);
    if (kind == KIND_DIAG) return RowBase{off, 2, 3, G::GD, G::QD};
    if (!(mode & MODE_T)) return RowBase{off, 2, 3, G::G4, G::Q4};
    return RowBase{off, 3, 7, G::G8, G::Q8};
}

// Sum colliding taps into the first of their group (the reference adds the products of all taps
// that land on the same pixel; merging the weights first is the same sum).
template <int KIND, int JH>
__device__ __forceinline__ void merge_weights(float (&w)[kMaxTaps]) {
    using P = LP<KIND, JH>;
    static_for<0, kMaxTaps>([&](auto ki) {
        constexpr int k = decltype(ki)::value;
        constexpr int into = P::p.merge_into[k];
        if constexpr (into >= 0 && into != k) w[into] += w[k];
    });
}

// ---- compute bodies --------------------------------------------------------------------------------
// Every body evaluates HALF of its outputs and is run twice: the second half is the first half of
// the mirrored problem (positions counted from the far end of the row, rows from the far end of the
// plane), which for these odd-symmetric lines is the same arithmetic with the weights read in
// reverse order.  That halves the unrolled code (the instruction cache is what limits these
// kernels' size) while a tap that would fall off the near end of a row still vanishes at compile
// time and the far end needs no test.

// Reversed copy of the 31 original weights (tap k <-> tap 30-k).
__device__ __forceinline__ void reverse_weights(const float (&w)[kMaxTaps], float (&wr)[kMaxTaps]) {
#pragma unroll
    for (int k = 0; k < kMaxTaps; k++) wr[k] = w[kMaxTaps - 1 - k];
}

// AXIS / DIAG: 1-D convolution along storage rows of length ROW, in place.  A lane works through
// `nrows` rows (row0, row0 + row_step, ..) x 2 halves.  Each half loads a window of ROW/2 + reach
// inputs once, and holds its ROW/2 results back until the next window has been read, because the
// next window may overlap the columns they overwrite.  KIND_DIAG rows hold two diagonals separated
// by kGap zeros at columns rho+1 .. rho+kGap; results there are not written, so the gap stays zero.
template <int KIND, int JH, int ROW>
__device__ __forceinline__ void rows_in_place(float *__restrict__ sm, const RowBase &rb, int row0, int row_step,
                                              int nrows, const float (&w)[kMaxTaps], const float (&wr)[kMaxTaps]) {
    using P = LP<KIND, JH>;
    constexpr int HALF = ROW / 2;
    constexpr int REACH = (KIND == KIND_DIAG) ? kGap : JH;
    constexpr int WN = (HALF + REACH < ROW) ? HALF + REACH : ROW;
    static_assert(ROW % 2 == 0, "rows are processed in two halves");
    float pend[HALF];
    int pend_at = 0, pend_dir = 0, pend_c0 = 0, pend_rho = 0;
#pragma unroll 1
    for (int it = 0; it < 2 * nrows; it++) {
        const int rho = row0 + (it >> 1) * row_step;
        const bool mirror = (it & 1) != 0;
        const int c0 = mirror ? ROW - 1 : 0, dir = mirror ? -1 : 1;
        const int at = rb(rho) + c0;
        float x[WN];
#pragma unroll
        for (int i = 0; i < WN; i++) x[i] = sm[at + dir * i];
        if (it > 0) {
#pragma unroll
            for (int o = 0; o < HALF; o++) {
                const int col = pend_c0 + pend_dir * o;
                if (KIND != KIND_DIAG || col <= pend_rho || col > pend_rho + kGap) sm[pend_at + pend_dir * o] = pend[o];
            }
        }
        float wv[kMaxTaps];
#pragma unroll
        for (int k = 0; k < kMaxTaps; k++) wv[k] = mirror ? wr[k] : w[k];
#pragma unroll
        for (int o = 0; o < HALF; o++) pend[o] = 0.f;
        static_for<0, P::p.ntaps>([&](auto ti) {
            constexpr int t = decltype(ti)::value;
            constexpr int dp = P::p.tap_dp[t], k = P::p.tap_k[t];
#pragma unroll
            for (int o = 0; o < HALF; o++)
                if (o + dp >= 0 && o + dp < WN) pend[o] = fmaf(wv[k], x[o + dp], pend[o]);
        });
        pend_at = at; pend_dir = dir; pend_c0 = c0; pend_rho = rho;
    }
#pragma unroll
    for (int o = 0; o < HALF; o++) {
        const int col = pend_c0 + pend_dir * o;
        if (KIND != KIND_DIAG || col <= pend_rho || col > pend_rho + kGap) sm[pend_at + pend_dir * o] = pend[o];
    }
}

// SLANT.  Window of (mirrored) storage row 2*rp + e needed by the outputs of rows 2*rp + m, m = 0, 1,
// columns 0 .. R-1: the union over m of the taps with line offset d = e - m, clipped to the row.
struct SlWin { int lo, hi; };
constexpr int slant_find_row(const LinePlan &p, int d) {
    for (int r = 0; r < p.nrows; r++)
        if (p.row_d[r] == d) return r;
    return -1;
}
template <int JH>
constexpr SlWin slant_window(int e, int R, int L) {
    const LinePlan &p = LP<KIND_SLANT, JH>::p;
    int lo = 1 << 20, hi = -(1 << 20);
    for (int m = 0; m < 2; m++) {
        const int r = slant_find_row(p, e - m);
        if (r < 0) continue;
        if (p.row_lo[r] < lo) lo = p.row_lo[r];
        if (R - 1 + p.row_hi[r] > hi) hi = R - 1 + p.row_hi[r];
    }
    if (lo < 0) lo = 0;
    if (hi > L - 1) hi = L - 1;
    return SlWin{lo, hi};
}

// Slanted channel: a lane owns the row pair rp and evaluates, per pass, the outputs of its two rows
// in the columns 0 .. L/2-1 of the plain (pass 0) or mirrored (pass 1) plane, so that every loaded
// row segment serves both rows.  `in` addresses the input plane (kHaloRows zero rows above and below
// the image rows), `out` the result plane (no halo).
template <int L, int JH>
__device__ __forceinline__ void slant_rows(const float *__restrict__ sm, float *__restrict__ smo, const RowBase &in,
                                           const RowBase &out, int rp, const float (&w)[kMaxTaps],
                                           const float (&wr)[kMaxTaps]) {
    using P = LP<KIND_SLANT, JH>;
    constexpr int MD = P::p.max_d, R = L / 2;
#pragma unroll 1
    for (int pass = 0; pass < 2; pass++) {
        const bool mirror = pass != 0;
        const int rs = mirror ? -1 : 1, r0 = mirror ? L - 1 : 0;        // image row = rs * (mirrored row) + r0
        const int cs = rs, cb = r0;                                     // same for columns
        float wv[kMaxTaps];
#pragma unroll
        for (int k = 0; k < kMaxTaps; k++) wv[k] = mirror ? wr[k] : w[k];
        float acc[2][R];
#pragma unroll
        for (int m = 0; m < 2; m++)
#pragma unroll
            for (int o = 0; o < R; o++) acc[m][o] = 0.f;
        static_for<0, 2 * MD + 2>([&](auto ei) {
            constexpr int e = decltype(ei)::value - MD;
            constexpr SlWin wn = slant_window<JH>(e, R, L);
            if constexpr (wn.hi >= wn.lo) {
                constexpr int WN = wn.hi - wn.lo + 1;
                const int base = in(rs * (2 * rp + e) + r0 + kHaloRows) + cb + cs * wn.lo;
                float win[WN];
#pragma unroll
                for (int i = 0; i < WN; i++) win[i] = sm[base + cs * i];
                static_for<0, 2>([&](auto mi) {
                    constexpr int m = decltype(mi)::value;
                    constexpr int r = slant_find_row(P::p, e - m);
                    if constexpr (r >= 0) {
                        static_for<0, P::p.ntaps>([&](auto ti) {
                            constexpr int t = decltype(ti)::value;
                            if constexpr (P::p.tap_row[t] == r) {
                                constexpr int dp = P::p.tap_dp[t], k = P::p.tap_k[t];
#pragma unroll
                                for (int o = 0; o < R; o++)
                                    if (o + dp >= wn.lo && o + dp <= wn.hi)
                                        acc[m][o] = fmaf(wv[k], win[o + dp - wn.lo], acc[m][o]);
                            }
                        });
                    }
                });
            }
        });
#pragma unroll
        for (int m = 0; m < 2; m++) {
            const int ob = out(rs * (2 * rp + m) + r0) + cb;
#pragma unroll
            for (int o = 0; o < R; o++) smo[ob + cs * o] = acc[m][o];
        }
    }
}

// ---------------------------------------------------------------------------------------------------
// y = conv(x) (+ bias); with flip = 1 the weights are read in reverse order, which for stride 1 is
// the input gradient.  Grid: persistent CTAs, items dealt image-major (neighbouring CTAs read
// neighbouring 16-byte halves of the same pixels at the same time).
// ---------------------------------------------------------------------------------------------------
template <int L, int JH>
__global__ void __launch_bounds__(kThreads, 2)
wline_fprop_kernel(const __grid_constant__ CUtensorMap tmap, const float *__restrict__ wgt,
                   const float *__restrict__ bias, const int8_t *__restrict__ chan, float *__restrict__ y,
                   int *__restrict__ err_flag, const WlParams p) {
    using G = Geo<L>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *sm = reinterpret_cast<float *>(smem_raw);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw + p.off_bar_bytes);
    float *wts = sm + p.off_wts;
    __shared__ int err_s;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wi = lane & 7, hi = lane >> 3;             // mover lane -> pixel of an 8 x 4 tile
    const int NSTG = p.nstg;

    for (int i = tid; i < p.plane_floats; i += kThreads) sm[i] = 0.f;
    if (tid == 0) {
        for (int s = 0; s < NSTG; s++) mbar_init(&full[s], 1);
        err_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    const int my_items = (p.total_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int total_bands = my_items * G::NB;
    auto issue = [&](int gb) {   // one elected thread
        const int it = gb / G::NB, b = gb - it * G::NB;
        const int item = blockIdx.x + it * gridDim.x;
        const int n = item / p.nchunks, chunk = item - n * p.nchunks;
        const int s = gb % NSTG;
        mbar_expect_tx(&full[s], G::kStageBytes);
        tma_load_4d(smem_raw + p.off_stage_bytes + (size_t)s * G::kStageBytes, &tmap, &full[s], chunk * kCC, 0,
                    b * kBR, n);
    };
    if (tid == 0)
        for (int gb = 0; gb < NSTG && gb < total_bands; gb++) issue(gb);

    int gb = 0;                      // bands consumed so far
    int prev_sig = -1;               // plane types of the previous item (re-zero when they change)
    for (int it = 0; it < my_items; it++) {
        const int item = blockIdx.x + it * gridDim.x;
        const int n = item / p.nchunks, chunk = item - n * p.nchunks;
        const int c0 = chunk * kCC;

        // ---- per-item channel tables: line ids, mover maps, weights ------------------------------
        int o_all[kCC];
#pragma unroll
        for (int j = 0; j < kCC; j++) o_all[j] = chan[c0 + j];
        int sig = 0;
#pragma unroll
        for (int j = 0; j < kCC; j++) sig = sig * 16 + canon_kind(o_all[j]) * 4 + (canon_mode(o_all[j]) & MODE_T) * 2;
        if (sig != prev_sig && prev_sig >= 0) {
            // another mix of plane types: stale data would sit where zeros are expected
            for (int i = tid; i < p.plane_floats; i += kThreads) sm[i] = 0.f;
        }
        prev_sig = sig;
        {
            const int pad = p.K / 2;
            const int j = tid >> 5, k = tid & 31;           // 4 x 32 entries, one per thread
            float v = 0.f;
            if (k < kMaxTaps) {
                int kk = k - kHalf + pad;
                if (kk >= 0 && kk < p.K) {
                    const bool rev = ((canon_mode(o_all[j]) & MODE_REV) != 0) != (p.flip != 0);
                    if (rev) kk = p.K - 1 - kk;
                    v = __ldg(wgt + (size_t)(c0 + j) * p.K + kk);
                    if (p.add_identity && kk == pad) v += 1.f;
                }
            }
            wts[tid] = v;
        }
        ChanMap rmap[kCC];
#pragma unroll
        for (int j = 0; j < kCC; j++)
            rmap[j] = make_map<L>(o_all[j], p.in_off[j], canon_kind(o_all[j]) == KIND_SLANT ? kHaloRows : 0, hi, wi);
        __syncthreads();

        // ---- restage: staging bands -> planes ---------------------------------------------------------
        for (int b = 0; b < G::NB; b++) {
            const int s = gb % NSTG;
            const uint32_t parity = (gb / NSTG) & 1;
            if (err_s == 0 && !mbar_wait(&full[s], parity, err_flag)) err_s = 1;
            const float4 *stg = reinterpret_cast<const float4 *>(smem_raw + p.off_stage_bytes + (size_t)s * G::kStageBytes);
            for (int t = warp; t < G::kTilesBand; t += 4) {
                const int ty = t / G::kTilesX, tx = t - ty * G::kTilesX;
                const int hb = b * (kBR / 4) + ty;
                const float4 v = stg[(4 * ty + hi) * L + 8 * tx + wi];
                sm[map_addr(rmap[0], hb, tx, L)] = v.x;
                sm[map_addr(rmap[1], hb, tx, L)] = v.y;
                sm[map_addr(rmap[2], hb, tx, L)] = v.z;
                sm[map_addr(rmap[3], hb, tx, L)] = v.w;
            }
            __syncthreads();
            if (tid == 0 && gb + NSTG < total_bands) issue(gb + NSTG);
            gb++;
        }

        // ---- compute: warp j evaluates channel j ----------------------------------------------------------
        {
            const int o = o_all[0] * (warp == 0) + o_all[1] * (warp == 1) + o_all[2] * (warp == 2) + o_all[3] * (warp == 3);
            const int in_off = p.in_off[0] * (warp == 0) + p.in_off[1] * (warp == 1) + p.in_off[2] * (warp == 2) +
                               p.in_off[3] * (warp == 3);
            const int kind = canon_kind(o);
            // results of a slanted channel go to its second plane; the other kinds work in place
            const int out_off = kind != KIND_SLANT ? in_off
                                                   : p.out_off[0] * (warp == 0) + p.out_off[1] * (warp == 1) +
                                                         p.out_off[2] * (warp == 2) + p.out_off[3] * (warp == 3);
            float w[kMaxTaps];
            {
                const float4 *wp = reinterpret_cast<const float4 *>(wts + warp * 32);
#pragma unroll
                for (int q = 0; q < 8; q++) {
                    const float4 v = wp[q];
                    w[4 * q] = v.x; w[4 * q + 1] = v.y; w[4 * q + 2] = v.z;
                    if (4 * q + 3 < kMaxTaps) w[4 * q + 3] = v.w;
                }
            }
            if (lane < L / 2) {
                float wr[kMaxTaps];
                reverse_weights(w, wr);
                if (kind == KIND_AXIS) {
                    const RowBase rb = row_base_of<L>(o, in_off);
                    rows_in_place<KIND_AXIS, JH, L>(sm, rb, lane, L / 2, 2, w, wr);
                } else if (kind == KIND_DIAG) {
                    merge_weights<KIND_DIAG, JH>(w);
                    merge_weights<KIND_DIAG, JH>(wr);
                    const RowBase rb = row_base_of<L>(o, in_off);
                    rows_in_place<KIND_DIAG, JH, G::LD>(sm, rb, lane, L / 2, 2, w, wr);
                } else {
                    merge_weights<KIND_SLANT, JH>(w);
                    merge_weights<KIND_SLANT, JH>(wr);
                    const RowBase in = row_base_of<L>(o, in_off), out = row_base_of<L>(o, out_off);
                    slant_rows<L, JH>(sm, sm, in, out, lane, w, wr);
                }
            }
        }
        __syncthreads();

        // ---- destage: planes -> NHWC, bias added ---------------------------------------------------------
        {
            ChanMap dmap[kCC];
            float bv[kCC];
#pragma unroll
            for (int j = 0; j < kCC; j++) {
                dmap[j] = make_map<L>(o_all[j], canon_kind(o_all[j]) == KIND_SLANT ? p.out_off[j] : p.in_off[j], 0, hi, wi);
                bv[j] = bias ? __ldg(bias + c0 + j) : 0.f;
            }
            float *ybase = y + ((size_t)n * L * L) * p.C + c0;
            for (int t = warp; t < G::kTilesImage; t += 4) {
                const int hb = t / G::kTilesX, tx = t - hb * G::kTilesX;
                float4 v;
                v.x = sm[map_addr(dmap[0], hb, tx, L)] + bv[0];
                v.y = sm[map_addr(dmap[1], hb, tx, L)] + bv[1];
                v.z = sm[map_addr(dmap[2], hb, tx, L)] + bv[2];
                v.w = sm[map_addr(dmap[3], hb, tx, L)] + bv[3];
                const int h = 4 * hb + hi, wq = 8 * tx + wi;
                *reinterpret_cast<float4 *>(ybase + ((size_t)h * L + wq) * p.C) = v;
            }
        }
        __syncthreads();
    }
}

}  // namespace wl
}  // namespace o1d
