// Whole-line kernels: stride 1, K <= 31, every channel on one of the eight canonical lines,
// NHWC, square maps whose side L is a compile-time constant (the ConvNeXt stage maps).
//
// A work item is (image n, 8 consecutive channels) = 32 bytes per pixel in fp32, one DRAM sector:
// narrower items were measured to cap a plain strided copy of the tensor at 40 % of the HBM rate
// (16-byte pieces) against 68 % for 32-byte pieces.  A CTA of eight warps owns one item at a time.
// Per item:
//
//   1. TMA (cp.async.bulk.tensor, 4-D box 8 x L x 8 x 1) streams the item's row bands into a small
//      ring; the producer runs ahead across item boundaries, and the warp that finishes a band
//      last refills its slot (no CTA-wide barrier per band).
//   2. restage: every band is scattered into fp32 planes in (line, position) coordinates
//      (o1d_lines.cuh): rows for horizontal lines, columns for vertical ones, anti-diagonals
//      (wrapped, with a gap of zeros between the two pieces that share a storage row) for the
//      45-degree lines.  After this step every line of an axis or diagonal channel is one
//      contiguous storage row.
//   3. compute: a lane owns whole storage rows and slides each of them through a register window,
//      so every input is loaded from shared memory ONCE (not once per tap or per window) and no tap
//      needs a bounds test.  Axis and diagonal rows are private to their lane and are overwritten
//      in place.  Slanted lines (22.5 degrees: 29 taps spread over 11 rows) are evaluated for two
//      adjacent rows at a time, so that each loaded row segment serves both; their results go to
//      a second plane.
//   4. destage: planes are gathered back to NHWC 16-byte vectors, bias added, and stored.
//
// Everything is stored and computed in PAIRS (two floats side by side, one 64-bit shared-memory
// access, one packed fma.rn.f32x2): the two halves are two adjacent storage rows of one channel
// (axis, diagonal) or the same pixel of two slanted channels of the item.  The arithmetic is bound
// by instruction issue, and the pairing halves its instruction count.
//
// The instruction cache shapes the compute bodies: straight-line code that four warps run through
// at different places stops fitting at roughly 2 K instructions in total, after which the kernel
// waits for instruction fetches.  Every body is therefore a short unrolled block inside a rolled
// loop over chunks of outputs.
//
// Plane layouts are chosen so that every phase is (nearly) free of bank conflicts: a storage row
// (pair) starts at group * G + member * Q with G = 2 (mod 32) and Q a multiple of 8 chosen per
// plane type, so that the rows a mover tile of 8 pixels x 4 rows touches, and the rows consecutive
// compute lanes own, start in different banks.
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

constexpr int kCC = 8;                   // channels per item: 32 bytes of every pixel, one DRAM sector
constexpr int kWarps = kCC;              // one warp per channel
constexpr int kThreads = 32 * kWarps;
constexpr int kBR = 8;                   // rows per TMA band
constexpr int kMaxStages = 4;
constexpr int kGap = 10;                 // zeros between the two diagonal pieces of a storage row (largest |dp|)
constexpr int kHaloRows = 8;             // zero rows above and below a slanted-line plane (largest |dl| is 5, +1 for the row pair)
constexpr uint32_t kSpinLimit = 1u << 22;

constexpr int next_mod(int v, int m, int r) {
    int x = v;
    while (x % m != r) x++;
    return x;
}
constexpr int cmax(int a, int b) { return a > b ? a : b; }

// Plane geometry for side L.  All sizes in floats; every plane holds pairs, so a position is 2 floats.
template <int L>
struct Geo {
    static_assert(L % 8 == 0 && L / 2 <= 32 && L >= 16, "side must be a multiple of 8 with L/2 lanes");
    // axis, rows are image rows: row r at (r>>2)*G2 + ((r>>1)&1)*Q2, its pair half r&1
    static constexpr int Q2 = next_mod(2 * L, 32, 16), G2 = 2 * Q2 + 2;
    // axis, rows are image columns: row pair q = r>>1 at (q>>2)*G8 + (q&3)*Q8
    static constexpr int Q8 = next_mod(2 * L, 16, 8), G8 = 4 * Q8 + 2;
    // diagonals (wrapped rows of L + kGap positions), paired like Q2/G2
    static constexpr int LD = L + kGap;
    static constexpr int QD = next_mod(2 * LD, 32, 16), GD = 2 * QD + 2;
    // slanted channel pair: row r at (r>>2)*GS + (r&3)*QS, pair half = channel of the pair
    static constexpr int SR = L + 2 * kHaloRows;
    static constexpr int QS = next_mod(2 * L, 16, 8), GS = 4 * QS + 2;
    static constexpr int kAxisFloats = cmax((L / 4) * G2, (L / 8) * G8);
    static constexpr int kDiagFloats = (L / 4) * GD;
    static constexpr int kSlantInFloats = (SR / 4) * GS;       // both channels of a pair
    static constexpr int kSlantOutFloats = (L / 4) * GS;
    static constexpr int kTilesX = L / 8, kTilesBand = (kBR / 4) * kTilesX, kTilesImage = (L / 4) * kTilesX;
    static constexpr int NB = L / kBR;
    static constexpr int kStageBytes = kBR * L * kCC * 4;
};

// Shared memory a chunk with these line kinds needs for its planes (floats).  Slanted channels come
// in pairs; `ok` is cleared for a chunk with an odd number of them.
template <int L>
__host__ __device__ inline int chunk_plane_floats(const int (&kind)[kCC], bool *ok) {
    using G = Geo<L>;
    int total = 0, ns = 0;
    for (int j = 0; j < kCC; j++) {
        if (kind[j] == KIND_AXIS) total += G::kAxisFloats;
        else if (kind[j] == KIND_DIAG) total += G::kDiagFloats;
        else ns++;
    }
    if (ok) *ok = (ns % 2) == 0;
    return total + (ns / 2) * (G::kSlantInFloats + G::kSlantOutFloats);
}

struct WlParams {
    int N, C, K, nchunks, total_items;
    int flip, add_identity;
    int plane_floats;                    // floats to clear at kernel start (largest chunk)
    int off_wts;                         // [kCC][32] floats, then mover maps and band counters
    int off_stage_bytes, nstg, off_bar_bytes;
    int step_n, step_chunk;              // item += gridDim.x as (n += step_n, chunk += step_chunk, carry)
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
__device__ __noinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, int *err_flag) {
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

// Brings a box into L2 without a destination in shared memory: the later tma_load_4d of the same
// box then costs an L2 hit instead of a trip to HBM.  No completion to wait for.
__device__ __forceinline__ void tma_prefetch_4d(const CUtensorMap *map, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.prefetch.tensor.4d.L2.global.tile [%0, {%1, %2, %3, %4}];"
                 ::"l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void prefetch_l2(const void *p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

template <int I, int N, typename F>
__device__ __forceinline__ void static_for(F &&f) {
    if constexpr (I < N) {
        f(std::integral_constant<int, I>{});
        static_for<I + 1, N>(f);
    }
}

// ---- packed fp32 arithmetic -----------------------------------------------------------------------
// fma.rn.f32x2 issues two independent IEEE fp32 FMAs (the low and the high half of a 64-bit
// register) as ONE instruction; each half is rounded exactly as a scalar fmaf would be.
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ f32x2 ffma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ f32x2 fmul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 ld2(const float *p) { return *reinterpret_cast<const f32x2 *>(p); }
__device__ __forceinline__ void st2(float *p, f32x2 v) { *reinterpret_cast<f32x2 *>(p) = v; }

// Element `w` of a small register array, for a warp-uniform w (a sum of masked terms keeps the
// array in registers, where an indexed read would spill it to local memory).
template <int N>
__device__ __forceinline__ int pick(const int (&v)[N], int w) {
    int r = 0;
#pragma unroll
    for (int j = 0; j < N; j++) r += v[j] * (w == j);
    return r;
}

// ---- plane addressing ----------------------------------------------------------------------------
// Where a mover lane's pixel of a tile lands: addr = a*hb + b*wb + c, with hb, wb the tile's row
// (4 image rows) and column (8 pixels) index, plus `wrapfix` on the second piece of a wrapped
// diagonal (4*hb + tb*wb + tc >= L).  (hi, wi) is the lane's pixel inside the tile.
struct ChanMap {
    int a, b, c;
    int tb, tc, wrapfix;
};

// o: canonical line id; off: plane offset (even); half: 0/1, the channel's half of a slanted pair;
// halo: zero rows above the image rows (slanted input planes).
template <int L>
__device__ __forceinline__ ChanMap make_map(int o, int off, int half, int halo, int hi, int wi) {
    using G = Geo<L>;
    const int kind = canon_kind(o), mode = canon_mode(o);
    const bool fp = (mode & MODE_FP) != 0, tr = (mode & MODE_T) != 0;
    ChanMap m;
    m.tb = 0; m.tc = -(1 << 24); m.wrapfix = 0;
    if (kind == KIND_DIAG) {
        // row r = (h + w') mod L with w' = w or L-1-w; position w' (+ kGap on the wrapped piece)
        const int wi2 = fp ? 7 - wi : wi, s = hi + wi2;
        const int per_wb = 2 * G::GD + 16;                 // r grows by 8, the position by 8 pairs
        m.a = G::GD;
        m.b = fp ? -per_wb : per_wb;
        m.c = off + (s >> 2) * G::GD + ((s >> 1) & 1) * G::QD + (s & 1) + 2 * wi2 + (fp ? (L / 8 - 1) * per_wb : 0);
        m.tb = fp ? -8 : 8;
        m.tc = s + (fp ? 8 * (L / 8 - 1) : 0);
        m.wrapfix = 2 * kGap - (L / 4) * G::GD;
    } else if (kind == KIND_AXIS && !tr) {
        m.a = G::G2;
        m.b = fp ? -16 : 16;
        m.c = off + (hi >> 1) * G::Q2 + (hi & 1) + 2 * (fp ? L - 1 - wi : wi);
    } else if (kind == KIND_AXIS) {
        // row r = w, pair q = r >> 1 = 4*wb + (wi >> 1); position h
        m.a = fp ? -8 : 8;
        m.b = G::G8;
        m.c = off + (wi >> 1) * G::Q8 + (wi & 1) + 2 * (fp ? L - 1 - hi : hi);
    } else if (!tr) {
        // slanted, rows are image rows: r = h + halo
        m.a = G::GS;
        m.b = fp ? -16 : 16;
        m.c = off + half + (halo / 4) * G::GS + hi * G::QS + 2 * (fp ? L - 1 - wi : wi);
    } else {
        // slanted, rows are image columns: r = w + halo = 8*wb + wi + halo
        m.a = fp ? -8 : 8;
        m.b = 2 * G::GS;
        m.c = off + half + (halo / 4 + (wi >> 2)) * G::GS + (wi & 3) * G::QS + 2 * (fp ? L - 1 - hi : hi);
    }
    return m;
}

__device__ __forceinline__ int map_addr(const ChanMap &m, int hb, int wb, int Lside) {
    int a = m.a * hb + m.b * wb + m.c;
    if (m.wrapfix != 0 && 4 * hb + m.tb * wb + m.tc >= Lside) a += m.wrapfix;     // wrapped diagonals only
    return a;
}

// Start of the storage row pair q (rows 2q, 2q+1) of an axis or diagonal plane.
template <int L>
__device__ __forceinline__ int pair_base(int o, int off, int q) {
    using G = Geo<L>;
    if (canon_kind(o) == KIND_DIAG) return off + (q >> 1) * G::GD + (q & 1) * G::QD;
    if (!(canon_mode(o) & MODE_T)) return off + (q >> 1) * G::G2 + (q & 1) * G::Q2;
    return off + (q >> 2) * G::G8 + (q & 3) * G::Q8;
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
// AXIS / DIAG: 1-D convolution along the two storage rows of a pair (length ROW, one row per half),
// in place, with taps at dp = -R .. R (weight pairs wt[dp + R] = (w, w)).  The rows slide through
// a register window: each input is loaded from shared memory once, positions before the row start
// are zeros and loads past its end are skipped.  Results may overwrite the rows as the sweep goes,
// because every later load lies ahead of every earlier store.  GAP (diagonal rows): columns
// rho+1 .. rho+kGap of row rho separate the two diagonals that share it; they stay zero, so results
// there are not written.
template <int R, int ROW, int CH, bool GAP>
__device__ __forceinline__ void row_pair_sweep(float *__restrict__ sm, int base, int rho0, const f32x2 (&wt)[2 * R + 1]) {
    static_assert(ROW % CH == 0 && R + CH <= ROW, "chunking");
    constexpr int WN = CH + 2 * R;
    f32x2 win[WN];                       // win[i] <-> position c*CH - R + i of both rows
#pragma unroll
    for (int i = 0; i < R; i++) win[i] = 0ull;
#pragma unroll
    for (int i = R; i < WN; i++) win[i] = ld2(sm + base + 2 * (i - R));
#pragma unroll 1
    for (int c = 0; c < ROW / CH; c++) {
        f32x2 acc[CH];
#pragma unroll
        for (int o = 0; o < CH; o++) acc[o] = fmul2(wt[0], win[o]);
#pragma unroll
        for (int t = 1; t < 2 * R + 1; t++)
#pragma unroll
            for (int o = 0; o < CH; o++) acc[o] = ffma2(wt[t], win[o + t], acc[o]);
        const int at = base + 2 * c * CH;
#pragma unroll
        for (int o = 0; o < CH; o++) {
            if (!GAP) {
                st2(sm + at + 2 * o, acc[o]);
            } else {
                const int col = c * CH + o;
                const float v0 = __uint_as_float((uint32_t)acc[o]), v1 = __uint_as_float((uint32_t)(acc[o] >> 32));
                if (col <= rho0 || col > rho0 + kGap) sm[at + 2 * o] = v0;
                if (col <= rho0 + 1 || col > rho0 + 1 + kGap) sm[at + 2 * o + 1] = v1;
            }
        }
#pragma unroll
        for (int i = 0; i < 2 * R; i++) win[i] = win[i + CH];
#pragma unroll
        for (int i = 0; i < CH; i++) {
            const int pos = (c + 1) * CH + R + i;                 // uniform over the warp
            win[2 * R + i] = pos < ROW ? ld2(sm + base + 2 * pos) : 0ull;
        }
    }
}

// SLANT.  Offsets (relative to the first output column of a chunk) of the segment of storage row
// 2*rp + e that the chunk's outputs in rows 2*rp + m, m = 0, 1, need: the union over m of the taps
// with line offset d = e - m.
struct SlWin { int lo, hi; };
constexpr int slant_find_row(const LinePlan &p, int d) {
    for (int r = 0; r < p.nrows; r++)
        if (p.row_d[r] == d) return r;
    return -1;
}
template <int JH>
constexpr SlWin slant_window(int e, int CH) {
    const LinePlan &p = LP<KIND_SLANT, JH>::p;
    int lo = 1 << 20, hi = -(1 << 20);
    for (int m = 0; m < 2; m++) {
        const int r = slant_find_row(p, e - m);
        if (r < 0) continue;
        if (p.row_lo[r] < lo) lo = p.row_lo[r];
        if (CH - 1 + p.row_hi[r] > hi) hi = CH - 1 + p.row_hi[r];
    }
    return SlWin{lo, hi};
}

// Pair of slanted channels, one half (L/2 columns) of the plane: chunks c0 .. c0 + L/2/CH - 1 of CH
// columns.  Lane rp owns the row pair rp; every loaded row segment serves both rows and (as a 64-bit
// load) both channels.  Columns that fall off the row are skipped with warp-uniform tests (they
// depend on the chunk index only, and a given load can only ever miss on one side).  `in` is the
// input plane (kHaloRows zero rows above and below the image rows), `out` the result plane.
// w2[k] = (channel A's weight k, channel B's).
template <int L, int JH, int CH>
__device__ __forceinline__ void slant_sweep(float *__restrict__ sm, int in, int out, int rp, int c0,
                                            const f32x2 (&w2)[kMaxTaps]) {
    using P = LP<KIND_SLANT, JH>;
    using G = Geo<L>;
    static_assert((L / 2) % CH == 0, "chunking");
    constexpr int MD = P::p.max_d, NC = (L / 2) / CH, NE = 2 * MD + 2;
    int rb[NE];                          // address of (row 2*rp + e, column 0)
#pragma unroll
    for (int i = 0; i < NE; i++) {
        const int r = 2 * rp + i - MD + kHaloRows;
        rb[i] = in + (r >> 2) * G::GS + (r & 3) * G::QS;
    }
    const int ob0 = out + (rp >> 1) * G::GS + (rp & 1) * 2 * G::QS;          // row 2*rp; row 2*rp + 1 is QS further
#pragma unroll 1
    for (int c = c0; c < c0 + NC; c++) {
        const int cc = c * CH;
        f32x2 acc[2][CH];
#pragma unroll
        for (int m = 0; m < 2; m++)
#pragma unroll
            for (int o = 0; o < CH; o++) acc[m][o] = 0ull;
        static_for<0, NE>([&](auto ei) {
            constexpr int e = decltype(ei)::value - MD;
            constexpr SlWin wn = slant_window<JH>(e, CH);
            if constexpr (wn.hi >= wn.lo) {
                constexpr int WN = wn.hi - wn.lo + 1;
                const float *src = sm + rb[e + MD] + 2 * cc;
                f32x2 win[WN];
#pragma unroll
                for (int i = 0; i < WN; i++) {
                    const int off = wn.lo + i;                          // compile-time after unrolling
                    bool ok = true;
                    if (off < 0) ok = cc >= -off;
                    else if (off + L - CH > L - 1) ok = cc <= L - 1 - off;
                    win[i] = ok ? ld2(src + 2 * off) : 0ull;
                }
                static_for<0, 2>([&](auto mi) {
                    constexpr int m = decltype(mi)::value;
                    constexpr int r = slant_find_row(P::p, e - m);
                    if constexpr (r >= 0) {
                        static_for<0, P::p.ntaps>([&](auto ti) {
                            constexpr int t = decltype(ti)::value;
                            if constexpr (P::p.tap_row[t] == r) {
                                constexpr int dp = P::p.tap_dp[t], k = P::p.tap_k[t];
#pragma unroll
                                for (int o = 0; o < CH; o++) acc[m][o] = ffma2(w2[k], win[o + dp - wn.lo], acc[m][o]);
                            }
                        });
                    }
                });
            }
        });
        float *dst = sm + ob0 + 2 * cc;
#pragma unroll
        for (int m = 0; m < 2; m++)
#pragma unroll
            for (int o = 0; o < CH; o++) st2(dst + m * G::QS + 2 * o, acc[m][o]);
    }
}

// ---------------------------------------------------------------------------------------------------
// y = conv(x) (+ bias); with flip = 1 the weights are read in reverse order, which for stride 1 is
// the input gradient.  Grid: persistent CTAs, items dealt image-major (neighbouring CTAs read
// neighbouring 16-byte halves of the same pixels at the same time).
//
// Shared memory (floats unless noted): planes | wts [8][32] | mover maps (ints: 16 maps x (4 uniform
// + 2 x 32 per lane)) | band counters (ints) | staging ring (bytes) | mbarriers.
//
// Warp roles: warp j owns channel j of the item unless that channel is slanted; slanted channels
// are taken in pairs (in channel order), and the two warps of a pair each evaluate one half of
// the plane for both channels.
// ---------------------------------------------------------------------------------------------------
constexpr int kMaps = 2 * kCC;                    // a restage and a destage map per channel
constexpr int kMapInts = kMaps * 4 + kMaps * 32 * 2;     // uniform a, b, tb, wrapfix per map; c and tc per lane

template <int L, int JH>
__global__ void __launch_bounds__(kThreads, 1)
wline_fprop_kernel(const __grid_constant__ CUtensorMap tmap, const float *__restrict__ wgt,
                   const float *__restrict__ bias, const int8_t *__restrict__ chan, float *__restrict__ y,
                   int *__restrict__ err_flag, const WlParams p) {
    using G = Geo<L>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *sm = reinterpret_cast<float *>(smem_raw);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw + p.off_bar_bytes);
    float *wts = sm + p.off_wts;
    int *map_u = reinterpret_cast<int *>(wts + kCC * 32);      // [kMaps][4]
    int *map_c = map_u + kMaps * 4;                            // [kMaps][32]
    int *map_tc = map_c + kMaps * 32;                          // [kMaps][32]
    int *band_cnt = map_tc + kMaps * 32;                       // [kMaxStages] warps done with a slot
    __shared__ int err_s;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wi = lane & 7, hi = lane >> 3;             // mover lane -> pixel of an 8 x 4 tile
    const int NSTG = p.nstg;

    for (int i = tid; i < p.plane_floats; i += kThreads) sm[i] = 0.f;
    if (tid == 0) {
        for (int s = 0; s < NSTG; s++) { mbar_init(&full[s], 1); band_cnt[s] = 0; }
        err_s = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    const int my_items = (p.total_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    const int total_bands = my_items * G::NB;
    // consumer position (n, chunk) and producer position (pn, pchunk, pb): both advance without divisions
    int n = (int)blockIdx.x / p.nchunks, chunk = (int)blockIdx.x - n * p.nchunks;
    int pn = n, pchunk = chunk, pb = 0, pstage = 0, issued = 0;
    // every thread tracks the producer position; `me` is true in the one thread that issues
    auto issue = [&](bool me) {
        if (me) {
            mbar_expect_tx(&full[pstage], G::kStageBytes);
            tma_load_4d(smem_raw + p.off_stage_bytes + (size_t)pstage * G::kStageBytes, &tmap, &full[pstage],
                        pchunk * kCC, 0, pb * kBR, pn);
        }
        issued++;
        if (++pstage == NSTG) pstage = 0;
        if (++pb == G::NB) {
            pb = 0;
            pn += p.step_n; pchunk += p.step_chunk;
            if (pchunk >= p.nchunks) { pchunk -= p.nchunks; pn++; }
        }
    };
    for (int g = 0; g < NSTG && g < total_bands; g++) issue(tid == 0);

    // Line id of channel (lane & 7) and this thread's weight (channel `warp`, tap `lane`; slot 31 is the
    // bias) of the chunk starting at channel c0, in line order: reversed for lines stored mirrored and
    // for the input gradient.  Loaded one item ahead, so that their latency hides behind the arithmetic.
    auto load_tables = [&](int c0, int &o_lane, float &wv) {
        o_lane = chan[c0 + (lane & (kCC - 1))];
        const int o_w = __shfl_sync(0xffffffffu, o_lane, warp);
        const int pad = p.K / 2, k = lane;
        float v = 0.f;
        if (k < kMaxTaps) {
            int kk = k - kHalf + pad;
            if (kk >= 0 && kk < p.K) {
                const bool rev = ((canon_mode(o_w) & MODE_REV) != 0) != (p.flip != 0);
                if (rev) kk = p.K - 1 - kk;
                v = __ldg(wgt + (size_t)(c0 + warp) * p.K + kk);
                if (p.add_identity && kk == pad) v += 1.f;
            }
        } else {
            v = bias ? __ldg(bias + c0 + warp) : 0.f;
        }
        wv = v;
    };
    int o_lane_next = 0;
    float wv_next = 0.f;
    if (my_items > 0) load_tables(chunk * kCC, o_lane_next, wv_next);

    int stage = 0;                   // ring slot and mbarrier parity of the next band to consume
    uint32_t parity = 0;
    int prev_sig = -1;               // plane layout of the previous item (re-zero when it changes)
#pragma unroll 1
    for (int it = 0; it < my_items; it++) {
        const int c0 = chunk * kCC;

        // ---- per-item tables -----------------------------------------------------------------------------
        // line ids of the four channels, plane offsets, this warp's role
        int o_j[kCC], in_off[kCC], out_off[kCC], half_j[kCC];
#pragma unroll
        for (int j = 0; j < kCC; j++) o_j[j] = __shfl_sync(0xffffffffu, o_lane_next, j);
        int sig = 0, partner = -1;
        {
            int cur = 0, open_in = 0, open_out = 0, open_j = -1;
#pragma unroll
            for (int j = 0; j < kCC; j++) {
                const int kind = canon_kind(o_j[j]);
                sig = sig * 16 + kind * 4 + (canon_mode(o_j[j]) & MODE_T);
                half_j[j] = 0;
                if (kind == KIND_SLANT) {
                    if (open_j < 0) {             // first channel of a pair
                        open_in = cur; open_out = cur + G::kSlantInFloats; open_j = j;
                        cur += G::kSlantInFloats + G::kSlantOutFloats;
                    } else {                      // second channel: same planes, other half of the pairs
                        half_j[j] = 1;
                        if (warp == j) partner = open_j;
                        if (warp == open_j) partner = j;
                        open_j = -1;
                    }
                    in_off[j] = open_in; out_off[j] = open_out;
                } else {
                    in_off[j] = out_off[j] = cur;
                    cur += kind == KIND_AXIS ? G::kAxisFloats : G::kDiagFloats;
                }
            }
        }
        if (sig != prev_sig && prev_sig >= 0)       // another plane layout: stale data would sit where
            for (int i = tid; i < p.plane_floats; i += kThreads) sm[i] = 0.f;     // zeros are expected
        prev_sig = sig;
        const int o_mine = pick(o_j, warp), in_mine = pick(in_off, warp), out_mine = pick(out_off, warp),
                  half_mine = pick(half_j, warp);
        {
            wts[tid] = wv_next;
            const bool slant = canon_kind(o_mine) == KIND_SLANT;
#pragma unroll 1
            for (int q = 0; q < 2; q++) {                  // q = 0: restage map, q = 1: destage map
                const ChanMap m = make_map<L>(o_mine, q ? out_mine : in_mine, half_mine,
                                              (!q && slant) ? kHaloRows : 0, hi, wi);
                const int mi = q * kCC + warp;
                map_c[mi * 32 + lane] = m.c;
                map_tc[mi * 32 + lane] = m.tc;
                if (lane == 0) {
                    map_u[mi * 4 + 0] = m.a; map_u[mi * 4 + 1] = m.b; map_u[mi * 4 + 2] = m.tb; map_u[mi * 4 + 3] = m.wrapfix;
                }
            }
        }
        __syncthreads();

        // ---- restage: staging bands -> planes ---------------------------------------------------------
        // Warp tx moves tile column tx of every band (tiles of 8 pixels x 4 rows).  A lane carries one
        // 16-byte half (4 channels) of two pixels of the tile, so that the 32 lanes of one load or
        // store instruction cover 16 whole pixels: full 32-byte sectors in global memory, contiguous
        // 256-byte runs in the staging ring.  All plane addresses advance by per-lane constants, and
        // a wrapped diagonal switches to its second piece from tile row `thr` on.
        const bool mover = warp < G::kTilesX;           // tile column tx = warp
        const int mhalf = lane & 1, mpix = lane >> 1;   // channels 4*mhalf .. +3 of tile pixels mpix, mpix + 16
        const int mhi = mpix >> 3, mwi = mpix & 7;      // pixel mpix = (row mhi, column mwi); mpix + 16 is two rows down
        if (mover) {
            int ra[4][2], thr[4][2], aj[4], wf[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int j = 4 * mhalf + i;
                aj[i] = map_u[j * 4 + 0];
                wf[i] = map_u[j * 4 + 3];
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    const int px = mpix + 16 * u;
                    ra[i][u] = map_c[j * 32 + px] + map_u[j * 4 + 1] * warp;
                    thr[i][u] = (L - map_tc[j * 32 + px] - map_u[j * 4 + 2] * warp + 3) >> 2;
                }
            }
#pragma unroll 1
            for (int b = 0; b < G::NB; b++) {
                if (err_s == 0 && !mbar_wait(&full[stage], parity, err_flag)) err_s = 1;
                const float4 *stg = reinterpret_cast<const float4 *>(smem_raw + p.off_stage_bytes + (size_t)stage * G::kStageBytes) +
                                    (mhi * L + mwi + 8 * warp) * 2 + mhalf;
                float4 v[kBR / 4][2];
#pragma unroll
                for (int ty = 0; ty < kBR / 4; ty++)
#pragma unroll
                    for (int u = 0; u < 2; u++) v[ty][u] = stg[(4 * ty + 2 * u) * L * 2];
#pragma unroll
                for (int ty = 0; ty < kBR / 4; ty++) {
                    const int hb = b * (kBR / 4) + ty;
#pragma unroll
                    for (int u = 0; u < 2; u++) {
                        const float f[4] = {v[ty][u].x, v[ty][u].y, v[ty][u].z, v[ty][u].w};
#pragma unroll
                        for (int i = 0; i < 4; i++)
                            sm[ra[i][u] + ty * aj[i] + (hb >= thr[i][u] ? wf[i] : 0)] = f[i];
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int u = 0; u < 2; u++) ra[i][u] += (kBR / 4) * aj[i];
                // the warp that finishes a slot last refills it: no CTA-wide barrier per band
                __syncwarp();
                int last = 0;
                if (lane == 0) {
                    __threadfence_block();
                    last = atomicAdd(&band_cnt[stage], 1) == G::kTilesX - 1;
                    if (last) band_cnt[stage] = 0;
                }
                if (issued < total_bands) issue(last != 0);
                if (++stage == NSTG) { stage = 0; parity ^= 1; }
            }
        } else {
            // keep the ring bookkeeping in step
#pragma unroll 1
            for (int b = 0; b < G::NB; b++) {
                if (issued < total_bands) issue(false);
                if (++stage == NSTG) { stage = 0; parity ^= 1; }
            }
        }
        __syncthreads();

        // The ring only holds the next item's first bands; ask for the rest of it to be brought into
        // L2 now, one compute and one destage phase ahead, and load its line ids and weights.
        if (it + 1 < my_items) {
            int nn = n + p.step_n, nc = chunk + p.step_chunk;
            if (nc >= p.nchunks) { nc -= p.nchunks; nn++; }
            if (tid >= NSTG && tid < G::NB) tma_prefetch_4d(&tmap, nc * kCC, 0, tid * kBR, nn);
            load_tables(nc * kCC, o_lane_next, wv_next);
        }

        // ---- compute ----------------------------------------------------------------------------------------
        {
            const int kind = canon_kind(o_mine);
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
                if (kind == KIND_AXIS) {
                    f32x2 wt[2 * JH + 1];
#pragma unroll
                    for (int t = 0; t < 2 * JH + 1; t++) wt[t] = pack2(w[t - JH + kHalf], w[t - JH + kHalf]);
                    row_pair_sweep<JH, L, 14, false>(sm, pair_base<L>(o_mine, in_mine, lane), 2 * lane, wt);
                } else if (kind == KIND_DIAG) {
                    using PD = LP<KIND_DIAG, JH>;
                    merge_weights<KIND_DIAG, JH>(w);
                    f32x2 wt[2 * kGap + 1];
#pragma unroll
                    for (int t = 0; t < 2 * kGap + 1; t++) wt[t] = 0ull;
                    static_for<0, PD::p.ntaps>([&](auto ti) {
                        constexpr int t = decltype(ti)::value;
                        constexpr int at = PD::p.tap_dp[t] + kGap, k = PD::p.tap_k[t];
                        wt[at] = pack2(w[k], w[k]);
                    });
                    row_pair_sweep<kGap, G::LD, 11, true>(sm, pair_base<L>(o_mine, in_mine, lane), 2 * lane, wt);
                } else if (partner >= 0) {
                    // both channels' weights: mine from registers, the partner's from shared memory
                    float wp[kMaxTaps];
                    {
                        const float4 *pp = reinterpret_cast<const float4 *>(wts + partner * 32);
#pragma unroll
                        for (int q = 0; q < 8; q++) {
                            const float4 v = pp[q];
                            wp[4 * q] = v.x; wp[4 * q + 1] = v.y; wp[4 * q + 2] = v.z;
                            if (4 * q + 3 < kMaxTaps) wp[4 * q + 3] = v.w;
                        }
                    }
                    merge_weights<KIND_SLANT, JH>(w);
                    merge_weights<KIND_SLANT, JH>(wp);
                    f32x2 w2[kMaxTaps];
#pragma unroll
                    for (int k = 0; k < kMaxTaps; k++) w2[k] = half_mine ? pack2(wp[k], w[k]) : pack2(w[k], wp[k]);
                    // first warp of the pair: left half of the plane, second warp: right half
                    slant_sweep<L, JH, 7>(sm, in_mine, out_mine, lane, half_mine ? (L / 2) / 7 : 0, w2);
                }
            }
        }
        __syncthreads();

        // ---- destage: planes -> NHWC, bias added ---------------------------------------------------------
        if (mover) {
            int rd[4][2], thr[4][2], aj[4], wf[4];
            float bv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int mi = kCC + 4 * mhalf + i;
                aj[i] = map_u[mi * 4 + 0];
                wf[i] = map_u[mi * 4 + 3];
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    const int px = mpix + 16 * u;
                    rd[i][u] = map_c[mi * 32 + px] + map_u[mi * 4 + 1] * warp;
                    thr[i][u] = (L - map_tc[mi * 32 + px] - map_u[mi * 4 + 2] * warp + 3) >> 2;
                }
                bv[i] = wts[(4 * mhalf + i) * 32 + 31];
            }
            float *yp = y + ((size_t)n * L * L) * p.C + c0 + ((size_t)mhi * L + mwi + 8 * warp) * p.C + 4 * mhalf;
            const size_t ystep = (size_t)4 * L * p.C, yrow2 = (size_t)2 * L * p.C;
#pragma unroll 2
            for (int hb = 0; hb < L / 4; hb++) {
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    float f[4];
#pragma unroll
                    for (int i = 0; i < 4; i++) f[i] = sm[rd[i][u] + (hb >= thr[i][u] ? wf[i] : 0)] + bv[i];
                    *reinterpret_cast<float4 *>(yp + u * yrow2) = make_float4(f[0], f[1], f[2], f[3]);
                }
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int u = 0; u < 2; u++) rd[i][u] += aj[i];
                yp += ystep;
            }
        }
        __syncthreads();
        n += p.step_n; chunk += p.step_chunk;
        if (chunk >= p.nchunks) { chunk -= p.nchunks; n++; }
    }
}

}  // namespace wl
}  // namespace o1d
