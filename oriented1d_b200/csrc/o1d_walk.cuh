// "Walker" kernels: stride-1 forward / input gradient on square NHWC fp32 maps whose channels
// all lie on the eight canonical lines, without any re-layout of the data.
//
// One persistent CTA per SM owns two shared-memory tiles, each holding a whole work item
// (image n, 8 consecutive channels) exactly as it lies in global memory: [rows][P pixels][8 ch],
// P = L+1 (the extra column is outside the tensor and arrives as zeros; an odd pitch spreads
// vertical neighbours over the banks).  A producer warp moves items with TMA: tile t is loaded
// band by band (8 rows per copy), computed IN PLACE by eleven compute warps, and stored back band by
// band with TMA stores; the next item's bands are loaded into the tile as soon as the store of the
// same band has read it.  While one tile computes, the other one drains and refills, so the HBM
// traffic of one item hides behind the arithmetic of its neighbour.
//
// Arithmetic, per channel, by line kind (o1d_lines.cuh):
//   * axis (0, 90 degrees) and diagonal (45, 135) channels: a thread walks one image line (row,
//     column or diagonal) with the last 38 inputs in registers; per round it loads 8 new inputs,
//     forms 8 outputs of 31 FMAs each and shifts the window by 8 registers.  The result of position
//     i overwrites cell i of the tile: that cell belongs to this line of this channel alone and was
//     read into the window 16 positions earlier.  A warp holds (channels of one kind in the chunk) x
//     (32 / that many) lines; the weights are per lane; tasks are handed out from a shared counter.
//   * slanted channels (22.5, 67.5, 112.5, 157.5 degrees): the channel's plane is first copied out
//     of the tile into a small fp32 plane in the canonical frame of the 22.5 degree line (transposed
//     and/or mirrored as o1d_lines.cuh prescribes) with zero rows and columns around it; a thread
//     then owns two adjacent rows and walks 14 columns with a 12-row x 6-column register window
//     (one load per input row per step, 58 FMAs), writing its outputs straight into the tile.
// Every wait is bounded; a wait that runs out raises the device flag and the CTA drains.
//
// The reference computes the same sums one output per thread with sincosf per tap and four bounds
// tests (models/dwoconv1d_specialized/kernels/kernels.h:201-291).
#pragma once

#include <cuda.h>

#include <type_traits>

#include "o1d_common.cuh"
#include "o1d_lines.cuh"

namespace o1d {
namespace walk {

constexpr int kCC = 8;                 // channels per item (32 bytes per pixel)
constexpr int kBandRows = 8;           // rows per TMA copy
constexpr int kMaxBands = 8;
constexpr int kSlantWarps = 4, kComputeWarps = 11;     // with the producer: 12 warps, registers are granted in fours
constexpr int kThreads = (kComputeWarps + 1) * 32;   // + the producer warp
constexpr int kWin = kMaxTaps, kReach = kHalf;
constexpr int kLineBlock = 8;          // outputs a line thread forms per round
constexpr int kSeg = 14;               // columns one slant thread walks
constexpr int kSpan = 6;               // columns of an input row a slant thread keeps
constexpr int kHaloRows = 6, kHaloCols = 14;
constexpr uint32_t kSpinLimit = 1u << 22;

struct WalkParams {
    int N, L, C, K, nchunks, total_items;
    int P, nbands, band_bytes, tile_bytes;
    int flip, add_identity;
    int off_plane, off_wts, off_misc;      // byte offsets in dynamic shared memory (tiles at 0 and tile_bytes)
};

template <int I, int N, typename F>
__device__ __forceinline__ void sfor(F &&f) {
    if constexpr (I < N) {
        f(std::integral_constant<int, I>{});
        sfor<I + 1, N>(f);
    }
}

// ---- slanted base line: unique taps and the window a two-row thread needs -------------------
struct SlantTab {
    int ntaps;
    int uniq[kMaxTaps];                 // canonical tap k -> unique tap (or -1)
    int tap_dl[kMaxTaps], tap_dp[kMaxTaps];
    int min_d, max_d, nin;              // input rows, relative to the first output row: min_d .. max_d+1
    int lo2[16], hi2[16];               // per input row: columns the two output rows touch
};
constexpr SlantTab make_slant_tab(int JH) {
    SlantTab t{};
    const LinePlan lp = make_line_plan(KIND_SLANT, JH);
    t.ntaps = lp.ntaps;
    for (int k = 0; k < kMaxTaps; k++) {
        t.uniq[k] = -1;
        if (lp.merge_into[k] >= 0)
            for (int u = 0; u < lp.ntaps; u++)
                if (lp.tap_k[u] == lp.merge_into[k]) t.uniq[k] = u;
    }
    t.min_d = 99; t.max_d = -99;
    for (int r = 0; r < lp.nrows; r++) {
        if (lp.row_d[r] < t.min_d) t.min_d = lp.row_d[r];
        if (lp.row_d[r] > t.max_d) t.max_d = lp.row_d[r];
    }
    for (int u = 0; u < lp.ntaps; u++) { t.tap_dl[u] = lp.row_d[lp.tap_row[u]]; t.tap_dp[u] = lp.tap_dp[u]; }
    t.nin = t.max_d - t.min_d + 2;
    for (int i = 0; i < 16; i++) { t.lo2[i] = 99; t.hi2[i] = -99; }
    for (int r = 0; r < lp.nrows; r++)
        for (int rr = 0; rr < 2; rr++) {
            const int ri = lp.row_d[r] + rr - t.min_d;
            if (lp.row_lo[r] < t.lo2[ri]) t.lo2[ri] = lp.row_lo[r];
            if (lp.row_hi[r] > t.hi2[ri]) t.hi2[ri] = lp.row_hi[r];
        }
    return t;
}
constexpr bool slant_tab_fits(const SlantTab &t) {
    if (t.nin > 16 || -t.min_d >= kHaloRows || t.max_d + 1 > kHaloRows) return false;
    for (int i = 0; i < t.nin; i++)
        if (t.hi2[i] - t.lo2[i] + 1 > kSpan || t.hi2[i] + 1 > kHaloCols) return false;
    return true;
}
template <int JH> struct ST {
    static constexpr SlantTab t = make_slant_tab(JH);
    static_assert(slant_tab_fits(t), "slant window does not fit the register window / plane halo");
};
constexpr int floor_half(int v) { return v >= 0 ? v / 2 : -((1 - v) / 2); }

// ---- primitives --------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool bar_wait(uint64_t *bar, uint32_t parity, int *err_flag) {
    uint32_t ok = 0;
    for (uint32_t i = 0; i < kSpinLimit && !ok; i++) {
        asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(ok) : "r"(s32(bar)), "r"(parity) : "memory");
        if (!ok) __nanosleep(64);        // leave the issue slots to the warps that have work
    }
    if (!ok) atomicExch(err_flag, 1);
    return ok != 0;
}
__device__ __forceinline__ void named_sync(int id, int count) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}
// Shared-memory accesses by 32-bit address, kept in program order (the tile is updated in place).
__device__ __forceinline__ float lds(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(a));
    return v;
}
template <int IMM>
__device__ __forceinline__ float lds_imm(uint32_t a) {
    float v;
    asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(a), "n"(IMM));
    return v;
}
__device__ __forceinline__ void sts(uint32_t a, float v) { asm volatile("st.shared.f32 [%0], %1;" ::"r"(a), "f"(v)); }
// value at `a` when i < n (signed), else the word at `z` (a cell that holds zero)
__device__ __forceinline__ float lds_if_lt(uint32_t a, uint32_t z, int i, int n) {
    float v;
    asm volatile("{\n .reg .pred q;\n .reg .u32 t;\n setp.lt.s32 q, %3, %4;\n selp.u32 t, %1, %2, q;\n ld.shared.f32 %0, [t];\n}\n"
                 : "=f"(v) : "r"(a), "r"(z), "r"(i), "r"(n));
    return v;
}
__device__ __forceinline__ void sts_if_lt(uint32_t a, float v, int i, int n) {
    asm volatile("{\n .reg .pred q;\n setp.lt.s32 q, %2, %3;\n @q st.shared.f32 [%0], %1;\n}\n" ::"r"(a), "f"(v), "r"(i), "r"(n));
}

// ---- axis / diagonal channels --------------------------------------------------------------------
// A lane walks positions 0..n-1 of one line: byte address a0 + q*s4.  Positions outside read zero.
// `chs` lists the task's channel slots (4 bits each), nch of them, padded to 1 << lg lanes;
// `diag`: the lines are the 2L-1 diagonals, else the L rows / columns.
template <int L>
__device__ __forceinline__ void line_task(uint32_t tile_s, const float *__restrict__ wtab, uint32_t idpack, uint32_t chs,
                                          int nch, int lg, bool diag, int task, int lane) {
    constexpr int W = kWin, R = kReach, P = L | 1, P32 = P * kCC * 4;
    const int ncp = 1 << lg, lpt = 32 >> lg;
    const int si = lane & (ncp - 1), line = task * lpt + (lane >> lg);
    const bool act = si < nch && line < (diag ? 2 * L - 1 : L);
    const int c = (chs >> (4 * si)) & 15, id = (idpack >> (4 * c)) & 15;
    int a0 = 0, s4 = kCC * 4, n = 0;
    if (act) {
        if (id == 0) { a0 = line * P32; n = L; }
        else if (id == 4) { a0 = line * kCC * 4; s4 = P32; n = L; }
        else if (id == 6) {      // down-right, w - h = d
            const int d = line - (L - 1);
            a0 = d >= 0 ? d * kCC * 4 : -d * P32; n = L - (d < 0 ? -d : d); s4 = P32 + kCC * 4;
        } else {                 // id 2, down-left, w + h = e
            const int e = line;
            a0 = e <= L - 1 ? e * kCC * 4 : (e - (L - 1)) * P32 + (L - 1) * kCC * 4; n = e <= L - 1 ? e + 1 : 2 * L - 1 - e;
            s4 = P32 - kCC * 4;
        }
        a0 += c * 4;
    }
    const int T = __reduce_max_sync(0xffffffffu, n);
    const uint32_t zero_cell = tile_s + L * kCC * 4;       // (row 0, column L): outside the tensor, arrives as zero
    float w[W];
#pragma unroll
    for (int k = 0; k < W; k++) w[k] = act ? wtab[c * 32 + k] : 0.f;
    const float bias = act ? wtab[c * 32 + 31] : 0.f;
    // win[k] = x[i0 - R + k], k = 0 .. 2R + RB - 1, for the RB outputs i0 .. i0+RB-1 of one round.  A round
    // loads RB new inputs, forms RB outputs and shifts the window by RB registers: the loop body stays a
    // few KB of code (a window that rotates through an unrolled body of 31 steps does not fit the
    // instruction cache once several warps run it at different phases).
    constexpr int RB = kLineBlock;
    float win[2 * R + RB];
    uint32_t lead = tile_s + a0;                           // address of position i0 + R + r while loading
    sfor<0, 2 * R>([&](auto kc) {
        constexpr int k = decltype(kc)::value, q = k - R;
        if constexpr (q < 0) win[k] = 0.f;
        else { win[k] = lds_if_lt(lead, zero_cell, q, n); lead += s4; }
    });
    uint32_t cur = tile_s + a0;                            // address of position i0 + r while storing
    for (int i0 = 0; i0 < T; i0 += RB) {
        sfor<0, RB>([&](auto rc) {
            constexpr int r = decltype(rc)::value;
            win[2 * R + r] = lds_if_lt(lead, zero_cell, i0 + R + r, n);
            lead += s4;
        });
        sfor<0, RB>([&](auto rc) {
            constexpr int r = decltype(rc)::value;
            float p0 = bias, p1 = 0.f;
            sfor<0, W>([&](auto kc) {
                constexpr int k = decltype(kc)::value;
                if constexpr (k % 2 == 0) p0 = fmaf(w[k], win[r + k], p0);
                else p1 = fmaf(w[k], win[r + k], p1);
            });
            sts_if_lt(cur, p0 + p1, i0 + r, n);
            cur += s4;
        });
#pragma unroll
        for (int k = 0; k < 2 * R; k++) win[k] = win[k + RB];
    }
}

// ---- slanted channels ----------------------------------------------------------------------------
// Tile byte offset of canonical-frame cell (a, b) of channel c: 4c + ofs + a*SA + b*SB.
struct SlantFrame { int ofs, SA, SB; };
template <int L>
__device__ __forceinline__ SlantFrame slant_frame(int id) {
    constexpr int P32 = (L | 1) * kCC * 4, C4 = kCC * 4;
    switch (id) {
        case 1: return SlantFrame{0, P32, C4};
        case 3: return SlantFrame{0, C4, P32};
        case 5: return SlantFrame{(L - 1) * P32, C4, -P32};
        default: return SlantFrame{(L - 1) * C4, P32, -C4};
    }
}
template <int L> struct Plane {
    static constexpr int kPitch = L + kHaloCols, kRows = L + 2 * kHaloRows;
    static constexpr int kWords = kRows * kPitch + kRows / 2 + 1;
    __host__ __device__ static constexpr int word(int a, int b) { return (a + kHaloRows) * kPitch + ((a + kHaloRows) >> 1) + b; }
    // offset of input row rho (relative to an even row 2*pr) from that row's start
    __host__ __device__ static constexpr int row_ofs(int rho) { return rho * kPitch + floor_half(rho); }
};

template <int L, int JH>
__device__ __forceinline__ void slant_task(uint32_t tile_s, uint32_t plane_s, const float *__restrict__ wrow, int c,
                                           const SlantFrame fr, int task, int lane, uint32_t dummy_s) {
    constexpr SlantTab t = ST<JH>::t;
    constexpr int NT = t.ntaps, NIN = t.nin, S = kSpan;
    using PL = Plane<L>;
    constexpr int pairs = L / 2, nseg = L / kSeg, jpt = pairs * (32 / pairs), njobs = pairs * nseg;
    const int job = task * jpt + lane;
    const bool act = lane < jpt && job < njobs;
    const int pr = act ? job % pairs : 0, sg = act ? job / pairs : 0;
    const int bs = sg * kSeg;
    float w[NT];
#pragma unroll
    for (int u = 0; u < NT; u++) w[u] = wrow[u];
    const float bias = wrow[31];
    uint32_t pb = plane_s + 4 * (PL::word(2 * pr, 0) + bs);          // byte address of plane cell (2*pr, b)
    float win[NIN][S];
    sfor<0, NIN>([&](auto rc) {
        constexpr int ri = decltype(rc)::value, rho = ri + t.min_d, first = t.hi2[ri] - (S - 1);
        sfor<0, S>([&](auto xc) {
            constexpr int x = decltype(xc)::value;
            win[ri][x] = (bs + first + x >= 0) ? lds_imm<4 * (PL::row_ofs(rho) + first + x)>(pb) : 0.f;
        });
    });
    const int SA = act ? fr.SA : 0, SB = act ? fr.SB : 0;
    uint32_t out0 = act ? tile_s + 4 * c + fr.ofs + (2 * pr) * fr.SA + bs * fr.SB : dummy_s;
    int b = 0;
    while (b < kSeg) {
        sfor<0, S>([&](auto uc) {
            constexpr int U = decltype(uc)::value;
            if (b < kSeg) {
                float acc[2][2] = {{bias, 0.f}, {bias, 0.f}};
                sfor<0, NT>([&](auto tc) {
                    constexpr int u = decltype(tc)::value;
                    sfor<0, 2>([&](auto rrc) {
                        constexpr int rr = decltype(rrc)::value, ri = t.tap_dl[u] + rr - t.min_d;
                        constexpr int x = t.tap_dp[u] - (t.hi2[ri] - (S - 1));
                        static_assert(x >= 0 && x < S, "tap outside the window");
                        acc[rr][u & 1] = fmaf(w[u], win[ri][(U + x) % S], acc[rr][u & 1]);
                    });
                });
                sfor<0, 2>([&](auto rrc) {
                    constexpr int rr = decltype(rrc)::value;
                    const float o = acc[rr][0] + acc[rr][1];
                    sts(out0 + rr * SA, o);
                });
                sfor<0, NIN>([&](auto rc) {
                    constexpr int ri = decltype(rc)::value, rho = ri + t.min_d;
                    win[ri][U] = lds_imm<4 * (PL::row_ofs(rho) + t.hi2[ri] + 1)>(pb);
                });
                b++; pb += 4; out0 += SB;
            }
        });
    }
}

// Weight of stored tap kc (canonical 31-tap indexing) of a channel with line id `id`.
__device__ __forceinline__ float stored_weight(const float *__restrict__ wc, int K, int kc, int mode_rev, int flip) {
    int jj = kc - kHalf;
    if (mode_rev) jj = -jj;
    if (flip) jj = -jj;
    const int half = K >> 1;
    return (jj >= -half && jj <= half) ? __ldg(wc + jj + half) : 0.f;
}

template <int L, int JH>
__global__ void __launch_bounds__(kThreads, 1)
walk_fprop_kernel(const __grid_constant__ CUtensorMap in_map, const __grid_constant__ CUtensorMap out_map,
                  const float *__restrict__ wgt, const float *__restrict__ bias, const int8_t *__restrict__ chan,
                  int *err_flag, const WalkParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    using PL = Plane<L>;
    float *plane = reinterpret_cast<float *>(smem + p.off_plane);
    float *wtab = reinterpret_cast<float *>(smem + p.off_wts);          // [2][8][32]
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + p.off_misc);   // [2]
    uint64_t *done = full + 2;                                           // [2]
    int *queue = reinterpret_cast<int *>(done + 2);                      // [2] next line task of the tile
    float *dummy = reinterpret_cast<float *>(queue + 2);                 // word the idle lanes of a slant task write
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int s = 0; s < 2; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&full[s])), "r"(1));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(&done[s])), "r"(kComputeWarps));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int e = tid; e < PL::kWords; e += kThreads) plane[e] = 0.f;
    __syncthreads();
    const int my_items = (p.total_items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;

    if (warp == kComputeWarps) {          // ---- producer: lane 0 issues every copy ----
        if (lane == 0) {
            auto coords = [&](int it, int &n, int &ch) {
                const int item = blockIdx.x + it * gridDim.x;
                n = item / p.nchunks; ch = item - n * p.nchunks;
            };
            auto load_band = [&](int it, int b) {
                int n, ch; coords(it, n, ch);
                const int t = it & 1;
                asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                             ::"r"(s32(smem + (size_t)t * p.tile_bytes + (size_t)b * p.band_bytes)), "l"(&in_map), "r"(s32(&full[t])),
                               "r"(ch * kCC), "r"(0), "r"(b * kBandRows), "r"(n) : "memory");
            };
            auto expect = [&](int it) {
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(&full[it & 1])), "r"(p.tile_bytes) : "memory");
            };
            for (int it = 0; it < 2 && it < my_items; it++) {
                expect(it);
                for (int b = 0; b < p.nbands; b++) load_band(it, b);
            }
            for (int it = 0; it < my_items; it++) {
                const int t = it & 1;
                if (!bar_wait(&done[t], (it >> 1) & 1, err_flag)) break;     // tile t holds the results of item it
                int n, ch; coords(it, n, ch);
                for (int b = 0; b < p.nbands; b++) {
                    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                                 ::"l"(&out_map), "r"(s32(smem + (size_t)t * p.tile_bytes + (size_t)b * p.band_bytes)),
                                   "r"(ch * kCC), "r"(0), "r"(b * kBandRows), "r"(n) : "memory");
                    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                }
                if (it + 2 < my_items) {
                    expect(it + 2);
                    // band b may be overwritten once its store (one of the nbands newest groups) has read it
                    for (int b = 0; b < p.nbands; b++) {
                        switch (p.nbands - 1 - b) {
                            case 7: asm volatile("cp.async.bulk.wait_group.read 7;" ::: "memory"); break;
                            case 6: asm volatile("cp.async.bulk.wait_group.read 6;" ::: "memory"); break;
                            case 5: asm volatile("cp.async.bulk.wait_group.read 5;" ::: "memory"); break;
                            case 4: asm volatile("cp.async.bulk.wait_group.read 4;" ::: "memory"); break;
                            case 3: asm volatile("cp.async.bulk.wait_group.read 3;" ::: "memory"); break;
                            case 2: asm volatile("cp.async.bulk.wait_group.read 2;" ::: "memory"); break;
                            case 1: asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); break;
                            default: asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); break;
                        }
                        load_band(it + 2, b);
                    }
                }
            }
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
        }
        return;
    }

    // ---- compute warps ----
    bool failed = false;
    for (int it = 0; it < my_items; it++) {
        const int t = it & 1;
        const int item = blockIdx.x + it * gridDim.x, chunk = item % p.nchunks;
        const uint32_t tile_s = s32(smem + (size_t)t * p.tile_bytes);
        float *wt = wtab + t * (kCC * 32);
        // line ids of the chunk's channels, and the lists of channel slots by kind
        uint32_t idpack = 0, axis = 0, diag = 0, slant = 0;
        int nA = 0, nD = 0, nS = 0;
#pragma unroll
        for (int j = 0; j < kCC; j++) {
            const int id = chan[chunk * kCC + j] & 7;
            idpack |= (uint32_t)id << (4 * j);
            if (id & 1) { slant |= (uint32_t)j << (4 * nS); nS++; }
            else if (id & 2) { diag |= (uint32_t)j << (4 * nD); nD++; }
            else { axis |= (uint32_t)j << (4 * nA); nA++; }
        }
        if (tid < kCC * 32) {   // weight table of the item: thread (channel, entry)
            const int ch = tid >> 5, idx = tid & 31, cg = chunk * kCC + ch, id = (idpack >> (4 * ch)) & 15;
            const float *wc = wgt + (size_t)cg * p.K;
            float v = 0.f;
            if (idx == 31) v = bias ? __ldg(bias + cg) : 0.f;
            else if (id & 1) {
                constexpr SlantTab st = ST<JH>::t;
                const int rev = (id == 3) ? 1 : 0;            // MODE_REV of the slanted lines
                sfor<0, kMaxTaps>([&](auto kc) {
                    constexpr int k = decltype(kc)::value, u = st.uniq[k];
                    if constexpr (u >= 0) { if (u == idx) v += stored_weight(wc, p.K, k, rev, p.flip); }
                });
                if (p.add_identity && idx == st.uniq[kHalf]) v += 1.f;     // the identity tap rides on the centre weight
            } else {
                const int d = idx - kHalf, half = p.K >> 1;
                sfor<0, kMaxTaps>([&](auto kc) {
                    constexpr int k = decltype(kc)::value, j = k - kHalf, dd = kCanonDh[2][k];
                    const int pos = id == 0 ? j : id == 4 ? -j : dd;
                    if (pos == d && j >= -half && j <= half) v += __ldg(wc + (p.flip ? -j : j) + half);
                });
                if (p.add_identity && d == 0) v += 1.f;
            }
            wt[ch * 32 + idx] = v;
            if (tid == 0) queue[t] = 0;
        }
        named_sync(1, kComputeWarps * 32);
        if (!failed && !bar_wait(&full[t], (it >> 1) & 1, err_flag)) failed = true;
        if (warp < kSlantWarps) {
            for (int s = 0; s < nS; s++) {
                const int c = (slant >> (4 * s)) & 15, id = (idpack >> (4 * c)) & 15;
                const SlantFrame fr = slant_frame<L>(id);
                if (!failed) {
                    for (int a = warp; a < L; a += kSlantWarps) {
                        const uint32_t src = tile_s + 4 * c + fr.ofs + a * fr.SA;
                        float *dst = plane + PL::word(a, 0);
                        for (int b = lane; b < L; b += 32) dst[b] = lds(src + b * fr.SB);
                    }
                }
                named_sync(2, kSlantWarps * 32);
                if (!failed) {
                    constexpr int pairs = L / 2, jpt = pairs * (32 / pairs), ntask = (pairs * (L / kSeg) + jpt - 1) / jpt;
                    for (int task = warp; task < ntask; task += kSlantWarps)
                        slant_task<L, JH>(tile_s, s32(plane), wt + c * 32, c, fr, task, lane, s32(dummy));
                }
                named_sync(2, kSlantWarps * 32);
            }
        }
        if (!failed) {      // rows, columns and diagonals: tasks handed out from a counter
            const int lgA = nA <= 1 ? 0 : nA <= 2 ? 1 : nA <= 4 ? 2 : 3, lgD = nD <= 1 ? 0 : nD <= 2 ? 1 : nD <= 4 ? 2 : 3;
            const int ntA = nA ? (L + (32 >> lgA) - 1) / (32 >> lgA) : 0;
            const int ntD = nD ? (2 * L - 1 + (32 >> lgD) - 1) / (32 >> lgD) : 0;
            for (;;) {
                int task = 0;
                if (lane == 0) task = atomicAdd(&queue[t], 1);
                task = __shfl_sync(0xffffffffu, task, 0);
                if (task >= ntA + ntD) break;
                const bool dg = task >= ntA;
                line_task<L>(tile_s, wt, idpack, dg ? diag : axis, dg ? nD : nA, dg ? lgD : lgA, dg, dg ? task - ntA : task, lane);
            }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(s32(&done[t])) : "memory");
    }
}

}  // namespace walk
}  // namespace o1d
