// Compile-time description of the eight canonical rasterised lines (angles i*pi/8, K<=31)
// and of how each is brought to one of three "base" shapes by re-indexing the image.
//
// The tables are the reference's rasterisation dh=(int)(-sinf(t)*j), dw=(int)(cosf(t)*j)
// (models/dwoconv1d_reference/kernels/kernels.cpp:43-44) evaluated for t = (float)(i*pi/8),
// j = -15..15.  A shorter kernel uses the centre of the same table.  The plan builder
// re-derives every class at run time and marks it canonical only if it matches these
// tables tap for tap, so a mismatch can only route a layer to the general kernels, never
// produce a wrong line.
#pragma once

#include <stdint.h>

namespace o1d {

constexpr int kMaxTaps = 31;   // taps of the tiled kernels (K <= 31)
constexpr int kHalf = 15;

constexpr int8_t kCanonDh[8][kMaxTaps] = {
    {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0},
    {5, 5, 4, 4, 4, 3, 3, 3, 2, 2, 1, 1, 1, 0, 0, 0, 0, 0, -1, -1, -1, -2, -2, -3, -3, -3, -4, -4, -4, -5, -5},
    {10, 9, 9, 8, 7, 7, 6, 5, 4, 4, 3, 2, 2, 1, 0, 0, 0, -1, -2, -2, -3, -4, -4, -5, -6, -7, -7, -8, -9, -9, -10},
    {13, 12, 12, 11, 10, 9, 8, 7, 6, 5, 4, 3, 2, 1, 0, 0, 0, -1, -2, -3, -4, -5, -6, -7, -8, -9, -10, -11, -12, -12, -13},
    {15, 14, 13, 12, 11, 10, 9, 8, 7, 6, 5, 4, 3, 2, 1, 0, -1, -2, -3, -4, -5, -6, -7, -8, -9, -10, -11, -12, -13, -14, -15},
    {13, 12, 12, 11, 10, 9, 8, 7, 6, 5, 4, 3, 2, 1, 0, 0, 0, -1, -2, -3, -4, -5, -6, -7, -8, -9, -10, -11, -12, -12, -13},
    {10, 9, 9, 8, 7, 7, 6, 5, 4, 4, 3, 2, 2, 1, 0, 0, 0, -1, -2, -2, -3, -4, -4, -5, -6, -7, -7, -8, -9, -9, -10},
    {5, 5, 4, 4, 4, 3, 3, 3, 2, 2, 1, 1, 1, 0, 0, 0, 0, 0, -1, -1, -1, -2, -2, -3, -3, -3, -4, -4, -4, -5, -5},
};
constexpr int8_t kCanonDw[8][kMaxTaps] = {
    {-15, -14, -13, -12, -11, -10, -9, -8, -7, -6, -5, -4, -3, -2, -1, 0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15},
    {-13, -12, -12, -11, -10, -9, -8, -7, -6, -5, -4, -3, -2, -1, 0, 0, 0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 12, 13},
    {-10, -9, -9, -8, -7, -7, -6, -5, -4, -4, -3, -2, -2, -1, 0, 0, 0, 1, 2, 2, 3, 4, 4, 5, 6, 7, 7, 8, 9, 9, 10},
    {-5, -5, -4, -4, -4, -3, -3, -3, -2, -2, -1, -1, -1, 0, 0, 0, 0, 0, 1, 1, 1, 2, 2, 3, 3, 3, 4, 4, 4, 5, 5},
    {0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0, 0},
    {5, 5, 4, 4, 4, 3, 3, 3, 2, 2, 1, 1, 1, 0, 0, 0, 0, 0, -1, -1, -1, -2, -2, -3, -3, -3, -4, -4, -4, -5, -5},
    {10, 9, 9, 8, 7, 7, 6, 5, 4, 4, 3, 2, 2, 1, 0, 0, 0, -1, -2, -2, -3, -4, -4, -5, -6, -7, -7, -8, -9, -9, -10},
    {13, 12, 12, 11, 10, 9, 8, 7, 6, 5, 4, 3, 2, 1, 0, 0, 0, -1, -2, -3, -4, -5, -6, -7, -8, -9, -10, -11, -12, -12, -13},
};

// ---------------------------------------------------------------------------------
// Base shapes.  Inside shared memory every channel plane is stored in "line/position"
// coordinates (l, p) chosen so that its taps look like one of three base lines:
//   AXIS  (canonical 0):  taps (dl, dp) = (0, j)                       31 taps, 1 line
//   SLANT (canonical 1):  taps = kCanon*[1]                            29 taps, 11 lines
//   DIAG  (canonical 2):  taps (dl, dp) = (u, -u), u = kCanonDh[2]     21 taps, diagonal
// The mapping image (h, w) -> (l, p) is a transpose and/or a mirror of the position axis,
// plus possibly reading the weights in reverse order:
//   T   transpose:      (l, p) = (w, h)    instead of (h, w)
//   FP  mirror p:       p -> len-1-p
//   REV weight order:   tap k of the stored line uses w[K-1-k]
// ---------------------------------------------------------------------------------
enum : int { KIND_AXIS = 0, KIND_SLANT = 1, KIND_DIAG = 2 };
enum : int { MODE_T = 1, MODE_FP = 2, MODE_REV = 4 };

constexpr int canon_kind(int o) { return (o == 0 || o == 4) ? KIND_AXIS : (o == 2 || o == 6) ? KIND_DIAG : KIND_SLANT; }
constexpr int canon_mode(int o) {
    switch (o) {
        case 3: case 4: return MODE_T | MODE_REV;
        case 5: return MODE_T | MODE_FP;
        case 6: case 7: return MODE_FP;
        default: return 0;
    }
}
constexpr int kind_base(int kind) { return kind; }   // canonical class whose table is the base

// Offsets of stored tap k of class o in (l, p) coordinates, after the mode is applied.
constexpr int stored_dl(int o, int k) {
    const int m = canon_mode(o), kk = (m & MODE_REV) ? kMaxTaps - 1 - k : k;
    return (m & MODE_T) ? kCanonDw[o][kk] : kCanonDh[o][kk];
}
constexpr int stored_dp(int o, int k) {
    const int m = canon_mode(o), kk = (m & MODE_REV) ? kMaxTaps - 1 - k : k;
    const int v = (m & MODE_T) ? kCanonDh[o][kk] : kCanonDw[o][kk];
    return (m & MODE_FP) ? -v : v;
}
constexpr bool modes_consistent() {
    for (int o = 0; o < 8; o++) {
        const int b = kind_base(canon_kind(o));
        for (int k = 0; k < kMaxTaps; k++)
            if (stored_dl(o, k) != kCanonDh[b][k] || stored_dp(o, k) != kCanonDw[b][k]) return false;
    }
    return true;
}
static_assert(modes_consistent(), "every canonical line must reduce to its base line");

// ---------------------------------------------------------------------------------
// Per-base-line evaluation plan: unique taps grouped by line offset ("rows"), each row
// with the span [lo, hi] of position offsets it touches.  JH limits the taps to |j| <= JH
// (shorter kernels, or taps that cannot reach inside a small image).
// For DIAG the single row holds u = -dl as the position along the diagonal.
// ---------------------------------------------------------------------------------
struct LinePlan {
    int nrows;
    int row_d[kMaxTaps], row_lo[kMaxTaps], row_hi[kMaxTaps];
    int ntaps;                    // unique taps
    int tap_row[kMaxTaps], tap_dp[kMaxTaps], tap_k[kMaxTaps];   // tap_k: first k of the group
    int merge_into[kMaxTaps];     // for each k: the tap_k it is summed into, or -1 (unused)
    int span;                     // max over rows of hi-lo+1
    int max_d;                    // max |row_d|
};

constexpr LinePlan make_line_plan(int kind, int JH) {
    LinePlan p{};
    const int b = kind_base(kind);
    for (int k = 0; k < kMaxTaps; k++) p.merge_into[k] = -1;
    for (int k = 0; k < kMaxTaps; k++) {
        const int j = k - kHalf;
        if (j < -JH || j > JH) continue;
        int dl = kCanonDh[b][k], dp = kCanonDw[b][k];
        if (kind == KIND_DIAG) { dp = -dl; dl = 0; }      // position along the diagonal
        int found = -1;
        for (int t = 0; t < p.ntaps; t++)
            if (p.row_d[p.tap_row[t]] == dl && p.tap_dp[t] == dp) found = t;
        if (found >= 0) { p.merge_into[k] = p.tap_k[found]; continue; }
        int row = -1;
        for (int r = 0; r < p.nrows; r++) if (p.row_d[r] == dl) row = r;
        if (row < 0) {
            row = p.nrows++;
            p.row_d[row] = dl; p.row_lo[row] = dp; p.row_hi[row] = dp;
        }
        if (dp < p.row_lo[row]) p.row_lo[row] = dp;
        if (dp > p.row_hi[row]) p.row_hi[row] = dp;
        p.tap_row[p.ntaps] = row; p.tap_dp[p.ntaps] = dp; p.tap_k[p.ntaps] = k;
        p.merge_into[k] = k;
        p.ntaps++;
    }
    for (int r = 0; r < p.nrows; r++)
    {
        if (p.row_hi[r] - p.row_lo[r] + 1 > p.span) p.span = p.row_hi[r] - p.row_lo[r] + 1;
        const int ad = p.row_d[r] < 0 ? -p.row_d[r] : p.row_d[r];
        if (ad > p.max_d) p.max_d = ad;
    }
    return p;
}

template <int KIND, int JH> struct LP { static constexpr LinePlan p = make_line_plan(KIND, JH); };

}  // namespace o1d
