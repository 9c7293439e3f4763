// Host side of the tiled kernels: applicability test, tile/chunk selection, shared-memory
// layout, TMA descriptor, launch.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <mutex>

#include "o1d_tiled.cuh"
#include "o1d_tma_host.cuh"

namespace o1d {

struct TiledConfig {
    TiledParams p;
    int smem_bytes;
    int grid;
    int threads;     // CTA size: 512, 256 or 128 (smaller CTAs co-reside and overlap their phases)
    int ctas_per_sm;
    double score;
    int stage_stride;
    int jh;          // taps |j| <= jh are evaluated (instantiated: 7, 9, 15)
    double util;
};

// Largest |j| whose tap can land inside an image of extent S x S for at least one base line,
// capped by the kernel length; rounded up to an instantiated value.
inline int tiled_tap_reach(int H, int W, int K) {
    const int S = H > W ? H : W;
    int need = 0;
    for (int j = kHalf; j >= 1 && !need; j--)
        for (int b = 0; b < 3; b++) {
            const int dh = kCanonDh[b][kHalf + j], dw = kCanonDw[b][kHalf + j];
            if ((dh < 0 ? -dh : dh) < S && (dw < 0 ? -dw : dw) < S) need = j;
        }
    if (need > K / 2) need = K / 2;
    return need <= 7 ? 7 : need <= 9 ? 9 : kHalf;
}

inline int round32(int v) { return (v + 31) & ~31; }
// Smallest stride >= v with stride*VE congruent to 32/GV modulo 32 (GV = CC/VE vectors per
// pixel): the GV channel groups of one pixel then start 32/GV banks apart.
inline int skew_stride(int v, int CC, int VE) {
    const int GV = CC / VE;
    if (GV <= 1 || GV > 32) return v;
    const int want = 32 / GV;
    for (int s = v; s < v + 64; s++)
        if ((s * VE) % 32 == want % 32) return s;
    return v;
}
inline int make_odd(int v) { return v | 1; }

// Picks BR (band rows), CC (chunk channels), the CTA size and the stage count for given line
// pitches (0 = the default, smallest odd pitch); returns false when the tiled kernels do not apply
// and the general kernels must be used.
inline bool tiled_configure_pitch(const PlanHeader &ph, const void *plan_host, int N, int H, int W, int C, int K,
                                  int stride, int layout, int esize, int smem_limit, int sms, int op, int want_pn,
                                  int want_pt, TiledConfig *out) {
    if (stride != 1 || layout != O1D_NHWC || K > kMaxTaps || !ph.all_canon || ph.comps_off == 0) return false;
    if (H > 256 || W > 256 || (C * esize) % 16 != 0) return false;
    int R = 0;
    if (H % 8 == 0 && W % 8 == 0) R = 8;
    else if (H % 7 == 0 && W % 7 == 0) R = 7;
    else return false;
    const int VE = 16 / esize;
    const KindComp *comps = reinterpret_cast<const KindComp *>(static_cast<const char *>(plan_host) + ph.comps_off);
    const int G = (R == 8) ? 17 : 16;
    const int pitch_n = want_pn ? want_pn : make_odd(W + G), pitch_t = want_pt ? want_pt : make_odd(H + G);
    // R == 7 kernels surround every plane with kHaloLines zero lines (shared between neighbouring
    // planes) instead of bounds-checking lines; see tiled_nhwc_kernel.
    const int halo = (R == 7) ? kHaloLines : 0;
    const int halo_floats = halo * (pitch_n > pitch_t ? pitch_n : pitch_t);
    const int PLS0 = ((H * pitch_n > W * pitch_t) ? H * pitch_n : W * pitch_t) + halo_floats;

    bool found = false;
    TiledConfig best{};
    for (int NT = kTiledThreads; NT >= 128; NT /= 2)
    for (int ci = 0; ci < kNumChunkWidths; ci++) {
        const int CC = kChunkWidths[ci];
        if (CC % VE != 0 || C % CC != 0 || comps[ci].n <= 0 || NT % (CC / VE) != 0) continue;
        // a chunk narrower than a 32-byte DRAM sector halves the useful bytes per sector fetched
        // (measured slower even with two CTAs per SM); allowed only for 2-byte elements, where 8
        // channels are the most whose planes fit at 56x56
        if (CC * esize < 32 && !(esize == 2 && CC == 8)) continue;
        for (int BR = R; BR <= H; BR += R) {
            if (H % BR != 0) continue;
            const int nseg_line = BR * (W / R), nseg_diag = (W + R - 1) * (BR / R);
            int worst = 0;
            double active = 0;
            for (int t = 0; t < comps[ci].n; t++) {
                const int a = comps[ci].tri[t][0], s = comps[ci].tri[t][1], d = comps[ci].tri[t][2];
                const int slots = round32(a * nseg_line) + round32(s * nseg_line) + round32(d * nseg_diag);
                if (slots > worst) worst = slots;
                active += (double)((a + s) * nseg_line + d * nseg_diag) / comps[ci].n;
            }
            if (worst > NT) continue;
            // movers: as many whole rows as the CTA has (pixel, vector) threads for, evened out
            // over the passes a band needs
            const int tr_max = NT / (CC / VE) / W;
            if (tr_max < 1) continue;
            const int passes = (BR + (tr_max < BR ? tr_max : BR) - 1) / (tr_max < BR ? tr_max : BR);
            const int tr = (BR + passes - 1) / passes;
            const int out_pitch_n = make_odd(W), out_pitch_t = make_odd(BR);
            // Plane strides are padded so that the channel groups a warp touches together in
            // the restage / store loops (VE channels apart) fall into different banks.
            const int PLS = skew_stride(PLS0, CC, VE);
            const int OPS = skew_stride((BR * out_pitch_n > W * out_pitch_t) ? BR * out_pitch_n : W * out_pitch_t, CC, VE);
            if (op == OP_WGRAD && (2 * CC * OPS) / NT < 1) continue;
            TiledParams p{};
            p.off_planar = 0;
            const int planar_floats = (32 + halo_floats + CC * PLS + 3) & ~3;
            p.plane_base = 32 + halo_floats;
            p.halo = halo;
            p.off_zero = planar_floats;
            p.zero_floats_total = planar_floats + kZeroFloats;
            p.off_out = p.zero_floats_total;
            p.off_wts = (p.off_out + 2 * CC * OPS + 3) & ~3;     // read as float4
            p.off_misc = p.off_wts + CC * 32;
            const int misc_ints = 4 + kMaxCC + 2 * kMaxCC * 4 + kMaxCC + 2 * kMaxCC;
            int bytes = (p.off_misc + misc_ints) * 4;
            bytes = (bytes + 127) & ~127;
            p.off_stage_bytes = bytes;
            p.stage_bytes = BR * W * CC * esize;
            const int stage_stride = (p.stage_bytes + 127) & ~127;
            const int NB = H / BR;
            // CTAs that fit one SM: 64K registers at 128 per thread; 228 KB of shared memory with
            // 1 KB reserved per CTA.  Staging depth is traded against co-residency: take the
            // largest CTA count that still leaves two stages (one when the image is one band).
            const int nstg_cap = NB + 2 > 3 ? (NB + 2 < kMaxStages ? NB + 2 : kMaxStages) : 3;
            const int nstg_min = NB == 1 ? 1 : 2;
            int ctas = 0, nstg = 0;
            for (int t = kTiledThreads / NT; t >= 1 && !ctas; t--) {
                int budget = (228 * 1024) / t - 1024;
                if (budget > smem_limit) budget = smem_limit;
                const int n_fit = (budget - bytes - 8 * kMaxStages) / stage_stride;
                if (n_fit >= nstg_min) { ctas = t; nstg = n_fit < nstg_cap ? n_fit : nstg_cap; }
            }
            if (!ctas) continue;
            // Rank: lanes doing useful work per SM, with a bonus when two or more CTAs share an
            // SM (their load / restage / compute / store phases overlap); then larger tiles.
            const double util = active / NT;
            const double score = util * (double)(ctas * NT) / kTiledThreads * (ctas >= 4 ? 1.4 : ctas >= 2 ? 1.25 : 1.0);
            const bool better = !found || score > best.score + 1e-9 ||
                                (score > best.score - 1e-9 && BR * CC > best.p.BR * best.p.CC);
            if (!better) continue;
            p.N = N; p.H = H; p.W = W; p.C = C; p.K = K;
            p.CC = CC; p.nchunks = C / CC; p.total_items = N * p.nchunks;
            p.R = R; p.BR = BR; p.NB = NB; p.NSTG = nstg;
            // grouping shortens the prefetch distance, which costs more than the barriers it saves
            // when an item has more bands than there are stages
            p.grp = (NB <= nstg && nstg / 2 > 1) ? nstg / 2 : 1;
            p.pitch_n = pitch_n; p.pitch_t = pitch_t; p.plane_stride = PLS;
            p.out_pitch_n = out_pitch_n; p.out_pitch_t = out_pitch_t; p.out_plane_stride = OPS;
            p.nseg_line = nseg_line; p.nseg_diag = nseg_diag;
            p.rezero = (H != W);
            p.stage_stride = stage_stride;
            p.off_bar_bytes = p.off_stage_bytes + nstg * stage_stride;
            p.div_gv = FastDiv::make(CC / VE); p.div_w = FastDiv::make(W);
            p.div_nseg_line = FastDiv::make(nseg_line); p.div_nseg_diag = FastDiv::make(nseg_diag);
            p.div_br = FastDiv::make(BR); p.div_wline = FastDiv::make(W); p.div_wdiag = FastDiv::make(W + R - 1);
            p.div_chunks = FastDiv::make(p.nchunks); p.div_nb = FastDiv::make(NB); p.div_n = FastDiv::make(N);
            p.TR = tr;
            best.p = p;
            best.smem_bytes = p.off_bar_bytes + 8 * kMaxStages;
            best.stage_stride = stage_stride;
            best.threads = NT; best.ctas_per_sm = ctas; best.score = score;
            best.grid = p.total_items < sms * ctas ? p.total_items : sms * ctas;
            best.p.order = (op == OP_WGRAD) ? 1 : 0;
            if (p.nchunks <= best.grid) {
                // A grid that is a multiple of the chunk count keeps every CTA on one chunk: its
                // channel tables and weights are built once, and the weight gradient can use the
                // DRAM-friendly image-major order with a single flush.  Worth giving up some SMs
                // (forward: up to 15%; weight gradient: up to 30%, chunk-major order re-reads
                // every DRAM sector).
                // Not for the forward kernels when chunks differ in line kinds (block-wise angle
                // assignment): slanted chunks cost more than axis chunks, and CTAs pinned to one
                // chunk would finish at different times; a grid that is no multiple of the chunk
                // count rotates every CTA through all chunks.
                const bool mixed_cost = op != OP_WGRAD && comps[ci].n > 1;
                const int g = (best.grid / p.nchunks) * p.nchunks;
                if (!mixed_cost && g * 100 >= best.grid * (op == OP_WGRAD ? 70 : 85)) {
                    best.grid = g;
                    best.p.order = 0;
                }
            }
            best.jh = tiled_tap_reach(H, W, K);
            best.util = util;
            found = true;
        }
    }
    if (found) {
        if (op == OP_WGRAD) {   // partial slots per CTA = chunks it can touch
            int mv = 1;
            for (int b = 0; b < best.grid && best.p.order == 1; b++) {
                const int lo = wgrad_item_lo(b, best.grid, best.p.total_items);
                const int hi = wgrad_item_lo(b + 1, best.grid, best.p.total_items);
                if (hi > lo) {
                    const int v = (hi - 1) / N - lo / N + 1;
                    if (v > mv) mv = v;
                }
            }
            best.p.max_visits = mv;
        }
        *out = best;
    }
    return found;
}

// Shared-memory wavefronts of the register-window loads of one band for one channel chunk: every
// load instruction of a warp costs as many wavefronts as its worst bank is hit with different
// addresses, and all window loads of a thread are at constant offsets from its segment origin,
// so the degree of a warp follows from the origins alone.  Mirrors the thread -> (kind, channel,
// segment) assignment and the origin arithmetic of tiled_nhwc_kernel.
inline long tiled_window_wavefronts(const int8_t *ids, const TiledParams &p, int NT) {
    const int CC = p.CC, R = p.R, BR = p.BR, W = p.W, H = p.H;
    int sorted[kMaxCC], cnt[3] = {0, 0, 0}, n = 0;
    for (int kd = 0; kd < 3; kd++)
        for (int i = 0; i < CC; i++)
            if (canon_kind(ids[i]) == kd) { sorted[n++] = i; cnt[kd]++; }
    const int wd = W + R - 1;
    const int slotsA = round32(cnt[0] * p.nseg_line), slotsS = round32(cnt[1] * p.nseg_line);
    const int loads[3] = {R + 30, 11 * (R + 2), R + 20};      // window loads per segment: axis, slant, diagonal
    long total = 0;
    for (int w0 = 0; w0 < NT; w0 += 32) {
        int origin[32], m = 0, kind = -1;
        for (int tid = w0; tid < w0 + 32; tid++) {
            int idx = tid, kd, ch, seg;
            if (idx < slotsA) {
                const int j = idx / p.nseg_line;
                if (j >= cnt[0]) continue;
                kd = KIND_AXIS; ch = sorted[j]; seg = idx - j * p.nseg_line;
            } else if ((idx -= slotsA) < slotsS) {
                const int j = idx / p.nseg_line;
                if (j >= cnt[1]) continue;
                kd = KIND_SLANT; ch = sorted[cnt[0] + j]; seg = idx - j * p.nseg_line;
            } else {
                idx -= slotsS;
                const int j = idx / p.nseg_diag;
                if (j >= cnt[2]) continue;
                kd = KIND_DIAG; ch = sorted[cnt[0] + cnt[1] + j]; seg = idx - j * p.nseg_diag;
            }
            const int mode = canon_mode(ids[ch]);
            const int pbase = p.plane_base + ch * p.plane_stride;
            int a;
            if (kd == KIND_DIAG) {
                const int sub = seg / wd, qi = seg - sub * wd;
                a = pbase + (sub * R + R - 1) * p.pitch_n + qi - (R - 1);
            } else if (!(mode & MODE_T)) {
                const int sg = seg / BR, rl = seg - sg * BR;
                a = pbase + rl * p.pitch_n + sg * R;
            } else {
                const int sub = seg / W;
                int l = seg - sub * W + 5;
                if (l >= W) l -= W;
                a = pbase + l * p.pitch_t + ((mode & MODE_FP) ? H - BR : 0) + sub * R;
            }
            origin[m++] = a;
            kind = kd;
        }
        if (!m) continue;
        int degree = 1;
        for (int b = 0; b < 32; b++) {
            int distinct = 0, seen[32];
            for (int i = 0; i < m; i++) {
                if (((origin[i] % 32) + 32) % 32 != b) continue;
                bool dup = false;
                for (int j = 0; j < distinct; j++) dup = dup || seen[j] == origin[i];
                if (!dup) seen[distinct++] = origin[i];
            }
            if (distinct > degree) degree = distinct;
        }
        total += (long)degree * loads[kind];
    }
    return total;
}

// With segments of 7 the 7*k segments of a channel never fill whole warps, and with the default
// pitches most warps straddle two line groups whose origins collide (28x28: 2.0 to 2.6
// wavefronts per window load).  Shared memory has room at these sizes, so the line pitches are
// searched for the fewest window-load wavefronts on a few sample chunks (28x28x192: 107 -> 97 us).
// The result is cached per problem geometry; the search costs about 0.2 ms once.
inline bool tiled_configure(const PlanHeader &ph, const void *plan_host, int N, int H, int W, int C, int K,
                            int stride, int layout, int esize, int smem_limit, int sms, int op, TiledConfig *out) {
    TiledConfig base;
    if (!tiled_configure_pitch(ph, plan_host, N, H, W, C, K, stride, layout, esize, smem_limit, sms, op, 0, 0, &base))
        return false;
    *out = base;
    if (base.p.R != 7 || ph.chan_off == 0) return true;
    const int8_t *chan = reinterpret_cast<const int8_t *>(static_cast<const char *>(plan_host) + ph.chan_off);
    const int CC = base.p.CC, nchunks = C / CC;
    int sample[4], ns = 0;
    for (int i = 0; i < 4; i++) {
        const int ch = (int)((long long)i * (nchunks - 1) / 3);
        if (ns == 0 || sample[ns - 1] != ch) sample[ns++] = ch;
    }
    uint64_t sig = 1469598103934665603ull;                     // FNV-1a over the sampled chunks' line ids
    for (int i = 0; i < ns; i++)
        for (int j = 0; j < CC; j++) sig = (sig ^ (uint8_t)chan[sample[i] * CC + j]) * 1099511628211ull;
    struct Entry { int H, W, CC, BR, NT, esize, op; uint64_t sig; int pn, pt; };
    static Entry cache[64];
    static int cached = 0;
    static std::mutex mu;
    int pn = 0, pt = 0;
    {
        std::lock_guard<std::mutex> lock(mu);
        for (int i = 0; i < cached; i++) {
            const Entry &e = cache[i];
            if (e.H == H && e.W == W && e.CC == CC && e.BR == base.p.BR && e.NT == base.threads && e.esize == esize &&
                e.op == op && e.sig == sig) { pn = e.pn; pt = e.pt; }
        }
    }
    if (!pn) {
        long best = -1;
        for (int dn = 0; dn < 16; dn++)
            for (int dt = 0; dt < 16; dt += 2) {                // transposed planes keep an odd pitch
                TiledConfig c;
                const int cn = base.p.pitch_n + dn, ct = base.p.pitch_t + dt;
                if (!tiled_configure_pitch(ph, plan_host, N, H, W, C, K, stride, layout, esize, smem_limit, sms, op, cn,
                                           ct, &c))
                    continue;
                if (c.p.CC != CC || c.p.BR != base.p.BR || c.threads != base.threads || c.ctas_per_sm < base.ctas_per_sm)
                    continue;
                long cost = 0;
                for (int i = 0; i < ns; i++) cost += tiled_window_wavefronts(chan + sample[i] * CC, c.p, c.threads);
                if (best < 0 || cost < best) { best = cost; pn = cn; pt = ct; }
            }
        if (!pn) { pn = base.p.pitch_n; pt = base.p.pitch_t; }
        std::lock_guard<std::mutex> lock(mu);
        if (cached < 64) cache[cached++] = Entry{H, W, CC, base.p.BR, base.threads, esize, op, sig, pn, pt};
    }
    if (pn == base.p.pitch_n && pt == base.p.pitch_t) return true;
    TiledConfig tuned;
    if (tiled_configure_pitch(ph, plan_host, N, H, W, C, K, stride, layout, esize, smem_limit, sms, op, pn, pt, &tuned) &&
        tuned.p.CC == CC && tuned.ctas_per_sm >= base.ctas_per_sm)
        *out = tuned;
    return true;
}

// 4-D tensor map over an NHWC tensor: dims (C, W, H, N), box (CC, W, BR, 1).
inline int make_nhwc_tensor_map(CUtensorMap *map, const void *base, int N, int H, int W, int C, int esize,
                                int CC, int BR) {
    const cuuint64_t dims[4] = {(cuuint64_t)C, (cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)N};
    const cuuint64_t strides[3] = {(cuuint64_t)C * esize, (cuuint64_t)W * C * esize, (cuuint64_t)H * W * C * esize};
    const cuuint32_t box[4] = {(cuuint32_t)CC, (cuuint32_t)W, (cuuint32_t)BR, 1};
    return encode_map4(map, base, esize, dims, strides, box);
}

template <typename T, int R, int JH, int OP, bool ACT>
cudaError_t launch_tiled_one(const TiledConfig &cfg, const CUtensorMap &map, const float *w, const float *bias,
                             const PlanView &pv, void *io, float *partial, const void *pre, cudaStream_t st) {
    auto kern = tiled_nhwc_kernel<T, R, JH, OP, ACT>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg.smem_bytes);
    if (e != cudaSuccess) return e;
    kern<<<cfg.grid, cfg.threads, cfg.smem_bytes, st>>>(map, w, bias, pv.chan, (T *)io, partial, (const T *)pre, cfg.p);
    return cudaGetLastError();
}

// Activation on load / its derivative on store exist for the full 31-tap reach only (the second
// conv of a 1D++ block has K = 31); tiled_supports_act() tells the caller beforehand.
inline bool tiled_supports_act(const TiledConfig &cfg) { return cfg.jh == kHalf; }

template <typename T, int R, int OP>
cudaError_t launch_tiled_jh(const TiledConfig &cfg, const CUtensorMap &map, const float *w, const float *bias,
                            const PlanView &pv, void *io, float *partial, const void *pre, cudaStream_t st) {
    if (cfg.p.act || pre)
        return cfg.jh == kHalf ? launch_tiled_one<T, R, kHalf, OP, true>(cfg, map, w, bias, pv, io, partial, pre, st)
                               : cudaErrorNotSupported;
    switch (cfg.jh) {
        case 7: return launch_tiled_one<T, R, 7, OP, false>(cfg, map, w, bias, pv, io, partial, pre, st);
        case 9: return launch_tiled_one<T, R, 9, OP, false>(cfg, map, w, bias, pv, io, partial, pre, st);
        default: return launch_tiled_one<T, R, kHalf, OP, false>(cfg, map, w, bias, pv, io, partial, pre, st);
    }
}

// Dispatch over (element type, segment length, tap reach) for one operation.
template <int OP>
cudaError_t launch_tiled(const TiledConfig &cfg, int dtype, const CUtensorMap &map, const float *w,
                         const float *bias, const PlanView &pv, void *io, float *partial, const void *pre,
                         cudaStream_t st) {
    if (dtype == O1D_F32)
        return cfg.p.R == 8 ? launch_tiled_jh<float, 8, OP>(cfg, map, w, bias, pv, io, partial, pre, st)
                            : launch_tiled_jh<float, 7, OP>(cfg, map, w, bias, pv, io, partial, pre, st);
    return cfg.p.R == 8 ? launch_tiled_jh<__nv_bfloat16, 8, OP>(cfg, map, w, bias, pv, io, partial, pre, st)
                        : launch_tiled_jh<__nv_bfloat16, 7, OP>(cfg, map, w, bias, pv, io, partial, pre, st);
}

inline MergeTables merge_tables_for(int jh) {
    switch (jh) {
        case 7: { constexpr MergeTables m = make_merge_tables<7>(); return m; }
        case 9: { constexpr MergeTables m = make_merge_tables<9>(); return m; }
        default: { constexpr MergeTables m = make_merge_tables<kHalf>(); return m; }
    }
}

inline size_t tiled_wgrad_partial_bytes(const TiledConfig &cfg) {
    return (size_t)cfg.grid * cfg.p.max_visits * cfg.p.CC * kPartialStride * sizeof(float);
}

}  // namespace o1d
