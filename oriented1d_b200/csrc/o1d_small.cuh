// 7x7 maps (the last ConvNeXt stage): one thread holds a whole 49-pixel channel plane in
// registers.  Forward and stride-1 input gradient, NHWC, canonical lines, K <= 31.
//
// A 31-tap line over a 7x7 map touches at most 13 pixels, so tiles with line halos (the
// direct kernels: a 19x19 zero-filled tile per 7x7 image, one shared-memory load per FMA) or
// planes with restage and band passes (the tiled kernels) are mostly overhead here.  Instead:
//   * TMA brings a box [32 images][7][7][CCs channels] (50 KB) into one of two tile buffers;
//   * the CTA re-lays it into one fp32 plane per channel, [channel][image][49 (+2 pad)], with
//     strides chosen so that both the re-layout and the per-thread plane loads are free of bank
//     conflicts;
//   * thread (warp = channel, lane = image) loads its 49 inputs into registers and evaluates
//     the 49 outputs with code unrolled for its channel's line: every tap that lands inside
//     the map is one register-register FMA, every other tap does not exist (compile time);
//     a warp works on one channel, so the eight unrolled line shapes never diverge;
//   * outputs go back through the thread's own plane and leave as 128-bit NHWC stores.
// About 17 instructions per output instead of about 50.
#pragma once

#include "o1d_common.cuh"
#include "o1d_lines.cuh"
#include "o1d_tiled_host.cuh"   // mbarrier / TMA primitives, static_for, Vec16, encode_tiled_fn

namespace o1d {

constexpr int kSmallImgs = 32;                    // images per tile = lanes of a warp
constexpr int kSmallPix = 49;
constexpr int kSmallImgPitch = 51;                // floats between the images of a plane (odd)
constexpr int kSmallPlaneStride = kSmallImgs * kSmallImgPitch + 4;   // = 4 (mod 32): channel planes 4 banks apart

struct SmallParams {
    int N, C, K, CCs, nchunks, tiles_n;
    int flip, add_identity;
    int nbuf;                     // tile buffers: 2 (one CTA per SM) or 1 (two CTAs per SM overlap each other)
    int tile_bytes, off_planes_bytes, off_w_bytes, off_bar_bytes;
};

// The eight canonical lines reduce to three base shapes (axis, slant, diagonal: canonical lines
// 0, 1, 2) when the plane is read transposed and/or mirrored and the weights possibly reversed
// (o1d_lines.cuh).  A thread therefore loads and stores its plane through the index map
// (l, p) -> A*l + B*p + C0 of its channel's mode and runs one of three unrolled bodies instead of
// one of eight: the bodies are large, and eight of them at once overflow the instruction cache.
struct PlaneMap { int A, B, C0; };
__device__ __forceinline__ PlaneMap plane_map(int mode) {
    PlaneMap m;
    m.A = (mode & MODE_T) ? 1 : 7;
    m.B = (mode & MODE_T) ? 7 : 1;
    m.C0 = 0;
    if (mode & MODE_FP) { m.C0 = 6 * m.B; m.B = -m.B; }
    return m;
}

// y'[l,p] = bias + sum over the taps of base line O that land inside the 7x7 map, in stored
// coordinates.  w is indexed by the stored tap index; taps beyond K/2 carry weight 0.
template <int O>
__device__ __forceinline__ void small_plane(const float (&x)[kSmallPix], const float (&w)[kMaxTaps], float bias,
                                            float *__restrict__ out, const PlaneMap m) {
    static_for<0, kSmallPix>([&](auto pi) {
        constexpr int p = decltype(pi)::value, h = p / 7, q = p % 7;
        float acc = bias;
        static_for<0, kMaxTaps>([&](auto ki) {
            constexpr int k = decltype(ki)::value;
            constexpr int hh = h + kCanonDh[O][k], qq = q + kCanonDw[O][k];
            if constexpr (hh >= 0 && hh < 7 && qq >= 0 && qq < 7) acc = fmaf(w[k], x[hh * 7 + qq], acc);
        });
        out[m.A * h + m.B * q + m.C0] = acc;
    });
}

template <typename T>
__global__ void __launch_bounds__(512, 1)
small7_fprop_kernel(const __grid_constant__ CUtensorMap tmap, const float *__restrict__ wgt,
                    const float *__restrict__ bias, const int8_t *__restrict__ chan, T *__restrict__ y,
                    const SmallParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *planes = reinterpret_cast<float *>(smem_raw + p.off_planes_bytes);
    float *s_w = reinterpret_cast<float *>(smem_raw + p.off_w_bytes);          // [CCs][32]
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw + p.off_bar_bytes);
    constexpr int VE = Vec16<T>::N;

    const int tid = threadIdx.x, nt = blockDim.x;         // nt = 32 * CCs: one thread per (channel, image)
    const int lane = tid & 31, ch = tid >> 5;
    constexpr int CCs = 32 / (int)sizeof(T);              // channels per chunk: compile time, so that the
                                                          // re-layout index arithmetic has no runtime divisions
    // work items (chunk, tile of 32 images), chunk fastest, dealt round-robin to the CTAs
    const int items = p.nchunks * p.tiles_n;
    const int my_tiles = (items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    auto item_of = [&](int it, int &chunk, int &n0) {
        const int t = blockIdx.x + it * gridDim.x;
        chunk = t % p.nchunks;
        n0 = (t / p.nchunks) * kSmallImgs;
    };

    if (tid == 0) {
        mbar_init(&full[0], 1);
        mbar_init(&full[1], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    auto issue = [&](int it) {
        int chunk, n0;
        item_of(it, chunk, n0);
        const int b = it % p.nbuf;
        mbar_expect_tx(&full[b], p.tile_bytes);
        tma_load_4d(smem_raw + (size_t)b * p.tile_bytes, &tmap, &full[b], chunk * CCs, 0, 0, n0);
    };
    if (tid == 0)
        for (int it = 0; it < p.nbuf && it < my_tiles; it++) issue(it);

    float *mine = planes + ch * kSmallPlaneStride + lane * kSmallImgPitch;
    constexpr int elems = kSmallImgs * kSmallPix * CCs;   // elements of a tile
    bool failed = false;
    for (int it = 0; it < my_tiles; it++) {
        const int b = it % p.nbuf;
        int chunk, n0;
        item_of(it, chunk, n0);
        const int c0 = chunk * CCs;
        // weights of this chunk by canonical tap index, mirrored for the input gradient
        for (int e = tid; e < CCs * 32; e += nt) {
            const int i = e >> 5, k = e & 31;
            float v = 0.f;
            const int kk = k - kHalf + p.K / 2;
            if (k < kMaxTaps && kk >= 0 && kk < p.K) {
                const int src = p.flip ? p.K - 1 - kk : kk;
                v = __ldg(wgt + (size_t)(c0 + i) * p.K + src);
                if (p.add_identity && src == p.K / 2) v += 1.f;
            }
            s_w[e] = v;
        }
        const float bv = bias ? __ldg(bias + c0 + ch) : 0.f;
        const int line = chan[c0 + ch];                    // canonical line of this warp's channel
        if (!failed && !mbar_wait(&full[b], (it / p.nbuf) & 1)) failed = true;
        // ---- tile [image][pixel][channel] -> planes [channel][image][pixel] ----------------
        const T *tile = reinterpret_cast<const T *>(smem_raw + (size_t)b * p.tile_bytes);
        {   // thread -> channel tid % CCs and (image, pixel) tid / CCs, then 32 pixels further per trip
            int img = (tid / CCs) / kSmallPix, px = (tid / CCs) % kSmallPix;
            float *dst = planes + (tid % CCs) * kSmallPlaneStride;
#pragma unroll 7
            for (int i = 0; i < elems / (32 * CCs); i++) {
                dst[img * kSmallImgPitch + px] = (float)tile[tid + i * 32 * CCs];   // shared memory: a plain load
                px += 32;
                if (px >= kSmallPix) { px -= kSmallPix; img++; }
            }
        }
        __syncthreads();                                   // planes complete; tile buffer b is free
        if (tid == 0 && it + p.nbuf < my_tiles) issue(it + p.nbuf);
        // ---- one plane per thread -----------------------------------------------------------
        const int mode = canon_mode(line), kind = canon_kind(line);     // warp-uniform
        const PlaneMap pm = plane_map(mode);
        float w[kMaxTaps];
#pragma unroll
        for (int k = 0; k < kMaxTaps; k++) w[k] = s_w[ch * 32 + ((mode & MODE_REV) ? kMaxTaps - 1 - k : k)];
        float x[kSmallPix];
#pragma unroll
        for (int i = 0; i < kSmallPix; i++) x[i] = mine[pm.A * (i / 7) + pm.B * (i % 7) + pm.C0];
        if (kind == KIND_AXIS) small_plane<0>(x, w, bv, mine, pm);
        else if (kind == KIND_SLANT) small_plane<1>(x, w, bv, mine, pm);
        else small_plane<2>(x, w, bv, mine, pm);
        __syncthreads();                                   // output planes complete
        // ---- planes -> NHWC, 16 bytes per store ---------------------------------------------
        constexpr int GV = CCs / VE;                       // 16-byte vectors per pixel of the chunk
        {
            constexpr int STEP = 32 * CCs / GV, DI = STEP / kSmallPix, DP = STEP % kSmallPix;   // (image, pixel) per trip
            const int g = tid % GV;
            int img = (tid / GV) / kSmallPix, px = (tid / GV) % kSmallPix;
            const float *src = planes + g * VE * kSmallPlaneStride;
            T *dst = y + (size_t)n0 * kSmallPix * p.C + c0 + g * VE;
            for (; img < kSmallImgs; img += DI, px += DP) {
                if (px >= kSmallPix) { px -= kSmallPix; if (++img >= kSmallImgs) break; }
                if (n0 + img >= p.N) break;                // images are visited in ascending order
                float f[VE];
#pragma unroll
                for (int j = 0; j < VE; j++) f[j] = src[j * kSmallPlaneStride + img * kSmallImgPitch + px];
                *reinterpret_cast<uint4 *>(dst + ((size_t)img * kSmallPix + px) * p.C) = Vec16<T>::pack(f);
            }
        }
        __syncthreads();                                   // planes may be overwritten by the next tile
    }
}


// Weight gradient of one plane: acc[k] += sum over pixels p of x[p + offset_k] * dy[p] for the taps
// that land inside the map (compile time); dy comes from the thread's plane, one pixel at a time.
template <int O>
__device__ __forceinline__ void small_plane_wgrad(const float (&x)[kSmallPix], const float *__restrict__ dyp,
                                                  float (&acc)[kMaxTaps], float &db, const PlaneMap m) {
    static_for<0, kSmallPix>([&](auto pi) {
        constexpr int p = decltype(pi)::value, h = p / 7, q = p % 7;
        const float g = dyp[m.A * h + m.B * q + m.C0];
        db += g;
        static_for<0, kMaxTaps>([&](auto ki) {
            constexpr int k = decltype(ki)::value;
            constexpr int hh = h + kCanonDh[O][k], qq = q + kCanonDw[O][k];
            if constexpr (hh >= 0 && hh < 7 && qq >= 0 && qq < 7) acc[k] = fmaf(x[hh * 7 + qq], g, acc[k]);
        });
    });
}

// Weight gradient, same tiles and planes: x goes tile -> planes -> registers, then dy takes the
// same tile buffer and the same planes.  The 32 images of a warp are added with shuffles; one
// partial per (tile, channel); small7_wgrad_final_kernel adds the tiles of a chunk in order.
template <typename T>
__global__ void __launch_bounds__(512, 1)
small7_wgrad_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_dy,
                    const int8_t *__restrict__ chan, float *__restrict__ partial, const SmallParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *planes = reinterpret_cast<float *>(smem_raw + p.off_planes_bytes);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem_raw + p.off_bar_bytes);
    constexpr int CCs = 32 / (int)sizeof(T);
    const int tid = threadIdx.x;
    const int lane = tid & 31, ch = tid >> 5;
    const int items = p.nchunks * p.tiles_n;
    const int my_tiles = (items - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
    auto item_of = [&](int it, int &chunk, int &n0) {
        const int t = blockIdx.x + it * gridDim.x;
        chunk = t % p.nchunks;
        n0 = (t / p.nchunks) * kSmallImgs;
    };
    if (tid == 0) {
        mbar_init(&full[0], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    auto issue = [&](const CUtensorMap *map, int it) {       // the single tile buffer
        int chunk, n0;
        item_of(it, chunk, n0);
        mbar_expect_tx(&full[0], p.tile_bytes);
        tma_load_4d(smem_raw, map, &full[0], chunk * CCs, 0, 0, n0);
    };
    auto relayout = [&]() {
        const T *tile = reinterpret_cast<const T *>(smem_raw);
        int img = (tid / CCs) / kSmallPix, px = (tid / CCs) % kSmallPix;
        float *dst = planes + (tid % CCs) * kSmallPlaneStride;
#pragma unroll 7
        for (int i = 0; i < kSmallPix; i++) {
            dst[img * kSmallImgPitch + px] = (float)tile[tid + i * 32 * CCs];
            px += 32;
            if (px >= kSmallPix) { px -= kSmallPix; img++; }
        }
    };
    if (tid == 0 && my_tiles > 0) issue(&tmap_x, 0);
    float *mine = planes + ch * kSmallPlaneStride + lane * kSmallImgPitch;
    uint32_t uses = 0;
    bool failed = false;
    for (int it = 0; it < my_tiles; it++) {
        int chunk, n0;
        item_of(it, chunk, n0);
        const int line = chan[chunk * CCs + ch];
        if (!failed && !mbar_wait(&full[0], uses++ & 1)) failed = true;
        relayout();                                        // x: tile -> planes
        __syncthreads();
        if (tid == 0) issue(&tmap_dy, it);                 // dy of the same item into the freed tile buffer
        const int mode = canon_mode(line), kind = canon_kind(line);     // warp-uniform
        const PlaneMap pm = plane_map(mode);
        float x[kSmallPix];
#pragma unroll
        for (int i = 0; i < kSmallPix; i++) x[i] = mine[pm.A * (i / 7) + pm.B * (i % 7) + pm.C0];
        __syncthreads();                                   // every thread holds its x plane in registers
        if (!failed && !mbar_wait(&full[0], uses++ & 1)) failed = true;
        relayout();                                        // dy: tile -> the same planes
        __syncthreads();
        if (tid == 0 && it + 1 < my_tiles) issue(&tmap_x, it + 1);
        float acc[kMaxTaps], db = 0.f;
#pragma unroll
        for (int k = 0; k < kMaxTaps; k++) acc[k] = 0.f;
        if (kind == KIND_AXIS) small_plane_wgrad<0>(x, mine, acc, db, pm);
        else if (kind == KIND_SLANT) small_plane_wgrad<1>(x, mine, acc, db, pm);
        else small_plane_wgrad<2>(x, mine, acc, db, pm);
        // images beyond N are zero-filled tiles: they add nothing.  Sum over the warp's 32 images.
#pragma unroll
        for (int k = 0; k < kMaxTaps; k++)
#pragma unroll
            for (int d = 16; d > 0; d >>= 1) acc[k] += __shfl_xor_sync(0xffffffffu, acc[k], d);
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) db += __shfl_xor_sync(0xffffffffu, db, d);
        float *dst = partial + ((size_t)(blockIdx.x + it * gridDim.x) * CCs + ch) * 32;
        float mineval = db;                                // lane k keeps canonical tap k, lane 31 the bias gradient
        const int stored = (mode & MODE_REV) ? kMaxTaps - 1 - lane : lane;    // stored tap that is canonical tap `lane`
#pragma unroll
        for (int k = 0; k < kMaxTaps; k++) if (stored == k) mineval = acc[k];
        dst[lane] = mineval;
        __syncthreads();                                   // planes are overwritten by the next item's x
    }
}

// dw[c][kk] = sum over the tiles of c's chunk, in tile order, of the partial of canonical tap kk - K/2 + 15.
__global__ void small7_wgrad_final_kernel(const float *__restrict__ partial, float *__restrict__ dw,
                                          float *__restrict__ db, int C, int K, int CCs, int nchunks, int tiles_n) {
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= C * (K + 1)) return;
    const int c = idx / (K + 1), kk = idx % (K + 1);
    if (kk == K && db == nullptr) return;
    const int chunk = c / CCs, cl = c % CCs;
    const int slot = kk == K ? 31 : kk - K / 2 + kHalf;
    float sum = 0.f;
    for (int t = 0; t < tiles_n; t++) sum += partial[((size_t)(t * nchunks + chunk) * CCs + cl) * 32 + slot];
    if (kk == K) db[c] = sum; else dw[(size_t)c * K + kk] = sum;
}

// ---- host side -------------------------------------------------------------------------
struct SmallConfig { SmallParams p; int smem_bytes, grid, threads; };

inline bool small7_configure(const PlanHeader &ph, int N, int H, int W, int C, int K, int stride, int layout, int esize,
                             int smem_limit, int sms, SmallConfig *out) {
    if (H != 7 || W != 7 || stride != 1 || layout != O1D_NHWC || K > kMaxTaps || !ph.all_canon || ph.chan_off == 0)
        return false;
    const int CCs = 32 / esize;
    if (C % CCs != 0) return false;
    SmallParams p{};
    p.N = N; p.C = C; p.K = K; p.CCs = CCs; p.nchunks = C / CCs;
    p.tiles_n = ceil_div(N, kSmallImgs);
    p.tile_bytes = kSmallImgs * kSmallPix * CCs * esize;
    // 4-byte elements: 256 threads per CTA; one tile buffer leaves room for two CTAs per SM
    p.nbuf = (esize == 4) ? 1 : 2;
    p.off_planes_bytes = p.nbuf * p.tile_bytes;
    p.off_w_bytes = p.off_planes_bytes + CCs * kSmallPlaneStride * 4;
    p.off_bar_bytes = p.off_w_bytes + CCs * 32 * 4;
    out->smem_bytes = p.off_bar_bytes + 16;
    if (out->smem_bytes > smem_limit) return false;
    const int items = p.nchunks * p.tiles_n;
    const int slots = sms * (p.nbuf == 1 ? 2 : 1);
    out->grid = items < slots ? items : slots;
    out->threads = 32 * CCs;
    out->p = p;
    return true;
}

// 4-D tensor map over an NHWC tensor [N][7][7][C] with a box CCs x 7 x 7 x 32 images.
inline int make_small7_tensor_map(CUtensorMap *map, const void *base, int N, int C, int esize, int CCs) {
    const cuuint64_t dims[4] = {(cuuint64_t)C, 7, 7, (cuuint64_t)N};
    const cuuint64_t strides[3] = {(cuuint64_t)C * esize, (cuuint64_t)7 * C * esize, (cuuint64_t)49 * C * esize};
    const cuuint32_t box[4] = {(cuuint32_t)CCs, 7, 7, (cuuint32_t)kSmallImgs};
    return encode_map4(map, base, esize, dims, strides, box);
}

template <typename T>
cudaError_t launch_small7(const SmallConfig &cfg, const CUtensorMap &map, const float *w, const float *bias,
                          const int8_t *chan, void *y, cudaStream_t st) {
    auto kern = small7_fprop_kernel<T>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg.smem_bytes);
    if (e != cudaSuccess) return e;
    kern<<<cfg.grid, cfg.threads, cfg.smem_bytes, st>>>(map, w, bias, chan, (T *)y, cfg.p);
    return cudaGetLastError();
}


// Weight gradient: one tile buffer (x, then dy), one set of planes.
inline bool small7_wgrad_configure(const PlanHeader &ph, int N, int H, int W, int C, int K, int stride, int layout,
                                   int esize, int smem_limit, int sms, SmallConfig *out) {
    if (!small7_configure(ph, N, H, W, C, K, stride, layout, esize, smem_limit, sms, out)) return false;
    SmallParams &p = out->p;
    p.nbuf = 1;
    p.off_planes_bytes = p.tile_bytes;
    p.off_w_bytes = p.off_planes_bytes + p.CCs * kSmallPlaneStride * 4;
    p.off_bar_bytes = p.off_w_bytes;
    out->smem_bytes = p.off_bar_bytes + 16;
    const int items = p.nchunks * p.tiles_n;
    const int slots = sms * ((228 * 1024) / (out->smem_bytes + 1024) >= 2 && out->threads <= 256 ? 2 : 1);
    out->grid = items < slots ? items : slots;
    return true;
}
inline size_t small7_wgrad_partial_bytes(const SmallConfig &cfg) {
    return (size_t)cfg.p.nchunks * cfg.p.tiles_n * cfg.p.CCs * 32 * sizeof(float);
}
template <typename T>
cudaError_t launch_small7_wgrad(const SmallConfig &cfg, const CUtensorMap &mx, const CUtensorMap &mdy,
                                const int8_t *chan, float *partial, cudaStream_t st) {
    auto kern = small7_wgrad_kernel<T>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, cfg.smem_bytes);
    if (e != cudaSuccess) return e;
    kern<<<cfg.grid, cfg.threads, cfg.smem_bytes, st>>>(mx, mdy, chan, partial, cfg.p);
    return cudaGetLastError();
}

}  // namespace o1d
