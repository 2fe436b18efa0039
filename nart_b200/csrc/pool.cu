// NHWC uint8 max / average pooling with the reference CPU module's integer requantize
// (art/modules/quant/src/op/pool.c:96-249 of ModelTC/NART).  CUDA-core, HBM-bound: one thread
// owns VEC consecutive channels of one output pixel and reads one VEC-byte vector per tap, so a
// warp reads contiguous runs of the channel axis.
#include <math.h>

#include "common.cuh"
#include "kernels.h"

namespace b200 {

template <int VEC> struct VecT;
template <> struct VecT<16> { using type = uint4; };
template <> struct VecT<4> { using type = uint32_t; };
template <> struct VecT<1> { using type = uint8_t; };

template <int VEC>
__device__ __forceinline__ void load_words(const uint8_t *p, uint32_t (&wv)[(VEC + 3) / 4])
{
    if constexpr (VEC == 16) {
        uint4 q = __ldg(reinterpret_cast<const uint4 *>(p));
        wv[0] = q.x; wv[1] = q.y; wv[2] = q.z; wv[3] = q.w;
    } else if constexpr (VEC == 4) {
        wv[0] = __ldg(reinterpret_cast<const uint32_t *>(p));
    } else {
        wv[0] = __ldg(p);
    }
}

template <int VEC>
__device__ __forceinline__ void store_words(uint8_t *p, const uint32_t (&wv)[(VEC + 3) / 4])
{
    if constexpr (VEC == 16) {
        *reinterpret_cast<uint4 *>(p) = make_uint4(wv[0], wv[1], wv[2], wv[3]);
    } else if constexpr (VEC == 4) {
        *reinterpret_cast<uint32_t *>(p) = wv[0];
    } else {
        *p = (uint8_t)wv[0];
    }
}

// Byte-wise unsigned maximum without the emulated SIMD-in-a-word intrinsics (__vmaxu4 expands to
// about eight integer instructions on this architecture): the four bytes of a word are spread over
// two words of two 16-bit lanes each (one byte-permute apiece), maxima run on those with the native
// max.u16x2, and one byte-permute packs the result.
struct U16x4 {
    uint32_t lo, hi;   // bytes 0, 1 and bytes 2, 3 of the word, zero-extended to 16 bits
};
__device__ __forceinline__ U16x4 spread_bytes(uint32_t w) { return { __byte_perm(w, 0, 0x4140), __byte_perm(w, 0, 0x4342) }; }
__device__ __forceinline__ uint32_t pack_bytes(const U16x4 &v) { return __byte_perm(v.lo, v.hi, 0x6420); }
__device__ __forceinline__ uint32_t max_u16x2(uint32_t a, uint32_t b)
{
    uint32_t d;
    asm("max.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}
__device__ __forceinline__ U16x4 max_u16x4(const U16x4 &a, const U16x4 &b) { return { max_u16x2(a.lo, b.lo), max_u16x2(a.hi, b.hi) }; }

// MAX: running byte-wise maximum starting from 0 (pool.c:140-148), then a 256-entry table that
// holds sat_u(rshift_rn(mult16 * (max - izp), shift) + ozp) for every possible maximum, built on
// the host with the exact arithmetic.
template <int VEC>
__global__ void __launch_bounds__(256) pool_max_kernel(
    const uint8_t *__restrict__ x, uint8_t *__restrict__ y, PoolGeom g, const uint8_t *__restrict__ lut_g)
{
    __shared__ uint8_t lut[256];
    lut[threadIdx.x] = lut_g[threadIdx.x];
    __syncthreads();
    constexpr int W = (VEC + 3) / 4;
    const int cv = g.c / VEC;
    const size_t total = (size_t)g.n * g.oh * g.ow * cv;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        int ci = (int)(idx % cv);
        size_t pix = idx / cv;
        int ox = (int)(pix % g.ow);
        int oy = (int)((pix / g.ow) % g.oh);
        int n = (int)(pix / ((size_t)g.ow * g.oh));
        int hs = oy * g.stride_h - g.pad_h, ws = ox * g.stride_w - g.pad_w;
        int he = min(hs + g.kernel_h, g.h), we = min(ws + g.kernel_w, g.w);
        hs = max(hs, 0);
        ws = max(ws, 0);
        U16x4 run[W];
#pragma unroll
        for (int j = 0; j < W; ++j)
            run[j] = { 0u, 0u };
        for (int iy = hs; iy < he; ++iy)
            for (int ix = ws; ix < we; ++ix) {
                uint32_t v[W];
                load_words<VEC>(x + (((size_t)n * g.h + iy) * g.w + ix) * g.c + (size_t)ci * VEC, v);
#pragma unroll
                for (int j = 0; j < W; ++j)
                    run[j] = max_u16x4(run[j], spread_bytes(v[j]));
            }
        uint32_t mx[W], o[W];
#pragma unroll
        for (int j = 0; j < W; ++j)
            mx[j] = pack_bytes(run[j]);
#pragma unroll
        for (int j = 0; j < W; ++j) {
            if constexpr (VEC == 1)
                o[j] = lut[mx[j] & 0xff];
            else
                o[j] = pack4(
                    lut[mx[j] & 0xff], lut[(mx[j] >> 8) & 0xff], lut[(mx[j] >> 16) & 0xff],
                    lut[mx[j] >> 24]);
        }
        store_words<VEC>(y + pix * g.c + (size_t)ci * VEC, o);
    }
}

// MAX on 16-channel vectors for a compile-time window KH x KW and horizontal stride SW, with 32-bit
// index arithmetic: one thread owns 16 channels of TWO output pixels side by side and loads the
// union of their windows (KH x (KW + SW) vectors) in one unrolled batch, so that all of a thread's
// loads are in flight together and the columns the two windows share are loaded once.  Taps
// outside the image read as 0, the value the running maximum starts from.  IDENT skips the table
// (it maps every byte to itself).  Results equal pool_max_kernel<16>.
template <int KH, int KW, int SW, bool IDENT>
__global__ void __launch_bounds__(256) pool_max_pair_kernel(
    const uint4 *__restrict__ x, uint4 *__restrict__ y, PoolGeom g, const uint8_t *__restrict__ lut_g, uint32_t total)
{
    __shared__ uint8_t lut[256];
    if (!IDENT) {
        lut[threadIdx.x] = lut_g[threadIdx.x];
        __syncthreads();
    }
    constexpr int UW = KW + SW;   // columns of the union of the two windows
    const uint32_t cv = (uint32_t)g.c >> 4, owp = (uint32_t)g.ow >> 1;
    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const uint32_t ci = idx % cv;
        uint32_t pix = idx / cv;
        const uint32_t oxp = pix % owp;
        pix /= owp;
        const uint32_t oy = pix % (uint32_t)g.oh, n = pix / (uint32_t)g.oh;
        const int hs = (int)oy * g.stride_h - g.pad_h;
        const int ws = (int)oxp * 2 * SW - g.pad_w;
        const uint4 *img = x + (size_t)n * (uint32_t)g.h * (uint32_t)g.w * cv + ci;
        uint4 q[KH][UW];
#pragma unroll
        for (int r = 0; r < KH; ++r)
#pragma unroll
            for (int j = 0; j < UW; ++j) {
                const int iy = hs + r, ix = ws + j;
                q[r][j] = make_uint4(0, 0, 0, 0);
                if ((unsigned)iy < (unsigned)g.h && (unsigned)ix < (unsigned)g.w)
                    q[r][j] = __ldg(img + ((uint32_t)iy * (uint32_t)g.w + (uint32_t)ix) * cv);
            }
        // separable: the maximum down each of the UW columns first, then across the KW columns of each
        // output; the columns the two windows share are reduced once
        U16x4 col[UW][4];
#pragma unroll
        for (int j = 0; j < UW; ++j) {
            col[j][0] = spread_bytes(q[0][j].x); col[j][1] = spread_bytes(q[0][j].y);
            col[j][2] = spread_bytes(q[0][j].z); col[j][3] = spread_bytes(q[0][j].w);
#pragma unroll
            for (int r = 1; r < KH; ++r) {
                col[j][0] = max_u16x4(col[j][0], spread_bytes(q[r][j].x)); col[j][1] = max_u16x4(col[j][1], spread_bytes(q[r][j].y));
                col[j][2] = max_u16x4(col[j][2], spread_bytes(q[r][j].z)); col[j][3] = max_u16x4(col[j][3], spread_bytes(q[r][j].w));
            }
        }
        uint32_t m0[4], m1[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            U16x4 a = col[0][i], b = col[SW][i];
#pragma unroll
            for (int j = 1; j < KW; ++j) {
                a = max_u16x4(a, col[j][i]);
                b = max_u16x4(b, col[SW + j][i]);
            }
            m0[i] = pack_bytes(a);
            m1[i] = pack_bytes(b);
        }
        if (!IDENT) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                m0[j] = pack4(lut[m0[j] & 0xff], lut[(m0[j] >> 8) & 0xff], lut[(m0[j] >> 16) & 0xff], lut[m0[j] >> 24]);
                m1[j] = pack4(lut[m1[j] & 0xff], lut[(m1[j] >> 8) & 0xff], lut[(m1[j] >> 16) & 0xff], lut[m1[j] >> 24]);
            }
        }
        uint4 *out = y + ((n * (uint32_t)g.oh + oy) * (uint32_t)g.ow + oxp * 2) * cv + ci;
        out[0] = make_uint4(m0[0], m0[1], m0[2], m0[3]);
        out[cv] = make_uint4(m1[0], m1[1], m1[2], m1[3]);
    }
}

template <int KH, int KW, int SW>
int pool_max_pair_launch(const uint8_t *x, uint8_t *y, const PoolGeom &g, const uint8_t *lut_dev, size_t pairs, cudaStream_t st)
{
    const size_t blocks = (pairs + 255) / 256;
    const uint4 *x4 = reinterpret_cast<const uint4 *>(x);
    uint4 *y4 = reinterpret_cast<uint4 *>(y);
    if (g.lut_identity)
        pool_max_pair_kernel<KH, KW, SW, true><<<resident_grid<pool_max_pair_kernel<KH, KW, SW, true>, 256>(blocks), 256, 0, st>>>(
            x4, y4, g, lut_dev, (uint32_t)pairs);
    else
        pool_max_pair_kernel<KH, KW, SW, false><<<resident_grid<pool_max_pair_kernel<KH, KW, SW, false>, 256>(blocks), 256, 0, st>>>(
            x4, y4, g, lut_dev, (uint32_t)pairs);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

// AVE: sum of (x - izp) over the in-image part of the window; the multiplier and shift depend on
// the padded window size (pool.c:217-221) and come from a small host-built table indexed by how
// many rows / columns the window loses at the far edge.
template <int VEC>
__global__ void __launch_bounds__(256) pool_avg_kernel(
    const uint8_t *__restrict__ x, uint8_t *__restrict__ y, PoolGeom g, PoolAvgTab tab)
{
    constexpr int W = (VEC + 3) / 4;
    const int cv = g.c / VEC;
    const size_t total = (size_t)g.n * g.oh * g.ow * cv;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        int ci = (int)(idx % cv);
        size_t pix = idx / cv;
        int ox = (int)(pix % g.ow);
        int oy = (int)((pix / g.ow) % g.oh);
        int n = (int)(pix / ((size_t)g.ow * g.oh));
        int hs = oy * g.stride_h - g.pad_h, ws = ox * g.stride_w - g.pad_w;
        int he = min(hs + g.kernel_h, g.h + g.pad_h), we = min(ws + g.kernel_w, g.w + g.pad_w);
        int dh = g.kernel_h - (he - hs), dw = g.kernel_w - (we - ws);   // rows / columns lost
        int mult = tab.mult[dh][dw], shift = tab.shift[dh][dw];
        hs = max(hs, 0);
        ws = max(ws, 0);
        he = min(he, g.h);
        we = min(we, g.w);
        int sum[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j)
            sum[j] = 0;
        const int cnt = max(he - hs, 0) * max(we - ws, 0);
        // eight taps per round, loaded before any is used, so that a large window (the global average
        // of a 7x7 map is 49 taps per thread) keeps several loads in flight
        constexpr int UNR = 8;
        for (int iy = hs; iy < he; ++iy) {
            const uint8_t *row = x + (((size_t)n * g.h + iy) * g.w) * g.c + (size_t)ci * VEC;
            for (int ix = ws; ix < we; ix += UNR) {
                uint32_t v[UNR][W];
#pragma unroll
                for (int u = 0; u < UNR; ++u) {
#pragma unroll
                    for (int j = 0; j < W; ++j)
                        v[u][j] = 0;
                    if (ix + u < we)
                        load_words<VEC>(row + (size_t)(ix + u) * g.c, v[u]);
                }
#pragma unroll
                for (int u = 0; u < UNR; ++u)
#pragma unroll
                    for (int j = 0; j < VEC; ++j)
                        sum[j] += (int)((v[u][j / 4] >> (8 * (j % 4))) & 0xff);
            }
        }
        uint32_t o[W];
#pragma unroll
        for (int j = 0; j < W; ++j)
            o[j] = 0;
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            int s = sum[j] - cnt * g.izp;
            // (int32)mult * sum is an int32 product in the reference; rshift_rn then runs on the
            // sign-extended value.
            long long p = (long long)(mult * s);
            int v = (int)(rshift_rn64(p, shift) + g.ozp);
            v = min(max(v, 0), g.qmax);
            o[j / 4] |= (uint32_t)v << (8 * (j % 4));
        }
        store_words<VEC>(y + pix * g.c + (size_t)ci * VEC, o);
    }
}

static int pool_out_dim(int in, int kernel, int pad, int stride, int ceil_mode, int any_pad)
{
    // art/src/op.c:934-956: double arithmetic, then one step back if the last window would start
    // at or beyond in + pad (only when some padding is set).
    double v = (in + pad * 2.0 - kernel) / stride + 1;
    int o = (int)(ceil_mode ? ceil(v) : floor(v));
    if (any_pad && (o - 1) * stride >= in + pad)
        --o;
    return o;
}

int pool_prepare(
    int h, int w, int method, int kernel_h, int kernel_w, int pad_h, int pad_w, int stride_h,
    int stride_w, int ceil_mode, float ialpha, uint8_t izp, float oalpha, uint8_t ozp,
    uint8_t obits, PoolGeom *g, uint8_t lut[256], PoolAvgTab *tab)
{
    if (h <= 0 || w <= 0 || kernel_h <= 0 || kernel_w <= 0 || stride_h <= 0 || stride_w <= 0
        || pad_h < 0 || pad_w < 0 || obits < 1 || obits > 8 || (method != 0 && method != 1))
        return fail(B200_ERR_INVALID, "pool: bad geometry");
    if (!(ialpha > 0.f) || !(oalpha > 0.f))
        return fail(B200_ERR_INVALID, "pool: scales must be positive");
    int any_pad = pad_h || pad_w;
    g->h = h; g->w = w;
    g->oh = pool_out_dim(h, kernel_h, pad_h, stride_h, ceil_mode, any_pad);
    g->ow = pool_out_dim(w, kernel_w, pad_w, stride_w, ceil_mode, any_pad);
    if (g->oh <= 0 || g->ow <= 0)
        return fail(B200_ERR_INVALID, "pool: empty output");
    g->kernel_h = kernel_h; g->kernel_w = kernel_w; g->pad_h = pad_h; g->pad_w = pad_w;
    g->stride_h = stride_h; g->stride_w = stride_w;
    g->izp = izp; g->ozp = ozp; g->qmax = (1 << obits) - 1;
    g->lut_identity = 0;
    const int qmax = g->qmax;
    if (method == 0) {
        uint32_t m16;
        int8_t sh;
        get_quant_scale(ialpha / oalpha, -16, &m16, &sh);
        if (sh < 1 || sh > 62)
            return fail(B200_ERR_UNSUPPORTED, "pool: shift %d outside 1..62", (int)sh);
        for (int q = 0; q < 256; ++q) {
            int32_t prod = (int32_t)m16 * (q - (int)izp);
            int32_t r = (int32_t)(rshift_rn_host(prod, sh) + ozp);
            lut[q] = (uint8_t)(r > qmax ? qmax : (r < 0 ? 0 : r));
        }
        g->lut_identity = 1;
        for (int q = 0; q < 256; ++q)
            if (lut[q] != q)
                g->lut_identity = 0;
    } else {
        // the windows at the far edge may be cut by `in + pad` (ceil mode): index the table by the
        // number of rows / columns cut
        int max_dh = 0, max_dw = 0;
        for (int oy = 0; oy < g->oh; ++oy) {
            int hs = oy * stride_h - pad_h;
            int d = hs + kernel_h - (h + pad_h);
            if (d > max_dh) max_dh = d;
        }
        for (int ox = 0; ox < g->ow; ++ox) {
            int ws = ox * stride_w - pad_w;
            int d = ws + kernel_w - (w + pad_w);
            if (d > max_dw) max_dw = d;
        }
        if (max_dh >= PoolAvgTab::kMax || max_dw >= PoolAvgTab::kMax)
            return fail(B200_ERR_UNSUPPORTED, "pool: window cut by %d/%d rows/cols at the edge", max_dh, max_dw);
        if ((long long)kernel_h * kernel_w * 255 * 32768 >= (1ll << 31))
            return fail(B200_ERR_UNSUPPORTED, "pool: average window too large for the int32 product");
        for (int dh = 0; dh < PoolAvgTab::kMax; ++dh)
            for (int dw = 0; dw < PoolAvgTab::kMax; ++dw) {
                tab->mult[dh][dw] = 0;
                tab->shift[dh][dw] = 1;
                if (dh > max_dh || dw > max_dw)
                    continue;
                uint32_t pool_size = (uint32_t)((kernel_h - dh) * (kernel_w - dw));
                if (pool_size == 0)
                    continue;
                uint32_t m;
                int8_t sh;
                get_quant_scale(ialpha / oalpha / pool_size, 16, &m, &sh);   // pool.c:221
                if (sh < 1 || sh > 62)
                    return fail(B200_ERR_UNSUPPORTED, "pool: shift %d outside 1..62", (int)sh);
                tab->mult[dh][dw] = (int)m;
                tab->shift[dh][dw] = sh;
            }
    }
    return B200_OK;
}

int pool_launch(
    const uint8_t *x, uint8_t *y, int n, int c, int method, const PoolGeom &g0, const uint8_t *lut_dev,
    const PoolAvgTab &tab, cudaStream_t st)
{
    PoolGeom g = g0;
    g.n = n;
    g.c = c;
    if (n == 0)
        return B200_OK;
    int vec = (c % 16 == 0 && (((uintptr_t)x | (uintptr_t)y) & 15) == 0) ? 16
        : (c % 4 == 0 && (((uintptr_t)x | (uintptr_t)y) & 3) == 0)       ? 4
                                                                           : 1;
    size_t total = (size_t)n * g.oh * g.ow * (c / vec);
    const size_t blocks = (total + 255) / 256;
    const size_t cv16 = (size_t)c / 16;
    if (method == 0 && vec == 16 && g.ow % 2 == 0 && (size_t)n * g.h * g.w * cv16 < 0xffffffffull) {
        // two outputs per thread, unrolled window, 32-bit indices: the common window shapes
        const size_t pairs = (size_t)n * g.oh * (g.ow / 2) * cv16;
        if (pairs < 0xffffffffull - 256ull * 65536ull) {
            if (g.kernel_h == 3 && g.kernel_w == 3 && g.stride_w == 2)
                return pool_max_pair_launch<3, 3, 2>(x, y, g, lut_dev, pairs, st);
            if (g.kernel_h == 3 && g.kernel_w == 3 && g.stride_w == 1)
                return pool_max_pair_launch<3, 3, 1>(x, y, g, lut_dev, pairs, st);
            if (g.kernel_h == 2 && g.kernel_w == 2 && g.stride_w == 2)
                return pool_max_pair_launch<2, 2, 2>(x, y, g, lut_dev, pairs, st);
        }
    }
    if (method == 0) {
        if (vec == 16) pool_max_kernel<16><<<resident_grid<pool_max_kernel<16>, 256>(blocks), 256, 0, st>>>(x, y, g, lut_dev);
        else if (vec == 4) pool_max_kernel<4><<<resident_grid<pool_max_kernel<4>, 256>(blocks), 256, 0, st>>>(x, y, g, lut_dev);
        else pool_max_kernel<1><<<resident_grid<pool_max_kernel<1>, 256>(blocks), 256, 0, st>>>(x, y, g, lut_dev);
    } else {
        if (vec == 16) pool_avg_kernel<16><<<resident_grid<pool_avg_kernel<16>, 256>(blocks), 256, 0, st>>>(x, y, g, tab);
        else if (vec == 4) pool_avg_kernel<4><<<resident_grid<pool_avg_kernel<4>, 256>(blocks), 256, 0, st>>>(x, y, g, tab);
        else pool_avg_kernel<1><<<resident_grid<pool_avg_kernel<1>, 256>(blocks), 256, 0, st>>>(x, y, g, tab);
    }
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_pool_out_dims(
    int32_t h, int32_t w, int32_t kernel_h, int32_t kernel_w, int32_t pad_h, int32_t pad_w,
    int32_t stride_h, int32_t stride_w, int32_t ceil_mode, int32_t *oh, int32_t *ow)
{
    if (!oh || !ow || stride_h <= 0 || stride_w <= 0)
        return fail(B200_ERR_INVALID, "pool_out_dims: bad argument");
    int any_pad = pad_h || pad_w;
    *oh = pool_out_dim(h, kernel_h, pad_h, stride_h, ceil_mode, any_pad);
    *ow = pool_out_dim(w, kernel_w, pad_w, stride_w, ceil_mode, any_pad);
    return B200_OK;
}

int b200_pool_u8(
    const uint8_t *x, int32_t n, int32_t c, int32_t h, int32_t w, int32_t method, int32_t kernel_h,
    int32_t kernel_w, int32_t pad_h, int32_t pad_w, int32_t stride_h, int32_t stride_w,
    int32_t ceil_mode, float ialpha, uint8_t izp, float oalpha, uint8_t ozp, uint8_t obits,
    uint8_t *y, b200_stream_t stream)
{
    if (!x || !y || n < 0 || c <= 0)
        return fail(B200_ERR_INVALID, "pool: bad argument");
    PoolGeom g;
    PoolAvgTab tab;
    uint8_t lut[256];
    B200_TRY(pool_prepare(
        h, w, method, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, ceil_mode, ialpha, izp,
        oalpha, ozp, obits, &g, lut, &tab));
    cudaStream_t st = as_stream(stream);
    const uint8_t *lut_dev = nullptr;
    if (method == 0)
        B200_TRY(lut_cache_get(lut, &lut_dev));   // uploaded once per distinct table, then reused
    return pool_launch(x, y, n, c, method, g, lut_dev, tab, st);
}

}  // extern "C"
