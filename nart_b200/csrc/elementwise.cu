// Bandwidth-bound uint8 ops around the quantized convolution: quantize / dequantize with the
// NCHW <-> NHWC transpose fused in, plain layout changes, eltwise SUM (add) and relu.  All are
// CUDA-core kernels measured against HBM bandwidth: every global access is a full-sector,
// coalesced or 16-byte vector access.
#include "common.cuh"
#include "kernels.h"

namespace b200 {

// ---------------------------------------------------------------------------------------------
// Tiled transpose between [N][C][P] (P = H*W, the reference's NCHW) and [N][P][Cpad] (NHWC).
// One block moves a tile of 32 channels x 256 pixels through shared memory so that both the
// global read and the global write are contiguous.  The element conversion (quantize,
// dequantize or none) happens on the way.
// ---------------------------------------------------------------------------------------------
constexpr int TC = 32;    // channels per tile
constexpr int TP = 256;   // pixels per tile (= threads per block)

struct QuantizeFn {
    // op_quantize_run_u8 (quantize.c:145-157) with saturate_float_by_bits (quant_helper.h:38-41):
    // t = (x - beta) / alpha in fp32 with beta = -(alpha * zp); the reference then truncates
    // (double)t + 0.5, which for 0 <= t <= qmax equals floor(t) + (t - floor(t) >= 0.5), exact in
    // fp32.  __fsub_rn/__fdiv_rn keep the two roundings separate (no contraction).
    float alpha, beta;
    int qmax;
    __device__ __forceinline__ uint8_t operator()(float x) const
    {
        float t = __fdiv_rn(__fsub_rn(x, beta), alpha);
        if (t > (float)qmax)
            return (uint8_t)qmax;
        if (t < 0.f)
            return 0;
        if (!(t == t))
            return 0;  // NaN: undefined in the reference
        float f = floorf(t);
        int v = (int)f + ((t - f) >= 0.5f ? 1 : 0);
        return (uint8_t)v;
    }
};

struct DequantizeFn {
    // op_dequantize_run_u8 (dequantize.c:111-123): ((int16)q - zp) * alpha, int -> float multiply.
    float alpha;
    int zp;
    __device__ __forceinline__ float operator()(uint8_t q) const
    {
        return __fmul_rn((float)((int)q - zp), alpha);
    }
};

struct QuantizeS8Fn {
    // op_quantize_run_i8 (quantize.c:159-185): clip(round(x * alpha), -l, l) with alpha = (float)(1. / oalpha)
    // (formed on the host), the float product rounded half away from zero -- roundf of the float equals the
    // reference's round() of the same value widened to double -- and the clip done on the rounded value.
    float alpha;
    int l;
    __device__ __forceinline__ uint8_t operator()(float x) const
    {
        const float r = roundf(__fmul_rn(x, alpha));
        if (!(r == r))
            return 0;  // NaN: undefined in the reference
        const int v = (int)fminf(fmaxf(r, (float)-l), (float)l);
        return (uint8_t)(int8_t)v;
    }
};

struct DequantizeS8Fn {
    // op_dequantize_run_i8 (dequantize.c:124-136): the int8 value as float, times alpha
    float alpha;
    __device__ __forceinline__ float operator()(uint8_t q) const { return __fmul_rn((float)(int)(int8_t)q, alpha); }
};

struct IdentityFn {
    __device__ __forceinline__ uint8_t operator()(uint8_t q) const { return q; }
};

// in: [N][C][P] of TIn  ->  out: [N][P][c_pad] of uint8; channels c..c_pad-1 are written `fill`.
template <typename TIn, typename Fn>
__global__ void __launch_bounds__(TP) nchw_to_nhwc_kernel(
    const TIn *__restrict__ in, uint8_t *__restrict__ out, int C, int P, int c_pad, int fill, Fn fn)
{
    __shared__ uint8_t tile[TC][TP + 4];
    const int n = blockIdx.z;
    const int c0 = blockIdx.y * TC;
    const int p0 = blockIdx.x * TP;
    const int t = threadIdx.x;
    const int p = p0 + t;
    const TIn *src = in + ((size_t)n * C) * P;
    const int cend = min(TC, c_pad - c0);
#pragma unroll 4
    for (int c = 0; c < cend; ++c) {
        uint8_t v = (uint8_t)fill;
        if (c0 + c < C && p < P)
            v = fn(src[(size_t)(c0 + c) * P + p]);
        tile[c][t] = v;
    }
    __syncthreads();
    if (p >= P)
        return;
    uint8_t *dst = out + ((size_t)n * P + p) * c_pad + c0;
    if (cend == TC && (c_pad & 15) == 0) {
        uint32_t wv[8];
#pragma unroll
        for (int j = 0; j < 8; ++j)
            wv[j] = pack4(tile[4 * j][t], tile[4 * j + 1][t], tile[4 * j + 2][t], tile[4 * j + 3][t]);
        uint4 *d4 = reinterpret_cast<uint4 *>(dst);
        d4[0] = make_uint4(wv[0], wv[1], wv[2], wv[3]);
        d4[1] = make_uint4(wv[4], wv[5], wv[6], wv[7]);
    } else if ((c_pad & 3) == 0 && (cend & 3) == 0) {
        for (int j = 0; j < cend / 4; ++j)
            reinterpret_cast<uint32_t *>(dst)[j]
                = pack4(tile[4 * j][t], tile[4 * j + 1][t], tile[4 * j + 2][t], tile[4 * j + 3][t]);
    } else {
        for (int c = 0; c < cend; ++c)
            dst[c] = tile[c][t];
    }
}

// in: [N][P][c_pad] uint8 -> out: [N][C][P] of TOut (channels >= C are dropped).
template <typename TOut, typename Fn>
__global__ void __launch_bounds__(TP) nhwc_to_nchw_kernel(
    const uint8_t *__restrict__ in, TOut *__restrict__ out, int C, int P, int c_pad, Fn fn)
{
    __shared__ uint8_t tile[TC][TP + 4];
    const int n = blockIdx.z;
    const int c0 = blockIdx.y * TC;
    const int p0 = blockIdx.x * TP;
    const int t = threadIdx.x;
    const int p = p0 + t;
    const int cend = min(TC, C - c0);
    if (p < P) {
        const uint8_t *src = in + ((size_t)n * P + p) * c_pad + c0;
        if (c0 + TC <= c_pad && (c_pad & 15) == 0) {
            const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
            uint4 a = s4[0], b = s4[1];
            uint32_t wv[8] = { a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w };
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                tile[4 * j + 0][t] = (uint8_t)(wv[j]);
                tile[4 * j + 1][t] = (uint8_t)(wv[j] >> 8);
                tile[4 * j + 2][t] = (uint8_t)(wv[j] >> 16);
                tile[4 * j + 3][t] = (uint8_t)(wv[j] >> 24);
            }
        } else {
            for (int c = 0; c < cend; ++c)
                tile[c][t] = src[c];
        }
    }
    __syncthreads();
    if (p >= P)
        return;
    TOut *dst = out + ((size_t)n * C) * P;
    for (int c = 0; c < cend; ++c)
        dst[(size_t)(c0 + c) * P + p] = fn(tile[c][t]);
}

// Flat variants (no layout change): 4 elements per thread.
template <typename Fn>
__global__ void quantize_flat_kernel(const float *__restrict__ in, uint8_t *__restrict__ out, size_t count, Fn fn)
{
    size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 4 <= count) {
        float4 v = *reinterpret_cast<const float4 *>(in + i);
        *reinterpret_cast<uint32_t *>(out + i) = pack4(fn(v.x), fn(v.y), fn(v.z), fn(v.w));
    } else {
        for (; i < count; ++i)
            out[i] = fn(in[i]);
    }
}

template <typename Fn>
__global__ void dequantize_flat_kernel(const uint8_t *__restrict__ in, float *__restrict__ out, size_t count, Fn fn)
{
    size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i + 4 <= count) {
        uint32_t q = *reinterpret_cast<const uint32_t *>(in + i);
        *reinterpret_cast<float4 *>(out + i) = make_float4(
            fn((uint8_t)q), fn((uint8_t)(q >> 8)), fn((uint8_t)(q >> 16)), fn((uint8_t)(q >> 24)));
    } else {
        for (; i < count; ++i)
            out[i] = fn(in[i]);
    }
}

// ---------------------------------------------------------------------------------------------
// eltwise SUM (eltwise.c:137-174): per input i, term_i = rshift_rn((x_i - zp_i) * m_i, b_i) with
// b_i = s_i - s0; t = sum term_i; y = sat_u(rshift_rn(t, s0) + ozp).  With
// rshift_rn(v, b) = (v + 2^(b-1)) >> b the term is (x_i * m_i + add_i) >> b_i where
// add_i = 2^(b_i-1) - zp_i * m_i is built on the host, one multiply-add and one shift per input.
// m_i < 2^22, so every intermediate fits int32 for b_i <= 30.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int elt_finish(int t, const EltwiseArgs &a)
{
    int v = ((t + a.round0) >> a.s0) + a.ozp;
    return sat_relu(v, a.qmax, a.relu_lo);
}

// FAST: obits == 8 and the final rounding term 2^(s0-1) << b[0] fits into add[0] (folded there by
// the host, exact because it is a multiple of 2^b[0]); then y = sat_u8(max((t >> s0) + ozp, relu_lo))
// and the saturation comes with the pack.  64 bytes per input per thread and iteration.
// PLAIN (with FAST): ozp == 0 and no floor above 0, so y = sat_u8(t >> s0) and the pack does the rest.
template <int N_IN, bool FAST, bool PLAIN = false, bool REV = false>
__global__ void __launch_bounds__(256) eltwise_sum_kernel(EltwiseArgs a, uint8_t *__restrict__ y, size_t count)
{
    constexpr int VPT = 4;   // 16-byte vectors per input per thread (2: 0.80 ms, 4: 0.78 ms, 8: 0.79 ms for the 16 adds of ResNet-50)
    const size_t nvec = count / 16;
    // a block works on tiles of 256 * VPT vectors; vector u of a thread lies 256 vectors after vector
    // u - 1, so that every load and store instruction of a warp covers 512 contiguous bytes
    const size_t ntile = nvec / (256 * VPT);
    for (size_t tile_i = blockIdx.x; tile_i < ntile; tile_i += gridDim.x) {
        const size_t tile = REV ? ntile - 1 - tile_i : tile_i;   // REV: from the last tile to the first
        const size_t v0 = tile * (256 * VPT) + threadIdx.x;
        uint32_t xin[N_IN][4 * VPT];
#pragma unroll
        for (int i = 0; i < N_IN; ++i)
#pragma unroll
            for (int u = 0; u < VPT; ++u) {
                uint4 q = __ldg(reinterpret_cast<const uint4 *>(a.x[i]) + v0 + u * 256);
                xin[i][4 * u + 0] = q.x; xin[i][4 * u + 1] = q.y; xin[i][4 * u + 2] = q.z; xin[i][4 * u + 3] = q.w;
            }
        uint32_t o[4 * VPT];
#pragma unroll
        for (int wd = 0; wd < 4 * VPT; ++wd) {
            int r[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int t = 0;
#pragma unroll
                for (int i = 0; i < N_IN; ++i) {
                    const int xv = (int)__byte_perm(xin[i][wd], 0, 0x4440 | e);   // byte e, zero-extended
                    t += (xv * a.m[i] + a.add[i]) >> a.b[i];
                }
                r[e] = PLAIN ? (t >> a.s0) : (FAST ? max((t >> a.s0) + a.ozp, a.relu_lo) : elt_finish(t, a));
            }
            o[wd] = FAST ? pack_sat_u8x4(r[0], r[1], r[2], r[3]) : pack4(r[0], r[1], r[2], r[3]);
        }
#pragma unroll
        for (int u = 0; u < VPT; ++u)
            reinterpret_cast<uint4 *>(y)[v0 + u * 256] = make_uint4(o[4 * u], o[4 * u + 1], o[4 * u + 2], o[4 * u + 3]);
    }
    // tail (what is left after whole tiles: less than 256 * VPT * 16 bytes)
    if (blockIdx.x == 0) {
        for (size_t e = ntile * (256 * VPT * 16) + threadIdx.x; e < count; e += blockDim.x) {
            int t = 0;
#pragma unroll
            for (int i = 0; i < N_IN; ++i)
                t += ((int)a.x[i][e] * a.m[i] + a.add[i]) >> a.b[i];
            int v = FAST ? min(max((t >> a.s0) + a.ozp, 0), 255) : elt_finish(t, a);
            y[e] = (uint8_t)(FAST ? max(v, a.relu_lo) : v);
        }
    }
}

// relu (relu.c:76-115): v = max(x, izp); y = sat_u(rshift_rn((v - izp) * m, s) + ozp), (m, s) from
// get_quant_scale(ialpha / oalpha, 24).  A 256-entry table built on the host with the exact
// 64-bit arithmetic turns the op into a byte lookup; the table sits in shared memory.
__global__ void __launch_bounds__(256) lut_u8_kernel(
    const uint8_t *__restrict__ x, uint8_t *__restrict__ y, size_t count, const uint8_t *__restrict__ lut_g)
{
    __shared__ uint8_t lut[256];
    lut[threadIdx.x] = lut_g[threadIdx.x];
    __syncthreads();
    const size_t nvec = count / 16;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t v = (size_t)blockIdx.x * blockDim.x + threadIdx.x; v < nvec; v += stride) {
        uint4 q = __ldg(reinterpret_cast<const uint4 *>(x) + v);
        uint32_t in[4] = { q.x, q.y, q.z, q.w }, o[4];
#pragma unroll
        for (int wd = 0; wd < 4; ++wd)
            o[wd] = pack4(
                lut[in[wd] & 0xff], lut[(in[wd] >> 8) & 0xff], lut[(in[wd] >> 16) & 0xff],
                lut[in[wd] >> 24]);
        reinterpret_cast<uint4 *>(y)[v] = make_uint4(o[0], o[1], o[2], o[3]);
    }
    if (blockIdx.x == 0)
        for (size_t e = nvec * 16 + threadIdx.x; e < count; e += blockDim.x)
            y[e] = lut[x[e]];
}

int relu_build_lut(
    float ialpha, uint8_t izp, float oalpha, uint8_t ozp, uint8_t obits, uint8_t lut[256])
{
    if (obits < 1 || obits > 8)
        return fail(B200_ERR_INVALID, "relu: obits outside 1..8");
    if (!(oalpha > 0.f) || !(ialpha > 0.f))
        return fail(B200_ERR_INVALID, "relu: scales must be positive");
    uint32_t m;
    int8_t s;
    get_quant_scale(ialpha / oalpha, 24, &m, &s);
    if (s < 1 || s > 62)
        return fail(B200_ERR_UNSUPPORTED, "relu: shift %d outside 1..62", (int)s);
    const int qmax = (1 << obits) - 1;
    for (int q = 0; q < 256; ++q) {
        int v = q >= izp ? q : izp;
        uint32_t prod = (uint32_t)(v - (int)izp) * m;   // relu.c:106, unsigned 32-bit product
        int32_t r = (int32_t)(rshift_rn_host((int64_t)prod, s) + ozp);
        lut[q] = (uint8_t)(r > qmax ? qmax : (r < 0 ? 0 : r));
    }
    return B200_OK;
}

int lut_u8_launch(const uint8_t *x, uint8_t *y, size_t count, const uint8_t *lut_dev, cudaStream_t st)
{
    if ((((uintptr_t)x | (uintptr_t)y) & 15) != 0)
        return fail(B200_ERR_INVALID, "relu: buffers must be 16-byte aligned");
    if (count == 0)
        return B200_OK;
    const int grid = resident_grid<lut_u8_kernel, 256>((count / 16 + 1 + 255) / 256);
    lut_u8_kernel<<<grid, 256, 0, st>>>(x, y, count, lut_dev);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

}  // namespace b200

namespace b200 {

// Host side of eltwise SUM: the per-input multipliers, addends and shifts of the kernel's
// arithmetic (see the comment above EltwiseArgs' kernel) from the reference's scale decomposition.
// *fast_out: obits == 8 and the final rounding term folded into the first input's addend.
int eltwise_prepare(
    int n_in, const float *ialpha, const uint8_t *izp, const float *coeff, float oalpha, uint8_t ozp,
    uint8_t obits, int relu, EltwiseArgs *out, bool *fast_out)
{
    if (n_in > kMaxEltIn)
        return fail(B200_ERR_UNSUPPORTED, "eltwise: at most %d inputs, got %d", kMaxEltIn, n_in);
    if (!(oalpha > 0.f))
        return fail(B200_ERR_INVALID, "eltwise: oalpha must be positive");
    EltwiseArgs &a = *out;
    uint32_t m[kMaxEltIn];
    int8_t s[kMaxEltIn];
    int s0 = 127;
    for (int i = 0; i < n_in; ++i) {
        float scale = (coeff ? coeff[i] : 1.0f) * ialpha[i] / oalpha;
        if (!(scale > 0.f))
            return fail(B200_ERR_INVALID, "eltwise: scale of input %d must be positive", i);
        get_quant_scale(scale, 23, &m[i], &s[i]);
        if (s[i] < s0)
            s0 = s[i];
    }
    s0 -= 1;  // eltwise.c:150
    if (s0 < 1 || s0 > 30)
        return fail(B200_ERR_UNSUPPORTED, "eltwise: final shift %d outside 1..30 (scale ratio too extreme)", s0);
    for (int i = 0; i < kMaxEltIn; ++i) {
        a.x[i] = nullptr; a.m[i] = 0; a.add[i] = 0; a.b[i] = 1;
    }
    for (int i = 0; i < n_in; ++i) {
        int b = (int)s[i] - s0;
        if (b < 1 || b > 30)
            return fail(B200_ERR_UNSUPPORTED, "eltwise: per-input shift %d outside 1..30", b);
        a.m[i] = (int)m[i];
        a.b[i] = b;
        const long long add = (1ll << (b - 1)) - (long long)izp[i] * (long long)m[i];
        // the kernels form x * m + add in int32 where the reference's rshift_rn works on int64
        // (quant_helper.h:55-58): decline what would not fit (shifts of 25 and more with a small zero point)
        const long long hi = 255ll * (long long)m[i] + add, lo = add;
        if (hi >= (1ll << 31) || lo < -(1ll << 31))
            return fail(B200_ERR_UNSUPPORTED, "eltwise: input %d needs more than 32 bits before its shift of %d (scale ratio too extreme)", i, b);
        a.add[i] = (int)add;
    }
    {
        long long worst = 1ll << (s0 - 1);
        for (int i = 0; i < n_in; ++i)
            worst += ((255ll * a.m[i]) >> a.b[i]) + 1;
        if (worst >= (1ll << 31))
            return fail(B200_ERR_UNSUPPORTED, "eltwise: the int32 sum could overflow");
    }
    a.n_in = n_in;
    a.rev = 0;
    a.s0 = s0;
    a.round0 = 1 << (s0 - 1);
    a.ozp = ozp;
    a.qmax = (1 << obits) - 1;
    a.relu_lo = relu ? ozp : 0;
    // fold the final rounding term into the first input's addend when that stays inside int32
    bool fast = a.qmax == 255;
    {
        long long folded = (long long)a.add[0] + ((long long)a.round0 << a.b[0]);
        long long worst = folded < 0 ? -folded : folded;
        worst += 255ll * a.m[0];
        if (fast && worst < (1ll << 31))
            a.add[0] = (int)folded;
        else
            fast = false;
    }
    *fast_out = fast;
    return B200_OK;
}

}  // namespace b200

namespace b200 {

// Images of up to four channels (the network input, C = 3) into 4-channel NHWC pixels: a thread
// reads four consecutive pixels of every plane (one word each) and writes four pixels (16 bytes).
// The pixel count of a plane must be a multiple of 4 and the planes word aligned.  Four such quads
// per thread and round, a grid stride apart, with all their loads issued before the first is used:
// one quad per round keeps 12 bytes per thread in flight, too few to cover the memory latency.
__global__ void __launch_bounds__(256) nchw_to_nhwc_c4_kernel(
    const uint8_t *__restrict__ x, uint4 *__restrict__ y, int c, uint32_t quads_per_image, uint32_t total, uint8_t fill)
{
    constexpr int UNR = 4;
    const uint32_t fill4 = (uint32_t)fill * 0x01010101u;
    const uint32_t stride = gridDim.x * blockDim.x;
    for (uint32_t idx0 = blockIdx.x * blockDim.x + threadIdx.x; idx0 < total; idx0 += UNR * stride) {
        uint32_t p[UNR][4];
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const uint32_t idx = idx0 + u * stride;
            const uint32_t img = idx / quads_per_image, q = idx - img * quads_per_image;
            const uint32_t *planes = reinterpret_cast<const uint32_t *>(x) + (size_t)img * c * quads_per_image + q;
#pragma unroll
            for (int ch = 0; ch < 4; ++ch)
                p[u][ch] = (ch < c && idx < total) ? __ldg(planes + (size_t)ch * quads_per_image) : fill4;
        }
#pragma unroll
        for (int u = 0; u < UNR; ++u) {
            const uint32_t idx = idx0 + u * stride;
            // 4x4 byte transpose: word j of the result holds byte j of every plane
            const uint32_t t0 = __byte_perm(p[u][0], p[u][1], 0x5140), t1 = __byte_perm(p[u][2], p[u][3], 0x5140);
            const uint32_t t2 = __byte_perm(p[u][0], p[u][1], 0x7362), t3 = __byte_perm(p[u][2], p[u][3], 0x7362);
            if (idx < total)
                y[idx] = make_uint4(__byte_perm(t0, t1, 0x5410), __byte_perm(t0, t1, 0x7632),
                                    __byte_perm(t2, t3, 0x5410), __byte_perm(t2, t3, 0x7632));
        }
    }
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_quantize_u8(
    const float *x, uint8_t *y, int32_t n, int32_t c, int32_t h, int32_t w, float oalpha,
    uint8_t ozp, uint8_t obits, int32_t nhwc, b200_stream_t stream)
{
    if (!x || !y || n < 0 || c <= 0 || h <= 0 || w <= 0 || obits < 1 || obits > 8)
        return fail(B200_ERR_INVALID, "quantize: bad argument");
    if (!(oalpha > 0.f))
        return fail(B200_ERR_INVALID, "quantize: oalpha must be positive");
    if (n == 0)
        return B200_OK;
    QuantizeFn fn;
    fn.alpha = oalpha;
    fn.beta = -(oalpha * (float)ozp);
    fn.qmax = (1 << obits) - 1;
    const int P = h * w;
    if (nhwc && !(c == 1 || P == 1)) {
        dim3 grid((P + TP - 1) / TP, (c + TC - 1) / TC, n);
        nchw_to_nhwc_kernel<float, QuantizeFn><<<grid, TP, 0, as_stream(stream)>>>(x, y, c, P, c, 0, fn);
    } else {
        size_t count = (size_t)n * c * P;
        size_t threads = (count + 3) / 4;
        quantize_flat_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, as_stream(stream)>>>(x, y, count, fn);
    }
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_dequantize_u8(
    const uint8_t *x, float *y, int32_t n, int32_t c, int32_t h, int32_t w, float ialpha,
    uint8_t izp, int32_t nhwc, b200_stream_t stream)
{
    if (!x || !y || n < 0 || c <= 0 || h <= 0 || w <= 0)
        return fail(B200_ERR_INVALID, "dequantize: bad argument");
    if (n == 0)
        return B200_OK;
    DequantizeFn fn;
    fn.alpha = ialpha;
    fn.zp = izp;
    const int P = h * w;
    if (nhwc && !(c == 1 || P == 1)) {
        dim3 grid((P + TP - 1) / TP, (c + TC - 1) / TC, n);
        nhwc_to_nchw_kernel<float, DequantizeFn><<<grid, TP, 0, as_stream(stream)>>>(x, y, c, P, c, fn);
    } else {
        size_t count = (size_t)n * c * P;
        size_t threads = (count + 3) / 4;
        dequantize_flat_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, as_stream(stream)>>>(x, y, count, fn);
    }
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_quantize_s8(
    const float *x, int8_t *y8, int32_t n, int32_t c, int32_t h, int32_t w, float oalpha, uint8_t obits,
    int32_t nhwc, b200_stream_t stream)
{
    if (!x || !y8 || n < 0 || c <= 0 || h <= 0 || w <= 0 || obits < 2 || obits > 8)
        return fail(B200_ERR_INVALID, "quantize(int8): bad argument (obits 2..8)");
    if (!(oalpha > 0.f))
        return fail(B200_ERR_INVALID, "quantize(int8): oalpha must be positive");
    if (n == 0)
        return B200_OK;
    uint8_t *y = reinterpret_cast<uint8_t *>(y8);
    QuantizeS8Fn fn;
    fn.alpha = (float)(1. / (double)oalpha);
    fn.l = (1 << (obits - 1)) - 1;
    const int P = h * w;
    if (nhwc && !(c == 1 || P == 1)) {
        dim3 grid((P + TP - 1) / TP, (c + TC - 1) / TC, n);
        nchw_to_nhwc_kernel<float, QuantizeS8Fn><<<grid, TP, 0, as_stream(stream)>>>(x, y, c, P, c, 0, fn);
    } else {
        size_t count = (size_t)n * c * P;
        size_t threads = (count + 3) / 4;
        quantize_flat_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, as_stream(stream)>>>(x, y, count, fn);
    }
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_dequantize_s8(
    const int8_t *x8, float *y, int32_t n, int32_t c, int32_t h, int32_t w, float ialpha, int32_t nhwc,
    b200_stream_t stream)
{
    if (!x8 || !y || n < 0 || c <= 0 || h <= 0 || w <= 0)
        return fail(B200_ERR_INVALID, "dequantize(int8): bad argument");
    if (n == 0)
        return B200_OK;
    const uint8_t *x = reinterpret_cast<const uint8_t *>(x8);
    DequantizeS8Fn fn;
    fn.alpha = ialpha;
    const int P = h * w;
    if (nhwc && !(c == 1 || P == 1)) {
        dim3 grid((P + TP - 1) / TP, (c + TC - 1) / TC, n);
        nhwc_to_nchw_kernel<float, DequantizeS8Fn><<<grid, TP, 0, as_stream(stream)>>>(x, y, c, P, c, fn);
    } else {
        size_t count = (size_t)n * c * P;
        size_t threads = (count + 3) / 4;
        dequantize_flat_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, as_stream(stream)>>>(x, y, count, fn);
    }
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_nchw_to_nhwc_u8(
    const uint8_t *x, uint8_t *y, int32_t n, int32_t c, int32_t h, int32_t w, int32_t c_pad,
    uint8_t fill, b200_stream_t stream)
{
    if (!x || !y || n < 0 || c <= 0 || h <= 0 || w <= 0 || c_pad < c)
        return fail(B200_ERR_INVALID, "nchw_to_nhwc: bad argument");
    if (n == 0)
        return B200_OK;
    const int P = h * w;
    if (c_pad == 4 && P % 4 == 0 && (((uintptr_t)x) & 3) == 0 && (((uintptr_t)y) & 15) == 0
        && (size_t)n * (P / 4) < 0xf0000000ull) {   // 32-bit indices, with room for the unrolled rounds past the end
        const uint32_t quads = (uint32_t)(P / 4), total = (uint32_t)n * quads;
        const int blocks = resident_grid<nchw_to_nhwc_c4_kernel, 256>(((size_t)total + 1023) / 1024);   // four quads per thread and round
        nchw_to_nhwc_c4_kernel<<<blocks, 256, 0, as_stream(stream)>>>(x, reinterpret_cast<uint4 *>(y), c, quads, total, fill);
        B200_CUDA_TRY(cudaGetLastError());
        return B200_OK;
    }
    dim3 grid((P + TP - 1) / TP, (c_pad + TC - 1) / TC, n);
    nchw_to_nhwc_kernel<uint8_t, IdentityFn><<<grid, TP, 0, as_stream(stream)>>>(x, y, c, P, c_pad, fill, IdentityFn());
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_nhwc_to_nchw_u8(
    const uint8_t *x, uint8_t *y, int32_t n, int32_t c, int32_t h, int32_t w, int32_t c_pad,
    b200_stream_t stream)
{
    if (!x || !y || n < 0 || c <= 0 || h <= 0 || w <= 0 || c_pad < c)
        return fail(B200_ERR_INVALID, "nhwc_to_nchw: bad argument");
    if (n == 0)
        return B200_OK;
    const int P = h * w;
    dim3 grid((P + TP - 1) / TP, (c + TC - 1) / TC, n);
    nhwc_to_nchw_kernel<uint8_t, IdentityFn><<<grid, TP, 0, as_stream(stream)>>>(x, y, c, P, c_pad, IdentityFn());
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int b200_eltwise_sum_u8(
    const uint8_t *const *xs, int32_t n_in, size_t count, const float *ialpha, const uint8_t *izp,
    const float *coeff, float oalpha, uint8_t ozp, uint8_t obits, int32_t relu, uint8_t *y,
    b200_stream_t stream)
{
    if (!xs || !ialpha || !izp || !y || n_in < 1 || obits < 1 || obits > 8)
        return fail(B200_ERR_INVALID, "eltwise: bad argument");
    EltwiseArgs a;
    bool fast = false;
    B200_TRY(eltwise_prepare(n_in, ialpha, izp, coeff, oalpha, ozp, obits, relu, &a, &fast));
    return eltwise_launch(a, fast, xs, y, count, 0, as_stream(stream));
}

}  // extern "C"

namespace b200 {

int eltwise_launch(const EltwiseArgs &prepared, bool fast, const uint8_t *const *xs, uint8_t *y, size_t count, int reverse,
                   cudaStream_t st)
{
    EltwiseArgs a = prepared;
    const int n_in = a.n_in;
    a.rev = reverse ? 1 : 0;
    for (int i = 0; i < n_in; ++i) {
        if (((uintptr_t)xs[i] & 15) != 0)
            return fail(B200_ERR_INVALID, "eltwise: input %d is not 16-byte aligned", i);
        a.x[i] = xs[i];
    }
    if (((uintptr_t)y & 15) != 0)
        return fail(B200_ERR_INVALID, "eltwise: output is not 16-byte aligned");
    if (count == 0)
        return B200_OK;
    const size_t want = count / (256 * 64) + 1;   // tiles of 256 threads x 64 bytes
#define B200_ELT_LAUNCH(...) \
    eltwise_sum_kernel<__VA_ARGS__><<<resident_grid<eltwise_sum_kernel<__VA_ARGS__>, 256>(want), 256, 0, st>>>(a, y, count)
    if (fast) {
        switch (n_in) {
        case 1: B200_ELT_LAUNCH(1, true); break;
        case 2:
            if (a.ozp == 0 && a.relu_lo <= 0)
                B200_ELT_LAUNCH(2, true, true);
            else if (a.rev)
                B200_ELT_LAUNCH(2, true, false, true);
            else
                B200_ELT_LAUNCH(2, true);
            break;
        case 3: B200_ELT_LAUNCH(3, true); break;
        default: B200_ELT_LAUNCH(4, true); break;
        }
    } else {
        switch (n_in) {
        case 1: B200_ELT_LAUNCH(1, false); break;
        case 2: B200_ELT_LAUNCH(2, false); break;
        case 3: B200_ELT_LAUNCH(3, false); break;
        default: B200_ELT_LAUNCH(4, false); break;
        }
    }
#undef B200_ELT_LAUNCH
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

}  // namespace b200

using namespace b200;

extern "C" {

int b200_relu_u8(
    const uint8_t *x, size_t count, float ialpha, uint8_t izp, float oalpha, uint8_t ozp,
    uint8_t obits, uint8_t *y, b200_stream_t stream)
{
    if (!x || !y)
        return fail(B200_ERR_INVALID, "relu: bad argument");
    uint8_t lut[256];
    B200_TRY(relu_build_lut(ialpha, izp, oalpha, ozp, obits, lut));
    if (count == 0)
        return B200_OK;
    const uint8_t *lut_dev = nullptr;
    B200_TRY(lut_cache_get(lut, &lut_dev));   // uploaded once per distinct table, then reused
    return lut_u8_launch(x, y, count, lut_dev, as_stream(stream));
}

}  // extern "C"
