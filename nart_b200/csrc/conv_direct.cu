// CUDA-core convolution kernels (dp4a) for the shapes that are not dense contractions: grouped and
// depthwise convs, tiny channel counts (the 3-channel stem), and any shape the tensor-core path
// declines.  Arithmetic follows op_conv_2d_u8xu8_run of the reference CPU module
// (art/modules/quant/src/op/conv_2d_uint8_impl.c:39-165 of ModelTC/NART):
//   acc = bias[k] + sum (x - izp) * (w - wzp),  taps outside the image contribute 0,
//   y   = sat_u(rshift_rn(acc * mult_k, shift_k) + ozp, obits).
// The kernels multiply the raw uint8 activation by the signed weight (dp4a.u32.s32) and read an
// out-of-image tap as the byte `izp`; with bias_fold[k] = bias[k] - izp * sum(w[k]) this gives the
// same int32 accumulator.
#include "common.cuh"
#include "kernels.h"

namespace b200 {

__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c)
{
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// ---------------------------------------------------------------------------------------------
// Generic tiled kernel.  Block = 256 threads = 32 output pixels x 8 quads of output channels
// (32 channels of one group).  The reduction runs over "items" = 4-channel words of
// [r][s][cg4]; the weights of the block's 32 channels are staged through shared memory in
// chunks of 64 items as [item][channel] so that a quad reads one 16-byte vector per item.
// ---------------------------------------------------------------------------------------------
constexpr int DK = 32;       // output channels per block
constexpr int DP = 32;       // output pixels per block
constexpr int DCHUNK = 64;   // items per shared-memory stage

template <bool WORD_LOADS>
__global__ void __launch_bounds__(256) conv_direct_kernel(
    ConvGeom g, int cg4, const uint8_t *__restrict__ x, const uint32_t *__restrict__ wq,
    const int32_t *__restrict__ bias_fold, const uint32_t *__restrict__ mult,
    const int32_t *__restrict__ shift, uint8_t *__restrict__ y, int32_t *__restrict__ acc_out, int n)
{
    __shared__ __align__(16) uint32_t wsm[DCHUNK][DK];
    const int tid = threadIdx.x;
    const int kq = tid & 7;
    const int pl = tid >> 3;
    const int kg = g.k / g.group, cg = g.c / g.group;
    const int ktiles = (kg + DK - 1) / DK;
    const int grp = blockIdx.y / ktiles;
    const int kt = blockIdx.y % ktiles;
    const int k_in_g0 = kt * DK;               // first channel of the tile inside the group
    const int kvalid = min(DK, kg - k_in_g0);  // channels of this tile that exist
    const int k0 = grp * kg + k_in_g0;
    const size_t npix = (size_t)n * g.oh * g.ow;
    const size_t pix = (size_t)blockIdx.x * DP + pl;
    const bool pvalid = pix < npix;
    int ox = 0, oy = 0, img = 0;
    if (pvalid) {
        ox = (int)(pix % g.ow);
        oy = (int)((pix / g.ow) % g.oh);
        img = (int)(pix / ((size_t)g.ow * g.oh));
    }
    const int iy0 = oy * g.stride_h - g.pad_h, ix0 = ox * g.stride_w - g.pad_w;
    const int cwords = cg4 / 4;
    const int items = g.r * g.s * cwords;
    const uint32_t izp4 = (uint32_t)g.izp * 0x01010101u;
    const uint32_t x_flip = g.act_signed ? 0x80808080u : 0u;   // int8 bytes seen as uint8 with zero point 128
    const uint8_t *ximg = x + (size_t)img * g.h * g.w * g.c + (size_t)grp * cg;

    int acc[4] = { 0, 0, 0, 0 };
    // wzp != 128: sum of the bytes the products see (out-of-image taps read izp, like the products),
    // with the bytes past the group's last channel masked out of the last word
    int xsum = 0;
    const uint32_t last_ones = 0x01010101u >> (8 * (cg4 - cg));
    for (int item0 = 0; item0 < items; item0 += DCHUNK) {
        const int nitem = min(DCHUNK, items - item0);
        __syncthreads();
        for (int i = tid; i < DCHUNK * DK; i += 256) {
            int it = i / DK, kl = i % DK;
            uint32_t v = 0;
            if (it < nitem && kl < kvalid)
                v = __ldg(wq + (size_t)(k0 + kl) * items + item0 + it);
            wsm[it][kl] = v;
        }
        __syncthreads();
        if (pvalid) {
            int tap = item0 / cwords, cw = item0 % cwords;
            for (int it = 0; it < nitem; ++it) {
                int rr = tap / g.s, ss = tap % g.s;
                int iy = iy0 + rr, ix = ix0 + ss;
                uint32_t xv = izp4;
                if (iy >= 0 && iy < g.h && ix >= 0 && ix < g.w) {
                    const uint8_t *px = ximg + ((size_t)iy * g.w + ix) * g.c + cw * 4;
                    if (WORD_LOADS) {
                        xv = __ldg(reinterpret_cast<const uint32_t *>(px));
                    } else {
                        xv = 0;
#pragma unroll
                        for (int b = 0; b < 4; ++b)
                            if (cw * 4 + b < cg)
                                xv |= (uint32_t)__ldg(px + b) << (8 * b);
                    }
                    xv ^= x_flip;   // (bytes past the group's last channel meet zero weights)
                }
                uint4 wv = *reinterpret_cast<const uint4 *>(&wsm[it][kq * 4]);
                acc[0] = dp4a_us(xv, wv.x, acc[0]);
                acc[1] = dp4a_us(xv, wv.y, acc[1]);
                acc[2] = dp4a_us(xv, wv.z, acc[2]);
                acc[3] = dp4a_us(xv, wv.w, acc[3]);
                if (g.wzp_d != 0)
                    xsum = (int)__dp4a(xv, cw == cwords - 1 ? last_ones : 0x01010101u, (unsigned)xsum);
                if (++cw == cwords) {
                    cw = 0;
                    ++tap;
                }
            }
        }
    }
    if (!pvalid)
        return;
    int q[4] = { 0, 0, 0, 0 };
    int nk = min(4, kvalid - kq * 4);
    for (int j = 0; j < 4; ++j) {
        if (j >= nk)
            break;
        int k = k0 + kq * 4 + j;
        int a = acc[j] + bias_fold[k];
        if (g.wzp_d != 0)   // sum (x - izp) over all taps (the out-of-image ones give 0) times -(wzp - 128)
            a -= g.wzp_d * (xsum - g.izp * g.r * g.s * cg);
        if (acc_out)
            acc_out[pix * g.k + k] = a;
        if (g.s8_wrap) {
            // ssaturate_int_by_bits(v, 8): clip at +-255, then the int8 return type keeps the low byte
            const int v = requant_raw(a, mult[k], shift[k], 0);
            q[j] = max(min(v, 255), g.relu_lo) & 0xff;
        } else {
            q[j] = sat_relu(requant_raw(a, mult[k], shift[k], g.ozp), g.qmax, g.relu_lo) ^ (g.act_signed ? 0x80 : 0);
        }
    }
    uint8_t *py = y + pix * g.k + k0 + kq * 4;
    if (nk == 4 && (((size_t)g.k | (size_t)k0) & 3) == 0) {
        *reinterpret_cast<uint32_t *>(py) = pack4(q[0], q[1], q[2], q[3]);
    } else {
        for (int j = 0; j < nk; ++j)
            py[j] = (uint8_t)q[j];
    }
}

// ---------------------------------------------------------------------------------------------
// Depthwise kernel (group == c == k, c % 16 == 0).  A thread owns 16 consecutive channels of one
// output pixel: one 16-byte activation vector and one 16-byte weight vector per tap, products
// formed per channel.  Weights are [r][s][c] int8.  HBM-bound: each activation byte is read once
// from DRAM (neighbouring taps hit L1/L2), each output byte written once.
// ---------------------------------------------------------------------------------------------
template <bool WZP>
__global__ void __launch_bounds__(256) conv_depthwise_kernel(
    ConvGeom g, const uint8_t *__restrict__ x, const int8_t *__restrict__ w_rsc,
    const int32_t *__restrict__ bias_fold, const uint32_t *__restrict__ mult,
    const int32_t *__restrict__ shift, uint8_t *__restrict__ y, int n)
{
    const int cv = g.c / 16;
    const size_t total = (size_t)n * g.oh * g.ow * cv;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int ci = (int)(idx % cv);
        const size_t pix = idx / cv;
        const int ox = (int)(pix % g.ow);
        const int oy = (int)((pix / g.ow) % g.oh);
        const int img = (int)(pix / ((size_t)g.ow * g.oh));
        const int iy0 = oy * g.stride_h - g.pad_h, ix0 = ox * g.stride_w - g.pad_w;
        int acc[16];
        {
            const int4 *b4 = reinterpret_cast<const int4 *>(bias_fold + ci * 16);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int4 b = __ldg(b4 + j);
                acc[4 * j] = b.x; acc[4 * j + 1] = b.y; acc[4 * j + 2] = b.z; acc[4 * j + 3] = b.w;
            }
        }
        // WZP: every channel is its own group, so the correction -(wzp - 128) * sum (x - izp) is per
        // channel: fold it into the weight, w - wzp = s8 - wzp_d, with izp at the out-of-image taps
        // (x - izp = 0 there) and the constant izp * taps * wzp_d added back
        if (WZP) {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                acc[j] += g.izp * g.r * g.s * g.wzp_d;
        }
        for (int rr = 0; rr < g.r; ++rr) {
            const int iy = iy0 + rr;
            for (int ss = 0; ss < g.s; ++ss) {
                const int ix = ix0 + ss;
                uint4 wv = __ldg(reinterpret_cast<const uint4 *>(w_rsc + ((size_t)(rr * g.s + ss) * g.c) + ci * 16));
                uint4 xv;
                if (iy >= 0 && iy < g.h && ix >= 0 && ix < g.w) {
                    xv = __ldg(reinterpret_cast<const uint4 *>(
                        x + (((size_t)img * g.h + iy) * g.w + ix) * g.c + ci * 16));
                } else {
                    uint32_t z = (uint32_t)g.izp * 0x01010101u;
                    xv = make_uint4(z, z, z, z);
                }
                const uint32_t xw[4] = { xv.x, xv.y, xv.z, xv.w };
                const uint32_t ww[4] = { wv.x, wv.y, wv.z, wv.w };
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    int xb = (int)((xw[j / 4] >> (8 * (j % 4))) & 0xff);
                    int wb = (int)(int8_t)((ww[j / 4] >> (8 * (j % 4))) & 0xff);
                    if (WZP)
                        wb -= g.wzp_d;   // 9 bits: fine in the 32-bit multiply
                    acc[j] += xb * wb;
                }
            }
        }
        uint32_t o[4];
#pragma unroll
        for (int wd = 0; wd < 4; ++wd) {
            int q[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                int k = ci * 16 + wd * 4 + e;
                q[e] = sat_relu(requant_raw(acc[wd * 4 + e], __ldg(mult + k), __ldg(shift + k), g.ozp), g.qmax, g.relu_lo);
            }
            o[wd] = pack4(q[0], q[1], q[2], q[3]);
        }
        *reinterpret_cast<uint4 *>(y + pix * g.k + ci * 16) = make_uint4(o[0], o[1], o[2], o[3]);
    }
}

// ---------------------------------------------------------------------------------------------
// Depthwise 3x3 on dp4a.  A thread owns four consecutive channels of one output pixel.  The nine
// tap words (four channels each) are transposed four at a time with byte permutes into words that
// hold four taps of ONE channel, which dp4a multiplies with the matching weight word
// [c/4][tap group][channel]: 8 permutes + 4 dp4a per 16 multiply-adds instead of 16 extractions
// and 16 multiply-adds.  The requantize is the folded form of the tensor-core epilogue:
// y = sat_u8(max((acc * mult + off64) >> shift, floor)), the host having checked shift >= 33.
// Neighbouring threads read neighbouring words of a pixel and write neighbouring output words.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void transpose4x4(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t (&ch)[4])
{
    const uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(c, d, 0x5140);   // a0 b0 a1 b1 | c0 d0 c1 d1
    const uint32_t t2 = __byte_perm(a, b, 0x7362), t3 = __byte_perm(c, d, 0x7362);   // a2 b2 a3 b3 | c2 d2 c3 d3
    ch[0] = __byte_perm(t0, t1, 0x5410);
    ch[1] = __byte_perm(t0, t1, 0x7632);
    ch[2] = __byte_perm(t2, t3, 0x5410);
    ch[3] = __byte_perm(t2, t3, 0x7632);
}

__global__ void __launch_bounds__(256) conv_depthwise3x3_kernel(
    ConvGeom g, const uint32_t *__restrict__ x, const uint4 *__restrict__ w3, const int4 *__restrict__ q3,
    uint32_t *__restrict__ y, int n)
{
    const uint32_t cq = (uint32_t)g.c / 4;
    const uint32_t total = (uint32_t)n * g.oh * g.ow * cq;      // the launcher checks that it fits 32 bits
    const uint32_t izp4 = (uint32_t)g.izp * 0x01010101u;
    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const uint32_t ci = idx % cq;
        const uint32_t pix = idx / cq;
        const int ox = (int)(pix % (uint32_t)g.ow);
        const uint32_t rowi = pix / (uint32_t)g.ow;
        const int oy = (int)(rowi % (uint32_t)g.oh);
        const uint32_t img = rowi / (uint32_t)g.oh;
        const int iy0 = oy * g.stride_h - g.pad_h, ix0 = ox * g.stride_w - g.pad_w;
        // word offsets fit 32 bits (checked by the launcher)
        const uint32_t row_pitch = (uint32_t)g.w * cq;
        const uint32_t *xc = x + (img * (uint32_t)g.h * row_pitch + ci);
        uint32_t t[9];
        if (iy0 >= 0 && iy0 + 2 < g.h && ix0 >= 0 && ix0 + 2 < g.w) {
            const uint32_t *p0 = xc + ((uint32_t)iy0 * row_pitch + (uint32_t)ix0 * cq);
#pragma unroll
            for (int rr = 0; rr < 3; ++rr)
#pragma unroll
                for (int ss = 0; ss < 3; ++ss)
                    t[rr * 3 + ss] = __ldg(p0 + (rr * row_pitch + ss * cq));
        } else {
#pragma unroll
            for (int rr = 0; rr < 3; ++rr)
#pragma unroll
                for (int ss = 0; ss < 3; ++ss) {
                    const int iy = iy0 + rr, ix = ix0 + ss;
                    t[rr * 3 + ss] = (iy >= 0 && iy < g.h && ix >= 0 && ix < g.w)
                        ? __ldg(xc + ((uint32_t)iy * row_pitch + (uint32_t)ix * cq)) : izp4;
                }
        }
        const uint4 wa = __ldg(w3 + (size_t)ci * 3), wb = __ldg(w3 + (size_t)ci * 3 + 1), wc = __ldg(w3 + (size_t)ci * 3 + 2);
        uint32_t ch[4];
        int acc[4];
        transpose4x4(t[0], t[1], t[2], t[3], ch);
        acc[0] = dp4a_us(ch[0], wa.x, 0); acc[1] = dp4a_us(ch[1], wa.y, 0);
        acc[2] = dp4a_us(ch[2], wa.z, 0); acc[3] = dp4a_us(ch[3], wa.w, 0);
        transpose4x4(t[4], t[5], t[6], t[7], ch);
        acc[0] = dp4a_us(ch[0], wb.x, acc[0]); acc[1] = dp4a_us(ch[1], wb.y, acc[1]);
        acc[2] = dp4a_us(ch[2], wb.z, acc[2]); acc[3] = dp4a_us(ch[3], wb.w, acc[3]);
        // the ninth tap: byte j of the word against byte 0 of the weight word
        acc[0] = dp4a_us(t[8] & 0xffu, wc.x, acc[0]); acc[1] = dp4a_us((t[8] >> 8) & 0xffu, wc.y, acc[1]);
        acc[2] = dp4a_us((t[8] >> 16) & 0xffu, wc.z, acc[2]); acc[3] = dp4a_us(t[8] >> 24, wc.w, acc[3]);
        int q[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int4 c4 = __ldg(q3 + (size_t)ci * 4 + j);
            const long long off = (long long)(((unsigned long long)(uint32_t)c4.y << 32) | (uint32_t)c4.x);
            const long long prod = (long long)acc[j] * c4.z + off;
            q[j] = max((int)(prod >> 32) >> c4.w, g.relu_lo);
        }
        y[idx] = pack_sat_u8x4(q[0], q[1], q[2], q[3]);
    }
}

// ---------------------------------------------------------------------------------------------
// Depthwise 3x3 with horizontal stride S (1 or 2): a thread computes two output pixels side by
// side, in ROWS (1 or 2) output rows.  The two windows of a row cover 3 + S neighbouring input
// pixels per kernel row.  One transpose of the first four of those words gives, per channel, a
// word (x0, x1, x2, x3) that serves both pixels: dp4a against (w0, w1, w2, 0) is the left pixel's
// kernel row; the right pixel's is (0, w0, w1, w2) for S == 1, and for S == 2 (0, 0, w0, w1) plus
// the fifth word against w2 placed at the channel's own byte (no extraction).  With ROWS == 2 (the
// vertical stride is S as well) the output rows share 3 - S of their input rows.  The per-channel
// weights and requantize constants are read once per thread.  Arithmetic and results equal
// conv_depthwise3x3_kernel.  Weight table: [c/4][3 kernel rows][2 + (S == 2)][4 channels] words.
// ---------------------------------------------------------------------------------------------
template <int ROWS, int S>
__global__ void __launch_bounds__(256) conv_depthwise3x3_pair_kernel(
    ConvGeom g, const uint32_t *__restrict__ x, const uint4 *__restrict__ w3p, const int4 *__restrict__ q3,
    uint32_t *__restrict__ y, int n)
{
    constexpr int IN_ROWS = 3 + (ROWS - 1) * S, IN_COLS = 3 + S, NV = S == 2 ? 3 : 2;
    const uint32_t cq = (uint32_t)g.c / 4;
    const uint32_t owp = ((uint32_t)g.ow + 1) / 2, ohp = ((uint32_t)g.oh + ROWS - 1) / ROWS;
    const uint32_t total = (uint32_t)n * ohp * owp * cq;      // the launcher checks that it fits 32 bits
    const uint32_t izp4 = (uint32_t)g.izp * 0x01010101u;
    for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
        const uint32_t ci = idx % cq;
        const uint32_t pp = idx / cq;
        const int ox = (int)(pp % owp) * 2;
        const uint32_t rowi = pp / owp;
        const int oy = (int)(rowi % ohp) * ROWS;
        const uint32_t img = rowi / ohp;
        const int iy0 = oy * g.stride_h - g.pad_h, ix0 = ox * S - g.pad_w;   // ROWS == 2 only with stride_h == S
        const uint32_t row_pitch = (uint32_t)g.w * cq;
        const uint32_t *xc = x + (img * (uint32_t)g.h * row_pitch + ci);
        uint32_t t[IN_ROWS][IN_COLS];
        if (iy0 >= 0 && iy0 + IN_ROWS - 1 < g.h && ix0 >= 0 && ix0 + IN_COLS - 1 < g.w) {
            const uint32_t *p0 = xc + ((uint32_t)iy0 * row_pitch + (uint32_t)ix0 * cq);
#pragma unroll
            for (int rr = 0; rr < IN_ROWS; ++rr)
#pragma unroll
                for (int ss = 0; ss < IN_COLS; ++ss)
                    t[rr][ss] = __ldg(p0 + (rr * row_pitch + ss * cq));
        } else {
#pragma unroll
            for (int rr = 0; rr < IN_ROWS; ++rr)
#pragma unroll
                for (int ss = 0; ss < IN_COLS; ++ss) {
                    const int iy = iy0 + rr, ix = ix0 + ss;
                    t[rr][ss] = (iy >= 0 && iy < g.h && ix >= 0 && ix < g.w)
                        ? __ldg(xc + ((uint32_t)iy * row_pitch + (uint32_t)ix * cq)) : izp4;
                }
        }
        uint4 wv[3][NV];
#pragma unroll
        for (int rr = 0; rr < 3; ++rr)
#pragma unroll
            for (int v = 0; v < NV; ++v)
                wv[rr][v] = __ldg(w3p + ((size_t)ci * 3 + rr) * NV + v);
        int acc[ROWS][2][4];
#pragma unroll
        for (int o = 0; o < ROWS; ++o)
#pragma unroll
            for (int j = 0; j < 4; ++j)
                acc[o][0][j] = acc[o][1][j] = 0;
#pragma unroll
        for (int ir = 0; ir < IN_ROWS; ++ir) {
            uint32_t ch[4];
            transpose4x4(t[ir][0], t[ir][1], t[ir][2], t[ir][3], ch);
#pragma unroll
            for (int o = 0; o < ROWS; ++o) {
                const int kr = ir - o * S;     // kernel row this input row meets in output row o
                if (kr < 0 || kr > 2)
                    continue;
                const uint4 w0 = wv[kr][0], w1 = wv[kr][1];
                acc[o][0][0] = dp4a_us(ch[0], w0.x, acc[o][0][0]); acc[o][0][1] = dp4a_us(ch[1], w0.y, acc[o][0][1]);
                acc[o][0][2] = dp4a_us(ch[2], w0.z, acc[o][0][2]); acc[o][0][3] = dp4a_us(ch[3], w0.w, acc[o][0][3]);
                acc[o][1][0] = dp4a_us(ch[0], w1.x, acc[o][1][0]); acc[o][1][1] = dp4a_us(ch[1], w1.y, acc[o][1][1]);
                acc[o][1][2] = dp4a_us(ch[2], w1.z, acc[o][1][2]); acc[o][1][3] = dp4a_us(ch[3], w1.w, acc[o][1][3]);
                if (S == 2) {
                    const uint4 w2 = wv[kr][NV - 1];
                    const uint32_t x4 = t[ir][IN_COLS - 1];
                    acc[o][1][0] = dp4a_us(x4, w2.x, acc[o][1][0]); acc[o][1][1] = dp4a_us(x4, w2.y, acc[o][1][1]);
                    acc[o][1][2] = dp4a_us(x4, w2.z, acc[o][1][2]); acc[o][1][3] = dp4a_us(x4, w2.w, acc[o][1][3]);
                }
            }
        }
        int q[ROWS][2][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int4 c4 = __ldg(q3 + (size_t)ci * 4 + j);
            const long long off = (long long)(((unsigned long long)(uint32_t)c4.y << 32) | (uint32_t)c4.x);
#pragma unroll
            for (int o = 0; o < ROWS; ++o)
#pragma unroll
                for (int p = 0; p < 2; ++p)
                    q[o][p][j] = max((int)(((long long)acc[o][p][j] * c4.z + off) >> 32) >> c4.w, g.relu_lo);
        }
#pragma unroll
        for (int o = 0; o < ROWS; ++o) {
            if (oy + o >= g.oh)
                break;
            uint32_t *out = y + (((img * (uint32_t)g.oh + (uint32_t)(oy + o)) * (uint32_t)g.ow + (uint32_t)ox) * cq + ci);
            out[0] = pack_sat_u8x4(q[o][0][0], q[o][0][1], q[o][0][2], q[o][0][3]);
            if (ox + 1 < g.ow)
                out[cq] = pack_sat_u8x4(q[o][1][0], q[o][1][1], q[o][1][2], q[o][1][3]);
        }
    }
}

template <int ROWS, int S>
static void depthwise3x3_pair_launch(const ConvGeom &g, const ConvDirectPlan &p, const uint8_t *x, int n, uint8_t *y, cudaStream_t st)
{
    const size_t total = (size_t)n * ((g.oh + ROWS - 1) / ROWS) * ((g.ow + 1) / 2) * (g.c / 4);
    conv_depthwise3x3_pair_kernel<ROWS, S><<<resident_grid<conv_depthwise3x3_pair_kernel<ROWS, S>, 256>((total + 255) / 256), 256, 0, st>>>(
        g, reinterpret_cast<const uint32_t *>(x), reinterpret_cast<const uint4 *>(p.w_dw3p_dev), p.q_dw3_dev,
        reinterpret_cast<uint32_t *>(y), n);
}

// ---------------------------------------------------------------------------------------------
// Row lowering for the tensor-core path of 4-channel images (see kernels.h).  One thread builds
// one 32-byte window: eight 4-byte pixels, two 16-byte stores.  Neighbouring threads read
// overlapping windows, so the image is fetched from DRAM once.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) conv_lower_rows_kernel(
    const uint32_t *__restrict__ x, uint4 *__restrict__ out, int n, int h, int w, int ow, int stride_w, int pad_w,
    uint32_t izp4)
{
    const size_t total = (size_t)n * h * ow;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int ox = (int)(idx % ow);
        const size_t rowi = idx / ow;                       // n * h + ih
        const uint32_t *xrow = x + rowi * w;
        const int px0 = ox * stride_w - pad_w;
        uint32_t v[kLowerWindow];
#pragma unroll
        for (int j = 0; j < kLowerWindow; ++j) {
            const int px = px0 + j;
            v[j] = (px >= 0 && px < w) ? __ldg(xrow + px) : izp4;
        }
        // halves swapped where bit 2 of ox is set: the 32-byte swizzle, applied here in global memory
        const int sw = (ox >> 2) & 1;
        out[idx * 2 + sw] = make_uint4(v[0], v[1], v[2], v[3]);
        out[idx * 2 + (sw ^ 1)] = make_uint4(v[4], v[5], v[6], v[7]);
    }
}

int conv_lower_rows_launch(const ConvGeom &g, const uint8_t *x, int n, uint8_t *out, cudaStream_t st)
{
    if (n == 0)
        return B200_OK;
    if (g.c != 4 || (((uintptr_t)x) & 3) != 0 || (((uintptr_t)out) & 15) != 0)
        return fail(B200_ERR_INVALID, "conv(lower): needs a 4-channel, word-aligned input");
    const size_t total = (size_t)n * g.h * g.ow;
    const int blocks = resident_grid<conv_lower_rows_kernel, 256>((total + 255) / 256);
    conv_lower_rows_kernel<<<(unsigned)blocks, 256, 0, st>>>(
        reinterpret_cast<const uint32_t *>(x), reinterpret_cast<uint4 *>(out), n, g.h, g.w, g.ow, g.stride_w, g.pad_w,
        (uint32_t)g.izp * 0x01010101u);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

// ---------------------------------------------------------------------------------------------
// Window sums for the tensor-core path when wzp != 128 (see ConvGeom::wzp_d).  Two small passes:
// the channel sum of every input pixel (one read of the activations), then the sum of those over
// each output pixel's in-image taps, less izp for every byte summed.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) conv_channel_sum_kernel(
    const uint8_t *__restrict__ x, int32_t *__restrict__ csum, size_t pixels, int c)
{
    // a quarter warp per pixel: 8 lanes stride over the pixel's 16-byte (or 4-byte, or single) pieces
    const size_t pix = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    const int sub = threadIdx.x & 7;
    unsigned sum = 0;
    if (pix < pixels) {
        const uint8_t *px = x + pix * (size_t)c;
        if ((c & 15) == 0 && (((uintptr_t)x) & 15) == 0) {
            for (int i = sub; i < c / 16; i += 8) {
                const uint4 q = __ldg(reinterpret_cast<const uint4 *>(px) + i);
                sum = __dp4a(q.x, 0x01010101u, sum);
                sum = __dp4a(q.y, 0x01010101u, sum);
                sum = __dp4a(q.z, 0x01010101u, sum);
                sum = __dp4a(q.w, 0x01010101u, sum);
            }
        } else if ((c & 3) == 0 && (((uintptr_t)x) & 3) == 0) {
            for (int i = sub; i < c / 4; i += 8)
                sum = __dp4a(__ldg(reinterpret_cast<const uint32_t *>(px) + i), 0x01010101u, sum);
        } else {
            for (int i = sub; i < c; i += 8)
                sum += __ldg(px + i);
        }
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    sum += __shfl_xor_sync(0xffffffffu, sum, 4);
    if (pix < pixels && sub == 0)
        csum[pix] = (int32_t)sum;
}

__global__ void __launch_bounds__(256) conv_window_sum_kernel(
    ConvGeom g, const int32_t *__restrict__ csum, int32_t *__restrict__ wsum, size_t total)
{
    for (size_t pix = (size_t)blockIdx.x * blockDim.x + threadIdx.x; pix < total; pix += (size_t)gridDim.x * blockDim.x) {
        const int ox = (int)(pix % g.ow);
        const int oy = (int)((pix / g.ow) % g.oh);
        const size_t img = pix / ((size_t)g.ow * g.oh);
        const int iy0 = oy * g.stride_h - g.pad_h, ix0 = ox * g.stride_w - g.pad_w;
        int sum = 0, taps = 0;
        for (int rr = 0; rr < g.r; ++rr) {
            const int iy = iy0 + rr;
            if (iy < 0 || iy >= g.h)
                continue;
            for (int ss = 0; ss < g.s; ++ss) {
                const int ix = ix0 + ss;
                if (ix < 0 || ix >= g.w)
                    continue;
                sum += __ldg(csum + (img * g.h + iy) * g.w + ix);
                ++taps;
            }
        }
        wsum[pix] = sum - g.izp * g.c * taps;
    }
}

int conv_window_sum_launch(const ConvGeom &g, const uint8_t *x, int n, int32_t *csum, int32_t *wsum, cudaStream_t st)
{
    if (n == 0)
        return B200_OK;
    const size_t in_pix = (size_t)n * g.h * g.w, out_pix = (size_t)n * g.oh * g.ow;
    const size_t blocks = (in_pix * 8 + 255) / 256;
    if (blocks > 0x7fffffffull)
        return fail(B200_ERR_UNSUPPORTED, "conv(window sum): too many pixels");
    conv_channel_sum_kernel<<<(unsigned)blocks, 256, 0, st>>>(x, csum, in_pix, g.c);
    conv_window_sum_kernel<<<resident_grid<conv_window_sum_kernel, 256>((out_pix + 255) / 256), 256, 0, st>>>(
        g, csum, wsum, out_pix);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

int conv_direct_launch(
    const ConvGeom &g, const ConvDirectPlan &p, const uint8_t *x, int n, uint8_t *y, int32_t *acc_out,
    cudaStream_t st)
{
    if (n == 0)
        return B200_OK;
    const size_t npix = (size_t)n * g.oh * g.ow;
    const int kg = g.k / g.group, cg = g.c / g.group;
    const bool depthwise = p.w_dw_dev && !acc_out && !g.act_signed && ((((uintptr_t)x | (uintptr_t)y) & 15) == 0);
    const bool dw3 = depthwise && p.w_dw3_dev && p.q_dw3_dev && npix * (size_t)(g.c / 4) < 0xffffffffull
        && (size_t)n * g.h * g.w * (size_t)(g.c / 4) < 0xffffffffull;
    if (dw3 && p.w_dw3p_dev && (g.stride_w == 1 || g.stride_w == 2)) {
        // two output rows per thread where the vertical stride equals the horizontal one
        if (g.stride_w == 1 && g.stride_h == 1) depthwise3x3_pair_launch<2, 1>(g, p, x, n, y, st);
        else if (g.stride_w == 1) depthwise3x3_pair_launch<1, 1>(g, p, x, n, y, st);
        else if (g.stride_h == 2) depthwise3x3_pair_launch<2, 2>(g, p, x, n, y, st);
        else depthwise3x3_pair_launch<1, 2>(g, p, x, n, y, st);
    } else if (dw3) {
        const size_t total = npix * (g.c / 4);
        const int grid = resident_grid<conv_depthwise3x3_kernel, 256>((total + 255) / 256);
        conv_depthwise3x3_kernel<<<grid, 256, 0, st>>>(
            g, reinterpret_cast<const uint32_t *>(x), reinterpret_cast<const uint4 *>(p.w_dw3_dev), p.q_dw3_dev,
            reinterpret_cast<uint32_t *>(y), n);
    } else if (depthwise) {
        size_t total = npix * (g.c / 16);
        size_t blocks = (total + 255) / 256;
        size_t cap = (size_t)sm_count() * 8;
        int grid = (int)(blocks < cap ? blocks : cap);
        if (g.wzp_d != 0)
            conv_depthwise_kernel<true><<<grid, 256, 0, st>>>(g, x, p.w_dw_dev, p.bias_fold_dev, p.mult_dev, p.shift_dev, y, n);
        else
            conv_depthwise_kernel<false><<<grid, 256, 0, st>>>(g, x, p.w_dw_dev, p.bias_fold_dev, p.mult_dev, p.shift_dev, y, n);
    } else {
        const int ktiles = (kg + DK - 1) / DK;
        size_t gx = (npix + DP - 1) / DP;
        if (gx > 0x7fffffffull || (size_t)g.group * ktiles > 65535)
            return fail(B200_ERR_UNSUPPORTED, "conv(direct): grid too large");
        dim3 grid((unsigned)gx, (unsigned)(g.group * ktiles));
        const bool word = (g.c % 4 == 0) && (cg % 4 == 0) && (((uintptr_t)x & 3) == 0);
        const uint32_t *wq = reinterpret_cast<const uint32_t *>(p.w_dev);
        if (word)
            conv_direct_kernel<true><<<grid, 256, 0, st>>>(
                g, p.cg4, x, wq, p.bias_fold_dev, p.mult_dev, p.shift_dev, y, acc_out, n);
        else
            conv_direct_kernel<false><<<grid, 256, 0, st>>>(
                g, p.cg4, x, wq, p.bias_fold_dev, p.mult_dev, p.shift_dev, y, acc_out, n);
    }
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

}  // namespace b200
