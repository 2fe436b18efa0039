/*
 * TEST INFRASTRUCTURE ONLY -- not part of the shipped library.
 *
 * CPU restatement ("port") of the arithmetic of NART's art `quant` module for the quantized
 * convolution path: plain C, host arrays in the reference's NCHW layout, no reference headers.
 * It is the checker the CUDA kernels are compared with, and it covers what the reference itself
 * cannot execute: batch > 1 in conv, one weight scale per output channel, a ReLU clamp fused
 * after the conv.  Every function cites the reference code it follows (paths relative to the
 * reference project root).
 *
 * Parity status: PINNED.  tests/test_oracle_pin.py checks every function here, byte for byte,
 * against the unmodified reference compiled into oracle/_ref/libnart_ref.so (through
 * oracle/ref_shim.c), and against fixtures under tests/golden/ that were produced by that
 * reference build (tests/golden/gen_golden.py).  The reference ships no tests or golden vectors
 * of its own for this module.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define PORT_API __attribute__((visibility("default")))

/* Round-half-up arithmetic right shift.
 * Follows art/modules/quant/include/art/quant/quant_helper.h:55-58:
 *   y = x >> (b-1);  result = (y + ((y & 1) << 1)) >> 1     (all shifts arithmetic, b >= 1)
 * y even -> y/2, y odd -> (y+1)/2. */
PORT_API int64_t port_rshift_rn(int64_t x, uint8_t bits)
{
    int64_t y = x >> (bits - 1);
    return (y + ((y & 1) << 1)) >> 1;
}

/* Decompose a positive float scale into multiplier and shift, scale ~= mult / 2^shift with
 * mult in [2^(bits-2), 2^(bits-1)).  Follows quant_helper.h:60-118 (`get_quant_scale_int32` is
 * bits == 32, `get_quant_scale_int16` is bits == -16 here and truncates to uint16,
 * `get_quant_scale(x, bits)` otherwise).  The halving/doubling loops are exact in fp32; the final
 * product is fp32 x (an exact power of two) and is truncated. */
PORT_API void port_get_quant_scale(float x, int bits, uint32_t *mult, int8_t *shift)
{
    int8_t sh = 0;
    int eff = bits == -16 ? 16 : bits;
    if (fabs(x - 0) < 1e-10) {
        *mult = 0;
        *shift = 0;
        return;
    }
    while (x >= 1.0f) {
        x /= 2;
        sh -= 1;
    }
    while (x < 0.5f) {
        x *= 2;
        sh += 1;
    }
    sh += eff - 1;
    if (bits == -16)
        *mult = (uint16_t)(x * (float)(1l << 15));
    else
        *mult = (uint32_t)(x * (float)(1ll << (eff - 1)));
    *shift = sh;
}

/* quant_helper.h:33-36 */
static inline uint8_t sat_u(int32_t x, uint8_t bits)
{
    int32_t hi = (1 << bits) - 1;
    return x > hi ? (uint8_t)hi : (x < 0 ? 0 : (uint8_t)x);
}

/* The requantize step shared by conv and ip (conv_2d_uint8_impl.c:159-164, ip.cpp:201-207):
 * the 64-bit rounded shift plus zero point is narrowed to int32 before saturation, exactly as
 * passing it to `saturate_int_by_bits(int32_t, ...)` does. */
static inline uint8_t requant_u8(int32_t acc, uint32_t mult, int8_t shift, uint8_t ozp, uint8_t obits)
{
    int64_t v = port_rshift_rn((int64_t)acc * (int64_t)mult, (uint8_t)shift) + ozp;
    return sat_u((int32_t)v, obits);
}

/*
 * conv_2d, uint8 activations and weights (art/modules/quant/src/op/conv_2d_uint8_impl.c:39-165):
 *   acc[k][p] = bias[k] + sum_{c,r,s} (x - izp) * (w - wzp), taps outside the image contribute 0
 *               because im2col runs on the zero-point-subtracted int16 copy (:107-109, :129);
 *   y = sat_u(rshift_rn(acc * mult, shift) + ozp, obits), (mult, shift) from
 *               get_quant_scale_int32(ialpha * walpha / oalpha) evaluated in fp32 (:75).
 * Extensions beyond what the reference executes (each pinned by a test against reference runs):
 *   - n > 1 (the reference aborts; per-image results are independent);
 *   - n_walpha == k: one (mult, shift) per output channel, each produced by the same function on
 *     ialpha * walpha[k] / oalpha; n_walpha == 1 is the reference's behaviour;
 *   - relu != 0: y = max(y, ozp), which is what the reference's relu op (relu.c:76-115) computes
 *     when its input and output scale and zero point are equal;
 *   - acc_out != NULL: the int32 accumulators (bias included) are also returned.
 * x: [n][c][h][w]  wt: [k][c/group][r][s]  bias: int32[k] or NULL  y: [n][k][oh][ow].
 */
PORT_API int port_conv2d_u8(
    const uint8_t *x, int n, int c, int h, int w, const uint8_t *wt, const int32_t *bias, int k,
    int r, int s, int pad_h, int pad_w, int stride_h, int stride_w, int group, float ialpha,
    uint8_t izp, const float *walpha, int n_walpha, uint8_t wzp, float oalpha, uint8_t ozp,
    uint8_t obits, int relu, uint8_t *y, int32_t *acc_out)
{
    int oh = (h + 2 * pad_h - r) / stride_h + 1;
    int ow = (w + 2 * pad_w - s) / stride_w + 1;
    int cg = c / group, kg = k / group;
    size_t wcount = (size_t)k * cg * r * s;
    int16_t *w16 = (int16_t *)malloc(sizeof(int16_t) * wcount);
    uint32_t *mult = (uint32_t *)malloc(sizeof(uint32_t) * k);
    int8_t *shift = (int8_t *)malloc(k);
    size_t i;
    int ko;
    if (n_walpha != 1 && n_walpha != k)
        return -1;
    for (i = 0; i < wcount; ++i)
        w16[i] = (int16_t)((int)wt[i] - (int)wzp);
    for (ko = 0; ko < k; ++ko)
        port_get_quant_scale(
            ialpha * walpha[n_walpha == 1 ? 0 : ko] / oalpha, 32, &mult[ko], &shift[ko]);
#pragma omp parallel for collapse(2) schedule(static)
    for (int in = 0; in < n; ++in) {
        for (int ko2 = 0; ko2 < k; ++ko2) {
            int g = ko2 / kg;
            int32_t *accrow = (int32_t *)malloc(sizeof(int32_t) * ow);
            for (int y0 = 0; y0 < oh; ++y0) {
                for (int x0 = 0; x0 < ow; ++x0)
                    accrow[x0] = bias ? bias[ko2] : 0;
                for (int ci = 0; ci < cg; ++ci) {
                    const uint8_t *xp = x + (((size_t)in * c + g * cg + ci) * h) * w;
                    const int16_t *wp = w16 + (((size_t)ko2 * cg + ci) * r) * s;
                    for (int rr = 0; rr < r; ++rr) {
                        int iy = y0 * stride_h + rr - pad_h;
                        if (iy < 0 || iy >= h)
                            continue;
                        for (int ss = 0; ss < s; ++ss) {
                            int32_t wv = wp[rr * s + ss];
                            int lo = 0, hi = ow;
                            /* ix = x0*stride_w + ss - pad_w must lie in [0, w) */
                            while (lo < ow && lo * stride_w + ss - pad_w < 0)
                                ++lo;
                            while (hi > lo && (hi - 1) * stride_w + ss - pad_w >= w)
                                --hi;
                            const uint8_t *xrow = xp + (size_t)iy * w + ss - pad_w;
                            for (int x0 = lo; x0 < hi; ++x0)
                                accrow[x0] += ((int32_t)xrow[x0 * stride_w] - (int32_t)izp) * wv;
                        }
                    }
                }
                size_t o = (((size_t)in * k + ko2) * oh + y0) * ow;
                for (int x0 = 0; x0 < ow; ++x0) {
                    uint8_t q = requant_u8(accrow[x0], mult[ko2], shift[ko2], ozp, obits);
                    if (relu && q < ozp)
                        q = ozp;
                    y[o + x0] = q;
                    if (acc_out)
                        acc_out[o + x0] = accrow[x0];
                }
            }
            free(accrow);
        }
    }
    free(w16);
    free(mult);
    free(shift);
    return 0;
}

/* ip / fully connected, uint8 path (art/modules/quant/src/op/ip.cpp:133-209): the same
 * accumulate and requantize as conv on a flattened input.  x: [n][chw], wt: [k][chw]. */
PORT_API int port_ip_u8(
    const uint8_t *x, int n, int chw, const uint8_t *wt, const int32_t *bias, int k, float ialpha,
    uint8_t izp, const float *walpha, int n_walpha, uint8_t wzp, float oalpha, uint8_t ozp,
    uint8_t obits, uint8_t *y)
{
    return port_conv2d_u8(
        x, n, chw, 1, 1, wt, bias, k, 1, 1, 0, 0, 1, 1, 1, ialpha, izp, walpha, n_walpha, wzp,
        oalpha, ozp, obits, 0, y, NULL);
}

/*
 * eltwise SUM (art/modules/quant/src/op/eltwise.c:137-174, tables built in prepare :241-252):
 *   (m_i, s_i) = get_quant_scale(coeff_i * ialpha_i / oalpha, 23);  s0 = min_i(s_i) - 1;
 *   t = sum_i (int32) rshift_rn((int32)(x_i - izp_i) * (int32)m_i, s_i - s0);
 *   y = sat_u(rshift_rn(t, s0) + ozp, obits).
 * `add` (add.c:83-148) is the two-input case with coeff 1; it orders the inputs by scale first,
 * which does not change the sum.  relu != 0 clamps at ozp afterwards (relu.c with equal scales).
 */
PORT_API int port_eltwise_sum_u8(
    const uint8_t *const *xs, int n_in, size_t count, const float *ialpha, const uint8_t *izp,
    const float *coeff, float oalpha, uint8_t ozp, uint8_t obits, int relu, uint8_t *y)
{
    uint32_t m[8];
    int8_t sh[8], s0 = 127;
    int i;
    if (n_in > 8)
        return -1;
    for (i = 0; i < n_in; ++i) {
        float cf = coeff ? coeff[i] : 1.0f;
        port_get_quant_scale(cf * ialpha[i] / oalpha, 23, &m[i], &sh[i]);
        if (sh[i] < s0)
            s0 = sh[i];
    }
    s0 = (int8_t)(s0 - 1);
    for (size_t e = 0; e < count; ++e) {
        int32_t t = 0;
        for (i = 0; i < n_in; ++i)
            t += (int32_t)port_rshift_rn(
                (int32_t)((int32_t)xs[i][e] - (int32_t)izp[i]) * (int32_t)m[i],
                (uint8_t)(sh[i] - s0));
        uint8_t q = sat_u((int32_t)(port_rshift_rn(t, (uint8_t)s0) + ozp), obits);
        if (relu && q < ozp)
            q = ozp;
        y[e] = q;
    }
    return 0;
}

/* relu (art/modules/quant/src/op/relu.c:76-115): clamp at the input zero point, then rescale
 * with get_quant_scale(ialpha / oalpha, 24). */
PORT_API int port_relu_u8(
    const uint8_t *x, size_t count, float ialpha, uint8_t izp, float oalpha, uint8_t ozp,
    uint8_t obits, uint8_t *y)
{
    uint32_t m;
    int8_t sh;
    port_get_quant_scale(ialpha / oalpha, 24, &m, &sh);
    for (size_t e = 0; e < count; ++e) {
        uint8_t v = x[e] >= izp ? x[e] : izp;
        uint32_t prod = (uint32_t)((int32_t)v - (int32_t)izp) * m;
        y[e] = sat_u((int32_t)(port_rshift_rn((int64_t)prod, (uint8_t)sh) + ozp), obits);
    }
    return 0;
}

/* Output extent of pool as the reference's shape inference decides it (art/src/op.c:903-967):
 * ceil or floor of (in + 2*pad - kernel) / stride + 1 in double, then, if any padding is set,
 * one step back when the last window would start at or beyond in + pad. */
PORT_API int port_pool_out_dim(int in, int kernel, int pad, int stride, int ceil_mode, int any_pad)
{
    double v = (in + pad * 2.0 - kernel) / stride + 1;
    int o = (int)(ceil_mode ? ceil(v) : floor(v));
    if (any_pad && (o - 1) * stride >= in + pad)
        --o;
    return o;
}

/*
 * pool.  method 0 = MAX (art/modules/quant/src/op/pool.c:96-168): max over the in-image part of
 * the window starting from 0, then (mult16, shift) = get_quant_scale_int16(ialpha / oalpha),
 * y = sat_u(rshift_rn((int32)mult16 * (max - izp), shift) + ozp).
 * method 1 = AVE (pool.c:170-249): pool_size counts padded cells up to in + pad;
 * (mult, shift) = get_quant_scale(ialpha / oalpha / pool_size, 16) per output pixel;
 * sum over in-image cells of (x - izp); y = sat_u(rshift_rn((int32)mult * sum, shift) + ozp).
 */
PORT_API int port_pool_u8(
    const uint8_t *x, int n, int c, int h, int w, int method, int kernel_h, int kernel_w, int pad_h,
    int pad_w, int stride_h, int stride_w, int ceil_mode, float ialpha, uint8_t izp, float oalpha,
    uint8_t ozp, uint8_t obits, uint8_t *y, int *out_hw)
{
    int any_pad = pad_h || pad_w;
    int oh = port_pool_out_dim(h, kernel_h, pad_h, stride_h, ceil_mode, any_pad);
    int ow = port_pool_out_dim(w, kernel_w, pad_w, stride_w, ceil_mode, any_pad);
    out_hw[0] = oh;
    out_hw[1] = ow;
    if (!y)
        return 0;
    uint32_t m16;
    int8_t sh16;
    port_get_quant_scale(ialpha / oalpha, -16, &m16, &sh16);
    for (int in = 0; in < n; ++in)
        for (int ci = 0; ci < c; ++ci) {
            const uint8_t *xp = x + ((size_t)in * c + ci) * h * w;
            uint8_t *yp = y + ((size_t)in * c + ci) * oh * ow;
            for (int y0 = 0; y0 < oh; ++y0)
                for (int x0 = 0; x0 < ow; ++x0) {
                    int hs = y0 * stride_h - pad_h, wsx = x0 * stride_w - pad_w;
                    if (method == 0) {
                        int he = hs + kernel_h < h ? hs + kernel_h : h;
                        int we = wsx + kernel_w < w ? wsx + kernel_w : w;
                        int h0 = hs > 0 ? hs : 0, w0 = wsx > 0 ? wsx : 0;
                        uint8_t mx = 0;
                        for (int i = h0; i < he; ++i)
                            for (int j = w0; j < we; ++j)
                                if (xp[i * w + j] > mx)
                                    mx = xp[i * w + j];
                        int32_t prod = (int32_t)m16 * ((int32_t)mx - (int32_t)izp);
                        yp[y0 * ow + x0]
                            = sat_u((int32_t)(port_rshift_rn(prod, (uint8_t)sh16) + ozp), obits);
                    } else {
                        int he = hs + kernel_h < h + pad_h ? hs + kernel_h : h + pad_h;
                        int we = wsx + kernel_w < w + pad_w ? wsx + kernel_w : w + pad_w;
                        uint32_t pool_size = (uint32_t)((he - hs) * (we - wsx));
                        uint32_t m;
                        int8_t sh;
                        port_get_quant_scale(ialpha / oalpha / pool_size, 16, &m, &sh);
                        int h0 = hs > 0 ? hs : 0, w0 = wsx > 0 ? wsx : 0;
                        he = he < h ? he : h;
                        we = we < w ? we : w;
                        int32_t sum = 0;
                        for (int i = h0; i < he; ++i)
                            for (int j = w0; j < we; ++j)
                                sum += (int32_t)xp[i * w + j] - (int32_t)izp;
                        int32_t prod = (int32_t)m * sum;
                        yp[y0 * ow + x0]
                            = sat_u((int32_t)(port_rshift_rn(prod, (uint8_t)sh) + ozp), obits);
                    }
                }
        }
    return 0;
}

/* quantize float32 -> uint8 (art/modules/quant/src/op/quantize.c:145-157 with
 * quant_helper.h:38-41): beta = -(alpha * zp) and t = (x - beta) / alpha in fp32; t > 2^bits-1
 * saturates high, t < 0 saturates to 0, otherwise truncate (double)t + 0.5. */
PORT_API int port_quantize_u8(
    const float *x, size_t count, float oalpha, uint8_t ozp, uint8_t obits, uint8_t *y)
{
    volatile float beta = -(oalpha * ozp);
    int hi = (1 << obits) - 1;
    for (size_t e = 0; e < count; ++e) {
        volatile float d = x[e] - beta;
        volatile float t = d / oalpha;
        y[e] = t > hi ? (uint8_t)hi : (t < 0 ? 0 : (uint8_t)((double)t + 0.5));
    }
    return 0;
}

/* dequantize uint8 -> float32 (art/modules/quant/src/op/dequantize.c:111-123). */
PORT_API int port_dequantize_u8(const uint8_t *x, size_t count, float ialpha, uint8_t izp, float *y)
{
    for (size_t e = 0; e < count; ++e)
        y[e] = (float)((int)(int16_t)x[e] - (int)izp) * ialpha;
    return 0;
}

/* ------------------------------------------------------------------------------------------
 * The int8 ("dtINT8", symmetric) path of the reference: no zero points anywhere.
 * ------------------------------------------------------------------------------------------ */

/* quant_helper.h:31 and :43-47: clip to +-(2^bits - 1), then the function's int8_t return type
 * truncates.  For bits <= 7 nothing is lost; for bits == 8 the bound is +-255 and the cast wraps
 * (200 -> -56), which is what the reference computes. */
static inline int8_t ssat(int32_t x, uint8_t bits)
{
    int32_t m = (1 << bits) - 1;
    int32_t c = x > m ? m : (x < -m ? -m : x);
    return (int8_t)(uint8_t)(uint32_t)c;
}

/* conv_2d, int8 activations and weights (art/modules/quant/src/op/conv_2d_int8_impl.c:34-174):
 *   acc = bias[k] + sum x * w  over the in-image taps (im2col_i8 writes zeros for the others,
 *   utils/im2col.cpp:22-116), y = ssat(rshift_rn(acc * mult, shift), obits) with (mult, shift)
 *   from get_quant_scale_int32(ialpha * walpha / oalpha).
 * Extensions as in port_conv2d_u8: n > 1, one scale per output channel (n_walpha == k).
 * x: [n][c][h][w] int8, wt: [k][c/group][r][s] int8, y: [n][k][oh][ow] int8. */
PORT_API int port_conv2d_i8(
    const int8_t *x, int n, int c, int h, int w, const int8_t *wt, const int32_t *bias, int k, int r,
    int s, int pad_h, int pad_w, int stride_h, int stride_w, int group, float ialpha,
    const float *walpha, int n_walpha, float oalpha, uint8_t obits, int8_t *y)
{
    int oh = (h + 2 * pad_h - r) / stride_h + 1;
    int ow = (w + 2 * pad_w - s) / stride_w + 1;
    int cg = c / group, kg = k / group;
    uint32_t *mult = (uint32_t *)malloc(sizeof(uint32_t) * k);
    int8_t *shift = (int8_t *)malloc(k);
    if (n_walpha != 1 && n_walpha != k)
        return -1;
    for (int ko = 0; ko < k; ++ko)
        port_get_quant_scale(ialpha * walpha[n_walpha == 1 ? 0 : ko] / oalpha, 32, &mult[ko], &shift[ko]);
#pragma omp parallel for collapse(2) schedule(static)
    for (int in = 0; in < n; ++in)
        for (int ko = 0; ko < k; ++ko) {
            int g = ko / kg;
            for (int y0 = 0; y0 < oh; ++y0)
                for (int x0 = 0; x0 < ow; ++x0) {
                    int32_t acc = bias ? bias[ko] : 0;
                    for (int ci = 0; ci < cg; ++ci)
                        for (int rr = 0; rr < r; ++rr) {
                            int iy = y0 * stride_h + rr - pad_h;
                            if (iy < 0 || iy >= h)
                                continue;
                            for (int ss = 0; ss < s; ++ss) {
                                int ix = x0 * stride_w + ss - pad_w;
                                if (ix < 0 || ix >= w)
                                    continue;
                                acc += (int32_t)x[(((size_t)in * c + g * cg + ci) * h + iy) * w + ix]
                                    * (int32_t)wt[(((size_t)ko * cg + ci) * r + rr) * s + ss];
                            }
                        }
                    int64_t v = port_rshift_rn((int64_t)acc * (int64_t)mult[ko], (uint8_t)shift[ko]);
                    y[(((size_t)in * k + ko) * oh + y0) * ow + x0] = ssat((int32_t)v, obits);
                }
        }
    free(mult);
    free(shift);
    return 0;
}

/* ip, int8 path (art/modules/quant/src/op/ip.cpp:210-274). x: [n][chw], wt: [k][chw]. */
PORT_API int port_ip_i8(
    const int8_t *x, int n, int chw, const int8_t *wt, const int32_t *bias, int k, float ialpha,
    const float *walpha, int n_walpha, float oalpha, uint8_t obits, int8_t *y)
{
    return port_conv2d_i8(x, n, chw, 1, 1, wt, bias, k, 1, 1, 0, 0, 1, 1, 1, ialpha, walpha, n_walpha, oalpha, obits, y);
}

/* quantize float32 -> int8, qtype SYMMETRIC (quantize.c:159-185): alpha = 1. / oalpha is a double
 * division narrowed to float; x * alpha is a float product that `round` (half away from zero)
 * takes as a double; the result is clipped to +-(2^(bits-1) - 1) by the int-typed clip of
 * quant_helper.h:31, whose double argument converts to int by truncation. */
PORT_API int port_quantize_i8(const float *x, size_t count, float oalpha, uint8_t obits, int8_t *y)
{
    volatile float alpha = (float)(1. / (double)oalpha);
    int l = (int)((1l << (obits - 1)) - 1);
    for (size_t e = 0; e < count; ++e) {
        volatile float prod = x[e] * alpha;
        int v = (int)round((double)prod);
        y[e] = (int8_t)(v > l ? l : (v < -l ? -l : v));
    }
    return 0;
}

/* dequantize int8 -> float32 (dequantize.c:124-136): the int8 value converted to float, times alpha. */
PORT_API int port_dequantize_i8(const int8_t *x, size_t count, float ialpha, float *y)
{
    for (size_t e = 0; e < count; ++e)
        y[e] = (float)x[e] * ialpha;
    return 0;
}
