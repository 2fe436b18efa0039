// conv_2d / ip plans: the one-time work the reference does (or repeats) in prepare and run --
// zero-point subtraction of the weights, scale decomposition, bias preload
// (art/modules/quant/src/op/conv_2d.c:95-147, conv_2d_uint8_impl.c:61-124 of ModelTC/NART) --
// done once here: weights repacked for the kernels, per-channel (mult, shift) tables, folded
// bias.  b200_conv2d_run then only launches.
#include <string.h>

#include <vector>

#include "common.cuh"
#include "kernels.h"

using namespace b200;

namespace {

template <typename T>
int upload(const std::vector<T> &v, T **dev)
{
    *dev = nullptr;
    if (v.empty())
        return B200_OK;
    B200_CUDA_TRY(cudaMalloc((void **)dev, v.size() * sizeof(T)));
    B200_CUDA_TRY(cudaMemcpy(*dev, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice));
    return B200_OK;
}

void destroy_conv(b200_conv *cv)
{
    if (!cv)
        return;
    cudaFree(cv->direct.w_dev);
    cudaFree(cv->direct.w_dw_dev);
    cudaFree(cv->direct.w_dw3_dev);
    cudaFree(cv->direct.w_dw3p_dev);
    cudaFree(cv->direct.q_dw3_dev);
    cudaFree(cv->direct.bias_fold_dev);
    cudaFree(cv->direct.mult_dev);
    cudaFree(cv->direct.shift_dev);
    if (cv->igemm)
        conv_igemm_destroy(cv->igemm);
    cudaFree(cv->scratch);
    cudaFree(cv->sums);
    delete cv;
}

}  // namespace

extern "C" {

int b200_conv2d_create(
    const b200_conv_params *p, const uint8_t *weights, const int32_t *bias, b200_conv_t **out)
{
    if (!p || !weights || !out)
        return fail(B200_ERR_INVALID, "conv: NULL argument");
    *out = nullptr;
    if (p->c <= 0 || p->h <= 0 || p->w <= 0 || p->k <= 0 || p->r <= 0 || p->s <= 0 || p->group <= 0
        || p->stride_h <= 0 || p->stride_w <= 0 || p->pad_h < 0 || p->pad_w < 0)
        return fail(B200_ERR_INVALID, "conv: non-positive dimension");
    if (p->c % p->group || p->k % p->group)
        return fail(B200_ERR_INVALID, "conv: c=%d and k=%d must be multiples of group=%d", p->c, p->k, p->group);
    if (p->h + 2 * p->pad_h < p->r || p->w + 2 * p->pad_w < p->s)
        return fail(B200_ERR_INVALID, "conv: kernel larger than the padded input");
    if (p->obits < 1 || p->obits > 8)
        return fail(B200_ERR_INVALID, "conv: obits=%d outside 1..8", (int)p->obits);
    if (!p->walpha || (p->n_walpha != 1 && p->n_walpha != p->k))
        return fail(B200_ERR_INVALID, "conv: n_walpha must be 1 or k");
    if (!(p->ialpha > 0.f) || !(p->oalpha > 0.f))
        return fail(B200_ERR_INVALID, "conv: ialpha and oalpha must be positive");
    if (p->algo != B200_CONV_ALGO_AUTO && p->algo != B200_CONV_ALGO_DIRECT && p->algo != B200_CONV_ALGO_IGEMM)
        return fail(B200_ERR_INVALID, "conv: unknown algo %d", p->algo);
    if (p->act_type != B200_ACT_U8 && p->act_type != B200_ACT_S8)
        return fail(B200_ERR_INVALID, "conv: unknown act_type %d", p->act_type);
    const bool s8 = p->act_type == B200_ACT_S8;
    if (s8 && p->obits == 8 && !p->s8_wrap)
        return fail(
            B200_ERR_UNSUPPORTED,
            "conv: int8 activations with obits = 8 clip at +-255 and then wrap into int8 in the reference "
            "(quant_helper.h:43-47); set s8_wrap to reproduce that, or use obits <= 7");
    if (s8 && p->obits == 8 && p->algo == B200_CONV_ALGO_IGEMM)
        return fail(B200_ERR_UNSUPPORTED, "conv: the wrapping int8 output exists on the CUDA-core path only");

    b200_conv *cv = new b200_conv();
    ConvGeom &g = cv->g;
    g.c = p->c; g.h = p->h; g.w = p->w; g.k = p->k; g.r = p->r; g.s = p->s;
    g.pad_h = p->pad_h; g.pad_w = p->pad_w; g.stride_h = p->stride_h; g.stride_w = p->stride_w;
    g.group = p->group;
    g.oh = (p->h + 2 * p->pad_h - p->r) / p->stride_h + 1;   // art/src/op.c:547-555
    g.ow = (p->w + 2 * p->pad_w - p->s) / p->stride_w + 1;
    g.izp = p->izp; g.ozp = p->ozp; g.qmax = (1 << p->obits) - 1;
    g.relu_lo = p->relu ? p->ozp : 0;
    g.wzp_d = (int)p->wzp - 128;
    g.act_signed = 0;
    g.s8_wrap = 0;
    if (s8) {
        const int m = (1 << p->obits) - 1;     // ssaturate_int_by_bits: +-(2^obits - 1)
        g.act_signed = 1;
        g.s8_wrap = p->obits == 8 ? 1 : 0;
        g.izp = 128; g.ozp = 128; g.wzp_d = 0;
        g.qmax = g.s8_wrap ? 255 : 128 + m;
        // the wrapping form works on the signed value itself (floor 0 or -255), the clipping one on value + 128
        g.relu_lo = g.s8_wrap ? (p->relu ? 0 : -255) : (p->relu ? 128 : 128 - m);
    }
    cv->oalpha = p->oalpha;
    cudaGetDevice(&cv->device);

    const int cg = g.c / g.group, taps = g.r * g.s;
    const size_t wcount = (size_t)g.k * cg * taps;
    // int32 accumulation wraps modulo 2^32 in every order, like the reference's int32 GEMM
    // (gemm/default/gemm.c:306-355), so no bound on the reduction length is needed.
    // Any stored byte minus 128 is an int8; a weight zero point other than 128 is carried as
    // wzp_d = wzp - 128 and applied through the sum of the activations (ConvGeom::wzp_d).
    std::vector<int8_t> w_s8(wcount);   // [k][cg][r][s], value = stored - 128
    for (size_t i = 0; i < wcount; ++i)
        w_s8[i] = s8 ? (int8_t)weights[i] : (int8_t)((int)weights[i] - 128);

    std::vector<uint32_t> mult(g.k);
    std::vector<int32_t> shift(g.k);
    for (int k = 0; k < g.k; ++k) {
        float wa = p->walpha[p->n_walpha == 1 ? 0 : k];
        if (!(wa > 0.f)) {
            destroy_conv(cv);
            return fail(B200_ERR_INVALID, "conv: walpha[%d] must be positive", k);
        }
        float scale = p->ialpha * wa / p->oalpha;   // conv_2d_uint8_impl.c:75, fp32, left to right
        uint32_t m;
        int8_t s;
        get_quant_scale(scale, 32, &m, &s);
        if (m == 0 || s < 1 || s > 62) {
            destroy_conv(cv);
            return fail(
                B200_ERR_UNSUPPORTED, "conv: scale %g of channel %d gives shift %d outside 1..62", (double)scale, k, (int)s);
        }
        mult[k] = m;
        shift[k] = s;
    }

    // ---- direct-kernel tables (always built: the accumulator-dumping entry uses them) --------
    const int cg4 = (cg + 3) / 4 * 4;
    std::vector<int8_t> w_pack((size_t)g.k * taps * cg4, 0);
    std::vector<int32_t> bias_fold(g.k);
    for (int k = 0; k < g.k; ++k) {
        long long wsum = 0;
        for (int c = 0; c < cg; ++c)
            for (int t = 0; t < taps; ++t) {
                int8_t v = w_s8[((size_t)k * cg + c) * taps + t];
                w_pack[((size_t)k * taps + t) * cg4 + c] = v;
                wsum += v;
            }
        long long bf = (long long)(bias ? bias[k] : 0) - (long long)g.izp * wsum;
        bias_fold[k] = (int32_t)(uint32_t)(unsigned long long)bf;   // modulo 2^32
    }
    cv->direct.cg4 = cg4;
    int rc = upload(w_pack, &cv->direct.w_dev);
    if (rc == B200_OK) rc = upload(bias_fold, &cv->direct.bias_fold_dev);
    if (rc == B200_OK) rc = upload(mult, &cv->direct.mult_dev);
    if (rc == B200_OK) rc = upload(shift, &cv->direct.shift_dev);
    if (rc == B200_OK && g.group == g.c && g.group == g.k && g.c % 16 == 0) {
        std::vector<int8_t> w_dw((size_t)taps * g.c);
        for (int c = 0; c < g.c; ++c)
            for (int t = 0; t < taps; ++t)
                w_dw[(size_t)t * g.c + c] = w_s8[(size_t)c * taps + t];
        rc = upload(w_dw, &cv->direct.w_dw_dev);
        // the dp4a form of the 3x3 case (conv_depthwise3x3_kernel)
        bool fast = g.r == 3 && g.s == 3 && g.qmax == 255 && g.wzp_d == 0;
        for (int k = 0; k < g.k && fast; ++k)
            fast = shift[k] >= 33 && shift[k] <= 53;
        if (rc == B200_OK && fast) {
            std::vector<uint32_t> w3((size_t)(g.c / 4) * 3 * 4, 0);
            std::vector<int4> q3(g.c);
            for (int c = 0; c < g.c; ++c) {
                for (int grp = 0; grp < 3; ++grp) {
                    uint32_t word = 0;
                    for (int j = 0; j < 4; ++j) {
                        const int t = grp * 4 + j;
                        if (t < 9)
                            word |= (uint32_t)(uint8_t)w_s8[(size_t)c * 9 + t] << (8 * j);
                    }
                    w3[((size_t)(c / 4) * 3 + grp) * 4 + (c % 4)] = word;
                }
                // (acc + bias_fold) * mult, rounded shift, + ozp  ==  (acc * mult + off64) >> shift
                const long long off64 = (long long)bias_fold[c] * (long long)mult[c] + (1ll << (shift[c] - 1))
                    + ((long long)g.ozp << shift[c]);
                q3[c] = make_int4((int)(uint32_t)(unsigned long long)off64, (int)(off64 >> 32), (int)mult[c], shift[c] - 32);
            }
            rc = upload(w3, &cv->direct.w_dw3_dev);
            if (rc == B200_OK) rc = upload(q3, &cv->direct.q_dw3_dev);
            if (rc == B200_OK && (g.stride_w == 1 || g.stride_w == 2)) {
                // one kernel row against 3 + stride_w neighbouring input pixels (conv_depthwise3x3_pair_kernel)
                const int nv = g.stride_w == 2 ? 3 : 2;
                std::vector<uint32_t> w3p((size_t)(g.c / 4) * 3 * nv * 4, 0);
                for (int c = 0; c < g.c; ++c)
                    for (int rr = 0; rr < 3; ++rr) {
                        uint32_t wb[3];
                        for (int j = 0; j < 3; ++j)
                            wb[j] = (uint32_t)(uint8_t)w_s8[(size_t)c * 9 + rr * 3 + j];
                        uint32_t *dst = &w3p[((size_t)(c / 4) * 3 + rr) * nv * 4 + (c % 4)];
                        dst[0] = wb[0] | (wb[1] << 8) | (wb[2] << 16);                   // left pixel: inputs 0..2
                        if (g.stride_w == 1) {
                            dst[4] = (wb[0] << 8) | (wb[1] << 16) | (wb[2] << 24);       // right pixel: inputs 1..3
                        } else {
                            dst[4] = (wb[0] << 16) | (wb[1] << 24);                      // right pixel: inputs 2, 3 ...
                            dst[8] = wb[2] << (8 * (c % 4));                             // ... and 4, at the channel's byte
                        }
                    }
                rc = upload(w3p, &cv->direct.w_dw3p_dev);
            }
        }
    }
    if (rc != B200_OK) {
        destroy_conv(cv);
        return rc;
    }

    // ---- tensor-core plan ---------------------------------------------------------------------
    char why[256] = "";
    const bool ig_ok = conv_igemm_supported(g, why, sizeof(why)) != 0 && !g.s8_wrap;
    // A 4-channel image with a short kernel row is no contraction the tensor cores can take as it
    // is (4 bytes per tap).  Gathering, for every input row and output column, the 8-pixel window
    // the kernel row slides over gives a 32-channel tensor [n][h][ow][8 pixels x 4 channels] on
    // which the same conv is an r x 1 kernel with stride (stride_h, 1): that is dense enough.
    // Window cells outside the image hold the byte izp, whose contribution the epilogue's
    // zero-point term removes exactly; cells past the kernel width get zero weights.
    const bool low_ok = g.group == 1 && g.c == 4 && g.s <= kLowerWindow && g.k >= 16 && g.stride_h <= 2
        && g.h >= g.stride_h && !g.act_signed;
    if (!ig_ok && low_ok && p->algo != B200_CONV_ALGO_DIRECT) {
        ConvGeom gl = g;
        gl.c = kLowerWindow * 4;
        gl.w = g.ow;
        gl.s = 1;
        gl.pad_w = 0;
        gl.stride_w = 1;
        std::vector<int8_t> w_low((size_t)g.k * gl.c * g.r, 0);   // [k][32][r][1]
        for (int k = 0; k < g.k; ++k)
            for (int c = 0; c < 4; ++c)
                for (int rr = 0; rr < g.r; ++rr)
                    for (int j = 0; j < g.s; ++j)
                        w_low[((size_t)k * gl.c + j * 4 + c) * g.r + rr] = w_s8[(((size_t)k * 4 + c) * g.r + rr) * g.s + j];
        rc = conv_igemm_create(gl, w_low, bias, mult.data(), shift.data(), &cv->igemm, true);
        if (rc == B200_OK) {
            cv->algo = B200_CONV_ALGO_IGEMM;
            cv->lowered = true;
            cv->g_low = gl;
            // for callers of b200_conv2d_run_static_scratch: everything that entry point would otherwise do
            // once per device (kernel set-up, the static array's address) happens here, where allocation is
            // allowed; a failure only matters to that entry point, which reports it itself
            if (conv_igemm_warm() != B200_OK || conv_static_scratch_prepare() != B200_OK)
                cudaGetLastError();
        } else if (rc != B200_ERR_UNSUPPORTED || p->algo == B200_CONV_ALGO_IGEMM) {
            destroy_conv(cv);
            return rc;
        }
    } else if (p->algo == B200_CONV_ALGO_IGEMM && !ig_ok) {
        destroy_conv(cv);
        return fail(B200_ERR_UNSUPPORTED, "conv: implicit-GEMM path declined: %s", why);
    }
    if (ig_ok && p->algo != B200_CONV_ALGO_DIRECT) {
        rc = conv_igemm_create(g, w_s8, bias, mult.data(), shift.data(), &cv->igemm);
        if (rc == B200_OK) {
            cv->algo = B200_CONV_ALGO_IGEMM;
        } else if (rc != B200_ERR_UNSUPPORTED || p->algo == B200_CONV_ALGO_IGEMM) {
            destroy_conv(cv);
            return rc;
        }   // declined under AUTO: the CUDA-core kernel runs it
    }
    *out = cv;
    return B200_OK;
}

int b200_ip_create(
    int32_t c, int32_t h, int32_t w, int32_t k, float ialpha, uint8_t izp, const float *walpha,
    int32_t n_walpha, uint8_t wzp, float oalpha, uint8_t ozp, uint8_t obits,
    const uint8_t *weights, const int32_t *bias, b200_conv_t **conv)
{
    // ip.cpp:133-209: y[n][k] = requant(bias[k] + sum_j (x[n][j] - izp) * (w[k][j] - wzp)) over the
    // flattened c*h*w input -- a convolution whose kernel is the whole image.
    b200_conv_params p;
    memset(&p, 0, sizeof(p));
    p.c = c; p.h = h; p.w = w; p.k = k; p.r = h; p.s = w;
    p.pad_h = p.pad_w = 0; p.stride_h = p.stride_w = 1; p.group = 1;
    p.ialpha = ialpha; p.izp = izp; p.wzp = wzp; p.ozp = ozp; p.obits = obits; p.oalpha = oalpha;
    p.walpha = walpha; p.n_walpha = n_walpha; p.relu = 0; p.algo = B200_CONV_ALGO_AUTO;
    return b200_conv2d_create(&p, weights, bias, conv);
}

int b200_ip_create_s8(
    int32_t c, int32_t h, int32_t w, int32_t k, float ialpha, const float *walpha, int32_t n_walpha,
    float oalpha, uint8_t obits, int32_t s8_wrap, const int8_t *weights, const int32_t *bias,
    b200_conv_t **conv)
{
    b200_conv_params p;
    memset(&p, 0, sizeof(p));
    p.c = c; p.h = h; p.w = w; p.k = k; p.r = h; p.s = w;
    p.pad_h = p.pad_w = 0; p.stride_h = p.stride_w = 1; p.group = 1;
    p.ialpha = ialpha; p.obits = obits; p.oalpha = oalpha;
    p.walpha = walpha; p.n_walpha = n_walpha; p.relu = 0; p.algo = B200_CONV_ALGO_AUTO;
    p.act_type = B200_ACT_S8; p.s8_wrap = s8_wrap;
    return b200_conv2d_create(&p, reinterpret_cast<const uint8_t *>(weights), bias, conv);
}

int b200_conv2d_out_dims(const b200_conv_t *conv, int32_t *oh, int32_t *ow)
{
    if (!conv || !oh || !ow)
        return fail(B200_ERR_INVALID, "conv: NULL argument");
    *oh = conv->g.oh;
    *ow = conv->g.ow;
    return B200_OK;
}

int b200_conv2d_algo(const b200_conv_t *conv) { return conv ? conv->algo : B200_ERR_INVALID; }

int b200_conv2d_describe(const b200_conv_t *conv, char *buf, size_t len)
{
    if (!conv || !buf || len == 0)
        return fail(B200_ERR_INVALID, "conv(describe): bad argument");
    if (conv->algo == B200_CONV_ALGO_IGEMM && conv->igemm) {
        conv_igemm_describe(conv->igemm, buf, len);
        if (conv->lowered) {
            size_t used = strlen(buf);
            snprintf(buf + used, len - used, ", on the row-lowered image");
        }
    } else {
        snprintf(buf, len, "CUDA cores (dp4a)%s", conv->g.group == conv->g.c && conv->g.group == conv->g.k ? ", depthwise" : "");
    }
    return B200_OK;
}

int b200_conv2d_run(b200_conv_t *conv, const uint8_t *x, int32_t n, uint8_t *y, b200_stream_t stream)
{
    if (!conv || n < 0 || (n > 0 && (!x || !y)))
        return fail(B200_ERR_INVALID, "conv: bad argument");
    if (n == 0)
        return B200_OK;
    if (conv->fused_residual)
        return fail(B200_ERR_INVALID, "conv: this plan has a residual add, run it with b200_conv2d_run_residual");
    B200_TRY(b200_conv2d_reserve(conv, n));   // grow-only scratch: the first call at a larger batch allocates (and synchronizes)
    const ConvGeom &g = conv->g;
    const int32_t *wsum = nullptr;
    if (conv->algo == B200_CONV_ALGO_IGEMM && g.wzp_d != 0) {
        int32_t *w = conv->sums + conv->sums_images * g.h * g.w;
        B200_TRY(conv_window_sum_launch(g, x, n, conv->sums, w, as_stream(stream)));
        wsum = w;
    }
    if (conv->lowered) {
        B200_TRY(conv_lower_rows_launch(g, x, n, conv->scratch, as_stream(stream)));
        return conv_igemm_launch(conv->igemm, conv->scratch, n, y, as_stream(stream), nullptr, nullptr, wsum);
    }
    if (conv->algo == B200_CONV_ALGO_IGEMM)
        return conv_igemm_launch(conv->igemm, x, n, y, as_stream(stream), nullptr, nullptr, wsum);
    return conv_direct_launch(conv->g, conv->direct, x, n, y, nullptr, as_stream(stream));
}

int b200_conv2d_reserve(b200_conv_t *conv, int32_t n)
{
    if (!conv || n < 0)
        return fail(B200_ERR_INVALID, "conv(reserve): bad argument");
    const ConvGeom &g = conv->g;
    if (conv->lowered) {
        const size_t need = (size_t)n * g.h * g.ow * (kLowerWindow * 4);
        if (need > conv->scratch_bytes) {
            B200_CUDA_TRY(cudaFree(conv->scratch));
            conv->scratch = nullptr;
            conv->scratch_bytes = 0;
            B200_TRY(b200_malloc((void **)&conv->scratch, need));
            conv->scratch_bytes = need;
        }
    }
    if (conv->algo == B200_CONV_ALGO_IGEMM && g.wzp_d != 0 && (size_t)n > conv->sums_images) {
        B200_CUDA_TRY(cudaFree(conv->sums));
        conv->sums = nullptr;
        conv->sums_images = 0;
        B200_TRY(b200_malloc((void **)&conv->sums, (size_t)n * ((size_t)g.h * g.w + (size_t)g.oh * g.ow) * sizeof(int32_t)));
        conv->sums_images = (size_t)n;
    }
    return B200_OK;
}

int b200_conv2d_fuse_residual_add(
    b200_conv_t *conv, int32_t conv_input, const float *ialpha, const uint8_t *izp,
    const float *coeff, float oalpha, uint8_t ozp, uint8_t obits, int32_t relu)
{
    if (!conv || !ialpha || !izp || conv_input < 0 || conv_input > 1)
        return fail(B200_ERR_INVALID, "conv(fuse): bad argument");
    if (conv->algo != B200_CONV_ALGO_IGEMM || conv->lowered || !conv->igemm)
        return fail(B200_ERR_UNSUPPORTED, "conv(fuse): only plans on the tensor-core path take a residual add");
    if (conv->g.wzp_d != 0)
        return fail(B200_ERR_UNSUPPORTED, "conv(fuse): a weight zero point other than 128 and a fused residual add do not combine");
    if (conv->g.act_signed)
        return fail(B200_ERR_UNSUPPORTED, "conv(fuse): the residual add is a uint8 op (eltwise.c reads uint8 only)");
    if (conv->fused_residual)
        return fail(B200_ERR_INVALID, "conv(fuse): the plan already has a residual add");
    if (izp[conv_input] != (uint8_t)conv->g.ozp || ialpha[conv_input] != conv->oalpha)
        return fail(B200_ERR_UNSUPPORTED, "conv(fuse): the eltwise input's scale / zero point are not the conv's output ones");
    EltwiseArgs e;
    bool fast = false;
    B200_TRY(eltwise_prepare(2, ialpha, izp, coeff, oalpha, ozp, obits, relu, &e, &fast));
    if (!fast)
        return fail(B200_ERR_UNSUPPORTED, "conv(fuse): the eltwise rounding term does not fold (or obits != 8)");
    B200_TRY(conv_igemm_set_residual(conv->igemm, e, conv_input));
    conv->fused_residual = true;
    return B200_OK;
}

int b200_conv2d_run_residual(
    b200_conv_t *conv, const uint8_t *x, int32_t n, const uint8_t *res, uint8_t *y, b200_stream_t stream)
{
    if (!conv || n < 0 || (n > 0 && (!x || !y || !res)))
        return fail(B200_ERR_INVALID, "conv(residual): bad argument");
    if (!conv->fused_residual)
        return fail(B200_ERR_INVALID, "conv(residual): the plan has no residual add (b200_conv2d_fuse_residual_add)");
    if (n == 0)
        return B200_OK;
    return conv_igemm_launch(conv->igemm, x, n, y, as_stream(stream), nullptr, res);
}

int b200_conv2d_run_acc(
    b200_conv_t *conv, const uint8_t *x, int32_t n, uint8_t *y, int32_t *acc, b200_stream_t stream)
{
    if (!conv || !x || !y || !acc || n < 0)
        return fail(B200_ERR_INVALID, "conv: bad argument");
    return conv_direct_launch(conv->g, conv->direct, x, n, y, acc, as_stream(stream));
}

int b200_conv2d_destroy(b200_conv_t *conv)
{
    destroy_conv(conv);
    return B200_OK;
}

}  // extern "C"
