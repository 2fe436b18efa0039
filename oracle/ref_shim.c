/*
 * TEST INFRASTRUCTURE ONLY -- not part of the shipped library.
 *
 * Flat C entry points that drive the UNMODIFIED reference `quant` module of NART's art runtime
 * through its own public op API (workspace_new_op / op_setting_*_set / op_config / op_prepare /
 * op_run), one op per call, on plain host arrays in the reference's NCHW layout.  The reference
 * sources are compiled where they lie by oracle/Makefile into oracle/_ref/libnart_ref.so together
 * with this file; nothing of the reference is copied into this repository.
 *
 * The way the op API is driven follows the reference's own C example
 * (examples/01-nart-case-cpu-example/src/main.c:25-74) and the settings each quant op reads in
 * its config function (art/modules/quant/src/op/conv_2d.c:27-70, pool.c:58-86, eltwise.c:51-92,
 * add.c:48-74, quantize.c:119-135, dequantize.c:84-101, ip.cpp:73-100).
 *
 * Constraints of the reference that this shim works around without changing results:
 *   - conv_2d sizes its int32 scratch without the batch factor and aborts for batch > 1
 *     (conv_2d_uint8_impl.c:32,104): images are run one at a time through one prepared op.
 *   - without a bias input the x86 accumulator is never cleared (conv_2d_uint8_impl.c:114-124):
 *     a zero bias is supplied when the caller passes NULL.
 *   - only walpha[0] is read (conv_2d_uint8_impl.c:61): per-tensor weight scale only.
 *   - im2col_i16 never writes the padding cells of its column buffer (every memset in
 *     utils/im2col.cpp:487-855 is commented out) and the buffer comes from malloc, so the result
 *     depends on what the heap held before: the scratch is cleared once after prepare, which is
 *     the state a fresh process gives it.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "art/module.h"
#include "art/op.h"
#include "art/op_settings.h"
#include "art/op_tp.h"
#include "art/quant/quant_module.h"
#include "art/quant/quant_op_settings.h"
#include "art/quant/quant_op_tp.h"
#include "art/quant/quant_helper.h"
/* the quant module's private op struct, for access to its im2col scratch */
#include "src/op/conv_2d.h"

#define REF_API __attribute__((visibility("default")))

static workspace_t *g_ws = NULL;
static const module_t *g_module = &quant_module_tp;
static int g_whole_batch = 0;   /* run conv on the whole batch at once (the reference itself cannot) */
static int g_conv_relu = 0;     /* set SETTING_CONV_2D_RELU_FLAG (the reference quant module ignores it) */

/* Drives another art module through the very same calls: the tests point this at the b200
 * plugin's `b200_module_tp`, which makes every function below a test of the plugin boundary. */
REF_API void ref_use_module(const module_t *module, int whole_batch, int conv_relu)
{
    if (g_ws) {
        workspace_delete(g_ws);
        g_ws = NULL;
    }
    g_module = module ? module : &quant_module_tp;
    g_whole_batch = whole_batch;
    g_conv_relu = conv_relu;
}

static workspace_t *ws(void)
{
    if (!g_ws)
        g_ws = workspace_new(g_module, NULL);
    return g_ws;
}

static tensor_t *new_tensor(uint32_t dtype, int dim_size, const int *dims)
{
    /* tensors live in the workspace's own mem type, as the reference's drivers create them
     * (tools/promark.cpp:179) */
    tensor_t *t = tensor_new(workspace_memtype(ws()), dtype);
    int i;
    t->shape.dim_size = dim_size;
    for (i = 0; i < dim_size; ++i)
        t->shape.dim[i] = (uint32_t)dims[i];
    if (dim_size == 1) {
        t->shape.batch_axis = 0;
        t->shape.channel_axis = -1;
    } else {
        t->shape.batch_axis = 0;
        t->shape.channel_axis = 1;
    }
    tensor_alloc(t);
    return t;
}

static void set_in_quant(op_t *op, int n, const float *alpha, const uint8_t *zp, const uint8_t *bits)
{
    CHECK(op_setting_array_set(op, SETTING_QUANT_IALPHA, dtFLOAT32, n, alpha));
    CHECK(op_setting_array_set(op, SETTING_QUANT_IZERO_POINT, dtUINT8, n, zp));
    CHECK(op_setting_array_set(op, SETTING_QUANT_IBITS, dtUINT8, n, bits));
}

static void set_out_quant(op_t *op, float alpha, uint8_t zp, uint8_t bits)
{
    CHECK(op_setting_array_set(op, SETTING_QUANT_OALPHA, dtFLOAT32, 1, &alpha));
    CHECK(op_setting_array_set(op, SETTING_QUANT_OZERO_POINT, dtUINT8, 1, &zp));
    CHECK(op_setting_array_set(op, SETTING_QUANT_OBITS, dtUINT8, 1, &bits));
}

static void set_w_quant(op_t *op, float alpha, uint8_t zp, uint8_t bits)
{
    CHECK(op_setting_array_set(op, SETTING_QUANT_WALPHA, dtFLOAT32, 1, &alpha));
    CHECK(op_setting_array_set(op, SETTING_QUANT_WZERO_POINT, dtUINT8, 1, &zp));
    CHECK(op_setting_array_set(op, SETTING_QUANT_WBITS, dtUINT8, 1, &bits));
}

/* The header's own scale decomposition, exported so tests can pin the restatement to it. */
REF_API void ref_get_quant_scale(float x, int bits, uint32_t *mult, int8_t *shift)
{
    if (bits == 32) {
        get_quant_scale_int32(x, mult, shift);
    } else if (bits == -16) { /* the uint16 variant used by max-pool */
        uint16_t m16 = 0;
        get_quant_scale_int16(x, &m16, shift);
        *mult = m16;
    } else {
        get_quant_scale(x, mult, shift, bits);
    }
}

REF_API int64_t ref_rshift_rn(int64_t x, uint8_t bits) { return rshift_rn(x, bits); }

/* conv_2d, uint8 path (art/modules/quant/src/op/conv_2d_uint8_impl.c:39-165). x: [n][c][h][w],
 * wt: [k][c/group][r][s] uint8, bias: int32[k] or NULL, y: [n][k][oh][ow]. */
REF_API int ref_conv2d_u8(
    const uint8_t *x, int n, int c, int h, int w, const uint8_t *wt, const int32_t *bias, int k,
    int r, int s, int pad_h, int pad_w, int stride_h, int stride_w, int group, float ialpha,
    uint8_t izp, float walpha, uint8_t wzp, float oalpha, uint8_t ozp, uint8_t obits, uint8_t *y)
{
    int per_run = g_whole_batch ? n : 1;
    int xd[4] = { per_run, c, h, w }, wd[4] = { k, c / group, r, s }, bd[1] = { k };
    tensor_t *tx = new_tensor(dtUINT8, 4, xd);
    tensor_t *tw = new_tensor(dtUINT8, 4, wd);
    tensor_t *tb = new_tensor(dtINT32, 1, bd);
    tensor_t *in[3] = { tx, tw, tb };
    float ia[3] = { ialpha, walpha, 1.f };
    uint8_t iz[3] = { izp, wzp, 0 }, ib[3] = { 8, 8, 32 };
    size_t xsz = (size_t)per_run * c * h * w, ysz;
    int i;
    op_t *op;
    /* weights and bias are in place before prepare, as after deserialization
     * (art/src/serialize_v2.c:211-280): a module may repack them there */
    memcpy(mem_cpu_data(tw->mem), wt, (size_t)k * (c / group) * r * s);
    if (bias)
        memcpy(mem_cpu_data(tb->mem), bias, sizeof(int32_t) * k);
    else
        memset(mem_cpu_data(tb->mem), 0, sizeof(int32_t) * k);
    op = workspace_new_op(ws(), OP_CONV_2D, 3, in);
    if (!op)
        return -1;
    if (g_conv_relu)
        CHECK(op_setting_single_set(op, SETTING_CONV_2D_RELU_FLAG, dtBOOL, 1));
    CHECK(op_setting_single_set(op, SETTING_CONV_2D_NUM_OUTPUT, dtUINT32, (uint32_t)k));
    CHECK(op_setting_single_set(op, SETTING_CONV_2D_KERNEL_H, dtUINT32, (uint32_t)r));
    CHECK(op_setting_single_set(op, SETTING_CONV_2D_KERNEL_W, dtUINT32, (uint32_t)s));
    CHECK(op_setting_single_set(op, SETTING_CONV_2D_PAD_H, dtUINT32, (uint32_t)pad_h));
    CHECK(op_setting_single_set(op, SETTING_CONV_2D_PAD_W, dtUINT32, (uint32_t)pad_w));
    CHECK(op_setting_single_set(op, SETTING_CONV_2D_STRIDE_H, dtUINT32, (uint32_t)stride_h));
    CHECK(op_setting_single_set(op, SETTING_CONV_2D_STRIDE_W, dtUINT32, (uint32_t)stride_w));
    CHECK(op_setting_single_set(op, SETTING_CONV_2D_GROUP, dtUINT32, (uint32_t)group));
    set_in_quant(op, 3, ia, iz, ib);
    set_w_quant(op, walpha, wzp, 8);
    set_out_quant(op, oalpha, ozp, obits);
    CHECK(op_config(op));
    op_prepare(op);
    if (g_module == &quant_module_tp) {
        op_conv_2d_t *conv_op = (op_conv_2d_t *)op;
        memset(mem_cpu_data(conv_op->temp_data), 0, mem_sizeof(conv_op->temp_data));
    }
    ysz = shape_count(&op->output_tensors[0].shape);
    for (i = 0; i < n; i += per_run) {
        memcpy(mem_cpu_data(tx->mem), x + xsz * (i / per_run), xsz);
        op_run(op);
        memcpy(y + ysz * (i / per_run), mem_cpu_data(op->output_tensors[0].mem), ysz);
    }
    op_delete(op);
    tensor_delete(tx);
    tensor_delete(tw);
    tensor_delete(tb);
    return 0;
}

/* ip (fully connected), uint8 path (art/modules/quant/src/op/ip.cpp:133-209).
 * x: [n][chw], wt: [k][chw], y: [n][k]. */
REF_API int ref_ip_u8(
    const uint8_t *x, int n, int chw, const uint8_t *wt, const int32_t *bias, int k, float ialpha,
    uint8_t izp, float walpha, uint8_t wzp, float oalpha, uint8_t ozp, uint8_t obits, uint8_t *y)
{
    int xd[4] = { n, chw, 1, 1 }, wd[4] = { k, chw, 1, 1 }, bd[1] = { k };
    tensor_t *tx = new_tensor(dtUINT8, 4, xd);
    tensor_t *tw = new_tensor(dtUINT8, 4, wd);
    tensor_t *tb = new_tensor(dtINT32, 1, bd);
    tensor_t *in[3] = { tx, tw, tb };
    float ia[3] = { ialpha, walpha, 1.f };
    uint8_t iz[3] = { izp, wzp, 0 }, ib[3] = { 8, 8, 32 };
    op_t *op = workspace_new_op(ws(), OP_IP, 3, in);
    if (!op)
        return -1;
    CHECK(op_setting_single_set(op, SETTING_IP_NUM_OUTPUT, dtUINT32, (uint32_t)k));
    set_in_quant(op, 3, ia, iz, ib);
    set_w_quant(op, walpha, wzp, 8);
    set_out_quant(op, oalpha, ozp, obits);
    CHECK(op_config(op));
    memcpy(mem_cpu_data(tw->mem), wt, (size_t)k * chw);
    if (bias)
        memcpy(mem_cpu_data(tb->mem), bias, sizeof(int32_t) * k);
    else
        memset(mem_cpu_data(tb->mem), 0, sizeof(int32_t) * k);
    op_prepare(op);
    memcpy(mem_cpu_data(tx->mem), x, (size_t)n * chw);
    op_run(op);
    memcpy(y, mem_cpu_data(op->output_tensors[0].mem), (size_t)n * k);
    op_delete(op);
    tensor_delete(tx);
    tensor_delete(tw);
    tensor_delete(tb);
    return 0;
}

/* eltwise SUM (eltwise.c:137-174) when use_add == 0, add (add.c:83-148) when use_add != 0.
 * xs: n_in arrays of `count` bytes; the shape is passed as [1][count][1][1]. */
REF_API int ref_eltwise_sum_u8(
    const uint8_t *const *xs, int n_in, size_t count, const float *ialpha, const uint8_t *izp,
    const float *coeff, float oalpha, uint8_t ozp, uint8_t obits, int use_add, uint8_t *y)
{
    int d[4] = { 1, (int)count, 1, 1 }, i;
    tensor_t *in[8];
    uint8_t ib[8];
    op_t *op;
    if (n_in > 8 || (use_add && n_in != 2))
        return -1;
    for (i = 0; i < n_in; ++i) {
        in[i] = new_tensor(dtUINT8, 4, d);
        memcpy(mem_cpu_data(in[i]->mem), xs[i], count);
        ib[i] = 8;
    }
    op = workspace_new_op(ws(), use_add ? OP_ADD : OP_ELTWISE, n_in, in);
    if (!op)
        return -1;
    if (!use_add) {
        CHECK(op_setting_single_set(
            op, SETTING_ELTWISE_OPERATION, dtUINT32, (uint32_t)SETTING_ELTWISE_OP_SUM));
        if (coeff)
            CHECK(op_setting_array_set(op, SETTING_ELTWISE_COEFF, dtFLOAT32, n_in, coeff));
    }
    set_in_quant(op, n_in, ialpha, izp, ib);
    set_out_quant(op, oalpha, ozp, obits);
    CHECK(op_config(op));
    op_prepare(op);
    op_run(op);
    memcpy(y, mem_cpu_data(op->output_tensors[0].mem), count);
    op_delete(op);
    for (i = 0; i < n_in; ++i)
        tensor_delete(in[i]);
    return 0;
}

/* relu (relu.c:76-115). */
REF_API int ref_relu_u8(
    const uint8_t *x, size_t count, float ialpha, uint8_t izp, float oalpha, uint8_t ozp,
    uint8_t obits, uint8_t *y)
{
    int d[4] = { 1, (int)count, 1, 1 };
    tensor_t *tx = new_tensor(dtUINT8, 4, d);
    tensor_t *in[1] = { tx };
    uint8_t ib = 8;
    op_t *op = workspace_new_op(ws(), OP_RELU, 1, in);
    if (!op)
        return -1;
    memcpy(mem_cpu_data(tx->mem), x, count);
    set_in_quant(op, 1, &ialpha, &izp, &ib);
    set_out_quant(op, oalpha, ozp, obits);
    CHECK(op_config(op));
    op_prepare(op);
    op_run(op);
    memcpy(y, mem_cpu_data(op->output_tensors[0].mem), count);
    op_delete(op);
    tensor_delete(tx);
    return 0;
}

/* pool, method 0 = MAX (pool.c:96-168), 1 = AVE (pool.c:170-249).  Output dims are written to
 * out_hw[2] as the reference's own shape inference decides them (art/src/op.c:903-967); y must
 * hold at least n*c*out_h*out_w bytes (call once with y == NULL to get the dims). */
REF_API int ref_pool_u8(
    const uint8_t *x, int n, int c, int h, int w, int method, int kernel_h, int kernel_w, int pad_h,
    int pad_w, int stride_h, int stride_w, int ceil_mode, float ialpha, uint8_t izp, float oalpha,
    uint8_t ozp, uint8_t obits, uint8_t *y, int *out_hw)
{
    int d[4] = { n, c, h, w };
    tensor_t *tx = new_tensor(dtUINT8, 4, d);
    tensor_t *in[1] = { tx };
    uint8_t ib = 8;
    op_t *op = workspace_new_op(ws(), OP_POOL, 1, in);
    if (!op)
        return -1;
    CHECK(op_setting_single_set(op, SETTING_POOL_METHOD, dtUINT32, (uint32_t)method));
    CHECK(op_setting_single_set(op, SETTING_POOL_KERNEL_H, dtUINT32, (uint32_t)kernel_h));
    CHECK(op_setting_single_set(op, SETTING_POOL_KERNEL_W, dtUINT32, (uint32_t)kernel_w));
    CHECK(op_setting_single_set(op, SETTING_POOL_PAD_H, dtUINT32, (uint32_t)pad_h));
    CHECK(op_setting_single_set(op, SETTING_POOL_PAD_W, dtUINT32, (uint32_t)pad_w));
    CHECK(op_setting_single_set(op, SETTING_POOL_STRIDE_H, dtUINT32, (uint32_t)stride_h));
    CHECK(op_setting_single_set(op, SETTING_POOL_STRIDE_W, dtUINT32, (uint32_t)stride_w));
    CHECK(op_setting_single_set(op, SETTING_POOL_CEIL_MODE, dtBOOL, (int)(ceil_mode != 0)));
    set_in_quant(op, 1, &ialpha, &izp, &ib);
    set_out_quant(op, oalpha, ozp, obits);
    CHECK(op_config(op));
    out_hw[0] = (int)op->output_tensors[0].shape.dim[2];
    out_hw[1] = (int)op->output_tensors[0].shape.dim[3];
    if (y) {
        op_prepare(op);
        memcpy(mem_cpu_data(tx->mem), x, (size_t)n * c * h * w);
        op_run(op);
        memcpy(
            y, mem_cpu_data(op->output_tensors[0].mem),
            shape_count(&op->output_tensors[0].shape));
    }
    op_delete(op);
    tensor_delete(tx);
    return 0;
}

/* quantize float32 -> uint8, qtype BIASED (quantize.c:145-157). */
REF_API int ref_quantize_u8(
    const float *x, size_t count, float oalpha, uint8_t ozp, uint8_t obits, uint8_t *y)
{
    int d[4] = { 1, (int)count, 1, 1 };
    tensor_t *tx = new_tensor(dtFLOAT32, 4, d);
    tensor_t *in[1] = { tx };
    op_t *op = workspace_new_op(ws(), OP_QUANT_QUANTIZE, 1, in);
    if (!op)
        return -1;
    memcpy(mem_cpu_data(tx->mem), x, count * sizeof(float));
    set_out_quant(op, oalpha, ozp, obits);
    CHECK(op_setting_single_set(op, SETTING_QUANT_QTYPE, dtINT32, (int32_t)SETTING_QUANT_BIASED));
    CHECK(op_config(op));
    op_prepare(op);
    op_run(op);
    memcpy(y, mem_cpu_data(op->output_tensors[0].mem), count);
    op_delete(op);
    tensor_delete(tx);
    return 0;
}

/* dequantize uint8 -> float32 (dequantize.c:111-123). */
REF_API int ref_dequantize_u8(const uint8_t *x, size_t count, float ialpha, uint8_t izp, float *y)
{
    int d[4] = { 1, (int)count, 1, 1 };
    tensor_t *tx = new_tensor(dtUINT8, 4, d);
    tensor_t *in[1] = { tx };
    uint8_t ib = 8;
    op_t *op = workspace_new_op(ws(), OP_QUANT_DEQUANTIZE, 1, in);
    if (!op)
        return -1;
    memcpy(mem_cpu_data(tx->mem), x, count);
    set_in_quant(op, 1, &ialpha, &izp, &ib);
    CHECK(op_setting_single_set(op, SETTING_QUANT_QTYPE, dtINT32, (int32_t)SETTING_QUANT_BIASED));
    CHECK(op_config(op));
    op_prepare(op);
    op_run(op);
    memcpy(y, mem_cpu_data(op->output_tensors[0].mem), count * sizeof(float));
    op_delete(op);
    tensor_delete(tx);
    return 0;
}

/* ------------------------------------------------------------------------------------------
 * The int8 (dtINT8, symmetric) path: conv_2d (conv_2d_int8_impl.c:34-174), ip (ip.cpp:210-274),
 * quantize with qtype SYMMETRIC (quantize.c:159-185), dequantize (dequantize.c:124-136).
 * Zero points are not read on this path; ibits = wbits = 8 selects gemm_i8xi8 (conv_2d.c:120-142).
 * The conv sizes its int32 scratch for one image (conv_2d_int8_impl.c:22-31): one image per run.
 * ------------------------------------------------------------------------------------------ */
REF_API int ref_conv2d_i8(
    const int8_t *x, int n, int c, int h, int w, const int8_t *wt, const int32_t *bias, int k, int r,
    int s, int pad_h, int pad_w, int stride_h, int stride_w, int group, float ialpha, float walpha,
    float oalpha, uint8_t obits, int8_t *y)
{
    int per_run = g_whole_batch ? n : 1;
    int xd[4] = { per_run, c, h, w }, wd[4] = { k, c / group, r, s }, bd[1] = { k };
    tensor_t *tx = new_tensor(dtINT8, 4, xd);
    tensor_t *tw = new_tensor(dtINT8, 4, wd);
    tensor_t *tb = new_tensor(dtINT32, 1, bd);
    tensor_t *in[3] = { tx, tw, tb };
    float ia[3] = { ialpha, walpha, 1.f };
    uint8_t iz[3] = { 0, 0, 0 }, ib[3] = { 8, 8, 32 };
    size_t xsz = (size_t)per_run * c * h * w, ysz;
    int i;
    op_t *op;
    memcpy(mem_cpu_data(tw->mem), wt, (size_t)k * (c / group) * r * s);
    if (bias)
        memcpy(mem_cpu_data(tb->mem), bias, sizeof(int32_t) * k);
    else
        memset(mem_cpu_data(tb->mem), 0, sizeof(int32_t) * k);
    op = workspace_new_op(ws(), OP_CONV_2D, 3, in);
    if (!op)
        return -1;
    CHECK(op_setting_single_set(op, SETTING_CONV_2D_NUM_OUTPUT, dtUINT32, (uint32_t)k));
    CHECK(op_setting_single_set(op, SETTING_CONV_2D_KERNEL_H, dtUINT32, (uint32_t)r));
    CHECK(op_setting_single_set(op, SETTING_CONV_2D_KERNEL_W, dtUINT32, (uint32_t)s));
    CHECK(op_setting_single_set(op, SETTING_CONV_2D_PAD_H, dtUINT32, (uint32_t)pad_h));
    CHECK(op_setting_single_set(op, SETTING_CONV_2D_PAD_W, dtUINT32, (uint32_t)pad_w));
    CHECK(op_setting_single_set(op, SETTING_CONV_2D_STRIDE_H, dtUINT32, (uint32_t)stride_h));
    CHECK(op_setting_single_set(op, SETTING_CONV_2D_STRIDE_W, dtUINT32, (uint32_t)stride_w));
    CHECK(op_setting_single_set(op, SETTING_CONV_2D_GROUP, dtUINT32, (uint32_t)group));
    set_in_quant(op, 3, ia, iz, ib);
    set_w_quant(op, walpha, 0, 8);
    set_out_quant(op, oalpha, 0, obits);
    CHECK(op_config(op));
    op_prepare(op);
    ysz = shape_count(&op->output_tensors[0].shape);
    for (i = 0; i < n; i += per_run) {
        memcpy(mem_cpu_data(tx->mem), x + xsz * (i / per_run), xsz);
        op_run(op);
        memcpy(y + ysz * (i / per_run), mem_cpu_data(op->output_tensors[0].mem), ysz);
    }
    op_delete(op);
    tensor_delete(tx);
    tensor_delete(tw);
    tensor_delete(tb);
    return 0;
}

REF_API int ref_ip_i8(
    const int8_t *x, int n, int chw, const int8_t *wt, const int32_t *bias, int k, float ialpha,
    float walpha, float oalpha, uint8_t obits, int8_t *y)
{
    int xd[4] = { n, chw, 1, 1 }, wd[4] = { k, chw, 1, 1 }, bd[1] = { k };
    tensor_t *tx = new_tensor(dtINT8, 4, xd);
    tensor_t *tw = new_tensor(dtINT8, 4, wd);
    tensor_t *tb = new_tensor(dtINT32, 1, bd);
    tensor_t *in[3] = { tx, tw, tb };
    float ia[3] = { ialpha, walpha, 1.f };
    uint8_t iz[3] = { 0, 0, 0 }, ib[3] = { 8, 8, 32 };
    op_t *op = workspace_new_op(ws(), OP_IP, 3, in);
    if (!op)
        return -1;
    CHECK(op_setting_single_set(op, SETTING_IP_NUM_OUTPUT, dtUINT32, (uint32_t)k));
    set_in_quant(op, 3, ia, iz, ib);
    set_w_quant(op, walpha, 0, 8);
    set_out_quant(op, oalpha, 0, obits);
    CHECK(op_config(op));
    memcpy(mem_cpu_data(tw->mem), wt, (size_t)k * chw);
    if (bias)
        memcpy(mem_cpu_data(tb->mem), bias, sizeof(int32_t) * k);
    else
        memset(mem_cpu_data(tb->mem), 0, sizeof(int32_t) * k);
    op_prepare(op);
    memcpy(mem_cpu_data(tx->mem), x, (size_t)n * chw);
    op_run(op);
    memcpy(y, mem_cpu_data(op->output_tensors[0].mem), (size_t)n * k);
    op_delete(op);
    tensor_delete(tx);
    tensor_delete(tw);
    tensor_delete(tb);
    return 0;
}

REF_API int ref_quantize_i8(const float *x, size_t count, float oalpha, uint8_t obits, int8_t *y)
{
    int d[4] = { 1, (int)count, 1, 1 };
    tensor_t *tx = new_tensor(dtFLOAT32, 4, d);
    tensor_t *in[1] = { tx };
    op_t *op = workspace_new_op(ws(), OP_QUANT_QUANTIZE, 1, in);
    if (!op)
        return -1;
    memcpy(mem_cpu_data(tx->mem), x, count * sizeof(float));
    set_out_quant(op, oalpha, 0, obits);
    CHECK(op_setting_single_set(op, SETTING_QUANT_QTYPE, dtINT32, (int32_t)SETTING_QUANT_SYMMETRIC));
    CHECK(op_config(op));
    if (op->output_tensors[0].dtype != dtINT8)
        return -2;
    op_prepare(op);
    op_run(op);
    memcpy(y, mem_cpu_data(op->output_tensors[0].mem), count);
    op_delete(op);
    tensor_delete(tx);
    return 0;
}

REF_API int ref_dequantize_i8(const int8_t *x, size_t count, float ialpha, uint8_t ibits, float *y)
{
    int d[4] = { 1, (int)count, 1, 1 };
    tensor_t *tx = new_tensor(dtINT8, 4, d);
    tensor_t *in[1] = { tx };
    uint8_t iz = 0;
    op_t *op = workspace_new_op(ws(), OP_QUANT_DEQUANTIZE, 1, in);
    if (!op)
        return -1;
    memcpy(mem_cpu_data(tx->mem), x, count);
    set_in_quant(op, 1, &ialpha, &iz, &ibits);
    CHECK(op_setting_single_set(op, SETTING_QUANT_QTYPE, dtINT32, (int32_t)SETTING_QUANT_SYMMETRIC));
    CHECK(op_config(op));
    op_prepare(op);
    op_run(op);
    memcpy(y, mem_cpu_data(op->output_tensors[0].mem), count * sizeof(float));
    op_delete(op);
    tensor_delete(tx);
    return 0;
}

/* ------------------------------------------------------------------------------------------
 * A serialized case (engine.bin, format v2: art/src/serialize_v2.c:26-103) through the
 * reference's own loader and parade, the way its drivers do it (tools/promark.cpp:58-72):
 * deserialize_parade with the current module's workspace, parade_prepare, then per run copy the
 * inputs in, parade_run, copy the outputs out (art/src/parade.c:184-197).
 * With the reference `quant` module the conv scratch of every conv op is cleared once after
 * prepare, and the batch must be 1 (see the constraints at the top of this file).
 * ------------------------------------------------------------------------------------------ */
#include <stdio.h>

#include "art/parade.h"
#include "art/serialize.h"
#include "src/parade_impl.h"   /* art/src: the parade struct, for the op list */

static size_t read_file_chunk(size_t sz, void *data, void *param)
{
    return fread(data, 1, sz, (FILE *)param);
}

REF_API parade_t *ref_parade_open(const char *path)
{
    FILE *fp = fopen(path, "rb");
    buffer_t *buf;
    parade_t *parade;
    workspace_t *wss[2];
    deserialize_param_t params;
    size_t i;
    if (!fp)
        return NULL;
    buf = nart_buffer_new(0x8000);
    buffer_set_buffer_read_func(buf, read_file_chunk, (void *)fp);
    wss[0] = ws();
    wss[1] = NULL;
    params.workspaces = wss;
    params.input_mem_tp = workspace_memtype(ws());
    parade = deserialize_parade(buf, &params);
    nart_buffer_delete(buf);
    fclose(fp);
    if (!parade)
        return NULL;
    parade_prepare(parade);
    if (g_module == &quant_module_tp) {
        for (i = 0; i < parade->op_count; ++i) {
            op_t *op = parade->ops[i];
            if (op->entry->tp->op_tp_code == OP_CONV_2D) {
                op_conv_2d_t *conv_op = (op_conv_2d_t *)op;
                if (conv_op->temp_data)
                    memset(mem_cpu_data(conv_op->temp_data), 0, mem_sizeof(conv_op->temp_data));
            }
        }
    }
    return parade;
}

/* Byte size of input / output `index` of the loaded case (whole batch). */
REF_API size_t ref_parade_io_bytes(parade_t *parade, int is_output, int index)
{
    size_t count = 0;
    tensor_array_t arr = NULL;
    if (is_output)
        parade_get_output_tensors(parade, &count, &arr);
    else
        parade_get_input_tensors(parade, &count, &arr);
    if (index < 0 || (size_t)index >= count)
        return 0;
    return shape_count(&arr[index]->shape) * datatype_sizeof(arr[index]->dtype);
}

/* One run: inputs[i] / outputs[i] are host arrays of ref_parade_io_bytes bytes. */
REF_API int ref_parade_run(parade_t *parade, const void *const *inputs, void *const *outputs)
{
    size_t n_in = 0, n_out = 0, i;
    tensor_array_t in = NULL, out = NULL;
    parade_get_input_tensors(parade, &n_in, &in);
    parade_get_output_tensors(parade, &n_out, &out);
    for (i = 0; i < n_in; ++i)
        memcpy(mem_cpu_data(in[i]->mem), inputs[i], shape_count(&in[i]->shape) * datatype_sizeof(in[i]->dtype));
    parade_run(parade);
    for (i = 0; i < n_out; ++i)
        memcpy(outputs[i], mem_cpu_data(out[i]->mem), shape_count(&out[i]->shape) * datatype_sizeof(out[i]->dtype));
    return 0;
}

/* The three steps of ref_parade_run on their own, for a driver that keeps its data in the tensors' host
 * views the way the reference's promark does (tools/promark.cpp:457-492): the host view of an input
 * (asking for it makes the host copy the current one, so the next run uploads it), parade_run, and the
 * host view of an output (which downloads it). */
REF_API void *ref_parade_input_ptr(parade_t *parade, int index)
{
    size_t count = 0;
    tensor_array_t arr = NULL;
    parade_get_input_tensors(parade, &count, &arr);
    return index >= 0 && (size_t)index < count ? mem_cpu_data(arr[index]->mem) : NULL;
}

REF_API void ref_parade_run_only(parade_t *parade) { parade_run(parade); }

REF_API void *ref_parade_output_ptr(parade_t *parade, int index)
{
    size_t count = 0;
    tensor_array_t arr = NULL;
    parade_get_output_tensors(parade, &count, &arr);
    return index >= 0 && (size_t)index < count ? mem_cpu_data(arr[index]->mem) : NULL;
}

REF_API void ref_parade_close(parade_t *parade)
{
    if (parade)
        parade_delete(parade);
}

/* Numeric value of a named constant of the reference's headers, for pinning the tables of the
 * engine writer; returns 0 and sets *found = 0 for an unknown name. */
REF_API uint64_t ref_constant(const char *name, int *found)
{
#define REF_CONST(x)             \
    if (strcmp(name, #x) == 0) { \
        *found = 1;              \
        return (uint64_t)(x);    \
    }
    REF_CONST(OP_CONV_2D) REF_CONST(OP_IP) REF_CONST(OP_ELTWISE) REF_CONST(OP_ADD) REF_CONST(OP_RELU)
    REF_CONST(OP_POOL) REF_CONST(OP_QUANT_QUANTIZE) REF_CONST(OP_QUANT_DEQUANTIZE)
    REF_CONST(SETTING_CONV_2D_RELU_FLAG) REF_CONST(SETTING_CONV_2D_NUM_OUTPUT) REF_CONST(SETTING_CONV_2D_KERNEL_H)
    REF_CONST(SETTING_CONV_2D_KERNEL_W) REF_CONST(SETTING_CONV_2D_PAD_H) REF_CONST(SETTING_CONV_2D_PAD_W)
    REF_CONST(SETTING_CONV_2D_STRIDE_H) REF_CONST(SETTING_CONV_2D_STRIDE_W) REF_CONST(SETTING_CONV_2D_GROUP)
    REF_CONST(SETTING_IP_NUM_OUTPUT) REF_CONST(SETTING_ELTWISE_OPERATION) REF_CONST(SETTING_ELTWISE_OP_SUM)
    REF_CONST(SETTING_ELTWISE_COEFF) REF_CONST(SETTING_POOL_METHOD) REF_CONST(SETTING_POOL_KERNEL_H)
    REF_CONST(SETTING_POOL_KERNEL_W) REF_CONST(SETTING_POOL_PAD_H) REF_CONST(SETTING_POOL_PAD_W)
    REF_CONST(SETTING_POOL_STRIDE_H) REF_CONST(SETTING_POOL_STRIDE_W) REF_CONST(SETTING_POOL_CEIL_MODE)
    REF_CONST(SETTING_POOL_MAX) REF_CONST(SETTING_POOL_AVE)
    REF_CONST(SETTING_QUANT_IALPHA) REF_CONST(SETTING_QUANT_IZERO_POINT) REF_CONST(SETTING_QUANT_IBITS)
    REF_CONST(SETTING_QUANT_OALPHA) REF_CONST(SETTING_QUANT_OZERO_POINT) REF_CONST(SETTING_QUANT_OBITS)
    REF_CONST(SETTING_QUANT_WALPHA) REF_CONST(SETTING_QUANT_WZERO_POINT) REF_CONST(SETTING_QUANT_WBITS)
    REF_CONST(SETTING_QUANT_QTYPE) REF_CONST(SETTING_QUANT_BIASED)
    REF_CONST(dtUINT8) REF_CONST(dtINT8) REF_CONST(dtUINT32) REF_CONST(dtINT32) REF_CONST(dtFLOAT32)
    REF_CONST(dtBOOL) REF_CONST(dtSTR)
#undef REF_CONST
    *found = 0;
    return 0;
}
