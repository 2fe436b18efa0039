/*
 * libart_module_b200.so -- the art-facing plugin of the Blackwell quantized-convolution backend.
 *
 * It exports one `const module_t b200_module_tp`, the symbol the reference's drivers look up as
 * "<name>_module_tp" in "libart_module_<name>.so" (tools/promark.cpp:122-134,152-154,
 * python/src/art/module.cpp:46-68 of ModelTC/NART), with `.op_group = OP_GROUP_CODE_QUANT` so that
 * a case exported for the reference `quant` module binds to these ops unchanged
 * (art/src/serialize_v2.c:111-128, art/src/module.c:53-75).  Ops: quantize, dequantize, conv_2d,
 * ip, relu, add, eltwise, pool -- the uint8 subset of art/modules/quant/src/quant_module.c:49-66 --
 * reading the same settings (SETTING_QUANT_*, art/modules/quant/include/art/quant/
 * quant_op_settings.h:26-40) and following the same lifecycle (alloc, config, prepare, run,
 * destroy, dealloc; art/include/art/op.h:114-143, art/src/op.c:39-77).
 *
 * This file is host-side C in the runtime's own idiom.  It contains no CUDA: everything on the
 * device goes through the C-ABI of libnart_b200.so (include/nart_b200.h).  Errors follow the
 * reference's convention: a failed C-ABI call is reported with LOG_error, which exits
 * (art/include/art/log.h:29-34).
 *
 * Layout.  Like the reference's GPU quant module, device tensors are NHWC under NCHW shapes
 * (python/nart/modules/cuda_quant.py:182-186).  Unlike it, the host never sees that: the mem type
 * below records which layout its device copy is in, and mem_cpu_data() always returns the
 * reference quant module's NCHW bytes.
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "art/log.h"
#include "art/mem.h"
#include "art/module.h"
#include "art/op.h"
#include "art/op_settings.h"
#include "art/op_tp.h"
#include "art/quant/quant_op_settings.h"
#include "art/quant/quant_op_tp.h"

#include "nart_b200.h"

#define B200_CALL(expr)                                                                       \
    do {                                                                                      \
        int _s = (expr);                                                                      \
        if (_s != B200_OK)                                                                    \
            LOG_error("b200: %s failed: %s (%s)\n", #expr, b200_strerror(_s), b200_last_error()); \
    } while (0)

/* ------------------------------------------------------------------------------------------
 * mem type: device buffer + host mirror, the contract of art/include/art/mem.h:48-64 as the
 * reference's device modules implement it (art/modules/cuda_quant/src/cuda_quant_mem.cpp:25-123):
 * data() uploads when the host copy is newer, cpu_data() downloads when the device copy is newer
 * and makes the host copy the current one again.
 * ------------------------------------------------------------------------------------------ */
typedef struct b200_mem_t {
    mem_t m;
    size_t sz;
    void *dev;
    void *host;         /* pinned mirror, allocated the first time the host asks for the data */
    size_t host_sz;
    void *nchw_tmp;     /* device staging for cpu_data() of an NHWC tensor, kept between calls */
    size_t nchw_tmp_sz;
    bool gpu_updated;   /* the device copy is the current one */
    bool upload_pending; /* an upload from the host mirror may still be reading it (see b200_mem_data) */
    bool host_current;  /* the host mirror holds what the device copy holds (set by an upload or a download, cleared
                         * when an op writes the device copy): b200_mem_cpu_data then has nothing to fetch */
    bool nhwc;          /* the device copy is NHWC uint8 with the dims below (set by the op that wrote it) */
    int n, c, h, w;
} b200_mem_t;

static mem_t *b200_mem_new(void)
{
    b200_mem_t *res = (b200_mem_t *)malloc(sizeof(b200_mem_t));
    memset(res, 0, sizeof(*res));
    return (mem_t *)res;
}

static void b200_mem_free(b200_mem_t *m)
{
    if (m->sz > 0) {
        B200_CALL(b200_free(m->dev));
        m->dev = NULL;
        m->sz = 0;
    }
    if (m->host)
        B200_CALL(b200_free_host(m->host));
    if (m->nchw_tmp)
        B200_CALL(b200_free(m->nchw_tmp));
    m->host = NULL;
    m->host_sz = 0;
    m->nchw_tmp = NULL;
    m->nchw_tmp_sz = 0;
}

static void b200_mem_delete(b200_mem_t *m)
{
    b200_mem_free(m);
    free(m);
}

/* grow-only, like the reference (art/modules/cuda_quant/src/cuda_quant_mem.cpp:49-64) */
static bool b200_mem_alloc(b200_mem_t *m, size_t sz)
{
    if (m->sz >= sz)
        return true;
    if (m->sz > 0)
        B200_CALL(b200_free(m->dev));
    /* 256 spare bytes: vector loads of a ragged last pixel may read past the tensor */
    B200_CALL(b200_malloc(&m->dev, sz + 256));
    B200_CALL(b200_memset(m->dev, 0, sz + 256, NULL));
    m->sz = sz;
    m->gpu_updated = false;
    m->nhwc = false;
    return true;
}

/* The host mirror exists only for tensors the host touches (case inputs and outputs, weights): it is
 * pinned, so that the copies of b200_mem_data / b200_mem_cpu_data run at full PCIe speed, and sized on
 * first use.  Intermediate tensors of a parade never get one. */
static void host_mirror(b200_mem_t *m)
{
    if (m->host_sz >= m->sz && m->host)
        return;
    void *fresh = NULL;
    B200_CALL(b200_malloc_host(&fresh, m->sz));
    CHECK_NE(NULL, fresh);
    if (m->host) {
        memcpy(fresh, m->host, m->host_sz);
        B200_CALL(b200_free_host(m->host));
    }
    if (m->sz > m->host_sz)
        memset((char *)fresh + m->host_sz, 0, m->sz - m->host_sz);
    m->host = fresh;
    m->host_sz = m->sz;
}

static void *b200_mem_data(b200_mem_t *m)
{
    if (!m->gpu_updated && m->host) {
        /* Asynchronous, from the pinned mirror, on the stream every op of this module runs on: the ops that
         * follow are queued while the copy is under way instead of after it.  The host gets at the mirror
         * only through b200_mem_cpu_data, which waits for a pending upload before it hands the pointer out. */
        B200_CALL(b200_memcpy_h2d(m->dev, m->host, m->sz, NULL));
        m->upload_pending = true;
        m->gpu_updated = true;
        m->host_current = true;
        m->nhwc = false;   /* what the host wrote is in the reference's layout */
    }
    return m->dev;
}

static void *b200_mem_cpu_data(b200_mem_t *m)
{
    if (m->upload_pending) {
        B200_CALL(b200_stream_synchronize(NULL));
        m->upload_pending = false;
    }
    host_mirror(m);
    if (m->gpu_updated && m->host_current) {
        /* the device copy came from this very mirror and nothing has written it since */
        m->gpu_updated = false;
    }
    if (m->gpu_updated) {
        size_t count = (size_t)m->n * m->c * m->h * m->w;
        if (m->nhwc && count <= m->sz && m->c > 1 && m->h * m->w > 1) {
            /* bring the device copy back to the reference's NCHW before the host reads it */
            if (m->nchw_tmp_sz < count) {
                if (m->nchw_tmp)
                    B200_CALL(b200_free(m->nchw_tmp));
                B200_CALL(b200_malloc(&m->nchw_tmp, count));
                m->nchw_tmp_sz = count;
            }
            void *tmp = m->nchw_tmp;
            B200_CALL(b200_nhwc_to_nchw_u8(m->dev, tmp, m->n, m->c, m->h, m->w, m->c, NULL));
            B200_CALL(b200_memcpy_d2h(m->host, tmp, count, NULL));
            B200_CALL(b200_stream_synchronize(NULL));
        } else {
            B200_CALL(b200_memcpy_d2h(m->host, m->dev, m->sz, NULL));
            B200_CALL(b200_stream_synchronize(NULL));
        }
        m->gpu_updated = false;
        m->host_current = true;
    }
    return m->host;
}

static size_t b200_mem_size(b200_mem_t *m) { return m->sz; }

static void *b200_mem_cpy_to_cpu(void *dst, const void *from, size_t sz)
{
    B200_CALL(b200_memcpy_d2h(dst, from, sz, NULL));
    B200_CALL(b200_stream_synchronize(NULL));
    return dst;
}

static void *b200_mem_cpy_from_cpu(void *dst, const void *from, size_t sz)
{
    B200_CALL(b200_memcpy_h2d(dst, from, sz, NULL));
    B200_CALL(b200_stream_synchronize(NULL));
    return dst;
}

static const mem_tp b200_mem_tp_st = {
    .name = "b200_mem",
    .new_func = b200_mem_new,
    .delete_func = (mem_func_delete)b200_mem_delete,
    .alloc_func = (mem_func_alloc)b200_mem_alloc,
    .free_func = (mem_func_free)b200_mem_free,
    .data_func = (mem_func_data)b200_mem_data,
    .cpu_data_func = (mem_func_data)b200_mem_cpu_data,
    .size_func = (mem_func_size)b200_mem_size,
    .copy_from_cpu_func = b200_mem_cpy_from_cpu,
    .copy_to_cpu_func = b200_mem_cpy_to_cpu,
    .share_from_func = NULL,
};
DLL_PUBLIC const mem_tp *const b200_mem_tp = &b200_mem_tp_st;

/* ------------------------------------------------------------------------------------------
 * helpers shared by the ops
 * ------------------------------------------------------------------------------------------ */
typedef struct {
    void *buf;
    size_t sz;
} scratch_t;

static void scratch_reserve(scratch_t *s, size_t sz)
{
    if (s->sz >= sz)
        return;
    if (s->buf)
        B200_CALL(b200_free(s->buf));
    B200_CALL(b200_malloc(&s->buf, sz + 256));
    s->sz = sz;
}

static void scratch_release(scratch_t *s)
{
    if (s->buf)
        B200_CALL(b200_free(s->buf));
    s->buf = NULL;
    s->sz = 0;
}

static void dims_of(const tensor_t *t, int *n, int *c, int *h, int *w)
{
    /* NCHW shape metadata; fewer than four dims are padded with 1 */
    const shape_t *s = &t->shape;
    *n = s->dim_size > 0 ? (int)s->dim[0] : 1;
    *c = s->dim_size > 1 ? (int)s->dim[1] : 1;
    *h = s->dim_size > 2 ? (int)s->dim[2] : 1;
    *w = s->dim_size > 3 ? (int)s->dim[3] : 1;
}

/* Device pointer to a uint8 input in NHWC.  Tensors written by this module's ops already are;
 * tensors the host (or another module) wrote are in the reference's NCHW and are transposed into
 * `scratch` first.  Foreign mem types are uploaded from their host view. */
static const uint8_t *input_nhwc_padded(tensor_t *t, scratch_t *scratch, int c_pad, uint8_t fill)
{
    int n, c, h, w;
    dims_of(t, &n, &c, &h, &w);
    if (c_pad < c)
        c_pad = c;
    size_t count = (size_t)n * c * h * w, padded = (size_t)n * c_pad * h * w;
    if (t->mem->tp != b200_mem_tp) {
        scratch_reserve(scratch, padded + count);
        uint8_t *stage = (uint8_t *)scratch->buf + padded;
        B200_CALL(b200_memcpy_h2d(stage, mem_cpu_data(t->mem), count, NULL));
        if (c_pad == c && (c == 1 || h * w == 1))
            return stage;
        B200_CALL(b200_nchw_to_nhwc_u8(stage, (uint8_t *)scratch->buf, n, c, h, w, c_pad, fill, NULL));
        return (const uint8_t *)scratch->buf;
    }
    b200_mem_t *m = (b200_mem_t *)t->mem;
    const uint8_t *dev = (const uint8_t *)mem_data(t->mem);
    if (c_pad == c && (m->nhwc || c == 1 || h * w == 1))
        return dev;
    if (m->nhwc) {
        /* an NHWC tensor of this module (a quantize op ahead of the first conv) that needs more channels:
         * back to NCHW, then out again with the padding; image-sized, once per run */
        scratch_reserve(scratch, padded + count);
        uint8_t *stage = (uint8_t *)scratch->buf + padded;
        B200_CALL(b200_nhwc_to_nchw_u8(dev, stage, n, c, h, w, c, NULL));
        B200_CALL(b200_nchw_to_nhwc_u8(stage, (uint8_t *)scratch->buf, n, c, h, w, c_pad, fill, NULL));
        return (const uint8_t *)scratch->buf;
    }
    scratch_reserve(scratch, padded);
    B200_CALL(b200_nchw_to_nhwc_u8(dev, (uint8_t *)scratch->buf, n, c, h, w, c_pad, fill, NULL));
    return (const uint8_t *)scratch->buf;
}

static const uint8_t *input_nhwc(tensor_t *t, scratch_t *scratch) { return input_nhwc_padded(t, scratch, 0, 0); }

/* Device pointer of an output tensor; tags its mem as freshly written on the device. */
static void *output_dev(tensor_t *t, bool nhwc)
{
    CHECK(t->mem->tp == b200_mem_tp);
    b200_mem_t *m = (b200_mem_t *)t->mem;
    dims_of(t, &m->n, &m->c, &m->h, &m->w);
    m->nhwc = nhwc;
    m->gpu_updated = true;
    m->host_current = false;
    return m->dev;
}

/* The int8 path of the reference clips 8-bit outputs at +-255 and then wraps them into int8
 * (quant_helper.h:43-47).  That is reproduced only when NART_B200_S8_WRAP=1 is set in the environment;
 * otherwise an int8 conv_2d / ip with obits = 8 is refused with the library's explanation. */
static int s8_wrap_allowed(void)
{
    const char *e = getenv("NART_B200_S8_WRAP");
    return e && atoi(e) != 0;
}

static void alloc_io(op_t *op)
{
    size_t i;
    for (i = 0; i < op->input_size; ++i)
        tensor_alloc(op->input_tensors[i]);
    for (i = 0; i < op->output_size; ++i)
        tensor_alloc(&op->output_tensors[i]);
}

/* the quantization settings every quant op carries */
typedef struct {
    float *ialpha, *walpha, *oalpha;
    uint8_t *izp, *wzp, *ozp;
    uint8_t *ibits, *wbits, *obits;
    size_t n_walpha;   /* entries of SETTING_QUANT_WALPHA */
} qsettings_t;

static void get_in_q(op_t *op, qsettings_t *q)
{
    size_t len;
    CHECK(op_setting_array_get(op, SETTING_QUANT_IALPHA, dtFLOAT32, &len, &q->ialpha));
    CHECK(op_setting_array_get(op, SETTING_QUANT_IZERO_POINT, dtUINT8, &len, &q->izp));
    CHECK(op_setting_array_get(op, SETTING_QUANT_IBITS, dtUINT8, &len, &q->ibits));
}

static void get_w_q(op_t *op, qsettings_t *q)
{
    size_t len;
    CHECK(op_setting_array_get(op, SETTING_QUANT_WALPHA, dtFLOAT32, &len, &q->walpha));
    q->n_walpha = len;
    CHECK(op_setting_array_get(op, SETTING_QUANT_WZERO_POINT, dtUINT8, &len, &q->wzp));
    CHECK(op_setting_array_get(op, SETTING_QUANT_WBITS, dtUINT8, &len, &q->wbits));
}

static void get_out_q(op_t *op, qsettings_t *q)
{
    size_t len;
    CHECK(op_setting_array_get(op, SETTING_QUANT_OALPHA, dtFLOAT32, &len, &q->oalpha));
    CHECK(op_setting_array_get(op, SETTING_QUANT_OZERO_POINT, dtUINT8, &len, &q->ozp));
    CHECK(op_setting_array_get(op, SETTING_QUANT_OBITS, dtUINT8, &len, &q->obits));
}

/* ------------------------------------------------------------------------------------------
 * conv_2d  (art/modules/quant/src/op/conv_2d.c:19-147, conv_2d_uint8_impl.c:39-165)
 * ------------------------------------------------------------------------------------------ */
typedef struct {
    op_t o;
    uint32_t num_output, pad_h, pad_w, kernel_h, kernel_w, stride_h, stride_w, group;
    bool relu_flag;
    qsettings_t q;
    b200_conv_t *plan;
    int plan_c, plan_h, plan_w;
    int c_pad;              /* channels the plan was built for: 4 for an image of fewer channels, else c */
    scratch_t in_scratch;
} op_b200_conv_2d_t;

op_t *op_b200_conv_2d_tp_alloc(workspace_t *ws)
{
    (void)ws;
    op_b200_conv_2d_t *res = (op_b200_conv_2d_t *)malloc(sizeof(*res));
    memset(res, 0, sizeof(*res));
    return (op_t *)res;
}

void op_b200_conv_2d_tp_config(op_t *op)
{
    op_b200_conv_2d_t *c = (op_b200_conv_2d_t *)op;
    CHECK(op_setting_single_get(op, SETTING_CONV_2D_NUM_OUTPUT, dtUINT32, &c->num_output));
    CHECK(op_setting_single_get(op, SETTING_CONV_2D_KERNEL_H, dtUINT32, &c->kernel_h));
    CHECK(op_setting_single_get(op, SETTING_CONV_2D_KERNEL_W, dtUINT32, &c->kernel_w));
    CHECK(op_setting_single_get(op, SETTING_CONV_2D_PAD_H, dtUINT32, &c->pad_h));
    CHECK(op_setting_single_get(op, SETTING_CONV_2D_PAD_W, dtUINT32, &c->pad_w));
    CHECK(op_setting_single_get(op, SETTING_CONV_2D_STRIDE_H, dtUINT32, &c->stride_h));
    CHECK(op_setting_single_get(op, SETTING_CONV_2D_STRIDE_W, dtUINT32, &c->stride_w));
    CHECK(op_setting_single_get(op, SETTING_CONV_2D_GROUP, dtUINT32, &c->group));
    /* the CPU quant module never reads this flag (art/modules/quant/src/op/conv_2d.c:27-70); the
     * GPU quant module fuses on it (art/modules/cuda_quant/src/op/conv_2d_quant.cu:793-794) */
    CHECK(op_setting_single_get(op, SETTING_CONV_2D_RELU_FLAG, dtBOOL, &c->relu_flag));
    {
        /* the quant module's conv has no dilation (conv_2d.c:27-70 never reads HOLE_*) */
        uint32_t hole_h = 1, hole_w = 1;
        CHECK(op_setting_single_get(op, SETTING_CONV_2D_HOLE_H, dtUINT32, &hole_h));
        CHECK(op_setting_single_get(op, SETTING_CONV_2D_HOLE_W, dtUINT32, &hole_w));
        if (hole_h != 1 || hole_w != 1)
            LOG_error("b200: dilated conv_2d is not built\n");
    }
    get_in_q(op, &c->q);
    get_w_q(op, &c->q);
    get_out_q(op, &c->q);
}

static void conv_release_plan(op_b200_conv_2d_t *c)
{
    if (c->plan) {
        B200_CALL(b200_conv2d_destroy(c->plan));
        c->plan = NULL;
    }
}

void op_b200_conv_2d_tp_destroy(op_t *op)
{
    op_b200_conv_2d_t *c = (op_b200_conv_2d_t *)op;
    conv_release_plan(c);
    scratch_release(&c->in_scratch);
}

void op_b200_conv_2d_tp_dealloc(op_t *op)
{
    if (NULL != op)
        free(op);
}

static void op_b200_conv_2d_run(op_t *op)
{
    op_b200_conv_2d_t *c = (op_b200_conv_2d_t *)op;
    int n, ch, h, w;
    dims_of(op->input_tensors[0], &n, &ch, &h, &w);
    const uint8_t *x = input_nhwc_padded(op->input_tensors[0], &c->in_scratch, c->c_pad, c->q.izp[0]);
    uint8_t *y = (uint8_t *)output_dev(&op->output_tensors[0], true);
    B200_CALL(b200_conv2d_run(c->plan, x, n, y, NULL));
}

void op_b200_conv_2d_tp_prepare(op_t *op)
{
    op_b200_conv_2d_t *c = (op_b200_conv_2d_t *)op;
    int n, ch, h, w;
    alloc_io(op);
    /* dispatch on the dtype of input 0, as the reference does (conv_2d.c:114-142) */
    if (op->input_tensors[0]->dtype != dtUINT8 && op->input_tensors[0]->dtype != dtINT8)
        LOG_error("b200: conv_2d takes uint8 or int8 activations\n");
    dims_of(op->input_tensors[0], &n, &ch, &h, &w);
    /* prepare runs again after a reshape (art/src/parade.c:199-215): rebuild only if the geometry changed */
    if (c->plan && c->plan_c == ch && c->plan_h == h && c->plan_w == w) {
        op->run_func = op_b200_conv_2d_run;
        return;
    }
    conv_release_plan(c);
    b200_conv_params p;
    memset(&p, 0, sizeof(p));
    p.c = ch; p.h = h; p.w = w;
    p.k = (int32_t)c->num_output; p.r = (int32_t)c->kernel_h; p.s = (int32_t)c->kernel_w;
    p.pad_h = (int32_t)c->pad_h; p.pad_w = (int32_t)c->pad_w;
    p.stride_h = (int32_t)c->stride_h; p.stride_w = (int32_t)c->stride_w; p.group = (int32_t)c->group;
    p.ialpha = c->q.ialpha[0]; p.izp = c->q.izp[0];
    p.wzp = c->q.wzp[0];
    p.oalpha = c->q.oalpha[0]; p.ozp = c->q.ozp[0]; p.obits = c->q.obits[0];
    p.walpha = c->q.walpha;
    /* The reference reads walpha[0] only (conv_2d_uint8_impl.c:61) and its exporter writes one entry
     * per weight tensor.  An array with one entry per output channel is taken as per-channel scales
     * (an extension; no file the reference writes has one). */
    p.n_walpha = (c->q.n_walpha == (size_t)c->num_output && c->num_output > 1) ? (int32_t)c->num_output : 1;
    p.relu = c->relu_flag ? 1 : 0;
    p.algo = B200_CONV_ALGO_AUTO;
    if (op->input_tensors[0]->dtype == dtINT8) {
        p.act_type = B200_ACT_S8;
        p.s8_wrap = s8_wrap_allowed();
    }
    const uint8_t *wt = (const uint8_t *)mem_cpu_data(op->input_tensors[1]->mem);
    const int32_t *bias = op->input_size == 3 ? (const int32_t *)mem_cpu_data(op->input_tensors[2]->mem) : NULL;
    /* An image of fewer than four channels (the network's first conv) is padded to four on its way to
     * NHWC, with weights equal to the zero point -- i.e. zero -- on the added channel: four channels are
     * what the library's row-lowered tensor-core path for image stems takes. */
    uint8_t *wpad = NULL;
    c->c_pad = ch;
    if (ch < 4 && p.group == 1 && p.act_type == B200_ACT_U8) {
        const size_t taps = (size_t)p.r * p.s;
        int k, cc;
        wpad = (uint8_t *)malloc((size_t)p.k * 4 * taps);
        memset(wpad, p.wzp, (size_t)p.k * 4 * taps);
        for (k = 0; k < p.k; ++k)
            for (cc = 0; cc < ch; ++cc)
                memcpy(wpad + ((size_t)k * 4 + cc) * taps, wt + ((size_t)k * ch + cc) * taps, taps);
        p.c = 4;
        c->c_pad = 4;
        wt = wpad;
    }
    B200_CALL(b200_conv2d_create(&p, wt, bias, &c->plan));
    free(wpad);
    c->plan_c = ch; c->plan_h = h; c->plan_w = w;
    op->run_func = op_b200_conv_2d_run;
}

/* ------------------------------------------------------------------------------------------
 * ip  (art/modules/quant/src/op/ip.cpp:73-209)
 * ------------------------------------------------------------------------------------------ */
typedef struct {
    op_t o;
    uint32_t num_output;
    qsettings_t q;
    b200_conv_t *plan;
    int plan_c, plan_h, plan_w;
    scratch_t in_scratch;
} op_b200_ip_t;

op_t *op_b200_ip_tp_alloc(workspace_t *ws)
{
    (void)ws;
    op_b200_ip_t *res = (op_b200_ip_t *)malloc(sizeof(*res));
    memset(res, 0, sizeof(*res));
    return (op_t *)res;
}

void op_b200_ip_tp_config(op_t *op)
{
    op_b200_ip_t *c = (op_b200_ip_t *)op;
    CHECK(op_setting_single_get(op, SETTING_IP_NUM_OUTPUT, dtUINT32, &c->num_output));
    get_in_q(op, &c->q);
    get_w_q(op, &c->q);
    get_out_q(op, &c->q);
}

void op_b200_ip_tp_destroy(op_t *op)
{
    op_b200_ip_t *c = (op_b200_ip_t *)op;
    if (c->plan)
        B200_CALL(b200_conv2d_destroy(c->plan));
    c->plan = NULL;
    scratch_release(&c->in_scratch);
}

void op_b200_ip_tp_dealloc(op_t *op)
{
    if (NULL != op)
        free(op);
}

static void op_b200_ip_run(op_t *op)
{
    op_b200_ip_t *c = (op_b200_ip_t *)op;
    int n, ch, h, w;
    dims_of(op->input_tensors[0], &n, &ch, &h, &w);
    const uint8_t *x = input_nhwc(op->input_tensors[0], &c->in_scratch);
    uint8_t *y = (uint8_t *)output_dev(&op->output_tensors[0], false);   /* [n][k]: layouts coincide */
    B200_CALL(b200_conv2d_run(c->plan, x, n, y, NULL));
}

void op_b200_ip_tp_prepare(op_t *op)
{
    op_b200_ip_t *c = (op_b200_ip_t *)op;
    int n, ch, h, w;
    alloc_io(op);
    if (op->input_tensors[0]->dtype != dtUINT8 && op->input_tensors[0]->dtype != dtINT8)
        LOG_error("b200: ip takes uint8 or int8 activations\n");
    dims_of(op->input_tensors[0], &n, &ch, &h, &w);
    if (c->plan && c->plan_c == ch && c->plan_h == h && c->plan_w == w) {
        op->run_func = op_b200_ip_run;
        return;
    }
    if (c->plan)
        B200_CALL(b200_conv2d_destroy(c->plan));
    const uint8_t *wt = (const uint8_t *)mem_cpu_data(op->input_tensors[1]->mem);
    const int32_t *bias = op->input_size == 3 ? (const int32_t *)mem_cpu_data(op->input_tensors[2]->mem) : NULL;
    const int32_t n_wa = (c->q.n_walpha == (size_t)c->num_output && c->num_output > 1) ? (int32_t)c->num_output : 1;
    if (op->input_tensors[0]->dtype == dtINT8)   /* ip.cpp:313-331 */
        B200_CALL(b200_ip_create_s8(
            ch, h, w, (int32_t)c->num_output, c->q.ialpha[0], c->q.walpha, n_wa, c->q.oalpha[0], c->q.obits[0],
            s8_wrap_allowed(), (const int8_t *)wt, bias, &c->plan));
    else
        B200_CALL(b200_ip_create(
            ch, h, w, (int32_t)c->num_output, c->q.ialpha[0], c->q.izp[0], c->q.walpha, n_wa, c->q.wzp[0],
            c->q.oalpha[0], c->q.ozp[0], c->q.obits[0], wt, bias, &c->plan));
    c->plan_c = ch; c->plan_h = h; c->plan_w = w;
    op->run_func = op_b200_ip_run;
}

/* ------------------------------------------------------------------------------------------
 * eltwise SUM and add  (art/modules/quant/src/op/eltwise.c:51-265, add.c:40-165)
 * ------------------------------------------------------------------------------------------ */
#define B200_MAX_ELT 4
typedef struct {
    op_t o;
    uint32_t operation;
    float *coeff;
    bool is_add;
    qsettings_t q;
    scratch_t in_scratch[B200_MAX_ELT];
} op_b200_eltwise_t;

static op_t *eltwise_alloc(bool is_add)
{
    op_b200_eltwise_t *res = (op_b200_eltwise_t *)malloc(sizeof(*res));
    memset(res, 0, sizeof(*res));
    res->is_add = is_add;
    return (op_t *)res;
}

op_t *op_b200_eltwise_tp_alloc(workspace_t *ws) { (void)ws; return eltwise_alloc(false); }
op_t *op_b200_add_tp_alloc(workspace_t *ws) { (void)ws; return eltwise_alloc(true); }

void op_b200_eltwise_tp_config(op_t *op)
{
    op_b200_eltwise_t *e = (op_b200_eltwise_t *)op;
    size_t len;
    CHECK(op_setting_single_get(op, SETTING_ELTWISE_OPERATION, dtUINT32, &e->operation));
    e->coeff = NULL;
    if (op_setting_if_set(op, SETTING_ELTWISE_COEFF)) {
        CHECK(op_setting_array_get(op, SETTING_ELTWISE_COEFF, dtFLOAT32, &len, &e->coeff));
        CHECK_EQ(op->input_size, len);
    }
    get_in_q(op, &e->q);
    get_out_q(op, &e->q);
}

void op_b200_add_tp_config(op_t *op)
{
    op_b200_eltwise_t *e = (op_b200_eltwise_t *)op;
    e->operation = SETTING_ELTWISE_OP_SUM;
    e->coeff = NULL;
    get_in_q(op, &e->q);
    get_out_q(op, &e->q);
}

static void eltwise_destroy(op_t *op)
{
    op_b200_eltwise_t *e = (op_b200_eltwise_t *)op;
    int i;
    for (i = 0; i < B200_MAX_ELT; ++i)
        scratch_release(&e->in_scratch[i]);
}
void op_b200_eltwise_tp_destroy(op_t *op) { eltwise_destroy(op); }
void op_b200_add_tp_destroy(op_t *op) { eltwise_destroy(op); }
void op_b200_eltwise_tp_dealloc(op_t *op) { if (NULL != op) free(op); }
void op_b200_add_tp_dealloc(op_t *op) { if (NULL != op) free(op); }

static void op_b200_eltwise_run(op_t *op)
{
    op_b200_eltwise_t *e = (op_b200_eltwise_t *)op;
    const uint8_t *xs[B200_MAX_ELT];
    size_t i;
    size_t count = shape_count(&op->output_tensors[0].shape);
    for (i = 0; i < op->input_size; ++i)
        xs[i] = input_nhwc(op->input_tensors[i], &e->in_scratch[i]);
    uint8_t *y = (uint8_t *)output_dev(&op->output_tensors[0], true);
    B200_CALL(b200_eltwise_sum_u8(
        xs, (int32_t)op->input_size, count, e->q.ialpha, e->q.izp, e->coeff, e->q.oalpha[0], e->q.ozp[0],
        e->q.obits[0], 0, y, NULL));
}

static void eltwise_prepare(op_t *op)
{
    op_b200_eltwise_t *e = (op_b200_eltwise_t *)op;
    alloc_io(op);
    if (op->input_tensors[0]->dtype != dtUINT8)
        LOG_error("b200: eltwise/add take uint8 tensors\n");
    if (e->operation != SETTING_ELTWISE_OP_SUM)
        LOG_error("b200: eltwise operation %u is not built (SUM only)\n", e->operation);
    if (op->input_size > B200_MAX_ELT)
        LOG_error("b200: eltwise with more than %d inputs is not built\n", B200_MAX_ELT);
    op->run_func = op_b200_eltwise_run;
}
void op_b200_eltwise_tp_prepare(op_t *op) { eltwise_prepare(op); }
void op_b200_add_tp_prepare(op_t *op) { eltwise_prepare(op); }

/* ------------------------------------------------------------------------------------------
 * relu  (art/modules/quant/src/op/relu.c:33-130)
 * ------------------------------------------------------------------------------------------ */
typedef struct {
    op_t o;
    qsettings_t q;
    scratch_t in_scratch;
} op_b200_relu_t;

op_t *op_b200_relu_tp_alloc(workspace_t *ws)
{
    (void)ws;
    op_b200_relu_t *res = (op_b200_relu_t *)malloc(sizeof(*res));
    memset(res, 0, sizeof(*res));
    return (op_t *)res;
}

void op_b200_relu_tp_config(op_t *op)
{
    op_b200_relu_t *r = (op_b200_relu_t *)op;
    get_in_q(op, &r->q);
    get_out_q(op, &r->q);
}

void op_b200_relu_tp_destroy(op_t *op) { scratch_release(&((op_b200_relu_t *)op)->in_scratch); }
void op_b200_relu_tp_dealloc(op_t *op) { if (NULL != op) free(op); }

static void op_b200_relu_run(op_t *op)
{
    op_b200_relu_t *r = (op_b200_relu_t *)op;
    size_t count = shape_count(&op->output_tensors[0].shape);
    const uint8_t *x = input_nhwc(op->input_tensors[0], &r->in_scratch);
    uint8_t *y = (uint8_t *)output_dev(&op->output_tensors[0], true);
    B200_CALL(b200_relu_u8(x, count, r->q.ialpha[0], r->q.izp[0], r->q.oalpha[0], r->q.ozp[0], r->q.obits[0], y, NULL));
}

void op_b200_relu_tp_prepare(op_t *op)
{
    alloc_io(op);
    if (op->input_tensors[0]->dtype != dtUINT8)
        LOG_error("b200: relu takes a uint8 tensor\n");
    op->run_func = op_b200_relu_run;
}

/* ------------------------------------------------------------------------------------------
 * pool  (art/modules/quant/src/op/pool.c:49-275)
 * ------------------------------------------------------------------------------------------ */
typedef struct {
    op_t o;
    uint32_t method, pad_h, pad_w, kernel_h, kernel_w, stride_h, stride_w;
    bool ceil_mode;
    qsettings_t q;
    scratch_t in_scratch;
} op_b200_pool_t;

op_t *op_b200_pool_tp_alloc(workspace_t *ws)
{
    (void)ws;
    op_b200_pool_t *res = (op_b200_pool_t *)malloc(sizeof(*res));
    memset(res, 0, sizeof(*res));
    return (op_t *)res;
}

void op_b200_pool_tp_config(op_t *op)
{
    op_b200_pool_t *p = (op_b200_pool_t *)op;
    CHECK(op_setting_single_get(op, SETTING_POOL_KERNEL_H, dtUINT32, &p->kernel_h));
    CHECK(op_setting_single_get(op, SETTING_POOL_KERNEL_W, dtUINT32, &p->kernel_w));
    CHECK(op_setting_single_get(op, SETTING_POOL_METHOD, dtUINT32, &p->method));
    CHECK(op_setting_single_get(op, SETTING_POOL_PAD_H, dtUINT32, &p->pad_h));
    CHECK(op_setting_single_get(op, SETTING_POOL_PAD_W, dtUINT32, &p->pad_w));
    CHECK(op_setting_single_get(op, SETTING_POOL_STRIDE_H, dtUINT32, &p->stride_h));
    CHECK(op_setting_single_get(op, SETTING_POOL_STRIDE_W, dtUINT32, &p->stride_w));
    CHECK(op_setting_single_get(op, SETTING_POOL_CEIL_MODE, dtBOOL, &p->ceil_mode));
    get_in_q(op, &p->q);
    get_out_q(op, &p->q);
}

void op_b200_pool_tp_destroy(op_t *op) { scratch_release(&((op_b200_pool_t *)op)->in_scratch); }
void op_b200_pool_tp_dealloc(op_t *op) { if (NULL != op) free(op); }

static void op_b200_pool_run(op_t *op)
{
    op_b200_pool_t *p = (op_b200_pool_t *)op;
    int n, c, h, w;
    dims_of(op->input_tensors[0], &n, &c, &h, &w);
    const uint8_t *x = input_nhwc(op->input_tensors[0], &p->in_scratch);
    uint8_t *y = (uint8_t *)output_dev(&op->output_tensors[0], true);
    B200_CALL(b200_pool_u8(
        x, n, c, h, w, (int32_t)p->method, (int32_t)p->kernel_h, (int32_t)p->kernel_w, (int32_t)p->pad_h,
        (int32_t)p->pad_w, (int32_t)p->stride_h, (int32_t)p->stride_w, p->ceil_mode ? 1 : 0, p->q.ialpha[0],
        p->q.izp[0], p->q.oalpha[0], p->q.ozp[0], p->q.obits[0], y, NULL));
}

void op_b200_pool_tp_prepare(op_t *op)
{
    alloc_io(op);
    if (op->input_tensors[0]->dtype != dtUINT8)
        LOG_error("b200: pool takes a uint8 tensor\n");
    op->run_func = op_b200_pool_run;
}

/* ------------------------------------------------------------------------------------------
 * quantize / dequantize  (art/modules/quant/src/op/quantize.c:40-272, dequantize.c:30-175)
 * The op types are module-defined in the reference; these carry the same codes
 * (art/modules/quant/include/art/quant/quant_op_tp.h:23-24) so that a quant case binds to them.
 * ------------------------------------------------------------------------------------------ */
typedef struct {
    op_t o;
    float *alpha;
    uint8_t *zp;
    uint8_t *bits;
    int32_t qtype;
    scratch_t in_scratch;
} op_b200_qdq_t;

static bool infer_shape_b200_quantize(op_t *op)
{
    CHECK_EQ(1, op->input_size);
    CHECK(1 >= op->output_size);
    if (0 == op->output_size) {
        op->output_size = 1;
        op->output_tensors = (tensor_t *)malloc(sizeof(tensor_t));
        memset(op->output_tensors, 0, sizeof(tensor_t));
        op->output_tensors[0].mem = mem_new(op->input_tensors[0]->mem->tp);
        /* quantize.c:51-65: SYMMETRIC gives int8, DEFAULT / BIASED uint8 (config has run: op.c:46-53) */
        op->output_tensors[0].dtype = ((op_b200_qdq_t *)op)->qtype == SETTING_QUANT_SYMMETRIC ? dtINT8 : dtUINT8;
    }
    op->output_tensors[0].shape = op->input_tensors[0]->shape;
    return true;
}

static bool infer_shape_b200_dequantize(op_t *op)
{
    CHECK_EQ(1, op->input_size);
    CHECK(1 >= op->output_size);
    if (0 == op->output_size) {
        op->output_size = 1;
        op->output_tensors = (tensor_t *)malloc(sizeof(tensor_t));
        memset(op->output_tensors, 0, sizeof(tensor_t));
        op->output_tensors[0].mem = mem_new(op->input_tensors[0]->mem->tp);
        op->output_tensors[0].dtype = dtFLOAT32;
    }
    op->output_tensors[0].shape = op->input_tensors[0]->shape;
    return true;
}

static const op_tp_t op_b200_quantize_tp = {
    .op_tp_code = OP_QUANT_QUANTIZE,
    .name = "quantize",
    .min_input_size = 1,
    .max_input_size = 1,
    .min_output_size = 1,
    .max_output_size = 1,
    .infer_output_func = infer_shape_b200_quantize,
    .constraints = { OP_SETTING_CONSTRAINT_REPEATED(SETTING_QUANT_OALPHA, dtFLOAT32),
                     OP_SETTING_CONSTRAINT_REPEATED(SETTING_QUANT_OZERO_POINT, dtUINT8),
                     OP_SETTING_CONSTRAINT_REPEATED(SETTING_QUANT_OBITS, dtUINT8),
                     OP_SETTING_CONSTRAINT_OPTIONAL(SETTING_QUANT_QTYPE, dtINT32, SETTING_QUANT_DEFAULT),
                     OP_SETTING_CONSTRAINT_END() }
};

static const op_tp_t op_b200_dequantize_tp = {
    .op_tp_code = OP_QUANT_DEQUANTIZE,
    .name = "dequantize",
    .min_input_size = 1,
    .max_input_size = 1,
    .min_output_size = 1,
    .max_output_size = 1,
    .infer_output_func = infer_shape_b200_dequantize,
    .constraints = { OP_SETTING_CONSTRAINT_REPEATED(SETTING_QUANT_IALPHA, dtFLOAT32),
                     OP_SETTING_CONSTRAINT_REPEATED(SETTING_QUANT_IZERO_POINT, dtUINT8),
                     OP_SETTING_CONSTRAINT_REPEATED(SETTING_QUANT_IBITS, dtUINT8),
                     OP_SETTING_CONSTRAINT_OPTIONAL(SETTING_QUANT_QTYPE, dtINT32, 0),
                     OP_SETTING_CONSTRAINT_END() }
};

static op_t *qdq_alloc(void)
{
    op_b200_qdq_t *res = (op_b200_qdq_t *)malloc(sizeof(*res));
    memset(res, 0, sizeof(*res));
    return (op_t *)res;
}
op_t *op_b200_quantize_tp_alloc(workspace_t *ws) { (void)ws; return qdq_alloc(); }
op_t *op_b200_dequantize_tp_alloc(workspace_t *ws) { (void)ws; return qdq_alloc(); }

void op_b200_quantize_tp_config(op_t *op)
{
    op_b200_qdq_t *q = (op_b200_qdq_t *)op;
    size_t len;
    CHECK(op_setting_array_get(op, SETTING_QUANT_OALPHA, dtFLOAT32, &len, &q->alpha));
    CHECK(op_setting_array_get(op, SETTING_QUANT_OZERO_POINT, dtUINT8, &len, &q->zp));
    CHECK(op_setting_array_get(op, SETTING_QUANT_OBITS, dtUINT8, &len, &q->bits));
    CHECK(op_setting_single_get(op, SETTING_QUANT_QTYPE, dtINT32, &q->qtype));
}

void op_b200_dequantize_tp_config(op_t *op)
{
    op_b200_qdq_t *q = (op_b200_qdq_t *)op;
    size_t len;
    CHECK(op_setting_array_get(op, SETTING_QUANT_IALPHA, dtFLOAT32, &len, &q->alpha));
    CHECK(op_setting_array_get(op, SETTING_QUANT_IZERO_POINT, dtUINT8, &len, &q->zp));
    CHECK(op_setting_array_get(op, SETTING_QUANT_IBITS, dtUINT8, &len, &q->bits));
    CHECK(op_setting_single_get(op, SETTING_QUANT_QTYPE, dtINT32, &q->qtype));
}

void op_b200_quantize_tp_destroy(op_t *op) { scratch_release(&((op_b200_qdq_t *)op)->in_scratch); }
void op_b200_dequantize_tp_destroy(op_t *op) { scratch_release(&((op_b200_qdq_t *)op)->in_scratch); }
void op_b200_quantize_tp_dealloc(op_t *op) { if (NULL != op) free(op); }
void op_b200_dequantize_tp_dealloc(op_t *op) { if (NULL != op) free(op); }

static const void *float_or_bytes_dev(tensor_t *t, scratch_t *scratch, size_t bytes)
{
    if (t->mem->tp == b200_mem_tp)
        return mem_data(t->mem);
    scratch_reserve(scratch, bytes);
    B200_CALL(b200_memcpy_h2d(scratch->buf, mem_cpu_data(t->mem), bytes, NULL));
    return scratch->buf;
}

static bool qdq_key_built(int32_t key)
{
    switch (key) {
    case 0x0008: case 0x0108:
    case 0x0202: case 0x0203: case 0x0204: case 0x0206: case 0x0207: case 0x0208:
        return true;
    default:
        return false;
    }
}

static void op_b200_quantize_run(op_t *op)
{
    op_b200_qdq_t *q = (op_b200_qdq_t *)op;
    int n, c, h, w;
    dims_of(op->input_tensors[0], &n, &c, &h, &w);
    const float *x = (const float *)float_or_bytes_dev(
        op->input_tensors[0], &q->in_scratch, sizeof(float) * shape_count(&op->input_tensors[0]->shape));
    uint8_t *y = (uint8_t *)output_dev(&op->output_tensors[0], true);
    if (q->qtype == SETTING_QUANT_SYMMETRIC)
        B200_CALL(b200_quantize_s8(x, (int8_t *)y, n, c, h, w, q->alpha[0], q->bits[0], 1, NULL));
    else
        B200_CALL(b200_quantize_u8(x, y, n, c, h, w, q->alpha[0], q->zp[0], q->bits[0], 1, NULL));
}

static void op_b200_dequantize_run(op_t *op)
{
    op_b200_qdq_t *q = (op_b200_qdq_t *)op;
    int n, c, h, w;
    dims_of(op->input_tensors[0], &n, &c, &h, &w);
    tensor_t *ti = op->input_tensors[0];
    bool in_nhwc = ti->mem->tp == b200_mem_tp && ((b200_mem_t *)ti->mem)->nhwc;
    const uint8_t *x = (const uint8_t *)float_or_bytes_dev(ti, &q->in_scratch, shape_count(&ti->shape));
    if (ti->mem->tp == b200_mem_tp)
        in_nhwc = ((b200_mem_t *)ti->mem)->nhwc;   /* mem_data() may have re-uploaded NCHW bytes */
    float *y = (float *)output_dev(&op->output_tensors[0], false);
    if (q->qtype == SETTING_QUANT_SYMMETRIC)
        B200_CALL(b200_dequantize_s8((const int8_t *)x, y, n, c, h, w, q->alpha[0], in_nhwc ? 1 : 0, NULL));
    else
        B200_CALL(b200_dequantize_u8(x, y, n, c, h, w, q->alpha[0], q->zp[0], in_nhwc ? 1 : 0, NULL));
}

void op_b200_quantize_tp_prepare(op_t *op)
{
    op_b200_qdq_t *q = (op_b200_qdq_t *)op;
    alloc_io(op);
    CHECK(op->input_tensors[0]->dtype == dtFLOAT32);
    int32_t key = q->qtype << 8 | q->bits[0];
    /* quantize.c:233-245: DEFAULT / BIASED with 8 bits -> uint8; SYMMETRIC with 2, 3, 4, 6, 7 or 8 bits -> int8 */
    if (!qdq_key_built(key))
        LOG_error("b200: quantization of %d bits with type %d is not built (uint8, and int8 of 2..8 bits)\n", q->bits[0], q->qtype);
    op->run_func = op_b200_quantize_run;
}

void op_b200_dequantize_tp_prepare(op_t *op)
{
    op_b200_qdq_t *q = (op_b200_qdq_t *)op;
    alloc_io(op);
    int32_t key = q->qtype << 8 | q->bits[0];
    if (!qdq_key_built(key))
        LOG_error("b200: dequantization of %d bits with type %d is not built (uint8, and int8 of 2..8 bits)\n", q->bits[0], q->qtype);
    op->run_func = op_b200_dequantize_run;
}

/* ------------------------------------------------------------------------------------------
 * module and workspace  (art/modules/quant/src/quant_module.c:27-120,
 * art/modules/cuda_quant/src/cuda_quant_module.c:79-141)
 * ------------------------------------------------------------------------------------------ */
typedef struct {
    workspace_t ws;
    char *name;
    int device;
} b200_workspace_t;

/* the shared op types live in libart and give shape inference and setting defaults
 * (art/src/op.c:2252-2660) */
extern const op_tp_t op_conv_2d_tp;
extern const op_tp_t op_ip_tp;
extern const op_tp_t op_relu_tp;
extern const op_tp_t op_add_tp;
extern const op_tp_t op_eltwise_tp;
extern const op_tp_t op_pool_tp;

extern const module_t b200_module_tp;
static int b200_ws_num = 0;

static const char *ws_b200_name(const b200_workspace_t *ws) { return ws->name; }
static const mem_tp *ws_b200_mem_tp(b200_workspace_t *ws) { (void)ws; return b200_mem_tp; }

/* Settings: item 1 with dtype dtINT32 selects the device, like SETTING_CUDA_WORKSPACE_DEVID of
 * the reference's GPU modules (art/modules/cuda/include/art/cuda/cuda_ws_settings.h:22); both
 * reference drivers pass NULL, so NART_B200_DEVICE in the environment works as well. */
static workspace_t *ws_b200_new(const setting_entry_t *settings)
{
    char tmp[32];
    b200_workspace_t *res = (b200_workspace_t *)malloc(sizeof(*res));
    memset(res, 0, sizeof(*res));
    snprintf(tmp, sizeof(tmp), "b200:%d", b200_ws_num++);
    res->name = (char *)malloc(strlen(tmp) + 1);
    strcpy(res->name, tmp);
    res->ws.module_type = &b200_module_tp;
    res->device = -1;
    for (; settings != NULL && settings->item != 0; ++settings) {
        if (settings->item == 1 && settings->dtype == dtINT32)
            res->device = settings->v.single.value.i32;
    }
    if (res->device < 0 && getenv("NART_B200_DEVICE"))
        res->device = atoi(getenv("NART_B200_DEVICE"));
    if (res->device >= 0)
        B200_CALL(b200_set_device(res->device));
    else
        B200_CALL(b200_get_device(&res->device));
    return (workspace_t *)res;
}

static void ws_b200_delete(b200_workspace_t *ws)
{
    if (ws->name)
        free(ws->name);
    free(ws);
}

#define B200_ENTRY(tp_obj, opname)                                                             \
    {                                                                                          \
        .tp = &tp_obj, .alloc_func = (op_alloc_op_func)op_b200_##opname##_tp_alloc,            \
        .config_func = op_b200_##opname##_tp_config, .destroy_func = op_b200_##opname##_tp_destroy, \
        .dealloc_func = op_b200_##opname##_tp_dealloc, .prepare_func = op_b200_##opname##_tp_prepare, \
    }

static op_tp_entry_t b200_op_entries[] = {
    B200_ENTRY(op_b200_quantize_tp, quantize),
    B200_ENTRY(op_b200_dequantize_tp, dequantize),
    B200_ENTRY(op_conv_2d_tp, conv_2d),
    B200_ENTRY(op_ip_tp, ip),
    B200_ENTRY(op_relu_tp, relu),
    B200_ENTRY(op_add_tp, add),
    B200_ENTRY(op_eltwise_tp, eltwise),
    B200_ENTRY(op_pool_tp, pool),
    { NULL },
};

const module_t DLL_PUBLIC b200_module_tp = {
    .op_group = OP_GROUP_CODE_QUANT,
    .name_func = (ws_name_func)ws_b200_name,
    .memtype_func = (ws_memtp_func)ws_b200_mem_tp,
    .new_func = (ws_new_func)ws_b200_new,
    .delete_func = (ws_delete_func)ws_b200_delete,
    .op_tp_entry = b200_op_entries,
};
