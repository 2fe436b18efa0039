// A prepared, runnable op list bound to one device -- what the reference calls a parade
// (art/src/parade.c:169-197 of ModelTC/NART: parade_prepare, parade_run) -- assembled through
// the C-ABI.  Tensors live on the device as NHWC uint8; the case inputs and outputs cross the
// boundary in the reference's NCHW layout through staging buffers, with the layout change (and
// quantize / dequantize where asked) done by device kernels.
#include <string.h>

#include <memory>
#include <vector>

#include "common.cuh"
#include "kernels.h"

using namespace b200;

namespace {

struct CaseTensor {
    int c = 0, h = 0, w = 0;
    int c_phys = 0;          // channels of the device NHWC buffer (>= c; the 3-channel image is padded to 4)
    uint8_t *dev = nullptr;  // [max_batch][h][w][c_phys]
    size_t bytes_per_image() const { return (size_t)h * w * c_phys; }
};

enum class OpKind { Conv, Eltwise, Relu, Pool };

struct CaseOp {
    OpKind kind;
    std::vector<int> ins;
    int out = -1;
    // conv / ip
    b200_conv_t *conv = nullptr;
    int residual = -1;        // tensor added in the conv's epilogue (a fused eltwise SUM), or -1
    bool skipped = false;     // an eltwise op whose work a conv has taken over
    // eltwise
    std::vector<float> ialpha, coeff;
    std::vector<uint8_t> izp;
    bool has_coeff = false;
    float oalpha = 1.f;
    uint8_t ozp = 0, obits = 8;
    int relu = 0;
    // eltwise: the prepared constants (built once in b200_case_prepare)
    b200::EltwiseArgs elt;
    bool elt_fast = false;
    // direction in which the op's kernel walks its tiles: 1 = last to first (see b200_case_prepare)
    int reverse = 0;
    // relu / max-pool lookup table
    uint8_t lut[256];
    uint8_t *lut_dev = nullptr;
    // pool
    int method = 0;
    PoolGeom pg;
    PoolAvgTab ptab;
};

struct CaseIO {
    int tensor = -1;
    bool is_f32 = false;
    float alpha = 1.f;
    uint8_t zp = 0, bits = 8;
    void *staging = nullptr;   // device, host layout (NCHW), max_batch images
    size_t bytes_per_image = 0;
};

}  // namespace

struct b200_case {
    std::vector<CaseTensor> tensors;
    std::vector<CaseOp> ops;
    std::vector<CaseIO> inputs, outputs;
    int max_batch = 0;
    bool prepared = false;
    bool fuse = false;                 // fold residual adds into the convs that feed them (b200_case_set_fusion)
    int fused_adds = 0;
    int device = 0;
    // per-launch timing (off by default)
    bool profiling = false;
    std::vector<cudaEvent_t> events;   // launches + 1
    std::vector<int> kinds;            // kind of each launch of the last run
    cudaStream_t last_stream = nullptr;
    bool have_profile = false;
    // CUDA graph of one run, per (batch, stream); off by default
    bool use_graph = false;
    struct Graph {
        int batch;
        cudaStream_t stream;
        int runs_seen;           // eager runs at this batch before capturing (the first one allocates)
        cudaGraphExec_t exec;
    };
    std::vector<Graph> graphs;
    // pipelined host runs (b200_case_submit_host): a copy stream, a compute stream, and the events
    // that order them
    cudaStream_t copy_stream = nullptr, comp_stream = nullptr, out_stream = nullptr;
    cudaEvent_t h2d_done = nullptr, after_inputs = nullptr;
    // the results of a submitted step travel to the host on out_stream, behind comp_done; the output kernels of the
    // next step wait for d2h_done before they overwrite the device staging buffers
    cudaEvent_t comp_done = nullptr, d2h_done = nullptr;
    bool submitted = false;
};

namespace {

int new_tensor(b200_case *cs, int c, int h, int w, int c_phys)
{
    CaseTensor t;
    t.c = c; t.h = h; t.w = w; t.c_phys = c_phys;
    cs->tensors.push_back(t);
    return (int)cs->tensors.size() - 1;
}

int check_building(b200_case *cs, const char *what)
{
    if (!cs)
        return fail(B200_ERR_INVALID, "%s: case is NULL", what);
    if (cs->prepared)
        return fail(B200_ERR_INVALID, "%s: the case is already prepared", what);
    return B200_OK;
}

int check_tensor(const b200_case *cs, int id, const char *what)
{
    if (id < 0 || id >= (int)cs->tensors.size())
        return fail(B200_ERR_INVALID, "%s: tensor id %d does not exist", what, id);
    return B200_OK;
}

// A two-input eltwise SUM whose later-produced input comes from a conv that nothing else reads is
// folded into that conv's epilogue: the conv then writes the eltwise op's output tensor and the
// eltwise op is skipped.  The values are those of the two separate ops (see
// b200_conv2d_fuse_residual_add); convs that cannot take the fusion keep the separate kernel.
void fuse_residual_adds(b200_case *cs)
{
    const int n_ops = (int)cs->ops.size();
    std::vector<int> readers(cs->tensors.size(), 0), producer(cs->tensors.size(), -1);
    for (int i = 0; i < n_ops; ++i) {
        for (int t : cs->ops[i].ins)
            readers[t]++;
        producer[cs->ops[i].out] = i;
    }
    for (const auto &io : cs->outputs)
        readers[io.tensor]++;
    for (int i = 0; i < n_ops; ++i) {
        CaseOp &add = cs->ops[i];
        if (add.kind != OpKind::Eltwise || add.ins.size() != 2 || add.ins[0] == add.ins[1])
            continue;
        // the input produced last is the one whose producer can see the other input complete
        const int p0 = producer[add.ins[0]], p1 = producer[add.ins[1]];
        const int ci = p0 > p1 ? 0 : 1;
        const int pi = ci == 0 ? p0 : p1;
        if (pi < 0 || pi >= i)
            continue;
        CaseOp &conv = cs->ops[pi];
        if (conv.kind != OpKind::Conv || conv.residual >= 0 || readers[conv.out] != 1)
            continue;
        const float *coeff = add.has_coeff ? add.coeff.data() : nullptr;
        if (b200_conv2d_fuse_residual_add(conv.conv, ci, add.ialpha.data(), add.izp.data(), coeff, add.oalpha,
                                          add.ozp, add.obits, add.relu) != B200_OK)
            continue;   // not this conv: the eltwise kernel stays
        conv.residual = add.ins[1 - ci];
        conv.out = add.out;
        add.skipped = true;
        cs->fused_adds++;
    }
}

}  // namespace

extern "C" {

int b200_case_create(b200_case_t **cs)
{
    if (!cs)
        return fail(B200_ERR_INVALID, "case_create: NULL argument");
    *cs = new b200_case();
    cudaGetDevice(&(*cs)->device);
    return B200_OK;
}

int b200_case_destroy(b200_case_t *cs)
{
    if (!cs)
        return B200_OK;
    for (auto &t : cs->tensors)
        cudaFree(t.dev);
    for (auto &op : cs->ops) {
        if (op.conv)
            b200_conv2d_destroy(op.conv);
        cudaFree(op.lut_dev);
    }
    for (auto &io : cs->inputs)
        cudaFree(io.staging);
    for (auto &io : cs->outputs)
        cudaFree(io.staging);
    for (auto e : cs->events)
        cudaEventDestroy(e);
    for (auto &gr : cs->graphs)
        if (gr.exec)
            cudaGraphExecDestroy(gr.exec);
    if (cs->h2d_done) cudaEventDestroy(cs->h2d_done);
    if (cs->after_inputs) cudaEventDestroy(cs->after_inputs);
    if (cs->comp_done) cudaEventDestroy(cs->comp_done);
    if (cs->d2h_done) cudaEventDestroy(cs->d2h_done);
    if (cs->out_stream) cudaStreamDestroy(cs->out_stream);
    if (cs->copy_stream) cudaStreamDestroy(cs->copy_stream);
    if (cs->comp_stream) cudaStreamDestroy(cs->comp_stream);
    delete cs;
    return B200_OK;
}

int b200_case_input_u8(b200_case_t *cs, int32_t c, int32_t h, int32_t w, int32_t *tensor)
{
    B200_TRY(check_building(cs, "case_input_u8"));
    if (!tensor || c <= 0 || h <= 0 || w <= 0)
        return fail(B200_ERR_INVALID, "case_input_u8: bad argument");
    // few-channel images are padded to a multiple of 4 so that every pixel is word aligned
    int c_phys = c % 4 == 0 ? c : (c + 3) / 4 * 4;
    CaseIO io;
    io.tensor = new_tensor(cs, c, h, w, c_phys);
    io.is_f32 = false;
    io.bytes_per_image = (size_t)c * h * w;
    cs->inputs.push_back(io);
    *tensor = io.tensor;
    return B200_OK;
}

int b200_case_input_f32(
    b200_case_t *cs, int32_t c, int32_t h, int32_t w, float oalpha, uint8_t ozp, uint8_t obits,
    int32_t *tensor)
{
    B200_TRY(check_building(cs, "case_input_f32"));
    if (!tensor || c <= 0 || h <= 0 || w <= 0 || obits < 1 || obits > 8 || !(oalpha > 0.f))
        return fail(B200_ERR_INVALID, "case_input_f32: bad argument");
    CaseIO io;
    io.tensor = new_tensor(cs, c, h, w, c);
    io.is_f32 = true;
    io.alpha = oalpha; io.zp = ozp; io.bits = obits;
    io.bytes_per_image = (size_t)c * h * w * sizeof(float);
    cs->inputs.push_back(io);
    *tensor = io.tensor;
    return B200_OK;
}

int b200_case_conv2d(
    b200_case_t *cs, int32_t in, const b200_conv_params *params, const uint8_t *weights,
    const int32_t *bias, int32_t *out)
{
    B200_TRY(check_building(cs, "case_conv2d"));
    B200_TRY(check_tensor(cs, in, "case_conv2d"));
    if (!params || !weights || !out)
        return fail(B200_ERR_INVALID, "case_conv2d: NULL argument");
    const CaseTensor ti = cs->tensors[in];
    if (params->c != ti.c || params->h != ti.h || params->w != ti.w)
        return fail(
            B200_ERR_INVALID, "case_conv2d: params %dx%dx%d do not match input tensor %dx%dx%d",
            params->c, params->h, params->w, ti.c, ti.h, ti.w);
    CaseOp op;
    op.kind = OpKind::Conv;
    op.ins = { in };
    b200_conv_params p = *params;
    // Channel padding.  A tensor whose channel count is not a multiple of 16 lives in a device buffer
    // with the count rounded up (c_phys), so that every conv around it can take the tensor-core path
    // (MobileNetV2's 24-channel tensors).  Padding input channels get zero weights (stored as wzp),
    // padding output channels zero weights and a zero bias: they add nothing to any result and
    // their own values are never read with a non-zero weight.
    const size_t taps = (size_t)p.r * p.s;
    const bool depthwise = p.group > 1 && p.group == params->c && p.k == params->c;
    if (ti.c_phys != ti.c && p.group != 1 && !depthwise)
        return fail(B200_ERR_UNSUPPORTED, "case_conv2d: grouped conv on a channel-padded input");
    const int c_in = ti.c_phys;
    int k_phys = p.k;
    if (depthwise)
        k_phys = ti.c_phys;
    else if (p.group == 1 && p.k % 16 != 0 && p.k >= 8)
        k_phys = (p.k + 15) / 16 * 16;
    std::vector<uint8_t> wpad;
    std::vector<int32_t> bpad;
    std::vector<float> wapad;
    const uint8_t *wsrc = weights;
    const int32_t *bsrc = bias;
    if (c_in != ti.c || k_phys != p.k) {
        const int cg_src = depthwise ? 1 : ti.c, cg_dst = depthwise ? 1 : c_in;
        wpad.assign((size_t)k_phys * cg_dst * taps, p.wzp);
        for (int k = 0; k < p.k; ++k)
            memcpy(&wpad[(size_t)k * cg_dst * taps], &weights[(size_t)k * cg_src * taps], (size_t)cg_src * taps);
        wsrc = wpad.data();
        if (k_phys != p.k) {
            bpad.assign(k_phys, 0);
            if (bias)
                memcpy(bpad.data(), bias, sizeof(int32_t) * p.k);
            bsrc = bpad.data();
            if (p.n_walpha == p.k && p.walpha) {
                wapad.assign(p.walpha, p.walpha + p.k);
                wapad.resize(k_phys, p.walpha[p.k - 1]);
                p.walpha = wapad.data();
                p.n_walpha = k_phys;
            }
        }
        p.c = c_in;
        p.k = k_phys;
        if (depthwise)
            p.group = c_in;
    }
    B200_TRY(b200_conv2d_create(&p, wsrc, bsrc, &op.conv));
    int32_t oh, ow;
    b200_conv2d_out_dims(op.conv, &oh, &ow);
    op.out = new_tensor(cs, params->k, oh, ow, k_phys);
    *out = op.out;
    cs->ops.push_back(op);
    return B200_OK;
}

int b200_case_ip(
    b200_case_t *cs, int32_t in, int32_t k, float ialpha, uint8_t izp, const float *walpha,
    int32_t n_walpha, uint8_t wzp, float oalpha, uint8_t ozp, uint8_t obits,
    const uint8_t *weights, const int32_t *bias, int32_t *out)
{
    B200_TRY(check_building(cs, "case_ip"));
    B200_TRY(check_tensor(cs, in, "case_ip"));
    if (!weights || !out)
        return fail(B200_ERR_INVALID, "case_ip: NULL argument");
    const CaseTensor ti = cs->tensors[in];
    if (ti.c_phys != ti.c)
        return fail(B200_ERR_UNSUPPORTED, "case_ip: channel-padded input");
    CaseOp op;
    op.kind = OpKind::Conv;
    op.ins = { in };
    B200_TRY(b200_ip_create(
        ti.c, ti.h, ti.w, k, ialpha, izp, walpha, n_walpha, wzp, oalpha, ozp, obits, weights, bias, &op.conv));
    op.out = new_tensor(cs, k, 1, 1, k);
    *out = op.out;
    cs->ops.push_back(op);
    return B200_OK;
}

int b200_case_eltwise_sum(
    b200_case_t *cs, const int32_t *ins, int32_t n_in, const float *ialpha, const uint8_t *izp,
    const float *coeff, float oalpha, uint8_t ozp, uint8_t obits, int32_t relu, int32_t *out)
{
    B200_TRY(check_building(cs, "case_eltwise_sum"));
    if (!ins || !ialpha || !izp || !out || n_in < 1 || n_in > 4)
        return fail(B200_ERR_INVALID, "case_eltwise_sum: bad argument");
    CaseOp op;
    op.kind = OpKind::Eltwise;
    for (int i = 0; i < n_in; ++i) {
        B200_TRY(check_tensor(cs, ins[i], "case_eltwise_sum"));
        const CaseTensor &a = cs->tensors[ins[0]], &b = cs->tensors[ins[i]];
        if (a.c != b.c || a.h != b.h || a.w != b.w || a.c_phys != b.c_phys)
            return fail(B200_ERR_INVALID, "case_eltwise_sum: input %d has a different shape", i);
        op.ins.push_back(ins[i]);
        op.ialpha.push_back(ialpha[i]);
        op.izp.push_back(izp[i]);
        op.coeff.push_back(coeff ? coeff[i] : 1.0f);
    }
    op.has_coeff = coeff != nullptr;
    op.oalpha = oalpha; op.ozp = ozp; op.obits = obits; op.relu = relu;
    const CaseTensor a = cs->tensors[ins[0]];
    op.out = new_tensor(cs, a.c, a.h, a.w, a.c_phys);
    *out = op.out;
    cs->ops.push_back(op);
    return B200_OK;
}

int b200_case_relu(
    b200_case_t *cs, int32_t in, float ialpha, uint8_t izp, float oalpha, uint8_t ozp,
    uint8_t obits, int32_t *out)
{
    B200_TRY(check_building(cs, "case_relu"));
    B200_TRY(check_tensor(cs, in, "case_relu"));
    if (!out)
        return fail(B200_ERR_INVALID, "case_relu: NULL argument");
    CaseOp op;
    op.kind = OpKind::Relu;
    op.ins = { in };
    B200_TRY(relu_build_lut(ialpha, izp, oalpha, ozp, obits, op.lut));
    const CaseTensor a = cs->tensors[in];
    op.out = new_tensor(cs, a.c, a.h, a.w, a.c_phys);
    *out = op.out;
    cs->ops.push_back(op);
    return B200_OK;
}

int b200_case_pool(
    b200_case_t *cs, int32_t in, int32_t method, int32_t kernel_h, int32_t kernel_w, int32_t pad_h,
    int32_t pad_w, int32_t stride_h, int32_t stride_w, int32_t ceil_mode, float ialpha,
    uint8_t izp, float oalpha, uint8_t ozp, uint8_t obits, int32_t *out)
{
    B200_TRY(check_building(cs, "case_pool"));
    B200_TRY(check_tensor(cs, in, "case_pool"));
    if (!out)
        return fail(B200_ERR_INVALID, "case_pool: NULL argument");
    const CaseTensor a = cs->tensors[in];
    CaseOp op;
    op.kind = OpKind::Pool;
    op.ins = { in };
    op.method = method;
    B200_TRY(pool_prepare(
        a.h, a.w, method, kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w, ceil_mode, ialpha,
        izp, oalpha, ozp, obits, &op.pg, op.lut, &op.ptab));
    op.out = new_tensor(cs, a.c, op.pg.oh, op.pg.ow, a.c_phys);
    *out = op.out;
    cs->ops.push_back(op);
    return B200_OK;
}

int b200_case_output_u8(b200_case_t *cs, int32_t tensor)
{
    B200_TRY(check_building(cs, "case_output_u8"));
    B200_TRY(check_tensor(cs, tensor, "case_output_u8"));
    const CaseTensor &t = cs->tensors[tensor];
    CaseIO io;
    io.tensor = tensor;
    io.is_f32 = false;
    io.bytes_per_image = (size_t)t.c * t.h * t.w;
    cs->outputs.push_back(io);
    return B200_OK;
}

int b200_case_output_f32(b200_case_t *cs, int32_t tensor, float ialpha, uint8_t izp)
{
    B200_TRY(check_building(cs, "case_output_f32"));
    B200_TRY(check_tensor(cs, tensor, "case_output_f32"));
    const CaseTensor &t = cs->tensors[tensor];
    if (t.c_phys != t.c)
        return fail(B200_ERR_UNSUPPORTED, "case_output_f32: a channel-padded tensor (%d channels) can only leave as uint8", t.c);
    CaseIO io;
    io.tensor = tensor;
    io.is_f32 = true;
    io.alpha = ialpha; io.zp = izp;
    io.bytes_per_image = (size_t)t.c * t.h * t.w * sizeof(float);
    cs->outputs.push_back(io);
    return B200_OK;
}

int b200_case_prepare(b200_case_t *cs, int32_t max_batch)
{
    B200_TRY(check_building(cs, "case_prepare"));
    if (max_batch <= 0)
        return fail(B200_ERR_INVALID, "case_prepare: max_batch must be positive");
    cs->max_batch = max_batch;
    if (cs->fuse)
        fuse_residual_adds(cs);
    for (auto &t : cs->tensors) {
        // 256 spare bytes: vector loads of the last pixel may read past a ragged channel count
        size_t bytes = t.bytes_per_image() * max_batch + 256;
        B200_TRY(b200_malloc((void **)&t.dev, bytes));
        B200_CUDA_TRY(cudaMemset(t.dev, 0, bytes));
    }
    for (auto *ios : { &cs->inputs, &cs->outputs })
        for (auto &io : *ios)
            B200_TRY(b200_malloc(&io.staging, io.bytes_per_image * max_batch));
    for (auto &op : cs->ops) {
        // conv scratch tensors are sized once, for the largest batch: a graph captured at one batch size
        // keeps their addresses, which a later, larger batch must not move
        if (op.kind == OpKind::Conv && op.conv)
            B200_TRY(b200_conv2d_reserve(op.conv, max_batch));
        if (op.kind == OpKind::Relu || (op.kind == OpKind::Pool && op.method == 0)) {
            B200_TRY(b200_malloc((void **)&op.lut_dev, 256));
            B200_CUDA_TRY(cudaMemcpy(op.lut_dev, op.lut, 256, cudaMemcpyHostToDevice));
        }
    }
    // Zig-zag traversal.  A tensor of this path is larger than what stays in L2 behind its producer, but
    // the part written last is still there: every op walks its tiles in the direction opposite to the op
    // that produced its (most recently written) input, so that it starts on that part.  The pools and
    // the layout kernels always run first to last.  Results do not depend on the direction.
    {
        const char *e = getenv("B200_CASE_ZIGZAG");
        const bool zigzag = !(e && atoi(e) == 0);
        std::vector<int> dir(cs->tensors.size(), 0);     // direction in which each tensor was written
        for (auto &op : cs->ops) {
            if (op.kind == OpKind::Eltwise) {
                B200_TRY(eltwise_prepare((int)op.ins.size(), op.ialpha.data(), op.izp.data(), op.has_coeff ? op.coeff.data() : nullptr,
                                         op.oalpha, op.ozp, op.obits, op.relu, &op.elt, &op.elt_fast));
            }
            if (op.skipped)
                continue;
            int latest = op.ins[0];
            for (int t : op.ins)
                latest = t > latest ? t : latest;           // tensor ids grow in creation order
            if (op.residual >= 0 && op.residual > latest)
                latest = op.residual;
            int rev = zigzag ? !dir[latest] : 0;
            if (op.kind == OpKind::Conv) {
                // a row-lowered conv reads the scratch tensor its own lowering kernel has just written, first to last
                if (op.conv->lowered)
                    rev = zigzag ? 1 : 0;
                if (op.conv->igemm)
                    conv_igemm_set_reverse(op.conv->igemm, rev);
                else
                    rev = 0;
            } else if (op.kind != OpKind::Eltwise) {
                rev = 0;
            }
            op.reverse = rev;
            dir[op.out] = rev;
        }
    }
    // Every tensor-core conv names the weights of the next one, so that they are on their way into L2 while it
    // runs (B200_CASE_PREFETCH=0 turns that off).
    {
        const char *e = getenv("B200_CASE_PREFETCH");
        const bool on = !(e && atoi(e) == 0);
        ConvIgemmPlan *prev = nullptr;
        for (auto &op : cs->ops) {
            if (op.skipped || op.kind != OpKind::Conv || !op.conv->igemm)
                continue;
            if (prev) {
                const uint8_t *w = nullptr;
                size_t bytes = 0;
                if (on)
                    conv_igemm_weights(op.conv->igemm, &w, &bytes);
                conv_igemm_set_next_readonly(prev, w, bytes);
            }
            prev = op.conv->igemm;
        }
        if (prev)
            conv_igemm_set_next_readonly(prev, nullptr, 0);
    }
    cs->prepared = true;
    return B200_OK;
}

int b200_case_tensor_dims(const b200_case_t *cs, int32_t tensor, int32_t *c, int32_t *h, int32_t *w)
{
    if (!cs || !c || !h || !w)
        return fail(B200_ERR_INVALID, "case_tensor_dims: NULL argument");
    B200_TRY(check_tensor(cs, tensor, "case_tensor_dims"));
    *c = cs->tensors[tensor].c;
    *h = cs->tensors[tensor].h;
    *w = cs->tensors[tensor].w;
    return B200_OK;
}

static const CaseIO *get_io(const b200_case_t *cs, int is_output, int index)
{
    const std::vector<CaseIO> &v = is_output ? cs->outputs : cs->inputs;
    if (index < 0 || index >= (int)v.size())
        return nullptr;
    return &v[index];
}

int b200_case_io_bytes(const b200_case_t *cs, int32_t is_output, int32_t index, size_t *bytes_per_image)
{
    if (!cs || !bytes_per_image)
        return fail(B200_ERR_INVALID, "case_io_bytes: NULL argument");
    const CaseIO *io = get_io(cs, is_output, index);
    if (!io)
        return fail(B200_ERR_INVALID, "case_io_bytes: no such %s %d", is_output ? "output" : "input", index);
    *bytes_per_image = io->bytes_per_image;
    return B200_OK;
}

int b200_case_io_device_ptr(const b200_case_t *cs, int32_t is_output, int32_t index, void **dev_ptr)
{
    if (!cs || !dev_ptr)
        return fail(B200_ERR_INVALID, "case_io_device_ptr: NULL argument");
    const CaseIO *io = get_io(cs, is_output, index);
    if (!io || !cs->prepared)
        return fail(B200_ERR_INVALID, "case_io_device_ptr: no such buffer (is the case prepared?)");
    *dev_ptr = io->staging;
    return B200_OK;
}

int b200_case_tensor_device_ptr(const b200_case_t *cs, int32_t tensor, void **dev_ptr)
{
    if (!cs || !dev_ptr)
        return fail(B200_ERR_INVALID, "case_tensor_device_ptr: NULL argument");
    B200_TRY(check_tensor(cs, tensor, "case_tensor_device_ptr"));
    *dev_ptr = cs->tensors[tensor].dev;
    return B200_OK;
}

// phase: 0 = whole run, 1 = input layout kernels only, 2 = ops and outputs only
static int run_eager(b200_case_t *cs, int32_t batch, b200_stream_t stream, int phase = 0);

// The ops (phase 2) and then the output kernels (phase 3), which stay outside a captured graph: they write the
// device staging buffers that the previous submitted step's device-to-host copy may still be reading.
static int run_outputs(b200_case_t *cs, int32_t batch, b200_stream_t stream)
{
    if (cs->submitted && cs->d2h_done)
        B200_CUDA_TRY(cudaStreamWaitEvent(as_stream(stream), cs->d2h_done, 0));
    return run_eager(cs, batch, stream, 3);
}

int b200_case_run_device(b200_case_t *cs, int32_t batch, b200_stream_t stream)
{
    if (!cs || !cs->prepared)
        return fail(B200_ERR_INVALID, "case_run: the case is not prepared");
    if (batch < 0 || batch > cs->max_batch)
        return fail(B200_ERR_INVALID, "case_run: batch %d outside 0..%d", batch, cs->max_batch);
    if (batch == 0)
        return B200_OK;
    // the legacy default stream cannot be captured: graph mode needs a stream of its own
    if (!cs->use_graph || cs->profiling || stream == nullptr) {
        if (cs->profiling || !cs->after_inputs) {
            // one whole pass (the event pairs of the profiler bracket every launch in order); a pipelined
            // caller may refill the input staging buffer once this pass is through
            const int rc = run_eager(cs, batch, stream);
            if (rc == B200_OK && cs->after_inputs)
                B200_CUDA_TRY(cudaEventRecord(cs->after_inputs, as_stream(stream)));
            return rc;
        }
        B200_TRY(run_eager(cs, batch, stream, 1));
        B200_CUDA_TRY(cudaEventRecord(cs->after_inputs, as_stream(stream)));
        B200_TRY(run_eager(cs, batch, stream, 2));
        return run_outputs(cs, batch, stream);
    }
    // Graph mode: the first run at a batch size is eager (plans build their tensor maps and scratch
    // then), the second is captured, later ones replay the captured launches back to back.
    cudaStream_t cst = as_stream(stream);
    b200_case::Graph *gr = nullptr;
    for (auto &g0 : cs->graphs)
        if (g0.batch == batch && g0.stream == cst)
            gr = &g0;
    if (!gr) {
        cs->graphs.push_back({ batch, cst, 0, nullptr });
        gr = &cs->graphs.back();
    }
    // the input layout kernels stay outside the graph: a pipelined caller refills the input staging
    // buffer as soon as they are done (b200_case_submit_host)
    if (gr->exec) {
        B200_TRY(run_eager(cs, batch, stream, 1));
        if (cs->after_inputs)
            B200_CUDA_TRY(cudaEventRecord(cs->after_inputs, cst));
        B200_CUDA_TRY(cudaGraphLaunch(gr->exec, cst));
        return run_outputs(cs, batch, stream);
    }
    if (gr->runs_seen++ == 0) {
        B200_TRY(run_eager(cs, batch, stream, 1));
        if (cs->after_inputs)
            B200_CUDA_TRY(cudaEventRecord(cs->after_inputs, cst));
        B200_TRY(run_eager(cs, batch, stream, 2));
        return run_outputs(cs, batch, stream);
    }
    B200_TRY(run_eager(cs, batch, stream, 1));
    if (cs->after_inputs)
        B200_CUDA_TRY(cudaEventRecord(cs->after_inputs, cst));
    cudaGraph_t graph = nullptr;
    B200_CUDA_TRY(cudaStreamBeginCapture(cst, cudaStreamCaptureModeThreadLocal));
    int rc = run_eager(cs, batch, stream, 2);
    cudaError_t ce = cudaStreamEndCapture(cst, &graph);
    if (rc != B200_OK || ce != cudaSuccess || !graph) {
        if (graph)
            cudaGraphDestroy(graph);
        cudaGetLastError();
        cs->use_graph = false;   // something on the path cannot be captured: stay eager
        if (rc != B200_OK)
            return rc;
        B200_TRY(run_eager(cs, batch, stream, 2));
        return run_outputs(cs, batch, stream);
    }
    ce = cudaGraphInstantiate(&gr->exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ce != cudaSuccess) {
        gr->exec = nullptr;
        cudaGetLastError();
        cs->use_graph = false;
        B200_TRY(run_eager(cs, batch, stream, 2));
        return run_outputs(cs, batch, stream);
    }
    B200_CUDA_TRY(cudaGraphLaunch(gr->exec, cst));
    return run_outputs(cs, batch, stream);
}

static int run_eager(b200_case_t *cs, int32_t batch, b200_stream_t stream, int phase)
{
    const bool prof = cs->profiling && phase == 0;
    size_t ev = 0;
    cudaStream_t cst = as_stream(stream);
    if (prof) {
        cs->kinds.clear();
        B200_CUDA_TRY(cudaEventRecord(cs->events[ev++], cst));
    }
    auto mark = [&](int kind) -> int {
        if (prof) {
            cs->kinds.push_back(kind);
            B200_CUDA_TRY(cudaEventRecord(cs->events[ev++], cst));
        }
        return B200_OK;
    };
    // phase 0: everything; 1: the input layout kernels; 2: the ops; 3: the output kernels
    for (auto &io : cs->inputs) {
        if (phase >= 2)
            break;
        CaseTensor &t = cs->tensors[io.tensor];
        if (io.is_f32)
            B200_TRY(b200_quantize_u8(
                (const float *)io.staging, t.dev, batch, t.c, t.h, t.w, io.alpha, io.zp, io.bits, 1, stream));
        else
            B200_TRY(b200_nchw_to_nhwc_u8(
                (const uint8_t *)io.staging, t.dev, batch, t.c, t.h, t.w, t.c_phys, 0, stream));
        B200_TRY(mark(0));
    }
    if (phase == 1)
        return B200_OK;
    for (auto &op : cs->ops) {
        int kind = 0;
        if (phase == 3)
            break;
        if (op.skipped)
            continue;
        CaseTensor &to = cs->tensors[op.out];
        const CaseTensor &ti = cs->tensors[op.ins[0]];
        switch (op.kind) {
        case OpKind::Conv:
            if (op.residual >= 0)
                B200_TRY(b200_conv2d_run_residual(op.conv, ti.dev, batch, cs->tensors[op.residual].dev, to.dev, stream));
            else
                B200_TRY(b200_conv2d_run(op.conv, ti.dev, batch, to.dev, stream));
            kind = b200_conv2d_algo(op.conv) == B200_CONV_ALGO_IGEMM ? 1 : 2;
            break;
        case OpKind::Eltwise: {
            const uint8_t *xs[4];
            for (size_t i = 0; i < op.ins.size(); ++i)
                xs[i] = cs->tensors[op.ins[i]].dev;
            B200_TRY(eltwise_launch(op.elt, op.elt_fast, xs, to.dev, to.bytes_per_image() * batch, op.reverse, as_stream(stream)));
            kind = 3;
            break;
        }
        case OpKind::Relu:
            B200_TRY(lut_u8_launch(ti.dev, to.dev, to.bytes_per_image() * batch, op.lut_dev, as_stream(stream)));
            kind = 4;
            break;
        case OpKind::Pool:
            B200_TRY(pool_launch(ti.dev, to.dev, batch, ti.c_phys, op.method, op.pg, op.lut_dev, op.ptab, as_stream(stream)));
            kind = 5;
            break;
        }
        B200_TRY(mark(kind));
    }
    for (auto &io : cs->outputs) {
        if (phase == 2)
            break;
        const CaseTensor &t = cs->tensors[io.tensor];
        if (io.is_f32)
            B200_TRY(b200_dequantize_u8(t.dev, (float *)io.staging, batch, t.c, t.h, t.w, io.alpha, io.zp, 1, stream));
        else
            B200_TRY(b200_nhwc_to_nchw_u8(t.dev, (uint8_t *)io.staging, batch, t.c, t.h, t.w, t.c_phys, stream));
        B200_TRY(mark(6));
    }
    if (prof) {
        cs->last_stream = cst;
        cs->have_profile = true;
    }
    return B200_OK;
}

int b200_case_set_fusion(b200_case_t *cs, int32_t enable)
{
    B200_TRY(check_building(cs, "case_set_fusion"));
    cs->fuse = enable != 0;
    return B200_OK;
}

int b200_case_use_graph(b200_case_t *cs, int32_t enable)
{
    if (!cs)
        return fail(B200_ERR_INVALID, "case_use_graph: NULL argument");
    cs->use_graph = enable != 0;
    return B200_OK;
}

int b200_case_set_profiling(b200_case_t *cs, int32_t enable)
{
    if (!cs || !cs->prepared)
        return fail(B200_ERR_INVALID, "case_set_profiling: the case is not prepared");
    if (enable && cs->events.empty()) {
        size_t n = cs->inputs.size() + cs->ops.size() + cs->outputs.size() + 1;
        for (size_t i = 0; i < n; ++i) {
            cudaEvent_t e;
            B200_CUDA_TRY(cudaEventCreate(&e));
            cs->events.push_back(e);
        }
    }
    cs->profiling = enable != 0;
    cs->have_profile = false;
    return B200_OK;
}

int b200_case_profile(b200_case_t *cs, float *ms_per_launch, int32_t *kinds, int32_t capacity, int32_t *count)
{
    if (!cs || !ms_per_launch || !kinds || !count)
        return fail(B200_ERR_INVALID, "case_profile: NULL argument");
    if (!cs->have_profile)
        return fail(B200_ERR_INVALID, "case_profile: no profiled run yet");
    B200_CUDA_TRY(cudaStreamSynchronize(cs->last_stream));
    const int n = (int)cs->kinds.size();
    *count = n;
    if (capacity < n)
        return fail(B200_ERR_INVALID, "case_profile: capacity %d < %d launches", capacity, n);
    for (int i = 0; i < n; ++i) {
        B200_CUDA_TRY(cudaEventElapsedTime(&ms_per_launch[i], cs->events[i], cs->events[i + 1]));
        kinds[i] = cs->kinds[i];
    }
    return B200_OK;
}

int b200_case_run_host(
    b200_case_t *cs, int32_t batch, const void *const *inputs, void *const *outputs,
    b200_stream_t stream)
{
    if (!cs || !cs->prepared)
        return fail(B200_ERR_INVALID, "case_run_host: the case is not prepared");
    if (!inputs || !outputs)
        return fail(B200_ERR_INVALID, "case_run_host: NULL argument");
    if (batch < 0 || batch > cs->max_batch)
        return fail(B200_ERR_INVALID, "case_run_host: batch %d outside 0..%d", batch, cs->max_batch);
    for (size_t i = 0; i < cs->inputs.size(); ++i)
        B200_TRY(b200_memcpy_h2d(cs->inputs[i].staging, inputs[i], cs->inputs[i].bytes_per_image * batch, stream));
    B200_TRY(b200_case_run_device(cs, batch, stream));
    for (size_t i = 0; i < cs->outputs.size(); ++i)
        B200_TRY(b200_memcpy_d2h(outputs[i], cs->outputs[i].staging, cs->outputs[i].bytes_per_image * batch, stream));
    B200_TRY(b200_stream_synchronize(stream));
    int word = 0;
    B200_TRY(b200_device_status(stream, &word));
    if (word != 0)
        return fail(B200_ERR_DEVICE_WAIT, "case_run_host: a device-side wait ran out (code 0x%x)", word);
    return B200_OK;
}

int b200_case_submit_host(b200_case_t *cs, int32_t batch, const void *const *inputs, void *const *outputs)
{
    if (!cs || !cs->prepared)
        return fail(B200_ERR_INVALID, "case_submit_host: the case is not prepared");
    if (!inputs || !outputs)
        return fail(B200_ERR_INVALID, "case_submit_host: NULL argument");
    if (batch < 0 || batch > cs->max_batch)
        return fail(B200_ERR_INVALID, "case_submit_host: batch %d outside 0..%d", batch, cs->max_batch);
    if (!cs->copy_stream) {
        B200_CUDA_TRY(cudaStreamCreateWithFlags(&cs->copy_stream, cudaStreamNonBlocking));
        B200_CUDA_TRY(cudaStreamCreateWithFlags(&cs->comp_stream, cudaStreamNonBlocking));
        B200_CUDA_TRY(cudaEventCreateWithFlags(&cs->h2d_done, cudaEventDisableTiming));
        B200_CUDA_TRY(cudaEventCreateWithFlags(&cs->after_inputs, cudaEventDisableTiming));
        B200_CUDA_TRY(cudaStreamCreateWithFlags(&cs->out_stream, cudaStreamNonBlocking));
        B200_CUDA_TRY(cudaEventCreateWithFlags(&cs->comp_done, cudaEventDisableTiming));
        B200_CUDA_TRY(cudaEventCreateWithFlags(&cs->d2h_done, cudaEventDisableTiming));
    }
    // the input staging buffer is free again once the previous run's layout kernels have read it
    if (cs->submitted)
        B200_CUDA_TRY(cudaStreamWaitEvent(cs->copy_stream, cs->after_inputs, 0));
    for (size_t i = 0; i < cs->inputs.size(); ++i)
        B200_CUDA_TRY(cudaMemcpyAsync(
            cs->inputs[i].staging, inputs[i], cs->inputs[i].bytes_per_image * batch, cudaMemcpyHostToDevice, cs->copy_stream));
    B200_CUDA_TRY(cudaEventRecord(cs->h2d_done, cs->copy_stream));
    B200_CUDA_TRY(cudaStreamWaitEvent(cs->comp_stream, cs->h2d_done, 0));
    B200_TRY(b200_case_run_device(cs, batch, reinterpret_cast<b200_stream_t>(cs->comp_stream)));
    // the results leave on a stream of their own, so that the next step's kernels do not queue behind the copy
    B200_CUDA_TRY(cudaEventRecord(cs->comp_done, cs->comp_stream));
    B200_CUDA_TRY(cudaStreamWaitEvent(cs->out_stream, cs->comp_done, 0));
    for (size_t i = 0; i < cs->outputs.size(); ++i)
        B200_CUDA_TRY(cudaMemcpyAsync(
            outputs[i], cs->outputs[i].staging, cs->outputs[i].bytes_per_image * batch, cudaMemcpyDeviceToHost, cs->out_stream));
    B200_CUDA_TRY(cudaEventRecord(cs->d2h_done, cs->out_stream));
    cs->submitted = true;
    return B200_OK;
}

int b200_case_wait(b200_case_t *cs)
{
    if (!cs)
        return fail(B200_ERR_INVALID, "case_wait: NULL argument");
    if (!cs->comp_stream)
        return B200_OK;
    B200_CUDA_TRY(cudaStreamSynchronize(cs->copy_stream));
    B200_CUDA_TRY(cudaStreamSynchronize(cs->comp_stream));
    B200_CUDA_TRY(cudaStreamSynchronize(cs->out_stream));
    int word = 0;
    B200_TRY(b200_device_status(reinterpret_cast<b200_stream_t>(cs->comp_stream), &word));
    if (word != 0)
        return fail(B200_ERR_DEVICE_WAIT, "case_wait: a device-side wait ran out (code 0x%x)", word);
    return B200_OK;
}

int b200_case_launch_count(const b200_case_t *cs, int32_t *launches)
{
    if (!cs || !launches)
        return fail(B200_ERR_INVALID, "case_launch_count: NULL argument");
    int n = (int)(cs->inputs.size() + cs->ops.size() + cs->outputs.size());
    for (const auto &op : cs->ops) {
        if (op.conv && op.conv->lowered)
            ++n;   // the row-lowering kernel runs ahead of the convolution kernel
        if (op.skipped)
            --n;   // an eltwise op that runs inside a conv's epilogue
    }
    *launches = n;
    return B200_OK;
}

}  // extern "C"
