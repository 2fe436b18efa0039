// Internal interfaces between the translation units of libnart_b200: prepared descriptors and
// launchers that the flat C-ABI calls and the case runner share.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

#include "nart_b200.h"

namespace b200 {

// ---- pool -----------------------------------------------------------------------------------
struct PoolGeom {
    int n, c, h, w, oh, ow;
    int kernel_h, kernel_w, pad_h, pad_w, stride_h, stride_w;
    int izp, ozp, qmax;
    int lut_identity;   // MAX: the requantize table maps every byte to itself (equal scales and zero points)
};
struct PoolAvgTab {
    static constexpr int kMax = 4;
    int mult[kMax][kMax];
    int shift[kMax][kMax];
};
int pool_prepare(
    int h, int w, int method, int kernel_h, int kernel_w, int pad_h, int pad_w, int stride_h,
    int stride_w, int ceil_mode, float ialpha, uint8_t izp, float oalpha, uint8_t ozp,
    uint8_t obits, PoolGeom *g, uint8_t lut[256], PoolAvgTab *tab);
int pool_launch(
    const uint8_t *x, uint8_t *y, int n, int c, int method, const PoolGeom &g, const uint8_t *lut_dev,
    const PoolAvgTab &tab, cudaStream_t st);

// ---- relu -----------------------------------------------------------------------------------
int relu_build_lut(
    float ialpha, uint8_t izp, float oalpha, uint8_t ozp, uint8_t obits, uint8_t lut[256]);
int lut_u8_launch(const uint8_t *x, uint8_t *y, size_t count, const uint8_t *lut_dev, cudaStream_t st);

// ---- eltwise SUM ----------------------------------------------------------------------------
// Arithmetic of eltwise.c:137-174 of the reference in the form the kernels use: per input i
// term_i = (x_i * m[i] + add[i]) >> b[i] (add[i] = 2^(b[i]-1) - zp_i * m[i]); t = sum term_i;
// y = sat_u(((t + round0) >> s0) + ozp), floored at relu_lo.
constexpr int kMaxEltIn = 4;
struct EltwiseArgs {
    const uint8_t *x[kMaxEltIn];
    int m[kMaxEltIn];
    int add[kMaxEltIn];
    int b[kMaxEltIn];
    int n_in;
    int rev;       // 1: tiles from the last to the first (see conv_igemm_set_reverse)
    int s0;        // final shift (>= 1)
    int round0;    // 2^(s0-1)
    int ozp, qmax, relu_lo;
};
int eltwise_prepare(
    int n_in, const float *ialpha, const uint8_t *izp, const float *coeff, float oalpha, uint8_t ozp,
    uint8_t obits, int relu, EltwiseArgs *out, bool *fast_out);
// Launches the prepared op on `count` bytes per input; reverse != 0 walks the tiles from the last to the first.
int eltwise_launch(const EltwiseArgs &prepared, bool fast, const uint8_t *const *xs, uint8_t *y, size_t count, int reverse,
                   cudaStream_t st);

// ---- conv -----------------------------------------------------------------------------------
// Geometry and quantization of one prepared convolution, shared by both kernels.
struct ConvGeom {
    int c, h, w, k, r, s;
    int pad_h, pad_w, stride_h, stride_w, group;
    int oh, ow;
    int izp, ozp, qmax, relu_lo;
    // Weight zero point minus 128.  The kernels multiply by s8 = stored weight - 128; for wzp != 128
    //   sum (x - izp) * (w - wzp) = sum (x - izp) * s8  -  wzp_d * sum_valid (x - izp),
    // and the second sum (over the window's in-image taps and the group's channels) is formed beside
    // the products (CUDA-core kernels) or read from a window-sum tensor (tensor-core kernel).
    int wzp_d;
    // int8 activations (the reference's dtINT8 path).  An int8 value v and the byte v ^ 0x80 = v + 128
    // are the same number seen with zero point 128, so the plan is the uint8 one with izp = 128,
    // int8 weights (wzp_d = 0), ozp = 128, floor 128 - m and ceiling qmax = 128 + m for the symmetric
    // clip at +-m; the kernels flip bit 7 of every input byte they load (or let the tensor cores read the
    // bytes as signed) and of every output byte they store.
    int act_signed;
    int s8_wrap;    // obits == 8 on that path: clip at +-255, then keep the low byte (CUDA-core kernel only)
};

// Direct (CUDA-core) convolution: weights [k][r][s][cg4] int8 (cg4 = c/group rounded up to 4,
// zero filled), bias_fold[k] = bias[k] - izp * sum(w[k]) so that out-of-image taps, read as izp,
// contribute nothing.
struct ConvDirectPlan {
    int8_t *w_dev = nullptr;
    int8_t *w_dw_dev = nullptr;   // depthwise only: [r][s][c] int8
    // depthwise 3x3 with every requantize shift >= 33 and 8-bit output: weights as dp4a words
    // [c/4][3 tap groups][4 channels] (taps 0-3, 4-7, 8 of one channel per word) and per channel
    // {folded 64-bit addend, mult, shift - 32}
    uint32_t *w_dw3_dev = nullptr;
    int4 *q_dw3_dev = nullptr;
    // the same for two output pixels side by side (stride_w 1 or 2), see conv_depthwise3x3_pair_kernel:
    // [c/4][3 kernel rows][2 or 3][4 channels] words of one kernel row against 3 + stride_w input pixels
    uint32_t *w_dw3p_dev = nullptr;
    int32_t *bias_fold_dev = nullptr;
    uint32_t *mult_dev = nullptr;
    int32_t *shift_dev = nullptr;
    int cg4 = 0;
};
int conv_direct_launch(
    const ConvGeom &g, const ConvDirectPlan &p, const uint8_t *x, int n, uint8_t *y, int32_t *acc_out,
    cudaStream_t st);

// Row lowering of a 4-channel NHWC image: out[n][ih][ow][j*4 + c] = x[n][ih][ow*stride_w - pad_w + j][c]
// for j < kLowerWindow, the byte izp where the pixel lies outside the image.  The two 16-byte
// halves of an output pixel are stored swapped when bit 2 of ow is set: that is the 32-byte
// shared-memory swizzle, applied in global memory, so that the tensor-core kernel can fetch whole
// rows of pixels with wide unswizzled copies (see conv_igemm_create, a_row_swizzled).
constexpr int kLowerWindow = 8;
int conv_lower_rows_launch(const ConvGeom &g, const uint8_t *x, int n, uint8_t *out, cudaStream_t st);

// Window sums for a weight zero point other than 128 (group == 1): csum[n][h][w] = sum_c x, then
// wsum[n][oh][ow] = sum over the window's in-image taps of (csum - izp * c).  Both int32.
int conv_window_sum_launch(const ConvGeom &g, const uint8_t *x, int n, int32_t *csum, int32_t *wsum, cudaStream_t st);

// Implicit-GEMM (tcgen05) convolution plan; defined in conv_igemm_sm100.cu.
struct ConvIgemmPlan;
int conv_igemm_supported(const ConvGeom &g, char *why, size_t why_len);
int conv_igemm_create(
    const ConvGeom &g, const std::vector<int8_t> &w_s8 /* [k][c][r][s] */, const int32_t *bias,
    const uint32_t *mult, const int32_t *shift, ConvIgemmPlan **plan, bool a_row_swizzled = false);
// a_row_swizzled: the activation tensor has 32 channels, the kernel is r x 1 with no horizontal
// stride or padding, and the tensor was written by conv_lower_rows_launch (halves swapped by ow bit 2).
// status_word: device int that a bounded wait writes its code into; nullptr = the per-device word
// that b200_device_status reads.
// res: the second input of a fused residual add (conv_igemm_set_residual), else nullptr.
// wsum: the window sums of conv_window_sum_launch when the plan's geometry has wzp_d != 0, else nullptr.
int conv_igemm_launch(ConvIgemmPlan *plan, const uint8_t *x, int n, uint8_t *y, cudaStream_t st,
                      int *status_word = nullptr, const uint8_t *res = nullptr, const int32_t *wsum = nullptr);
// Fuses y = eltwise_sum(conv(x), res) into the epilogue: `e` holds the eltwise constants and
// conv_input says which of its two inputs is this conv's output.  B200_ERR_UNSUPPORTED when the
// plan's epilogue form cannot take it (the caller then keeps the separate eltwise kernel).
int conv_igemm_set_residual(ConvIgemmPlan *plan, const EltwiseArgs &e, int conv_input);
void conv_igemm_destroy(ConvIgemmPlan *plan);
// Direction in which a launch walks its output tiles: 0 first to last, 1 last to first.  Results do not
// depend on it; a consumer that walks against its producer's direction starts on data still in L2.
void conv_igemm_set_reverse(ConvIgemmPlan *plan, int reverse);
// The repacked weights of a plan (device pointer, bytes), and the read-only operand of the launch that follows this
// plan's: the kernel asks for it to be brought into L2 while it runs (nullptr: none).
void conv_igemm_weights(const ConvIgemmPlan *plan, const uint8_t **ptr, size_t *bytes);
void conv_igemm_set_next_readonly(ConvIgemmPlan *plan, const uint8_t *ptr, size_t bytes);
// One line of text naming the plan's tiling and kernel variant.
void conv_igemm_describe(const ConvIgemmPlan *plan, char *buf, size_t len);
// Per-process / per-device set-up of the tensor-core kernels (driver entry point, shared-memory
// attribute): done by the first launch otherwise; plan creation calls it so that runs do not.
int conv_igemm_warm();
// Times `mmas_per_sm` back-to-back kind::i8 M128 x N256 x K32 MMAs on every SM (operands resident in shared
// memory); *ops is the number of integer operations (2 per multiply-add) the launch performed.
int mma_i8_peak_launch(int mmas_per_sm, float *ms, double *ops, cudaStream_t st);
// Launches the one-warp kernel whose bounded wait cannot be satisfied (see b200_selftest_wait_expiry).
int wait_expiry_probe_launch(long long limit_cycles, cudaStream_t st);
// Resolves the device address of the static scratch array for the current device (conv_static_scratch.cu).
int conv_static_scratch_prepare();

}  // namespace b200

// A prepared convolution (the handle of the C-ABI).
struct b200_conv {
    b200::ConvGeom g;
    int algo = B200_CONV_ALGO_DIRECT;
    int device = 0;
    b200::ConvDirectPlan direct;
    b200::ConvIgemmPlan *igemm = nullptr;
    // Row lowering of 4-channel inputs (the image stem): the igemm plan then runs on `g_low`, and
    // its activation operand is a scratch tensor the lowering kernel fills on every run.
    bool lowered = false;
    b200::ConvGeom g_low;
    uint8_t *scratch = nullptr;     // [n][h][ow][32]
    size_t scratch_bytes = 0;
    int32_t *sums = nullptr;        // wzp != 128 on the tensor-core path: [n][h][w] channel sums, then [n][oh][ow] window sums
    size_t sums_images = 0;         // images the two tensors hold
    float oalpha = 0.f;             // output scale, kept for b200_conv2d_fuse_residual_add
    bool fused_residual = false;    // the plan computes eltwise_sum(conv(x), res)
};
