/*
 * nart_b200 -- C-ABI of the Blackwell (sm_100a) backend for the quantized-convolution path of
 * NART's art runtime.
 *
 * Everything here is `extern "C"`, takes plain pointers, sizes and POD structs and returns an
 * int status (0 = B200_OK, negative = error; b200_last_error() gives the detail).  Nothing
 * aborts.  The art-facing module (nart_b200/module/, C) and the Python host mirror (nart_b200/)
 * sit on top of exactly these entry points.
 *
 * Each entry point names the reference interface it stands in for, as file:line inside the
 * reference project (ModelTC/NART).  The reference's per-op contract is
 * `op_tp_entry_t { alloc, config, destroy, dealloc, prepare }` + `op->run_func`
 * (art/include/art/op.h:114-143): `*_create` here does the work of config + prepare (it is the
 * only place weights are repacked and tables built), `*_run` is run_func, `*_destroy` is
 * destroy + dealloc.
 *
 * Data layout.  Activations on the device are NHWC uint8 (`[N][H][W][C]`, C contiguous), the
 * layout the reference's own GPU quant module keeps under NCHW shapes
 * (art/modules/cuda_quant/src/op/quantize.cu, python/nart/modules/cuda_quant.py:182-186).
 * Host-facing tensors (weights, bias, case inputs/outputs) are in the reference's NCHW / OIHW
 * layout (art/modules/quant).  int8 weights are passed the way the reference quant module stores
 * them: uint8 = value + 128 with wzp = 128 (python/nart/modules/quant.py:53-58).
 *
 * Arithmetic is the reference CPU quant module's integer arithmetic, bit for bit
 * (art/modules/quant/include/art/quant/quant_helper.h:29-118).
 */
#ifndef NART_B200_H
#define NART_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define B200_API __attribute__((visibility("default")))
#else
#define B200_API
#endif

/* ---- status ------------------------------------------------------------------------------
 * The reference has no error returns: CHECK -> abort(), LOG_error -> exit(-1)
 * (art/include/art/log.h:29-34,82-101).  The module layer turns a non-zero status into that
 * convention; this layer never kills the process. */
#define B200_OK 0
#define B200_ERR_INVALID (-1)       /* a bad argument or an inconsistent descriptor          */
#define B200_ERR_UNSUPPORTED (-2)   /* valid in the reference, not implemented on this path  */
#define B200_ERR_CUDA (-3)          /* a CUDA runtime/driver call failed                     */
#define B200_ERR_NOMEM (-4)
#define B200_ERR_DEVICE_WAIT (-5)   /* a bounded wait inside a kernel ran out (see status word) */

B200_API const char *b200_strerror(int status);
/* Detail text of the last failure on the calling thread ("" if none). */
B200_API const char *b200_last_error(void);
B200_API int b200_version(void);

/* ---- device, memory, streams ---------------------------------------------------------------
 * Stand in for the device workspace + mem type of a GPU module:
 * workspace new/delete with a device id (art/modules/cuda_quant/src/cuda_quant_module.c:98-141)
 * and the mem_tp vtable alloc/free/copy_from_cpu/copy_to_cpu (art/include/art/mem.h:48-64,
 * art/modules/cuda_quant/src/cuda_quant_mem.cpp:25-123).  A stream is an opaque handle; NULL
 * means the CUDA default stream, as the reference GPU modules use. */
typedef void *b200_stream_t;

B200_API int b200_device_count(int *count);
B200_API int b200_set_device(int device);
B200_API int b200_get_device(int *device);
B200_API int b200_malloc(void **dev_ptr, size_t bytes);
B200_API int b200_free(void *dev_ptr);
B200_API int b200_malloc_host(void **host_ptr, size_t bytes); /* pinned */
B200_API int b200_free_host(void *host_ptr);
B200_API int b200_memset(void *dev_ptr, int value, size_t bytes, b200_stream_t stream);
B200_API int b200_memcpy_h2d(void *dev_dst, const void *host_src, size_t bytes, b200_stream_t stream);
B200_API int b200_memcpy_d2h(void *host_dst, const void *dev_src, size_t bytes, b200_stream_t stream);
B200_API int b200_memcpy_d2d(void *dev_dst, const void *dev_src, size_t bytes, b200_stream_t stream);
B200_API int b200_stream_create(b200_stream_t *stream);
B200_API int b200_stream_destroy(b200_stream_t stream);
B200_API int b200_stream_synchronize(b200_stream_t stream);
/* Reads and clears the device status word that kernels with bounded waits write when a wait
 * runs out (0 = none did).  Synchronizes `stream` first. */
B200_API int b200_device_status(b200_stream_t stream, int *status_word);

/* Exercises the give-up path of the bounded device-side waits without a fault: launches a one-warp
 * kernel that waits, through the very wait routine the convolution kernel's roles use, on a barrier
 * nothing arrives at.  After `limit_cycles` SM clock cycles (1 .. 2e9, i.e. at most about a second)
 * the wait gives up, the kernel records code 0x1ff in the device status word and returns normally;
 * the next b200_device_status then reads 0x1ff, and b200_case_run_host / b200_case_wait report
 * B200_ERR_DEVICE_WAIT.  The context stays usable.  The reference has no counterpart: its GPU
 * modules have no device-side waits (art/modules/cuda_quant/src/cuda_quant_workspace.c). */
B200_API int b200_selftest_wait_expiry(uint64_t limit_cycles, b200_stream_t stream);

/* The tensor pipe's dense int8 rate on this GPU, measured: every SM issues `mmas_per_sm` back-to-back
 * tcgen05 kind::i8 MMAs of M128 x N256 x K32 on operands resident in shared memory -- the convolution
 * kernel's instruction without its loads and its epilogue.  *ms is the launch's device time (CUDA
 * events on `stream`, which the call synchronizes), *ops the integer operations performed (2 per
 * multiply-add); ops / ms is the ceiling the convolution's TOP/s are compared with.  A few thousand
 * MMAs give the burst rate, a second or more of them the rate under the power cap.  No counterpart in
 * the reference. */
B200_API int b200_measure_mma_i8_peak(int32_t mmas_per_sm, float *ms, double *ops, b200_stream_t stream);

/* ---- scale decomposition -------------------------------------------------------------------
 * get_quant_scale_int32 / get_quant_scale_int16 / get_quant_scale
 * (art/modules/quant/include/art/quant/quant_helper.h:60-118): `bits` 32, -16 (the uint16
 * variant) or the generic bit count.  Host-only; the results feed every kernel's tables. */
B200_API void b200_get_quant_scale(float x, int bits, uint32_t *mult, int8_t *shift);

/* ---- conv_2d --------------------------------------------------------------------------------
 * op_quant_conv_2d_tp_{config,prepare} + op_conv_2d_u8xu8_run
 * (art/modules/quant/src/op/conv_2d.c:27-147, conv_2d_uint8_impl.c:39-165):
 *   acc = bias[k] + sum (x - izp) * (w - wzp), zero outside the image;
 *   y   = sat_u(rshift_rn(acc * mult_k, shift_k) + ozp, obits), then max(y, ozp) if relu.
 * n_walpha is 1 (the reference's per-tensor scale) or k (one scale per output channel, each
 * decomposed by the same function).  relu follows the fused flag of the reference GPU module
 * (SETTING_CONV_2D_RELU_FLAG, art/modules/cuda_quant/src/op/conv_2d_quant.cu:793-794) with the
 * CPU module's relu arithmetic (art/modules/quant/src/op/relu.c:76-115, equal in/out scale). */
/* Tuning switches of the tensor-core plan, read from the environment by b200_conv2d_create (all
 * optional; a value a plan cannot honour is ignored; results never change, only speed):
 *   B200_IGEMM_BN=<16..256, multiple of 16>  output channels per tile
 *   B200_IGEMM_GROUPS=<2|4>                  epilogue groups (4 needs four accumulators in tensor memory)
 *   B200_IGEMM_ACC=<2|4>                     accumulator stages in tensor memory
 *   B200_IGEMM_KGROUP=<1..10>                k-blocks per pipeline stage (must divide a tile's k-blocks)
 *   B200_IGEMM_MMA_WARPS=<1|2>               MMA-issuing warps
 *   B200_IGEMM_PAIR=0                        never pair tiles on one weight tile
 *   B200_IGEMM_CTA_PAIR=<0|1>                never / wherever possible run on CTA pairs (tcgen05 cta_group::2)
 *   B200_IGEMM_EPI_CONST=0                   never use the uniform-shift epilogue (per-channel constants as kernel parameters)
 * and by b200_case_prepare:
 *   B200_CASE_ZIGZAG=0                       every op walks its tiles first to last (default: each op walks against the
 *                                            direction of the op that wrote its input, to start on what is still in L2)
 *   B200_CASE_PREFETCH=0                     no L2 prefetch of the next conv's weights while a conv runs (default: every
 *                                            tensor-core conv of a case asks for the following one's repacked weights) */
/* Activation type.  B200_ACT_S8 is the reference's dtINT8 path -- op_conv_2d_i8xi8_run
 * (art/modules/quant/src/op/conv_2d_int8_impl.c:34-174), dispatched on the dtype of input 0
 * (conv_2d.c:114-142): activations, weights and outputs are int8, there are no zero points
 * (izp / wzp / ozp are ignored), `weights` points at int8 values, and
 *   y = ssaturate_int_by_bits(rshift_rn(acc * mult_k, shift_k), obits)     (quant_helper.h:43-47)
 * which clips to +-(2^obits - 1) and then narrows to int8.  For obits <= 7 that is a plain clip.  For
 * obits == 8 -- what the reference's exporter writes for 8-bit tensors (python/nart/modules/
 * quant.py:47,200) -- the bound is +-255 and the narrowing wraps (200 becomes -56): such a plan is
 * refused unless s8_wrap is set, in which case it reproduces the wrap bit for bit on the CUDA-core
 * path.  relu != 0 floors the output at 0.  x and y of the run calls are then int8 NHWC tensors. */
#define B200_ACT_U8 0
#define B200_ACT_S8 1

#define B200_CONV_ALGO_AUTO 0
#define B200_CONV_ALGO_DIRECT 1 /* CUDA-core dp4a kernel: any group, any channel count   */
#define B200_CONV_ALGO_IGEMM 2  /* tcgen05 kind::i8 implicit GEMM: group 1, c % 16 == 0, k % 16 == 0 */

typedef struct b200_conv_params {
    int32_t c, h, w;        /* input channels and spatial size (batch is a run-time argument) */
    int32_t k, r, s;        /* output channels, kernel height and width                       */
    int32_t pad_h, pad_w, stride_h, stride_w, group;
    float ialpha;           /* SETTING_QUANT_IALPHA[0]                                        */
    uint8_t izp;            /* SETTING_QUANT_IZERO_POINT[0]                                   */
    uint8_t wzp;            /* SETTING_QUANT_WZERO_POINT[0]; 128 = int8 weights stored as value + 128.
                             * Other values cost one extra pass over the activations on the
                             * tensor-core path (window sums of x) and rule out the fused residual add */
    uint8_t ozp;            /* SETTING_QUANT_OZERO_POINT[0]                                   */
    uint8_t obits;          /* SETTING_QUANT_OBITS[0], 1..8                                   */
    float oalpha;           /* SETTING_QUANT_OALPHA[0]                                        */
    const float *walpha;    /* SETTING_QUANT_WALPHA, n_walpha entries (host)                  */
    int32_t n_walpha;       /* 1 or k                                                         */
    int32_t relu;           /* non-zero: clamp at ozp after requantize                        */
    int32_t algo;           /* B200_CONV_ALGO_*                                               */
    int32_t act_type;       /* B200_ACT_U8 (0, the default of a zeroed struct) or B200_ACT_S8 */
    int32_t s8_wrap;        /* B200_ACT_S8 only: accept obits == 8 with the reference's wrapping cast */
} b200_conv_params;

typedef struct b200_conv b200_conv_t;

/* weights: host, [k][c/group][r][s] uint8; bias: host int32[k] or NULL (= zeros). */
B200_API int b200_conv2d_create(
    const b200_conv_params *params, const uint8_t *weights, const int32_t *bias,
    b200_conv_t **conv);
B200_API int b200_conv2d_out_dims(const b200_conv_t *conv, int32_t *oh, int32_t *ow);
/* The algorithm the plan resolved to (B200_CONV_ALGO_DIRECT or _IGEMM). */
B200_API int b200_conv2d_algo(const b200_conv_t *conv);
/* One line of text naming the kernel variant and tiling the plan resolved to (for logs and tuning). */
B200_API int b200_conv2d_describe(const b200_conv_t *conv, char *buf, size_t len);
/* x: device NHWC [n][h][w][c]; y: device NHWC [n][oh][ow][k].  Plans with a scratch tensor (the
 * row-lowered 4-channel stem; window sums for wzp != 128) grow it, with a device synchronization,
 * the first time a larger batch arrives; the old tensor is freed then. */
B200_API int b200_conv2d_run(
    b200_conv_t *conv, const uint8_t *x, int32_t n, uint8_t *y, b200_stream_t stream);
/* Sizes the plan's scratch tensors for batches of up to n images now, so that no later run
 * allocates or frees (a CUDA graph captured from a run keeps the scratch address it saw).
 * No counterpart in the reference; a no-op for plans without scratch. */
B200_API int b200_conv2d_reserve(b200_conv_t *conv, int32_t n);
/* As b200_conv2d_run, also writing the int32 accumulators (bias included) as NHWC int32.
 * Debug/verification entry; always takes the CUDA-core path. */
B200_API int b200_conv2d_run_acc(
    b200_conv_t *conv, const uint8_t *x, int32_t n, uint8_t *y, int32_t *acc,
    b200_stream_t stream);
B200_API int b200_conv2d_destroy(b200_conv_t *conv);
/* No counterpart in the reference.  b200_conv2d_run for callers that must not allocate: a serving
 * loop that cannot afford the device-wide synchronization of cudaMalloc / cudaFree, or a host
 * application that has already given all device memory to its own pool, where an allocation made
 * from inside a plugin fails.  It applies to plans that use a scratch tensor -- the row-lowered
 * convs of 4-channel images (c == 4, group == 1, kernel width <= 8, k >= 16; any other plan is
 * refused with B200_ERR_INVALID) -- and keeps that tensor in a fixed 32 MiB device array inside
 * the library instead of growing one with cudaMalloc.  The call fails with B200_ERR_UNSUPPORTED
 * when n * h * ow * 32 bytes exceed 32 MiB (41 images of a 224x224 stride-2 stem).  It makes no
 * cudaMalloc / cudaFree, calls no allocating library routine and, once a given (x, y, n) has been
 * seen, touches no host heap either (the first call with a new (x, y, n) encodes tensor maps into
 * storage the plan reserved at creation).
 * - b200_conv2d_create of such a plan resolves the array's device address and does the kernels'
 *   one-time set-up on the device that is current then, so that this entry point has nothing left to
 *   set up there.  On any other device the first call does it: make that call during preparation,
 *   outside any stream capture.  Every GPU the array is resolved on holds the 32 MiB until the process exits.
 * - All calls on a device share the one array: two calls whose kernels overlap on the GPU (different
 *   streams, no dependency between them) race on it.  Calls on one stream are safe.
 * - A bounded device-side wait that runs out is recorded in the array's own status word, not in the
 *   one b200_device_status reads: check it with b200_static_scratch_status, which allocates nothing. */
B200_API int b200_conv2d_run_static_scratch(
    b200_conv_t *conv, const uint8_t *x, int32_t n, uint8_t *y, b200_stream_t stream);

/* No counterpart in the reference.  Synchronizes `stream`, copies the static scratch array's status
 * word (4 bytes) into *status_word and, if it is not zero, clears it and returns
 * B200_ERR_DEVICE_WAIT: some b200_conv2d_run_static_scratch call since the last check had a device-side
 * wait run out and its output is not valid.  B200_OK with *status_word == 0 otherwise. */
B200_API int b200_static_scratch_status(b200_stream_t stream, int *status_word);

/* Residual add fused into the conv (no such op in the reference's CPU module; its GPU module
 * fuses ReLU into conv and eltwise the same way, python/nart/modules/cuda_quant.py:300-330).
 * After b200_conv2d_fuse_residual_add the plan computes, in one kernel,
 *     y = eltwise_sum(conv(x), res)      -- op_quant_eltwise_accumulate_output_sum,
 *                                           art/modules/quant/src/op/eltwise.c:137-174
 * bit for bit as the two separate ops would: the conv's value is requantized and saturated to
 * uint8 first, then both inputs go through the eltwise integer formula.  conv_input (0 or 1) says
 * which eltwise input is the conv's output; ialpha / izp / coeff (NULL = all 1) are the eltwise
 * op's two-entry arrays in its own input order, ialpha[conv_input] and izp[conv_input] must be the
 * conv's oalpha and ozp.  Returns B200_ERR_UNSUPPORTED, leaving the plan unchanged, when the plan
 * cannot take it (not on the tensor-core path, output channels not a multiple of 32, obits != 8,
 * a requantize shift below 33): the caller then runs b200_eltwise_sum_u8 as a separate step.
 * A fused plan runs only through b200_conv2d_run_residual (res: NHWC, the dims of y). */
B200_API int b200_conv2d_fuse_residual_add(
    b200_conv_t *conv, int32_t conv_input, const float *ialpha, const uint8_t *izp,
    const float *coeff, float oalpha, uint8_t ozp, uint8_t obits, int32_t relu);
B200_API int b200_conv2d_run_residual(
    b200_conv_t *conv, const uint8_t *x, int32_t n, const uint8_t *res, uint8_t *y,
    b200_stream_t stream);

/* ---- ip (fully connected) -------------------------------------------------------------------
 * op_quant_ip_u8xu8_run (art/modules/quant/src/op/ip.cpp:133-209): a conv whose kernel covers
 * the whole c x h x w input.  weights: host [k][c*h*w] in the reference's flattened-NCHW column
 * order.  The returned plan is run with b200_conv2d_run (x NHWC [n][h][w][c], y [n][k]). */
B200_API int b200_ip_create(
    int32_t c, int32_t h, int32_t w, int32_t k, float ialpha, uint8_t izp, const float *walpha,
    int32_t n_walpha, uint8_t wzp, float oalpha, uint8_t ozp, uint8_t obits,
    const uint8_t *weights, const int32_t *bias, b200_conv_t **conv);

/* op_quant_ip_i8xi8_run (art/modules/quant/src/op/ip.cpp:210-274): the inner product on int8
 * activations and weights (see B200_ACT_S8).  weights: host int8 [k][c*h*w]. */
B200_API int b200_ip_create_s8(
    int32_t c, int32_t h, int32_t w, int32_t k, float ialpha, const float *walpha, int32_t n_walpha,
    float oalpha, uint8_t obits, int32_t s8_wrap, const int8_t *weights, const int32_t *bias,
    b200_conv_t **conv);

/* ---- quantize / dequantize ------------------------------------------------------------------
 * op_quantize_run_u8 (art/modules/quant/src/op/quantize.c:145-157) and op_dequantize_run_u8
 * (dequantize.c:111-123).  The float side is always NCHW (the reference's layout); the uint8
 * side is NHWC when `nhwc` is non-zero (the fused transpose of the reference GPU module,
 * art/modules/cuda_quant/src/utils/cuda_quant_helper.cu:196-373), else NCHW. */
B200_API int b200_quantize_u8(
    const float *x, uint8_t *y, int32_t n, int32_t c, int32_t h, int32_t w, float oalpha,
    uint8_t ozp, uint8_t obits, int32_t nhwc, b200_stream_t stream);
B200_API int b200_dequantize_u8(
    const uint8_t *x, float *y, int32_t n, int32_t c, int32_t h, int32_t w, float ialpha,
    uint8_t izp, int32_t nhwc, b200_stream_t stream);

/* op_quantize_run_i8 (quantize.c:159-185, qtype SYMMETRIC): y = clip(round(x * (float)(1. / oalpha)),
 * +-(2^(obits-1) - 1)), round half away from zero; and op_dequantize_run_i8 (dequantize.c:124-136):
 * y = (float)q * ialpha.  Layout arguments as for the uint8 pair. */
B200_API int b200_quantize_s8(
    const float *x, int8_t *y, int32_t n, int32_t c, int32_t h, int32_t w, float oalpha,
    uint8_t obits, int32_t nhwc, b200_stream_t stream);
B200_API int b200_dequantize_s8(
    const int8_t *x, float *y, int32_t n, int32_t c, int32_t h, int32_t w, float ialpha,
    int32_t nhwc, b200_stream_t stream);

/* ---- layout ---------------------------------------------------------------------------------
 * uint8 NCHW <-> NHWC, for tensors that cross the module boundary in the reference's layout.
 * c_pad >= c pads/strips trailing channels (written as `fill`), used for the 3-channel image
 * input. */
B200_API int b200_nchw_to_nhwc_u8(
    const uint8_t *x, uint8_t *y, int32_t n, int32_t c, int32_t h, int32_t w, int32_t c_pad,
    uint8_t fill, b200_stream_t stream);
B200_API int b200_nhwc_to_nchw_u8(
    const uint8_t *x, uint8_t *y, int32_t n, int32_t c, int32_t h, int32_t w, int32_t c_pad,
    b200_stream_t stream);

/* ---- eltwise SUM / add / relu ---------------------------------------------------------------
 * op_quant_eltwise_accumulate_output_sum (art/modules/quant/src/op/eltwise.c:137-174, tables
 * :241-252) and op_quant_add_run (add.c:83-148, the two-input case).  Layout-agnostic: `count`
 * bytes per input.  relu != 0 clamps at ozp (the reference GPU module's fused flag,
 * art/modules/cuda_quant/src/op/eltwise.cu:224-245).  n_in <= 4; xs is a host array of device
 * pointers. */
B200_API int b200_eltwise_sum_u8(
    const uint8_t *const *xs, int32_t n_in, size_t count, const float *ialpha, const uint8_t *izp,
    const float *coeff, float oalpha, uint8_t ozp, uint8_t obits, int32_t relu, uint8_t *y,
    b200_stream_t stream);
/* op_quant_relu_run (art/modules/quant/src/op/relu.c:76-115). */
B200_API int b200_relu_u8(
    const uint8_t *x, size_t count, float ialpha, uint8_t izp, float oalpha, uint8_t ozp,
    uint8_t obits, uint8_t *y, b200_stream_t stream);

/* ---- pool -----------------------------------------------------------------------------------
 * op_quant_pool_max_run / op_quant_pool_average_run (art/modules/quant/src/op/pool.c:96-249),
 * output extent by the reference's shape inference (art/src/op.c:903-967, b200_pool_out_dims).
 * method: 0 = MAX, 1 = AVE (SETTING_POOL_MAX / _AVE, art/include/art/op_settings.h:62-63).
 * x, y: device NHWC. */
B200_API int b200_pool_out_dims(
    int32_t h, int32_t w, int32_t kernel_h, int32_t kernel_w, int32_t pad_h, int32_t pad_w,
    int32_t stride_h, int32_t stride_w, int32_t ceil_mode, int32_t *oh, int32_t *ow);
B200_API int b200_pool_u8(
    const uint8_t *x, int32_t n, int32_t c, int32_t h, int32_t w, int32_t method, int32_t kernel_h,
    int32_t kernel_w, int32_t pad_h, int32_t pad_w, int32_t stride_h, int32_t stride_w,
    int32_t ceil_mode, float ialpha, uint8_t izp, float oalpha, uint8_t ozp, uint8_t obits,
    uint8_t *y, b200_stream_t stream);

/* ---- case (parade) --------------------------------------------------------------------------
 * A prepared, runnable op list bound to one device: what the reference calls a parade
 * (art/include/art/parade.h, art/src/parade.c:169-197 parade_prepare / parade_run), built
 * through calls instead of deserialized.  Tensors are named by the int ids these calls return.
 * Host-side tensors of a case (its inputs and outputs) are NCHW, as in the reference. */
typedef struct b200_case b200_case_t;

B200_API int b200_case_create(b200_case_t **cs);
B200_API int b200_case_destroy(b200_case_t *cs);
/* A uint8 NCHW input of c x h x w per image.  */
B200_API int b200_case_input_u8(b200_case_t *cs, int32_t c, int32_t h, int32_t w, int32_t *tensor);
/* A float32 NCHW input, quantized on the device by the op of b200_quantize_u8. */
B200_API int b200_case_input_f32(
    b200_case_t *cs, int32_t c, int32_t h, int32_t w, float oalpha, uint8_t ozp, uint8_t obits,
    int32_t *tensor);
/* params->c/h/w must match the input tensor. */
B200_API int b200_case_conv2d(
    b200_case_t *cs, int32_t in, const b200_conv_params *params, const uint8_t *weights,
    const int32_t *bias, int32_t *out);
B200_API int b200_case_ip(
    b200_case_t *cs, int32_t in, int32_t k, float ialpha, uint8_t izp, const float *walpha,
    int32_t n_walpha, uint8_t wzp, float oalpha, uint8_t ozp, uint8_t obits,
    const uint8_t *weights, const int32_t *bias, int32_t *out);
B200_API int b200_case_eltwise_sum(
    b200_case_t *cs, const int32_t *ins, int32_t n_in, const float *ialpha, const uint8_t *izp,
    const float *coeff, float oalpha, uint8_t ozp, uint8_t obits, int32_t relu, int32_t *out);
B200_API int b200_case_relu(
    b200_case_t *cs, int32_t in, float ialpha, uint8_t izp, float oalpha, uint8_t ozp,
    uint8_t obits, int32_t *out);
B200_API int b200_case_pool(
    b200_case_t *cs, int32_t in, int32_t method, int32_t kernel_h, int32_t kernel_w, int32_t pad_h,
    int32_t pad_w, int32_t stride_h, int32_t stride_w, int32_t ceil_mode, float ialpha,
    uint8_t izp, float oalpha, uint8_t ozp, uint8_t obits, int32_t *out);
/* Marks a uint8 tensor as a case output (returned NCHW uint8). */
B200_API int b200_case_output_u8(b200_case_t *cs, int32_t tensor);
/* Marks a uint8 tensor as a case output returned dequantized (NCHW float32). */
B200_API int b200_case_output_f32(b200_case_t *cs, int32_t tensor, float ialpha, uint8_t izp);
/* parade_prepare: allocates every device buffer for up to max_batch images. */
B200_API int b200_case_prepare(b200_case_t *cs, int32_t max_batch);
B200_API int b200_case_tensor_dims(
    const b200_case_t *cs, int32_t tensor, int32_t *c, int32_t *h, int32_t *w);
/* Bytes per image of the i-th input / output on the host side. */
B200_API int b200_case_io_bytes(
    const b200_case_t *cs, int32_t is_output, int32_t index, size_t *bytes_per_image);
/* Device staging buffer of the i-th input / output (host layout, NCHW), for callers that keep
 * data resident. */
B200_API int b200_case_io_device_ptr(
    const b200_case_t *cs, int32_t is_output, int32_t index, void **dev_ptr);
/* Device NHWC buffer of any tensor after a run (verification). */
B200_API int b200_case_tensor_device_ptr(const b200_case_t *cs, int32_t tensor, void **dev_ptr);
/* parade_run on data already resident in the input staging buffers; asynchronous on `stream`. */
B200_API int b200_case_run_device(b200_case_t *cs, int32_t batch, b200_stream_t stream);
/* parade_run with host buffers: copies every input host->device, runs, copies every output
 * device->host and synchronizes.  inputs[i] / outputs[i]: batch x bytes_per_image. */
B200_API int b200_case_run_host(
    b200_case_t *cs, int32_t batch, const void *const *inputs, void *const *outputs,
    b200_stream_t stream);
/* Pipelined form of b200_case_run_host for back-to-back batches: returns as soon as the work is
 * queued on the case's own copy and compute streams, so that the host->device copy of the next
 * batch overlaps the kernels of this one (the reference's drivers run parade_run and the copies
 * strictly one after the other, tools/promark.cpp:457-492).  The host buffers must be pinned and
 * stay valid -- and the outputs unread -- until b200_case_wait returns.  A later submit may reuse
 * the same host buffers only after a wait.  b200_case_wait also returns the bounded-wait status. */
B200_API int b200_case_submit_host(
    b200_case_t *cs, int32_t batch, const void *const *inputs, void *const *outputs);
B200_API int b200_case_wait(b200_case_t *cs);
/* Number of kernels one b200_case_run_device launches. */
B200_API int b200_case_launch_count(const b200_case_t *cs, int32_t *launches);
/* Folds residual adds into the convs that feed them (default: off; call before b200_case_prepare).
 * Off by default because on B200 the conv epilogue is bound by instruction issue, not by memory:
 * ResNet-50 at batch 256 runs 3.43 ms per step fused against 3.23 ms with the adds as kernels of
 * their own, although the fused form moves 2.7 GB less.
 * A two-input eltwise SUM whose later-produced input is the output of a tensor-core conv that
 * nothing else reads then runs in that conv's epilogue (b200_conv2d_fuse_residual_add) and its own
 * kernel is skipped; results are unchanged.  No counterpart in the reference's CPU module, whose
 * parade runs every op as its own pass (art/src/parade.c:184-197). */
B200_API int b200_case_set_fusion(b200_case_t *cs, int32_t enable);
/* Replays b200_case_run_device as one CUDA graph per (batch, stream) instead of launching op by op
 * (the reference's parade_run loop, art/src/parade.c:184-197, launches one op at a time): the first
 * run at a batch size is eager, the second is captured, later ones replay.  Off by default; ignored
 * while profiling is on and on the default (NULL) stream, which cannot be captured.  The buffers of a
 * case never move, so a captured graph stays valid. */
B200_API int b200_case_use_graph(b200_case_t *cs, int32_t enable);
/* Per-op device timing, the counterpart of the reference's per-op profiler pointcut around
 * op->run_func (art/include/art/op.h:145-163) and its CUDA-event timer
 * (art/modules/cuda_quant/src/cuda_timer.h).  When enabled, every launch of a run is bracketed by
 * CUDA events on the run's stream; b200_case_profile then returns, for the last run, the
 * milliseconds of each launch in launch order (inputs, ops, outputs) and its kind:
 * 0 input layout/quantize, 1 conv (tensor-core path), 2 conv (CUDA-core path), 3 eltwise, 4 relu,
 * 5 pool, 6 output layout/dequantize.  It synchronizes the stream of the last run. */
B200_API int b200_case_set_profiling(b200_case_t *cs, int32_t enable);
B200_API int b200_case_profile(
    b200_case_t *cs, float *ms_per_launch, int32_t *kinds, int32_t capacity, int32_t *count);

#ifdef __cplusplus
}
#endif
#endif /* NART_B200_H */
