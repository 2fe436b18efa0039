// b200_conv2d_run_static_scratch: the row-lowered convolution (4-channel image stems) with its
// scratch tensor in a fixed device array that is part of this library's image, so that the call
// itself allocates nothing.
//
// Who needs this.  The regular entry point, b200_conv2d_run, grows a per-plan scratch tensor with
// cudaMalloc the first time it sees a batch size.  Some hosts of this library cannot have that:
//   * a serving loop with a latency budget -- cudaMalloc and cudaFree block the calling thread and
//     synchronize the whole device, which stalls every other stream of the process;
//   * a process whose device memory has already been handed, all of it, to the host application's
//     own pool (a framework's caching allocator, a fixed partition of a shared GPU): a cudaMalloc
//     issued from inside a plugin simply fails there.
// Such callers prepare the plan while allocation is still allowed -- b200_conv2d_create of a
// row-lowered plan also resolves this array's address on the current device (which is what makes the
// CUDA runtime load the array onto that device) and does the kernels' one-time set-up -- and then run
// it through this entry point.
#include "common.cuh"
#include "kernels.h"

namespace {

// 32 MiB + a 256-byte header.  Every GPU on which this library is used holds the array from the
// moment the module is loaded until the process exits.
constexpr size_t kStaticScratchBytes = 32u << 20;
// [0, 4): status word of the bounded device-side waits.  Zero when the array is loaded; a kernel only
// ever changes it from zero to a code; b200_static_scratch_status reads it and puts the zero back.
constexpr size_t kHeaderBytes = 256;
static __device__ __align__(256) unsigned char g_static_scratch[kHeaderBytes + kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not an address the GPU can
// use; the device address is asked for once per device and kept here.
constexpr int kMaxDevices = 64;
unsigned char *g_scratch_dev[kMaxDevices] = { nullptr };

int static_scratch_ptr(unsigned char **ptr)
{
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices)
        return b200::fail(B200_ERR_INVALID, "device index %d out of range", dev);
    if (!g_scratch_dev[dev]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);   // with device `dev` current
        if (e != cudaSuccess || !p)
            return b200::fail(B200_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
        g_scratch_dev[dev] = static_cast<unsigned char *>(p);
    }
    *ptr = g_scratch_dev[dev];
    return B200_OK;
}

}  // namespace

namespace b200 {
int conv_static_scratch_prepare()
{
    unsigned char *p = nullptr;
    return static_scratch_ptr(&p);
}
}  // namespace b200

extern "C" int b200_static_scratch_status(b200_stream_t stream, int *status_word)
{
    using namespace b200;
    if (!status_word)
        return fail(B200_ERR_INVALID, "static scratch status: status_word is NULL");
    *status_word = 0;
    unsigned char *base = nullptr;
    B200_TRY(static_scratch_ptr(&base));
    B200_CUDA_TRY(cudaStreamSynchronize(as_stream(stream)));
    B200_CUDA_TRY(cudaMemcpy(status_word, base, sizeof(int), cudaMemcpyDeviceToHost));   // pageable 4-byte copy: no allocation
    if (*status_word != 0) {
        B200_CUDA_TRY(cudaMemset(base, 0, sizeof(int)));
        return fail(B200_ERR_DEVICE_WAIT, "conv(static scratch): a device-side wait ran out (code 0x%x); the outputs of the calls since the last check are not valid", *status_word);
    }
    return B200_OK;
}

extern "C" int b200_conv2d_run_static_scratch(
    b200_conv_t *conv, const uint8_t *x, int32_t n, uint8_t *y, b200_stream_t stream)
{
    using namespace b200;
    if (!conv || n < 0 || (n > 0 && (!x || !y)))
        return fail(B200_ERR_INVALID, "conv(static scratch): bad argument");
    if (!conv->lowered)
        return fail(
            B200_ERR_INVALID,
            "conv(static scratch): this plan uses no scratch tensor (only row-lowered 4-channel convs do); "
            "use b200_conv2d_run");
    if (conv->g.wzp_d != 0)
        return fail(
            B200_ERR_UNSUPPORTED,
            "conv(static scratch): a weight zero point other than 128 needs the window-sum tensors of b200_conv2d_run");
    if (n == 0)
        return B200_OK;
    const ConvGeom &g = conv->g;
    const size_t need = (size_t)n * g.h * g.ow * (kLowerWindow * 4);
    if (need > kStaticScratchBytes)
        return fail(
            B200_ERR_UNSUPPORTED,
            "conv(static scratch): batch %d needs %zu bytes of scratch, the static array holds %zu "
            "(at most %zu images of this shape per call)",
            n, need, kStaticScratchBytes, kStaticScratchBytes / ((size_t)g.h * g.ow * (kLowerWindow * 4)));
    unsigned char *base = nullptr;
    B200_TRY(static_scratch_ptr(&base));
    cudaStream_t st = as_stream(stream);
    // The array keeps what the previous call left.  Of the lowered tensor this call reads exactly the
    // n * h * ow * 32 bytes its lowering kernel has just written, whatever lies behind them.  The status
    // word is not cleared here: a code left by an earlier call stays until b200_static_scratch_status
    // has reported it.
    uint8_t *lowered = base + kHeaderBytes;
    B200_TRY(conv_lower_rows_launch(g, x, n, lowered, st));
    return conv_igemm_launch(conv->igemm, lowered, n, y, st, reinterpret_cast<int *>(base));
}
