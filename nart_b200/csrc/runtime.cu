// Device, memory and stream entry points of the C-ABI, status reporting, and the host
// restatement of the reference's scale decomposition.
#include <math.h>
#include <stdarg.h>
#include <string.h>

#include <mutex>
#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace b200 {

static thread_local char g_err[512] = "";

void set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int fail(int status, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return status;
}

static const int kMaxDevices = 64;
static int *g_status_words[kMaxDevices] = { nullptr };
static int g_sm_count[kMaxDevices] = { 0 };

int status_word_ptr(int **dev_ptr)
{
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices)
        return fail(B200_ERR_INVALID, "device index %d out of range", dev);
    if (!g_status_words[dev]) {
        int *p = nullptr;
        B200_CUDA_TRY(cudaMalloc(&p, sizeof(int)));
        B200_CUDA_TRY(cudaMemset(p, 0, sizeof(int)));
        g_status_words[dev] = p;
    }
    *dev_ptr = g_status_words[dev];
    return B200_OK;
}

// 256-byte lookup tables (relu, max pool) of the flat C-ABI calls: uploaded once per distinct table and
// device and kept for the life of the process, so that a steady-state call allocates and copies nothing.
namespace {
struct LutEntry {
    int device;
    uint8_t bytes[256];
    uint8_t *dev;
};
std::mutex g_lut_mutex;
std::vector<LutEntry> g_luts;
}  // namespace

int lut_cache_get(const uint8_t lut[256], const uint8_t **dev_ptr)
{
    int dev = 0;
    B200_CUDA_TRY(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_lut_mutex);
    for (const auto &e : g_luts)
        if (e.device == dev && memcmp(e.bytes, lut, 256) == 0) {
            *dev_ptr = e.dev;
            return B200_OK;
        }
    LutEntry e;
    e.device = dev;
    memcpy(e.bytes, lut, 256);
    B200_CUDA_TRY(cudaMalloc((void **)&e.dev, 256));
    B200_CUDA_TRY(cudaMemcpy(e.dev, lut, 256, cudaMemcpyHostToDevice));
    g_luts.push_back(e);
    *dev_ptr = e.dev;
    return B200_OK;
}

int sm_count()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices)
        return 148;
    if (!g_sm_count[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        g_sm_count[dev] = n;
    }
    return g_sm_count[dev];
}

// quant_helper.h:60-118.  x is halved / doubled in fp32 (exact) until it lies in [0.5, 1);
// the multiplier is the truncation of x * 2^(bits-1), formed in fp32 like the reference's
// `x * (1ll << 31)` (float times an integer converted to float).  bits == -16 is the uint16
// variant (get_quant_scale_int16).
void get_quant_scale(float x, int bits, uint32_t *mult, int8_t *shift)
{
    int eff = bits == -16 ? 16 : bits;
    int8_t sh = 0;
    if (fabs((double)(x - 0)) < 1e-10) {
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
    float scaled = x * (float)(1ll << (eff - 1));
    *mult = bits == -16 ? (uint32_t)(uint16_t)scaled : (uint32_t)scaled;
    *shift = sh;
}

}  // namespace b200

using namespace b200;

extern "C" {

const char *b200_strerror(int status)
{
    switch (status) {
    case B200_OK: return "ok";
    case B200_ERR_INVALID: return "invalid argument";
    case B200_ERR_UNSUPPORTED: return "unsupported configuration";
    case B200_ERR_CUDA: return "CUDA call failed";
    case B200_ERR_NOMEM: return "out of memory";
    case B200_ERR_DEVICE_WAIT: return "a bounded device-side wait ran out";
    default: return "unknown status";
    }
}

const char *b200_last_error(void) { return g_err; }

int b200_version(void) { return 100; }

int b200_device_count(int *count)
{
    if (!count)
        return fail(B200_ERR_INVALID, "count is NULL");
    B200_CUDA_TRY(cudaGetDeviceCount(count));
    return B200_OK;
}

int b200_set_device(int device)
{
    B200_CUDA_TRY(cudaSetDevice(device));
    return B200_OK;
}

int b200_get_device(int *device)
{
    if (!device)
        return fail(B200_ERR_INVALID, "device is NULL");
    B200_CUDA_TRY(cudaGetDevice(device));
    return B200_OK;
}

int b200_malloc(void **dev_ptr, size_t bytes)
{
    if (!dev_ptr)
        return fail(B200_ERR_INVALID, "dev_ptr is NULL");
    *dev_ptr = nullptr;
    if (bytes == 0)
        return B200_OK;
    cudaError_t e = cudaMalloc(dev_ptr, bytes);
    if (e == cudaErrorMemoryAllocation) {
        cudaGetLastError();
        return fail(B200_ERR_NOMEM, "cudaMalloc of %zu bytes failed", bytes);
    }
    B200_CUDA_TRY(e);
    return B200_OK;
}

int b200_free(void *dev_ptr)
{
    if (dev_ptr)
        B200_CUDA_TRY(cudaFree(dev_ptr));
    return B200_OK;
}

int b200_malloc_host(void **host_ptr, size_t bytes)
{
    if (!host_ptr)
        return fail(B200_ERR_INVALID, "host_ptr is NULL");
    *host_ptr = nullptr;
    if (bytes == 0)
        return B200_OK;
    B200_CUDA_TRY(cudaMallocHost(host_ptr, bytes));
    return B200_OK;
}

int b200_free_host(void *host_ptr)
{
    if (host_ptr)
        B200_CUDA_TRY(cudaFreeHost(host_ptr));
    return B200_OK;
}

int b200_memset(void *dev_ptr, int value, size_t bytes, b200_stream_t stream)
{
    if (bytes)
        B200_CUDA_TRY(cudaMemsetAsync(dev_ptr, value, bytes, as_stream(stream)));
    return B200_OK;
}

int b200_memcpy_h2d(void *dev_dst, const void *host_src, size_t bytes, b200_stream_t stream)
{
    if (bytes)
        B200_CUDA_TRY(
            cudaMemcpyAsync(dev_dst, host_src, bytes, cudaMemcpyHostToDevice, as_stream(stream)));
    return B200_OK;
}

int b200_memcpy_d2h(void *host_dst, const void *dev_src, size_t bytes, b200_stream_t stream)
{
    if (bytes)
        B200_CUDA_TRY(
            cudaMemcpyAsync(host_dst, dev_src, bytes, cudaMemcpyDeviceToHost, as_stream(stream)));
    return B200_OK;
}

int b200_memcpy_d2d(void *dev_dst, const void *dev_src, size_t bytes, b200_stream_t stream)
{
    if (bytes)
        B200_CUDA_TRY(
            cudaMemcpyAsync(dev_dst, dev_src, bytes, cudaMemcpyDeviceToDevice, as_stream(stream)));
    return B200_OK;
}

int b200_stream_create(b200_stream_t *stream)
{
    if (!stream)
        return fail(B200_ERR_INVALID, "stream is NULL");
    cudaStream_t s;
    B200_CUDA_TRY(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking));
    *stream = reinterpret_cast<b200_stream_t>(s);
    return B200_OK;
}

int b200_stream_destroy(b200_stream_t stream)
{
    if (stream)
        B200_CUDA_TRY(cudaStreamDestroy(as_stream(stream)));
    return B200_OK;
}

int b200_stream_synchronize(b200_stream_t stream)
{
    B200_CUDA_TRY(cudaStreamSynchronize(as_stream(stream)));
    return B200_OK;
}

int b200_device_status(b200_stream_t stream, int *status_word)
{
    if (!status_word)
        return fail(B200_ERR_INVALID, "status_word is NULL");
    int *p = nullptr;
    B200_TRY(status_word_ptr(&p));
    B200_CUDA_TRY(cudaStreamSynchronize(as_stream(stream)));
    B200_CUDA_TRY(cudaMemcpy(status_word, p, sizeof(int), cudaMemcpyDeviceToHost));
    if (*status_word != 0)
        B200_CUDA_TRY(cudaMemset(p, 0, sizeof(int)));
    return B200_OK;
}

int b200_selftest_wait_expiry(uint64_t limit_cycles, b200_stream_t stream)
{
    if (limit_cycles == 0 || limit_cycles > 2000000000ull)
        return fail(B200_ERR_INVALID, "selftest: limit of %llu cycles outside 1..2e9 (about one second)", (unsigned long long)limit_cycles);
    return wait_expiry_probe_launch((long long)limit_cycles, as_stream(stream));
}

int b200_measure_mma_i8_peak(int32_t mmas_per_sm, float *ms, double *ops, b200_stream_t stream)
{
    if (!ms || !ops || mmas_per_sm < 64 || mmas_per_sm > 40000000)
        return fail(B200_ERR_INVALID, "measure_mma_i8_peak: bad argument (64 .. 4e7 MMAs per SM)");
    return mma_i8_peak_launch(mmas_per_sm, ms, ops, as_stream(stream));
}

void b200_get_quant_scale(float x, int bits, uint32_t *mult, int8_t *shift)
{
    get_quant_scale(x, bits, mult, shift);
}

}  // extern "C"
