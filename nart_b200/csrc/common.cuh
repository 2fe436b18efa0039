// Shared host/device helpers of the sm_100a quantized-convolution backend: status reporting
// for the C-ABI, and the device restatement of the reference CPU module's integer requantize
// arithmetic (art/modules/quant/include/art/quant/quant_helper.h:29-118 of ModelTC/NART).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "nart_b200.h"

namespace b200 {

// ---- host: error plumbing ------------------------------------------------------------------
void set_error(const char *fmt, ...);
int fail(int status, const char *fmt, ...);

#define B200_CUDA_TRY(expr)                                                                    \
    do {                                                                                       \
        cudaError_t _e = (expr);                                                               \
        if (_e != cudaSuccess) {                                                               \
            cudaGetLastError(); /* a non-sticky error must not surface at a later, unrelated call */ \
            return ::b200::fail(                                                               \
                B200_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, \
                __LINE__);                                                                     \
        }                                                                                      \
    } while (0)

#define B200_TRY(expr)           \
    do {                         \
        int _s = (expr);         \
        if (_s != B200_OK)       \
            return _s;           \
    } while (0)

inline cudaStream_t as_stream(b200_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

// Per-device int the kernels with bounded waits write a code into when a wait runs out.
int status_word_ptr(int **dev_ptr);

// Device copy of a 256-byte lookup table, uploaded the first time this table is seen on the current device
// and cached for the life of the process (runtime.cu).
int lut_cache_get(const uint8_t lut[256], const uint8_t **dev_ptr);

// Number of SMs of the current device (cached).
int sm_count();

// Grid of a grid-stride kernel: the blocks that are resident at one time (occupancy x SMs), or
// fewer when there is less work.  A larger grid would run a second, partly filled wave.
template <auto Kernel, int Threads>
int resident_grid(size_t blocks_wanted)
{
    static const int per_sm = [] {
        int occ = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, Kernel, Threads, 0) != cudaSuccess || occ < 1)
            occ = 1;
        return occ;
    }();
    const size_t cap = (size_t)sm_count() * per_sm;
    const size_t blocks = blocks_wanted < cap ? blocks_wanted : cap;
    return (int)(blocks < 1 ? 1 : blocks);
}

// Host restatement of quant_helper.h:60-118 (see b200_get_quant_scale).
void get_quant_scale(float x, int bits, uint32_t *mult, int8_t *shift);
// Host restatement of quant_helper.h:55-58.
inline int64_t rshift_rn_host(int64_t x, int bits)
{
    int64_t y = x >> (bits - 1);
    return (y + ((y & 1) << 1)) >> 1;
}

// ---- device: requantize ----------------------------------------------------------------------
// rshift_rn(x, b) of the reference is ((x >> (b-1)) + (((x >> (b-1)) & 1) << 1)) >> 1 on int64,
// which equals floor((x + 2^(b-1)) / 2^b) whenever x + 2^(b-1) does not overflow (here
// |x| < 2^62).  For b >= 33 the low 32 bits of x cannot change the floor, so the high word of
// the product is enough:  floor((hi*2^32 + lo + 2^(b-1)) / 2^b) = (hi + 2^(b-33)) >> (b-32).
//
// Returns the value the reference passes to saturate_int_by_bits: the rounded shift plus the
// output zero point, narrowed to int32 (conv_2d_uint8_impl.c:159-164).
__device__ __forceinline__ int requant_raw(int acc, uint32_t mult, int shift, int ozp)
{
    if (shift >= 33) {
        return ((__mulhi(acc, (int)mult) + (1 << (shift - 33))) >> (shift - 32)) + ozp;
    }
    long long p = (long long)acc * (long long)mult;
    return (int)(((p + (1ll << (shift - 1))) >> shift) + (long long)ozp);
}

// saturate_int_by_bits (quant_helper.h:33-36) followed, when relu_lo >= 0, by the clamp at the
// output zero point that the reference's relu op performs for equal scales (relu.c:103-109).
__device__ __forceinline__ int sat_relu(int v, int qmax, int relu_lo)
{
    v = min(max(v, 0), qmax);
    return max(v, relu_lo);
}

__device__ __forceinline__ uint32_t pack4(int a, int b, int c, int d)
{
    return (uint32_t)a | ((uint32_t)b << 8) | ((uint32_t)c << 16) | ((uint32_t)d << 24);
}

// sat_u8 of four int32 values packed little-endian (byte 0 = a): cvt.pack.sat.u8.s32 converts two
// values with saturation to 0..255 and merges them above the low half of a third operand.
__device__ __forceinline__ uint32_t pack_sat_u8x4(int a, int b, int c, int d)
{
    uint32_t hi, out;
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(d), "r"(c), "r"(0));
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(b), "r"(a), "r"(hi));
    return out;
}

// 32-bit rounded shift for operands known to satisfy |x| + 2^(b-1) < 2^31, 1 <= b <= 30.
__device__ __forceinline__ int rshift_rn32(int x, int b) { return (x + (1 << (b - 1))) >> b; }
// 64-bit rounded shift, 1 <= b <= 62.
__device__ __forceinline__ long long rshift_rn64(long long x, int b)
{
    return (x + (1ll << (b - 1))) >> b;
}

}  // namespace b200
