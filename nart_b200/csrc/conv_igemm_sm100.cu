// Implicit-GEMM int8 convolution on the 5th-generation tensor cores (sm_100a):
//   D[pixels, Cout] (int32, TMEM) += A[pixels, R*S*C] (uint8 activations) x B[Cout, R*S*C]^T (int8)
// with tcgen05.mma kind::i8, operands staged by TMA into swizzled shared memory, accumulators in
// tensor memory, and the reference's zero-point correction, bias, requantize and ReLU clamp
// fused into the epilogue (art/modules/quant/src/op/conv_2d_uint8_impl.c:107-164 of ModelTC/NART).
//
// GEMM view.  An M tile is 128 output pixels arranged as a TW x TH x TN box of
// (ow, oh, image); for filter tap (r, s) and a BK-channel slice the A operand is the box of input
// pixels one tiled TMA load fetches from the NHWC tensor (coordinates may run outside the image:
// TMA fills zeros).  Strided convs address the input through one tensor map per (row, column)
// parity so that every load stays a plain dense box.  B is the weight matrix repacked once to
// [Cout][R][S][C] int8.  K is walked tap by tap, BK channels at a time.
//
// Zero point.  The MMA multiplies the raw uint8 activation, and TMA pads with the byte 0, whereas
// the reference pads with the real value 0, i.e. the byte izp.  With
//   raw = sum_{valid taps} x * w      true = sum_{valid taps} (x - izp) * w = raw - izp * sum_{valid} w
// the correction depends only on which taps are inside the image, i.e. on the output pixel's
// border class.  The host builds off[class][k] = bias[k] - izp * sum_{taps valid in class} w[k]; the
// epilogue uses it folded with the requantize constants into one 64-bit addend per (class, k):
//   rshift_rn((acc + off) * mult, shift) + ozp  ==  (acc * mult + off64) >> shift,
//   off64 = off * mult + 2^(shift-1) + (ozp << shift).
//
// Warp roles (576 threads, one CTA per SM, persistent over tiles):
//   warp 0      TMA producer (one lane per pipeline slot)
//   warp 1      tensor-memory allocation, MMA issue (one elected lane)
//   warps 2..17 epilogue, two groups of 8 warps (two per tensor-memory lane quarter) or, for narrow
//               channel tiles with a short mainloop, four groups of 4 warps; group i
//               owns accumulator stage i: tcgen05.ld -> requantize -> pack -> swizzled smem -> TMA store
//   warp 18     a second MMA-issuing warp in the instantiations for narrow tiles (MODE 1, 2)
// One accumulator stage per group in tensor memory lets the epilogue of tile i overlap the mainloop
// of the next tiles and their epilogues (the other groups).  MODE 3 runs on clusters of two CTAs that
// share every MMA (tcgen05 cta_group::2, M = 256), each CTA loading its own operands with plain TMA
// loads; the other instantiations launch without clusters.  No load is multicast.  Two epilogue forms
// exist: the 64-bit addend above with per-channel shifts, and a uniform-shift form with two 32-bit
// constants per channel as kernel parameters (see IgemmArgs::epi_const).  Every wait is bounded:
// when one runs out the kernel records a code in the status word, all roles leave their loops,
// tensor memory is freed and the kernel returns.
#include <cuda.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include "common.cuh"
#include "kernels.h"

namespace b200 {

namespace {

constexpr int kMaxAccStages = 4;              // accumulator stages in tensor memory = epilogue groups: 2 or 4
#ifndef B200_EPI_WARPS
#define B200_EPI_WARPS 16
#endif
constexpr int kEpiWarps = B200_EPI_WARPS;     // split into 2 groups of 8 warps or 4 groups of 4
constexpr int kMma2Warp = 2 + kEpiWarps;        // the second MMA-issuing warp, behind the epilogue warps
constexpr int kThreads = 64 + kEpiWarps * 32;
constexpr int kThreads2 = kThreads + 32;         // with the second MMA-issuing warp
constexpr int kTileM = 128;
constexpr int kMaxStages = 8;
constexpr int kGroupBytes = 32 * 1024;        // target size of one pipeline stage (a group of k-blocks)
constexpr int kMaxGroup = 10;                 // three stages of a group must fit the producer's 32 lanes
constexpr long long kWaitCycles = 4000000000ll;   // ~2 s at 1.9 GHz

// device status codes (which wait gave up)
constexpr int kErrProducerWait = 0x101;
constexpr int kErrMmaFullWait = 0x102;
constexpr int kErrMmaTmemWait = 0x103;
constexpr int kErrEpilogueWait = 0x104;
constexpr int kErrSelfTestWait = 0x1ff;   // wait_expiry_probe_kernel

struct alignas(64) IgemmMaps {
    CUtensorMap a[4];   // activations, one per (row parity, column parity) of a strided conv
    CUtensorMap b;      // weights [Cout][R*S*C]
    CUtensorMap y;      // output NHWC
};

struct IgemmArgs {
    // problem
    int n, oh, ow, cout;
    int r, s, pad_h, pad_w, stride_h, stride_w;
    int c;               // input channels, rounded up to a multiple of 32 (the k-blocks' extent)
    // tiling
    int tw, th, tn;      // M-tile box (ow, oh, image), tw*th*tn == 128, each a power of two
    int tw_sh, th_sh;    // log2(tw), log2(th)
    int tiles_w, tiles_h, tiles_n, n_tiles_n;   // tile counts along ow, oh, image and Cout
    int step_nt, step_w, step_h, step_n;        // mixed-radix digits of the grid size (see TileWalker)
    int bk;              // channels per k-block (32, 64, 128) == swizzle span of the operands
    int bn;              // output channels per tile (multiple of 16, <= 256)
    int stages;          // smem pipeline depth
    int groups;          // epilogue groups (2 or 4); group i takes every groups-th tile of the CTA
    int acc_stages;      // accumulator stages in tensor memory (a multiple of groups, at most 4)
    int kgroup;          // k-blocks per pipeline stage (divides the k-blocks of a tile): one barrier round trip per group
    uint32_t rcp_cchunks, rcp_s;   // ceil(2^30 / (c / bk)), ceil(2^30 / s): k-block index -> tap, tap -> row
    int b_resident;      // 1: all k-blocks of B stay in shared memory (one channel tile, weights fit)
    int a_wide;          // 1: 32-channel rows stored pre-swizzled; A is fetched as whole rows of pixels
    int ob, ob_sh;       // bytes per row of an output staging sub-tile (16..128, divides bn) and its log2
    uint32_t idesc;      // tcgen05 instruction descriptor
    uint32_t tmem_cols;  // columns to allocate (power of two >= 2*bn)
    // epilogue tables
    const long long *off;    // [n_cls][kpad]: off * mult + 2^(shift-1) + (ozp << shift)
    const uint32_t *mult;    // [kpad]
    const int32_t *shift;    // [kpad]
    const uint8_t *row_cls;  // [oh]
    const uint8_t *col_cls;  // [ow]
    int n_col_cls, n_cls, kpad;
    int ozp, qmax, relu_lo;
    int generic_requant;     // 1: some channel has shift < 33, use the 64-bit requantize everywhere
    int use_tma_store;       // 0: plain stores (Cout not a multiple of 16)
    uint8_t *y;
    int *status;
    // fused residual add (eltwise SUM of this conv's output and `res`, see EltwiseArgs): index 0 is
    // the conv's own output, index 1 the residual tensor (NHWC, the dims of y); res == nullptr: off
    const uint8_t *res;
    int r_m[2], r_add[2], r_b[2];
    int r_s0, r_ozp, r_lo;
    // weight zero point other than 128: acc -= wzp_d * wsum[pixel] before the requantize, wsum = window
    // sums of (x - izp) per output pixel [n][oh][ow] (conv_window_sum_launch); nullptr: off
    const int32_t *wsum;
    int wzp_d;
    // Uniform-shift epilogue (epi_const != 0): every channel's shift was brought to the layer's smallest
    // one, S, by dropping low zero bits of its multiplier, so that
    //   y = ((acc + off32[class][k]) * mult_u[k] + rnd) >> S,   rnd = 2^(S-1) + (ozp << S)
    // needs two 32-bit constants per channel.  With one channel tile they are kernel parameters (EpiTab),
    // read as immediate constant-bank operands by the unrolled epilogue: no loads, no registers.
    uint32_t out_flip;       // int8 outputs: 0x80808080 (the generic requantize form flips bit 7 of every byte), else 0
    int epi_const;           // 0: off; else one byte per warp of a lane quarter: (first 32-column chunk << 4) | chunk count
    int ushift;              // S - 32: the shift of the product's high word
    int rnd_lo, rnd_hi;      // rnd
    const int32_t *off32;    // [n_cls][kpad] accumulator offsets (layers with several border classes read them from here)
    // 1: the M tiles are visited from the last image / row / column tile down to the first, so that a layer
    // starts on the part of its input that the layer before wrote last (and that still sits in L2)
    int rev;
    // Read-only bytes the launch after this one starts on (the next layer's repacked weights): every CTA asks
    // for its slice to be brought into L2 while this layer runs, so that the next launch's first weight loads
    // do not all miss at once.  nullptr / 0: none.
    const uint8_t *next_ro;
    uint32_t next_ro_bytes;
    // CTA pair (MODE 3): two CTAs of a cluster share every MMA (tcgen05 cta_group::2, M = 256): CTA r of the
    // pair owns M tile 2 * pm + r of pair tile pm and loads that tile's activations and half r of the
    // weight tile; the pair tiles are walked as (nt fastest, pm) with the digits step_nt, step_pm of the
    // number of clusters.
    int pm_tiles;            // pair tiles along M: ceil(m_tiles / 2)
    int step_pm;
};

// Per-channel constants of the uniform-shift epilogue for layers with one channel tile (<= 256 channels).
struct EpiTab {
    int32_t off32[256];      // the single border class's offsets (unused otherwise)
    int32_t mult[256];
};

// Tile index -> (Cout tile, ow tile, oh tile, image tile), Cout tile fastest.  A persistent CTA
// visits tiles blockIdx.x, blockIdx.x + gridDim.x, ...: the digits advance by the mixed-radix
// digits of gridDim.x (computed on the host) with carries, so no role divides inside its loop.
struct TileWalker {
    int nt, twi, thi, tni;
    int pm = 0, rank = -1;   // CTA-pair mode (rank >= 0): pair tile index along M and this CTA's rank in its pair
    __device__ __forceinline__ void decode_pair(const IgemmArgs &g)
    {
        int mt = 2 * pm + rank;          // an M tile past the last one decodes to an image index past the batch
        twi = mt % g.tiles_w;
        mt /= g.tiles_w;
        thi = mt % g.tiles_h;
        tni = mt / g.tiles_h;
    }
    __device__ __forceinline__ void init_pair(const IgemmArgs &g, int pair_tile, int cta_rank)
    {
        rank = cta_rank;
        nt = pair_tile % g.n_tiles_n;
        pm = pair_tile / g.n_tiles_n;
        decode_pair(g);
    }
    __device__ __forceinline__ void init(const IgemmArgs &g, int tile)
    {
        nt = tile % g.n_tiles_n;
        int mt = tile / g.n_tiles_n;
        twi = mt % g.tiles_w;
        mt /= g.tiles_w;
        thi = mt % g.tiles_h;
        tni = mt / g.tiles_h;
    }
    __device__ __forceinline__ void advance(const IgemmArgs &g)
    {
        if (rank >= 0) {
            nt += g.step_nt;
            int carry = 0;
            if (nt >= g.n_tiles_n) { nt -= g.n_tiles_n; carry = 1; }
            pm += g.step_pm + carry;
            decode_pair(g);
            return;
        }
        nt += g.step_nt;
        int carry = 0;
        if (nt >= g.n_tiles_n) { nt -= g.n_tiles_n; carry = 1; }
        twi += g.step_w + carry;
        carry = 0;
        if (twi >= g.tiles_w) { twi -= g.tiles_w; carry = 1; }
        thi += g.step_h + carry;
        carry = 0;
        if (thi >= g.tiles_h) { thi -= g.tiles_h; carry = 1; }
        tni += g.step_n + carry;
    }
    // tile coordinates as the roles use them (reversed traversal mirrors every M digit)
    __device__ __forceinline__ int wi(const IgemmArgs &g) const { return g.rev ? g.tiles_w - 1 - twi : twi; }
    __device__ __forceinline__ int hi(const IgemmArgs &g) const { return g.rev ? g.tiles_h - 1 - thi : thi; }
    // (an M tile past the end -- the odd tail of a CTA pair -- keeps its out-of-range image index)
    __device__ __forceinline__ int ni(const IgemmArgs &g) const { return (g.rev && tni < g.tiles_n) ? g.tiles_n - 1 - tni : tni; }
};

// ---- PTX wrappers --------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking form: the producer lanes poll many barriers from one warp, where a try_wait that
// suspends on one lane's barrier would hold back the lanes whose barrier is ready.
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: returns false when the barrier did not flip within kWaitCycles or another role
// has already given up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, long long limit = kWaitCycles)
{
    if (mbar_try_wait(bar, parity))
        return true;
    const long long t0 = clock64();
    int spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 255) == 0) {
            if (*abort_flag != 0 || clock64() - t0 > limit)
                return false;
        }
    }
    return true;
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
// Loads of a CTA pair: the data lands in this CTA's shared memory, the bytes are counted on the mbarrier of
// the pair's leading CTA (`bar` is a shared::cluster address).  Plain tiled loads -- every CTA fetches its own box.
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
// The shared::cluster address of `addr` (a shared::cta address of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t cluster_addr(uint32_t addr, uint32_t rank)
{
    uint32_t out;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(addr), "r"(rank));
    return out;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar)
{
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_store_4d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
        ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// all but the most recent store group have finished reading their shared-memory source
__device__ __forceinline__ void tma_store_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void prefetch_map(const CUtensorMap *map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// The same three for a CTA pair: one warp of each CTA of the pair issues them.
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t cols)
{
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t cols)
{
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
// One MMA over both CTAs of a pair (M = 256): rows 0..127 of A and D live in the leading CTA, rows 128..255 in
// its peer, each CTA holds half of B's rows; the descriptors are this (the leading) CTA's shared addresses.
__device__ __forceinline__ void mma_i8_pair(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                            uint32_t accumulate, uint32_t issue)
{
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "setp.ne.b32 q, %6, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "@q tcgen05.mma.cta_group::2.kind::i8 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate), "r"(issue)
        : "memory");
}
// Arrival on `bar` (a shared::cluster address, this CTA's or the peer's) when every MMA of the pair issued so
// far has completed.  One such commit per CTA that has to hear of it: no multicast form is used.
__device__ __forceinline__ void mma_commit_pair(uint32_t bar, uint32_t issue)
{
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "@q tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(bar), "r"(issue)
        : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T, 8-bit integer operands, int32 accumulate.  The descriptors
// come as low words plus the high word both share; `issue` predicates the instruction.
__device__ __forceinline__ void mma_i8(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t desc_hi, uint32_t idesc,
                                       uint32_t accumulate, uint32_t issue)
{
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t.reg .b64 da, db;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "setp.ne.b32 q, %6, 0;\n\t"
        "mov.b64 da, {%1, %3};\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "@q tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(desc_hi), "r"(idesc), "r"(accumulate), "r"(issue)
        : "memory");
}
// The barrier gets one arrival when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar, uint32_t issue)
{
    asm volatile(
        "{\n\t.reg .pred q;\n\t"
        "setp.ne.b32 q, %1, 0;\n\t"
        "@q tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(bar), "r"(issue)
        : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
          "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
          "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// Named barriers of one epilogue group (ids 1 + 2g and 2 + 2g for group g).
__device__ __forceinline__ void epi_bar_sync(int group, int group_threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(1 + 2 * group), "r"(group_threads) : "memory");
}
// AND-reduction of a predicate over the threads of one epilogue group: every thread gets
// the same answer, so all of them leave the tile loop together.
__device__ __forceinline__ bool epi_bar_all(int group, int group_threads, bool pred)
{
    uint32_t out;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %1, 0;\n\t"
        "barrier.cta.red.and.pred q, %3, %2, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(out)
        : "r"((uint32_t)pred), "r"(group_threads), "r"(2 + 2 * group)
        : "memory");
    return out != 0;
}

// Shared-memory matrix descriptor of a K-major operand tile whose rows are `bk` bytes
// (bk = 128 / 64 / 32 selects the 128B / 64B / 32B swizzle both TMA and the MMA use); eight rows
// form one swizzle atom, atoms follow each other every 8*bk bytes (the stride byte offset).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, int bk)
{
    const uint64_t layout = bk == 128 ? 2ull : (bk == 64 ? 4ull : 6ull);
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3FFFF) >> 4);          // start address, 16-byte units
    d |= (uint64_t)1 << 16;                           // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)((8 * bk) >> 4) << 32;             // stride byte offset
    d |= (uint64_t)1 << 46;                           // descriptor version of sm_100
    d |= layout << 61;
    return d;
}

// ---- epilogue arithmetic ------------------------------------------------------------------------
struct EpiConsts {
    const int32_t *s_mult;     // shared: per-channel multiplier of the current channel tile
    const int32_t *s_shift;    // shared: shift - 32 (fast form) or shift (generic form)
    const long long *s_off;    // shared: folded 64-bit addends when the layer has one border class
    uint8_t *s_out;            // staging buffer of this epilogue group
    int ob, ob_sh, sw, row;
    int qmax, relu_lo;
    uint32_t out_flip;         // 0x80808080 for int8 outputs (generic form only), else 0
    int r_m0, r_add0, r_b0, r_m1, r_add1, r_b1, r_s0, r_ozp, r_lo;   // fused residual add
};

// One chunk of NCOL (32 or 16) accumulator columns of this thread's row: requantize, pack, write to
// the swizzled staging tile.  The host folded everything additive into one 64-bit constant per
// (border class, channel):  off64 = off * mult + 2^(shift-1) + (ozp << shift), so that
//   rshift_rn((acc + off) * mult, shift) + ozp == (acc * mult + off64) >> shift
// -- one wide multiply-add, then a shift (of the high word alone when every shift is >= 32: FAST).
// FAST also assumes obits == 8, where the pack's saturation to 0..255 is the whole clamp.
// SMEM_OFF reads the addends from shared memory (layers with a single border class) instead of
// the per-class rows in global memory.  All flags are compile-time so that the body is one
// straight-line block of independent chains.  FLOOR = false drops the ReLU floor when it is 0, where
// the pack's own clamp already applies it.
template <bool FAST, bool SMEM_OFF, int NCOL, bool FLOOR = true, bool RES = false>
__device__ __forceinline__ void epi_chunk(const uint32_t (&v)[32], int c0, const long long *off_row, const EpiConsts &ec,
                                          const uint32_t (&rv)[8])
{
    uint32_t packed[NCOL / 4];
#pragma unroll
    for (int q4 = 0; q4 < NCOL / 4; ++q4) {
        longlong2 oa, ob;
        if (SMEM_OFF) {
            oa = *reinterpret_cast<const longlong2 *>(ec.s_off + c0 + q4 * 4);
            ob = *reinterpret_cast<const longlong2 *>(ec.s_off + c0 + q4 * 4 + 2);
        } else {
            oa = __ldg(reinterpret_cast<const longlong2 *>(off_row + c0 + q4 * 4));
            ob = __ldg(reinterpret_cast<const longlong2 *>(off_row + c0 + q4 * 4 + 2));
        }
        const int4 m4 = *reinterpret_cast<const int4 *>(ec.s_mult + c0 + q4 * 4);
        const int4 s4 = *reinterpret_cast<const int4 *>(ec.s_shift + c0 + q4 * 4);
        const long long p0 = (long long)(int)v[q4 * 4 + 0] * m4.x + oa.x;
        const long long p1 = (long long)(int)v[q4 * 4 + 1] * m4.y + oa.y;
        const long long p2 = (long long)(int)v[q4 * 4 + 2] * m4.z + ob.x;
        const long long p3 = (long long)(int)v[q4 * 4 + 3] * m4.w + ob.y;
        int q0, q1, q2, q3;
        if (FAST) {
            q0 = (int)(p0 >> 32) >> s4.x;
            q1 = (int)(p1 >> 32) >> s4.y;
            q2 = (int)(p2 >> 32) >> s4.z;
            q3 = (int)(p3 >> 32) >> s4.w;
        } else {
            // generic: full 64-bit shift, narrowed to int32 as the reference narrows before saturating
            q0 = min((int)(p0 >> s4.x), ec.qmax);
            q1 = min((int)(p1 >> s4.y), ec.qmax);
            q2 = min((int)(p2 >> s4.z), ec.qmax);
            q3 = min((int)(p3 >> s4.w), ec.qmax);
        }
        if (RES) {
            // fused eltwise SUM with the residual bytes rv: the conv's own value is first saturated as
            // it would have been stored (floor, then 0..255), then both inputs go through
            // (x * m + add) >> b, the sum through >> s0 plus the output zero point and floor
            const uint32_t rw = rv[q4];
            const int a0 = min(max(q0, ec.relu_lo), 255), a1 = min(max(q1, ec.relu_lo), 255);
            const int a2 = min(max(q2, ec.relu_lo), 255), a3 = min(max(q3, ec.relu_lo), 255);
            const int t0 = ((a0 * ec.r_m0 + ec.r_add0) >> ec.r_b0) + (((int)(rw & 0xff) * ec.r_m1 + ec.r_add1) >> ec.r_b1);
            const int t1 = ((a1 * ec.r_m0 + ec.r_add0) >> ec.r_b0) + (((int)((rw >> 8) & 0xff) * ec.r_m1 + ec.r_add1) >> ec.r_b1);
            const int t2 = ((a2 * ec.r_m0 + ec.r_add0) >> ec.r_b0) + (((int)((rw >> 16) & 0xff) * ec.r_m1 + ec.r_add1) >> ec.r_b1);
            const int t3 = ((a3 * ec.r_m0 + ec.r_add0) >> ec.r_b0) + (((int)(rw >> 24) * ec.r_m1 + ec.r_add1) >> ec.r_b1);
            packed[q4] = pack_sat_u8x4(max((t0 >> ec.r_s0) + ec.r_ozp, ec.r_lo), max((t1 >> ec.r_s0) + ec.r_ozp, ec.r_lo),
                                       max((t2 >> ec.r_s0) + ec.r_ozp, ec.r_lo), max((t3 >> ec.r_s0) + ec.r_ozp, ec.r_lo));
        } else
        // the pack saturates to 0..255; a ReLU floor above 0 is applied first (FLOOR)
        if (FLOOR)
            packed[q4] = pack_sat_u8x4(max(q0, ec.relu_lo), max(q1, ec.relu_lo), max(q2, ec.relu_lo), max(q3, ec.relu_lo));
        else
            packed[q4] = pack_sat_u8x4(q0, q1, q2, q3);
        if (!FAST)
            packed[q4] ^= ec.out_flip;
    }
    // staging: sub-tile (col / ob), row-major rows of `ob` bytes, 16-byte chunks XOR-swizzled with the
    // row index exactly as the TMA store's swizzle mode expects
#pragma unroll
    for (int ch = 0; ch < NCOL / 16; ++ch) {
        const int col = c0 + ch * 16;
        const int sub = col >> ec.ob_sh;
        const int chunk = (col & (ec.ob - 1)) >> 4;
        uint8_t *srow = ec.s_out + (((size_t)sub * kTileM + ec.row) << ec.ob_sh);
        *reinterpret_cast<uint4 *>(srow + ((chunk ^ ec.sw) << 4))
            = make_uint4(packed[ch * 4], packed[ch * 4 + 1], packed[ch * 4 + 2], packed[ch * 4 + 3]);
    }
}

// The uniform-shift form of one 16-column half chunk (see IgemmArgs::epi_const).  `c0` is a compile-time
// constant after unrolling, so tab.mult[c0 + i] and tab.off32[c0 + i] are constant-bank operands of
// the add and the multiply-add; the 16 chains share nothing but the two uniform registers of `rnd`.
template <bool SINGLE, bool FLOOR, bool WZP>
__device__ __forceinline__ void epi_half_const(const uint32_t (&v)[16], const EpiTab &tab, const int c0, const int32_t *off_row32,
                                               const long long rnd, const int ush, const int relu_lo, const int wz_t,
                                               uint8_t *s_out, const int ob, const int ob_sh, const int sw, const int row)
{
    uint32_t packed[4];
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
        int o0, o1, o2, o3;
        if (SINGLE) {
            o0 = tab.off32[c0 + q4 * 4 + 0]; o1 = tab.off32[c0 + q4 * 4 + 1];
            o2 = tab.off32[c0 + q4 * 4 + 2]; o3 = tab.off32[c0 + q4 * 4 + 3];
        } else {
            const int4 o = __ldg(reinterpret_cast<const int4 *>(off_row32 + c0 + q4 * 4));
            o0 = o.x; o1 = o.y; o2 = o.z; o3 = o.w;
        }
        if (WZP) {
            o0 += wz_t; o1 += wz_t; o2 += wz_t; o3 += wz_t;
        }
        const long long p0 = (long long)((int)v[q4 * 4 + 0] + o0) * tab.mult[c0 + q4 * 4 + 0] + rnd;
        const long long p1 = (long long)((int)v[q4 * 4 + 1] + o1) * tab.mult[c0 + q4 * 4 + 1] + rnd;
        const long long p2 = (long long)((int)v[q4 * 4 + 2] + o2) * tab.mult[c0 + q4 * 4 + 2] + rnd;
        const long long p3 = (long long)((int)v[q4 * 4 + 3] + o3) * tab.mult[c0 + q4 * 4 + 3] + rnd;
        const int q0 = (int)(p0 >> 32) >> ush, q1 = (int)(p1 >> 32) >> ush;
        const int q2 = (int)(p2 >> 32) >> ush, q3 = (int)(p3 >> 32) >> ush;
        if (FLOOR)
            packed[q4] = pack_sat_u8x4(max(q0, relu_lo), max(q1, relu_lo), max(q2, relu_lo), max(q3, relu_lo));
        else
            packed[q4] = pack_sat_u8x4(q0, q1, q2, q3);
    }
    const int sub = c0 >> ob_sh;
    const int chunk = (c0 & (ob - 1)) >> 4;
    uint8_t *srow = s_out + (((size_t)sub * kTileM + row) << ob_sh);
    *reinterpret_cast<uint4 *>(srow + ((chunk ^ sw) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

// The 32-column chunks [CH0, CH1) of a tile's accumulator rows for one warp, uniform-shift form, in
// halves of 16 columns: the tensor-memory read of the next half is in flight while this one is
// requantized (two register sets of 16).  The accumulator stage goes back to the MMA warp as soon as
// the last read has landed, before the last half's arithmetic.
template <int CH0, int CH1, bool SINGLE, bool FLOOR, bool WZP>
__device__ __forceinline__ void epi_tile_const(const uint32_t t_row, const int bn, const EpiTab &tab, const int32_t *off_row32,
                                               const long long rnd, const int ush, const int relu_lo, const int wz_t,
                                               uint8_t *s_out, const int ob, const int ob_sh, const int sw, const int row,
                                               const uint32_t tempty, const int lane)
{
    // the caller guarantees that the range is exact (CH1 * 32 <= bn): everything here is compile-time
    uint32_t va[16], vb[16];
    tmem_ld16(t_row + CH0 * 32, va);
#pragma unroll
    for (int h = CH0 * 2; h < CH1 * 2; ++h) {
        const int c0 = h * 16;
        tmem_ld_wait();
        const bool more = h + 1 < CH1 * 2;
        if (((h - CH0 * 2) & 1) == 0) {
            if (more)
                tmem_ld16(t_row + c0 + 16, vb);
        } else {
            if (more)
                tmem_ld16(t_row + c0 + 16, va);
        }
        if (!more) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0)
                mbar_arrive(tempty);
        }
        if (((h - CH0 * 2) & 1) == 0)
            epi_half_const<SINGLE, FLOOR, WZP>(va, tab, c0, off_row32, rnd, ush, relu_lo, wz_t, s_out, ob, ob_sh, sw, row);
        else
            epi_half_const<SINGLE, FLOOR, WZP>(vb, tab, c0, off_row32, rnd, ush, relu_lo, wz_t, s_out, ob, ob_sh, sw, row);
    }
}

// ---- shared memory layout (dynamic, base aligned to 1024) ---------------------------------------
//   [stages x A tile (128 x bk)] [stages x B tile (bn x bk)] [2 x output staging 128 x bn]
//   [2 x (mult bn x 4, shift bn x 4, offsets bn x 8)] [barriers][tmem address][abort flag]
struct SmemLayout {
    uint32_t a, b, out, tables, bars, tmem_slot, abort_flag, total;
};
// b_slots: B tiles held in shared memory -- one per pipeline stage, or every k-block of the layer
// when the weights stay resident.
__host__ __device__ inline SmemLayout smem_layout(int a_slots, int b_slots, int bk, int bn, int groups, int bn_b = 0)
{
    if (bn_b == 0)
        bn_b = bn;      // rows of a B tile in this CTA's shared memory (half of bn in a CTA pair)
    SmemLayout L;
    uint32_t o = 0;
    L.a = o;
    o += (uint32_t)a_slots * kTileM * bk;
    L.b = o;
    uint32_t b_tile = ((uint32_t)bn_b * bk + 1023u) & ~1023u;
    o += (uint32_t)b_slots * b_tile;
    L.out = o;
    o += (uint32_t)groups * kTileM * bn;   // one output staging buffer per epilogue group
    o = (o + 1023u) & ~1023u;
    L.tables = o;                      // per epilogue group: mult[bn], shift[bn] (int32), off[bn] (int64)
    o += (uint32_t)groups * bn * 16;
    o = (o + 15u) & ~15u;
    L.bars = o;
    o += (2 * kMaxStages + 2 * kMaxAccStages + 1) * 8;
    L.tmem_slot = o;
    o += 8;
    L.abort_flag = o;
    o += 8;
    L.total = o;
    return L;
}

// HAS_RES: the instantiation whose epilogue can add a residual tensor; plans without a fused add run the
// other one, which carries none of that code.
// MODE 0: one MMA-issuing warp.  MODE 1 and 2 add a second one (one more warp in the block):
//   1: the CTA's tiles alternate between the two warps, each on its own half of the stage ring;
//   2: the CTA's tiles go in pairs that share every weight k-block: a stage holds the activation
//      tiles of both and ONE weight tile, each warp issues the MMAs of its own tile of the pair.
template <bool HAS_RES, bool HAS_WZP = false, int MODE = 0>
__global__ void __launch_bounds__((MODE == 1 || MODE == 2) ? kThreads2 : kThreads, 1) conv_igemm_i8_kernel(const __grid_constant__ IgemmMaps maps, const __grid_constant__ IgemmArgs g, const __grid_constant__ EpiTab tab)
{
    extern __shared__ uint8_t smem_raw[];
    // the swizzle patterns are functions of the absolute shared address: align the base to 1024
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (base - raw_addr);
    const int kblocks_all = g.r * g.s * (g.c / g.bk);
    const int slots = g.stages * g.kgroup;
    constexpr bool PAIR = MODE == 3;
    uint32_t cta_rank = 0;
    if (PAIR)
        asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(cta_rank));
    const bool leader = !PAIR || cta_rank == 0;
    const int bnl = PAIR ? g.bn >> 1 : g.bn;     // rows of B this CTA holds
    const SmemLayout L = smem_layout(MODE == 2 ? 2 * slots : slots, g.b_resident ? kblocks_all : slots, g.bk, g.bn, g.groups, bnl);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t a_tile_bytes = (uint32_t)kTileM * g.bk;
    const uint32_t b_tile_bytes = ((uint32_t)bnl * g.bk + 1023u) & ~1023u;
    const uint32_t bar0 = base + L.bars;
    auto full_bar = [&](int s) { return bar0 + 8u * s; };
    auto empty_bar = [&](int s) { return bar0 + 8u * (kMaxStages + s); };
    auto tfull_bar = [&](int s) { return bar0 + 8u * (2 * kMaxStages + s); };
    auto tempty_bar = [&](int s) { return bar0 + 8u * (2 * kMaxStages + kMaxAccStages + s); };
    const uint32_t bres_bar = bar0 + 8u * (2 * kMaxStages + 2 * kMaxAccStages);   // resident weights have landed
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem + L.tmem_slot);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L.abort_flag);

    if (threadIdx.x == 0) {
        for (int s = 0; s < g.stages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), MODE == 2 ? 2 : 1);   // pair mode: both issuing warps release a stage
        }
        mbar_init(bres_bar, 1);
        for (int s = 0; s < g.acc_stages; ++s) {
            mbar_init(tfull_bar(s), 1);
            // one arrival per warp of the stage's epilogue group (of both CTAs of a pair: the leading CTA's
            // barrier tells its MMA warp that the accumulator halves of both are free)
            mbar_init(tempty_bar(s), (kEpiWarps / g.groups) * (PAIR ? 2 : 1));
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_map(&maps.a[0]);
        prefetch_map(&maps.b);
        prefetch_map(&maps.y);
    }
    if (warp == 1) {
        if (PAIR) {
            tmem_alloc_pair(base + L.tmem_slot, g.tmem_cols);
            tmem_relinquish_pair();
        } else {
            tmem_alloc(base + L.tmem_slot, g.tmem_cols);
            tmem_relinquish();
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR)
        cluster_sync_all();     // the peer's barriers are initialised before anything arrives on them
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (threadIdx.x == 2 * 32 && g.next_ro_bytes != 0) {
        // this CTA's slice of the next launch's read-only operand, in 16-byte granules
        const uint32_t granules = g.next_ro_bytes >> 4;
        const uint32_t per = (granules + gridDim.x - 1) / gridDim.x;
        const uint32_t first = blockIdx.x * per;
        if (first < granules) {
            const uint32_t cnt = min(per, granules - first);
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(g.next_ro + ((size_t)first << 4)), "r"(cnt << 4) : "memory");
        }
    }

    const int m_tiles = g.tiles_w * g.tiles_h * g.tiles_n;
    // the tile sequence of this CTA: tile0, tile0 + tstride, ...  (a CTA pair walks pair tiles together)
    const int total_tiles = PAIR ? g.pm_tiles * g.n_tiles_n : m_tiles * g.n_tiles_n;
    const int tile0 = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int tstride = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    auto walker_init = [&](TileWalker &w) {
        if (PAIR)
            w.init_pair(g, tile0, (int)cta_rank);
        else
            w.init(g, tile0);
    };
    const int cchunks = g.c / g.bk;
    const int kblocks = g.r * g.s * cchunks;

    if (warp == 0) {
        // ================= TMA producer =================
        // The pipeline's k-blocks form one sequence over this CTA's tiles; slot l = q mod slots
        // (slots = stages * kgroup <= 32) holds k-block q.  Lane l owns slot l for the whole kernel and
        // issues the loads of k-blocks l, l + slots, ...: the lanes work side by side, so the latency
        // of one lane's bookkeeping (decode the k-block, wait for the stage, issue) is shared by
        // `slots` k-blocks.  The first lane of a group posts the group's byte count; a load of another
        // lane may complete before that (the transaction count is signed), the phase cannot, because
        // the arrival is still pending.
        //
        // With two MMA-issuing warps the ring is split in two halves, one per warp: the lanes of half
        // r load the k-blocks of the CTA's tiles r, r + 2, ... only, so that every stage barrier has
        // one consumer that meets its phases in order.
        const int slots = g.stages * g.kgroup;
        //
        // Pair mode: one ring; slot l holds, for k-block q of the PAIR sequence, the activation tiles of
        // the pair's two tiles and the one weight tile both use (the host has checked that the two
        // tiles share their channel tile).
        constexpr int rings = MODE == 1 ? 2 : 1;
        constexpr int tiles_per_step = (MODE == 0 || MODE == 3) ? 1 : 2;   // tiles a lane moves on by when its k-block wraps
        const int ring_slots = slots / rings;
        if (lane < slots && tile0 < total_tiles) {
            const int stage = lane / g.kgroup;
            const int ring = lane / ring_slots, rl = lane - ring * ring_slots;
            const bool first = lane == stage * g.kgroup;
            const uint32_t fb = full_bar(stage), eb = empty_bar(stage);
            const uint32_t a_dst = base + L.a + lane * a_tile_bytes * (MODE == 2 ? 2 : 1), b_dst = base + L.b + lane * b_tile_bytes;
            // a CTA pair: the leading CTA's barrier counts the bytes of both CTAs
            const uint32_t tx_bytes = (a_tile_bytes + (g.b_resident ? 0u : (uint32_t)bnl * g.bk)) * (uint32_t)g.kgroup * (PAIR ? 2u : 1u);
            const uint32_t fb_lead = PAIR ? cluster_addr(fb, 0) : fb;
            if (g.b_resident && lane == 0) {
                // one channel tile and weights that fit: every k-block of B is loaded once and stays
                mbar_expect_tx(bres_bar, (uint32_t)kblocks * g.bn * g.bk);
                for (int kb = 0; kb < kblocks; ++kb)
                    tma_load_2d(base + L.b + kb * b_tile_bytes, &maps.b, bres_bar, kb * g.bk, 0);
            }
            const int sh_h = g.stride_h - 1, sh_w = g.stride_w - 1;   // strides are 1 or 2
            // this lane's first k-block
            int kb = rl % kblocks;
            int tile = tile0;
            TileWalker tw;
            walker_init(tw);
            for (int i = (rl / kblocks) * tiles_per_step + ring; i > 0; --i) {
                tile += tstride;
                tw.advance(g);
            }
            uint32_t phase = 0;
            // Every pass of the loop each lane polls its own stage once (without suspending: a blocked
            // lane would hold back the ready ones); a lane whose stage is free issues its loads and
            // moves on to its next k-block, the others poll again in the next pass.  No lane ever waits
            // for another lane's stage.
            const unsigned lanes_mask = slots >= 32 ? 0xffffffffu : ((1u << slots) - 1u);
            bool active = tile < total_tiles;
            long long t0 = clock64();
            int spins = 0;
            while (__any_sync(lanes_mask, active)) {
                if (active) {
                    if (mbar_test_wait(eb, phase ^ 1)) {
                        // k-block -> (tap row, tap column, channel chunk); the divisions are multiplications
                        // by reciprocals the host rounded up (exact for operands below 2^15)
                        const int tap = (int)(((uint64_t)(uint32_t)kb * g.rcp_cchunks) >> 30);
                        const int cc = (kb - tap * cchunks) * g.bk;
                        const int rr = (int)(((uint64_t)(uint32_t)tap * g.rcp_s) >> 30);
                        const int ss = tap - rr * g.s;
                        // input row of output row oh for this tap: ih = oh*stride + d, d = rr - pad
                        //   = stride * (oh + (d - p) / stride) + p with p = d mod stride (0 <= p < stride)
                        const int dh = rr - g.pad_h, ph = dh & sh_h;
                        const int dw = ss - g.pad_w, pw = dw & sh_w;
                        const int yh = (tw.hi(g) << g.th_sh) + ((dh - ph) >> sh_h);
                        const int xw = (tw.wi(g) << g.tw_sh) + ((dw - pw) >> sh_w);
                        const int n0 = tw.ni(g) * g.tn;
                        const CUtensorMap *amap = &maps.a[ph * 2 + pw];
                        if (PAIR) {
                            if (first && leader)
                                mbar_expect_tx(fb, tx_bytes);
                            tma_load_4d_pair(a_dst, amap, fb_lead, cc, xw, yh, n0);
                            tma_load_2d_pair(b_dst, &maps.b, fb_lead, kb * g.bk, tw.nt * g.bn + (int)cta_rank * bnl);
                        } else if (MODE == 2) {
                            // the pair's second tile (absent behind an odd number of tiles): same tap, its own pixels
                            const bool second = tile + (int)gridDim.x < total_tiles;
                            mbar_expect_tx(fb, tx_bytes + (second ? a_tile_bytes : 0u));
                            tma_load_4d(a_dst, amap, fb, cc, xw, yh, n0);
                            if (second) {
                                TileWalker t2 = tw;
                                t2.advance(g);
                                tma_load_4d(a_dst + a_tile_bytes, amap, fb, cc, (t2.wi(g) << g.tw_sh) + ((dw - pw) >> sh_w),
                                            (t2.hi(g) << g.th_sh) + ((dh - ph) >> sh_h), t2.ni(g) * g.tn);
                            }
                        } else {
                        if (first)
                            mbar_expect_tx(fb, tx_bytes);
                        if (g.a_wide)   // rows of tw pixels x 32 bytes, in 8-byte elements
                            tma_load_3d(a_dst, amap, fb, xw << 2, yh, n0);
                        else
                            tma_load_4d(a_dst, amap, fb, cc, xw, yh, n0);
                        }
                        if (!g.b_resident && !PAIR)
                            tma_load_2d(b_dst, &maps.b, fb, kb * g.bk, tw.nt * g.bn);
                        phase ^= 1;
                        kb += ring_slots;
                        while (kb >= kblocks) {
                            kb -= kblocks;
                            for (int i = 0; i < tiles_per_step; ++i) {
                                tile += tstride;
                                tw.advance(g);
                            }
                        }
                        active = tile < total_tiles;
                        t0 = clock64();
                        spins = 0;
                    } else if ((++spins & 255) == 0 && (*abort_flag != 0 || clock64() - t0 > kWaitCycles)) {
                        atomicCAS(g.status, 0, kErrProducerWait);
                        *abort_flag = 1;
                        active = false;
                    }
                }
            }
        }
    } else if (warp == 1 || ((MODE == 1 || MODE == 2) && warp == kMma2Warp)) {
        // ================= MMA issuer =================
        // The whole warp walks the loop (uniform control flow); lane 0 alone issues.  Descriptors of
        // one operand differ only in the start-address field, so only their low words are computed.
        // In a CTA pair the leading CTA's warp issues for both; the peer's has nothing to do.
        if (leader) {
            const uint32_t lead = lane == 0 ? 1u : 0u;
            // warp r of `rings` issuing warps takes the CTA's tiles r, r + rings, ... and the stages
            // [r * ring_stages, (r + 1) * ring_stages); accumulator stages advance by `rings` as well
            // In pair mode both warps walk the whole ring, stage by stage together: warp r issues for the
            // r-th tile of each pair, on the r-th activation tile of the stage and the shared weight tile.
            constexpr int rings = MODE == 1 ? 2 : 1;
            constexpr int tile_step = (MODE == 0 || MODE == 3) ? 1 : 2;
            const int ring = warp == 1 ? 0 : 1;
            const int ring_stages = g.stages / rings, stage0 = MODE == 1 ? ring * ring_stages : 0;
            int stage = stage0;
            uint32_t phase = 0;
            int as = ring;
            uint32_t aphase = 0;
            bool ok = true;
            const uint64_t adesc0 = make_smem_desc(base + L.a, g.bk);
            const uint64_t bdesc0 = make_smem_desc(base + L.b, g.bk);
            const uint32_t desc_hi = (uint32_t)(adesc0 >> 32);        // the same for A and B
            const uint32_t a_lo0 = (uint32_t)adesc0, b_lo0 = (uint32_t)bdesc0;
            const uint32_t a_step = a_tile_bytes >> 4, b_step = b_tile_bytes >> 4;   // descriptor address units
            const uint32_t a_grp = a_step * g.kgroup * (MODE == 2 ? 2 : 1), b_grp = b_step * g.kgroup;
            const int ksteps = g.bk / 32;
            const int groups = kblocks / g.kgroup;
            const uint32_t idesc = g.idesc;
            if (g.b_resident && tile0 < total_tiles && !mbar_wait(bres_bar, 0, abort_flag)) {
                if (lead)
                    atomicCAS(g.status, 0, kErrMmaFullWait);
                *abort_flag = 1;
                ok = false;
            }
            for (int tile = tile0 + ring * tstride; (MODE == 2 ? tile - ring * tstride : tile) < total_tiles && ok;
                 tile += tile_step * tstride) {
                // pair mode: the second warp of a pair without a second tile still takes part in the
                // stage hand-over (its commits arrive at once), it just issues nothing
                const bool have_tile = MODE != 2 || tile < total_tiles;
                const uint32_t issue = have_tile ? lead : 0u;
                if (have_tile && !mbar_wait(tempty_bar(as), aphase ^ 1, abort_flag)) {
                    if (lead)
                        atomicCAS(g.status, 0, kErrMmaTmemWait);
                    *abort_flag = 1;
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(as * g.bn);
                uint32_t accumulate = 0;
                for (int grp = 0; grp < groups; ++grp) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) {
                        if (lead)
                            atomicCAS(g.status, 0, kErrMmaFullWait);
                        *abort_flag = 1;
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    uint32_t a_lo = a_lo0 + stage * a_grp + (MODE == 2 ? ring * a_step : 0u);
                    uint32_t b_lo = b_lo0 + (g.b_resident ? grp : stage) * b_grp;
                    for (int j = 0; j < g.kgroup; ++j, a_lo += a_step, b_lo += b_step) {
                        // a k-block is 1, 2 or 4 MMAs of K = 32 bytes: +2 (16-byte units) inside the swizzle atom
                        if (PAIR) {
                            mma_i8_pair(d_tmem, a_lo, b_lo, desc_hi, idesc, accumulate, issue);
                            if (ksteps >= 2)
                                mma_i8_pair(d_tmem, a_lo + 2, b_lo + 2, desc_hi, idesc, 1, issue);
                            if (ksteps == 4) {
                                mma_i8_pair(d_tmem, a_lo + 4, b_lo + 4, desc_hi, idesc, 1, issue);
                                mma_i8_pair(d_tmem, a_lo + 6, b_lo + 6, desc_hi, idesc, 1, issue);
                            }
                            accumulate = 1;
                            continue;
                        }
                        mma_i8(d_tmem, a_lo, b_lo, desc_hi, idesc, accumulate, issue);
                        accumulate = 1;
                        if (ksteps >= 2)
                            mma_i8(d_tmem, a_lo + 2, b_lo + 2, desc_hi, idesc, 1, issue);
                        if (ksteps == 4) {
                            mma_i8(d_tmem, a_lo + 4, b_lo + 4, desc_hi, idesc, 1, issue);
                            mma_i8(d_tmem, a_lo + 6, b_lo + 6, desc_hi, idesc, 1, issue);
                        }
                    }
                    if (PAIR) {
                        // the stage is free again in both CTAs once these MMAs are done: one commit per CTA
                        mma_commit_pair(cluster_addr(empty_bar(stage), 0), lead);
                        mma_commit_pair(cluster_addr(empty_bar(stage), 1), lead);
                    } else
                    mma_commit(empty_bar(stage), lead);   // frees the smem stage when the group's MMAs are done
                    if (++stage == stage0 + ring_stages) {
                        stage = stage0;
                        phase ^= 1;
                    }
                }
                if (!ok)
                    break;
                if (PAIR) {
                    mma_commit_pair(cluster_addr(tfull_bar(as), 0), issue);   // both CTAs' halves of the accumulator
                    mma_commit_pair(cluster_addr(tfull_bar(as), 1), issue);
                } else
                mma_commit(tfull_bar(as), issue);         // accumulator complete
                as += tile_step;
                if (as >= g.acc_stages) {
                    as -= g.acc_stages;
                    aphase ^= 1;
                }
            }
        }
    } else if (warp < kMma2Warp) {
        // ================= epilogue (warps 2..17) =================
        // Two independent groups of 8 warps; group i owns accumulator stage i, i.e. every second
        // tile of this CTA, with its own staging buffer, tables and named barriers, so that one
        // group's waits and barriers overlap the other group's arithmetic.
        const int group_warps = kEpiWarps / g.groups;      // 8 or 4: a multiple of four, one or two warps per lane quarter
        const int group_threads = group_warps * 32;
        const int group = (warp - 2) / group_warps;
        const int gw = (warp - 2) % group_warps;     // warp inside the group
        const int et = gw * 32 + lane;               // thread inside the group
        const int quarter = warp & 3;                // TMEM lanes 32*quarter .. +31 belong to this warp
        const int sub_warp = gw >> 2;                // which of the group's warps of that quarter
        const int row = quarter * 32 + lane;         // accumulator row = pixel of the tile
        uint8_t *tables = smem + L.tables + (size_t)group * g.bn * 16;
        int32_t *s_mult = reinterpret_cast<int32_t *>(tables);
        int32_t *s_shift = s_mult + g.bn;
        long long *s_off = reinterpret_cast<long long *>(tables + (size_t)g.bn * 8);
        const bool single_class = g.n_cls == 1;      // 1x1 / unpadded convs: one offset row for all pixels
        const int n_sub = g.bn >> g.ob_sh;           // output sub-tiles of `ob` bytes per row
        const int sw_shift = g.ob == 128 ? 0 : (g.ob == 64 ? 1 : 2);
        const int sw_mask = g.ob == 128 ? 7 : (g.ob == 64 ? 3 : (g.ob == 32 ? 1 : 0));
        const int sw = (row >> sw_shift) & sw_mask;
        const uint32_t out_bytes = (uint32_t)kTileM * g.bn;
        // this thread's pixel inside a tile (tw, th are powers of two)
        const int lw = row & (g.tw - 1), lh = (row >> g.tw_sh) & (g.th - 1), ln = row >> (g.tw_sh + g.th_sh);
        int as = group;                              // accumulator stage of this group's current tile
        uint32_t aphase = 0;
        int cur_nt = -1;
        bool store_pending = false;
        uint8_t *s_out = smem + L.out + (size_t)group * out_bytes;

        const EpiConsts ec = { s_mult, s_shift, s_off, s_out, g.ob, g.ob_sh, sw, row, g.qmax, g.relu_lo, g.out_flip,
                               g.r_m[0], g.r_add[0], g.r_b[0], g.r_m[1], g.r_add[1], g.r_b[1], g.r_s0, g.r_ozp, g.r_lo };
        const bool fast_epi = !g.generic_requant && g.qmax == 255;
        const bool no_floor = g.relu_lo <= 0;

        // Each warp owns its 32 rows of the staging buffer for the column sub-tiles it computes
        // (sub-tile j belongs to warp j mod warps-per-quarter of the quarter), and stores them with
        // its own TMA store of the quarter box: no barrier between the warps of a group on the way
        // of a tile.  Group barriers remain only where the shared tables are reloaded.
        const int wpq = group_warps >> 2;                       // warps per lane quarter: 1 or 2
        const int own_sh = g.ob_sh > 5 ? g.ob_sh : 5;           // ownership granule: a sub-tile, at least one chunk
        const int p0 = quarter * 32;                            // first pixel of this warp's rows inside a tile
        const int qlw = p0 & (g.tw - 1), qlh = (p0 >> g.tw_sh) & (g.th - 1), qln = p0 >> (g.tw_sh + g.th_sh);
        bool failed = false;   // a wait ran out: skip the work of the remaining tiles, keep meeting the group barriers

        TileWalker tw;
        walker_init(tw);
        for (int i = 0; i < group; ++i)
            tw.advance(g);
        // a CTA pair's accumulator stages are handed back on the leading CTA's barrier
        auto tempty_arrive = [&](int stage_idx) {
            if (PAIR && !leader)
                mbar_arrive_cluster(cluster_addr(tempty_bar(stage_idx), 0));
            else
                mbar_arrive(tempty_bar(stage_idx));
        };
        for (int tile = tile0 + group * tstride; tile < total_tiles; tile += g.groups * tstride) {
            const int nt = tw.nt;
            const int ow0 = tw.wi(g) << g.tw_sh, oh0 = tw.hi(g) << g.th_sh, n0 = tw.ni(g) * g.tn;
            const int k0 = nt * g.bn;
            const int ow = ow0 + lw, oh = oh0 + lh, img = n0 + ln;
            const bool pix_valid = ow < g.ow && oh < g.oh && img < g.n;
            const uint8_t *res_row = g.res;
            if ((HAS_RES && g.res != nullptr) && pix_valid)
                res_row += (((size_t)img * g.oh + oh) * g.ow + ow) * g.cout + k0;
            // wzp != 128: this pixel's correction, the same for every channel
            int wz_t = 0;
            if (HAS_WZP && pix_valid)
                wz_t = -g.wzp_d * __ldg(g.wsum + ((size_t)img * g.oh + oh) * g.ow + ow);
            const long long *off_row = g.off + k0;
            if (!single_class)
                off_row += (size_t)((int)g.row_cls[min(oh, g.oh - 1)] * g.n_col_cls + (int)g.col_cls[min(ow, g.ow - 1)]) * g.kpad;

            // per-channel tables change with the channel tile: the group meets before (everyone is
            // past the previous tile's reads) and after the reload
            if (nt != cur_nt && (HAS_RES || !g.epi_const)) {
                epi_bar_sync(group, group_threads);
                for (int j = et; j < g.bn; j += group_threads) {
                    const int sft = g.shift[k0 + j];
                    s_mult[j] = (int)g.mult[k0 + j];
                    s_shift[j] = fast_epi ? sft - 32 : sft;   // the fast form shifts the high word only
                    if (single_class)
                        s_off[j] = g.off[k0 + j];
                }
                epi_bar_sync(group, group_threads);
                cur_nt = nt;
            }
            if (!failed) {
                // this warp's previous store must have finished reading its part of the staging buffer
                if (store_pending) {
                    if (lane == 0)
                        tma_store_wait_read();
                    __syncwarp();
                }
                if (!__all_sync(0xffffffffu, mbar_wait(tfull_bar(as), aphase, abort_flag))) {
                    if (lane == 0) {
                        atomicCAS(g.status, 0, kErrEpilogueWait);
                        *abort_flag = 1;
                    }
                    failed = true;
                }
            }
            if (!failed) {
                tc_fence_after();
                const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(as * g.bn);
                if (!HAS_RES && g.epi_const) {
                const long long rnd = ((long long)g.rnd_hi << 32) | (unsigned long long)(uint32_t)g.rnd_lo;
                const int32_t *off_row32 = g.off32;
                if (!single_class)
                    off_row32 += (size_t)((int)g.row_cls[min(oh, g.oh - 1)] * g.n_col_cls + (int)g.col_cls[min(ow, g.ow - 1)]) * g.kpad;
#define B200_EPI_TILE(CH0, CH1)                                                                                                   \
    do {                                                                                                                          \
        if (single_class) {                                                                                                       \
            if (no_floor)                                                                                                         \
                epi_tile_const<CH0, CH1, true, false, HAS_WZP>(t_row, g.bn, tab, off_row32, rnd, g.ushift, g.relu_lo, wz_t, s_out, g.ob, g.ob_sh, sw, row, tempty_bar(as), lane); \
            else                                                                                                                  \
                epi_tile_const<CH0, CH1, true, true, HAS_WZP>(t_row, g.bn, tab, off_row32, rnd, g.ushift, g.relu_lo, wz_t, s_out, g.ob, g.ob_sh, sw, row, tempty_bar(as), lane);  \
        } else {                                                                                                                  \
            if (no_floor)                                                                                                         \
                epi_tile_const<CH0, CH1, false, false, HAS_WZP>(t_row, g.bn, tab, off_row32, rnd, g.ushift, g.relu_lo, wz_t, s_out, g.ob, g.ob_sh, sw, row, tempty_bar(as), lane); \
            else                                                                                                                  \
                epi_tile_const<CH0, CH1, false, true, HAS_WZP>(t_row, g.bn, tab, off_row32, rnd, g.ushift, g.relu_lo, wz_t, s_out, g.ob, g.ob_sh, sw, row, tempty_bar(as), lane);  \
        }                                                                                                                         \
    } while (0)
                // epi_const = (first chunk << 4) | chunk count of this warp's column range, per sub-warp
                switch ((g.epi_const >> (8 * sub_warp)) & 0xff) {
                case 0x01: B200_EPI_TILE(0, 1); break;
                case 0x02: B200_EPI_TILE(0, 2); break;
                case 0x03: B200_EPI_TILE(0, 3); break;
                case 0x04: B200_EPI_TILE(0, 4); break;
                case 0x22: B200_EPI_TILE(2, 4); break;
                case 0x08: B200_EPI_TILE(0, 8); break;
                default: B200_EPI_TILE(4, 8); break;   // 0x44
                }
#undef B200_EPI_TILE
                } else
                for (int c0 = 0; c0 < g.bn; c0 += 32) {
                    if (((c0 >> own_sh) & (wpq - 1)) != sub_warp)
                        continue;
                    uint32_t v[32];
                    uint32_t rv[8] = { 0, 0, 0, 0, 0, 0, 0, 0 };
                    const int ncol = min(32, g.bn - c0);   // 32, or 16 for the last chunk of bn % 32 == 16
                    if (ncol == 32)
                        tmem_ld32(t_row + c0, v);
                    else
                        tmem_ld16(t_row + c0, v);
                    if ((HAS_RES && g.res != nullptr) && pix_valid) {
                        // the residual bytes of this pixel's 32 channels, in flight with the accumulator read
                        const uint4 *rp = reinterpret_cast<const uint4 *>(res_row + c0);
                        const uint4 ra = __ldg(rp), rb = __ldg(rp + 1);
                        rv[0] = ra.x; rv[1] = ra.y; rv[2] = ra.z; rv[3] = ra.w;
                        rv[4] = rb.x; rv[5] = rb.y; rv[6] = rb.z; rv[7] = rb.w;
                    }
                    tmem_ld_wait();
                    if (HAS_WZP) {
                        if (ncol == 32) {
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                v[i] += (uint32_t)wz_t;
                        } else {
#pragma unroll
                            for (int i = 0; i < 16; ++i)
                                v[i] += (uint32_t)wz_t;
                        }
                    }
                    // the common case is one straight-line block of 32 independent chains
                    if ((HAS_RES && g.res != nullptr)) {          // host guarantees the fast form and whole 32-column chunks
                        if (single_class)
                            epi_chunk<true, true, 32, true, true>(v, c0, off_row, ec, rv);
                        else
                            epi_chunk<true, false, 32, true, true>(v, c0, off_row, ec, rv);
                    } else if (fast_epi && ncol == 32) {
                        if (single_class) {
                            if (no_floor)
                                epi_chunk<true, true, 32, false>(v, c0, off_row, ec, rv);
                            else
                                epi_chunk<true, true, 32>(v, c0, off_row, ec, rv);
                        } else {
                            if (no_floor)
                                epi_chunk<true, false, 32, false>(v, c0, off_row, ec, rv);
                            else
                                epi_chunk<true, false, 32>(v, c0, off_row, ec, rv);
                        }
                    } else if (fast_epi) {
                        epi_chunk<true, false, 16>(v, c0, off_row, ec, rv);
                    } else if (ncol == 32) {
                        epi_chunk<false, false, 32>(v, c0, off_row, ec, rv);
                    } else {
                        epi_chunk<false, false, 16>(v, c0, off_row, ec, rv);
                    }
                }
                // accumulator stage drained: hand it back to the MMA warp (the uniform-shift form has
                // done so already, after its last tensor-memory read)
                if (HAS_RES || !g.epi_const) {
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0)
                        tempty_arrive(as);
                }

                if (g.use_tma_store) {
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        for (int sub = 0; sub < n_sub; ++sub) {
                            // ownership is by granules of max(ob, 32) bytes (with ob == 16 two neighbouring
                            // sub-tiles form one granule)
                            if (((((sub << g.ob_sh) >> own_sh) & (wpq - 1)) == sub_warp) && k0 + (sub << g.ob_sh) < g.cout)
                                tma_store_4d(&maps.y, smem_u32(s_out + (((size_t)sub * kTileM + p0) << g.ob_sh)),
                                             k0 + (sub << g.ob_sh), ow0 + qlw, oh0 + qlh, n0 + qln);
                        }
                        tma_store_commit();
                    }
                    store_pending = true;
                } else {
                    // plain stores for channel counts the TMA store cannot address (Cout % 16 != 0):
                    // every thread copies the columns its warp computed for its pixel
                    __syncwarp();
                    if (pix_valid) {
                        uint8_t *dst = g.y + (((size_t)img * g.oh + oh) * g.ow + ow) * g.cout + k0;
                        const int nvalid = min(g.bn, g.cout - k0);
                        for (int j = 0; j < nvalid; ++j) {
                            if (((j >> own_sh) & (wpq - 1)) != sub_warp)
                                continue;
                            const int sub = j >> g.ob_sh, cin = j & (g.ob - 1);
                            const int chunk = cin >> 4;
                            dst[j] = s_out[(((size_t)sub * kTileM + row) << g.ob_sh) + ((chunk ^ sw) << 4) + (cin & 15)];
                        }
                    }
                    __syncwarp();
                }
            }
            as += g.groups;                          // the group's next tile: stage (as + groups) mod acc_stages
            if (as >= g.acc_stages) {
                as -= g.acc_stages;
                aphase ^= 1;
            }
            for (int i = 0; i < g.groups; ++i)
                tw.advance(g);
        }
        if (store_pending && lane == 0)
            tma_store_wait_all();
    }

    // ---- common exit: every role gets here (all waits are bounded) ---------------------------------
    tc_fence_before();
    __syncthreads();
    if (PAIR)
        cluster_sync_all();     // neither CTA leaves (or gives tensor memory back) while its peer still works on the pair
    if (warp == 1) {
        tc_fence_after();
        if (PAIR)
            tmem_dealloc_pair(tmem_base, g.tmem_cols);
        else
            tmem_dealloc(tmem_base, g.tmem_cols);
    }
}

// The give-up path of the bounded waits, on its own: one warp waits, through the same mbar_wait the
// convolution's roles use, on a barrier that nothing will ever arrive at, with the caller's (short)
// limit.  When the limit is reached the wait returns false, the code goes to the status word and the
// kernel ends normally -- no trap, nothing left waiting.
__global__ void __launch_bounds__(32) wait_expiry_probe_kernel(int *status, long long limit_cycles)
{
    __shared__ __align__(8) unsigned long long bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncwarp();
    const bool ok = mbar_wait(smem_u32(&bar), 0, &abort_flag, limit_cycles);
    if (!__all_sync(0xffffffffu, ok) && threadIdx.x == 0) {
        atomicCAS(status, 0, kErrSelfTestWait);
        abort_flag = 1;
    }
}

// The tensor pipe's own rate for this kernel's instruction: every SM issues `mmas` MMAs of the shape the
// 256-wide tiles use (kind::i8, M128 x N256 x K32, u8 x s8 -> s32) back to back on operands that stay in
// shared memory (pseudo-random bytes: all-zero operands would draw less power and run at other clocks),
// alternating between two accumulators every 32 MMAs.  No loads, no epilogue: the number it gives is the
// ceiling the convolution's mainloop is measured against.
constexpr int kPeakGroup = 32;   // MMAs per commit
__global__ void __launch_bounds__(128, 1) mma_i8_peak_kernel(int mmas, int *status)
{
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t *smem = smem_raw + (base - raw_addr);
    constexpr uint32_t kA = 128 * 128, kB = 256 * 128;
    __shared__ __align__(8) unsigned long long bars[2];
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    for (uint32_t i = threadIdx.x; i < (kA + kB) / 4; i += blockDim.x)
        reinterpret_cast<uint32_t *>(smem)[i] = (i + blockIdx.x) * 2654435761u;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bars[0]), 1);
        mbar_init(smem_u32(&bars[1]), 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    fence_async_smem();
    if (threadIdx.x < 32) {
        tmem_alloc(smem_u32(&tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;
    if (threadIdx.x < 32) {
        const uint32_t lead = threadIdx.x == 0 ? 1u : 0u;
        const uint64_t adesc = make_smem_desc(base, 128), bdesc = make_smem_desc(base + kA, 128);
        const uint32_t desc_hi = (uint32_t)(adesc >> 32), a_lo = (uint32_t)adesc, b_lo = (uint32_t)bdesc;
        const uint32_t idesc = (2u << 4) | (0u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);
        const int groups = mmas / kPeakGroup;
        uint32_t phase[2] = { 0, 0 };
        bool ok = true;
        for (int gi = 0; gi < groups && ok; ++gi) {
            const int b = gi & 1;
            if (gi >= 2) {     // the group two back has drained: at most two groups are queued
                if (!mbar_wait(smem_u32(&bars[b]), phase[b], &abort_flag)) {
                    if (lead)
                        atomicCAS(status, 0, kErrSelfTestWait);
                    ok = false;
                    break;
                }
                phase[b] ^= 1;
            }
            const uint32_t d = tmem_base + (uint32_t)b * 256u;
#pragma unroll 4
            for (int j = 0; j < kPeakGroup; ++j)
                mma_i8(d, a_lo + 2 * (j & 3), b_lo + 2 * (j & 3), desc_hi, idesc, j ? 1u : 0u, lead);
            mma_commit(smem_u32(&bars[b]), lead);
        }
        // the last groups must have finished before tensor memory goes back
        for (int t = groups < 2 ? 0 : groups - 2; t < groups && ok; ++t) {
            const int b = t & 1;
            if (!mbar_wait(smem_u32(&bars[b]), phase[b], &abort_flag)) {
                if (lead)
                    atomicCAS(status, 0, kErrSelfTestWait);
                ok = false;
            }
            phase[b] ^= 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x < 32) {
        tc_fence_after();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---- host side -------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(
    CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
    const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess
            && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

CUtensorMapSwizzle swizzle_for(int bytes)
{
    return bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
        : bytes == 64   ? CU_TENSOR_MAP_SWIZZLE_64B
        : bytes == 32   ? CU_TENSOR_MAP_SWIZZLE_32B
                        : CU_TENSOR_MAP_SWIZZLE_NONE;
}

int encode(CUtensorMap *m, void *base, int rank, const cuuint64_t *dims, const cuuint64_t *strides_bytes,
           const cuuint32_t *box, CUtensorMapSwizzle sw, CUtensorMapDataType dtype = CU_TENSOR_MAP_DATA_TYPE_UINT8)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn)
        return fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    cuuint32_t estr[5] = { 1, 1, 1, 1, 1 };
    CUresult r = fn(m, dtype, (cuuint32_t)rank, base, dims, strides_bytes, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu %llu, box %u %u)",
                    (int)r, rank, (unsigned long long)dims[0], (unsigned long long)dims[1], box[0], box[1]);
    return B200_OK;
}

}  // namespace

struct ConvIgemmPlan {
    ConvGeom g;
    int groups = 2, acc_stages = 2;
    int cpad = 0;                   // input channels rounded up to a multiple of 32
    int bk = 0, bn = 0, stages = 0, kgroup = 1, ob = 0, kpad = 0, b_resident = 0, a_wide = 0, mma_warps = 1, pair = 0;
    // Two CTAs of a cluster per MMA (kernel MODE 3).  Whether a launch uses it depends on the batch: the pair
    // wins 3-6 % once every cluster walks many tiles and loses a little on short launches (cluster launch,
    // two cluster-wide syncs), so the plan carries both configurations and build_launch picks.
    int pair_ok = 0, pair_want = -1, stages_pair = 0;
    int cta_pair = 0;               // the configuration of the current launch
    int max_clusters = 0;           // co-resident CTA pairs of that kernel on this device
    int n_row_cls = 0, n_col_cls = 0;
    int generic_requant = 0;
    int8_t *w_dev = nullptr;        // [kpad][r][s][c]
    long long *off_dev = nullptr;   // [n_cls][kpad]
    uint32_t *mult_dev = nullptr;   // [kpad]
    int32_t *shift_dev = nullptr;   // [kpad]
    uint8_t *row_cls_dev = nullptr, *col_cls_dev = nullptr;
    // uniform-shift epilogue (IgemmArgs::epi_const)
    int rev = 0;                    // reversed tile traversal (conv_igemm_set_reverse)
    const uint8_t *next_ro = nullptr;   // what the next launch reads first (conv_igemm_set_next_readonly)
    uint32_t next_ro_bytes = 0;
    size_t w_bytes = 0;             // size of w_dev
    int epi_const = 0, ushift = 0;
    long long rnd = 0;
    int32_t *off32_dev = nullptr;   // [n_cls][kpad]
    EpiTab tab;
    // fused residual add (conv_igemm_set_residual)
    bool has_res = false;
    int r_m[2] = { 0, 0 }, r_add[2] = { 0, 0 }, r_b[2] = { 1, 1 };
    int r_s0 = 1, r_ozp = 0, r_lo = 0;
    // tensor maps of the last (x, y, n) seen
    const uint8_t *last_res = nullptr;
    const uint8_t *last_x = nullptr;
    uint8_t *last_y = nullptr;
    int last_n = -1;
    int *last_status = nullptr;
    IgemmMaps maps;
    IgemmArgs args;
    dim3 grid;
    size_t smem = 0;
    bool attr_set = false;
    // a few earlier launch configurations (callers that rotate through a handful of buffers)
    struct Saved {
        const uint8_t *x;
        const uint8_t *res;
        uint8_t *y;
        int n;
        int *status;
        IgemmMaps maps;
        IgemmArgs args;
        dim3 grid;
        size_t smem;
        int cta_pair;
    };
    static constexpr size_t kMaxSaved = 8;
    std::vector<Saved> saved;
    size_t next_saved = 0;
};

int conv_igemm_supported(const ConvGeom &g, char *why, size_t why_len)
{
    const char *msg = nullptr;
    if (g.group != 1) msg = "group != 1";
    else if (g.c % 16 != 0) msg = "input channels not a multiple of 16";   // the pixel stride of a TMA map
    else if (g.k < 16) msg = "fewer than 16 output channels";
    else if (g.stride_h > 2 || g.stride_w > 2) msg = "stride > 2";
    else if (g.h < g.stride_h || g.w < g.stride_w) msg = "input smaller than the stride";
    else if ((long long)g.r * g.s * ((g.c + 31) / 32) >= 32768) msg = "more than 32767 k-blocks per tile";
    if (msg) {
        snprintf(why, why_len, "%s", msg);
        return 0;
    }
    return 1;
}

// Distinct sets of in-image taps along one axis: cls[o] = class of output coordinate o, and
// valid[class] = bit mask of taps that fall inside the image.
static void tap_classes(int out, int in, int kernel, int pad, int stride, std::vector<uint8_t> &cls,
                        std::vector<std::vector<char>> &valid)
{
    cls.resize(out);
    valid.clear();
    for (int o = 0; o < out; ++o) {
        std::vector<char> v(kernel);
        for (int t = 0; t < kernel; ++t) {
            int i = o * stride + t - pad;
            v[t] = (i >= 0 && i < in) ? 1 : 0;
        }
        int id = -1;
        for (size_t j = 0; j < valid.size(); ++j)
            if (valid[j] == v) {
                id = (int)j;
                break;
            }
        if (id < 0) {
            valid.push_back(v);
            id = (int)valid.size() - 1;
        }
        cls[o] = (uint8_t)id;
    }
}

int conv_igemm_create(
    const ConvGeom &g, const std::vector<int8_t> &w_s8, const int32_t *bias, const uint32_t *mult,
    const int32_t *shift, ConvIgemmPlan **out, bool a_row_swizzled)
{
    if (a_row_swizzled && !(g.c == 32 && g.s == 1 && g.stride_w == 1 && g.pad_w == 0 && g.w == g.ow))
        return fail(B200_ERR_INVALID, "conv(igemm): pre-swizzled rows need 32 channels and an r x 1 kernel");
    // The epilogue adds the accumulator offset in 64-bit arithmetic, where the reference's int32
    // accumulator would wrap; and its folded addend needs shift <= 53 to stay inside int64.
    {
        long long max_bias = 0;
        for (int k = 0; k < g.k && bias; ++k) {
            long long b = bias[k] < 0 ? -(long long)bias[k] : (long long)bias[k];
            if (b > max_bias)
                max_bias = b;
        }
        const long long wmag = 128ll + (g.wzp_d < 0 ? -g.wzp_d : g.wzp_d);   // |s8| plus the zero-point correction
        if (max_bias + (long long)g.r * g.s * g.c * 255ll * wmag >= (1ll << 31))
            return fail(B200_ERR_UNSUPPORTED, "conv(igemm): the int32 accumulator could wrap");
        for (int k = 0; k < g.k; ++k)
            if (shift[k] > 53)
                return fail(B200_ERR_UNSUPPORTED, "conv(igemm): shift %d of channel %d exceeds 53", shift[k], k);
    }
    ConvIgemmPlan *p = new ConvIgemmPlan();
    p->g = g;
    p->saved.reserve(ConvIgemmPlan::kMaxSaved);   // launches never grow it: a later run touches no heap
    p->a_wide = a_row_swizzled ? 1 : 0;
    // K of an 8-bit MMA is 32 bytes: the channel count is rounded up to a multiple of 32 in the
    // repacked weights (zero weights); on the activation side the TMA box runs past the tensor's
    // channel extent and reads zeros there
    p->cpad = (g.c + 31) / 32 * 32;
    p->bk = p->cpad % 128 == 0 ? 128 : (p->cpad % 64 == 0 ? 64 : 32);
    // output-channel tile: a multiple of 16 up to 256 that wastes little of Cout
    {
        const int k16 = (g.k + 15) / 16 * 16;
        if (k16 <= 256) {
            p->bn = k16;
        } else {
            int best = 256, best_waste = 1 << 30;
            for (int bn = 256; bn >= 128; bn -= 16) {
                int tiles = (g.k + bn - 1) / bn;
                int waste = tiles * bn - g.k;
                if (waste < best_waste) {
                    best_waste = waste;
                    best = bn;
                }
            }
            p->bn = best;
        }
    }
    // a 1x1 output map (an inner product run as a full-image conv) has one row per image, far too few
    // row tiles to fill the SMs at any usual batch: narrow channel tiles spread the weight matrix over
    // many CTAs instead (2048 -> 1000 at batch 256: 8 CTAs and 0.035 ms at 256 wide, 64 CTAs and < 0.02 ms at 32)
    if (g.oh * g.ow == 1 && g.k >= 32)
        p->bn = 32;
    if (const char *e = getenv("B200_IGEMM_BN")) {   // tuning aid: channel-tile width, a multiple of 16 up to 256
        int v = atoi(e);
        if (v >= 16 && v <= 256 && v % 16 == 0 && v <= (g.k + 15) / 16 * 16)
            p->bn = v;
    }
    const int n_tiles_n = (g.k + p->bn - 1) / p->bn;
    p->kpad = n_tiles_n * p->bn;
    // pipeline depth from the shared memory left after the staging buffer
    {
        const int kblocks = g.r * g.s * (p->cpad / p->bk);
        // weights resident when there is one channel tile and they leave room for >= 3 A stages
        // four epilogue groups (four tiles in flight behind the mainloop) when the tiles are narrow:
        // their per-tile latency chain, not their arithmetic, sets the epilogue rate
        p->groups = (p->bn <= 64 || (p->bn <= 128 && kblocks * p->bk <= 256)) ? 4 : 2;
        if (const char *e = getenv("B200_IGEMM_GROUPS")) {   // tuning aid: 2, or 4 when four accumulators fit
            int v = atoi(e);
            if (v == 2 || (v == 4 && 4 * p->bn <= 512))
                p->groups = v;
        }
        // staging sub-tile width: the largest of 128/64/32/16 that divides bn and, where possible,
        // gives the warps that share a lane quarter the same number of sub-tiles
        {
            const int wpq = (kEpiWarps / p->groups) / 4;
            p->ob = 0;
            for (int ob = 128; ob >= 16 && !p->ob; ob >>= 1)
                if (p->bn % ob == 0 && (p->bn / ob) % wpq == 0)
                    p->ob = ob;
            if (!p->ob)
                p->ob = p->bn % 128 == 0 ? 128 : (p->bn % 64 == 0 ? 64 : (p->bn % 32 == 0 ? 32 : 16));
        }
        p->acc_stages = 4 * p->bn <= 512 ? 4 : p->groups;
        if (const char *e = getenv("B200_IGEMM_ACC")) {
            int v = atoi(e);
            if ((v == 2 || v == 4) && v * p->bn <= 512 && v >= p->groups)
                p->acc_stages = v;
        }
        p->b_resident = n_tiles_n == 1 && smem_layout(3, kblocks, p->bk, p->bn, p->groups).total + 1024 <= 227 * 1024;
        // Narrow k-blocks (few bytes per barrier round trip) travel in groups: the largest divisor of
        // the tile's k-blocks that keeps a stage at or under kGroupBytes.
        const int kb_bytes = kTileM * p->bk + (p->b_resident ? 0 : p->bn * p->bk);
        int kgroup = 1;
        for (int d = 1; d <= kblocks; ++d)
            if (kblocks % d == 0 && d * kb_bytes <= kGroupBytes && d <= kMaxGroup)
                kgroup = d;
        if (const char *e = getenv("B200_IGEMM_KGROUP")) {   // tuning aid: a divisor of the k-blocks, else ignored
            int v = atoi(e);
            if (v >= 1 && v <= kMaxGroup && kblocks % v == 0)
                kgroup = v;
        }
        int stages = kMaxStages;
        auto fits = [&](int st, int kg) {
            return smem_layout(st * kg, p->b_resident ? kblocks : st * kg, p->bk, p->bn, p->groups).total + 1024 <= 227 * 1024;
        };
        while (kgroup > 1 && !fits(3, kgroup)) {   // keep at least three stages in flight
            int d = kgroup - 1;
            while (kblocks % d != 0)
                --d;
            kgroup = d;
        }
        while (stages > 2 && (!fits(stages, kgroup) || stages * kgroup > 32))
            --stages;
        // a deep ring lets the producer run several tiles ahead when a tile has few k-blocks
        // Narrow channel tiles make short MMAs, and one thread issues those no faster than one per
        // ~100 cycles whatever their size: two issuing warps, each on its own half of the ring and on
        // every second tile, keep the tensor pipe fed (3x3 64-channel layer: 0.082 -> 0.061 ms; 256-wide
        // tiles gain nothing).
        p->mma_warps = (p->bn <= 128 && stages >= 4) ? 2 : 1;
        if (const char *e = getenv("B200_IGEMM_MMA_WARPS")) {   // tuning aid: 1, or 2 when the ring has four stages or more
            int v = atoi(e);
            if (v == 1 || (v == 2 && stages >= 4))
                p->mma_warps = v;
        }
        if (p->mma_warps == 2)
            stages &= ~1;
        // Pair mode (see the kernel's MODE 2): wide k-blocks of a layer with one channel tile, where the
        // operand loads from L2 set the pace: two tiles per stage share one weight tile.
        // (3x3 128-channel layer 0.047 -> 0.043 ms.  256-wide tiles lose: their two accumulators fill the
        // tensor memory, so the next pair's mainloop cannot overlap this pair's epilogue: 0.039 -> 0.044 ms.)
        const bool pair_off = getenv("B200_IGEMM_PAIR") && atoi(getenv("B200_IGEMM_PAIR")) == 0;   // tuning aid
        if (!pair_off && !p->b_resident && kgroup == 1 && !p->a_wide && n_tiles_n == 1 && p->bn <= 128) {
            int st = kMaxStages;
            auto fits2 = [&](int n) { return smem_layout(2 * n, n, p->bk, p->bn, p->groups).total + 1024 <= 227 * 1024; };
            while (st > 2 && !fits2(st))
                --st;
            if (fits2(st)) {
                p->pair = 1;
                p->mma_warps = 2;
                stages = st;
            }
        }
        // CTA pair (the kernel's MODE 3): two CTAs of a cluster run every MMA together (cta_group::2, M = 256),
        // each loading its own activation tile and half of the weight tile.  A 256-wide MMA of one CTA reads
        // 12 KB of operands from shared memory while TMA writes the next 12 KB into it, which is more than the
        // shared memory moves per MMA time; the pair halves the weight bytes per SM on both sides.  For the
        // layers whose mainloop sets the pace: 256-wide tiles with at least 1 KB of reduction per pixel.
        {
            const char *e = getenv("B200_IGEMM_CTA_PAIR");     // tuning aid: 0 never, 1 wherever possible
            p->pair_want = e ? atoi(e) : -1;
            const bool can = !p->b_resident && !p->a_wide && !p->pair && p->bn % 32 == 0 && p->bn >= 64 && g.wzp_d == 0;
            const bool automatic = p->bn == 256 && kblocks * p->bk >= 1024;
            if (can && (p->pair_want == 1 || (p->pair_want == -1 && automatic))) {
                auto fits_p = [&](int st, int kg) {
                    return smem_layout(st * kg, st * kg, p->bk, p->bn, p->groups, p->bn / 2).total + 1024 <= 227 * 1024;
                };
                int st = kMaxStages;
                while (st > 2 && (!fits_p(st, kgroup) || st * kgroup > 32))
                    --st;
                if (fits_p(st, kgroup) && p->mma_warps == 1) {
                    p->pair_ok = 1;
                    p->stages_pair = st;
                }
            }
        }
        p->stages = stages;
        p->kgroup = kgroup;
    }
    if (smem_layout((p->pair ? 2 : 1) * p->stages * p->kgroup, p->b_resident ? g.r * g.s * (p->cpad / p->bk) : p->stages * p->kgroup, p->bk, p->bn, p->groups).total + 1024 > 227 * 1024) {
        delete p;
        return fail(B200_ERR_UNSUPPORTED, "conv(igemm): tile does not fit shared memory");
    }

    const int taps = g.r * g.s;
    // ---- weights [kpad][r][s][c] ---------------------------------------------------------------
    std::vector<int8_t> wp((size_t)p->kpad * taps * p->cpad, 0);
    for (int k = 0; k < g.k; ++k)
        for (int c = 0; c < g.c; ++c)
            for (int t = 0; t < taps; ++t)
                wp[((size_t)k * taps + t) * p->cpad + c] = w_s8[((size_t)k * g.c + c) * taps + t];
    // ---- border classes and offsets ---------------------------------------------------------------
    std::vector<uint8_t> row_cls, col_cls;
    std::vector<std::vector<char>> row_valid, col_valid;
    tap_classes(g.oh, g.h, g.r, g.pad_h, g.stride_h, row_cls, row_valid);
    tap_classes(g.ow, g.w, g.s, g.pad_w, g.stride_w, col_cls, col_valid);
    p->n_row_cls = (int)row_valid.size();
    p->n_col_cls = (int)col_valid.size();
    if (p->n_row_cls > 255 || p->n_col_cls > 255) {
        delete p;
        return fail(B200_ERR_UNSUPPORTED, "conv(igemm): too many border classes");
    }
    std::vector<long long> wtap((size_t)g.k * taps, 0);   // sum over channels per (k, tap)
    for (int k = 0; k < g.k; ++k)
        for (int c = 0; c < g.c; ++c)
            for (int t = 0; t < taps; ++t)
                wtap[(size_t)k * taps + t] += w_s8[((size_t)k * g.c + c) * taps + t];
    std::vector<long long> off((size_t)p->n_row_cls * p->n_col_cls * p->kpad, 0);
    std::vector<int32_t> off32_all(off.size(), 0);   // the same offsets as plain int32 (uniform-shift epilogue)
    for (int rc = 0; rc < p->n_row_cls; ++rc)
        for (int cc = 0; cc < p->n_col_cls; ++cc)
            for (int k = 0; k < g.k; ++k) {
                long long sum = 0;
                for (int rr = 0; rr < g.r; ++rr)
                    if (row_valid[rc][rr])
                        for (int ss = 0; ss < g.s; ++ss)
                            if (col_valid[cc][ss])
                                sum += wtap[(size_t)k * taps + rr * g.s + ss];
                // int8 activations reach the tensor cores as signed bytes and TMA pads with a true zero: no correction
                long long v = (long long)(bias ? bias[k] : 0) - (long long)(g.act_signed ? 0 : g.izp) * sum;
                // the int32 accumulator offset, folded with the multiplier, the rounding term and the
                // output zero point into the 64-bit addend of the epilogue's multiply-add
                const long long off32 = (long long)(int32_t)(uint32_t)(unsigned long long)v;
                off32_all[((size_t)rc * p->n_col_cls + cc) * p->kpad + k] = (int32_t)off32;
                off[((size_t)rc * p->n_col_cls + cc) * p->kpad + k]
                    = off32 * (long long)mult[k] + (1ll << (shift[k] - 1)) + ((long long)g.ozp << shift[k]);
            }
    std::vector<uint32_t> multp(p->kpad, 0);
    std::vector<int32_t> shiftp(p->kpad, 33);
    for (int k = 0; k < g.k; ++k) {
        multp[k] = mult[k];
        shiftp[k] = shift[k];
        if (shift[k] < 32)
            p->generic_requant = 1;
    }
    if (g.act_signed)
        p->generic_requant = 1;     // the generic form carries the ceiling below 255 and the output's bit flip
    // Uniform shift: the multipliers come from an fp32 scale, so their low 7 bits are zero; a channel
    // whose shift lies d above the layer's smallest one, S, is served exactly by (mult >> d, S) when those
    // d bits are zero:  (t * mult + 2^(shift-1)) / 2^shift == (t * (mult >> d) + 2^(S-1)) / 2^S.
    memset(&p->tab, 0, sizeof(p->tab));
    {
        int smin = 127;
        for (int k = 0; k < g.k; ++k)
            smin = shift[k] < smin ? shift[k] : smin;
        bool uni = smin >= 33 && !p->generic_requant && g.qmax == 255 && g.k % 16 == 0 && n_tiles_n == 1 && p->bn % 32 == 0 && !p->a_wide;
        for (int k = 0; k < g.k && uni; ++k) {
            const int d = shift[k] - smin;
            uni = d <= 7 && (mult[k] & ((1u << d) - 1u)) == 0;
        }
        // each warp of a lane quarter takes a contiguous range of 32-column chunks: (first << 4) | count,
        // one byte per warp of the quarter; only the ranges the kernel has code for qualify
        const int wpq = (kEpiWarps / p->groups) / 4;
        const int chunks = p->bn / 32;
        int ranges = 0;
        if (wpq == 1 && (chunks <= 4 || chunks == 8))
            ranges = chunks;
        else if (wpq == 2 && p->bn == 256 && p->ob == 128)
            ranges = 0x04 | (0x44 << 8);
        else if (wpq == 2 && p->bn == 128 && p->ob == 64)
            ranges = 0x02 | (0x22 << 8);
        if (ranges == 0)
            uni = false;
        if (getenv("B200_IGEMM_EPI_CONST") && atoi(getenv("B200_IGEMM_EPI_CONST")) == 0)   // tuning aid
            uni = false;
        if (uni) {
            p->epi_const = ranges;
            p->ushift = smin - 32;
            p->rnd = (1ll << (smin - 1)) + ((long long)g.ozp << smin);
            for (int k = 0; k < g.k; ++k)
                p->tab.mult[k] = (int32_t)(mult[k] >> (shift[k] - smin));
            for (int k = 0; k < g.k; ++k)
                p->tab.off32[k] = off32_all[k];          // class 0: all there is when the layer has one class
        }
    }
    auto up = [](const void *src, size_t bytes, void **dst) -> int {
        B200_CUDA_TRY(cudaMalloc(dst, bytes));
        B200_CUDA_TRY(cudaMemcpy(*dst, src, bytes, cudaMemcpyHostToDevice));
        return B200_OK;
    };
    p->w_bytes = wp.size();
    int rc = up(wp.data(), wp.size(), (void **)&p->w_dev);
    if (rc == B200_OK) rc = up(off.data(), off.size() * 8, (void **)&p->off_dev);
    if (rc == B200_OK) rc = up(off32_all.data(), off32_all.size() * 4, (void **)&p->off32_dev);
    if (rc == B200_OK) rc = up(multp.data(), multp.size() * 4, (void **)&p->mult_dev);
    if (rc == B200_OK) rc = up(shiftp.data(), shiftp.size() * 4, (void **)&p->shift_dev);
    if (rc == B200_OK) rc = up(row_cls.data(), row_cls.size(), (void **)&p->row_cls_dev);
    if (rc == B200_OK) rc = up(col_cls.data(), col_cls.size(), (void **)&p->col_cls_dev);
    if (rc != B200_OK) {
        conv_igemm_destroy(p);
        return rc;
    }
    *out = p;
    return B200_OK;
}

void conv_igemm_destroy(ConvIgemmPlan *p)
{
    if (!p)
        return;
    cudaFree(p->w_dev);
    cudaFree(p->off_dev);
    cudaFree(p->off32_dev);
    cudaFree(p->mult_dev);
    cudaFree(p->shift_dev);
    cudaFree(p->row_cls_dev);
    cudaFree(p->col_cls_dev);
    delete p;
}

// Chooses the M-tile box (tw, th, tn), powers of two with product 128, that covers the output with
// the fewest tiles; ties go to the wider box.
static void choose_tile(int ow, int oh, int n, int *tw, int *th, int *tn, int min_a = 0, int max_a = 7)
{
    long long best = -1;
    for (int a = min_a; a <= max_a; ++a)
        for (int b = 0; a + b <= 7; ++b) {
            int w = 1 << a, h = 1 << b, nn = 1 << (7 - a - b);
            long long tiles = (long long)((ow + w - 1) / w) * ((oh + h - 1) / h) * ((n + nn - 1) / nn);
            if (best < 0 || tiles < best || (tiles == best && w > *tw)) {
                best = tiles;
                *tw = w;
                *th = h;
                *tn = nn;
            }
        }
}

void conv_igemm_describe(const ConvIgemmPlan *p, char *buf, size_t len)
{
    const char *mode = p->cta_pair ? "cta-pair (cta_group::2, M=256)" : p->pair ? "tile pairs on one weight tile"
        : p->pair_ok ? "one issuing warp (cta pairs on long launches)"
        : p->mma_warps == 2 ? "two issuing warps" : "one issuing warp";
    snprintf(buf, len, "tcgen05 igemm: bn=%d bk=%d stages=%d kgroup=%d groups=%d acc_stages=%d %s%s%s%s", p->bn, p->bk,
             p->cta_pair ? p->stages_pair : p->stages, p->kgroup, p->groups, p->acc_stages, mode, p->b_resident ? ", weights resident" : "",
             (p->epi_const && !p->cta_pair) ? ", uniform-shift epilogue" : (p->generic_requant ? ", generic requantize" : ""),
             p->rev ? ", reversed" : "");
}

void conv_igemm_set_reverse(ConvIgemmPlan *p, int reverse)
{
    if (p->rev != (reverse ? 1 : 0)) {
        p->rev = reverse ? 1 : 0;
        p->last_n = -1;        // cached launch configurations carry the old direction
        p->saved.clear();
    }
}

void conv_igemm_weights(const ConvIgemmPlan *p, const uint8_t **ptr, size_t *bytes)
{
    *ptr = reinterpret_cast<const uint8_t *>(p->w_dev);
    *bytes = p->w_bytes;
}

void conv_igemm_set_next_readonly(ConvIgemmPlan *p, const uint8_t *ptr, size_t bytes)
{
    // 16-byte granules (the bulk prefetch's unit); anything beyond 64 MiB would only evict what the layers between need
    if (((uintptr_t)ptr & 15) != 0 || bytes > (64u << 20))
        ptr = nullptr;
    const uint32_t b = ptr ? (uint32_t)(bytes & ~(size_t)15) : 0u;
    if (p->next_ro != ptr || p->next_ro_bytes != b) {
        p->next_ro = ptr;
        p->next_ro_bytes = b;
        p->last_n = -1;
        p->saved.clear();
    }
}

int conv_igemm_set_residual(ConvIgemmPlan *p, const EltwiseArgs &e, int conv_input)
{
    // the fused form exists for the straight-line epilogue only: high-word requantize, 8-bit output,
    // whole 32-channel chunks stored through TMA
    if (p->generic_requant || p->g.qmax != 255 || p->g.k % 32 != 0 || p->bn % 32 != 0)
        return fail(B200_ERR_UNSUPPORTED, "conv(igemm): residual add needs the fast requantize form and Cout %% 32 == 0");
    p->pair_ok = 0;     // the kernel variant with the residual add runs one CTA per tile
    if (e.n_in != 2 || e.qmax != 255 || conv_input < 0 || conv_input > 1)
        return fail(B200_ERR_UNSUPPORTED, "conv(igemm): residual add takes a two-input, 8-bit eltwise SUM");
    const int other = 1 - conv_input;
    p->r_m[0] = e.m[conv_input]; p->r_add[0] = e.add[conv_input]; p->r_b[0] = e.b[conv_input];
    p->r_m[1] = e.m[other]; p->r_add[1] = e.add[other]; p->r_b[1] = e.b[other];
    p->r_s0 = e.s0; p->r_ozp = e.ozp; p->r_lo = e.relu_lo;
    p->has_res = true;
    p->last_n = -1;        // cached launch configurations carry the old constants
    p->saved.clear();
    return B200_OK;
}

static int build_launch(ConvIgemmPlan *p, const uint8_t *x, int n, uint8_t *y, int *status_word, const uint8_t *res)
{
    const ConvGeom &g = p->g;
    if ((((uintptr_t)x | (uintptr_t)y) & 15) != 0)
        return fail(B200_ERR_INVALID, "conv(igemm): x and y must be 16-byte aligned");
    IgemmArgs &a = p->args;
    memset(&a, 0, sizeof(a));
    a.n = n; a.oh = g.oh; a.ow = g.ow; a.cout = g.k;
    p->cta_pair = 0;
    a.r = g.r; a.s = g.s; a.pad_h = g.pad_h; a.pad_w = g.pad_w; a.stride_h = g.stride_h; a.stride_w = g.stride_w;
    a.c = p->cpad;
    if (p->a_wide)   // whole swizzle atoms (8 pixels) per row segment, at most 256 8-byte elements
        choose_tile(g.ow, g.oh, n, &a.tw, &a.th, &a.tn, 3, 6);
    else
        choose_tile(g.ow, g.oh, n, &a.tw, &a.th, &a.tn);
    a.tiles_w = (g.ow + a.tw - 1) / a.tw;
    a.tiles_h = (g.oh + a.th - 1) / a.th;
    a.tiles_n = (n + a.tn - 1) / a.tn;
    a.n_tiles_n = p->kpad / p->bn;
    const int sms = sm_count();
    if (!p->attr_set) {
        B200_TRY(conv_igemm_warm());
        p->attr_set = true;
    }
    if (p->pair_ok) {
        if (p->max_clusters == 0) {
            cudaLaunchConfig_t cfg = {};
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
            cfg.gridDim = dim3((unsigned)(sms & ~1));
            cfg.blockDim = dim3(kThreads);
            cfg.dynamicSmemBytes = smem_layout(p->stages_pair * p->kgroup, p->stages_pair * p->kgroup, p->bk, p->bn, p->groups, p->bn / 2).total + 1024;
            cfg.attrs = at;
            cfg.numAttrs = 1;
            int nc = 0;
            if (cudaOccupancyMaxActiveClusters(&nc, conv_igemm_i8_kernel<false, false, 3>, &cfg) != cudaSuccess || nc < 1) {
                cudaGetLastError();
                nc = sms / 2;
            }
            p->max_clusters = nc < sms / 2 ? nc : sms / 2;
        }
        const int pair_tiles = (a.tiles_w * a.tiles_h * a.tiles_n + 1) / 2 * (p->kpad / p->bn);
        // long launches only: at least six pair tiles for every cluster
        p->cta_pair = (p->pair_want == 1 || pair_tiles >= 6 * p->max_clusters) ? 1 : 0;
    }
    a.bk = p->bk; a.bn = p->bn; a.stages = p->cta_pair ? p->stages_pair : p->stages; a.kgroup = p->kgroup; a.groups = p->groups; a.acc_stages = p->acc_stages;
    a.rcp_cchunks = (uint32_t)(((1ull << 30) + (uint64_t)(p->cpad / p->bk) - 1) / (uint64_t)(p->cpad / p->bk));
    a.rcp_s = (uint32_t)(((1ull << 30) + (uint64_t)g.s - 1) / (uint64_t)g.s); a.ob = p->ob; a.b_resident = p->b_resident; a.a_wide = p->a_wide;
    for (a.tw_sh = 0; (1 << a.tw_sh) < a.tw; ++a.tw_sh) {}
    for (a.th_sh = 0; (1 << a.th_sh) < a.th; ++a.th_sh) {}
    for (a.ob_sh = 0; (1 << a.ob_sh) < a.ob; ++a.ob_sh) {}
    // instruction descriptor: D = S32 (2 at bit 4), A = unsigned 8-bit (0 at bit 7), B = signed 8-bit
    // (1 at bit 10), both K-major, N >> 3 at bit 17, M >> 4 at bit 24
    a.idesc = (2u << 4) | ((g.act_signed ? 1u : 0u) << 7) | (1u << 10) | ((uint32_t)(p->bn >> 3) << 17)
        | ((uint32_t)((p->cta_pair ? 2 * kTileM : kTileM) >> 4) << 24);
    uint32_t cols = 32;
    while (cols < (uint32_t)(p->acc_stages * p->bn))
        cols <<= 1;
    a.tmem_cols = cols;
    a.off = p->off_dev; a.mult = p->mult_dev; a.shift = p->shift_dev;
    a.row_cls = p->row_cls_dev; a.col_cls = p->col_cls_dev;
    a.n_col_cls = p->n_col_cls; a.n_cls = p->n_row_cls * p->n_col_cls; a.kpad = p->kpad;
    a.ozp = g.ozp; a.qmax = g.qmax; a.relu_lo = g.relu_lo;
    a.generic_requant = p->generic_requant;
    a.out_flip = g.act_signed ? 0x80808080u : 0u;
    a.epi_const = p->cta_pair ? 0 : p->epi_const; a.ushift = p->ushift;
    a.rnd_lo = (int)(uint32_t)(unsigned long long)p->rnd; a.rnd_hi = (int)(p->rnd >> 32);
    a.off32 = p->off32_dev;
    a.rev = p->rev;
    a.next_ro = p->next_ro; a.next_ro_bytes = p->next_ro_bytes;
    a.use_tma_store = (g.k % 16 == 0) ? 1 : 0;
    a.y = y;
    a.res = res;
    for (int i = 0; i < 2; ++i) {
        a.r_m[i] = p->r_m[i]; a.r_add[i] = p->r_add[i]; a.r_b[i] = p->r_b[i];
    }
    a.r_s0 = p->r_s0; a.r_ozp = p->r_ozp; a.r_lo = p->r_lo;
    if (status_word)
        a.status = status_word;       // caller-provided word (the allocation-free entry point)
    else
        B200_TRY(status_word_ptr(&a.status));

    // ---- tensor maps -------------------------------------------------------------------------------
    const CUtensorMapSwizzle sw_ab = swizzle_for(p->bk);
    for (int ph = 0; ph < g.stride_h; ++ph)
        for (int pw = 0; pw < g.stride_w; ++pw) {
            // input pixels (ph + stride_h * i, pw + stride_w * j): a dense 4-D tensor (c, j, i, image)
            if (ph >= g.h || pw >= g.w) {
                p->maps.a[ph * 2 + pw] = p->maps.a[0];
                continue;
            }
            if (p->a_wide) {
                // rows of this parity as a 3-D tensor (ow * 32 bytes in 8-byte elements, row, image);
                // no swizzle: the bytes are already laid out as the MMA's 32-byte swizzle wants them
                cuuint64_t dims[3] = { (cuuint64_t)g.w * 4, (cuuint64_t)((g.h - ph + g.stride_h - 1) / g.stride_h), (cuuint64_t)n };
                cuuint64_t strides[2] = { (cuuint64_t)g.stride_h * g.w * 32, (cuuint64_t)g.h * g.w * 32 };
                cuuint32_t box[3] = { (cuuint32_t)a.tw * 4, (cuuint32_t)a.th, (cuuint32_t)a.tn };
                void *base = (void *)(x + (size_t)ph * g.w * 32);
                B200_TRY(encode(&p->maps.a[ph * 2 + pw], base, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_NONE,
                                CU_TENSOR_MAP_DATA_TYPE_UINT64));
                continue;
            }
            cuuint64_t dims[4] = { (cuuint64_t)g.c, (cuuint64_t)((g.w - pw + g.stride_w - 1) / g.stride_w),
                                   (cuuint64_t)((g.h - ph + g.stride_h - 1) / g.stride_h), (cuuint64_t)n };
            cuuint64_t strides[3] = { (cuuint64_t)g.stride_w * g.c, (cuuint64_t)g.stride_h * g.w * g.c,
                                      (cuuint64_t)g.h * g.w * g.c };
            cuuint32_t box[4] = { (cuuint32_t)p->bk, (cuuint32_t)a.tw, (cuuint32_t)a.th, (cuuint32_t)a.tn };
            void *base = (void *)(x + ((size_t)ph * g.w + pw) * g.c);
            B200_TRY(encode(&p->maps.a[ph * 2 + pw], base, 4, dims, strides, box, sw_ab));
        }
    for (int i = 0; i < 4; ++i) {
        int ph = i / 2, pw = i % 2;
        if (ph >= g.stride_h || pw >= g.stride_w)
            p->maps.a[i] = p->maps.a[0];
    }
    {
        const int ktot = g.r * g.s * p->cpad;
        cuuint64_t dims[2] = { (cuuint64_t)ktot, (cuuint64_t)p->kpad };
        cuuint64_t strides[1] = { (cuuint64_t)ktot };
        cuuint32_t box[2] = { (cuuint32_t)p->bk, (cuuint32_t)(p->cta_pair ? p->bn / 2 : p->bn) };   // a CTA of a pair loads half the rows
        B200_TRY(encode(&p->maps.b, p->w_dev, 2, dims, strides, box, sw_ab));
    }
    if (a.use_tma_store) {
        cuuint64_t dims[4] = { (cuuint64_t)g.k, (cuuint64_t)g.ow, (cuuint64_t)g.oh, (cuuint64_t)n };
        cuuint64_t strides[3] = { (cuuint64_t)g.k, (cuuint64_t)g.ow * g.k, (cuuint64_t)g.oh * g.ow * g.k };
        // one store covers the 32 pixels of a tensor-memory lane quarter: a sub-box of the tile
        cuuint32_t qw = a.tw >= 32 ? 32 : a.tw;
        cuuint32_t qh = a.tw >= 32 ? 1 : (a.tw * a.th >= 32 ? 32 / a.tw : a.th);
        cuuint32_t qn = a.tw * a.th >= 32 ? 1 : 32 / (a.tw * a.th);
        cuuint32_t box[4] = { (cuuint32_t)p->ob, qw, qh, qn };
        B200_TRY(encode(&p->maps.y, y, 4, dims, strides, box, swizzle_for(p->ob)));
    } else {
        p->maps.y = p->maps.b;
    }
    const int total_tiles = a.tiles_w * a.tiles_h * a.tiles_n * a.n_tiles_n;
    p->grid = dim3((unsigned)(total_tiles < sms ? total_tiles : sms));
    p->smem = smem_layout((p->pair ? 2 : 1) * a.stages * p->kgroup, p->b_resident ? g.r * g.s * (p->cpad / p->bk) : a.stages * p->kgroup, p->bk, p->bn, p->groups,
                          p->cta_pair ? p->bn / 2 : 0).total + 1024;
    if (p->cta_pair) {
        // pair tiles (two neighbouring M tiles, one channel tile) over the CTA pairs that fit the device at once
        a.pm_tiles = (a.tiles_w * a.tiles_h * a.tiles_n + 1) / 2;
        const int pair_tiles = a.pm_tiles * a.n_tiles_n;
        const int clusters = pair_tiles < p->max_clusters ? pair_tiles : p->max_clusters;
        p->grid = dim3((unsigned)(2 * clusters));
        a.step_nt = clusters % a.n_tiles_n;
        a.step_pm = clusters / a.n_tiles_n;
    } else
    {
        int gsz = (int)p->grid.x;
        a.step_nt = gsz % a.n_tiles_n;
        gsz /= a.n_tiles_n;
        a.step_w = gsz % a.tiles_w;
        gsz /= a.tiles_w;
        a.step_h = gsz % a.tiles_h;
        a.step_n = gsz / a.tiles_h;
    }
    p->last_x = x;
    p->last_res = res;
    p->last_y = y;
    p->last_n = n;
    p->last_status = status_word;
    return B200_OK;
}

int conv_igemm_launch(ConvIgemmPlan *p, const uint8_t *x, int n, uint8_t *y, cudaStream_t st, int *status_word,
                      const uint8_t *res, const int32_t *wsum)
{
    if (n == 0)
        return B200_OK;
    if ((p->g.wzp_d != 0) != (wsum != nullptr))
        return fail(B200_ERR_INVALID, "conv(igemm): window sums are needed exactly when the weight zero point is not 128");
    if (wsum != nullptr && res != nullptr)
        return fail(B200_ERR_UNSUPPORTED, "conv(igemm): a fused residual add and a weight zero point other than 128 do not combine");
    if (res != nullptr && !p->has_res)
        return fail(B200_ERR_INVALID, "conv(igemm): a residual tensor was given but no residual add is set");
    if (res == nullptr && p->has_res)
        return fail(B200_ERR_INVALID, "conv(igemm): this conv was fused with a residual add and needs the residual tensor");
    if (res != nullptr && (((uintptr_t)res) & 15) != 0)
        return fail(B200_ERR_INVALID, "conv(igemm): the residual tensor must be 16-byte aligned");
    if (p->last_x != x || p->last_y != y || p->last_n != n || p->last_status != status_word || p->last_res != res) {
        bool hit = false;
        for (const auto &sv : p->saved)
            if (sv.x == x && sv.y == y && sv.n == n && sv.status == status_word && sv.res == res) {
                p->maps = sv.maps;
                p->args = sv.args;
                p->grid = sv.grid;
                p->smem = sv.smem;
                p->cta_pair = sv.cta_pair;
                p->last_x = x; p->last_y = y; p->last_n = n; p->last_status = status_word; p->last_res = res;
                hit = true;
                break;
            }
        if (!hit) {
            B200_TRY(build_launch(p, x, n, y, status_word, res));
            ConvIgemmPlan::Saved sv = { x, res, y, n, status_word, p->maps, p->args, p->grid, p->smem, p->cta_pair };
            if (p->saved.size() < ConvIgemmPlan::kMaxSaved) {
                p->saved.push_back(sv);
            } else {
                p->saved[p->next_saved] = sv;
                p->next_saved = (p->next_saved + 1) % ConvIgemmPlan::kMaxSaved;
            }
        }
    }
    // the window sums live in the caller's scratch, not in the launch cache's key: set them per launch
    p->args.wsum = wsum;
    p->args.wzp_d = p->g.wzp_d;
    if (res != nullptr)
        conv_igemm_i8_kernel<true><<<p->grid, kThreads, p->smem, st>>>(p->maps, p->args, p->tab);
    else if (wsum != nullptr)
        conv_igemm_i8_kernel<false, true><<<p->grid, kThreads, p->smem, st>>>(p->maps, p->args, p->tab);
    else if (p->cta_pair) {
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute at[1];
        at[0].id = cudaLaunchAttributeClusterDimension;
        at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
        cfg.gridDim = p->grid;
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = p->smem;
        cfg.stream = st;
        cfg.attrs = at;
        cfg.numAttrs = 1;
        B200_CUDA_TRY(cudaLaunchKernelEx(&cfg, conv_igemm_i8_kernel<false, false, 3>, p->maps, p->args, p->tab));
    } else if (p->pair)
        conv_igemm_i8_kernel<false, false, 2><<<p->grid, kThreads2, p->smem, st>>>(p->maps, p->args, p->tab);
    else if (p->mma_warps == 2)
        conv_igemm_i8_kernel<false, false, 1><<<p->grid, kThreads2, p->smem, st>>>(p->maps, p->args, p->tab);
    else
        conv_igemm_i8_kernel<false><<<p->grid, kThreads, p->smem, st>>>(p->maps, p->args, p->tab);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

// Everything the first launch of any plan would otherwise do once per process or device: the driver
// entry point of the tensor-map encoder and the kernels' shared-memory attribute (which also loads
// this module's code onto the current device).  Called at plan creation, while allocation is allowed.
int conv_igemm_warm()
{
    if (!encode_fn())
        return fail(B200_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    B200_CUDA_TRY(cudaFuncSetAttribute(conv_igemm_i8_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    B200_CUDA_TRY(cudaFuncSetAttribute(conv_igemm_i8_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    B200_CUDA_TRY((cudaFuncSetAttribute(conv_igemm_i8_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024)));
    B200_CUDA_TRY((cudaFuncSetAttribute(conv_igemm_i8_kernel<false, false, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024)));
    B200_CUDA_TRY((cudaFuncSetAttribute(conv_igemm_i8_kernel<false, false, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024)));
    B200_CUDA_TRY((cudaFuncSetAttribute(conv_igemm_i8_kernel<false, false, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024)));
    return B200_OK;
}

int mma_i8_peak_launch(int mmas_per_sm, float *ms, double *ops, cudaStream_t st)
{
    int *status = nullptr;
    B200_TRY(status_word_ptr(&status));
    const int mmas = mmas_per_sm / kPeakGroup * kPeakGroup;
    const size_t smem = 128 * 128 + 256 * 128 + 1024;
    B200_CUDA_TRY(cudaFuncSetAttribute(mma_i8_peak_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    cudaEvent_t e0, e1;
    B200_CUDA_TRY(cudaEventCreate(&e0));
    B200_CUDA_TRY(cudaEventCreate(&e1));
    const int sms = sm_count();
    B200_CUDA_TRY(cudaEventRecord(e0, st));
    mma_i8_peak_kernel<<<sms, 128, smem, st>>>(mmas, status);
    cudaError_t le = cudaGetLastError();
    B200_CUDA_TRY(cudaEventRecord(e1, st));
    cudaError_t se = cudaEventSynchronize(e1);
    float t = 0.f;
    if (le == cudaSuccess && se == cudaSuccess)
        se = cudaEventElapsedTime(&t, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    B200_CUDA_TRY(le);
    B200_CUDA_TRY(se);
    *ms = t;
    *ops = (double)sms * (double)mmas * 2.0 * 128.0 * 256.0 * 32.0;
    return B200_OK;
}

int wait_expiry_probe_launch(long long limit_cycles, cudaStream_t st)
{
    int *status = nullptr;
    B200_TRY(status_word_ptr(&status));
    wait_expiry_probe_kernel<<<1, 32, 0, st>>>(status, limit_cycles);
    B200_CUDA_TRY(cudaGetLastError());
    return B200_OK;
}

}  // namespace b200
