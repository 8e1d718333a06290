// Implicit-GEMM convolution on the sm_100a tensor cores.
//
//   D[pixel][filter] = sum over taps (kh,kw) and channel blocks of
//                      X[pixel shifted by the tap][channels] * W[tap][filter][channels]
//
// * GEMM M = 128 output pixels (a wt x ht x bt box of the output, batch folded in
//   for small maps), N = bn filters (<= 256), K walks taps x channel blocks.
// * Both operands are K-major (channels innermost): activations are kept
//   channels-last between layers, weights are repacked once at load.  No im2col
//   matrix exists anywhere: for every (tap, channel block) a TMA tiled load
//   fetches the shifted box of the input straight into the swizzled
//   shared-memory layout tcgen05.mma reads; out-of-image coordinates are
//   zero-filled by the TMA unit, which is the convolution's padding.  A strided
//   convolution reads from stride*stride lattices of the input (one tensor map
//   per row/column parity), so every load is still a dense box.
// * Accumulators live in TMEM (fp32); two accumulator buffers of 256 columns let
//   the epilogue of tile i overlap the MMAs of tile i+1.
// * Warp roles in a 192-thread CTA: warp 0 issues TMA, warp 1 issues tcgen05.mma
//   and owns the TMEM allocation, warps 2-5 drain TMEM and apply the fused
//   epilogue (folded batchnorm or bias, activation, stores in NHWC and/or NCHW).
// * Persistent: one CTA per SM walks tiles blockIdx.x, +gridDim.x, ...; tiles
//   that share a pixel box are adjacent so the box is fetched from HBM once and
//   re-read from L2 by the neighbouring CTAs.  No cluster, no multicast.
// * Every mbarrier wait is bounded: when it expires the CTA records a code in
//   the status word, raises a shared abort flag that all roles poll, drains,
//   frees its TMEM and returns.  The kernel never traps.
//
// Replaces forward_convolutional_layer_gpu (src/convolutional_kernels.cu:73-135
// of the reference) for groups == 1 and c >= 8.
#include <cuda.h>

#include "common.h"
#include "conv.h"
#include "device_utils.cuh"

namespace dnb {

constexpr int TC_THREADS = 192;
constexpr int MAX_STAGES = 8;
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;  // about one second

// ------------------------------------------------------------------ PTX wrappers
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
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    return done;
}

// Bounded wait.  Returns false when the wait expired or another role aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status, int code)
{
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = clock64();
    int spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0xff) == 0) {
            if (*abort_flag) return false;
            if (clock64() - t0 > WAIT_LIMIT_CYCLES) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2, int c3)
{
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int c0, int c1, int c2)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

// Shared-memory matrix descriptor, K-major operand whose rows are `row_bytes`
// long and equal to the swizzle span; 8-row groups are 8*row_bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, int row_bytes)
{
    const uint64_t layout = row_bytes == 128 ? 2 : (row_bytes == 64 ? 4 : 6);  // SWIZZLE_128B / 64B / 32B
    uint64_t d = (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;                                  // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)((8 * row_bytes) >> 4) << 32;             // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                                  // descriptor version for sm_100
    d |= layout << 61;
    return d;
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate, int is_bf16)
{
    if (is_bf16) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
    }
}
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// TMA store of one staged output chunk (shared -> global), bulk-group completion.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap *map, uint32_t src, int c0, int c1, int c2, int c3)
{
    asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
                 ::"l"(map), "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read1() { asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// barrier among the 128 epilogue threads only (barrier 0 is __syncthreads)
__device__ __forceinline__ void epilogue_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// ------------------------------------------------------------------ kernel
struct TcShared {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

enum { WAIT_EMPTY = 101, WAIT_FULL = 102, WAIT_ACC_EMPTY = 103, WAIT_ACC_FULL = 104 };
enum { ACT_GENERIC = -1 };

template <int ACT>
__device__ __forceinline__ float act_apply(float x, int runtime_act)
{
    if (ACT == DNB_LINEAR) return x;
    if (ACT == DNB_LEAKY) return fmaxf(x, 0.1f * x);   // x > 0 ? x : 0.1x
    if (ACT == DNB_LOGISTIC) return 1.f / (1.f + __expf(-x));
    return activate(x, runtime_act);
}

template <int ACT>
__global__ void __launch_bounds__(TC_THREADS, 1)
conv_tc_kernel(const __grid_constant__ TcArgs a)
{
    extern __shared__ uint8_t smem_raw[];
    // operand ring, 1024-byte aligned (the 128-byte swizzle pattern repeats every 1024 bytes)
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t stage_bytes = a.a_bytes + a.b_bytes;
    uint8_t *after_ring = smem_raw + (ring - smem_u32(smem_raw)) + (size_t)a.stages * stage_bytes;
    uint8_t *stage_out = after_ring;                                  // 2 x 128 rows x store_row_bytes
    float *s_scale = reinterpret_cast<float *>(after_ring + 2 * 128 * a.store_row_bytes);
    float *s_shift = s_scale + a.n_tot;
    TcShared *sh = reinterpret_cast<TcShared *>(s_shift + a.n_tot);
    volatile int *abort_flag = &sh->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < a.stages; ++s) {
            mbar_init(smem_u32(&sh->full[s]), 1);
            mbar_init(smem_u32(&sh->empty[s]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&sh->acc_full[i]), 1);
            mbar_init(smem_u32(&sh->acc_empty[i]), 4);
        }
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {  // TMEM: all 512 columns (two accumulators of 256), whole warp
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // per-filter epilogue vectors, once per CTA (zero beyond the layer's filters)
    for (int i = threadIdx.x; i < a.n_tot; i += TC_THREADS) {
        s_scale[i] = i < a.n_pad ? __ldg(a.ep.scale + i) : 0.f;
        s_shift[i] = i < a.n_pad ? __ldg(a.ep.shift + i) : 0.f;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;

    const int k_iters = a.taps * a.c_blocks;
    const int ptiles_wh = a.tiles_w * a.tiles_h;

    if (warp == 0) {
        // ---------------- TMA producer
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < a.total_tiles && ok; tile += gridDim.x) {
            const int nt = tile % a.n_tiles, pt = tile / a.n_tiles;
            const int ow0 = (pt % a.tiles_w) * a.wt;
            const int oh0 = ((pt / a.tiles_w) % a.tiles_h) * a.ht;
            const int b0 = (pt / ptiles_wh) * a.bt;
            for (int tap = 0; tap < a.taps && ok; ++tap) {
                const int kh = tap / a.g.size, kw = tap - kh * a.g.size;
                // input row = oh*stride + kh - pad = stride*(oh + q) + parity
                const int dh = kh - a.g.pad, dw = kw - a.g.pad;
                const int ph = ((dh % a.g.stride) + a.g.stride) % a.g.stride, qh = (dh - ph) / a.g.stride;
                const int pw = ((dw % a.g.stride) + a.g.stride) % a.g.stride, qw = (dw - pw) / a.g.stride;
                const CUtensorMap *mx = &a.tmx[ph * a.g.stride + pw];
                for (int cb = 0; cb < a.c_blocks; ++cb) {
                    ok = mbar_wait(smem_u32(&sh->empty[stage]), phase ^ 1, abort_flag, a.status, WAIT_EMPTY);
                    ok = __all_sync(0xffffffffu, ok);
                    if (!ok) break;
                    if (lane == 0) {
                        const uint32_t bar = smem_u32(&sh->full[stage]);
                        const uint32_t sa = ring + stage * stage_bytes, sb = sa + a.a_bytes;
                        mbar_expect_tx(bar, 128u * a.row_bytes + (uint32_t)a.bn * a.row_bytes);
                        tma_load_4d(sa, mx, bar, cb * a.bk, ow0 + qw, oh0 + qh, b0);
                        tma_load_3d(sb, &a.tmw, bar, cb * a.bk, nt * a.bn, tap);
                    }
                    __syncwarp();
                    if (++stage == a.stages) { stage = 0; phase ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer
        const uint32_t fmt = a.is_bf16 ? 1u : 2u;  // BF16 : TF32
        const uint32_t idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(a.bn >> 3) << 17) | ((128u >> 4) << 24);
        const int k_steps = a.row_bytes / 32;  // one MMA consumes 32 bytes of K per row
        int stage = 0;
        uint32_t phase = 0;
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < a.total_tiles && ok; tile += gridDim.x, ++it) {
            const int acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            ok = mbar_wait(smem_u32(&sh->acc_empty[acc]), acc_phase ^ 1, abort_flag, a.status, WAIT_ACC_EMPTY);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * 256;
            for (int ki = 0; ki < k_iters; ++ki) {
                ok = mbar_wait(smem_u32(&sh->full[stage]), phase, abort_flag, a.status, WAIT_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                tc_fence_after();
                if (lane == 0) {
                    const uint32_t sa = ring + stage * stage_bytes, sb = sa + a.a_bytes;
                    const uint64_t da = make_smem_desc(sa, a.row_bytes), db = make_smem_desc(sb, a.row_bytes);
                    for (int k = 0; k < k_steps; ++k)
                        umma(d_tmem, da + 2 * k, db + 2 * k, idesc, (ki | k) != 0, a.is_bf16);
                    umma_commit(smem_u32(&sh->empty[stage]));  // frees the stage when these MMAs retire
                    if (ki == k_iters - 1) umma_commit(smem_u32(&sh->acc_full[acc]));
                }
                __syncwarp();
                if (++stage == a.stages) { stage = 0; phase ^= 1; }
            }
        }
    } else {
        // ---------------- epilogue: warps 2..5 own TMEM lanes 32*(warp%4) .. +31
        const int quarter = warp & 3;
        const int m = quarter * 32 + lane;  // pixel index inside the tile = TMEM lane = staging row
        const int wl = m % a.wt, hl = (m / a.wt) % a.ht, bl = m / (a.wt * a.ht);
        const ConvGeom &g = a.g;
        const bool store_thread = threadIdx.x == 64;
        const bool out_bf16 = a.y_dtype == DNB_BF16;
        const int srb = a.store_row_bytes;                       // bytes of one staged row = swizzle span
        const int cols_per_chunk = srb / (out_bf16 ? 2 : 4);
        const int q_mask = srb / 16 - 1;
        const int q_xor = (m >> (srb == 128 ? 0 : (srb == 64 ? 1 : 2))) & q_mask;   // 16-byte chunk swizzle of row m
        uint32_t chunk_count = 0;
        int it = 0;
        for (int tile = blockIdx.x; tile < a.total_tiles; tile += gridDim.x, ++it) {
            const int acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            const int nt = tile % a.n_tiles, pt = tile / a.n_tiles;
            const int ow0 = (pt % a.tiles_w) * a.wt, oh0 = ((pt / a.tiles_w) % a.tiles_h) * a.ht, b0 = (pt / ptiles_wh) * a.bt;
            const int ow = ow0 + wl, oh = oh0 + hl, b = b0 + bl;
            const bool pix_ok = ow < g.out_w && oh < g.out_h && b < g.batch;

            mbar_wait(smem_u32(&sh->acc_full[acc]), acc_phase, abort_flag, a.status, WAIT_ACC_FULL);
            epilogue_bar();                 // all four warps agree on the abort flag from here
            if (*abort_flag) break;
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * 256;
            for (int c0 = 0; c0 < a.bn; c0 += cols_per_chunk) {
                uint8_t *row = nullptr;
                if (a.y_nhwc) {
                    const uint32_t buf = chunk_count & 1;
                    if (store_thread && chunk_count >= 2) tma_store_wait_read1();   // the store that last read this buffer is done
                    epilogue_bar();
                    row = stage_out + (size_t)buf * 128 * srb + (size_t)m * srb;
                }
                for (int p0 = 0; p0 < cols_per_chunk; p0 += 16) {
                    const int j0 = c0 + p0;            // first column of this piece inside the tile
                    float v[16];
                    if (j0 < a.bn) {
                        uint32_t r[16];
                        tmem_ld16(t_row + j0, r);
                        tmem_ld_wait();
                        const int nl = nt * a.bn + j0;  // first filter of this piece
                        const float4 *sc4 = reinterpret_cast<const float4 *>(s_scale + nl);
                        const float4 *sf4 = reinterpret_cast<const float4 *>(s_shift + nl);
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const float4 sc = sc4[q], sf = sf4[q];
                            const float scv[4] = {sc.x, sc.y, sc.z, sc.w}, sfv[4] = {sf.x, sf.y, sf.z, sf.w};
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const int j = 4 * q + e;
                                float t = act_apply<ACT>(fmaf(__uint_as_float(r[j]), scv[e], sfv[e]), a.ep.activation);
                                if (a.ep.round_tf32) t = round_tf32(t);
                                v[j] = (nl + j < g.n) ? t : 0.f;
                            }
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j) v[j] = 0.f;
                    }
                    if (row) {
                        if (!out_bf16) {
                            const int qb = p0 / 4;     // first 16-byte chunk of this piece in the row
#pragma unroll
                            for (int q = 0; q < 4; ++q)
                                *reinterpret_cast<float4 *>(row + (((qb + q) ^ q_xor) << 4)) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                        } else {
                            const int qb = p0 / 8;
#pragma unroll
                            for (int q = 0; q < 2; ++q) {
                                __align__(16) __nv_bfloat16 hv[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j) hv[j] = __float2bfloat16_rn(v[8 * q + j]);
                                *reinterpret_cast<uint4 *>(row + (((qb + q) ^ q_xor) << 4)) = *reinterpret_cast<uint4 *>(hv);
                            }
                        }
                    }
                    if (a.y_nchw && pix_ok && j0 < a.bn) {
                        const int n0 = nt * a.bn + j0;
                        const size_t plane = (size_t)g.out_h * g.out_w;
                        float *dst = a.y_nchw + ((size_t)b * g.n + n0) * plane + (size_t)oh * g.out_w + ow;
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (n0 + j < g.n) dst[j * plane] = v[j];
                    }
                }
                if (a.y_nhwc) {
                    fence_async_smem();            // staged rows visible to the TMA unit
                    epilogue_bar();
                    if (store_thread) {
                        // the TMA unit clips the box at the tensor's extents: ragged tiles need no predicates
                        tma_store_4d(&a.tmy, smem_u32(stage_out + (size_t)(chunk_count & 1) * 128 * srb), nt * a.bn + c0, ow0, oh0, b0);
                        tma_store_commit();
                    }
                    ++chunk_count;
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&sh->acc_empty[acc]));
        }
        if (store_thread) tma_store_wait_all();
    }

    // ---------------- teardown (also the abort path)
    if (*abort_flag) {   // give loads that are still in flight time to land before shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000LL) { }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// ------------------------------------------------------------------ host side
size_t conv_tc_fixed_smem(int store_row_bytes, int n_tot)
{
    return 1024 + 2 * 128 * (size_t)store_row_bytes + 2 * sizeof(float) * (size_t)n_tot + sizeof(TcShared) + 64;
}

size_t conv_tc_smem_bytes(const TcArgs &a)
{
    return (size_t)a.stages * (a.a_bytes + a.b_bytes) + conv_tc_fixed_smem(a.store_row_bytes, a.n_tot);
}

int conv_tc_max_smem()
{
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return 0;
    return v;
}

int launch_conv_tc(const TcArgs &a, cudaStream_t s)
{
    static thread_local int configured_for = -1;
    const size_t smem = conv_tc_smem_bytes(a);
    int dev = 0;
    DNB_CUDA(cudaGetDevice(&dev));
    if (configured_for != dev) {
        const int m = conv_tc_max_smem();
        DNB_CUDA(cudaFuncSetAttribute(conv_tc_kernel<DNB_LINEAR>, cudaFuncAttributeMaxDynamicSharedMemorySize, m));
        DNB_CUDA(cudaFuncSetAttribute(conv_tc_kernel<DNB_LEAKY>, cudaFuncAttributeMaxDynamicSharedMemorySize, m));
        DNB_CUDA(cudaFuncSetAttribute(conv_tc_kernel<DNB_LOGISTIC>, cudaFuncAttributeMaxDynamicSharedMemorySize, m));
        DNB_CUDA(cudaFuncSetAttribute(conv_tc_kernel<ACT_GENERIC>, cudaFuncAttributeMaxDynamicSharedMemorySize, m));
        configured_for = dev;
    }
    int grid = a.total_tiles < sm_count() ? a.total_tiles : sm_count();
    switch (a.ep.activation) {
    case DNB_LINEAR: conv_tc_kernel<DNB_LINEAR><<<grid, TC_THREADS, smem, s>>>(a); break;
    case DNB_LEAKY: conv_tc_kernel<DNB_LEAKY><<<grid, TC_THREADS, smem, s>>>(a); break;
    case DNB_LOGISTIC: conv_tc_kernel<DNB_LOGISTIC><<<grid, TC_THREADS, smem, s>>>(a); break;
    default: conv_tc_kernel<ACT_GENERIC><<<grid, TC_THREADS, smem, s>>>(a); break;
    }
    DNB_LAUNCH_CHECK("conv_tc");
    return DNB_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_tensor_map(CUtensorMap *map, int is_bf16, int rank, void *base, const uint64_t *dims,
                      const uint64_t *strides_bytes, const uint32_t *box, int swizzle_bytes)
{
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        DNB_CUDA(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q));
        if (!p || q != cudaDriverEntryPointSuccess) DNB_FAIL(DNB_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
        fn = (EncodeTiledFn)p;
    }
    cuuint64_t d[5], st[4];
    cuuint32_t bx[5], es[5];
    for (int i = 0; i < rank; ++i) { d[i] = dims[i]; bx[i] = box[i]; es[i] = 1; }
    for (int i = 0; i + 1 < rank; ++i) st[i] = strides_bytes[i];
    CUtensorMapSwizzle sw = swizzle_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B
                            : swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
    CUresult r = fn(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, (cuuint32_t)rank, base,
                    d, st, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        DNB_FAIL(DNB_ECUDA, "cuTensorMapEncodeTiled failed with %d (rank %d, dims %llu %llu %llu, box %u %u %u, swizzle %d)", (int)r, rank,
                 (unsigned long long)d[0], (unsigned long long)d[1], (unsigned long long)(rank > 2 ? d[2] : 0), bx[0], bx[1], rank > 2 ? bx[2] : 0, swizzle_bytes);
    return DNB_OK;
}

}  // namespace dnb
