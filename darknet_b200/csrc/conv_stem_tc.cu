// First-layer convolution on the sm_100a tensor cores: 3x3 filters over at most 3 input channels
// (the RGB stems of YOLOv3, YOLOv3-tiny and Darknet-19), K = c*9 <= 27 padded to 32.
//
// The K extent is one 128-byte row of TF32 values, far too short for the TMA-fed ring of the general
// kernel (nine 32-byte-wide loads per tile).  Here the 128 threads of a CTA build the im2col rows
// themselves: thread m gathers the 27 input values of output pixel m of the tile from the image as
// the caller laid it out (NCHW or channels-last, through element strides; out-of-image taps read as
// zero, which is the padding), rounds them to TF32 and writes its row into shared memory in the
// 128-byte-swizzled K-major layout tcgen05.mma reads.  One thread then issues four K=8 MMAs against the
// filter matrix, which sits in shared memory for the life of the CTA,
// into a TMEM accumulator.  A thread requests the inputs of tile i+1 before it runs the epilogue of tile i
// (TMEM -> registers -> folded batchnorm / bias, activation), so the loads' latency is covered.  The
// finished rows are staged where the tile's im2col rows were and leave through one TMA store per warp
// (32 rows; plain 16-byte stores when a row is wider than 128 bytes).  Tiles are runs of 128 consecutive
// output pixels of the flattened [batch][out_h][out_w] index, so a tile's output is one contiguous span.
// Several CTAs share an SM and fill each other's barrier and MMA waits.
//
// Every mbarrier wait is bounded; on expiry the CTA records a code in the status word and leaves.
//
// Replaces forward_convolutional_layer_gpu (src/convolutional_kernels.cu:73-135 of the reference) for
// size 3, groups 1, c <= 3, n a multiple of 16 up to 64, channels-last output; im2col row order
// c*9 + kh*3 + kw as in src/im2col.c:15-39.  A second kernel below covers 5x5 and 7x7 filters over RGB
// (ResNet's 7x7 stride-2 first layer), whose K spans several 128-byte rows.
#include "common.h"
#include "conv.h"
#include "device_utils.cuh"
#include "tc_ptx.cuh"

namespace dnb {

constexpr int ST_THREADS = 128;
constexpr int ST_A_BYTES = 128 * 128;   // one im2col tile: 128 rows of 32 TF32 values

struct StemShared {
    uint64_t acc_full;
    uint32_t tmem_base;
    int abort_flag;
};

enum { ST_WAIT_ACC = 104, ST_BAD_SMEM_BASE = 106 };
enum { ST_ACT_GENERIC = -1 };

template <int ACT>
__device__ __forceinline__ float stem_act(float x, int runtime_act)
{
    if (ACT == DNB_LINEAR) return x;
    if (ACT == DNB_LEAKY) return fmaxf(x, 0.1f * x);
    return activate_call(x, runtime_act);
}

// C: input channels (1..3); ACT: activation folded at compile time or ST_ACT_GENERIC; OUT_BF16: storage
// type of the channels-last output.
template <int C, int ACT, bool OUT_BF16>
__global__ void __launch_bounds__(ST_THREADS, 5)
conv_stem_tc_kernel(const __grid_constant__ StemTcArgs a)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023u) {   // the swizzle pattern repeats every 1024 bytes
        if (threadIdx.x == 0) atomicCAS(a.status, 0, ST_BAD_SMEM_BASE);
        return;
    }
    constexpr int K = C * 9;
    const int tid = threadIdx.x, warp = tid >> 5;
    const int n_pad = a.n_pad;
    uint8_t *sA = smem;                           // 2 x 128 rows x 128 bytes
    uint8_t *sB = smem + 2 * ST_A_BYTES;          // n_pad rows x 128 bytes
    float *s_scale = reinterpret_cast<float *>(sB + (size_t)n_pad * 128);
    float *s_shift = s_scale + n_pad;
    StemShared *sh = reinterpret_cast<StemShared *>(s_shift + n_pad);
    volatile int *abort_flag = &sh->abort_flag;
    const ConvGeom g = a.g;

    // filters: row f holds w[f][0..K) rounded to TF32, zero beyond K and beyond the layer's filters
    for (int i = tid; i < n_pad * 8; i += ST_THREADS) {
        const int f = i >> 3, q = i & 7;
        uint32_t v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = 4 * q + e;
            v[e] = (k < K && f < g.n) ? __float_as_uint(round_tf32(__ldg(a.w + (size_t)k * a.npg_pad + f))) : 0u;
        }
        *reinterpret_cast<uint4 *>(sB + f * 128 + ((q ^ (f & 7)) << 4)) = make_uint4(v[0], v[1], v[2], v[3]);
    }
    for (int i = tid; i < n_pad; i += ST_THREADS) {
        s_scale[i] = i < g.n ? __ldg(a.ep.scale + i) : 0.f;
        s_shift[i] = i < g.n ? __ldg(a.ep.shift + i) : 0.f;
    }
    if (tid == 0) {
        mbar_init(smem_u32(&sh->acc_full), 1);
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const uint32_t tmem_cols = (uint32_t)a.tmem_cols;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_async_smem();   // the filter rows are read by the tensor cores
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;

    // register copies: every asm statement below is a compiler memory barrier
    const float *const x = a.x;
    const long long xs_b = a.xs_b;
    const int xs_c = (int)a.xs_c, xs_h = (int)a.xs_h, xs_w = (int)a.xs_w;
    const int npix = a.npix, tiles = a.tiles, plane = g.out_h * g.out_w;
    const int runtime_act = a.ep.activation, do_round = a.ep.round_tf32;
    uint8_t *const y = reinterpret_cast<uint8_t *>(a.y);
    const size_t y_row_bytes = (size_t)a.y_cpitch * (OUT_BF16 ? 2 : 4);
    int *const status = a.status;
    const long long wait_limit = a.wait_limit;
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n_pad >> 3) << 17) | ((128u >> 4) << 24);   // TF32 x TF32 -> f32, M 128, N n_pad
    const uint64_t db = make_smem_desc(smem_u32(sB), 128);
    const uint64_t da0 = make_smem_desc(smem_u32(sA), 128);
    const uint32_t bar0 = smem_u32(&sh->acc_full);
    const uint32_t row_off = (uint32_t)tid * 128u, sw = (uint32_t)(tid & 7);

    // staged output rows for the TMA store: row m of the tile at m * row_bytes, 16-byte pieces swizzled as the map says
    const bool tma = a.tma_store != 0;
    const uint32_t out_row_bytes = (uint32_t)a.y_cpitch * (OUT_BF16 ? 2u : 4u);
    const uint32_t q_xor = out_row_bytes == 128 ? (uint32_t)(tid & 7) : (out_row_bytes == 64 ? (uint32_t)((tid >> 1) & 3) : (uint32_t)((tid >> 2) & 1));
    const CUtensorMap *ymap = &a.tmy;
    const int lane = tid & 31;

    bool failed = false;
    int prev_tile = 0;
    int it = 0;
    for (int tile = blockIdx.x;; tile += gridDim.x, ++it) {
        const bool have = tile < tiles;   // uniform over the CTA
        const int buf = it & 1;
        // ---- this thread's 27 input values of the next tile: requested first, used after the epilogue below
        float v[K];
        if (have) {
            const int p = tile * ST_THREADS + tid;
            const bool valid = p < npix;
            const int b = p / plane, rem = p - b * plane;
            const int oy = rem / g.out_w, ox = rem - oy * g.out_w;
            const int iy0 = oy * g.stride - g.pad, ix0 = ox * g.stride - g.pad;
            // three row and three column validity flags and one base pointer: a tap costs one predicated load
            const bool rv0 = valid && (unsigned)iy0 < (unsigned)g.h, rv1 = valid && (unsigned)(iy0 + 1) < (unsigned)g.h,
                       rv2 = valid && (unsigned)(iy0 + 2) < (unsigned)g.h;
            const bool cv0 = (unsigned)ix0 < (unsigned)g.w, cv1 = (unsigned)(ix0 + 1) < (unsigned)g.w, cv2 = (unsigned)(ix0 + 2) < (unsigned)g.w;
            const float *xp = x + (size_t)b * xs_b + (long long)iy0 * xs_h + (long long)ix0 * xs_w;   // dereferenced only where valid
#pragma unroll
            for (int c = 0; c < C; ++c)
#pragma unroll
                for (int kh = 0; kh < 3; ++kh) {
                    const bool rv = kh == 0 ? rv0 : (kh == 1 ? rv1 : rv2);
                    const float *rp = xp + c * xs_c + kh * xs_h;
                    v[c * 9 + kh * 3 + 0] = (rv && cv0) ? __ldg(rp) : 0.f;
                    v[c * 9 + kh * 3 + 1] = (rv && cv1) ? __ldg(rp + xs_w) : 0.f;
                    v[c * 9 + kh * 3 + 2] = (rv && cv2) ? __ldg(rp + 2 * xs_w) : 0.f;
                }
        }
        if (it > 0) {
            // ---- epilogue of the previous tile (its MMAs were issued at the end of the previous iteration)
            const int pb = (it - 1) & 1;
            if (!mbar_wait(bar0, (uint32_t)((it - 1) & 1), abort_flag, status, ST_WAIT_ACC, 0, wait_limit)) {
                failed = true;
            } else {
                tc_fence_after();
                const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16);
                const int prev_p = prev_tile * ST_THREADS + tid;
                const bool store = prev_p < npix;
                uint8_t *dst = y + (size_t)prev_p * y_row_bytes;
                // the finished rows go where the tile's im2col rows were: its MMAs have retired
                uint8_t *srow = sA + pb * ST_A_BYTES + (uint32_t)tid * out_row_bytes;
#pragma unroll 1
                for (int c0 = 0; c0 < n_pad; c0 += 16) {
                    uint32_t r[16];
                    tmem_ld16(t_row + c0, r);
                    tmem_ld_wait();
                    float o[16];
                    const float4 *sc4 = reinterpret_cast<const float4 *>(s_scale + c0);
                    const float4 *sf4 = reinterpret_cast<const float4 *>(s_shift + c0);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float4 sc = sc4[q], sf = sf4[q];
                        const float scv[4] = {sc.x, sc.y, sc.z, sc.w}, sfv[4] = {sf.x, sf.y, sf.z, sf.w};
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int j = 4 * q + e;
                            float t = stem_act<ACT>(fmaf(__uint_as_float(r[j]), scv[e], sfv[e]), runtime_act);
                            if (do_round) t = round_tf32(t);
                            // beyond the layer's filters scale and shift are zero: only an activation with f(0) != 0 needs the mask
                            o[j] = (ACT == ST_ACT_GENERIC && c0 + j >= g.n) ? 0.f : t;
                        }
                    }
                    if (!OUT_BF16) {
#pragma unroll
                        for (int q = 0; q < 4; ++q) {
                            const uint4 pk = make_uint4(__float_as_uint(o[4 * q]), __float_as_uint(o[4 * q + 1]), __float_as_uint(o[4 * q + 2]), __float_as_uint(o[4 * q + 3]));
                            if (tma) *reinterpret_cast<uint4 *>(srow + ((((uint32_t)(c0 >> 2) + q) ^ q_xor) << 4)) = pk;
                            else if (store) reinterpret_cast<uint4 *>(dst + (size_t)c0 * 4)[q] = pk;
                        }
                    } else {
#pragma unroll
                        for (int q = 0; q < 2; ++q) {
                            uint4 pk;
                            __nv_bfloat162 h0 = __floats2bfloat162_rn(o[8 * q], o[8 * q + 1]);
                            __nv_bfloat162 h1 = __floats2bfloat162_rn(o[8 * q + 2], o[8 * q + 3]);
                            __nv_bfloat162 h2 = __floats2bfloat162_rn(o[8 * q + 4], o[8 * q + 5]);
                            __nv_bfloat162 h3 = __floats2bfloat162_rn(o[8 * q + 6], o[8 * q + 7]);
                            pk.x = *reinterpret_cast<uint32_t *>(&h0); pk.y = *reinterpret_cast<uint32_t *>(&h1);
                            pk.z = *reinterpret_cast<uint32_t *>(&h2); pk.w = *reinterpret_cast<uint32_t *>(&h3);
                            if (tma) *reinterpret_cast<uint4 *>(srow + ((((uint32_t)(c0 >> 3) + q) ^ q_xor) << 4)) = pk;
                            else if (store) reinterpret_cast<uint4 *>(dst + (size_t)c0 * 2)[q] = pk;
                        }
                    }
                }
                if (tma) {
                    // each warp stores its own 32 rows: no CTA-wide barrier between the rows and the store
                    fence_async_smem();
                    __syncwarp();
                    const int row0 = prev_tile * ST_THREADS + warp * 32;
                    if (lane == 0 && row0 < npix) {   // the TMA unit clips the box at the last pixel
                        tma_store_2d(ymap, smem_u32(sA + pb * ST_A_BYTES) + (uint32_t)(warp * 32) * out_row_bytes, 0, row0);
                        tma_store_commit();
                    }
                }
            }
        }
        if (have) {
            // ---- im2col row into A[buf]; the buffer last held the staged rows of two tiles ago
            if (tma) {
                if (lane == 0) tma_store_wait_read1();   // all but the store just issued have read their rows
                __syncwarp();
                // Staged rows narrower than an im2col row (fewer than 128 bytes of output per pixel) put this thread's
                // im2col row over rows that OTHER warps staged two tiles ago: every warp's stores must have read them.
                if (out_row_bytes < 128) __syncthreads();
            }
            uint8_t *row = sA + buf * ST_A_BYTES + row_off;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                uint32_t w4[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) w4[e] = 4 * q + e < K ? __float_as_uint(round_tf32(v[4 * q + e < K ? 4 * q + e : 0])) : 0u;
                *reinterpret_cast<uint4 *>(row + ((q ^ sw) << 4)) = make_uint4(w4[0], w4[1], w4[2], w4[3]);
            }
            fence_async_smem();   // rows visible to the tensor cores
        }
        tc_fence_before();        // this thread's TMEM loads precede the barrier, the next MMAs follow it
        if (__syncthreads_or(failed)) break;
        if (!have) break;
        if (tid == 0) {
            tc_fence_after();
            const uint64_t da = da0 + (uint64_t)(buf * (ST_A_BYTES >> 4));
            umma<MMA_TF32>(tmem_base, da, db, idesc, 0u);
            umma<MMA_TF32>(tmem_base, da + 2, db + 2, idesc, 1u);
            umma<MMA_TF32>(tmem_base, da + 4, db + 4, idesc, 1u);
            umma<MMA_TF32>(tmem_base, da + 6, db + 6, idesc, 1u);
            umma_commit(bar0);
        }
        __syncwarp();
        prev_tile = tile;
    }
    if (tma && lane == 0) tma_store_wait_all();

    // ---- teardown (also the abort path)
    if (*abort_flag) {   // give MMAs that may still read shared memory time to retire
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000LL) { }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// ------------------------------------------------------------------ wider first layers (5x5, 7x7 over RGB)
// K = c*size*size no longer fits one 128-byte row (147 for ResNet's 7x7 layer): the tile's im2col rows are built
// and multiplied in blocks of 32 values.  Two 16 KB row buffers alternate; the MMAs of block kb read one while
// the threads gather block kb+1 into the other; the filter matrix (all blocks) stays in shared memory.  The
// epilogue follows the last block's MMAs, staged over both row buffers and stored by TMA, one or two boxes of
// 32 rows x 128 bytes per warp.
struct StemWideShared {
    uint64_t mma_done[2];   // the MMAs that read row buffer i have retired
    uint64_t acc_full;
    uint32_t tmem_base;
    int abort_flag;
};

template <int C, int KS, int ACT, bool OUT_BF16>
__global__ void __launch_bounds__(ST_THREADS, 3)
conv_stem_tc_wide_kernel(const __grid_constant__ StemTcArgs a)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    if (smem_u32(smem) & 1023u) {
        if (threadIdx.x == 0) atomicCAS(a.status, 0, ST_BAD_SMEM_BASE);
        return;
    }
    constexpr int K = C * KS * KS, KB = (K + 31) / 32;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_pad = a.n_pad;
    uint8_t *sA = smem;                              // 2 x 128 rows x 128 bytes; also the staging rows of the epilogue
    uint8_t *sB = smem + 2 * ST_A_BYTES;             // KB blocks of n_pad rows x 128 bytes
    float *s_scale = reinterpret_cast<float *>(sB + (size_t)KB * n_pad * 128);
    float *s_shift = s_scale + n_pad;
    StemWideShared *sh = reinterpret_cast<StemWideShared *>(s_shift + n_pad);
    volatile int *abort_flag = &sh->abort_flag;
    const ConvGeom g = a.g;

    for (int i = tid; i < KB * n_pad * 8; i += ST_THREADS) {
        const int kb = i / (n_pad * 8), r = i - kb * n_pad * 8, f = r >> 3, q = r & 7;
        uint32_t v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = kb * 32 + 4 * q + e;
            v[e] = (k < K && f < g.n) ? __float_as_uint(round_tf32(__ldg(a.w + (size_t)k * a.npg_pad + f))) : 0u;
        }
        *reinterpret_cast<uint4 *>(sB + (size_t)kb * n_pad * 128 + f * 128 + ((q ^ (f & 7)) << 4)) = make_uint4(v[0], v[1], v[2], v[3]);
    }
    for (int i = tid; i < n_pad; i += ST_THREADS) {
        s_scale[i] = i < g.n ? __ldg(a.ep.scale + i) : 0.f;
        s_shift[i] = i < g.n ? __ldg(a.ep.shift + i) : 0.f;
    }
    if (tid == 0) {
        mbar_init(smem_u32(&sh->mma_done[0]), 1);
        mbar_init(smem_u32(&sh->mma_done[1]), 1);
        mbar_init(smem_u32(&sh->acc_full), 1);
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    const uint32_t tmem_cols = (uint32_t)a.tmem_cols;
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    fence_async_smem();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = sh->tmem_base;

    const float *const x = a.x;
    const long long xs_b = a.xs_b;
    const int xs_c = (int)a.xs_c, xs_h = (int)a.xs_h, xs_w = (int)a.xs_w;
    const int npix = a.npix, tiles = a.tiles, plane = g.out_h * g.out_w;
    const int runtime_act = a.ep.activation, do_round = a.ep.round_tf32;
    int *const status = a.status;
    const long long wait_limit = a.wait_limit;
    const uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(n_pad >> 3) << 17) | ((128u >> 4) << 24);
    const uint64_t db0 = make_smem_desc(smem_u32(sB), 128);
    const uint64_t da0 = make_smem_desc(smem_u32(sA), 128);
    const uint64_t b_step = (uint64_t)((n_pad * 128) >> 4);
    const uint32_t done0 = smem_u32(&sh->mma_done[0]), acc_bar = smem_u32(&sh->acc_full);
    const uint32_t row_off = (uint32_t)tid * 128u, sw = (uint32_t)(tid & 7);
    const uint32_t out_row_bytes = (uint32_t)a.y_cpitch * (OUT_BF16 ? 2u : 4u);   // 32, 64, 128 or 256
    const uint32_t half_bytes = out_row_bytes > 128 ? 128u : out_row_bytes;       // bytes of a row per staging half
    const uint32_t q_mask = half_bytes / 16 - 1;
    const uint32_t q_xor = (half_bytes == 128 ? (uint32_t)tid : (half_bytes == 64 ? (uint32_t)(tid >> 1) : (uint32_t)(tid >> 2))) & q_mask;
    const CUtensorMap *ymap = &a.tmy;

    bool failed = false, stop = false;
    uint32_t kcount = 0;        // blocks of 32 K values processed so far (buffer = kcount & 1)
    int it = 0;
    for (int tile = blockIdx.x; tile < tiles && !stop; tile += gridDim.x, ++it) {
        const int p = tile * ST_THREADS + tid;
        const bool valid = p < npix;
        const int b = p / plane, rem = p - b * plane;
        const int oy = rem / g.out_w, ox = rem - oy * g.out_w;
        const int iy0 = oy * g.stride - g.pad, ix0 = ox * g.stride - g.pad;
        uint32_t rmask = 0, cmask = 0;   // bit k: row iy0+k / column ix0+k is inside the image
#pragma unroll
        for (int k = 0; k < KS; ++k) {
            rmask |= (valid && (unsigned)(iy0 + k) < (unsigned)g.h) ? (1u << k) : 0u;
            cmask |= ((unsigned)(ix0 + k) < (unsigned)g.w) ? (1u << k) : 0u;
        }
        const float *xp = x + (size_t)b * xs_b + (long long)iy0 * xs_h + (long long)ix0 * xs_w;   // dereferenced only where valid
        // the previous tile's stores read the row buffers this tile overwrites
        if (lane == 0) tma_store_wait_read0();
        __syncwarp();
#pragma unroll
        for (int kb = 0; kb < KB; ++kb) {
            const uint32_t buf = kcount & 1u, use = kcount >> 1;
            if (use > 0 && !mbar_wait(done0 + 8 * buf, (use - 1) & 1u, abort_flag, status, ST_WAIT_ACC, 0, wait_limit)) failed = true;
            float v[32];
#pragma unroll
            for (int t = 0; t < 32; ++t) {
                const int k = kb * 32 + t;
                if (k < K) {
                    const int c = k / (KS * KS), r = k - c * KS * KS, kh = r / KS, kw = r - kh * KS;
                    const bool in = ((rmask >> kh) & (cmask >> kw) & 1u) != 0;
                    v[t] = in ? __ldg(xp + c * xs_c + kh * xs_h + kw * xs_w) : 0.f;
                } else {
                    v[t] = 0.f;
                }
            }
            uint8_t *row = sA + buf * ST_A_BYTES + row_off;
#pragma unroll
            for (int q = 0; q < 8; ++q)
                *reinterpret_cast<uint4 *>(row + ((q ^ sw) << 4)) =
                    make_uint4(__float_as_uint(round_tf32(v[4 * q])), __float_as_uint(round_tf32(v[4 * q + 1])),
                               __float_as_uint(round_tf32(v[4 * q + 2])), __float_as_uint(round_tf32(v[4 * q + 3])));
            fence_async_smem();
            tc_fence_before();
            if (__syncthreads_or(failed)) { stop = true; break; }
            if (tid == 0) {
                tc_fence_after();
                const uint64_t da = da0 + (uint64_t)(buf * (ST_A_BYTES >> 4)), db = db0 + kb * b_step;
                umma<MMA_TF32>(tmem_base, da, db, idesc, kb > 0 ? 1u : 0u);
                umma<MMA_TF32>(tmem_base, da + 2, db + 2, idesc, 1u);
                umma<MMA_TF32>(tmem_base, da + 4, db + 4, idesc, 1u);
                umma<MMA_TF32>(tmem_base, da + 6, db + 6, idesc, 1u);
                umma_commit(done0 + 8 * buf);
                if (kb == KB - 1) umma_commit(acc_bar);
            }
            __syncwarp();
            ++kcount;
        }
        if (stop) break;
        // ---- epilogue: all of the tile's MMAs have retired, the row buffers are free for the staged output
        if (!mbar_wait(acc_bar, (uint32_t)(it & 1), abort_flag, status, ST_WAIT_ACC, 0, wait_limit)) failed = true;
        if (!failed) {
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(warp * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < n_pad; c0 += 16) {
                uint32_t r[16];
                tmem_ld16(t_row + c0, r);
                tmem_ld_wait();
                float o[16];
                const float4 *sc4 = reinterpret_cast<const float4 *>(s_scale + c0);
                const float4 *sf4 = reinterpret_cast<const float4 *>(s_shift + c0);
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 sc = sc4[q], sf = sf4[q];
                    const float scv[4] = {sc.x, sc.y, sc.z, sc.w}, sfv[4] = {sf.x, sf.y, sf.z, sf.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = 4 * q + e;
                        float t = stem_act<ACT>(fmaf(__uint_as_float(r[j]), scv[e], sfv[e]), runtime_act);
                        if (do_round) t = round_tf32(t);
                        o[j] = (ACT == ST_ACT_GENERIC && c0 + j >= g.n) ? 0.f : t;
                    }
                }
                // byte offset of these 16 columns inside the pixel's row, split into 128-byte halves
                const uint32_t byte0 = (uint32_t)c0 * (OUT_BF16 ? 2u : 4u);
                uint8_t *half = sA + (byte0 >> 7) * ST_A_BYTES + (uint32_t)tid * half_bytes;
                const uint32_t q0 = (byte0 & 127u) >> 4;
                if (!OUT_BF16) {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                        *reinterpret_cast<uint4 *>(half + (((q0 + q) ^ q_xor) << 4)) =
                            make_uint4(__float_as_uint(o[4 * q]), __float_as_uint(o[4 * q + 1]), __float_as_uint(o[4 * q + 2]), __float_as_uint(o[4 * q + 3]));
                } else {
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        uint4 pk;
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(o[8 * q], o[8 * q + 1]);
                        __nv_bfloat162 h1 = __floats2bfloat162_rn(o[8 * q + 2], o[8 * q + 3]);
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(o[8 * q + 4], o[8 * q + 5]);
                        __nv_bfloat162 h3 = __floats2bfloat162_rn(o[8 * q + 6], o[8 * q + 7]);
                        pk.x = *reinterpret_cast<uint32_t *>(&h0); pk.y = *reinterpret_cast<uint32_t *>(&h1);
                        pk.z = *reinterpret_cast<uint32_t *>(&h2); pk.w = *reinterpret_cast<uint32_t *>(&h3);
                        *reinterpret_cast<uint4 *>(half + (((q0 + q) ^ q_xor) << 4)) = pk;
                    }
                }
            }
            fence_async_smem();
            __syncwarp();
            const int row0 = tile * ST_THREADS + warp * 32;
            if (lane == 0 && row0 < npix) {
                for (uint32_t hb = 0; hb * 128u < out_row_bytes; ++hb)
                    tma_store_2d(ymap, smem_u32(sA + hb * ST_A_BYTES) + (uint32_t)(warp * 32) * half_bytes,
                                 (int)(hb * 128u / (OUT_BF16 ? 2u : 4u)), row0);
                tma_store_commit();
            }
        }
        tc_fence_before();   // this tile's TMEM loads precede the next tile's first barrier and MMA
    }
    if (lane == 0) tma_store_wait_all();

    if (*abort_flag) {
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000LL) { }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
}

// ------------------------------------------------------------------ host side
static bool stem_is_wide(const ConvGeom &g) { return g.c == 3 && (g.size == 5 || g.size == 7); }

bool conv_stem_tc_covers(const ConvGeom &g)
{
    const bool narrow = g.size == 3 && g.c >= 1 && g.c <= 3;
    return (narrow || stem_is_wide(g)) && g.groups == 1 && g.n % 16 == 0 && g.n <= 64 && g.stride >= 1 && g.stride <= 2;
}

template <int KS, int ACT, bool OBF>
static int launch_wide_one(const StemTcArgs &a, cudaStream_t s)
{
    auto kern = conv_stem_tc_wide_kernel<3, KS, ACT, OBF>;
    constexpr int KB = (3 * KS * KS + 31) / 32;
    const size_t smem = 2 * ST_A_BYTES + (size_t)KB * a.n_pad * 128 + 2 * sizeof(float) * a.n_pad + sizeof(StemWideShared) + 16;
    DNB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    DNB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    int per_sm = (int)((228 * 1024) / (smem + 1024));
    if (per_sm > 3) per_sm = 3;   // the kernel's register budget (__launch_bounds__)
    if (per_sm > 512 / a.tmem_cols) per_sm = 512 / a.tmem_cols;
    if (per_sm < 1) DNB_FAIL(DNB_ECUDA, "first-layer kernel: %zu bytes of shared memory do not fit", smem);
    long long grid = (long long)sm_count() * per_sm;
    if (grid > a.tiles) grid = a.tiles;
    kern<<<(unsigned)grid, ST_THREADS, smem, s>>>(a);
    DNB_LAUNCH_CHECK("conv_stem_tc_wide");
    return DNB_OK;
}

template <int KS, bool OBF>
static int launch_wide_act(const StemTcArgs &a, cudaStream_t s)
{
    if (a.ep.activation == DNB_LEAKY) return launch_wide_one<KS, DNB_LEAKY, OBF>(a, s);
    if (a.ep.activation == DNB_LINEAR) return launch_wide_one<KS, DNB_LINEAR, OBF>(a, s);
    return launch_wide_one<KS, ST_ACT_GENERIC, OBF>(a, s);
}

template <int C, int ACT, bool OBF>
static int launch_one(const StemTcArgs &a, size_t smem, int grid_limit_per_sm, cudaStream_t s)
{
    auto kern = conv_stem_tc_kernel<C, ACT, OBF>;
    DNB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    // all of the SM's configurable memory as shared memory, so that several CTAs are resident
    DNB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
    int per_sm = (int)((228 * 1024) / (smem + 1024));   // each resident CTA also reserves 1 KB
    if (per_sm > 2048 / ST_THREADS) per_sm = 2048 / ST_THREADS;
    if (per_sm > 5) per_sm = 5;   // the kernel's register budget (__launch_bounds__)
    if (per_sm < 1) DNB_FAIL(DNB_ECUDA, "first-layer kernel: %zu bytes of shared memory do not fit", smem);
    if (per_sm > grid_limit_per_sm) per_sm = grid_limit_per_sm;
    long long grid = (long long)sm_count() * per_sm;
    if (grid > a.tiles) grid = a.tiles;
    kern<<<(unsigned)grid, ST_THREADS, smem, s>>>(a);
    DNB_LAUNCH_CHECK("conv_stem_tc");
    return DNB_OK;
}

template <int C, bool OBF>
static int launch_act(const StemTcArgs &a, size_t smem, int lim, cudaStream_t s)
{
    if (a.ep.activation == DNB_LEAKY) return launch_one<C, DNB_LEAKY, OBF>(a, smem, lim, s);
    if (a.ep.activation == DNB_LINEAR) return launch_one<C, DNB_LINEAR, OBF>(a, smem, lim, s);
    return launch_one<C, ST_ACT_GENERIC, OBF>(a, smem, lim, s);
}

int launch_conv_stem_tc(StemTcArgs a, cudaStream_t s)
{
    const ConvGeom &g = a.g;
    if (!conv_stem_tc_covers(g)) DNB_FAIL(DNB_EUNSUPPORTED, "first-layer kernel: geometry outside its coverage");
    const long long npix = (long long)g.batch * g.out_h * g.out_w;
    if (npix + ST_THREADS >= (1LL << 31)) DNB_FAIL(DNB_EUNSUPPORTED, "first-layer kernel: %lld output pixels", npix);
    if (a.xs_c >= (1LL << 31) / 4 || a.xs_h >= (1LL << 31) / 4) DNB_FAIL(DNB_EUNSUPPORTED, "first-layer kernel: image too large for 32-bit offsets");
    a.npix = (int)npix;
    a.tiles = (int)((npix + ST_THREADS - 1) / ST_THREADS);
    a.n_pad = round_up(g.n, 16);
    a.tmem_cols = 32;
    while (a.tmem_cols < a.n_pad) a.tmem_cols *= 2;
    size_t smem = 2 * ST_A_BYTES + (size_t)a.n_pad * 128 + 2 * sizeof(float) * a.n_pad + sizeof(StemShared) + 16;
    // TMEM holds 512 columns per SM: never more CTAs on an SM than can all hold their accumulators at once.
    // The grid is sized for that, and the shared-memory request is padded so that one more would not fit.
    const int lim = 512 / a.tmem_cols;
    const size_t sm_bytes = 228 * 1024, reserved = 1024;   // per SM, and per resident CTA
    if ((smem + reserved) * (lim + 1) <= sm_bytes) smem = sm_bytes / (lim + 1) - reserved + 16;
    const bool obf = a.y_dtype == DNB_BF16;
    if (stem_is_wide(g)) {
        // rows of up to 256 bytes, in halves of at most 128: one or two 32-row boxes per warp
        const int rb = a.y_cpitch * (obf ? 2 : 4);
        if (a.y_cpitch != g.n || (rb != 32 && rb != 64 && rb != 128 && rb != 256)) DNB_FAIL(DNB_EUNSUPPORTED, "first-layer kernel: output rows of %d bytes", rb);
        const int half = rb > 128 ? 128 : rb;
        const uint64_t dims[2] = {(uint64_t)a.y_cpitch, (uint64_t)npix};
        const uint64_t strides[1] = {(uint64_t)rb};
        const uint32_t box[2] = {(uint32_t)(half / (obf ? 2 : 4)), 32u};
        DNB_TRY(encode_tensor_map(&a.tmy, obf, 2, a.y, dims, strides, box, half));
        a.tma_store = 1;
        if (g.size == 7) return obf ? launch_wide_act<7, true>(a, s) : launch_wide_act<7, false>(a, s);
        return obf ? launch_wide_act<5, true>(a, s) : launch_wide_act<5, false>(a, s);
    }
    // rows of 32, 64 or 128 bytes leave through TMA stores from swizzled staging rows; wider ones by plain stores
    const int row_bytes = a.y_cpitch * (obf ? 2 : 4);
    a.tma_store = (a.y_cpitch == g.n && (row_bytes == 32 || row_bytes == 64 || row_bytes == 128)) ? 1 : 0;
    if (const char *e = getenv("DNB_STEM_TMA")) a.tma_store = a.tma_store && atoi(e) != 0;
    if (a.tma_store) {
        const uint64_t dims[2] = {(uint64_t)a.y_cpitch, (uint64_t)npix};
        const uint64_t strides[1] = {(uint64_t)row_bytes};
        const uint32_t box[2] = {(uint32_t)a.y_cpitch, 32u};
        DNB_TRY(encode_tensor_map(&a.tmy, obf, 2, a.y, dims, strides, box, row_bytes));
    }
    switch (g.c) {
    case 1: return obf ? launch_act<1, true>(a, smem, lim, s) : launch_act<1, false>(a, smem, lim, s);
    case 2: return obf ? launch_act<2, true>(a, smem, lim, s) : launch_act<2, false>(a, smem, lim, s);
    default: return obf ? launch_act<3, true>(a, smem, lim, s) : launch_act<3, false>(a, smem, lim, s);
    }
}

}  // namespace dnb
