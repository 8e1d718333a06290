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
// * Accumulators live in TMEM (fp32); two accumulator buffers of bn columns let the
//   epilogue of tile i overlap the MMAs of tile i+1.
// * Warp roles in a 192-thread CTA: warp 0 issues TMA (one thread), warp 1 issues
//   tcgen05.mma (one thread) and owns the TMEM allocation, warps 2-5 drain TMEM
//   and apply the fused epilogue: folded batchnorm or bias, activation, optionally
//   the residual add of a following shortcut layer (its tile arrives by TMA in the
//   staging buffer the finished rows then overwrite), TF32 rounding, TMA store of
//   the channels-last rows and/or plain stores of Darknet's NCHW layout.
// * Persistent: one CTA per SM (two when the filter tile is at most 128 wide) walks
//   tiles blockIdx.x, +gridDim.x, ...; tiles that share a pixel box are adjacent so
//   the box is fetched from HBM once and re-read from L2 by the neighbouring CTAs.
//   No cluster, no multicast.
// * The depth of the operand ring decides how much load latency is hidden (2 / 3 / 4
//   slots: 0.45 / 0.35 / 0.32 ms on a 76x76 256-filter layer), so shared memory is
//   budgeted to the byte: no alignment slack, only the current filter tile's
//   scale/shift vectors, staging rows as narrow as four ring slots require.
// * Every mbarrier wait is bounded: when it expires the CTA records a code in
//   the status word, raises a shared abort flag that all roles poll, drains,
//   frees its TMEM and returns.  The kernel never traps.
//
// Replaces forward_convolutional_layer_gpu (src/convolutional_kernels.cu:73-135
// of the reference) for groups == 1 and c >= 8, and with it the shortcut layer that follows
// (forward_shortcut_layer_gpu, src/shortcut_layer.c:75-80; src/blas_kernels.cu:711-745) when the caller asks for the fusion.
#include <cuda.h>

#include "common.h"
#include "conv.h"
#include "device_utils.cuh"
#include "tc_ptx.cuh"

namespace dnb {

constexpr int TC_THREADS = 192;
constexpr int MAX_STAGES = 8;
constexpr int MAX_B_STAGES = 12;   // weight-tile ring of the halo mode
constexpr int MAX_RES_BUFS = 4;   // staging buffers with a fused residual; tiles are requested two chunks ahead

// ------------------------------------------------------------------ kernel
struct TcShared {
    uint64_t full[MAX_STAGES];     // operand ring (halo mode: the ring of activation boxes)
    uint64_t empty[MAX_STAGES];
    uint64_t full_b[MAX_B_STAGES]; // halo mode: the ring of weight tiles
    uint64_t empty_b[MAX_B_STAGES];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t res_full[MAX_RES_BUFS];   // residual tile landed in its staging buffer
    uint32_t tmem_base;
    int abort_flag;
    int split_last;                    // split-K: this CTA delivered the last partial sum of the tile it is finishing
};

enum { WAIT_EMPTY = 101, WAIT_FULL = 102, WAIT_ACC_EMPTY = 103, WAIT_ACC_FULL = 104, WAIT_RESIDUAL = 105, BAD_SMEM_BASE = 106 };
enum { ACT_GENERIC = -1, ACT2_NONE = -2, ACT_YOLO = -3 };   // ACT2_NONE: no fused residual; ACT_YOLO: linear, then the [yolo] layer's per-entry logistic


template <int ACT>
__device__ __forceinline__ float act_apply(float x, int runtime_act)
{
    if (ACT == DNB_LINEAR || ACT == ACT_YOLO) return x;
    if (ACT == DNB_LEAKY) return fmaxf(x, 0.1f * x);   // x > 0 ? x : 0.1x
    // the run-time variant: relu (Darknet's VGG and AlexNet cfgs) and logistic inline, the rest of the 14-way switch
    // out of line (a call per element costs the epilogue several times its normal instruction count)
    if (runtime_act == DNB_RELU) return x > 0.f ? x : 0.f;
    if (runtime_act == DNB_LOGISTIC) return 1.f / (1.f + expf(-x));
    return activate_call(x, runtime_act);
}

// ACT: activation folded at compile time (DNB_LINEAR, DNB_LEAKY) or ACT_GENERIC (runtime switch).
// ACT2: ACT2_NONE, or the activation of the fused shortcut layer (same three choices).  The epilogue's chunk
// body is unrolled over CPC columns and shares the instruction cache with the TMA and MMA loops: every
// per-element run-time choice that can be a template parameter is one, or the warps stall on instruction fetch.
// CPC: output columns per staged chunk (16, 32 or 64); OUT_BF16: storage type of the operands and of the
// NHWC output (bf16 for BF16 plans, f32 with TF32 products otherwise).
// One staged row is CPC * sizeof(output element) bytes = the swizzle span of the store map.
// PAIR: the kernel runs as clusters of two CTAs that share every MMA (cta_group::2): one tile index names two
// adjacent pixel tiles (one per CTA) under one 256-filter tile; each CTA loads its own 128 pixels and HALF of the
// weight tile, so a third fewer operand bytes cross L2 -> shared memory per MMA and the ring is six slots deep.
// The even CTA issues the MMAs for both; each CTA drains its own 128 accumulator rows.
// I8: operands are int8 sign tensors (+1 / -1, 0 in padding channels and, through the TMA zero fill, outside the
// image), products accumulate exactly in int32 (kind::i8): the xnor convolution on the tensor cores.  The epilogue
// converts the integer sums to float and continues as for the other kinds (output f32, OUT_BF16 false).
// SPLIT: the K loop (taps x channel blocks) of every output tile is cut into a.splits consecutive ranges that run as
// separate tiles, on different CTAs at the same time: for layers with fewer tiles than SMs and a long K loop (small
// batches of the 19x19 and 38x38 layers).  Every range's CTA writes its raw accumulators to a scratch tensor in
// global memory (L2), then adds one to the tile's counter; the CTA that finds the counter at splits - 1 is the last
// one, sums all ranges in their fixed order (so the result does not depend on who came last) and runs the normal
// epilogue.  Nobody waits for anybody: no spin, no deadlock.  The last CTA resets the counter for the next launch.
// SIGNS (int8 kind, 128-byte staged rows): beside its f32 output the layer writes the output's signs (+1 where the value
// is > 0, else -1, 0 beyond the layer's filters) as the int8 channels-last tensor that the xnor layer after it reads as
// its operand: that layer's sign pass over the f32 tensor disappears.  The signs of a chunk are staged in a third
// staging buffer (two 4 KB halves in rotation) and leave with the chunk's output rows, in the same bulk group.
template <int ACT, int CPC, bool OUT_BF16, int ACT2, bool PAIR, bool I8 = false, bool SPLIT = false, bool SIGNS = false>
__global__ void __launch_bounds__(TC_THREADS)
conv_tc_kernel(const __grid_constant__ TcArgs a)
{
    static_assert(!SIGNS || (I8 && CPC == 32 && !OUT_BF16 && !SPLIT), "the sign output belongs to the int8 kind with 128-byte staged rows");
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // operand ring, 1024-byte aligned (the 128-byte swizzle pattern repeats every 1024 bytes).  The kernel
    // has no static shared memory, so the dynamic window starts aligned; no slack is budgeted for rounding
    // up, and a launch that finds it otherwise reports that and does nothing.
    const uint32_t ring = smem_u32(smem_raw);
    if (ring & 1023u) {
        if (threadIdx.x == 0) atomicCAS(a.status, 0, BAD_SMEM_BASE);
        return;
    }
    const uint32_t stage_bytes = a.a_bytes + a.b_bytes;
    const size_t ring_bytes = a.halo ? (size_t)a.a_stages * a.a_slot + (size_t)a.b_stages * a.b_bytes : (size_t)a.stages * stage_bytes;
    uint8_t *after_ring = smem_raw + (ring - smem_u32(smem_raw)) + ring_bytes;
    // staging buffers of 128 rows x store_row_bytes: two for plain stores; four when a residual is fused, each
    // then receiving a residual tile first and the finished output rows, in place, afterwards
    uint8_t *stage_out = after_ring;
    float *s_scale = reinterpret_cast<float *>(stage_out + (size_t)a.stage_bufs * 128 * (CPC * (OUT_BF16 ? 2 : 4)));
    float *s_shift = s_scale + a.bn + 64;   // the current filter tile's vectors, padded by one widest chunk
    TcShared *sh = reinterpret_cast<TcShared *>(s_shift + a.bn + 64);
    volatile int *abort_flag = &sh->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta_rank = PAIR ? cluster_ctarank() : 0u;   // 0: the CTA that issues the pair's MMAs
    const bool leader = cta_rank == 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < MAX_STAGES; ++s) {
            mbar_init(smem_u32(&sh->full[s]), 1);
            mbar_init(smem_u32(&sh->empty[s]), 1);
        }
        for (int s = 0; s < MAX_B_STAGES; ++s) {
            mbar_init(smem_u32(&sh->full_b[s]), 1);
            mbar_init(smem_u32(&sh->empty_b[s]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&sh->acc_full[i]), 1);
            mbar_init(smem_u32(&sh->acc_empty[i]), PAIR ? 8 : 4);   // the epilogue warps of both CTAs of a pair
        }
        for (int i = 0; i < MAX_RES_BUFS; ++i) mbar_init(smem_u32(&sh->res_full[i]), 1);
        sh->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    const uint32_t tmem_cols = (uint32_t)a.tmem_cols, acc_stride = tmem_cols / 2;
    if (warp == 1) {  // TMEM: two accumulators of tmem_cols/2 columns each (512 in all for 256-filter tiles), whole warp
        if (PAIR) {   // the same warp of both CTAs, the same shared-memory offset for the result
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(tmem_cols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sh->tmem_base)), "r"(tmem_cols) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync_all();   // the other CTA's barriers are initialised before anything is signalled across the pair
    tc_fence_after();
    // Everything above touched only this CTA's shared memory and TMEM: it may run while the previous layer's kernel is
    // still draining.  From here on the previous layer's output is read and buffers it may still read are written.
    grid_dependency_wait();
    launch_dependents();   // this grid is persistent and fully resident: the next layer's CTAs take SMs only as ours leave
    const uint32_t tmem_base = sh->tmem_base;

    // Kernel parameters live in the constant bank, and every asm statement below is a compiler memory
    // barrier: anything read through `a` inside a loop would be re-fetched each iteration.  The loops
    // therefore work on register copies only.
    const int taps = a.taps, c_blocks = a.c_blocks, k_iters = taps * c_blocks;
    const int n_tiles = a.n_tiles, total_tiles = a.total_tiles, stages = a.stages, bn = a.bn, bk = a.bk;
    const int tiles_w = a.tiles_w, tiles_h = a.tiles_h, ptiles_wh = tiles_w * tiles_h;
    const int wt = a.wt, ht = a.ht, bt = a.bt, row_bytes = a.row_bytes;
    const uint32_t a_bytes = a.a_bytes;
    const int grid_stride = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    const int first_tile = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    // tile index -> pixel tile of this CTA.  The last pair of an odd number of pixel tiles gives its second CTA a
    // tile past the batch: its loads are zero-filled, its stores are skipped.
    auto pixel_tile = [&](int tile) { return PAIR ? 2 * (tile / n_tiles) + (int)cta_rank : tile / n_tiles; };
    const long long wait_limit = a.wait_limit;
    const int splits = SPLIT ? a.splits : 1;
    // tile index -> (output tile, K range); the ranges of one output tile are consecutive tile indices, i.e. they
    // run on neighbouring CTAs at the same time
    auto k_begin = [&](int split) { return SPLIT ? (int)((long long)split * k_iters / splits) : 0; };

    if (warp == 0) {
        // ---------------- TMA producer: one thread runs the loop, the other lanes wait at the __syncwarp
        const int ksize = a.g.size, cstride = a.g.stride, cpad = a.g.pad;
        const uint32_t tx_bytes = 128u * row_bytes + (uint32_t)(PAIR ? bn >> 1 : bn) * row_bytes;
        const CUtensorMap *maps = a.tmx;
        const CUtensorMap *wmap = &a.tmw;
        int *status = a.status;
        const uint32_t full0 = smem_u32(&sh->full[0]), empty0 = smem_u32(&sh->empty[0]);
        const bool withhold = (a.debug & 32) != 0;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        if (a.halo) {
            // one activation box per channel block, then the nine weight tiles that multiply it
            const int a_stages = a.a_stages, b_stages = a.b_stages;
            const uint32_t a_slot = a.a_slot, a_tx = a.a_box_bytes, b_slot = a.b_bytes, b_tx = (uint32_t)bn * row_bytes;
            const uint32_t ring_b = ring + a_stages * a_slot;
            const uint32_t fullb0 = smem_u32(&sh->full_b[0]), emptyb0 = smem_u32(&sh->empty_b[0]);
            int sb = 0;
            uint32_t phase_b = 0;
            for (int tile = blockIdx.x; lane == 0 && tile < total_tiles && ok; tile += grid_stride) {
                const int nt = tile % n_tiles, pt = tile / n_tiles;
                const int ow0 = (pt % tiles_w) * wt, oh0 = ((pt / tiles_w) % tiles_h) * ht, b0 = (pt / ptiles_wh) * bt;
                const int n0 = nt * bn;
                for (int cb = 0; cb < c_blocks && ok; ++cb) {
                    ok = mbar_wait_thread(empty0 + 8 * stage, phase ^ 1, abort_flag, status, WAIT_EMPTY, wait_limit);
                    if (!ok) break;
                    mbar_expect_tx(full0 + 8 * stage, a_tx);
                    tma_load_4d(ring + stage * a_slot, maps, full0 + 8 * stage, cb * bk, ow0 - cpad, oh0 - cpad, b0);
                    if (++stage == a_stages) { stage = 0; phase ^= 1; }
                    for (int tap = 0; tap < taps; ++tap) {
                        ok = mbar_wait_thread(emptyb0 + 8 * sb, phase_b ^ 1, abort_flag, status, WAIT_EMPTY, wait_limit);
                        if (!ok) break;
                        mbar_expect_tx(fullb0 + 8 * sb, b_tx);
                        tma_load_3d(ring_b + sb * b_slot, wmap, fullb0 + 8 * sb, cb * bk, n0, tap);
                        if (++sb == b_stages) { sb = 0; phase_b ^= 1; }
                    }
                }
            }
        } else
        for (int tile = first_tile; lane == 0 && tile < total_tiles && ok; tile += grid_stride) {
            const int base = SPLIT ? tile / splits : tile, split = SPLIT ? tile - base * splits : 0;
            const int nt = base % n_tiles, pt = pixel_tile(base);
            const int ow0 = (pt % tiles_w) * wt;
            const int oh0 = ((pt / tiles_w) % tiles_h) * ht;
            const int b0 = (pt / ptiles_wh) * bt;
            const int n0 = nt * bn + (PAIR ? (int)cta_rank * (bn >> 1) : 0);   // a pair's CTAs load one half of the filter tile each
            const int k0 = k_begin(split), k1 = SPLIT ? k_begin(split + 1) : k_iters;
            int tap = k0 / c_blocks, cb = k0 - tap * c_blocks;
            int kh = tap / ksize, kw = tap - kh * ksize;
            for (int ki = k0; ki < k1; ++ki) {
                // input row = oh*stride + kh - pad = stride*(oh + q) + parity
                const int dh = kh - cpad, dw = kw - cpad;
                int ph = 0, qh = dh, pw = 0, qw = dw;
                if (cstride == 2) { ph = dh & 1; qh = (dh - ph) >> 1; pw = dw & 1; qw = (dw - pw) >> 1; }
                const CUtensorMap *mx = maps + (ph * cstride + pw);
                ok = mbar_wait_thread(empty0 + 8 * stage, phase ^ 1, abort_flag, status, WAIT_EMPTY, wait_limit);
                if (!ok) break;
                // wait-expiry test (debug bit 32): the last operand load of this CTA's first tile is never
                // requested, so the MMA role's wait for it runs out and the CTA takes the abort path
                if (withhold && tile == first_tile && ki == k1 - 1) { ok = false; break; }
                const uint32_t bar = full0 + 8 * stage;
                const uint32_t sa = ring + stage * stage_bytes;
                if (PAIR) {
                    // one barrier, in the even CTA, counts the bytes of both CTAs' loads of this slot
                    if (leader) mbar_expect_tx(bar, 2u * tx_bytes);
                    tma_load_4d_pair(sa, mx, bar, cb * bk, ow0 + qw, oh0 + qh, b0);
                    tma_load_3d_pair(sa + a_bytes, wmap, bar, cb * bk, n0, tap);
                } else {
                    mbar_expect_tx(bar, tx_bytes);
                    tma_load_4d(sa, mx, bar, cb * bk, ow0 + qw, oh0 + qh, b0);
                    tma_load_3d(sa + a_bytes, wmap, bar, cb * bk, n0, tap);
                }
                if (++stage == stages) { stage = 0; phase ^= 1; }
                if (++cb == c_blocks) {
                    cb = 0; ++tap;
                    if (++kw == ksize) { kw = 0; ++kh; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer: one thread.  Its instruction stream per ring slot has to stay well
        // below the 4 x 128 cycles the tensor pipe needs for the slot's MMAs, so everything is in registers:
        // barrier addresses and operand descriptors advance by constants, the accumulator-ready commit
        // sits after the k loop.
        constexpr int is_bf16 = I8 ? MMA_I8 : (OUT_BF16 ? MMA_BF16 : MMA_TF32);   // operand kind of the MMAs
        const uint32_t idesc = mma_idesc<is_bf16>(PAIR ? 256u : 128u, (uint32_t)bn);
        const int k_steps = row_bytes / 32;      // one MMA consumes 32 bytes of K per row
        const uint64_t da0 = make_smem_desc(ring, row_bytes), db0 = make_smem_desc(ring + a_bytes, row_bytes);
        const uint64_t slot_step = stage_bytes >> 4;   // descriptor address field counts 16-byte units
        const uint32_t full0 = smem_u32(&sh->full[0]), empty0 = smem_u32(&sh->empty[0]);
        int *status = a.status;
        const int dbg_mma = a.debug;
        int stage = 0;
        uint32_t phase = 0;
        uint64_t da = da0, db = db0;
        int it = 0;
        bool ok = true;
        if (a.halo) {
            const int a_stages = a.a_stages, b_stages = a.b_stages, pitch = a.a_pitch, ksize = a.g.size;
            const uint32_t fullb0 = smem_u32(&sh->full_b[0]), emptyb0 = smem_u32(&sh->empty_b[0]);
            // A descriptor of a box: rows of 128 bytes, 8-row groups one box row (pitch pixels) apart
            uint64_t dbox0 = make_smem_desc(ring, 128);
            dbox0 = (dbox0 & ~((uint64_t)0x3FFF << 32)) | ((uint64_t)(pitch * 8) << 32);
            const uint64_t dw0 = make_smem_desc(ring + a_stages * a.a_slot, 128);
            const uint64_t a_step = (uint64_t)(a.a_slot >> 4), b_step = (uint64_t)(a.b_bytes >> 4);
            int sb = 0;
            uint32_t phase_b = 0;
            for (int tile = blockIdx.x; lane == 0 && tile < total_tiles && ok; tile += grid_stride, ++it) {
                const int acc = it & 1;
                const uint32_t acc_phase = (it >> 1) & 1;
                ok = mbar_wait_thread(smem_u32(&sh->acc_empty[acc]), acc_phase ^ 1, abort_flag, status, WAIT_ACC_EMPTY, wait_limit);
                if (!ok) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * acc_stride;
                uint32_t accumulate = 0u;
                for (int cb = 0; cb < c_blocks && ok; ++cb) {
                    ok = mbar_wait_thread(full0 + 8 * stage, phase, abort_flag, status, WAIT_FULL, wait_limit);
                    if (!ok) break;
                    const uint64_t dbox = dbox0 + stage * a_step;
                    int kh = 0, kw = 0;
                    for (int tap = 0; tap < taps; ++tap) {
                        ok = mbar_wait_thread(fullb0 + 8 * sb, phase_b, abort_flag, status, WAIT_FULL, wait_limit);
                        if (!ok) break;
                        tc_fence_after();
                        const uint64_t da = dbox + (uint64_t)((kh * pitch + kw) * 8);   // 128-byte rows in 16-byte units
                        const uint64_t db = dw0 + sb * b_step;
                        if (!(dbg_mma & 16)) {
                            umma<is_bf16>(d_tmem, da, db, idesc, accumulate);
                            umma<is_bf16>(d_tmem, da + 2, db + 2, idesc, 1u);
                            umma<is_bf16>(d_tmem, da + 4, db + 4, idesc, 1u);
                            umma<is_bf16>(d_tmem, da + 6, db + 6, idesc, 1u);
                        }
                        accumulate = 1u;
                        umma_commit(emptyb0 + 8 * sb);   // the weight tile is free when these MMAs retire
                        if (++sb == b_stages) { sb = 0; phase_b ^= 1; }
                        if (++kw == ksize) { kw = 0; ++kh; }
                    }
                    if (ok) umma_commit(empty0 + 8 * stage);   // and the box when all nine taps have read it
                    if (++stage == a_stages) { stage = 0; phase ^= 1; }
                }
                if (ok) umma_commit(smem_u32(&sh->acc_full[acc]));
            }
        } else
        for (int tile = first_tile; lane == 0 && leader && tile < total_tiles && ok; tile += grid_stride, ++it) {
            const int acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            ok = mbar_wait_thread(smem_u32(&sh->acc_empty[acc]), acc_phase ^ 1, abort_flag, status, WAIT_ACC_EMPTY, wait_limit);
            if (!ok) break;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + acc * acc_stride;
            const int split = SPLIT ? tile % splits : 0;
            const int kn = SPLIT ? k_begin(split + 1) - k_begin(split) : k_iters;   // this tile's share of the K loop
            for (int ki = 0; ki < kn; ++ki) {
                ok = mbar_wait_thread(full0 + 8 * stage, phase, abort_flag, status, WAIT_FULL, wait_limit);
                if (!ok) break;
                tc_fence_after();
                if (dbg_mma & 16) {
                } else if (PAIR) {   // the same descriptors address both CTAs' shared memory; row_bytes is 128 in pair mode
                    umma_pair<is_bf16>(d_tmem, da, db, idesc, ki != 0);
                    umma_pair<is_bf16>(d_tmem, da + 2, db + 2, idesc, 1u);
                    umma_pair<is_bf16>(d_tmem, da + 4, db + 4, idesc, 1u);
                    umma_pair<is_bf16>(d_tmem, da + 6, db + 6, idesc, 1u);
                } else if (k_steps == 4) {
                    umma<is_bf16>(d_tmem, da, db, idesc, ki != 0);
                    umma<is_bf16>(d_tmem, da + 2, db + 2, idesc, 1u);
                    umma<is_bf16>(d_tmem, da + 4, db + 4, idesc, 1u);
                    umma<is_bf16>(d_tmem, da + 6, db + 6, idesc, 1u);
                } else {
                    for (int k = 0; k < k_steps; ++k) umma<is_bf16>(d_tmem, da + 2 * k, db + 2 * k, idesc, (ki | k) != 0);
                }
                // frees the slot (in both CTAs of a pair) when these MMAs retire
                if (PAIR) umma_commit_pair(empty0 + 8 * stage); else umma_commit(empty0 + 8 * stage);
                da += slot_step; db += slot_step;
                if (++stage == stages) { stage = 0; phase ^= 1; da = da0; db = db0; }
            }
            if (ok) {   // accumulator complete (in both CTAs of a pair) when all MMAs above retire
                if (PAIR) umma_commit_pair(smem_u32(&sh->acc_full[acc])); else umma_commit(smem_u32(&sh->acc_full[acc]));
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: warps 2..5 own TMEM lanes 32*(warp%4) .. +31
        const int quarter = warp & 3;
        const int m = quarter * 32 + lane;  // pixel index inside the tile = TMEM lane = staging row
        const int wl = m % wt, hl = (m / wt) % ht, bl = m / (wt * ht);
        const ConvGeom g = a.g;   // register copy
        void *const y_nhwc = a.y_nhwc;
        float *const y_nchw = a.y_nchw;
        const int runtime_act = a.ep.activation, do_round = a.ep.round_tf32;
        const bool raw_acc = I8 && a.ep.raw_acc != 0;
        const int yolo_entries = ACT == ACT_YOLO ? a.ep.yolo_entries : 1;   // fused [yolo] head: a kernel variant of its own
        constexpr bool residual = ACT2 != ACT2_NONE;
        // A CTA pair reads the residual with plain 16-byte loads, one staged chunk ahead, instead of TMA tiles into the
        // staging buffers: residual tile loads inside the pair kernel raised an illegal-instruction fault on B200 whose
        // cause was not found, so that combination is not built.  Each thread reads its own pixel's 128 contiguous bytes.
        constexpr bool res_direct = residual && PAIR;
        constexpr bool res_tiles = residual && !PAIR;
        const CUtensorMap *rmap = &a.tmr;
        const uint32_t buf_mask = res_tiles ? 3u : 1u;   // staging buffers in rotation
        constexpr int res_ahead = 3;   // residual tiles requested ahead of the chunk being finished (of four buffers)
        const int act2 = a.ep.activation2;
        const float res_alpha = a.ep.alpha, res_beta = a.ep.beta;
        const CUtensorMap *ymap = &a.tmy;
        int *status = a.status;
        const bool store_thread = threadIdx.x == 64;
        // Per-warp stores (no residual tiles, no sign output): every warp stages its own 32 rows, which are a box of the
        // output like the whole tile is, and sends them off itself; the four warps then meet once per tile instead of
        // twice per chunk, so one warp's TMEM or store wait no longer stalls the other three.
        constexpr bool can_warp_store = ACT2 == ACT2_NONE || PAIR;
        const bool warp_stores = can_warp_store && !SIGNS && a.warp_stores != 0 && a.y_nhwc != nullptr;
        const int m0 = quarter * 32;
        const int wl0 = m0 % wt, hl0 = (m0 / wt) % ht, bl0 = m0 / (wt * ht);   // origin of this warp's rows inside the tile
        constexpr bool out_bf16 = OUT_BF16;
        constexpr int srb = CPC * (OUT_BF16 ? 2 : 4);            // bytes of one staged row = swizzle span
        constexpr int q_mask = srb / 16 - 1;
        const int q_xor = (m >> (srb == 128 ? 0 : (srb == 64 ? 1 : 2))) & q_mask;   // 16-byte chunk swizzle of row m
        uint32_t chunk_count = 0;
        int it = 0, loaded_nt = -1;
        // Residual tiles are requested as one stream of chunks that runs res_ahead chunks in front of the epilogue
        // and does not stop at tile boundaries: what bounds a layer with a fused residual is how many bytes of it
        // are in flight, so the requests must not drain while the epilogue waits for the next accumulator.
        uint32_t pf_count = 0;                 // chunks requested so far (buffer = count & 3)
        int pf_tile = first_tile, pf_c0 = 0;   // the next chunk to request
        const int dbg = a.debug;
        // diagnostics: bit 1 no residual loads at all, bit 64 none in the second CTA of a pair (wrong results, no waits)
        const bool no_res = (dbg & 1) != 0;
        auto request_residual = [&]() {
            if (pf_tile >= total_tiles || no_res) return;
            const int nt = pf_tile % n_tiles, pt = pixel_tile(pf_tile);
            const int ow0 = (pt % tiles_w) * wt, oh0 = ((pt / tiles_w) % tiles_h) * ht, b0 = (pt / ptiles_wh) * bt;
            const uint32_t rb = pf_count & 3u, bar = smem_u32(&sh->res_full[rb]);
            mbar_expect_tx(bar, 128u * srb);
            tma_load_4d(smem_u32(stage_out + (size_t)rb * 128 * srb), rmap, bar, nt * bn + pf_c0, ow0, oh0, b0);
            ++pf_count;
            pf_c0 += CPC;
            if (pf_c0 >= bn) { pf_c0 = 0; pf_tile += grid_stride; }
        };
        if (res_tiles && store_thread)
            for (int d = 0; d < res_ahead; ++d) request_residual();
        const uint8_t *const res_base = reinterpret_cast<const uint8_t *>(a.ep.residual);
        const size_t res_pix_bytes = (size_t)a.ep.res_cpitch * (OUT_BF16 ? 2 : 4);
        const float *const ep_scale = a.ep.scale, *const ep_shift = a.ep.shift;
        const int n_pad = a.n_pad;
        for (int tile = first_tile; tile < total_tiles; tile += grid_stride, ++it) {
            const int acc = it & 1;
            const uint32_t acc_phase = (it >> 1) & 1;
            const int base = SPLIT ? tile / splits : tile, split = SPLIT ? tile - base * splits : 0;
            const int nt = base % n_tiles, pt = pixel_tile(base);
            const int ow0 = (pt % tiles_w) * wt, oh0 = ((pt / tiles_w) % tiles_h) * ht, b0 = (pt / ptiles_wh) * bt;
            const int ow = ow0 + wl, oh = oh0 + hl, b = b0 + bl;
            const bool pix_ok = ow < g.out_w && oh < g.out_h && b < g.batch;
            if (nt != loaded_nt) {
                if (warp_stores) epilogue_bar();   // no per-chunk barrier in this mode: the other warps may still read the previous tile's vectors
                // this filter tile's epilogue vectors (zero beyond the layer's filters).  Every thread is past the
                // previous tile's last barrier, which follows the last read; the barrier below publishes the writes.
                for (int i = threadIdx.x - 64; i < bn + 64; i += 128) {
                    const int gi = nt * bn + i;
                    const bool in = i < bn && gi < n_pad;
                    s_scale[i] = in ? __ldg(ep_scale + gi) : 0.f;
                    s_shift[i] = in ? __ldg(ep_shift + gi) : 0.f;
                }
                loaded_nt = nt;
            }
            mbar_wait(smem_u32(&sh->acc_full[acc]), acc_phase, abort_flag, status, WAIT_ACC_FULL, 32, wait_limit);
            epilogue_bar();                 // all four warps agree on the abort flag from here
            if (*abort_flag) break;
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + acc * acc_stride;
            // split-K: this pixel's row of every range's partial sums, [range][128 rows][bn columns] per output tile
            // layout [range][group of 4 columns][128 rows][4]: the 32 rows of a warp are 512 contiguous bytes
            const uint4 *split_rows = nullptr;
            if (SPLIT) {
                uint4 *tile_rows = reinterpret_cast<uint4 *>(a.split_scratch) + ((size_t)(pt * n_tiles + nt) * splits) * 32 * bn + m;
                uint4 *mine = tile_rows + (size_t)split * 32 * bn;
#pragma unroll 1
                for (int c0 = 0; c0 < bn; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld16(t_row + c0, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int q = 0; q < 4; ++q) __stcg(mine + (size_t)(c0 / 4 + q) * 128, make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]));
                }
                __threadfence();          // the partial sums are visible device-wide before the counter moves
                epilogue_bar();
                if (store_thread) {
                    int *counter = a.split_counters + (pt * n_tiles + nt);
                    const int last = atomicAdd(counter, 1) == splits - 1;
                    if (last) *counter = 0;   // every range has arrived: ready for the next launch
                    sh->split_last = last;
                }
                epilogue_bar();
                const bool last = *reinterpret_cast<volatile int *>(&sh->split_last) != 0;
                if (!last) {              // another CTA finishes this tile
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if (PAIR) mbar_arrive_leader(smem_u32(&sh->acc_empty[acc])); else mbar_arrive(smem_u32(&sh->acc_empty[acc]));
                    }
                    continue;
                }
                __threadfence();
                split_rows = tile_rows;
            }
            // One staged chunk of CPC columns per iteration: CPC/16 TMEM loads in flight, one wait, the
            // arithmetic, the staged row, the store.  The loop is deliberately NOT unrolled: its body has to
            // stay resident in the instruction cache next to the MMA warp's loop.
            const size_t plane = (size_t)g.out_h * g.out_w;
            constexpr int RES_V = CPC * (OUT_BF16 ? 2 : 4) / 16;      // 16-byte pieces of a staged row
            // direct residual: this pixel's row of the residual tensor, the next chunk's 128 bytes always in flight
            const uint4 *res_row = nullptr;
            uint4 res_next[res_direct ? RES_V : 1];
            if (res_direct) {
                if (pix_ok && !no_res) res_row = reinterpret_cast<const uint4 *>(res_base + (((size_t)b * g.out_h + oh) * g.out_w + ow) * res_pix_bytes + (size_t)nt * bn * (OUT_BF16 ? 2 : 4));
#pragma unroll
                for (int q = 0; q < RES_V; ++q) res_next[q] = res_row ? __ldg(res_row + q) : make_uint4(0u, 0u, 0u, 0u);
            }
#pragma unroll 1
            for (int c0 = (dbg & 8) ? bn : 0; c0 < bn; c0 += CPC) {
                uint32_t r[CPC];
                if (SPLIT) {
                    // the ranges' partial sums, added in their fixed order (bn is a multiple of CPC in this variant); the
                    // next range's loads are in flight while this one is added
                    const uint4 *src = split_rows + (size_t)(c0 / 4) * 128;
                    uint4 v[CPC / 4], w[CPC / 4];
#pragma unroll
                    for (int q = 0; q < CPC / 4; ++q) v[q] = __ldcg(src + (size_t)q * 128);
                    if (splits > 1) {
#pragma unroll
                        for (int q = 0; q < CPC / 4; ++q) w[q] = __ldcg(src + (size_t)32 * bn + (size_t)q * 128);
                    }
#pragma unroll 1
                    for (int sp = 1; sp < splits; ++sp) {
                        uint4 cur[CPC / 4];
#pragma unroll
                        for (int q = 0; q < CPC / 4; ++q) cur[q] = w[q];
                        if (sp + 1 < splits) {
#pragma unroll
                            for (int q = 0; q < CPC / 4; ++q) w[q] = __ldcg(src + (size_t)(sp + 1) * 32 * bn + (size_t)q * 128);
                        }
#pragma unroll
                        for (int q = 0; q < CPC / 4; ++q) {
                            if (I8) { v[q].x += cur[q].x; v[q].y += cur[q].y; v[q].z += cur[q].z; v[q].w += cur[q].w; }
                            else {
                                v[q].x = __float_as_uint(__uint_as_float(v[q].x) + __uint_as_float(cur[q].x));
                                v[q].y = __float_as_uint(__uint_as_float(v[q].y) + __uint_as_float(cur[q].y));
                                v[q].z = __float_as_uint(__uint_as_float(v[q].z) + __uint_as_float(cur[q].z));
                                v[q].w = __float_as_uint(__uint_as_float(v[q].w) + __uint_as_float(cur[q].w));
                            }
                        }
                    }
#pragma unroll
                    for (int q = 0; q < CPC / 4; ++q) { r[4 * q] = v[q].x; r[4 * q + 1] = v[q].y; r[4 * q + 2] = v[q].z; r[4 * q + 3] = v[q].w; }
                } else {
#pragma unroll
                    for (int u = 0; u < CPC / 16; ++u) {
                        if (c0 + 16 * u < bn) {
                            tmem_ld16(t_row + c0 + 16 * u, *reinterpret_cast<uint32_t(*)[16]>(&r[16 * u]));
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j) r[16 * u + j] = 0u;
                        }
                    }
                    tmem_ld_wait();
                }
                uint4 res[RES_V];
                if (res_direct) {
#pragma unroll
                    for (int q = 0; q < RES_V; ++q) res[q] = res_next[q];
                    if (c0 + CPC < bn && res_row) {
                        const uint4 *nx = res_row + (size_t)(c0 + CPC) * (OUT_BF16 ? 2 : 4) / 16;
#pragma unroll
                        for (int q = 0; q < RES_V; ++q) res_next[q] = __ldg(nx + q);
                    }
                }
                if (res_tiles) {
                    // this chunk's residual tile (TMA zero-fills pixels and channels outside the tensor)
                    const uint32_t rb = chunk_count & 3u;
                    if (!no_res) mbar_wait(smem_u32(&sh->res_full[rb]), (chunk_count >> 2) & 1, abort_flag, status, WAIT_RESIDUAL, 0, wait_limit);
                    const uint8_t *rrow = stage_out + (size_t)rb * 128 * srb + (size_t)m * srb;
#pragma unroll
                    for (int q = 0; q < RES_V; ++q) res[q] = *reinterpret_cast<const uint4 *>(rrow + ((q ^ q_xor) << 4));
                }
                // epilogue arithmetic in place: r[] becomes the output values (as float bits); the shared
                // scale / shift copies are zero beyond the layer's filters and padded by 64 entries
                const int nl0 = nt * bn + c0;                 // first filter of this chunk
                const int nvalid = min(bn - c0, g.n - nl0);   // columns of this chunk that are real filters
                int yolo_entry = ACT == ACT_YOLO ? nl0 % yolo_entries : 0;   // entry (x, y, w, h, objectness, classes...) of the chunk's first column
                const float4 *sc4 = reinterpret_cast<const float4 *>(s_scale + c0);
                const float4 *sf4 = reinterpret_cast<const float4 *>(s_shift + c0);
#pragma unroll
                for (int q = 0; q < CPC / 4; ++q) {
                    const float4 sc = sc4[q], sf = sf4[q];
                    const float scv[4] = {sc.x, sc.y, sc.z, sc.w}, sfv[4] = {sf.x, sf.y, sf.z, sf.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int j = 4 * q + e;
                        const float accv = I8 ? (float)(int)r[j] : __uint_as_float(r[j]);   // int32 sums of an xnor layer are exact in f32 (below 2^24)
                        float t = act_apply<ACT>(fmaf(accv, scv[e], sfv[e]), runtime_act);
                        if (ACT == ACT_YOLO) {
                            // forward_yolo_layer_gpu's activations (src/yolo_layer.c:351-357): logistic on x, y, objectness, classes.
                            // The entry index is the same for the whole warp (it depends on the column only); the epilogue has
                            // four warps to hide its latencies with, so the fast exponential and division are used (2 ulp).
                            if (yolo_entry < 2 || yolo_entry >= 4) t = __fdividef(1.f, 1.f + __expf(-t));
                            if (++yolo_entry == yolo_entries) yolo_entry = 0;
                        }
                        if (residual) {
                            float rv = 0.f;
                            {
                                if (!OUT_BF16) {
                                    const uint4 v4 = res[j / 4];
                                    rv = __uint_as_float((j & 3) == 0 ? v4.x : (j & 3) == 1 ? v4.y : (j & 3) == 2 ? v4.z : v4.w);
                                } else {
                                    const uint4 v4 = res[j / 8];
                                    const uint32_t wd = ((j >> 1) & 3) == 0 ? v4.x : ((j >> 1) & 3) == 1 ? v4.y : ((j >> 1) & 3) == 2 ? v4.z : v4.w;
                                    rv = __uint_as_float((j & 1) ? (wd & 0xffff0000u) : (wd << 16));
                                }
                            }
                            t = act_apply<ACT2>(res_alpha * t + res_beta * rv, act2);
                        }
                        if (!OUT_BF16 && do_round) t = round_tf32(t);
                        // columns beyond the layer's filters: scale, shift, weights and residual are all zero there, so
                        // linear and leaky epilogues produce the zero by themselves; others need the mask
                        constexpr bool self_zero = (ACT == DNB_LINEAR || ACT == DNB_LEAKY) &&
                                                   (ACT2 == ACT2_NONE || ACT2 == DNB_LINEAR || ACT2 == DNB_LEAKY);
                        if (!(I8 && raw_acc)) r[j] = __float_as_uint((self_zero || j < nvalid) ? t : 0.f);   // raw: the integer sums themselves
                    }
                }
                const uint32_t buf = chunk_count & buf_mask;
                if (!res_tiles) {
                    if (warp_stores) {
                        if (lane == 0 && chunk_count >= 2) tma_store_wait_read1();   // this warp's store that last read its rows of the buffer is done
                        __syncwarp();
                    } else {
                        if (store_thread && chunk_count >= 2) tma_store_wait_read1();   // the store that last read this buffer is done
                        epilogue_bar();
                    }
                }   // with a residual the buffer is this thread's to overwrite: its tile landed after that store, and
                    // a thread reads and writes its own row only
                uint8_t *row = stage_out + (size_t)buf * 128 * srb + (size_t)m * srb;
                if (!out_bf16) {
#pragma unroll
                    for (int q = 0; q < srb / 16; ++q)         // 16-byte pieces of 4 floats
                        *reinterpret_cast<uint4 *>(row + ((q ^ q_xor) << 4)) = make_uint4(r[4 * q], r[4 * q + 1], r[4 * q + 2], r[4 * q + 3]);
                } else {
#pragma unroll
                    for (int q = 0; q < srb / 16; ++q) {       // 16-byte pieces of 8 bf16
                        const int j = 8 * q;
                        uint4 pk;
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
                        __nv_bfloat162 h1 = __floats2bfloat162_rn(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
                        __nv_bfloat162 h3 = __floats2bfloat162_rn(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
                        pk.x = *reinterpret_cast<uint32_t *>(&h0); pk.y = *reinterpret_cast<uint32_t *>(&h1);
                        pk.z = *reinterpret_cast<uint32_t *>(&h2); pk.w = *reinterpret_cast<uint32_t *>(&h3);
                        *reinterpret_cast<uint4 *>(row + ((q ^ q_xor) << 4)) = pk;
                    }
                }
                if (SIGNS) {
                    // 32 signs of this pixel = one 32-byte row of a 32-byte-swizzled box: its two 16-byte halves swap on rows 4..7 of every 8
                    uint32_t sw[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        uint32_t wd = 0u;
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const int j = 4 * q + e;
                            const uint32_t sgn = j < nvalid ? (__uint_as_float(r[j]) > 0.f ? 0x01u : 0xFFu) : 0u;
                            wd |= sgn << (8 * e);
                        }
                        sw[q] = wd;
                    }
                    uint8_t *srow = stage_out + (size_t)2 * 128 * srb + (size_t)(chunk_count & 1u) * 128 * 32 + (size_t)m * 32;
                    const int sx = (m >> 2) & 1;
                    *reinterpret_cast<uint4 *>(srow + ((0 ^ sx) << 4)) = make_uint4(sw[0], sw[1], sw[2], sw[3]);
                    *reinterpret_cast<uint4 *>(srow + ((1 ^ sx) << 4)) = make_uint4(sw[4], sw[5], sw[6], sw[7]);
                }
                fence_async_smem();            // staged rows visible to the TMA unit
                if (warp_stores) {
                    __syncwarp();
                    if (lane == 0) {
                        if (!(dbg & 2) && (!PAIR || b0 < g.batch))
                            tma_store_4d(&a.tmy_warp, smem_u32(stage_out + (size_t)buf * 128 * srb + (size_t)m0 * srb), nl0, ow0 + wl0, oh0 + hl0, b0 + bl0);
                        tma_store_commit();
                    }
                } else
                epilogue_bar();
                if (!warp_stores && store_thread) {
                    // the TMA unit clips the box at the tensor's extents: ragged tiles need no predicates
                    if (y_nhwc && !(dbg & 2) && (!PAIR || b0 < g.batch)) tma_store_4d(ymap, smem_u32(stage_out + (size_t)buf * 128 * srb), nl0, ow0, oh0, b0);
                    if (SIGNS && (!PAIR || b0 < g.batch))
                        tma_store_4d(&a.tms, smem_u32(stage_out + (size_t)2 * 128 * srb + (size_t)(chunk_count & 1u) * 128 * 32), nl0, ow0, oh0, b0);
                    tma_store_commit();
                    if (res_tiles) {
                        // the tile three chunks on goes into the buffer of the previous chunk, once that chunk's
                        // store has read it (only the store just issued may still be pending)
                        if (!(dbg & 4)) tma_store_wait_read1();
                        request_residual();
                    }
                }
                if (y_nchw && pix_ok) {
                    // Darknet-layout copy: this thread's pixel, one filter plane per column, straight from the registers
                    // (a warp's 32 pixels are wt-long runs of each plane).  BF16 plans write what the channels-last
                    // copy holds: the value rounded to bf16.
                    float *dst = y_nchw + ((size_t)b * g.n + nl0) * plane + (size_t)oh * g.out_w + ow;
                    const int cols = min(CPC, g.n - nl0);
#pragma unroll
                    for (int j = 0; j < CPC; ++j) {
                        if (j < cols) {
                            float v = __uint_as_float(r[j]);
                            if (out_bf16) v = __bfloat162float(__float2bfloat16_rn(v));
                            dst[(size_t)j * plane] = v;
                        }
                    }
                }
                ++chunk_count;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {   // a pair's accumulator is free when the epilogues of both CTAs have drained their rows
                if (PAIR) mbar_arrive_leader(smem_u32(&sh->acc_empty[acc])); else mbar_arrive(smem_u32(&sh->acc_empty[acc]));
            }
        }
        if (warp_stores ? lane == 0 : store_thread) tma_store_wait_all();
    }

    // ---------------- teardown (also the abort path)
    if (*abort_flag) {   // give loads that are still in flight time to land before shared memory is released
        const long long t0 = clock64();
        while (clock64() - t0 < 4000000LL) { }
    }
    tc_fence_before();
    __syncthreads();
    // A pair leaves together: neither CTA may exit, or free TMEM, while the other can still signal its barriers or
    // run MMAs into its TMEM.  Every wait above is bounded, so both CTAs get here.
    if (PAIR) cluster_sync_all();
    if (warp == 1) {
        tc_fence_after();
        if (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(tmem_cols) : "memory");
    }
    if (PAIR) cluster_sync_all();
}

// ------------------------------------------------------------------ host side
size_t conv_tc_fixed_smem(int store_row_bytes, int bn, int stage_bufs)
{
    return stage_bufs * 128 * (size_t)store_row_bytes + 2 * sizeof(float) * ((size_t)bn + 64) + sizeof(TcShared) + 16;
}

size_t conv_tc_smem_bytes(const TcArgs &a)
{
    if (a.halo) return (size_t)a.a_stages * a.a_slot + (size_t)a.b_stages * a.b_bytes + conv_tc_fixed_smem(a.store_row_bytes, a.bn, a.stage_bufs);
    return (size_t)a.stages * (a.a_bytes + a.b_bytes) + conv_tc_fixed_smem(a.store_row_bytes, a.bn, a.stage_bufs);
}

int conv_tc_max_smem()
{
    int dev = 0, v = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess) return 0;
    return v;
}

// Resident clusters of two CTAs of a pair-mode kernel with `smem` bytes of dynamic shared memory (cached per kernel).
template <typename K>
static int max_pair_clusters(K kernel, size_t smem)
{
    static int cached = 0;
    static size_t cached_smem = 0;
    if (cached && cached_smem == smem) return cached;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * (unsigned)(sm_count() / 2));
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = sm_count() / 2; }
    cached = n; cached_smem = smem;
    return n;
}

// DNB_PDL=0 launches every kernel plainly (no overlap of a kernel's set-up with the tail of the kernel before it).
static bool pdl_enabled()
{
    static int v = -1;
    if (v < 0) { const char *e = getenv("DNB_PDL"); v = e ? (atoi(e) != 0) : 1; }
    return v != 0;
}

// One launch.  Single CTAs: one CTA per SM slot (or per tile, if fewer).  Pair mode: clusters of two CTAs, as many as are
// resident at once (or pair tiles, if fewer).  Either way the grid is one wave of persistent CTAs.  Every launch carries
// the programmatic-stream-serialization attribute: the kernel's set-up overlaps the tail of the kernel before it in the
// stream, and the kernel itself waits for that kernel before it touches global memory.
template <typename K>
static int launch_one(K kern, const TcArgs &a, size_t smem, cudaStream_t s)
{
    // the opt-in for large dynamic shared memory is per kernel symbol and cheap, so it is set on every launch
    DNB_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, conv_tc_max_smem()));
    unsigned grid;
    if (a.pair) {
        const int clusters_max = max_pair_clusters(kern, smem);
        grid = 2u * (unsigned)(a.total_tiles < clusters_max ? a.total_tiles : clusters_max);
    } else {
        const int slots = sm_count() * a.ctas_per_sm;
        grid = (unsigned)(a.total_tiles < slots ? a.total_tiles : slots);
    }
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    attrs[1].id = cudaLaunchAttributeClusterDimension;
    attrs[1].val.clusterDim.x = 2; attrs[1].val.clusterDim.y = 1; attrs[1].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(TC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cfg.attrs = attrs;
    cfg.numAttrs = a.pair ? 2 : 1;
    DNB_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
    return DNB_OK;
}

int launch_conv_tc(const TcArgs &a, cudaStream_t s)
{
    const size_t smem = conv_tc_smem_bytes(a);
    const bool obf = a.is_bf16 == 1, i8 = a.is_bf16 == 2;   // int8 operands write f32 output
    const int cpc = a.store_row_bytes / (obf ? 2 : 4);
    if (cpc != 16 && cpc != 32 && cpc != 64) DNB_FAIL(DNB_EINVAL, "conv_tc: staged row of %d bytes", a.store_row_bytes);
    if (a.pair && !((!obf && cpc == 32) || (obf && cpc == 64))) DNB_FAIL(DNB_EINVAL, "conv_tc: pair mode needs 128-byte staged rows");
    if (a.splits > 1 && (!((!obf && cpc == 32) || (obf && cpc == 64)) || a.bn % cpc || a.halo || !a.split_scratch || !a.split_counters))
        DNB_FAIL(DNB_EINVAL, "conv_tc: split-K needs 128-byte staged rows, whole chunks per tile, no halo mode, and its scratch");
    // one instantiation per (activation, columns per staged chunk, output type, fused shortcut, pair mode, operand kind)
    // split-K variants exist for 128-byte staged rows, f32 / bf16 operands; with a fused residual only as pairs (the
    // single-CTA kernel streams residual tiles ahead of the epilogue, which a tile finished elsewhere would derail)
#define DNB_TC_GO(ACT, CPC, OBF, ACT2, I8)                                                          \
    do {                                                                                            \
        if (a.splits > 1) {                                                                         \
            if (I8) DNB_FAIL(DNB_EINVAL, "conv_tc: no split-K variant of the int8 kind");            \
            if (a.pair) DNB_TRY(launch_one(conv_tc_kernel<ACT, CPC, OBF, ACT2, true, false, !I8>, a, smem, s)); \
            else if (ACT2 != ACT2_NONE) DNB_FAIL(DNB_EINVAL, "conv_tc: split-K with a fused residual runs as CTA pairs only"); \
            else DNB_TRY(launch_one(conv_tc_kernel<ACT, CPC, OBF, ACT2_NONE, false, false, !I8>, a, smem, s)); \
        } else if (a.pair) DNB_TRY(launch_one(conv_tc_kernel<ACT, CPC, OBF, ACT2, true, I8>, a, smem, s)); \
        else DNB_TRY(launch_one(conv_tc_kernel<ACT, CPC, OBF, ACT2, false, I8>, a, smem, s));       \
    } while (0)
    // pair-mode kernels exist for 128-byte staged rows only, so the narrower variants are instantiated without it
#define DNB_TC_GO_SINGLE(ACT, CPC, OBF, ACT2, I8)                                                   \
    do {                                                                                            \
        if (a.splits > 1) DNB_FAIL(DNB_EINVAL, "conv_tc: no split-K variant for this staged row width"); \
        DNB_TRY(launch_one(conv_tc_kernel<ACT, CPC, OBF, ACT2, false, I8>, a, smem, s));            \
    } while (0)
#define DNB_TC_LAUNCH_ACT(ACT, ACT2)                                            \
    do {                                                                        \
        if (!obf && cpc == 32) DNB_TC_GO(ACT, 32, false, ACT2, false);          \
        else if (!obf && cpc == 16) DNB_TC_GO_SINGLE(ACT, 16, false, ACT2, false); \
        else if (obf && cpc == 64) DNB_TC_GO(ACT, 64, true, ACT2, false);       \
        else if (obf && cpc == 32) DNB_TC_GO_SINGLE(ACT, 32, true, ACT2, false); \
        else if (obf && cpc == 16) DNB_TC_GO_SINGLE(ACT, 16, true, ACT2, false); \
        else DNB_FAIL(DNB_EINVAL, "conv_tc: no kernel for %d columns per chunk", cpc); \
    } while (0)
    // (a yolo head's filters are anchors * (classes + 5), never whole tiles of 256: no pair variant)
#define DNB_TC_LAUNCH_ACT_SINGLE(ACT, ACT2)                                     \
    do {                                                                        \
        if (a.pair) DNB_FAIL(DNB_EINVAL, "conv_tc: no pair variant of this epilogue"); \
        if (!obf && cpc == 32) DNB_TC_GO_SINGLE(ACT, 32, false, ACT2, false);   \
        else if (!obf && cpc == 16) DNB_TC_GO_SINGLE(ACT, 16, false, ACT2, false); \
        else if (obf && cpc == 64) DNB_TC_GO_SINGLE(ACT, 64, true, ACT2, false); \
        else if (obf && cpc == 32) DNB_TC_GO_SINGLE(ACT, 32, true, ACT2, false); \
        else if (obf && cpc == 16) DNB_TC_GO_SINGLE(ACT, 16, true, ACT2, false); \
        else DNB_FAIL(DNB_EINVAL, "conv_tc: no kernel for %d columns per chunk", cpc); \
    } while (0)
#define DNB_TC_LAUNCH_I8_ACT(ACT)                                               \
    do {                                                                        \
        if (a.sign_out) {                                                       \
            if (cpc != 32 || a.stage_bufs != 3 || a.splits > 1 || a.ep.raw_acc) DNB_FAIL(DNB_EINVAL, "conv_tc: the sign output needs 128-byte staged rows and a third staging buffer"); \
            if (a.pair) DNB_TRY(launch_one(conv_tc_kernel<ACT, 32, false, ACT2_NONE, true, true, false, true>, a, smem, s)); \
            else DNB_TRY(launch_one(conv_tc_kernel<ACT, 32, false, ACT2_NONE, false, true, false, true>, a, smem, s)); \
        } else                                                                  \
        if (cpc == 32) DNB_TC_GO(ACT, 32, false, ACT2_NONE, true);              \
        else if (cpc == 16) DNB_TC_GO_SINGLE(ACT, 16, false, ACT2_NONE, true);  \
        else DNB_FAIL(DNB_EINVAL, "conv_tc: no int8 kernel for %d columns per chunk", cpc); \
    } while (0)
    if (i8) {
        if (a.ep.residual || a.ep.yolo_entries) DNB_FAIL(DNB_EUNSUPPORTED, "conv_tc: the int8 (xnor) kernel fuses neither a residual nor a yolo head");
        switch (a.ep.activation) {
        case DNB_LINEAR: DNB_TC_LAUNCH_I8_ACT(DNB_LINEAR); break;
        case DNB_LEAKY: DNB_TC_LAUNCH_I8_ACT(DNB_LEAKY); break;
        default: DNB_TC_LAUNCH_I8_ACT(ACT_GENERIC); break;
        }
    } else if (!a.ep.residual) {
        if (a.ep.yolo_entries > 0 && a.ep.activation != DNB_LINEAR) DNB_FAIL(DNB_EUNSUPPORTED, "conv_tc: a fused yolo head follows a linear convolution");
        switch (a.ep.yolo_entries > 0 ? (int)ACT_YOLO : a.ep.activation) {
        case DNB_LINEAR: DNB_TC_LAUNCH_ACT(DNB_LINEAR, ACT2_NONE); break;
        case DNB_LEAKY: DNB_TC_LAUNCH_ACT(DNB_LEAKY, ACT2_NONE); break;
        case ACT_YOLO: DNB_TC_LAUNCH_ACT_SINGLE(ACT_YOLO, ACT2_NONE); break;
        default: DNB_TC_LAUNCH_ACT(ACT_GENERIC, ACT2_NONE); break;
        }
    } else {
        // fused shortcut: the two pairs the reference's cfgs use (yolov3: leaky conv, linear shortcut; resnet:
        // linear conv, leaky shortcut) are compile-time, every other pair takes the run-time switches
        if (a.ep.yolo_entries) DNB_FAIL(DNB_EUNSUPPORTED, "conv_tc: a residual and a yolo head in one launch");
        if (a.stage_bufs != (a.pair ? 2 : 4)) DNB_FAIL(DNB_EINVAL, "conv_tc: a fused residual needs four staging buffers (two in pair mode)");
        if (a.ep.activation == DNB_LEAKY && a.ep.activation2 == DNB_LINEAR) DNB_TC_LAUNCH_ACT(DNB_LEAKY, DNB_LINEAR);
        else if (a.ep.activation == DNB_LINEAR && a.ep.activation2 == DNB_LEAKY) DNB_TC_LAUNCH_ACT(DNB_LINEAR, DNB_LEAKY);
        else DNB_TC_LAUNCH_ACT(ACT_GENERIC, ACT_GENERIC);
    }
#undef DNB_TC_LAUNCH_I8_ACT
#undef DNB_TC_LAUNCH_ACT_SINGLE
#undef DNB_TC_LAUNCH_ACT
#undef DNB_TC_GO_SINGLE
#undef DNB_TC_GO
    DNB_LAUNCH_CHECK("conv_tc");
    return DNB_OK;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

int encode_tensor_map(CUtensorMap *map, int elem_kind, int rank, void *base, const uint64_t *dims,
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
    const CUtensorMapDataType dt = elem_kind == 1 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : (elem_kind == 2 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32);
    CUresult r = fn(map, dt, (cuuint32_t)rank, base,
                    d, st, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        DNB_FAIL(DNB_ECUDA, "cuTensorMapEncodeTiled failed with %d (rank %d, dims %llu %llu %llu, box %u %u %u, swizzle %d)", (int)r, rank,
                 (unsigned long long)d[0], (unsigned long long)d[1], (unsigned long long)(rank > 2 ? d[2] : 0), bx[0], bx[1], rank > 2 ? bx[2] : 0, swizzle_bytes);
    return DNB_OK;
}

}  // namespace dnb
