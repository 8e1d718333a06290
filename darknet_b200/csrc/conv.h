// Internal argument blocks of the convolution kernels and the plan object.
#pragma once
#include <cuda.h>

#include <vector>

#include "common.h"

namespace dnb {

// Default bound of the kernels' device-side waits: about one second of SM clock cycles.
constexpr long long DEFAULT_WAIT_CYCLES = 2000000000LL;

// ---- conv_direct.cu
struct DirectArgs {
    const void *x;                       // input, any layout through element strides
    int x_dtype;
    long long xs_b, xs_c, xs_h, xs_w;    // element strides of x
    const float *wpk;                    // weights [groups][K][npg_pad], K = c/groups*size*size
    int npg_pad;                         // filters per group rounded up to 32
    void *y_nhwc;                        // optional NHWC output
    int y_dtype, y_cpitch;
    float *y_nchw;                       // optional NCHW f32 output
    ConvGeom g;
    ConvEpilogue ep;
};
int launch_conv_direct(const DirectArgs &a, cudaStream_t s);

// ---- conv_stem_tc.cu : first layer (3x3, at most 3 input channels) on tcgen05, im2col rows built by the threads
struct alignas(64) StemTcArgs {
    CUtensorMap tmy;                     // channels-last output as [pixel][channel], 32-row boxes
    int tma_store;                       // rows leave through tmy (else plain stores)
    const float *x;                      // f32 input, any layout through element strides
    long long xs_b, xs_c, xs_h, xs_w;
    const float *w;                      // weights [K][npg_pad], K = c*9 (the direct kernel's packing)
    int npg_pad;
    void *y;                             // channels-last output, pitch == n
    int y_dtype, y_cpitch;
    int n_pad, tmem_cols, tiles, npix;   // filled by the launcher
    int *status;
    long long wait_limit;                // bound of every device-side wait, SM clock cycles
    ConvGeom g;
    ConvEpilogue ep;
};
bool conv_stem_tc_covers(const ConvGeom &g);
int launch_conv_stem_tc(StemTcArgs a, cudaStream_t s);

// ---- conv_tc.cu : implicit GEMM on tcgen05 / TMEM, operands by TMA
struct alignas(64) TcArgs {
    CUtensorMap tmx[4];   // activation maps: one per (row parity, column parity) lattice of a strided conv
    CUtensorMap tmw;      // weights [taps][n_pad][c_pad], channels innermost
    CUtensorMap tmy;      // NHWC output, written by TMA stores from the staging rows
    CUtensorMap tmr;      // fused residual (same extents and box as tmy), loaded tile by tile in the epilogue
    CUtensorMap tmy_warp; // the same output as 32-pixel boxes: the rows one epilogue warp stages (per-warp stores)
    CUtensorMap tms;      // sign output (int8 channels-last, the next xnor layer's operand): 32-channel boxes of the same pixels as tmy
    int is_bf16;          // operand kind: 0 kind::tf32 on f32 operands, 1 kind::f16 on bf16 operands, 2 kind::i8 on int8 sign tensors (xnor)
    int row_bytes;        // bytes of channels per pipeline stage row: 128, 64 or 32 (= swizzle span)
    int bk;               // channels per stage row (row_bytes / element size)
    int c_blocks;         // ceil(c_pad / bk)
    int taps;             // size*size
    int bn;               // filters per tile: multiple of 16, <= 256
    int n_tiles;          // ceil(n / bn)
    int wt, ht, bt;       // output pixels per tile along w, h, batch; wt*ht*bt == 128
    int tiles_w, tiles_h, tiles_b;
    int total_tiles;      // n_tiles * tiles_w * tiles_h * tiles_b
    int stages;           // depth of the shared-memory ring
    // Halo mode (3x3, stride 1, tiles of 8 x 16 pixels): ONE activation box of (8+2) x (16+2) pixels per channel
    // block serves all nine taps (the MMA's A descriptor starts at row kh*10 + kw of the box, its 8-row groups are
    // 10 rows apart), so activations cross L2 -> shared memory once instead of nine times.  Activations and
    // weights then travel in two rings: a_stages boxes of a_slot bytes, b_stages weight tiles of b_bytes.
    int halo, a_stages, b_stages, a_slot, a_box_bytes, a_pitch;
    int tmem_cols;        // TMEM columns the CTA allocates: a power of two >= 2*bn (two accumulators)
    int debug;            // timing experiments only (DNB_TC_DEBUG): 1 no residual loads, 2 no output stores, 4 no wait before a residual request, 8 empty epilogue, 16 no MMAs;
                          // 32 (dnb_conv_plan_set_diagnostics): each CTA withholds the last operand load of its first tile, so a bounded wait runs out
    long long wait_limit; // bound of every device-side wait, SM clock cycles
    int stage_bufs;       // staging buffers of the epilogue: 2, or 4 with a fused residual (tiles land in them first)
    int pair;             // 1: clusters of two CTAs share every MMA (cta_group::2); total_tiles then counts PAIRS of pixel tiles,
                          // b_bytes and the weight map's box cover half a filter tile, bn is 256
    int ctas_per_sm;      // 2 for narrow tiles (TMEM and shared memory are sized so that two CTAs share an SM), else 1
    int a_bytes, b_bytes; // shared-memory bytes of one stage's activation / weight tile (1024-multiples)
    int store_row_bytes;  // bytes of one staged output row (128, 64 or 32) = swizzle span of tmy
    int n_pad;            // length of the scale / shift vectors
    int n_tot;            // n_tiles * bn rounded up: entries of the shared scale / shift copies
    void *y_nhwc;
    int y_dtype, y_cpitch;
    float *y_nchw;
    int *status;          // device word: 0, or the code of the wait that expired
    // split-K (layers with fewer tiles than SMs and a long K loop): total_tiles counts (output tile, K range) pairs
    int warp_stores;      // 1: every epilogue warp stores its own 32 rows (tmy_warp); 0: one store per chunk by one thread (tmy)
    void *sign_out;       // int8 kind: also write the output's signs here ([b][h][w][sign_cpitch] bytes), or null
    int sign_cpitch;
    int splits;           // K ranges per output tile; 1 = off
    void *split_scratch;  // [output tile][range][128 rows][bn] raw accumulators (f32, or int32 of the int8 kind)
    int *split_counters;  // [output tile] ranges delivered so far; zero between launches
    ConvGeom g;
    ConvEpilogue ep;
};
int launch_conv_tc(const TcArgs &a, cudaStream_t s);
size_t conv_tc_smem_bytes(const TcArgs &a);
size_t conv_tc_fixed_smem(int store_row_bytes, int bn, int stage_bufs);
int conv_tc_max_smem();

// cuTensorMapEncodeTiled through the runtime's driver entry point (no libcuda link).
int encode_tensor_map(CUtensorMap *map, int elem_kind /* 0 f32, 1 bf16, 2 bytes */, int rank, void *base, const uint64_t *dims,
                      const uint64_t *strides_bytes /* rank-1 */, const uint32_t *box, int swizzle_bytes);

// ---- conv_xnor.cu : bit-packed popcount GEMM
struct XnorArgs {
    const uint32_t *xbits;   // [b][h][w][cwords] sign bits of the input (1 = x > 0)
    const uint32_t *wbits;   // [n][taps][cwords] sign bits of the weights (1 = w > 0)
    int cwords;              // ceil(c / 32); unused high bits are 0 in both operands
    const float *wmean;      // [n] mean |w| per filter
    int32_t *acc_out;        // optional NCHW int32 accumulators
    void *y_nhwc;
    int y_dtype, y_cpitch;
    float *y_nchw;
    ConvGeom g;
    ConvEpilogue ep;
};
int launch_conv_xnor(const XnorArgs &a, cudaStream_t s);
// sign bits of an NHWC (f32/bf16) or NCHW f32 tensor into [b][h][w][cwords]
int launch_pack_sign_bits(const dnb_tensor *x, uint32_t *bits, int cwords, cudaStream_t s);
// signs of the same tensors as int8 (+1 where x > 0, else -1; 0 in the padding channels) into [b][h][w][cpad], cpad a
// multiple of 32: the operand of the tensor-core xnor convolution
int launch_pack_sign_i8(const dnb_tensor *x, int8_t *out, int cpad, cudaStream_t s);

}  // namespace dnb

// The plan object behind the C ABI.
struct dnb_conv_plan {
    dnb_conv_desc d;
    int mode;
    int kernel;              // 0 tc_tf32, 1 tc_bf16, 2 direct_fp32, 3 xnor_popc
    dnb::ConvGeom g;
    int n_pad;               // filters rounded up to 16
    int c_pad;               // input channels rounded up to 8 (cpitch the kernel expects of NHWC input)
    bool params_set;
    bool stem_tc;            // a direct plan whose channels-last f32-input launches use the tensor-core first-layer kernel
    // derived device tensors
    float *scale, *shift;    // [n_pad] folded batchnorm / bias
    void *w_tc;              // [taps][n_pad][c_pad] f32 (TF32-rounded) or bf16
    float *w_direct;         // [groups][K][npg_pad]
    uint32_t *w_bits;        // [n][taps][cwords]
    float *w_mean;           // [n]
    int npg_pad, cwords;
    // scratch owned by the plan
    void *x_nhwc_scratch;    // NHWC copy of an NCHW input handed to a tensor-core plan
    size_t x_nhwc_bytes;
    uint32_t *x_bits;        // packed input of an xnor plan
    size_t x_bits_bytes;
    // xnor on the tensor cores (kind::i8): int8 sign tensors instead of packed bits
    bool xnor_tc;            // this xnor plan runs the tensor-core kernel (DNB_XNOR_TC=0 keeps the popcount kernel)
    int c_pad_i8;            // input channels rounded up to 32
    int8_t *w_i8;            // [taps][n_pad][c_pad_i8] signs of the weights
    float *scale_i8;         // [n_pad] mean|w| * folded batchnorm scale
    int8_t *x_i8;            // int8 signs of the input, scratch
    size_t x_i8_bytes;
    int *status;             // device status word of the tensor-core kernel
    bool status_shared;      // the word belongs to a network object (one word for all its plans)
    // tensor-core launch block, rebuilt when the input pointer changes
    dnb::TcArgs tc;
    const void *tc_x_ptr;
    int tc_x_cpitch;
    const void *tc_y_ptr;    // NHWC output the store map was built for
    const void *tc_res_ptr;  // fused residual the load map was built for (NULL: none)
    int tc_res_cpitch;
    int tc_y_cpitch, tc_y_dtype;
    // xnor layers in a row (tensor-core kind): the producer's epilogue writes the consumer's int8 operand
    dnb_conv_plan *sign_consumer;   // this plan also fills that plan's x_i8 (set by the network object), or null
    bool signs_given;               // this plan's x_i8 is filled by the layer before it: no sign pass of its own
    const void *signs_of;           // ... as long as the input it is given is this tensor
    void *tc_sign_out;              // the sign output the cached launch block was built for
    void *split_scratch;     // split-K partial sums and counters of the cached launch block (owned by the plan)
    size_t split_scratch_bytes;
    int *split_counters;
    int split_counters_n;
    int tc_nchw_out;         // the cached launch block was built for a launch that also writes Darknet's layout
    int device;
    long long wait_limit;    // bound of the kernels' waits in cycles (0: the default, about one second)
    int debug_bits;          // OR-ed into the launch block's debug field (dnb_conv_plan_set_diagnostics)
};

// zero the split-K counters a timed-out launch may have left part-way (on `s`; a null plan or one without counters: nothing)
void conv_plan_reset_after_abort(dnb_conv_plan *p, cudaStream_t s = nullptr);

// producers of a tensor-core xnor layer's int8 operand (see conv_plan.cu)
int8_t *conv_plan_expect_signs(dnb_conv_plan *consumer, const void *tensor, int batch, int c, int h, int w);
bool conv_plan_link_signs(dnb_conv_plan *producer, dnb_conv_plan *consumer, const void *tensor);
