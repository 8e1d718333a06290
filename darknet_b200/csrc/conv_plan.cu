// Convolution plans: geometry checks, kernel choice, derived parameter tensors
// (folded batchnorm, repacked / rounded / bit-packed weights) and the forward
// dispatch behind dnb_conv_*.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include <vector>

#include <cuda_bf16.h>

#include "common.h"
#include "conv.h"

using namespace dnb;

enum { K_TC_TF32 = 0, K_TC_BF16 = 1, K_DIRECT = 2, K_XNOR = 3 };
static const char *const kKernelNames[] = {"tc_tf32", "tc_bf16", "direct_fp32", "xnor_popc"};
static const char kXnorTcName[] = "xnor_tc";

extern "C" int dnb_conv_plan_create(const dnb_conv_desc *d, int mode, dnb_conv_plan **out)
{
    if (!d || !out) DNB_FAIL(DNB_EINVAL, "conv plan: null argument");
    *out = nullptr;
    if (mode != DNB_MODE_TF32 && mode != DNB_MODE_BF16 && mode != DNB_MODE_FP32) DNB_FAIL(DNB_EINVAL, "conv plan: mode %d", mode);
    if (d->batch < 1 || d->h < 1 || d->w < 1 || d->c < 1 || d->n < 1 || d->size < 1 || d->stride < 1 || d->pad < 0 || d->groups < 1)
        DNB_FAIL(DNB_EINVAL, "conv plan: non-positive geometry (batch %d, %dx%dx%d, n %d, size %d, stride %d, pad %d, groups %d)",
                 d->batch, d->c, d->h, d->w, d->n, d->size, d->stride, d->pad, d->groups);
    if (d->c % d->groups || d->n % d->groups) DNB_FAIL(DNB_EINVAL, "conv plan: groups %d does not divide c %d and n %d", d->groups, d->c, d->n);
    if (d->activation < 0 || d->activation > DNB_SELU) DNB_FAIL(DNB_EINVAL, "conv plan: activation %d", d->activation);
    if (d->size > 15) DNB_FAIL(DNB_EUNSUPPORTED, "conv plan: kernel size %d > 15", d->size);
    const int out_h = (d->h + 2 * d->pad - d->size) / d->stride + 1;
    const int out_w = (d->w + 2 * d->pad - d->size) / d->stride + 1;
    if (out_h < 1 || out_w < 1) DNB_FAIL(DNB_EINVAL, "conv plan: empty output (%dx%d)", out_w, out_h);
    if (d->size == 1 && (d->stride != 1 || d->pad != 0))
        DNB_FAIL(DNB_EUNSUPPORTED, "conv plan: 1x1 kernel with stride %d / pad %d: the reference's CPU path skips im2col for size 1 and "
                 "multiplies the unstrided image (src/convolutional_layer.c:468-470), so its result is not a convolution; not reproduced", d->stride, d->pad);
    if (d->xnor && d->groups != 1) DNB_FAIL(DNB_EUNSUPPORTED, "conv plan: xnor with groups %d", d->groups);

    dnb_conv_plan *p = new dnb_conv_plan();
    memset(p, 0, sizeof(*p));
    p->d = *d;
    p->mode = mode;
    p->g = ConvGeom{d->batch, d->h, d->w, d->c, d->n, d->groups, d->size, d->stride, d->pad, out_h, out_w};
    p->n_pad = round_up(d->n, 16);
    p->c_pad = round_up(d->c, 8);
    p->npg_pad = round_up(d->n / d->groups, 32);
    p->cwords = (d->c + 31) / 32;
    p->c_pad_i8 = round_up(d->c, 32);
    if (d->xnor) p->kernel = K_XNOR;
    else if (mode == DNB_MODE_FP32 || d->groups != 1 || d->c < 8) p->kernel = K_DIRECT;
    else p->kernel = mode == DNB_MODE_BF16 ? K_TC_BF16 : K_TC_TF32;
    // the tensor-core kernel reads strided inputs through stride*stride lattices and carries maps for strides 1
    // and 2 only; wider strides (none in the benchmark networks) run on the CUDA-core kernel
    if ((p->kernel == K_TC_TF32 || p->kernel == K_TC_BF16) && d->stride > 2) p->kernel = K_DIRECT;
    // RGB first layers of the TF32 / BF16 modes: tensor cores with thread-built im2col rows (DNB_STEM_TC=0 keeps the FP32 kernel)
    const char *stem_env = getenv("DNB_STEM_TC");
    p->stem_tc = p->kernel == K_DIRECT && mode != DNB_MODE_FP32 && !d->xnor && conv_stem_tc_covers(p->g) && !(stem_env && atoi(stem_env) == 0);
    // xnor layers: int8 sign tensors through the tensor cores (kind::i8, exact int32 sums) unless DNB_XNOR_TC=0 asks
    // for the bit-packed popcount kernel; strides above 2 have no lattice maps and stay with the popcount kernel
    {
        const char *e = getenv("DNB_XNOR_TC");
        p->xnor_tc = p->kernel == K_XNOR && d->stride <= 2 && !(e && atoi(e) == 0);
    }
    cudaGetDevice(&p->device);
    *out = p;
    return DNB_OK;
}

extern "C" void dnb_conv_plan_destroy(dnb_conv_plan *p)
{
    if (!p) return;
    cudaFree(p->scale); cudaFree(p->shift); cudaFree(p->w_tc); cudaFree(p->w_direct); cudaFree(p->w_bits);
    cudaFree(p->w_mean); cudaFree(p->x_nhwc_scratch); cudaFree(p->x_bits); cudaFree(p->w_i8); cudaFree(p->scale_i8); cudaFree(p->x_i8);
    cudaFree(p->split_scratch); cudaFree(p->split_counters);
    if (!p->status_shared) cudaFree(p->status);
    delete p;
}

extern "C" const char *dnb_conv_plan_kernel(const dnb_conv_plan *p)
{
    if (!p) return "";
    if (p->kernel == K_XNOR && p->xnor_tc) return kXnorTcName;
    return p->stem_tc ? "stem_tc_tf32" : kKernelNames[p->kernel];
}

extern "C" int dnb_conv_plan_describe(const dnb_conv_plan *p, char *buf, int len)
{
    if (!p || !buf || len < 1) DNB_FAIL(DNB_EINVAL, "conv describe: bad argument");
    const TcArgs &a = p->tc;
    if ((p->kernel == K_TC_TF32 || p->kernel == K_TC_BF16 || (p->kernel == K_XNOR && p->xnor_tc)) && p->tc_x_ptr)
        snprintf(buf, len, "%s pair=%d halo=%d bn=%d tile=%dx%dx%d tiles=%d stages=%d ctas_per_sm=%d srb=%d splits=%d signs_in=%d signs_out=%d", kKernelNames[p->kernel], a.pair, a.halo,
                 a.bn, a.wt, a.ht, a.bt, a.total_tiles, a.stages, a.ctas_per_sm, a.store_row_bytes, a.splits, p->signs_given ? 1 : 0, a.sign_out ? 1 : 0);
    else
        snprintf(buf, len, "%s", dnb_conv_plan_kernel(p));
    return DNB_OK;
}

template <typename T>
static int upload(T **dst, const std::vector<T> &src)
{
    if (*dst) { cudaFree(*dst); *dst = nullptr; }
    DNB_CUDA(cudaMalloc((void **)dst, src.size() * sizeof(T)));
    DNB_CUDA(cudaMemcpy(*dst, src.data(), src.size() * sizeof(T), cudaMemcpyHostToDevice));
    return DNB_OK;
}

// ------------------------------------------------------------------ derived parameter tensors, built on the device
// One host-to-device copy of the layer's weights as Darknet holds them ([n][c/groups][size][size]) and one kernel per
// derived tensor: transposition into the kernels' layouts, rounding to the storage type, sign extraction.
namespace {

// tensor-core layout [tap][n_pad][c_pad], zero where padded; T = float (rounded to TF32-nearest) or bf16
template <typename T>
__global__ void repack_tc_kernel(const float *__restrict__ w, T *__restrict__ out, int n, int c, int taps, int n_pad, int c_pad)
{
    const size_t total = (size_t)taps * n_pad * c_pad;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int cc = (int)(i % c_pad);
        const size_t r = i / c_pad;
        const int f = (int)(r % n_pad), t = (int)(r / n_pad);
        float v = 0.f;
        if (f < n && cc < c) v = __ldg(w + ((size_t)f * c + cc) * taps + t);
        if (sizeof(T) == 4) {
            // nearest TF32, ties away from zero (what cvt.rna.tf32.f32 computes); infinities and NaNs pass through
            uint32_t u = __float_as_uint(v);
            if ((u & 0x7f800000u) != 0x7f800000u) u = (u + 0x1000u) & ~0x1fffu;
            reinterpret_cast<float *>(out)[i] = __uint_as_float(u);
        } else {
            reinterpret_cast<__nv_bfloat16 *>(out)[i] = __float2bfloat16_rn(v);
        }
    }
}

// CUDA-core layout [groups][K][npg_pad], K = c/groups * size * size, filters innermost
__global__ void repack_direct_kernel(const float *__restrict__ w, float *__restrict__ out, int groups, int npg, size_t K, int npg_pad)
{
    const size_t total = (size_t)groups * K * npg_pad;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int f = (int)(i % npg_pad);
        const size_t r = i / npg_pad;
        const size_t k = r % K;
        const int g = (int)(r / K);
        out[i] = f < npg ? __ldg(w + ((size_t)(g * npg + f)) * K + k) : 0.f;
    }
}

// xnor: per filter the mean |w|, summed in a float in index order as binarize_weights does (src/convolutional_layer.c:28-41):
// one thread per filter, so the order of the additions is the reference's
__global__ void xnor_mean_kernel(const float *__restrict__ w, float *__restrict__ mean, int n, size_t K)
{
    const int f = blockIdx.x * blockDim.x + threadIdx.x;
    if (f >= n) return;
    float acc = 0.f;
    for (size_t k = 0; k < K; ++k) acc += fabsf(__ldg(w + (size_t)f * K + k));
    mean[f] = acc / (float)K;
}

// xnor: sign bits [n][taps][cwords] (bit c % 32 of word c / 32 set where w > 0), one thread per word
__global__ void xnor_bits_kernel(const float *__restrict__ w, uint32_t *__restrict__ bits, int n, int c, int taps, int cwords)
{
    const size_t total = (size_t)n * taps * cwords;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int wd = (int)(i % cwords);
        const size_t r = i / cwords;
        const int t = (int)(r % taps), f = (int)(r / taps);
        uint32_t word = 0;
        for (int k = 0; k < 32; ++k) {
            const int cc = wd * 32 + k;
            if (cc < c && __ldg(w + ((size_t)f * c + cc) * taps + t) > 0.f) word |= 1u << k;
        }
        bits[i] = word;
    }
}

// xnor on the tensor cores: signs as int8 in the tensor-core weight layout [tap][n_pad][c_pad], zero where padded
__global__ void xnor_i8_kernel(const float *__restrict__ w, int8_t *__restrict__ out, int n, int c, int taps, int n_pad, int c_pad)
{
    const size_t total = (size_t)taps * n_pad * c_pad;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int cc = (int)(i % c_pad);
        const size_t r = i / c_pad;
        const int f = (int)(r % n_pad), t = (int)(r / n_pad);
        int8_t v = 0;
        if (f < n && cc < c) v = __ldg(w + ((size_t)f * c + cc) * taps + t) > 0.f ? 1 : -1;
        out[i] = v;
    }
}

// mean|w| folded into the batchnorm scale of the tensor-core xnor kernel
__global__ void scale_times_mean_kernel(const float *__restrict__ scale, const float *__restrict__ mean, float *__restrict__ out, int n, int n_pad)
{
    const int f = blockIdx.x * blockDim.x + threadIdx.x;
    if (f < n_pad) out[f] = f < n ? mean[f] * scale[f] : 0.f;
}

int grid_of(size_t total)
{
    const size_t blocks = (total + 255) / 256, cap = (size_t)sm_count() * 16;
    return (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
}

template <typename T>
int device_alloc(T **dst, size_t count)
{
    if (*dst) { cudaFree(*dst); *dst = nullptr; }
    DNB_CUDA(cudaMalloc((void **)dst, count * sizeof(T)));
    return DNB_OK;
}

}  // namespace

extern "C" int dnb_conv_plan_set_params(dnb_conv_plan *p, const float *weights, const float *biases, const float *scales,
                                        const float *mean, const float *var)
{
    if (!p || !weights || !biases) DNB_FAIL(DNB_EINVAL, "conv params: null argument");
    const dnb_conv_desc &d = p->d;
    if (d.batch_normalize && (!scales || !mean || !var)) DNB_FAIL(DNB_EINVAL, "conv params: batch_normalize layer needs scales, rolling_mean, rolling_variance");
    DNB_TRY(check_current_device(p->device, "conv params"));
    const int cpg = d.c / d.groups, npg = d.n / d.groups, taps = d.size * d.size;
    const size_t K = (size_t)cpg * taps, nw = (size_t)d.n * K;

    // Folded inference batchnorm.  The CPU reference computes
    // ((x - mean) / (sqrt(var) + 1e-6f)) * scale + bias (src/blas.c:147-158,
    // src/batchnorm_layer.c:151-154); folded: x*s + (bias - mean*s).
    std::vector<float> s(p->n_pad, 0.f), b(p->n_pad, 0.f);
    for (int n = 0; n < d.n; ++n) {
        if (d.batch_normalize) {
            const double sc = (double)scales[n] / (sqrt((double)var[n]) + (double).000001f);
            s[n] = (float)sc;
            b[n] = (float)((double)biases[n] - (double)mean[n] * sc);
        } else {
            s[n] = 1.f;
            b[n] = biases[n];
        }
    }
    DNB_TRY(upload(&p->scale, s));
    DNB_TRY(upload(&p->shift, b));

    // the weights as Darknet holds them, once; every derived tensor is built from this copy on the device
    float *raw = nullptr;
    DNB_CUDA(cudaMalloc((void **)&raw, nw * sizeof(float)));
    struct Raw { float *p; ~Raw() { cudaFree(p); } } raw_guard{raw};
    DNB_CUDA(cudaMemcpy(raw, weights, nw * sizeof(float), cudaMemcpyHostToDevice));

    if (p->kernel == K_TC_TF32) {
        const size_t total = (size_t)taps * p->n_pad * p->c_pad;
        float *dev = (float *)p->w_tc;
        DNB_TRY(device_alloc(&dev, total));
        p->w_tc = dev;
        repack_tc_kernel<float><<<grid_of(total), 256>>>(raw, dev, d.n, d.c, taps, p->n_pad, p->c_pad);
    } else if (p->kernel == K_TC_BF16) {
        const size_t total = (size_t)taps * p->n_pad * p->c_pad;
        __nv_bfloat16 *dev = (__nv_bfloat16 *)p->w_tc;
        DNB_TRY(device_alloc(&dev, total));
        p->w_tc = dev;
        repack_tc_kernel<__nv_bfloat16><<<grid_of(total), 256>>>(raw, dev, d.n, d.c, taps, p->n_pad, p->c_pad);
    } else if (p->kernel == K_DIRECT) {
        const size_t total = (size_t)d.groups * K * p->npg_pad;
        DNB_TRY(device_alloc(&p->w_direct, total));
        repack_direct_kernel<<<grid_of(total), 256>>>(raw, p->w_direct, d.groups, npg, K, p->npg_pad);
    } else {
        DNB_TRY(device_alloc(&p->w_bits, (size_t)d.n * taps * p->cwords));
        DNB_TRY(device_alloc(&p->w_mean, (size_t)d.n));
        xnor_bits_kernel<<<grid_of((size_t)d.n * taps * p->cwords), 256>>>(raw, p->w_bits, d.n, d.c, taps, p->cwords);
        xnor_mean_kernel<<<(d.n + 127) / 128, 128>>>(raw, p->w_mean, d.n, K);
        if (p->xnor_tc) {
            const size_t total = (size_t)taps * p->n_pad * p->c_pad_i8;
            DNB_TRY(device_alloc(&p->w_i8, total));
            DNB_TRY(device_alloc(&p->scale_i8, (size_t)p->n_pad));
            xnor_i8_kernel<<<grid_of(total), 256>>>(raw, p->w_i8, d.n, d.c, taps, p->n_pad, p->c_pad_i8);
            scale_times_mean_kernel<<<(p->n_pad + 127) / 128, 128>>>(p->scale, p->w_mean, p->scale_i8, d.n, p->n_pad);
        }
    }
    DNB_LAUNCH_CHECK("weight repack");
    DNB_CUDA(cudaDeviceSynchronize());   // the staging copy is released on return
    p->params_set = true;
    // The launch block caches a tensor map over the weights just replaced: have the next forward rebuild it.
    p->tc_x_ptr = p->tc_y_ptr = p->tc_res_ptr = nullptr;
    return DNB_OK;
}

// Shortens the bound of the plan's device-side waits (cycles; 0 restores the default of about one second) and
// sets diagnostic bits of the tensor-core kernel.  Bit 32 makes every CTA withhold one operand load, so that a
// wait runs out: the way the time-out path is exercised without faulting the device.
extern "C" int dnb_conv_plan_set_diagnostics(dnb_conv_plan *p, long long wait_limit_cycles, int debug_bits)
{
    if (!p || wait_limit_cycles < 0) DNB_FAIL(DNB_EINVAL, "conv diagnostics: bad argument");
    p->wait_limit = wait_limit_cycles;
    p->debug_bits = debug_bits;
    p->tc_x_ptr = p->tc_y_ptr = p->tc_res_ptr = nullptr;
    return DNB_OK;
}

// ------------------------------------------------------------------ tensor-core launch block
// Relative cost of writing NCHW output in runs of `run` contiguous pixels (tuning knob DNB_TC_NCHW_PENALTY scales it;
// 0 = the tile that suits channels-last output).
static double nchw_run_penalty(int run)
{
    static double scale = -1.0;
    if (scale < 0.0) { const char *e = getenv("DNB_TC_NCHW_PENALTY"); scale = e ? atof(e) : 1.0; }
    const double base = run >= 32 ? 0.0 : run >= 16 ? 0.03 : run >= 8 ? 0.10 : run >= 4 ? 0.5 : run >= 2 ? 1.0 : 2.0;
    return scale * base;
}

static void pick_pixel_tile(const ConvGeom &g, bool nchw_out, int *wt, int *ht, int *bt)
{
    // wt*ht*bt == 128, powers of two; least padded work, then widest rows.
    // A launch that writes Darknet's layout stores, per filter plane, one run of wt pixels per tile row: runs shorter
    // than a 32-byte sector make every store a partial-sector write, which costs far more than the padded work of a
    // wider tile (measured on the 255-filter heads of YOLOv3-608, batch 64: 4-pixel runs 2.0 ms, see nchw_run_penalty).
    double best = 1e300;
    for (int w = 1; w <= 128; w *= 2)
        for (int h = 1; w * h <= 128; h *= 2) {
            const int b = 128 / (w * h);
            const double work = (double)round_up(g.out_w, w) * round_up(g.out_h, h) * round_up(g.batch, b);
            double score = work * (1.0 + 1e-6 * (128 - w) + 1e-7 * (128 - h));
            if (nchw_out) score *= 1.0 + nchw_run_penalty(w < g.out_w ? w : g.out_w);
            if (score < best) { best = score; *wt = w; *ht = h; *bt = b; }
        }
}

static int build_tc_args(dnb_conv_plan *p, const dnb_tensor *x, void *y_nhwc, int y_dtype, int y_cpitch,
                         const void *residual, int res_cpitch, bool nchw_out, void *sign_out = nullptr, int sign_cpitch = 0)
{
    TcArgs &a = p->tc;
    // A 1x1 convolution (stride 1, no padding) does not care which pixels are neighbours: with Darknet's layout among
    // the outputs, the h x w plane is treated as one row of h*w pixels, so that a tile is a run of up to 128 contiguous
    // pixels of every filter plane (and of the channels-last input) instead of a wt x ht patch.  DNB_TC_FLAT=0: never.
    ConvGeom g = p->g;
    {
        const char *e = getenv("DNB_TC_FLAT");
        if (nchw_out && g.size == 1 && g.stride == 1 && g.pad == 0 && !(e && atoi(e) == 0)) {
            g.w = g.out_w = g.w * g.h;
            g.h = g.out_h = 1;
        }
    }
    const bool bf16 = p->kernel == K_TC_BF16, i8 = p->kernel == K_XNOR;
    const int es = i8 ? 1 : (bf16 ? 2 : 4);
    const int kind = i8 ? 2 : (bf16 ? 1 : 0);              // element kind of the operands (and of their tensor maps)
    const int c_pad = i8 ? p->c_pad_i8 : p->c_pad;         // channel pitch of the operand tensors
    a.is_bf16 = kind;
    const int cbytes = c_pad * es;
    a.row_bytes = cbytes >= 128 ? 128 : (cbytes >= 64 ? 64 : 32);
    a.bk = a.row_bytes / es;
    a.c_blocks = (c_pad + a.bk - 1) / a.bk;
    a.taps = g.size * g.size;
    pick_pixel_tile(g, nchw_out, &a.wt, &a.ht, &a.bt);
    // Halo mode (experimental, off unless DNB_TC_HALO is 1 or 2): one activation box per channel block serves all
    // nine taps of a 3x3 stride-1 layer, which cuts the bytes that cross L2 -> shared memory by 2.3x on the
    // 32- and 64-channel layers of large maps.  Measured on YOLOv3-608 batch 64 it does not pay yet: the 8 x 16
    // tile, the two rings it needs and the smaller share of shared memory left for each slow the 304x304 and
    // 152x152 layers by 25-35 % (an isolated 32 -> 64 layer without a residual gains 11 %).  1: where the
    // heuristic below allows; 2: wherever the geometry allows (the tests use this).
    a.halo = 0;
    {
        const char *e = getenv("DNB_TC_HALO");
        const int knob = e ? atoi(e) : 0;
        if (knob != 0 && !i8 && g.size == 3 && g.stride == 1 && g.pad == 1 && a.row_bytes == 128 && g.out_w >= 8 && g.out_h >= 16) {
            const double work_h = (double)round_up(g.out_w, 8) * round_up(g.out_h, 16) * g.batch;
            const double work_0 = (double)round_up(g.out_w, a.wt) * round_up(g.out_h, a.ht) * round_up(g.batch, a.bt);
            if (knob == 2 || (a.c_blocks <= 2 && work_h <= 1.08 * work_0)) { a.halo = 1; a.wt = 8; a.ht = 16; a.bt = 1; }
        }
    }
    a.tiles_w = (g.out_w + a.wt - 1) / a.wt;
    a.tiles_h = (g.out_h + a.ht - 1) / a.ht;
    a.tiles_b = (g.batch + a.bt - 1) / a.bt;
    const int ptiles = a.tiles_w * a.tiles_h * a.tiles_b;
    // Filters per tile.  One tile when they fit (<= 256).  Otherwise a multiple of 64 (so that every
    // staged output chunk lies inside one tile), weighing padded MMA columns against operand re-loads.
    if (p->n_pad <= 256) {
        a.bn = p->n_pad;
    } else {
        double best = 1e300;
        for (int bn = 64; bn <= 256; bn += 64) {
            const int nt = (p->n_pad + bn - 1) / bn;
            const double score = (double)nt * bn + 0.5 * nt * 128;
            if (score <= best) { best = score; a.bn = bn; }
        }
    }
    // Tuning knobs for experiments: DNB_TC_BN (filters per tile, a multiple of 64) and DNB_TC_STAGES.
    if (const char *e = getenv("DNB_TC_BN")) {
        const int v = atoi(e);
        if (v >= 64 && v <= 256 && v % 64 == 0 && p->n_pad > v) a.bn = v;
    }
    a.n_tiles = (p->n_pad + a.bn - 1) / a.bn;
    while (ptiles * a.n_tiles < sm_count() && a.bn >= 128 && a.bn % 128 == 0) {  // too few tiles to fill the SMs
        a.bn /= 2;
        a.n_tiles = (p->n_pad + a.bn - 1) / a.bn;
    }
    // A launch that writes Darknet's layout spends a store per output element in its epilogue; behind a short K loop
    // (the 1x1 heads of YOLOv3) that is the whole run time, and the four epilogue warps of one CTA per SM issue it
    // slowly: 128-filter tiles leave TMEM for a second CTA, i.e. eight epilogue warps.
    if (nchw_out && a.bn == 256 && g.size * g.size * a.c_blocks <= 16) {
        a.bn = 128;
        a.n_tiles = (p->n_pad + a.bn - 1) / a.bn;
    }
    // CTA pairs (cta_group::2): for layers whose filters come in whole tiles of 256 and whose K loop is long enough to
    // be bound by operand traffic.  Each CTA of a pair loads its own 128 pixels and half of the 256-filter weight tile:
    // a third fewer bytes from L2 into shared memory per MMA, and 32 KB ring slots (six of them) instead of 48 KB (four).
    // DNB_TC_PAIR: 0 never, 1 (default) layers with at least 16 K iterations (every 3x3 layer that qualifies, and 1x1
    // layers over 512 or more channels: 8 % faster than single CTAs on YOLOv3's 38x38 and 19x19 1x1 layers at batch 64),
    // 2 every layer the geometry allows.
    a.pair = 0;
    {
        const char *e = getenv("DNB_TC_PAIR");
        const int knob = e ? atoi(e) : 1;
        // (the pair kernel is built for 128-byte staged rows only: it needs a channels-last output at least that wide)
        // Enough pair tiles to occupy every pair of SMs; or, for long K loops (small batches of the 19x19 and 38x38
        // layers), at least half of them: a pair's six-deep ring of 32 KB slots keeps its tensor pipes fed where two
        // single CTAs per SM with two or three slots each starve on load latency, which outweighs the idle SMs.
        const int pair_tiles = (ptiles + 1) / 2 * (g.n / 256), clusters = sm_count() / 2;
        const int k_iters_p = g.size * g.size * a.c_blocks;
        // (with split-K, below, a sixteenth of them is enough: every pair tile becomes up to eight)
        const bool split_ok = !(getenv("DNB_TC_SPLITK") && atoi(getenv("DNB_TC_SPLITK")) == 0) && !i8;
        const bool enough = pair_tiles >= clusters || (k_iters_p >= 64 && (2 * pair_tiles >= clusters || (split_ok && 16 * pair_tiles >= clusters)));
        const bool legal = !a.halo && a.row_bytes == 128 && g.n % 256 == 0 && enough && y_nhwc && y_cpitch * (bf16 ? 2 : 4) >= 128;
        if (legal && (knob == 2 || (knob == 1 && (g.size >= 3 || k_iters_p >= 16)))) {
            a.pair = 1;
            a.bn = 256;
            a.n_tiles = p->n_pad / 256;
        }
    }
    a.total_tiles = a.pair ? (ptiles + 1) / 2 * a.n_tiles : ptiles * a.n_tiles;
    a.n_pad = p->n_pad;
    a.n_tot = a.n_tiles * a.bn;
    a.a_bytes = 128 * a.row_bytes;
    a.b_bytes = round_up((a.pair ? a.bn / 2 : a.bn) * a.row_bytes, 1024);
    const int max_smem = conv_tc_max_smem();
    if (max_smem <= 0) DNB_FAIL(DNB_ECUDA, "conv: cannot query shared memory of the current device");
    // staged output rows: the widest of 128 / 64 / 32 bytes that the output pitch allows and that keeps
    // at least four ring stages
    const int out_es = bf16 ? 2 : 4;   // channels-last output uses the plan's storage type
    const int pitch_bytes = y_nhwc ? y_cpitch * out_es : 32;
    const int min_srb = sign_out ? 128 : 16 * out_es;  // a staged row holds at least one 16-column piece of the accumulator; the sign output is built for 32 columns per chunk
    int srb = pitch_bytes >= 128 ? 128 : (pitch_bytes >= 64 ? 64 : 32);
    if (srb < min_srb) srb = min_srb;  // the box may be wider than a narrow tensor: the TMA unit clips it
    if (sign_out && (pitch_bytes < 128 || !i8)) DNB_FAIL(DNB_EINVAL, "conv: the sign output needs an int8-kind plan with at least 32 output channels");
    if (const char *e = getenv("DNB_TC_SRB")) {   // tuning knob: widest staged row to try (128, 64 or 32)
        const int v = atoi(e);
        if ((v == 128 || v == 64 || v == 32) && v >= min_srb && v < srb && !a.pair) srb = v;
    }
    const int min_stages = getenv("DNB_TC_MIN_STAGES") ? atoi(getenv("DNB_TC_MIN_STAGES")) : 4;
    // two accumulators of bn columns; TMEM is allocated in powers of two >= 32 columns
    a.tmem_cols = 32;
    while (a.tmem_cols < 2 * a.bn) a.tmem_cols *= 2;
    // Narrow tiles (bn <= 128) leave TMEM and, with a short ring, shared memory for a second CTA on the SM:
    // twice the warps hide the per-tile hand-offs that dominate layers with few K iterations.
    a.ctas_per_sm = 1;
    a.stage_bufs = (residual && !a.pair) ? 4 : 2;   // a pair reads the residual with plain loads: nothing lands in the staging buffers
    if (sign_out) a.stage_bufs = 3;   // the third buffer holds the staged signs
    a.sign_out = sign_out;
    a.sign_cpitch = sign_cpitch;
    a.debug = (getenv("DNB_TC_DEBUG") ? atoi(getenv("DNB_TC_DEBUG")) : 0) | p->debug_bits;
    a.wait_limit = p->wait_limit > 0 ? p->wait_limit : DEFAULT_WAIT_CYCLES;
    int stages = 0;
    const bool allow2 = getenv("DNB_TC_CTAS") ? atoi(getenv("DNB_TC_CTAS")) >= 2 : true;
    a.a_stages = a.b_stages = a.a_slot = a.a_box_bytes = a.a_pitch = 0;
    if (a.halo) {
        // two rings: activation boxes (one per channel block) and weight tiles (nine per box).  A weight tile is
        // consumed in a quarter of the time an ordinary ring slot is, so that ring wants to be deep: one CTA per
        // SM unless two still leave six weight slots each.
        a.a_pitch = a.wt + 2;
        a.a_box_bytes = (a.wt + 2) * (a.ht + 2) * a.row_bytes;
        a.a_slot = round_up(a.a_box_bytes, 1024);
        auto fit = [&](long budget, int srb_try, int a_want, int b_min) {
            const long left = budget - (long)conv_tc_fixed_smem(srb_try, a.bn, a.stage_bufs) - (long)a_want * a.a_slot;
            const int b = left > 0 ? (int)(left / a.b_bytes) : 0;
            if (b < b_min) return false;
            a.a_stages = a_want; a.b_stages = b > 12 ? 12 : b; srb = srb_try;
            return true;
        };
        bool done = false;
        if (allow2 && a.tmem_cols <= 256) {
            const long budget = (228L * 1024) / 2 - 2048;
            for (int srb2 = srb; srb2 >= min_srb && !done; srb2 /= 2) done = fit(budget, srb2, 2, 6);
            if (done) a.ctas_per_sm = 2;
        }
        for (int srb2 = srb; srb2 >= min_srb && !done; srb2 /= 2) done = fit(max_smem, srb2, 3, 6) || fit(max_smem, srb2, 2, 4);
        if (!done) a.halo = 0;   // the tile shape stays 8 x 16: still a valid tiling for the ordinary rings below
        stages = 2;
    }
    if (!a.halo) {
        if (allow2 && a.tmem_cols <= 256 && !a.pair) {
            const int max2 = getenv("DNB_TC_MAX2") ? atoi(getenv("DNB_TC_MAX2")) : 4;   // ring slots per CTA when two share the SM
            const long budget = (228L * 1024) / 2 - 2048;   // per CTA when two share the SM (1 KB each is reserved by the system)
            for (int srb2 = srb; srb2 >= min_srb; srb2 /= 2) {   // narrower staged rows if that is what makes two CTAs fit
                const int s2 = (int)((budget - (long)conv_tc_fixed_smem(srb2, a.bn, a.stage_bufs)) / (a.a_bytes + a.b_bytes));
                if (s2 >= 2) { a.ctas_per_sm = 2; stages = s2 > max2 ? max2 : s2; srb = srb2; break; }
            }
        }
        if (a.ctas_per_sm == 1) {
            // The depth of the ring is what hides the operand loads' latency: four slots before wide staged rows.
            // The exception is a fused residual behind a short K loop, where the epilogue (one round of barrier,
            // residual wait and store per staged chunk) would outlast the tile's MMAs: fewer, wider chunks then.
            const int k_iters = g.size * g.size * a.c_blocks;
            const bool short_k_rule = getenv("DNB_TC_SHORTK") ? atoi(getenv("DNB_TC_SHORTK")) != 0 : true;
            const int short_k = bf16 ? 32 : 64;   // measured: 76x76x128 -> 256 layers want the wide rows in both modes, 38x38x256 -> 512 only in TF32
            const int want = (residual && k_iters < short_k && min_stages > 3 && short_k_rule) ? 3 : min_stages;
            for (;; srb /= 2) {
                stages = (int)((max_smem - (long)conv_tc_fixed_smem(srb, a.bn, a.stage_bufs)) / (a.a_bytes + a.b_bytes));
                if (stages >= want || srb == min_srb) break;
            }
        }
    }
    if (stages > 8) stages = 8;
    if (const char *e = getenv("DNB_TC_STAGES")) {
        const int v = atoi(e);
        if (v >= 2 && v <= stages) stages = v;
    }
    if (stages < 2) DNB_FAIL(DNB_ECUDA, "conv: %d bytes of shared memory are too few for the operand ring", max_smem);
    a.stages = stages;
    a.store_row_bytes = srb;
    // Split-K: a layer with fewer tiles than the GPU has room for and a long K loop (the 19x19 and 38x38 layers at
    // small batches) cuts every tile's K loop into `splits` ranges that run as separate tiles; see the kernel.
    // The cost model counts waves of tiles, in units of one K-loop iteration (about 0.3 us): a tile cut into S ranges
    // costs K/S iterations plus the partial sums' trip through L2: one dump (about 10 units) and, in the CTA that
    // finishes the tile, S dependent rounds of loads per staged chunk (about 16 units per range; measured on the 19x19
    // layers of YOLOv3 at one image: 61 us unsplit, 46 us with eight ranges).  Only long K loops on a mostly empty GPU
    // qualify: batches of one or two images.
    // DNB_TC_SPLITK: 0 never, N > 1 forces N ranges wherever the variant exists (tests).
    {   // DNB_TC_WARP_STORES=1 (experiment, off): every epilogue warp stores its own 32 rows and the four warps meet once
        // per tile instead of twice per chunk.  Measured on YOLOv3-608 b64: the layers' event times drop by 0.5 %, the
        // step replayed as one CUDA graph takes 2 % longer (18.5 -> 18.9 ms), batch 8 and ResNet-50 do not move.
        const char *e = getenv("DNB_TC_WARP_STORES");
        a.warp_stores = e ? (atoi(e) != 0) : 0;
    }
    a.splits = 1;
    a.split_scratch = nullptr;
    a.split_counters = nullptr;
    {
        const char *e = getenv("DNB_TC_SPLITK");
        const int knob = e ? atoi(e) : -1;
        const int k_iters = g.size * g.size * a.c_blocks, cpc = srb / out_es;
        const bool legal = knob != 0 && !a.halo && !i8 && srb == 128 && a.bn % cpc == 0 && (!residual || a.pair) && k_iters >= 4;
        if (legal) {
            const int slots = a.pair ? sm_count() / 2 : sm_count() * a.ctas_per_sm;
            const int T = a.total_tiles;
            int best_s = 1;
            double best = (double)((T + slots - 1) / slots);
            best *= k_iters;
            const double alone_units = best;
            for (int S = 2; S <= 8 && k_iters / S >= 8; ++S) {
                const double cost = (double)(((long long)T * S + slots - 1) / slots) * ((double)k_iters / S + 10.0 + 16.0 * S);
                if (cost < best) { best = cost; best_s = S; }
            }
            if (best > 0.85 * alone_units) best_s = 1;   // not worth the extra traffic
            if (knob > 1) best_s = knob < k_iters / 2 ? knob : k_iters / 2;
            if (best_s > 8) best_s = 8;
            a.splits = best_s > 1 ? best_s : 1;
        }
        if (a.splits > 1) {
            const int out_tiles = (a.pair ? (ptiles + 1) / 2 * 2 : ptiles) * a.n_tiles;
            const size_t need = (size_t)out_tiles * a.splits * 128 * a.bn * sizeof(float);
            if (need > p->split_scratch_bytes) {
                cudaFree(p->split_scratch);
                p->split_scratch = nullptr; p->split_scratch_bytes = 0;
                DNB_CUDA(cudaMalloc(&p->split_scratch, need));
                p->split_scratch_bytes = need;
            }
            if (out_tiles > p->split_counters_n) {
                cudaFree(p->split_counters);
                p->split_counters = nullptr; p->split_counters_n = 0;
                DNB_CUDA(cudaMalloc((void **)&p->split_counters, (size_t)out_tiles * sizeof(int)));
                DNB_CUDA(cudaMemset(p->split_counters, 0, (size_t)out_tiles * sizeof(int)));
                p->split_counters_n = out_tiles;
            }
            a.split_scratch = p->split_scratch;
            a.split_counters = p->split_counters;
            a.total_tiles *= a.splits;
        }
    }
    a.g = g;
    if (!p->status) {
        DNB_CUDA(cudaMalloc((void **)&p->status, sizeof(int)));
        DNB_CUDA(cudaMemset(p->status, 0, sizeof(int)));
    }
    a.status = p->status;

    // activation maps: lattice (ph, pw) of the input holds rows ph, ph+stride, ... and columns pw, pw+stride, ...
    const size_t pix_bytes = (size_t)x->cpitch * es;
    const int s = g.stride;
    if (s > 2) DNB_FAIL(DNB_EUNSUPPORTED, "conv: stride %d on the tensor-core path (1 and 2 are covered)", s);
    for (int ph = 0; ph < s; ++ph)
        for (int pw = 0; pw < s; ++pw) {
            const int hl = (g.h - ph + s - 1) / s, wl = (g.w - pw + s - 1) / s;
            uint64_t dims[4] = {(uint64_t)c_pad, (uint64_t)(wl > 0 ? wl : 1), (uint64_t)(hl > 0 ? hl : 1), (uint64_t)g.batch};
            uint64_t strides[3] = {pix_bytes * s, pix_bytes * g.w * s, pix_bytes * g.w * g.h};
            uint32_t box[4] = {(uint32_t)a.bk, (uint32_t)a.wt, (uint32_t)a.ht, (uint32_t)a.bt};
            if (a.halo) { box[1] = (uint32_t)(a.wt + 2); box[2] = (uint32_t)(a.ht + 2); }
            char *base = (char *)x->data + ((size_t)ph * g.w + pw) * pix_bytes;
            if (hl <= 0 || wl <= 0) base = (char *)x->data;  // lattice empty: never addressed in-bounds
            DNB_TRY(encode_tensor_map(&a.tmx[ph * s + pw], kind, 4, base, dims, strides, box, a.row_bytes));
        }
    {
        uint64_t dims[3] = {(uint64_t)c_pad, (uint64_t)p->n_pad, (uint64_t)a.taps};
        uint64_t strides[2] = {(uint64_t)c_pad * es, (uint64_t)c_pad * es * p->n_pad};
        uint32_t box[3] = {(uint32_t)a.bk, (uint32_t)(a.pair ? a.bn / 2 : a.bn), 1u};
        DNB_TRY(encode_tensor_map(&a.tmw, kind, 3, i8 ? (void *)p->w_i8 : p->w_tc, dims, strides, box, a.row_bytes));
    }
    if (y_nhwc) {
        const size_t opix = (size_t)y_cpitch * out_es;
        // the channel extent is the layer's own (padded to 8), the pitch whatever the tensor has: the output may be a
        // channel range of a wider tensor (a [route] output), and the boxes must not spill into its neighbour
        const int y_chan = round_up(g.n, 8) < y_cpitch ? round_up(g.n, 8) : y_cpitch;
        uint64_t dims[4] = {(uint64_t)y_chan, (uint64_t)g.out_w, (uint64_t)g.out_h, (uint64_t)g.batch};
        uint64_t strides[3] = {opix, opix * g.out_w, opix * g.out_w * g.out_h};
        uint32_t box[4] = {(uint32_t)(srb / out_es), (uint32_t)a.wt, (uint32_t)a.ht, (uint32_t)a.bt};
        DNB_TRY(encode_tensor_map(&a.tmy, bf16, 4, y_nhwc, dims, strides, box, srb));
        {   // the 32 consecutive rows of one epilogue warp: wt*ht*bt = 128 in powers of two, so they are a box too
            const int w2 = a.wt < 32 ? a.wt : 32, h2 = a.ht < 32 / w2 ? a.ht : 32 / w2, b2 = 32 / (w2 * h2);
            uint32_t wbox[4] = {(uint32_t)(srb / out_es), (uint32_t)w2, (uint32_t)h2, (uint32_t)b2};
            DNB_TRY(encode_tensor_map(&a.tmy_warp, bf16, 4, y_nhwc, dims, strides, wbox, srb));
        }
        if (residual) {
            const size_t rpix = (size_t)res_cpitch * out_es;
            const int r_chan = round_up(g.n, 8) < res_cpitch ? round_up(g.n, 8) : res_cpitch;
            uint64_t rdims[4] = {(uint64_t)r_chan, (uint64_t)g.out_w, (uint64_t)g.out_h, (uint64_t)g.batch};
            uint64_t rstrides[3] = {rpix, rpix * g.out_w, rpix * g.out_w * g.out_h};
            DNB_TRY(encode_tensor_map(&a.tmr, bf16, 4, const_cast<void *>(residual), rdims, rstrides, box, srb));
        }
    }
    if (sign_out) {
        uint64_t dims[4] = {(uint64_t)sign_cpitch, (uint64_t)g.out_w, (uint64_t)g.out_h, (uint64_t)g.batch};
        uint64_t strides[3] = {(uint64_t)sign_cpitch, (uint64_t)sign_cpitch * g.out_w, (uint64_t)sign_cpitch * g.out_w * g.out_h};
        uint32_t box[4] = {32u, (uint32_t)a.wt, (uint32_t)a.ht, (uint32_t)a.bt};
        DNB_TRY(encode_tensor_map(&a.tms, 2, 4, sign_out, dims, strides, box, 32));
    }
    p->tc_sign_out = sign_out;
    p->tc_x_ptr = x->data;
    p->tc_x_cpitch = x->cpitch;
    p->tc_y_ptr = y_nhwc;
    p->tc_y_cpitch = y_cpitch;
    p->tc_y_dtype = y_dtype;
    p->tc_res_ptr = residual;
    p->tc_res_cpitch = res_cpitch;
    p->tc_nchw_out = nchw_out ? 1 : 0;
    return DNB_OK;
}

// A tensor-core xnor layer reads its input as int8 signs.  Where the layer before it can write them as it writes its
// own f32 output (another tensor-core xnor layer, from its epilogue; a maxpool layer), the sign pass over the f32 tensor
// disappears.  conv_plan_expect_signs prepares the consumer (its operand buffer is allocated and returned; it skips its
// own pass whenever it is given `tensor`, the channels-last tensor that carries the producer's output) and
// conv_plan_link_signs also tells a producing xnor plan.  DNB_XNOR_SIGNS=0: never.
int8_t *conv_plan_expect_signs(dnb_conv_plan *consumer, const void *tensor, int batch, int c, int h, int w)
{
    const char *e = getenv("DNB_XNOR_SIGNS");
    if (e && atoi(e) == 0) return nullptr;
    if (!consumer || !tensor || consumer->kernel != K_XNOR || !consumer->xnor_tc) return nullptr;
    const ConvGeom &b = consumer->g;
    if (c != b.c || h != b.h || w != b.w || batch != b.batch || c % 32 || consumer->c_pad_i8 != c) return nullptr;
    const size_t need = (size_t)b.batch * b.h * b.w * consumer->c_pad_i8;
    if (need > consumer->x_i8_bytes) {
        cudaFree(consumer->x_i8);
        consumer->x_i8 = nullptr; consumer->x_i8_bytes = 0;
        if (cudaMalloc((void **)&consumer->x_i8, need) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        consumer->x_i8_bytes = need;
        consumer->tc_x_ptr = nullptr;
    }
    consumer->signs_given = true;
    consumer->signs_of = tensor;
    return consumer->x_i8;
}

bool conv_plan_link_signs(dnb_conv_plan *producer, dnb_conv_plan *consumer, const void *tensor)
{
    if (!producer || producer->kernel != K_XNOR || !producer->xnor_tc) return false;
    const ConvGeom &a = producer->g;
    if (!conv_plan_expect_signs(consumer, tensor, a.batch, a.n, a.out_h, a.out_w)) return false;
    producer->sign_consumer = consumer;
    return true;
}

// ------------------------------------------------------------------ forward
static int check_conv_io(const dnb_conv_plan *p, const dnb_tensor *x, const dnb_tensor *y, const dnb_tensor *y2)
{
    const ConvGeom &g = p->g;
    DNB_TRY(check_tensor(x, "conv input"));
    DNB_TRY(check_tensor(y, "conv output"));
    if (y2) DNB_TRY(check_tensor(y2, "conv second output"));
    if (x->n != g.batch || x->c != g.c || x->h != g.h || x->w != g.w)
        DNB_FAIL(DNB_EINVAL, "conv: input is %dx%dx%dx%d, plan expects %dx%dx%dx%d", x->n, x->c, x->h, x->w, g.batch, g.c, g.h, g.w);
    const dnb_tensor *outs[2] = {y, y2};
    for (int i = 0; i < 2; ++i) {
        const dnb_tensor *o = outs[i];
        if (!o) continue;
        if (o->n != g.batch || o->c != g.n || o->h != g.out_h || o->w != g.out_w)
            DNB_FAIL(DNB_EINVAL, "conv: output is %dx%dx%dx%d, plan produces %dx%dx%dx%d", o->n, o->c, o->h, o->w, g.batch, g.n, g.out_h, g.out_w);
    }
    if (y2 && y2->layout == y->layout) DNB_FAIL(DNB_EINVAL, "conv: the second output must use the other layout");
    return DNB_OK;
}

struct Residual {
    const dnb_tensor *add = nullptr;
    float alpha = 1.f, beta = 1.f;
    int activation = DNB_LINEAR;
    int yolo_entries = 0;   // instead of a residual: the [yolo] layer's activations, entries per anchor
};

static int conv_forward_impl(dnb_conv_plan *p, const dnb_tensor *x, const dnb_tensor *y, const dnb_tensor *y2,
                             int32_t *acc_out, cudaStream_t s, const Residual *res = nullptr)
{
    if (!p) DNB_FAIL(DNB_EINVAL, "conv: null plan");
    if (!p->params_set) DNB_FAIL(DNB_EINVAL, "conv: dnb_conv_plan_set_params has not been called");
    DNB_TRY(check_current_device(p->device, "conv"));
    const ConvGeom &g = p->g;
    void *y_nhwc = nullptr;
    float *y_nchw = nullptr;
    int y_dtype = DNB_F32, y_cpitch = 0;
    const dnb_tensor *outs[2] = {y, y2};
    for (int i = 0; i < 2; ++i) {
        const dnb_tensor *o = outs[i];
        if (!o) continue;
        if (o->layout == DNB_NHWC) { y_nhwc = o->data; y_dtype = o->dtype; y_cpitch = o->cpitch; }
        else y_nchw = (float *)o->data;
    }
    ConvEpilogue ep{p->scale, p->shift, p->d.activation, 0, nullptr, 0, DNB_LINEAR, 1.f, 1.f, 0, 0};
    if (res && res->yolo_entries > 0) {
        if (p->kernel != K_TC_TF32 && p->kernel != K_TC_BF16)
            DNB_FAIL(DNB_EUNSUPPORTED, "conv + yolo: only tensor-core plans fuse the yolo activations (this plan is %s)", kKernelNames[p->kernel]);
        ep.yolo_entries = res->yolo_entries;
    }
    if (res && res->add) {
        if (p->kernel != K_TC_TF32 && p->kernel != K_TC_BF16)
            DNB_FAIL(DNB_EUNSUPPORTED, "conv + shortcut: only tensor-core plans fuse the residual (this plan is %s)", kKernelNames[p->kernel]);
        ep.residual = res->add->data; ep.res_cpitch = res->add->cpitch; ep.activation2 = res->activation;
        ep.alpha = res->alpha; ep.beta = res->beta;
    }
    // f32 channels-last results of a TF32 network feed the next tensor-core layer: round them once here (the tensor
    // core would truncate them instead, a bias that adds up over a network's depth).  A copy in Darknet's layout
    // written by the same launch holds the same rounded values.
    ep.round_tf32 = (p->mode == DNB_MODE_TF32 && y_nhwc && y_dtype == DNB_F32) ? 1 : 0;

    if (p->kernel == K_DIRECT && p->stem_tc && x->dtype == DNB_F32 && y_nhwc && !y_nchw && y_cpitch == g.n) {
        StemTcArgs a;
        a.x = (const float *)x->data;
        if (x->layout == DNB_NHWC) { a.xs_c = 1; a.xs_w = x->cpitch; a.xs_h = (long long)g.w * x->cpitch; a.xs_b = (long long)g.h * a.xs_h; }
        else { a.xs_w = 1; a.xs_h = g.w; a.xs_c = (long long)g.h * g.w; a.xs_b = (long long)g.c * a.xs_c; }
        a.w = p->w_direct; a.npg_pad = p->npg_pad;
        a.y = y_nhwc; a.y_dtype = y_dtype; a.y_cpitch = y_cpitch;
        if (!p->status) {
            DNB_CUDA(cudaMalloc((void **)&p->status, sizeof(int)));
            DNB_CUDA(cudaMemset(p->status, 0, sizeof(int)));
        }
        a.status = p->status;
        a.wait_limit = p->wait_limit > 0 ? p->wait_limit : DEFAULT_WAIT_CYCLES;
        a.g = g; a.ep = ep;
        return launch_conv_stem_tc(a, s);
    }
    if (p->kernel == K_DIRECT) {   // also a first-layer plan asked for Darknet's layout or given bf16 input
        DirectArgs a;
        a.x = x->data; a.x_dtype = x->dtype;
        if (x->layout == DNB_NHWC) { a.xs_c = 1; a.xs_w = x->cpitch; a.xs_h = (long long)g.w * x->cpitch; a.xs_b = (long long)g.h * a.xs_h; }
        else { a.xs_w = 1; a.xs_h = g.w; a.xs_c = (long long)g.h * g.w; a.xs_b = (long long)g.c * a.xs_c; }
        a.wpk = p->w_direct; a.npg_pad = p->npg_pad;
        a.y_nhwc = y_nhwc; a.y_dtype = y_dtype; a.y_cpitch = y_cpitch; a.y_nchw = y_nchw;
        a.g = g; a.ep = ep;
        return launch_conv_direct(a, s);
    }
    if (p->kernel == K_XNOR && p->xnor_tc) {
        // tensor-core xnor: the input's signs as an int8 channels-last tensor (one pass over the input), then the
        // implicit-GEMM kernel in its int8 kind; out-of-image taps are the TMA unit's zero fill, i.e. they add nothing,
        // as in the reference, where the padding is applied after the binarisation (src/im2col.c:3-12)
        const size_t need = (size_t)g.batch * g.h * g.w * p->c_pad_i8;
        if (need > p->x_i8_bytes) {
            cudaFree(p->x_i8);
            p->x_i8 = nullptr; p->x_i8_bytes = 0;
            DNB_CUDA(cudaMalloc((void **)&p->x_i8, need));
            p->x_i8_bytes = need;
            p->tc_x_ptr = nullptr;
        }
        // (the xnor layer before this one, if the network linked the two, has written the signs from its epilogue)
        const bool given = p->signs_given && x->layout == DNB_NHWC && x->data == p->signs_of;
        if (!given) DNB_TRY(launch_pack_sign_i8(x, p->x_i8, p->c_pad_i8, s));
        dnb_tensor xin{p->x_i8, DNB_NHWC, DNB_F32, g.batch, g.c, g.h, g.w, p->c_pad_i8};   // dtype unused: the plan's kind says int8
        if (y_nhwc && y_dtype != DNB_F32) DNB_FAIL(DNB_EINVAL, "conv: an xnor plan writes channels-last output as f32");
        float *nchw = acc_out ? reinterpret_cast<float *>(acc_out) : y_nchw;
        void *nhwc = acc_out ? nullptr : y_nhwc;
        // signs for the next xnor layer, when this launch writes the very tensor that layer reads
        dnb_conv_plan *next = p->sign_consumer;
        void *sign_out = (next && nhwc && nhwc == next->signs_of && next->x_i8) ? next->x_i8 : nullptr;
        if (p->tc_x_ptr != xin.data || p->tc_y_ptr != nhwc || p->tc_y_cpitch != (nhwc ? y_cpitch : 0) || !p->status || p->tc_nchw_out != (nchw ? 1 : 0) ||
            p->tc_sign_out != sign_out)
            DNB_TRY(build_tc_args(p, &xin, nhwc, DNB_F32, nhwc ? y_cpitch : 0, nullptr, 0, nchw != nullptr, sign_out, sign_out ? next->c_pad_i8 : 0));
        TcArgs &a = p->tc;
        a.y_nhwc = nhwc; a.y_dtype = DNB_F32; a.y_cpitch = nhwc ? y_cpitch : 0; a.y_nchw = nchw;
        ep.scale = p->scale_i8;
        ep.round_tf32 = 0;
        ep.raw_acc = acc_out ? 1 : 0;
        if (acc_out) ep.activation = DNB_LINEAR;
        a.ep = ep;
        a.status = p->status;
        return launch_conv_tc(a, s);
    }
    if (p->kernel == K_XNOR) {
        const size_t need = (size_t)g.batch * g.h * g.w * p->cwords * sizeof(uint32_t);
        if (need > p->x_bits_bytes) {
            cudaFree(p->x_bits);
            p->x_bits = nullptr; p->x_bits_bytes = 0;
            DNB_CUDA(cudaMalloc((void **)&p->x_bits, need));
            p->x_bits_bytes = need;
        }
        DNB_TRY(launch_pack_sign_bits(x, p->x_bits, p->cwords, s));
        XnorArgs a;
        a.xbits = p->x_bits; a.wbits = p->w_bits; a.cwords = p->cwords; a.wmean = p->w_mean; a.acc_out = acc_out;
        a.y_nhwc = y_nhwc; a.y_dtype = y_dtype; a.y_cpitch = y_cpitch; a.y_nchw = y_nchw;
        a.g = g; a.ep = ep; a.ep.round_tf32 = 0;
        return launch_conv_xnor(a, s);
    }
    // tensor-core path: channels-last input of the plan's storage type
    const int want = p->kernel == K_TC_BF16 ? DNB_BF16 : DNB_F32;
    dnb_tensor xin = *x;
    if (x->layout == DNB_NCHW) {
        const size_t need = (size_t)g.batch * g.h * g.w * p->c_pad * elem_size(want);
        if (need > p->x_nhwc_bytes) {
            cudaFree(p->x_nhwc_scratch);
            p->x_nhwc_scratch = nullptr; p->x_nhwc_bytes = 0;
            DNB_CUDA(cudaMalloc(&p->x_nhwc_scratch, need));
            p->x_nhwc_bytes = need;
        }
        xin.data = p->x_nhwc_scratch; xin.layout = DNB_NHWC; xin.dtype = want; xin.cpitch = p->c_pad;
        DNB_TRY(launch_convert(x, &xin, want == DNB_F32, 0, 0, s));
    } else if (x->dtype != want) {
        DNB_FAIL(DNB_EINVAL, "conv: channels-last input is %s, this plan (%s) reads %s", x->dtype == DNB_BF16 ? "bf16" : "f32",
                 kKernelNames[p->kernel], want == DNB_BF16 ? "bf16" : "f32");
    }
    if (y_nhwc && y_dtype != want)
        DNB_FAIL(DNB_EINVAL, "conv: a %s plan writes channels-last output as %s", kKernelNames[p->kernel], want == DNB_BF16 ? "bf16" : "f32");
    if (p->tc_x_ptr != xin.data || p->tc_x_cpitch != xin.cpitch || p->tc_y_ptr != y_nhwc || p->tc_y_cpitch != y_cpitch ||
        p->tc_y_dtype != y_dtype || !p->status || p->tc_res_ptr != ep.residual || p->tc_res_cpitch != ep.res_cpitch ||
        p->tc_nchw_out != (y_nchw ? 1 : 0))
        DNB_TRY(build_tc_args(p, &xin, y_nhwc, y_dtype, y_cpitch, ep.residual, ep.res_cpitch, y_nchw != nullptr));
    TcArgs &a = p->tc;
    a.y_nhwc = y_nhwc; a.y_dtype = y_dtype; a.y_cpitch = y_cpitch; a.y_nchw = y_nchw;
    a.ep = ep;
    a.status = p->status;   // a network points its plans at the status word of the step being enqueued
    return launch_conv_tc(a, s);
}

extern "C" int dnb_conv_forward(dnb_conv_plan *p, const dnb_tensor *x, const dnb_tensor *y, const dnb_tensor *y2, void *stream)
{
    if (!p) DNB_FAIL(DNB_EINVAL, "conv: null plan");
    DNB_TRY(check_conv_io(p, x, y, y2));
    return conv_forward_impl(p, x, y, y2, nullptr, (cudaStream_t)stream);
}

// Convolution followed by the residual add of a [shortcut] layer, one launch:
// y = act2(alpha * act(conv(x)) + beta * add).
extern "C" int dnb_conv_shortcut_forward(dnb_conv_plan *p, const dnb_tensor *x, const dnb_tensor *add, const dnb_tensor *y,
                                         float alpha, float beta, int activation2, void *stream)
{
    if (!p || !add) DNB_FAIL(DNB_EINVAL, "conv + shortcut: null argument");
    DNB_TRY(check_conv_io(p, x, y, nullptr));
    DNB_TRY(check_tensor(add, "conv + shortcut residual"));
    if (activation2 < 0 || activation2 > DNB_SELU) DNB_FAIL(DNB_EINVAL, "conv + shortcut: activation %d", activation2);
    const int want = p->kernel == K_TC_BF16 ? DNB_BF16 : DNB_F32;
    if (add->layout != DNB_NHWC || y->layout != DNB_NHWC || add->dtype != want)
        DNB_FAIL(DNB_EINVAL, "conv + shortcut: residual and output must be channels-last in the plan's storage type");
    if (add->n != y->n || add->c != y->c || add->h != y->h || add->w != y->w)
        DNB_FAIL(DNB_EUNSUPPORTED, "conv + shortcut: the residual must have the output's extents (other shapes: dnb_shortcut_forward)");
    Residual r;
    r.add = add; r.alpha = alpha; r.beta = beta; r.activation = activation2;
    return conv_forward_impl(p, x, y, nullptr, nullptr, (cudaStream_t)stream, &r);
}

// Convolution followed by the [yolo] layer that reads it, one launch: forward_yolo_layer_gpu at inference copies
// its input and applies the logistic to the x, y, objectness and class entries of every anchor
// (src/yolo_layer.c:347-357); here the convolution's epilogue does that and writes the [yolo] layer's NCHW output.
extern "C" int dnb_conv_yolo_forward(dnb_conv_plan *p, const dnb_tensor *x, const dnb_tensor *y, int anchors, int classes, void *stream)
{
    if (!p) DNB_FAIL(DNB_EINVAL, "conv + yolo: null plan");
    DNB_TRY(check_conv_io(p, x, y, nullptr));
    if (anchors < 1 || classes < 0 || p->g.n != anchors * (classes + 5))
        DNB_FAIL(DNB_EINVAL, "conv + yolo: %d filters are not %d anchors of %d entries", p->g.n, anchors, classes + 5);
    if (y->layout != DNB_NCHW || y->dtype != DNB_F32) DNB_FAIL(DNB_EINVAL, "conv + yolo: the output is Darknet's layout (NCHW f32)");
    if (p->d.activation != DNB_LINEAR) DNB_FAIL(DNB_EUNSUPPORTED, "conv + yolo: the convolution's own activation must be linear (as in every yolo cfg)");
    if (p->g.n % 256 == 0) DNB_FAIL(DNB_EUNSUPPORTED, "conv + yolo: %d filters (whole tiles of 256 may run as CTA pairs, which have no yolo epilogue)", p->g.n);
    Residual r;
    r.yolo_entries = classes + 5;
    return conv_forward_impl(p, x, y, nullptr, nullptr, (cudaStream_t)stream, &r);
}

extern "C" int dnb_conv_xnor_accumulate(dnb_conv_plan *p, const dnb_tensor *x, int32_t *acc, void *stream)
{
    if (!p || !acc) DNB_FAIL(DNB_EINVAL, "xnor accumulate: null argument");
    if (p->kernel != K_XNOR) DNB_FAIL(DNB_EINVAL, "xnor accumulate: the plan is not an xnor plan");
    DNB_TRY(check_tensor(x, "conv input"));
    const ConvGeom &g = p->g;
    if (x->n != g.batch || x->c != g.c || x->h != g.h || x->w != g.w) DNB_FAIL(DNB_EINVAL, "xnor accumulate: input extents differ from the plan");
    return conv_forward_impl(p, x, nullptr, nullptr, acc, (cudaStream_t)stream);
}

// A launch that gave up on a wait may have left split-K counters part-way: zero them before the plan runs again.
void conv_plan_reset_after_abort(dnb_conv_plan *p, cudaStream_t s)
{
    if (p && p->split_counters) cudaMemsetAsync(p->split_counters, 0, (size_t)p->split_counters_n * sizeof(int), s);
}

// Device status word of the tensor-core kernel: 0, or the code of the bounded
// wait that expired (DNB_ETIMEOUT is returned to the caller in that case).
extern "C" int dnb_conv_plan_check_status(dnb_conv_plan *p)
{
    if (!p || !p->status) return DNB_OK;
    int v = 0;
    DNB_CUDA(cudaMemcpy(&v, p->status, sizeof(int), cudaMemcpyDeviceToHost));
    if (v) {
        cudaMemset(p->status, 0, sizeof(int));
        conv_plan_reset_after_abort(p);
        DNB_FAIL(DNB_ETIMEOUT, "conv: a device-side wait expired (code %d: 101 ring slot free, 102 operands landed, 103 accumulator free, 104 accumulator ready, 105 residual tile, 106 shared memory window not 1024-byte aligned)", v);
    }
    return DNB_OK;
}
