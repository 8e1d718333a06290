// Direct convolution on the CUDA cores (fp32 FMA, fp32 accumulate).
//
// Used where the tensor-core kernel does not apply: very narrow inputs (the
// 3-channel first layer, which it reads straight from Darknet's NCHW input),
// grouped convolutions, and DNB_MODE_FP32 networks.
//
// A block owns 128 consecutive output pixels and a slab of FB = 32 filters; a
// thread owns one pixel and all 32 filters of the slab.  The slab's weights are
// staged through shared memory in K chunks together with a (c,kh,kw) table, so
// the inner loop is one predicated, warp-coalesced load of x and 32 FMAs fed by
// broadcast 16-byte shared loads.  Accumulation runs over
// k = c*size*size + kh*size + kw in increasing order, the reference's own order
// (src/im2col.c:25-28, src/gemm.c:81-87).  Results go through a shared tile so
// that the global stores are 16-byte and contiguous across the warp in either
// output layout (a pixel's channel run for NHWC, a filter's pixel run for NCHW).
#include "common.h"
#include "conv.h"
#include "device_utils.cuh"

namespace dnb {

constexpr int FB = 32;         // filters per thread / per block slab
constexpr int KCHUNK = 192;    // taps staged per pass: 192 * (32*4 + 4) B = 25 KB
constexpr int DTHREADS = 128;  // pixels per block

template <typename TX, typename TY>
__global__ void __launch_bounds__(DTHREADS)
conv_direct_kernel(DirectArgs a)
{
    __shared__ __align__(16) float w_s[KCHUNK][FB];
    __shared__ int tap_s[KCHUNK];
    __shared__ __align__(16) float out_s[DTHREADS][FB + 4];   // +4 floats: rows stay 16-byte aligned, banks spread

    const ConvGeom &g = a.g;
    const int cpg = g.c / g.groups;           // input channels per group
    const int npg = g.n / g.groups;           // filters per group
    const int fblocks_per_group = (npg + FB - 1) / FB;
    const int grp = blockIdx.y / fblocks_per_group;
    const int f0 = (blockIdx.y % fblocks_per_group) * FB;   // first filter within the group
    const int K = cpg * g.size * g.size;
    const int ksq = g.size * g.size;

    const long long npix = (long long)g.batch * g.out_h * g.out_w;
    const long long pix0 = (long long)blockIdx.x * DTHREADS;
    const long long pix = pix0 + threadIdx.x;
    const bool live = pix < npix;
    int b = 0, oh = 0, ow = 0;
    if (live) {
        ow = (int)(pix % g.out_w);
        long long t = pix / g.out_w;
        oh = (int)(t % g.out_h);
        b = (int)(t / g.out_h);
    }
    const int ih0 = oh * g.stride - g.pad, iw0 = ow * g.stride - g.pad;
    const TX *xb = reinterpret_cast<const TX *>(a.x) + b * a.xs_b + (long long)grp * cpg * a.xs_c;

    float acc[FB];
#pragma unroll
    for (int j = 0; j < FB; ++j) acc[j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += KCHUNK) {
        const int kn = min(KCHUNK, K - k0);
        __syncthreads();
        // weights of this slab: packed [group][k][npg_pad], npg_pad a multiple of FB
        for (int i = threadIdx.x; i < kn * FB; i += DTHREADS) {
            int kk = i / FB, j = i % FB;
            w_s[kk][j] = __ldg(a.wpk + ((size_t)grp * K + k0 + kk) * a.npg_pad + f0 + j);
        }
        for (int kk = threadIdx.x; kk < kn; kk += DTHREADS) {
            int k = k0 + kk, c = k / ksq, r = k - c * ksq, kh = r / g.size, kw = r - kh * g.size;
            tap_s[kk] = (c << 8) | (kh << 4) | kw;
        }
        __syncthreads();
        if (live) {
            for (int kk = 0; kk < kn; ++kk) {
                const int t = tap_s[kk];
                const int c = t >> 8, ih = ih0 + ((t >> 4) & 15), iw = iw0 + (t & 15);
                float xv = 0.f;
                if (ih >= 0 && ih < g.h && iw >= 0 && iw < g.w)
                    xv = to_float<TX>(xb[c * a.xs_c + ih * a.xs_h + iw * a.xs_w]);
                const float4 *wr = reinterpret_cast<const float4 *>(w_s[kk]);
#pragma unroll
                for (int q = 0; q < FB / 4; ++q) {
                    float4 w4 = wr[q];
                    acc[4 * q + 0] = fmaf(xv, w4.x, acc[4 * q + 0]);
                    acc[4 * q + 1] = fmaf(xv, w4.y, acc[4 * q + 1]);
                    acc[4 * q + 2] = fmaf(xv, w4.z, acc[4 * q + 2]);
                    acc[4 * q + 3] = fmaf(xv, w4.w, acc[4 * q + 3]);
                }
            }
        }
    }

    // Epilogue: folded batchnorm / bias, activation, into the shared tile.
    const int n0 = grp * npg + f0;  // first global filter of this slab
#pragma unroll
    for (int j = 0; j < FB; ++j) {
        float v = 0.f;
        if (f0 + j < npg) {
            v = acc[j] * __ldg(a.ep.scale + n0 + j) + __ldg(a.ep.shift + n0 + j);
            v = activate_fast(v, a.ep.activation);
            if (a.ep.round_tf32) v = round_tf32(v);
        }
        out_s[threadIdx.x][j] = v;
    }
    __syncthreads();
    const int live_pix = (int)min((long long)DTHREADS, npix - pix0);
    const int nvalid = min(FB, npg - f0);                  // filters of this slab that exist

    if (a.y_nhwc) {
        // Channels [n0, n0 + cols) of every pixel; the last slab of the last group also writes the zero
        // padding up to cpitch.  16-byte pieces, consecutive threads -> consecutive pieces of a pixel.
        const bool last = grp == g.groups - 1 && f0 + FB >= npg;
        const int cols = last ? min(FB, a.y_cpitch - n0) : nvalid;
        constexpr int EPV = 16 / sizeof(TY);               // elements per 16-byte piece
        if (cols % EPV == 0 && n0 % EPV == 0) {
            const int pieces = cols / EPV;
            TY *base = reinterpret_cast<TY *>(a.y_nhwc) + (size_t)pix0 * a.y_cpitch + n0;
            for (int i = threadIdx.x; i < live_pix * pieces; i += DTHREADS) {
                const int p = i / pieces, q = i - p * pieces;
                const float *src = &out_s[p][q * EPV];
                if (sizeof(TY) == 4) {
                    *reinterpret_cast<float4 *>(base + (size_t)p * a.y_cpitch + q * EPV) = *reinterpret_cast<const float4 *>(src);
                } else {
                    __align__(16) __nv_bfloat16 h[8];
#pragma unroll
                    for (int e = 0; e < 8; ++e) h[e] = __float2bfloat16_rn(src[e]);
                    *reinterpret_cast<uint4 *>(base + (size_t)p * a.y_cpitch + q * EPV) = *reinterpret_cast<uint4 *>(h);
                }
            }
        } else {
            TY *base = reinterpret_cast<TY *>(a.y_nhwc) + (size_t)pix0 * a.y_cpitch + n0;
            for (int i = threadIdx.x; i < live_pix * cols; i += DTHREADS) {
                const int p = i / cols, j = i - p * cols;
                base[(size_t)p * a.y_cpitch + j] = from_float<TY>(out_s[p][j]);
            }
        }
    }
    if (a.y_nchw && live) {
        const size_t plane = (size_t)g.out_h * g.out_w;
        float *dst = a.y_nchw + ((size_t)b * g.n + n0) * plane + (size_t)oh * g.out_w + ow;
        for (int j = 0; j < nvalid; ++j) dst[j * plane] = out_s[threadIdx.x][j];
    }
}

// First-layer specialisation: 3 input channels, 3x3, stride 1, pad 1 (the RGB stems of YOLOv3,
// YOLOv3-tiny and Darknet-19).  Everything is compile-time, so the 36 input values of a thread's two
// neighbouring output pixels are loaded up front (independent loads in flight instead of one
// load-use chain per tap) and every broadcast weight load feeds two FMAs.  256 pixels per block, results
// stored straight from registers.
constexpr int SPIX = 2;                       // output pixels per thread, adjacent in x
constexpr int STHREADS = 128;

template <typename TX, typename TY>
__global__ void __launch_bounds__(STHREADS)
conv_stem3x3_kernel(DirectArgs a)
{
    __shared__ __align__(16) float w_s[27][FB];

    const ConvGeom g = a.g;
    const int f0 = blockIdx.y * FB;
    for (int i = threadIdx.x; i < 27 * FB; i += STHREADS) w_s[i / FB][i % FB] = __ldg(a.wpk + (size_t)(i / FB) * a.npg_pad + f0 + (i % FB));

    // pixel pairs never straddle a row: out_w is padded to even per row by the launcher's grid math
    const int pairs_per_row = (g.out_w + 1) / 2;
    const unsigned npairs = (unsigned)g.batch * g.out_h * pairs_per_row;   // < 2^31, checked by the launcher
    const unsigned pair = blockIdx.x * STHREADS + threadIdx.x;
    const bool live = pair < npairs;
    int b = 0, oh = 0, ow = 0;
    if (live) {
        ow = (int)(pair % pairs_per_row) * 2;
        const unsigned t = pair / pairs_per_row;
        oh = (int)(t % g.out_h);
        b = (int)(t / g.out_h);
    }
    const TX *xb = reinterpret_cast<const TX *>(a.x) + b * a.xs_b;
    float xv[3][3][4];
#pragma unroll
    for (int c = 0; c < 3; ++c)
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int ih = oh + r - 1, iw = ow + q - 1;
                const bool in = live && ih >= 0 && ih < g.h && iw >= 0 && iw < g.w;
                xv[c][r][q] = in ? to_float<TX>(xb[c * a.xs_c + ih * a.xs_h + iw * a.xs_w]) : 0.f;
            }
    __syncthreads();

    float acc0[FB], acc1[FB];
#pragma unroll
    for (int j = 0; j < FB; ++j) { acc0[j] = 0.f; acc1[j] = 0.f; }
#pragma unroll
    for (int c = 0; c < 3; ++c)
#pragma unroll
        for (int r = 0; r < 3; ++r)
#pragma unroll
            for (int q = 0; q < 3; ++q) {
                const float4 *wr = reinterpret_cast<const float4 *>(w_s[(c * 3 + r) * 3 + q]);
                const float x0 = xv[c][r][q], x1 = xv[c][r][q + 1];
#pragma unroll
                for (int v = 0; v < FB / 4; ++v) {
                    const float4 w4 = wr[v];
                    acc0[4 * v + 0] = fmaf(x0, w4.x, acc0[4 * v + 0]); acc1[4 * v + 0] = fmaf(x1, w4.x, acc1[4 * v + 0]);
                    acc0[4 * v + 1] = fmaf(x0, w4.y, acc0[4 * v + 1]); acc1[4 * v + 1] = fmaf(x1, w4.y, acc1[4 * v + 1]);
                    acc0[4 * v + 2] = fmaf(x0, w4.z, acc0[4 * v + 2]); acc1[4 * v + 2] = fmaf(x1, w4.z, acc1[4 * v + 2]);
                    acc0[4 * v + 3] = fmaf(x0, w4.w, acc0[4 * v + 3]); acc1[4 * v + 3] = fmaf(x1, w4.w, acc1[4 * v + 3]);
                }
            }
    // Epilogue straight from registers: every thread owns whole pixels, so a pixel's 32 channels leave as
    // eight 16-byte stores into one 128-byte line (no shared-memory staging, no index arithmetic).
    const int nvalid = min(FB, g.n - f0);
    const int act = a.ep.activation, rnd = a.ep.round_tf32;
#pragma unroll
    for (int j = 0; j < FB; ++j) {
        float v0 = 0.f, v1 = 0.f;
        if (j < nvalid) {
            const float sc = __ldg(a.ep.scale + f0 + j), sh = __ldg(a.ep.shift + f0 + j);
            v0 = activate_fast(acc0[j] * sc + sh, act);
            v1 = activate_fast(acc1[j] * sc + sh, act);
            if (rnd) { v0 = round_tf32(v0); v1 = round_tf32(v1); }
        }
        acc0[j] = v0;
        acc1[j] = v1;
    }
    if (!live) return;
    const bool second = ow + 1 < g.out_w;
    const size_t pix = ((size_t)b * g.out_h + oh) * g.out_w + ow;
    if (a.y_nhwc) {
        // channels [f0, f0 + cols): the last slab also writes the zero padding up to cpitch
        const int cols = (f0 + FB >= g.n) ? min(FB, a.y_cpitch - f0) : nvalid;
        TY *d0 = reinterpret_cast<TY *>(a.y_nhwc) + pix * a.y_cpitch + f0;
        TY *d1 = d0 + a.y_cpitch;
        if (sizeof(TY) == 4) {
#pragma unroll
            for (int q = 0; q < FB / 4; ++q)
                if (4 * q < cols) {      // cpitch is a multiple of 8: whole pieces
                    reinterpret_cast<float4 *>(d0)[q] = make_float4(acc0[4 * q], acc0[4 * q + 1], acc0[4 * q + 2], acc0[4 * q + 3]);
                    if (second) reinterpret_cast<float4 *>(d1)[q] = make_float4(acc1[4 * q], acc1[4 * q + 1], acc1[4 * q + 2], acc1[4 * q + 3]);
                }
        } else {
#pragma unroll
            for (int q = 0; q < FB / 8; ++q)
                if (8 * q < cols) {
                    uint4 p0, p1;
                    __nv_bfloat162 h;
                    h = __floats2bfloat162_rn(acc0[8 * q], acc0[8 * q + 1]); p0.x = *reinterpret_cast<uint32_t *>(&h);
                    h = __floats2bfloat162_rn(acc0[8 * q + 2], acc0[8 * q + 3]); p0.y = *reinterpret_cast<uint32_t *>(&h);
                    h = __floats2bfloat162_rn(acc0[8 * q + 4], acc0[8 * q + 5]); p0.z = *reinterpret_cast<uint32_t *>(&h);
                    h = __floats2bfloat162_rn(acc0[8 * q + 6], acc0[8 * q + 7]); p0.w = *reinterpret_cast<uint32_t *>(&h);
                    h = __floats2bfloat162_rn(acc1[8 * q], acc1[8 * q + 1]); p1.x = *reinterpret_cast<uint32_t *>(&h);
                    h = __floats2bfloat162_rn(acc1[8 * q + 2], acc1[8 * q + 3]); p1.y = *reinterpret_cast<uint32_t *>(&h);
                    h = __floats2bfloat162_rn(acc1[8 * q + 4], acc1[8 * q + 5]); p1.z = *reinterpret_cast<uint32_t *>(&h);
                    h = __floats2bfloat162_rn(acc1[8 * q + 6], acc1[8 * q + 7]); p1.w = *reinterpret_cast<uint32_t *>(&h);
                    reinterpret_cast<uint4 *>(d0)[q] = p0;
                    if (second) reinterpret_cast<uint4 *>(d1)[q] = p1;
                }
        }
    }
    if (a.y_nchw) {
        const size_t plane = (size_t)g.out_h * g.out_w;
        float *dst = a.y_nchw + ((size_t)b * g.n + f0) * plane + (size_t)oh * g.out_w + ow;
#pragma unroll
        for (int j = 0; j < FB; ++j)
            if (j < nvalid) {
                dst[j * plane] = acc0[j];
                if (second) dst[j * plane + 1] = acc1[j];
            }
    }
}

int launch_conv_direct(const DirectArgs &a, cudaStream_t s)
{
    const ConvGeom &g = a.g;
    if (g.size > 15) DNB_FAIL(DNB_EUNSUPPORTED, "direct conv: kernel size %d > 15", g.size);
    const long long npix = (long long)g.batch * g.out_h * g.out_w;
    const int npg = g.n / g.groups;
    dim3 grid((unsigned)((npix + DTHREADS - 1) / DTHREADS), (unsigned)(g.groups * ((npg + FB - 1) / FB)));
    if (grid.y > 65535) DNB_FAIL(DNB_EUNSUPPORTED, "direct conv: too many filter blocks (%u)", grid.y);
    const bool xb = a.x_dtype == DNB_BF16, yb = a.y_dtype == DNB_BF16;
    if (g.c == 3 && g.size == 3 && g.stride == 1 && g.pad == 1 && g.groups == 1 && !xb &&
        (!a.y_nhwc || (a.y_cpitch % 8 == 0))) {
        const long long npairs = (long long)g.batch * g.out_h * ((g.out_w + 1) / 2);
        if (npairs >= (1LL << 31)) DNB_FAIL(DNB_EUNSUPPORTED, "first-layer kernel: %lld pixel pairs", npairs);
        dim3 sgrid((unsigned)((npairs + STHREADS - 1) / STHREADS), (unsigned)((g.n + FB - 1) / FB));
        if (yb) conv_stem3x3_kernel<float, __nv_bfloat16><<<sgrid, STHREADS, 0, s>>>(a);
        else conv_stem3x3_kernel<float, float><<<sgrid, STHREADS, 0, s>>>(a);
        DNB_LAUNCH_CHECK("conv_stem3x3");
        return DNB_OK;
    }
    if (!xb && !yb) conv_direct_kernel<float, float><<<grid, DTHREADS, 0, s>>>(a);
    else if (!xb && yb) conv_direct_kernel<float, __nv_bfloat16><<<grid, DTHREADS, 0, s>>>(a);
    else if (xb && !yb) conv_direct_kernel<__nv_bfloat16, float><<<grid, DTHREADS, 0, s>>>(a);
    else conv_direct_kernel<__nv_bfloat16, __nv_bfloat16><<<grid, DTHREADS, 0, s>>>(a);
    DNB_LAUNCH_CHECK("conv_direct");
    return DNB_OK;
}

}  // namespace dnb
