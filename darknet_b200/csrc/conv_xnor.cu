// XNOR convolution as a bit-packed popcount GEMM.
//
// The reference binarises weights to +-mean|w| and inputs to +-1 and then runs
// the ordinary fp32 im2col + GEMM (src/convolutional_layer.c:451-456, :461-475);
// zero padding is applied after binarisation, so a tap outside the image adds 0.
// With signs packed 32 per word (bit = value > 0) the integer accumulator is
//
//     acc[pixel][n] = sum over in-image taps of ( C - 2 * popc(xbits ^ wbits) )
//
// which is exact.  The layer output is act(bn(mean[n] * acc)).
//
// Integer / bit work on the CUDA cores: a 64 pixel x 64 filter block tile, each
// thread a 4 x 4 micro-tile, operands staged through shared memory one tap and
// up to 32 words at a time; per word pair one LOP3 (xor-and-mask), one POPC, one
// IADD.  Bounded by the POPC issue rate and, for wide layers, by HBM on the
// 32x smaller packed operands; not a tensor-core workload.
#include "common.h"
#include "conv.h"
#include "device_utils.cuh"

namespace dnb {

constexpr int XT = 64;      // pixels per block
constexpr int XN = 64;      // filters per block
constexpr int XW = 32;      // words per staged chunk
constexpr int XTHREADS = 256;

__global__ void __launch_bounds__(XTHREADS)
conv_xnor_kernel(XnorArgs a)
{
    __shared__ uint32_t xs[XW][XT + 1];   // [word][pixel]
    __shared__ uint32_t ws[XW][XN + 1];   // [word][filter]
    __shared__ uint32_t mask_s[XT];       // all-ones where the tap is inside the image
    __shared__ int valid_s[XT];           // in-image taps per pixel

    const ConvGeom &g = a.g;
    const long long npix = (long long)g.batch * g.out_h * g.out_w;
    const long long pix0 = (long long)blockIdx.x * XT;
    const int n0 = blockIdx.y * XN;
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;  // tx: filter quad, ty: pixel quad
    const int taps = g.size * g.size;

    int pop[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) pop[i][j] = 0;

    // the block's 64 pixels are decoded once; the tap loop only adds offsets (-1: beyond the last pixel)
    __shared__ int pb_s[XT], poh_s[XT], pow_s[XT];
    if (threadIdx.x < XT) {
        valid_s[threadIdx.x] = 0;
        const long long pix = pix0 + threadIdx.x;
        int b = -1, oh = 0, ow = 0;
        if (pix < npix) {
            ow = (int)(pix % g.out_w);
            const long long t = pix / g.out_w;
            oh = (int)(t % g.out_h);
            b = (int)(t / g.out_h);
        }
        pb_s[threadIdx.x] = b; poh_s[threadIdx.x] = oh; pow_s[threadIdx.x] = ow;
    }

    for (int tap = 0; tap < taps; ++tap) {
        const int kh = tap / g.size, kw = tap - kh * g.size;
        for (int w0 = 0; w0 < a.cwords; w0 += XW) {
            const int wn = min(XW, a.cwords - w0);
            __syncthreads();
            if (threadIdx.x < XT) {   // is this tap inside the image for pixel p?
                const int p = threadIdx.x;
                const int ih = poh_s[p] * g.stride + kh - g.pad, iw = pow_s[p] * g.stride + kw - g.pad;
                const bool inside = pb_s[p] >= 0 && ih >= 0 && ih < g.h && iw >= 0 && iw < g.w;
                mask_s[p] = inside ? 0xffffffffu : 0u;
                if (w0 == 0 && inside) valid_s[p] += 1;
            }
            // stage the wn input words of this tap for every pixel: (pixel, word) pairs, words fastest so that
            // the loads of a warp are contiguous; layers with few words per pixel touch only those
            for (int i = threadIdx.x; i < XT * wn; i += XTHREADS) {
                const int p = i / wn, w = i - p * wn;
                const int ih = poh_s[p] * g.stride + kh - g.pad, iw = pow_s[p] * g.stride + kw - g.pad;
                uint32_t v = 0;
                if (pb_s[p] >= 0 && ih >= 0 && ih < g.h && iw >= 0 && iw < g.w)
                    v = __ldg(a.xbits + (((size_t)pb_s[p] * g.h + ih) * g.w + iw) * a.cwords + w0 + w);
                xs[w][p] = v;
            }
            for (int i = threadIdx.x; i < XN * wn; i += XTHREADS) {
                const int f = i / wn, w = i - f * wn;
                const int n = n0 + f;
                ws[w][f] = n < g.n ? __ldg(a.wbits + ((size_t)n * taps + tap) * a.cwords + w0 + w) : 0u;
            }
            __syncthreads();
            uint32_t m[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) m[i] = mask_s[ty * 4 + i];
            for (int w = 0; w < wn; ++w) {
                uint32_t xv[4], wv[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) xv[i] = xs[w][ty * 4 + i];
#pragma unroll
                for (int j = 0; j < 4; ++j) wv[j] = ws[w][tx * 4 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) pop[i][j] += __popc((xv[i] ^ wv[j]) & m[i]);
            }
        }
    }
    __syncthreads();

    const size_t plane = (size_t)g.out_h * g.out_w;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const long long pix = pix0 + ty * 4 + i;
        if (pix >= npix) continue;
        const int ow = (int)(pix % g.out_w);
        const long long t = pix / g.out_w;
        const int oh = (int)(t % g.out_h), b = (int)(t / g.out_h);
        const int base = valid_s[ty * 4 + i] * g.c;
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            const int acc = base - 2 * pop[i][j];
            v[j] = 0.f;
            if (n < g.n) {
                if (a.acc_out) a.acc_out[((size_t)b * g.n + n) * plane + (size_t)oh * g.out_w + ow] = acc;
                float r = (float)acc * __ldg(a.wmean + n);
                r = r * __ldg(a.ep.scale + n) + __ldg(a.ep.shift + n);
                v[j] = activate(r, a.ep.activation);
                if (a.y_nchw) a.y_nchw[((size_t)b * g.n + n) * plane + (size_t)oh * g.out_w + ow] = v[j];
            }
        }
        const int nq = n0 + tx * 4;
        if (a.y_nhwc && nq + 4 <= a.y_cpitch) {
            if (a.y_dtype == DNB_F32) {
                *reinterpret_cast<float4 *>(reinterpret_cast<float *>(a.y_nhwc) + (size_t)pix * a.y_cpitch + nq) = make_float4(v[0], v[1], v[2], v[3]);
            } else {
                __align__(8) __nv_bfloat16 h[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __float2bfloat16_rn(v[j]);
                *reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(a.y_nhwc) + (size_t)pix * a.y_cpitch + nq) = *reinterpret_cast<uint2 *>(h);
            }
        }
    }
}

int launch_conv_xnor(const XnorArgs &a, cudaStream_t s)
{
    const ConvGeom &g = a.g;
    const long long npix = (long long)g.batch * g.out_h * g.out_w;
    dim3 grid((unsigned)((npix + XT - 1) / XT), (unsigned)((round_up(g.n, 8) + XN - 1) / XN));
    conv_xnor_kernel<<<grid, XTHREADS, 0, s>>>(a);
    DNB_LAUNCH_CHECK("conv_xnor");
    return DNB_OK;
}

// ------------------------------------------------------------------ sign-bit packing
// NHWC: eight lanes per (pixel, word), four channels (one 16-byte or 8-byte load) per lane, so a warp packs four
// words per iteration from 512 contiguous bytes; the eight nibbles are OR-ed together with three shuffles.
// Padding channels hold zeros (the channels-last contract), so they pack as "not positive" by themselves.
template <typename T>
__global__ void __launch_bounds__(256)
pack_bits_nhwc_kernel(const T *__restrict__ x, uint32_t *__restrict__ bits, size_t npix, int C, int Cp, int cwords)
{
    const int lane = threadIdx.x & 31, sub = lane >> 3, q = lane & 7;
    const size_t warp0 = (blockIdx.x * (size_t)blockDim.x + threadIdx.x) >> 5;
    const size_t nwarps = ((size_t)gridDim.x * blockDim.x) >> 5;
    const size_t total = npix * cwords;
    (void)C;
    for (size_t base = warp0 * 4; base < total; base += nwarps * 4) {
        const size_t item = base + sub;
        uint32_t nib = 0;
        if (item < total) {
            const size_t p = item / cwords;
            const int w = (int)(item - p * cwords), c0 = w * 32 + q * 4;
            if (c0 < Cp) {   // the pitch is a multiple of 8: a 4-channel piece is inside it or outside
                float v0, v1, v2, v3;
                if (sizeof(T) == 4) {
                    const float4 f = __ldg(reinterpret_cast<const float4 *>(x + p * Cp + c0));
                    v0 = f.x; v1 = f.y; v2 = f.z; v3 = f.w;
                } else {
                    const uint2 u = __ldg(reinterpret_cast<const uint2 *>(x + p * Cp + c0));
                    v0 = __uint_as_float(u.x << 16); v1 = __uint_as_float(u.x & 0xffff0000u);
                    v2 = __uint_as_float(u.y << 16); v3 = __uint_as_float(u.y & 0xffff0000u);
                }
                nib = (v0 > 0.f ? 1u : 0u) | (v1 > 0.f ? 2u : 0u) | (v2 > 0.f ? 4u : 0u) | (v3 > 0.f ? 8u : 0u);
            }
        }
        uint32_t word = nib << (4 * q);
        word |= __shfl_xor_sync(0xffffffffu, word, 1);
        word |= __shfl_xor_sync(0xffffffffu, word, 2);
        word |= __shfl_xor_sync(0xffffffffu, word, 4);
        if (q == 0 && item < total) bits[item] = word;
    }
}

// NCHW: one thread per (pixel, word): 32 strided loads, coalesced across the warp.
__global__ void pack_bits_nchw_kernel(const float *__restrict__ x, uint32_t *__restrict__ bits, int B, int C, size_t HW, int cwords)
{
    const size_t total = (size_t)B * HW * cwords;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const size_t hw = i % HW;
        const size_t t = i / HW;
        const int w = (int)(t % cwords), b = (int)(t / cwords);
        uint32_t word = 0;
        for (int k = 0; k < 32; ++k) {
            const int c = w * 32 + k;
            if (c < C && __ldg(x + ((size_t)b * C + c) * HW + hw) > 0.f) word |= 1u << k;
        }
        bits[((size_t)b * HW + hw) * cwords + w] = word;
    }
}

int launch_pack_sign_bits(const dnb_tensor *x, uint32_t *bits, int cwords, cudaStream_t s)
{
    const size_t npix = (size_t)x->n * x->h * x->w;
    if (x->layout == DNB_NHWC) {
        size_t warps = (npix * cwords + 3) / 4;   // four words per warp iteration
        size_t blocks = (warps * 32 + 255) / 256;
        size_t cap = (size_t)sm_count() * 8;
        int grid = (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
        if (x->dtype == DNB_F32) pack_bits_nhwc_kernel<float><<<grid, 256, 0, s>>>((const float *)x->data, bits, npix, x->c, x->cpitch, cwords);
        else pack_bits_nhwc_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16 *)x->data, bits, npix, x->c, x->cpitch, cwords);
    } else {
        size_t total = npix * cwords;
        size_t blocks = (total + 255) / 256;
        size_t cap = (size_t)sm_count() * 8;
        int grid = (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
        pack_bits_nchw_kernel<<<grid, 256, 0, s>>>((const float *)x->data, bits, x->n, x->c, (size_t)x->h * x->w, cwords);
    }
    DNB_LAUNCH_CHECK("pack_sign_bits");
    return DNB_OK;
}

// ------------------------------------------------------------------ int8 signs for the tensor-core xnor convolution
// One thread per (pixel, group of 16 channels): +1 where x > 0, -1 elsewhere (the CPU reference's test, so 0 maps to -1),
// 0 for channels beyond the layer's (they must add nothing to the sums); 16 bytes written per thread.
template <typename T, bool NCHW>
__global__ void __launch_bounds__(256)
pack_sign_i8_kernel(const T *__restrict__ x, int8_t *__restrict__ out, size_t npix, size_t HW, int C, int Cp_in, int cpad)
{
    const int groups = cpad / 16;
    const size_t total = npix * groups;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t p;
        int gq;
        if (NCHW) { p = i % npix; gq = (int)(i / npix); }      // consecutive threads: consecutive pixels of one channel group
        else { p = i / groups; gq = (int)(i - p * groups); }   // consecutive threads: consecutive groups of one pixel
        const int c0 = gq * 16;
        uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
        for (int k = 0; k < 16; ++k) {
            const int c = c0 + k;
            float v = 0.f;
            bool in = c < C;
            if (in) {
                if (NCHW) {
                    const size_t b = p / HW, hw = p - b * HW;
                    v = __ldg(reinterpret_cast<const float *>(x) + (b * C + c) * HW + hw);
                } else if (sizeof(T) == 4) {
                    v = __ldg(reinterpret_cast<const float *>(x) + p * Cp_in + c);
                } else {
                    v = __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(x)[p * Cp_in + c]);
                }
            }
            const uint32_t byte = in ? (v > 0.f ? 0x01u : 0xffu) : 0u;
            w[k >> 2] |= byte << (8 * (k & 3));
        }
        *reinterpret_cast<uint4 *>(out + p * cpad + c0) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

int launch_pack_sign_i8(const dnb_tensor *x, int8_t *out, int cpad, cudaStream_t s)
{
    const size_t npix = (size_t)x->n * x->h * x->w, HW = (size_t)x->h * x->w;
    const size_t total = npix * (cpad / 16);
    const size_t blocks = (total + 255) / 256, cap = (size_t)sm_count() * 16;
    const int grid = (int)(blocks < cap ? (blocks ? blocks : 1) : cap);
    if (x->layout == DNB_NCHW) pack_sign_i8_kernel<float, true><<<grid, 256, 0, s>>>((const float *)x->data, out, npix, HW, x->c, 0, cpad);
    else if (x->dtype == DNB_F32) pack_sign_i8_kernel<float, false><<<grid, 256, 0, s>>>((const float *)x->data, out, npix, HW, x->c, x->cpitch, cpad);
    else pack_sign_i8_kernel<__nv_bfloat16, false><<<grid, 256, 0, s>>>((const __nv_bfloat16 *)x->data, out, npix, HW, x->c, x->cpitch, cpad);
    DNB_LAUNCH_CHECK("pack_sign_i8");
    return DNB_OK;
}

}  // namespace dnb

// ------------------------------------------------------------------ entry point that allocates nothing
// Some callers may not allocate device memory at all while they run: code that executes inside a
// latency-critical serving loop whose memory was carved out up front, a host process that handed the
// whole device to an arena allocator of its own, or a plug-in loaded into a process whose owner forbids
// cudaMalloc after start-up.  For them the xnor convolution, which needs scratch for the bit-packed
// input, is also available with that scratch inside the library image: a fixed array in device memory
// that every GPU loading the library holds until the process exits.
namespace dnb {
constexpr size_t kXnorStaticWords = (size_t)1 << 20;   // 4 MiB: batch*h*w*ceil(c/32) may not exceed this
static __device__ __align__(256) uint32_t g_xnor_static_bits[kXnorStaticWords];
// In host code the array's name is only a handle for the runtime, not a device address: the address is
// looked up once per device (with that device current) and cached here.
static uint32_t *g_xnor_static_ptr[64];
}  // namespace dnb

extern "C" int dnb_conv_xnor_forward_static(const dnb_conv_desc *d, const dnb_tensor *x, const uint32_t *wbits,
                                            const float *wmean, const float *scale, const float *shift,
                                            const dnb_tensor *y, void *stream)
{
    using namespace dnb;
    if (!d || !x || !wbits || !wmean || !scale || !shift || !y) DNB_FAIL(DNB_EINVAL, "xnor static: null argument");
    if (d->batch < 1 || d->h < 1 || d->w < 1 || d->c < 1 || d->n < 1 || d->size < 1 || d->size > 15 || d->stride < 1 || d->pad < 0 ||
        d->groups != 1)
        DNB_FAIL(DNB_EINVAL, "xnor static: bad geometry (groups must be 1)");
    if (d->activation < 0 || d->activation > DNB_SELU) DNB_FAIL(DNB_EINVAL, "xnor static: activation %d", d->activation);
    const int out_h = (d->h + 2 * d->pad - d->size) / d->stride + 1, out_w = (d->w + 2 * d->pad - d->size) / d->stride + 1;
    if (out_h < 1 || out_w < 1) DNB_FAIL(DNB_EINVAL, "xnor static: empty output");
    DNB_TRY(check_tensor(x, "xnor static input"));
    DNB_TRY(check_tensor(y, "xnor static output"));
    if (x->n != d->batch || x->c != d->c || x->h != d->h || x->w != d->w) DNB_FAIL(DNB_EINVAL, "xnor static: input extents differ from the descriptor");
    if (y->n != d->batch || y->c != d->n || y->h != out_h || y->w != out_w) DNB_FAIL(DNB_EINVAL, "xnor static: output extents differ from the descriptor");
    const int cwords = (d->c + 31) / 32;
    const size_t words = (size_t)d->batch * d->h * d->w * cwords;
    if (words > kXnorStaticWords)
        DNB_FAIL(DNB_EINVAL, "xnor static: the packed input needs %zu words, the built-in scratch holds %zu (batch*h*w*ceil(c/32) <= 2^20); "
                 "use a plan (dnb_conv_plan_create) for larger layers", words, kXnorStaticWords);
    int dev = 0;
    DNB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) DNB_FAIL(DNB_EINVAL, "xnor static: device ordinal %d", dev);
    if (!g_xnor_static_ptr[dev]) {   // set-up: first call on this device
        uint32_t *ptr = nullptr;
        DNB_CUDA(cudaGetSymbolAddress((void **)&ptr, g_xnor_static_bits));
        if (!ptr) DNB_FAIL(DNB_ECUDA, "xnor static: the scratch array has no address on device %d", dev);
        g_xnor_static_ptr[dev] = ptr;
    }
    uint32_t *bits = g_xnor_static_ptr[dev];
    cudaStream_t s = (cudaStream_t)stream;
    // every word the convolution reads is rewritten by the packing pass, so nothing has to be cleared
    DNB_TRY(launch_pack_sign_bits(x, bits, cwords, s));
    XnorArgs a;
    a.xbits = bits; a.wbits = wbits; a.cwords = cwords; a.wmean = wmean; a.acc_out = nullptr;
    a.y_nhwc = y->layout == DNB_NHWC ? y->data : nullptr;
    a.y_dtype = y->dtype; a.y_cpitch = y->cpitch;
    a.y_nchw = y->layout == DNB_NCHW ? (float *)y->data : nullptr;
    a.g = ConvGeom{d->batch, d->h, d->w, d->c, d->n, 1, d->size, d->stride, d->pad, out_h, out_w};
    a.ep = ConvEpilogue{scale, shift, d->activation, 0};
    return launch_conv_xnor(a, s);
}
