// HBM-bound layers of the forward path: maxpool, upsample, shortcut, route,
// layout conversion (+ YOLO head), global average pool, softmax.
//
// All of them move each byte once with 16-byte vector accesses along the contiguous
// axis (channels for NHWC, width for NCHW).  The channels-last maxpool, upsample and
// general shortcut walk one output row per block iteration, so that the per-element
// index arithmetic is one 32-bit division and all loads of an element's window are in
// flight together (a rolled window loop and 64-bit divisions per vector held the
// maxpool at 58 % of the HBM copy rate; it runs at 97-100 % now).  The flat kernels
// (equal-shape shortcut, route copies, conversions) use grid-stride loops over a
// grid that is a multiple of the SM count.  None of them is GEMM-shaped.
#include "common.h"
#include "device_utils.cuh"

namespace dnb {

static inline int grid_for(size_t work_items, int threads)
{
    size_t blocks = (work_items + threads - 1) / threads;
    size_t cap = (size_t)sm_count() * 16;  // 16 resident CTAs of 128 threads per SM
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

// Grid of the row-wise kernels: one block per output row, at most 8 resident blocks of 256 threads per SM.
static inline int row_grid(int batch, int rows_per_image)
{
    const long long rows = (long long)batch * rows_per_image;
    const long long cap = (long long)sm_count() * 8;
    return (int)(rows < cap ? (rows > 0 ? rows : 1) : cap);
}

// 16-byte vector of T with elementwise helpers.
template <typename T> struct Vec16 {
    static constexpr int N = 16 / sizeof(T);
    union { uint4 raw; T v[N]; };
};

// ------------------------------------------------------------------ maxpool
// Darknet semantics (src/maxpool_layer.c:79-114): window origin -padding/2,
// taps outside the image skipped, -FLT_MAX if none is inside.
// One output row (b, oh) per block iteration, threads along the row's (ow, channel vector) pairs: the only
// per-element index arithmetic is one 32-bit division (64-bit divisions per 16-byte vector made this kernel
// instruction-bound at 58 % of the HBM rate).
// SIZE: the window's extent at compile time (2, 3) so that all of a window's loads are in flight together (a
// rolled loop issues load, compare, load, compare, ... and each thread then has one load in flight), or 0 for
// any size at run time.
template <typename T, int SIZE>
__global__ void __launch_bounds__(256)
maxpool_nhwc_kernel(const T *__restrict__ x, T *__restrict__ y, int B, int H, int W, int cvecs,
                    int OH, int OW, int size_rt, int stride, int off, int8_t *__restrict__ signs, int spitch)
{
    // signs (f32 tensors only): also write the signs of the output (+1 where > 0, else -1) as an int8 channels-last
    // tensor of pitch spitch, the operand of the tensor-core xnor layer that follows; every channel is a real one there
    using V = Vec16<T>;
    const int size = SIZE > 0 ? SIZE : size_rt;
    const int rows = B * OH, row_vecs = OW * cvecs;
    const uint4 *xin = reinterpret_cast<const uint4 *>(x);
    uint4 *yout = reinterpret_cast<uint4 *>(y);
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const int b = row / OH, oh = row - b * OH;
        const int ih0 = off + oh * stride;
        const size_t in_img = (size_t)b * H * W * cvecs;
        uint4 *yrow = yout + (size_t)row * row_vecs;
        for (int j = threadIdx.x; j < row_vecs; j += blockDim.x) {
            const int ow = j / cvecs, cv = j - ow * cvecs;
            const int iw0 = off + ow * stride;
            float best[V::N];
#pragma unroll
            for (int k = 0; k < V::N; ++k) best[k] = -FLT_MAX;
            if (SIZE > 0) {
                constexpr int WIN = SIZE > 0 ? SIZE * SIZE : 1;
                V v[WIN];
                bool in[WIN];
#pragma unroll
                for (int n = 0; n < SIZE; ++n)
#pragma unroll
                    for (int m = 0; m < SIZE; ++m) {
                        const int ih = ih0 + n, iw = iw0 + m;
                        in[n * SIZE + m] = ih >= 0 && ih < H && iw >= 0 && iw < W;
                        if (in[n * SIZE + m]) v[n * SIZE + m].raw = __ldg(xin + in_img + ((size_t)ih * W + iw) * cvecs + cv);
                    }
#pragma unroll
                for (int t = 0; t < WIN; ++t)
                    if (in[t]) {
#pragma unroll
                        for (int k = 0; k < V::N; ++k) best[k] = fmaxf(best[k], to_float<T>(v[t].v[k]));
                    }
            } else
            for (int n = 0; n < size; ++n) {
                const int ih = ih0 + n;
                if (ih < 0 || ih >= H) continue;
                const uint4 *xrow = xin + in_img + (size_t)ih * W * cvecs + cv;
                for (int m = 0; m < size; ++m) {
                    const int iw = iw0 + m;
                    if (iw < 0 || iw >= W) continue;
                    V v;
                    v.raw = __ldg(xrow + iw * cvecs);
#pragma unroll
                    for (int k = 0; k < V::N; ++k) best[k] = fmaxf(best[k], to_float<T>(v.v[k]));
                }
            }
            V o;
#pragma unroll
            for (int k = 0; k < V::N; ++k) o.v[k] = from_float<T>(best[k]);
            yrow[j] = o.raw;
            if (V::N == 4 && signs) {
                const uint32_t sg = (best[0] > 0.f ? 0x01u : 0xFFu) | (best[1] > 0.f ? 0x0100u : 0xFF00u) |
                                    (best[2] > 0.f ? 0x010000u : 0xFF0000u) | (best[V::N - 1] > 0.f ? 0x01000000u : 0xFF000000u);
                *reinterpret_cast<uint32_t *>(signs + ((size_t)row * OW + ow) * spitch + 4 * cv) = sg;
            }
        }
    }
}

__global__ void maxpool_nchw_kernel(const float *__restrict__ x, float *__restrict__ y, int planes, int H, int W,
                                    int OH, int OW, int size, int stride, int off)
{
    const size_t total = (size_t)planes * OH * OW;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        int ow = (int)(i % OW);
        size_t p = i / OW;
        int oh = (int)(p % OH);
        size_t plane = p / OH;
        const float *src = x + plane * H * W;
        float best = -FLT_MAX;
        for (int n = 0; n < size; ++n) {
            int ih = off + oh * stride + n;
            if (ih < 0 || ih >= H) continue;
            for (int m = 0; m < size; ++m) {
                int iw = off + ow * stride + m;
                if (iw < 0 || iw >= W) continue;
                best = fmaxf(best, __ldg(src + (size_t)ih * W + iw));
            }
        }
        y[i] = best;
    }
}

int launch_maxpool(const dnb_tensor *x, const dnb_tensor *y, int size, int stride, int padding, cudaStream_t s, int8_t *signs, int spitch)
{
    DNB_TRY(check_tensor(x, "maxpool input"));
    DNB_TRY(check_tensor(y, "maxpool output"));
    if (size < 1 || stride < 1 || padding < 0) DNB_FAIL(DNB_EINVAL, "maxpool: bad size/stride/padding %d/%d/%d", size, stride, padding);
    const int oh = (x->h + padding - size) / stride + 1, ow = (x->w + padding - size) / stride + 1;
    if (y->h != oh || y->w != ow || y->c != x->c || y->n != x->n)
        DNB_FAIL(DNB_EINVAL, "maxpool: output is %dx%dx%dx%d, expected %dx%dx%dx%d", y->n, y->c, y->h, y->w, x->n, x->c, oh, ow);
    if (x->layout != y->layout || x->dtype != y->dtype) DNB_FAIL(DNB_EINVAL, "maxpool: input and output differ in layout or dtype");
    const int off = -(padding / 2);
#define MAXPOOL_LAUNCH(T, ...)                                                                          \
    do {                                                                                                \
        if (size == 2) maxpool_nhwc_kernel<T, 2><<<row_grid(y->n, oh), 256, 0, s>>>(__VA_ARGS__);       \
        else if (size == 3) maxpool_nhwc_kernel<T, 3><<<row_grid(y->n, oh), 256, 0, s>>>(__VA_ARGS__);  \
        else maxpool_nhwc_kernel<T, 0><<<row_grid(y->n, oh), 256, 0, s>>>(__VA_ARGS__);                 \
    } while (0)
    if (x->layout == DNB_NHWC) {
        if (x->cpitch != y->cpitch) DNB_FAIL(DNB_EINVAL, "maxpool: cpitch differs (%d vs %d)", x->cpitch, y->cpitch);
        if (x->dtype == DNB_F32) {
            int cv = x->cpitch / 4;
            if (signs && (x->c % 32 || x->cpitch != x->c || spitch < x->c)) DNB_FAIL(DNB_EINVAL, "maxpool: the sign output needs a multiple of 32 channels, unpadded");
            MAXPOOL_LAUNCH(float, (const float *)x->data, (float *)y->data, x->n, x->h, x->w, cv, oh, ow, size, stride, off, signs, spitch);
        } else {
            int cv = x->cpitch / 8;
            if (signs) DNB_FAIL(DNB_EINVAL, "maxpool: the sign output is built for f32 tensors");
            MAXPOOL_LAUNCH(__nv_bfloat16, (const __nv_bfloat16 *)x->data, (__nv_bfloat16 *)y->data, x->n, x->h, x->w, cv, oh, ow, size, stride, off, nullptr, 0);
        }
    } else {
        if (x->dtype != DNB_F32) DNB_FAIL(DNB_EINVAL, "maxpool: NCHW tensors must be f32");
        if (signs) DNB_FAIL(DNB_EINVAL, "maxpool: the sign output is built for channels-last tensors");
        size_t total = (size_t)y->n * y->c * oh * ow;
        maxpool_nchw_kernel<<<grid_for(total, 128), 128, 0, s>>>((const float *)x->data, (float *)y->data, x->n * x->c, x->h, x->w, oh, ow, size, stride, off);
    }
#undef MAXPOOL_LAUNCH
    DNB_LAUNCH_CHECK("maxpool");
    return DNB_OK;
}

// ------------------------------------------------------------------ upsample
// One output row (b, oh) per block iteration; see maxpool_nhwc_kernel.
template <typename T>
__global__ void __launch_bounds__(256)
upsample_nhwc_kernel(const T *__restrict__ x, T *__restrict__ y, int B, int H, int W, int cvecs, int xpitch_vecs, int ypitch_vecs,
                     int stride, float scale)
{
    // cvecs 16-byte vectors of channels per pixel are copied; input and output pixels may be further apart than that
    // (a tensor that is a channel range of a wider one, e.g. the slice of a [route] output it was placed in)
    using V = Vec16<T>;
    const int OH = H * stride, OW = W * stride;
    const int rows = B * OH, row_vecs = OW * cvecs;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const int b = row / OH, oh = row - b * OH;
        const uint4 *xrow = reinterpret_cast<const uint4 *>(x) + ((size_t)b * H + oh / stride) * W * xpitch_vecs;
        uint4 *yrow = reinterpret_cast<uint4 *>(y) + (size_t)row * OW * ypitch_vecs;
#pragma unroll 4
        for (int j = threadIdx.x; j < row_vecs; j += blockDim.x) {
            const int ow = j / cvecs, cv = j - ow * cvecs;
            V v;
            v.raw = __ldg(xrow + (ow / stride) * xpitch_vecs + cv);
            if (scale != 1.f) {
#pragma unroll
                for (int k = 0; k < V::N; ++k) v.v[k] = from_float<T>(scale * to_float<T>(v.v[k]));
            }
            yrow[ow * ypitch_vecs + cv] = v.raw;
        }
    }
}

__global__ void upsample_nchw_kernel(const float *__restrict__ x, float *__restrict__ y, int planes, int H, int W,
                                     int stride, float scale)
{
    const int OH = H * stride, OW = W * stride;
    const size_t total = (size_t)planes * OH * OW;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        int ow = (int)(i % OW);
        size_t p = i / OW;
        int oh = (int)(p % OH);
        size_t plane = p / OH;
        y[i] = scale * __ldg(x + (plane * H + oh / stride) * W + ow / stride);
    }
}

int launch_upsample(const dnb_tensor *x, const dnb_tensor *y, int stride, float scale, cudaStream_t s)
{
    DNB_TRY(check_tensor(x, "upsample input"));
    DNB_TRY(check_tensor(y, "upsample output"));
    if (stride < 1) DNB_FAIL(DNB_EUNSUPPORTED, "upsample: stride %d (the reverse/downsample form is not on the forward path)", stride);
    if (y->h != x->h * stride || y->w != x->w * stride || y->c != x->c || y->n != x->n)
        DNB_FAIL(DNB_EINVAL, "upsample: output extents do not match input x%d", stride);
    if (x->layout != y->layout || x->dtype != y->dtype) DNB_FAIL(DNB_EINVAL, "upsample: input and output differ in layout or dtype");
    if (x->layout == DNB_NHWC) {
        // the channels copied per pixel: the narrower of the two pitches (equal pitches: all of them, padding included)
        const int per = x->dtype == DNB_F32 ? 4 : 8;
        const int cv = (x->cpitch < y->cpitch ? x->cpitch : y->cpitch) / per;
        if (cv * per < x->c || x->cpitch % per || y->cpitch % per) DNB_FAIL(DNB_EINVAL, "upsample: channel pitches %d and %d for %d channels", x->cpitch, y->cpitch, x->c);
        if (x->dtype == DNB_F32) {
            upsample_nhwc_kernel<float><<<row_grid(y->n, y->h), 256, 0, s>>>((const float *)x->data, (float *)y->data, x->n, x->h, x->w, cv, x->cpitch / per,
                                                                            y->cpitch / per, stride, scale);
        } else {
            upsample_nhwc_kernel<__nv_bfloat16><<<row_grid(y->n, y->h), 256, 0, s>>>((const __nv_bfloat16 *)x->data, (__nv_bfloat16 *)y->data, x->n, x->h, x->w,
                                                                                    cv, x->cpitch / per, y->cpitch / per, stride, scale);
        }
    } else {
        if (x->dtype != DNB_F32) DNB_FAIL(DNB_EINVAL, "upsample: NCHW tensors must be f32");
        size_t total = (size_t)y->n * y->c * y->h * y->w;
        upsample_nchw_kernel<<<grid_for(total, 128), 128, 0, s>>>((const float *)x->data, (float *)y->data, x->n * x->c, x->h, x->w, stride, scale);
    }
    DNB_LAUNCH_CHECK("upsample");
    return DNB_OK;
}

// ------------------------------------------------------------------ shortcut
// Equal shapes: y = act(alpha*x + beta*add), flat over 16-byte vectors.
template <typename T>
__global__ void shortcut_flat_kernel(const T *__restrict__ x, const T *__restrict__ add, T *__restrict__ y,
                                     size_t nvec, float alpha, float beta, int act)
{
    using V = Vec16<T>;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < nvec; i += (size_t)gridDim.x * blockDim.x) {
        V a, b, o;
        a.raw = __ldg(reinterpret_cast<const uint4 *>(x) + i);
        b.raw = __ldg(reinterpret_cast<const uint4 *>(add) + i);
#pragma unroll
        for (int k = 0; k < V::N; ++k)
            o.v[k] = from_float<T>(activate(alpha * to_float<T>(a.v[k]) + beta * to_float<T>(b.v[k]), act));
        reinterpret_cast<uint4 *>(y)[i] = o.raw;
    }
}

// General shapes (src/blas.c:68-92): the add tensor may be wider/narrower or
// have more/fewer channels.  One thread per output element; element strides
// describe either layout.
struct ShortcutGeom {
    int B, C2, H2, W2;                    // output (= x) extents
    int minc, minh, minw, stride, sample;
    long long xs_b, xs_c, xs_h, xs_w;     // x / y element strides
    long long as_b, as_c, as_h, as_w;     // add element strides
    int inner_is_c;                       // 1: iterate c fastest (NHWC)
};

template <typename T>
__global__ void shortcut_general_kernel(const T *__restrict__ x, const T *__restrict__ add, T *__restrict__ y,
                                        ShortcutGeom g, float alpha, float beta, int act)
{
    const size_t total = (size_t)g.B * g.C2 * g.H2 * g.W2;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        int b, c, h, w;
        size_t p = i;
        if (g.inner_is_c) {
            c = (int)(p % g.C2); p /= g.C2; w = (int)(p % g.W2); p /= g.W2; h = (int)(p % g.H2); b = (int)(p / g.H2);
        } else {
            w = (int)(p % g.W2); p /= g.W2; h = (int)(p % g.H2); p /= g.H2; c = (int)(p % g.C2); b = (int)(p / g.C2);
        }
        const long long xi = b * g.xs_b + c * g.xs_c + h * g.xs_h + w * g.xs_w;
        float v = to_float<T>(x[xi]);
        if (c < g.minc && h % g.sample == 0 && w % g.sample == 0 && h / g.sample < g.minh && w / g.sample < g.minw) {
            const long long ai = b * g.as_b + c * g.as_c + (long long)(h / g.sample) * g.stride * g.as_h +
                                 (long long)(w / g.sample) * g.stride * g.as_w;
            v = alpha * v + beta * to_float<T>(add[ai]);
        }
        y[xi] = from_float<T>(activate(v, act));
    }
}

// General shapes, channels-last: one output row (b, h) per block iteration, threads along the row's (w, 16-byte
// channel vector) pairs.  The add tensor contributes where the reference's loops reach (src/blas.c:68-92): channels
// below minc, and pixels (h, w) that are multiples of `sample`, read from (h/sample*stride, w/sample*stride).
template <typename T>
__global__ void __launch_bounds__(256)
shortcut_rows_nhwc_kernel(const T *__restrict__ x, const T *__restrict__ add, T *__restrict__ y, ShortcutGeom g,
                          int cpitch, int add_cpitch, int add_h, int add_w, float alpha, float beta, int act)
{
    using V = Vec16<T>;
    const int cvecs = cpitch / V::N, rows = g.B * g.H2, row_vecs = g.W2 * cvecs;
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const int b = row / g.H2, h = row - b * g.H2;
        const bool h_hit = h % g.sample == 0 && h / g.sample < g.minh;
        const T *arow = add + ((size_t)b * add_h + (size_t)(h / g.sample) * g.stride) * add_w * add_cpitch;
        const uint4 *xrow = reinterpret_cast<const uint4 *>(x) + (size_t)row * row_vecs;
        uint4 *yrow = reinterpret_cast<uint4 *>(y) + (size_t)row * row_vecs;
        for (int j = threadIdx.x; j < row_vecs; j += blockDim.x) {
            const int w = j / cvecs, c0 = (j - w * cvecs) * V::N;
            V a, o;
            a.raw = __ldg(xrow + j);
            const bool hit = h_hit && c0 < g.minc && w % g.sample == 0 && w / g.sample < g.minw;
            float r[V::N];
#pragma unroll
            for (int k = 0; k < V::N; ++k) r[k] = to_float<T>(a.v[k]);
            if (hit) {
                const T *ap = arow + (size_t)(w / g.sample) * g.stride * add_cpitch + c0;
                if (c0 + V::N <= g.minc) {          // the whole vector lies inside both tensors (pitches are multiples of 8)
                    V d;
                    d.raw = __ldg(reinterpret_cast<const uint4 *>(ap));
#pragma unroll
                    for (int k = 0; k < V::N; ++k) r[k] = alpha * r[k] + beta * to_float<T>(d.v[k]);
                } else {
#pragma unroll
                    for (int k = 0; k < V::N; ++k)
                        if (c0 + k < g.minc) r[k] = alpha * r[k] + beta * to_float<T>(ap[k]);
                }
            }
#pragma unroll
            for (int k = 0; k < V::N; ++k) o.v[k] = from_float<T>(c0 + k < g.C2 ? activate(r[k], act) : 0.f);   // padding channels stay zero
            yrow[j] = o.raw;
        }
    }
}

int launch_shortcut(const dnb_tensor *x, const dnb_tensor *add, const dnb_tensor *y, float alpha, float beta,
                    int activation, cudaStream_t s)
{
    DNB_TRY(check_tensor(x, "shortcut input"));
    DNB_TRY(check_tensor(add, "shortcut add"));
    DNB_TRY(check_tensor(y, "shortcut output"));
    if (x->layout != y->layout || x->layout != add->layout || x->dtype != y->dtype || x->dtype != add->dtype)
        DNB_FAIL(DNB_EINVAL, "shortcut: tensors differ in layout or dtype");
    if (x->n != y->n || x->c != y->c || x->h != y->h || x->w != y->w || add->n != x->n)
        DNB_FAIL(DNB_EINVAL, "shortcut: input and output extents differ");
    if (x->layout == DNB_NHWC && x->cpitch != y->cpitch) DNB_FAIL(DNB_EINVAL, "shortcut: cpitch of input and output differ");
    if (x->layout == DNB_NCHW && x->dtype != DNB_F32) DNB_FAIL(DNB_EINVAL, "shortcut: NCHW tensors must be f32");
    if (activation < 0 || activation > DNB_SELU) DNB_FAIL(DNB_EINVAL, "shortcut: activation %d", activation);
    const bool same = add->c == x->c && add->h == x->h && add->w == x->w &&
                      (x->layout == DNB_NCHW || add->cpitch == x->cpitch);
    // A padded channel must stay zero: only activations with act(0) == 0 may run over the padding.
    const bool pad_safe = x->layout == DNB_NCHW || x->cpitch == x->c ||
                          (activation != DNB_LOGISTIC && activation != DNB_PLSE);
    if (same && pad_safe) {
        const size_t bytes = tensor_elems(x) * elem_size(x->dtype);
        if (bytes % 16 == 0) {
            size_t nvec = bytes / 16;
            if (x->dtype == DNB_F32)
                shortcut_flat_kernel<float><<<grid_for(nvec, 256), 256, 0, s>>>((const float *)x->data, (const float *)add->data, (float *)y->data, nvec, alpha, beta, activation);
            else
                shortcut_flat_kernel<__nv_bfloat16><<<grid_for(nvec, 256), 256, 0, s>>>((const __nv_bfloat16 *)x->data, (const __nv_bfloat16 *)add->data, (__nv_bfloat16 *)y->data, nvec, alpha, beta, activation);
            DNB_LAUNCH_CHECK("shortcut");
            return DNB_OK;
        }
    }
    // w1,h1,c1 = add; w2,h2,c2 = out.  The reference asserts stride == h1/h2 and sample == h2/h1.
    ShortcutGeom g;
    g.B = x->n; g.C2 = x->c; g.H2 = x->h; g.W2 = x->w;
    g.stride = add->w / x->w; g.sample = x->w / add->w;
    if (g.stride != add->h / x->h || g.sample != x->h / add->h)
        DNB_FAIL(DNB_EINVAL, "shortcut: width and height ratios differ (%dx%d vs %dx%d)", add->w, add->h, x->w, x->h);
    if (g.stride < 1) g.stride = 1;
    if (g.sample < 1) g.sample = 1;
    g.minw = add->w < x->w ? add->w : x->w;
    g.minh = add->h < x->h ? add->h : x->h;
    g.minc = add->c < x->c ? add->c : x->c;
    if (x->layout == DNB_NHWC) {
        g.inner_is_c = 1;
        g.xs_c = 1; g.xs_w = x->cpitch; g.xs_h = (long long)x->w * x->cpitch; g.xs_b = (long long)x->h * g.xs_h;
        g.as_c = 1; g.as_w = add->cpitch; g.as_h = (long long)add->w * add->cpitch; g.as_b = (long long)add->h * g.as_h;
    } else {
        g.inner_is_c = 0;
        g.xs_w = 1; g.xs_h = x->w; g.xs_c = (long long)x->h * x->w; g.xs_b = (long long)x->c * g.xs_c;
        g.as_w = 1; g.as_h = add->w; g.as_c = (long long)add->h * add->w; g.as_b = (long long)add->c * g.as_c;
    }
    if (x->layout == DNB_NHWC && (long long)g.B * g.H2 < (1LL << 31) && (long long)g.W2 * x->cpitch < (1LL << 31)) {
        if (x->dtype == DNB_F32)
            shortcut_rows_nhwc_kernel<float><<<row_grid(g.B, g.H2), 256, 0, s>>>((const float *)x->data, (const float *)add->data, (float *)y->data, g,
                                                                              x->cpitch, add->cpitch, add->h, add->w, alpha, beta, activation);
        else
            shortcut_rows_nhwc_kernel<__nv_bfloat16><<<row_grid(g.B, g.H2), 256, 0, s>>>((const __nv_bfloat16 *)x->data, (const __nv_bfloat16 *)add->data,
                                                                                      (__nv_bfloat16 *)y->data, g, x->cpitch, add->cpitch, add->h, add->w,
                                                                                      alpha, beta, activation);
        DNB_LAUNCH_CHECK("shortcut");
        return DNB_OK;
    }
    size_t total = (size_t)g.B * g.C2 * g.H2 * g.W2;
    if (x->dtype == DNB_F32)
        shortcut_general_kernel<float><<<grid_for(total, 256), 256, 0, s>>>((const float *)x->data, (const float *)add->data, (float *)y->data, g, alpha, beta, activation);
    else
        shortcut_general_kernel<__nv_bfloat16><<<grid_for(total, 256), 256, 0, s>>>((const __nv_bfloat16 *)x->data, (const __nv_bfloat16 *)add->data, (__nv_bfloat16 *)y->data, g, alpha, beta, activation);
    DNB_LAUNCH_CHECK("shortcut");
    return DNB_OK;
}

// ------------------------------------------------------------------ route (strided 2-D copy)
template <typename V>
__global__ void copy2d_kernel(const V *__restrict__ src, V *__restrict__ dst, size_t rows, size_t row_len,
                              size_t src_pitch, size_t dst_pitch)
{
    const size_t total = rows * row_len;
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        size_t r = i / row_len, k = i - r * row_len;
        dst[r * dst_pitch + k] = __ldg(src + r * src_pitch + k);
    }
}

static int copy2d(const void *src, void *dst, size_t rows, size_t row_bytes, size_t src_pitch_bytes,
                  size_t dst_pitch_bytes, cudaStream_t s)
{
    const size_t all = row_bytes | src_pitch_bytes | dst_pitch_bytes | (size_t)(uintptr_t)src | (size_t)(uintptr_t)dst;
    if (all % 16 == 0) {
        size_t n = rows * (row_bytes / 16);
        copy2d_kernel<uint4><<<grid_for(n, 256), 256, 0, s>>>((const uint4 *)src, (uint4 *)dst, rows, row_bytes / 16, src_pitch_bytes / 16, dst_pitch_bytes / 16);
    } else if (all % 8 == 0) {
        size_t n = rows * (row_bytes / 8);
        copy2d_kernel<uint2><<<grid_for(n, 256), 256, 0, s>>>((const uint2 *)src, (uint2 *)dst, rows, row_bytes / 8, src_pitch_bytes / 8, dst_pitch_bytes / 8);
    } else if (all % 4 == 0) {
        size_t n = rows * (row_bytes / 4);
        copy2d_kernel<uint32_t><<<grid_for(n, 256), 256, 0, s>>>((const uint32_t *)src, (uint32_t *)dst, rows, row_bytes / 4, src_pitch_bytes / 4, dst_pitch_bytes / 4);
    } else {
        size_t n = rows * (row_bytes / 2);
        copy2d_kernel<uint16_t><<<grid_for(n, 256), 256, 0, s>>>((const uint16_t *)src, (uint16_t *)dst, rows, row_bytes / 2, src_pitch_bytes / 2, dst_pitch_bytes / 2);
    }
    DNB_LAUNCH_CHECK("route copy");
    return DNB_OK;
}

int launch_route(const dnb_tensor *const *inputs, int count, const dnb_tensor *y, cudaStream_t s)
{
    if (count < 1 || !inputs) DNB_FAIL(DNB_EINVAL, "route: no inputs");
    DNB_TRY(check_tensor(y, "route output"));
    int csum = 0;
    for (int i = 0; i < count; ++i) {
        DNB_TRY(check_tensor(inputs[i], "route input"));
        const dnb_tensor *t = inputs[i];
        if (t->layout != y->layout || t->dtype != y->dtype || t->n != y->n)
            DNB_FAIL(DNB_EINVAL, "route: input %d differs from the output in layout, dtype or batch", i);
        if (t->h != y->h || t->w != y->w)
            DNB_FAIL(DNB_EUNSUPPORTED, "route: input %d is %dx%d, output %dx%d (inputs of unequal size give a flat, "
                     "shapeless output in the reference; not on this path)", i, t->w, t->h, y->w, y->h);
        csum += t->c;
    }
    if (csum != y->c) DNB_FAIL(DNB_EINVAL, "route: inputs have %d channels in total, output %d", csum, y->c);
    const size_t es = elem_size(y->dtype);
    int coff = 0;
    for (int i = 0; i < count; ++i) {
        const dnb_tensor *t = inputs[i];
        if (y->layout == DNB_NHWC && t->data == (char *)y->data + (size_t)coff * es && t->cpitch == y->cpitch) {
            coff += t->c;   // this input IS its channel range of the output (its producer wrote it there): nothing to copy
            continue;
        }
        if (y->layout == DNB_NHWC) {
            size_t rows = (size_t)t->n * t->h * t->w;
            DNB_TRY(copy2d(t->data, (char *)y->data + (size_t)coff * es, rows, (size_t)t->c * es, (size_t)t->cpitch * es, (size_t)y->cpitch * es, s));
        } else {
            size_t plane = (size_t)t->h * t->w;
            DNB_TRY(copy2d(t->data, (char *)y->data + (size_t)coff * plane * es, (size_t)t->n, (size_t)t->c * plane * es, (size_t)t->c * plane * es, (size_t)y->c * plane * es, s));
        }
        coff += t->c;
    }
    return DNB_OK;
}

// ------------------------------------------------------------------ layout conversion (+ YOLO head)
// Per image a [C][HW] <-> [HW][Cp] transpose through a 32x33 shared tile.
// yolo_entries > 0: channel ch gets the logistic when (ch % yolo_entries) is
// 0, 1 or >= 4 (x, y, objectness, classes; src/yolo_layer.c:137-146).
template <typename T>
__global__ void nchw_to_nhwc_kernel(const float *__restrict__ x, T *__restrict__ y, int C, int HW, int Cp, int rnd)
{
    __shared__ float tile[32][33];
    const int b = blockIdx.z;
    const int c0 = blockIdx.y * 32, p0 = blockIdx.x * 32;
    const float *src = x + (size_t)b * C * HW;
    T *dst = y + (size_t)b * HW * Cp;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        int c = c0 + j, p = p0 + threadIdx.x;
        tile[j][threadIdx.x] = (c < C && p < HW) ? __ldg(src + (size_t)c * HW + p) : 0.f;
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        int p = p0 + j, c = c0 + threadIdx.x;
        if (p < HW && c < Cp) {
            float v = tile[threadIdx.x][j];
            if (rnd) v = round_tf32(v);
            dst[(size_t)p * Cp + c] = from_float<T>(v);
        }
    }
}

// Channels-last to Darknet's layout: a tile of 128 pixels x 32 channels per block.  Loads are 16-byte
// (8-byte for bf16) pieces of a pixel's channels, four pixels per warp instruction; stores are 128-byte
// runs of one channel plane.  The 129-float row pitch keeps both shared-memory phases conflict-free.
template <typename T>
__global__ void __launch_bounds__(256)
nhwc_to_nchw_kernel(const T *__restrict__ x, float *__restrict__ y, int C, int HW, int Cp, int yolo_entries)
{
    __shared__ float tile[32][129];
    const int b = blockIdx.z;
    const int c0 = blockIdx.y * 32, p0 = blockIdx.x * 128;
    const T *src = x + (size_t)b * HW * Cp;
    float *dst = y + (size_t)b * C * HW;
    const int t = threadIdx.x;
    {
        const int pl = t >> 3, q = t & 7, c = c0 + 4 * q;
#pragma unroll
        for (int pass = 0; pass < 4; ++pass) {
            const int pp = pl + 32 * pass, p = p0 + pp;
            float v[4] = {0.f, 0.f, 0.f, 0.f};
            if (p < HW && c < Cp) {   // the pitch is a multiple of 8: a 4-channel piece is inside it or outside
                if (sizeof(T) == 4) {
                    const float4 f = __ldg(reinterpret_cast<const float4 *>(src + (size_t)p * Cp + c));
                    v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
                } else {
                    const uint2 u = __ldg(reinterpret_cast<const uint2 *>(src + (size_t)p * Cp + c));
                    v[0] = __uint_as_float(u.x << 16); v[1] = __uint_as_float(u.x & 0xffff0000u);
                    v[2] = __uint_as_float(u.y << 16); v[3] = __uint_as_float(u.y & 0xffff0000u);
                }
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) tile[4 * q + e][pp] = v[e];
        }
    }
    __syncthreads();
    const int lane = t & 31, w = t >> 5;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int j = w + 8 * k, c = c0 + j;
        if (c >= C) continue;
        bool logistic = false;
        if (yolo_entries > 0) {
            const int e = c % yolo_entries;
            logistic = e < 2 || e >= 4;
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int pp = lane + 32 * e, p = p0 + pp;
            if (p < HW) {
                float v = tile[j][pp];
                if (logistic) v = 1.f / (1.f + expf(-v));
                dst[(size_t)c * HW + p] = v;
            }
        }
    }
}

// Same layout on both sides: copy with optional rounding / YOLO logistic / dtype change.
template <typename TI, typename TO>
__global__ void elementwise_convert_kernel(const TI *__restrict__ x, TO *__restrict__ y, size_t total, int rnd,
                                           int yolo_entries, int HW, int C)
{
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        float v = to_float<TI>(x[i]);
        if (yolo_entries > 0) {  // NCHW only
            int c = (int)((i / HW) % C), e = c % yolo_entries;
            if (e < 2 || e >= 4) v = 1.f / (1.f + expf(-v));
        }
        if (rnd) v = round_tf32(v);
        y[i] = from_float<TO>(v);
    }
}

int launch_convert(const dnb_tensor *x, const dnb_tensor *y, int rnd, int yolo_anchors, int yolo_classes, cudaStream_t s)
{
    DNB_TRY(check_tensor(x, "convert input"));
    DNB_TRY(check_tensor(y, "convert output"));
    if (x->n != y->n || x->c != y->c || x->h != y->h || x->w != y->w) DNB_FAIL(DNB_EINVAL, "convert: extents differ");
    const int entries = yolo_anchors > 0 ? 5 + yolo_classes : 0;
    if (entries && (y->layout != DNB_NCHW || y->dtype != DNB_F32 || x->c != yolo_anchors * entries))
        DNB_FAIL(DNB_EINVAL, "yolo: output must be NCHW f32 with %d channels", yolo_anchors * entries);
    const int HW = x->h * x->w;
    dim3 block(32, 8);
    if (x->layout == DNB_NCHW && y->layout == DNB_NHWC) {
        if (x->dtype != DNB_F32) DNB_FAIL(DNB_EINVAL, "convert: NCHW tensors must be f32");
        dim3 grid((HW + 31) / 32, (y->cpitch + 31) / 32, x->n);
        if (y->dtype == DNB_F32) nchw_to_nhwc_kernel<float><<<grid, block, 0, s>>>((const float *)x->data, (float *)y->data, x->c, HW, y->cpitch, rnd);
        else nchw_to_nhwc_kernel<__nv_bfloat16><<<grid, block, 0, s>>>((const float *)x->data, (__nv_bfloat16 *)y->data, x->c, HW, y->cpitch, 0);
    } else if (x->layout == DNB_NHWC && y->layout == DNB_NCHW) {
        if (y->dtype != DNB_F32) DNB_FAIL(DNB_EINVAL, "convert: NCHW tensors must be f32");
        dim3 grid((HW + 127) / 128, (x->c + 31) / 32, x->n);
        if (x->dtype == DNB_F32) nhwc_to_nchw_kernel<float><<<grid, 256, 0, s>>>((const float *)x->data, (float *)y->data, x->c, HW, x->cpitch, entries);
        else nhwc_to_nchw_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16 *)x->data, (float *)y->data, x->c, HW, x->cpitch, entries);
    } else if (x->layout == DNB_NCHW) {
        if (x->dtype != DNB_F32 || y->dtype != DNB_F32) DNB_FAIL(DNB_EINVAL, "convert: NCHW tensors must be f32");
        size_t total = tensor_elems(x);
        elementwise_convert_kernel<float, float><<<grid_for(total, 256), 256, 0, s>>>((const float *)x->data, (float *)y->data, total, rnd, entries, HW, x->c);
    } else {
        if (x->cpitch != y->cpitch) DNB_FAIL(DNB_EINVAL, "convert: NHWC to NHWC needs equal cpitch");
        size_t total = tensor_elems(x);
        if (x->dtype == DNB_F32 && y->dtype == DNB_F32) elementwise_convert_kernel<float, float><<<grid_for(total, 256), 256, 0, s>>>((const float *)x->data, (float *)y->data, total, rnd, 0, 1, 1);
        else if (x->dtype == DNB_F32) elementwise_convert_kernel<float, __nv_bfloat16><<<grid_for(total, 256), 256, 0, s>>>((const float *)x->data, (__nv_bfloat16 *)y->data, total, 0, 0, 1, 1);
        else if (y->dtype == DNB_F32) elementwise_convert_kernel<__nv_bfloat16, float><<<grid_for(total, 256), 256, 0, s>>>((const __nv_bfloat16 *)x->data, (float *)y->data, total, 0, 0, 1, 1);
        else elementwise_convert_kernel<__nv_bfloat16, __nv_bfloat16><<<grid_for(total, 256), 256, 0, s>>>((const __nv_bfloat16 *)x->data, (__nv_bfloat16 *)y->data, total, 0, 0, 1, 1);
    }
    DNB_LAUNCH_CHECK("convert");
    return DNB_OK;
}

// ------------------------------------------------------------------ global average pool
// One block per (image, 32-channel slab); 8 row-threads per channel walk the
// pixels, then a shared-memory tree.  Element strides describe either layout.
template <typename T>
__global__ void avgpool_kernel(const T *__restrict__ x, T *__restrict__ y, int C, int HW, long long sb, long long sc,
                               long long sp, long long ysb)
{
    __shared__ float part[8][33];
    const int b = blockIdx.y, c = blockIdx.x * 32 + threadIdx.x;
    float acc = 0.f;
    if (c < C)
        for (int p = threadIdx.y; p < HW; p += 8) acc += to_float<T>(x[b * sb + c * sc + p * sp]);
    part[threadIdx.y][threadIdx.x] = acc;
    __syncthreads();
    if (threadIdx.y == 0 && c < C) {
        float t = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) t += part[j][threadIdx.x];
        y[b * ysb + c] = from_float<T>(t / HW);
    }
}

int launch_avgpool(const dnb_tensor *x, const dnb_tensor *y, cudaStream_t s)
{
    DNB_TRY(check_tensor(x, "avgpool input"));
    DNB_TRY(check_tensor(y, "avgpool output"));
    if (y->h != 1 || y->w != 1 || y->c != x->c || y->n != x->n) DNB_FAIL(DNB_EINVAL, "avgpool: output must be n x c x 1 x 1");
    if (x->layout != y->layout || x->dtype != y->dtype) DNB_FAIL(DNB_EINVAL, "avgpool: input and output differ in layout or dtype");
    const int HW = x->h * x->w;
    long long sb, sc, sp, ysb;
    if (x->layout == DNB_NHWC) { sc = 1; sp = x->cpitch; sb = (long long)HW * x->cpitch; ysb = y->cpitch; }
    else { sp = 1; sc = HW; sb = (long long)x->c * HW; ysb = y->c; }
    dim3 grid((x->c + 31) / 32, x->n), block(32, 8);
    if (x->dtype == DNB_F32) avgpool_kernel<float><<<grid, block, 0, s>>>((const float *)x->data, (float *)y->data, x->c, HW, sb, sc, sp, ysb);
    else avgpool_kernel<__nv_bfloat16><<<grid, block, 0, s>>>((const __nv_bfloat16 *)x->data, (__nv_bfloat16 *)y->data, x->c, HW, sb, sc, sp, ysb);
    DNB_LAUNCH_CHECK("avgpool");
    return DNB_OK;
}

// ------------------------------------------------------------------ softmax
// One block per (image, group): max, exp-sum, normalise (src/blas.c:305-332).
template <typename T>
__global__ void softmax_kernel(const T *__restrict__ x, T *__restrict__ y, int n, long long batch_stride,
                               int group_stride, float temp)
{
    __shared__ float red[32];
    const T *in = x + blockIdx.y * batch_stride + (long long)blockIdx.x * group_stride;
    T *out = y + blockIdx.y * batch_stride + (long long)blockIdx.x * group_stride;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    float m = -FLT_MAX;
    for (int i = threadIdx.x; i < n; i += blockDim.x) m = fmaxf(m, to_float<T>(in[i]));
    for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if (lane == 0) red[warp] = m;
    __syncthreads();
    m = red[0];
    for (int j = 1; j < nwarps; ++j) m = fmaxf(m, red[j]);
    __syncthreads();
    float sum = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) sum += expf(to_float<T>(in[i]) / temp - m / temp);
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if (lane == 0) red[warp] = sum;
    __syncthreads();
    sum = 0.f;
    for (int j = 0; j < nwarps; ++j) sum += red[j];
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        out[i] = from_float<T>(expf(to_float<T>(in[i]) / temp - m / temp) / sum);
}

int launch_softmax(const dnb_tensor *x, const dnb_tensor *y, int groups, float temperature, cudaStream_t s)
{
    DNB_TRY(check_tensor(x, "softmax input"));
    DNB_TRY(check_tensor(y, "softmax output"));
    if (x->h != 1 || x->w != 1) DNB_FAIL(DNB_EUNSUPPORTED, "softmax: only n x c x 1 x 1 tensors (classifier tail) are on this path");
    if (y->n != x->n || y->c != x->c || y->h != 1 || y->w != 1 || x->layout != y->layout || x->dtype != y->dtype)
        DNB_FAIL(DNB_EINVAL, "softmax: input and output differ");
    if (groups < 1 || x->c % groups) DNB_FAIL(DNB_EINVAL, "softmax: %d channels do not split into %d groups", x->c, groups);
    if (x->layout == DNB_NHWC && x->cpitch != y->cpitch) DNB_FAIL(DNB_EINVAL, "softmax: cpitch differs");
    const long long bs = x->layout == DNB_NHWC ? x->cpitch : x->c;
    dim3 grid(groups, x->n);
    if (x->dtype == DNB_F32) softmax_kernel<float><<<grid, 256, 0, s>>>((const float *)x->data, (float *)y->data, x->c / groups, bs, x->c / groups, temperature);
    else softmax_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16 *)x->data, (__nv_bfloat16 *)y->data, x->c / groups, bs, x->c / groups, temperature);
    DNB_LAUNCH_CHECK("softmax");
    return DNB_OK;
}

}  // namespace dnb
