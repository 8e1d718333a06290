/*
 * CPU restatement of Darknet's forward (inference) arithmetic for the layers on
 * the convolutional hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker that the CUDA kernels are
 * compared against; it is never linked into, imported by or called from the
 * shipped library.  Only the test-suite, the smoke check and the CPU-baseline
 * leg of the benchmark may build or load it.
 *
 * Parity pin: every function below is checked bit-for-bit (or, where the stock
 * build's -Ofast reassociates a reduction, to the stated tolerance) against the
 * unmodified reference compiled from its own sources (see ref_harness.c and the
 * Makefile in this directory), and against the golden vectors that build
 * produced (tests/golden).
 *
 * All tensors are Darknet's: fp32, NCHW, one contiguous block per image.
 * Each function cites the reference code it follows (path within the
 * pjreddie/darknet tree).
 *
 * Build: gcc -O2 -fopenmp -fPIC -shared (no -ffast-math, no -march): the
 * accumulation order is the reference's, sequential in k, one rounding per
 * multiply and one per add.
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* Same numbering as the reference's ACTIVATION enum (include/darknet.h:48-50). */
enum {
    ORC_LOGISTIC = 0, ORC_RELU, ORC_RELIE, ORC_LINEAR, ORC_RAMP, ORC_TANH, ORC_PLSE,
    ORC_LEAKY, ORC_ELU, ORC_LOGGY, ORC_STAIR, ORC_HARDTAN, ORC_LHTAN, ORC_SELU
};

/* ------------------------------------------------------------------------- */
/* Activations: src/activations.h:19-53 (scalar forms), src/activations.c:65-106
 * (dispatch and the in-place array loop).  The reference writes the constants
 * as doubles (".1*x", "1./(1. + exp(-x))"), so the arithmetic runs in double
 * and is rounded to float once on return; the same is done here. */
static float orc_activate_one(float x, int a)
{
    switch (a) {
    case ORC_LINEAR:   return x;
    case ORC_LOGISTIC: return (float)(1. / (1. + exp(-x)));
    case ORC_LOGGY:    return (float)(2. / (1. + exp(-x)) - 1);
    case ORC_RELU:     return x * (x > 0);
    case ORC_ELU:      return (float)((x >= 0) * x + (x < 0) * (exp(x) - 1));
    case ORC_SELU:     return (float)((x >= 0) * 1.0507 * x + (x < 0) * 1.0507 * 1.6732 * (exp(x) - 1));
    case ORC_RELIE:    return (x > 0) ? x : (float)(.01 * x);
    case ORC_RAMP:     return (float)(x * (x > 0) + .1 * x);
    case ORC_LEAKY:    return (x > 0) ? x : (float)(.1 * x);
    case ORC_TANH:     return (float)((exp(2 * x) - 1) / (exp(2 * x) + 1));
    case ORC_PLSE:
        if (x < -4) return (float)(.01 * (x + 4));
        if (x > 4)  return (float)(.01 * (x - 4) + 1);
        return (float)(.125 * x + .5);
    case ORC_STAIR: {
        int n = (int)floor(x);
        if (n % 2 == 0) return (float)floor(x / 2.);
        return (float)((x - n) + floor(x / 2.));
    }
    case ORC_HARDTAN:
        if (x < -1) return -1;
        if (x > 1) return 1;
        return x;
    case ORC_LHTAN:
        if (x < 0) return (float)(.001 * x);
        if (x > 1) return (float)(.001 * (x - 1) + 1);
        return x;
    }
    return 0;
}

void orc_activate_array(float *x, long n, int a)
{
    for (long i = 0; i < n; ++i) x[i] = orc_activate_one(x[i], a);
}

/* ------------------------------------------------------------------------- */
/* Unfold one image into the K x N matrix the GEMM multiplies.
 * src/im2col.c:3-39: row r = (c*ksize + kh)*ksize + kw, column = h'*W' + w',
 * value = im[c][h'*stride + kh - pad][w'*stride + kw - pad], 0 outside. */
void orc_im2col(const float *im, int channels, int height, int width,
                int ksize, int stride, int pad, float *col)
{
    const int out_h = (height + 2 * pad - ksize) / stride + 1;
    const int out_w = (width + 2 * pad - ksize) / stride + 1;
    const int rows = channels * ksize * ksize;
    for (int r = 0; r < rows; ++r) {
        const int kw = r % ksize;
        const int kh = (r / ksize) % ksize;
        const int ch = r / ksize / ksize;
        const float *plane = im + (size_t)ch * height * width;
        float *dst = col + (size_t)r * out_h * out_w;
        for (int oh = 0; oh < out_h; ++oh) {
            const int ih = oh * stride + kh - pad;
            for (int ow = 0; ow < out_w; ++ow) {
                const int iw = ow * stride + kw - pad;
                const int inside = ih >= 0 && iw >= 0 && ih < height && iw < width;
                dst[oh * out_w + ow] = inside ? plane[(size_t)ih * width + iw] : 0.f;
            }
        }
    }
}

/* C += alpha * A * B, row-major, no transposes.  src/gemm.c:74-89: rows of C
 * are the OpenMP-parallel loop; for one row the k loop is outermost, so every
 * C[i][j] receives its K products in increasing k, each product rounded to
 * fp32 (alpha*A[i][k] rounded first), each add rounded to fp32.  The row loop
 * carries no dependence, so the result does not depend on the thread count. */
void orc_gemm_nn(int M, int N, int K, float alpha,
                 const float *A, int lda, const float *B, int ldb, float *C, int ldc)
{
#pragma omp parallel for
    for (int i = 0; i < M; ++i) {
        float *crow = C + (size_t)i * ldc;
        for (int k = 0; k < K; ++k) {
            const float a = alpha * A[(size_t)i * lda + k];
            const float *brow = B + (size_t)k * ldb;
            for (int j = 0; j < N; ++j) crow[j] += a * brow[j];
        }
    }
}

/* ------------------------------------------------------------------------- */
/* Weight binarisation: src/convolutional_layer.c:28-41.  Per filter, every
 * weight becomes +mean or -mean with mean = (sum of |w|)/size accumulated in a
 * float in index order; the sign test is "> 0" (zero maps to -mean). */
void orc_binarize_weights(const float *weights, int n, int size, float *binary)
{
    for (int f = 0; f < n; ++f) {
        float mean = 0;
        for (int i = 0; i < size; ++i) mean += fabs(weights[(size_t)f * size + i]);
        mean = mean / size;
        for (int i = 0; i < size; ++i)
            binary[(size_t)f * size + i] = (weights[(size_t)f * size + i] > 0) ? mean : -mean;
    }
}

/* Input binarisation: src/convolutional_layer.c:43-49, "> 0" -> +1 else -1. */
void orc_binarize_input(const float *input, long n, float *binary)
{
    for (long i = 0; i < n; ++i) binary[i] = (input[i] > 0) ? 1.f : -1.f;
}

/* ------------------------------------------------------------------------- */
typedef struct {
    int batch, h, w, c;          /* input  [batch][c][h][w]                        */
    int n, groups, size, stride, pad;
    int batch_normalize;         /* 1: rolling-stat batchnorm, 0: bias only        */
    int activation;              /* ORC_* / reference ACTIVATION value             */
    int xnor;                    /* 1: binarise weights and input first            */
} orc_conv_t;

int orc_conv_out_h(const orc_conv_t *p) { return (p->h + 2 * p->pad - p->size) / p->stride + 1; }
int orc_conv_out_w(const orc_conv_t *p) { return (p->w + 2 * p->pad - p->size) / p->stride + 1; }

/* Bytes of scratch orc_conv_forward needs (im2col matrix of one image-group,
 * plus, for xnor, the binarised weights and input). */
size_t orc_conv_workspace_bytes(const orc_conv_t *p)
{
    const size_t col = (size_t)orc_conv_out_h(p) * orc_conv_out_w(p) * p->size * p->size * (p->c / p->groups);
    size_t extra = 0;
    if (p->xnor) extra = (size_t)p->n * (p->c / p->groups) * p->size * p->size + (size_t)p->batch * p->c * p->h * p->w;
    return (col + extra) * sizeof(float);
}

/* Inference batchnorm + bias as the CPU reference applies them:
 * src/batchnorm_layer.c:151-154 -> normalize_cpu (src/blas.c:147-158), then
 * scale_bias and add_bias (src/convolutional_layer.c:411-433).  Three separate
 * roundings per element.  normalize_cpu calls the double sqrt and adds the
 * float constant .000001f, so the quotient is formed in double and rounded. */
static void orc_bn_bias(float *out, const orc_conv_t *p, int spatial,
                        const float *biases, const float *scales,
                        const float *mean, const float *variance)
{
    for (int b = 0; b < p->batch; ++b) {
        for (int f = 0; f < p->n; ++f) {
            float *o = out + ((size_t)b * p->n + f) * spatial;
            if (p->batch_normalize) {
                for (int i = 0; i < spatial; ++i)
                    o[i] = (float)((o[i] - mean[f]) / (sqrt(variance[f]) + .000001f));
                for (int i = 0; i < spatial; ++i) o[i] *= scales[f];
            }
            for (int i = 0; i < spatial; ++i) o[i] += biases[f];
        }
    }
}

/* The whole convolutional forward: src/convolutional_layer.c:445-485.
 * out is zeroed, then per image and per group C += W * im2col(x); a 1x1
 * kernel skips im2col and multiplies the image itself with ldb = out_h*out_w
 * (so the reference ignores stride/pad for size 1; kept as is).  Then
 * batchnorm-or-bias, then the activation.  With xnor the weights and the whole
 * input batch are binarised first (zero padding is applied afterwards by
 * im2col, so border taps add 0, not -1). */
void orc_conv_forward(const orc_conv_t *p, const float *input, const float *weights,
                      const float *biases, const float *scales,
                      const float *rolling_mean, const float *rolling_variance,
                      float *output, float *workspace)
{
    const int out_h = orc_conv_out_h(p), out_w = orc_conv_out_w(p);
    const int m = p->n / p->groups;
    const int k = p->size * p->size * p->c / p->groups;
    const int n = out_h * out_w;
    const size_t nweights = (size_t)p->n * (p->c / p->groups) * p->size * p->size;
    float *col = workspace;

    memset(output, 0, sizeof(float) * (size_t)p->batch * p->n * n);
    if (p->xnor) {
        float *bw = workspace + (size_t)n * k;
        float *bx = bw + nweights;
        orc_binarize_weights(weights, p->n, k, bw);
        orc_binarize_input(input, (long)p->batch * p->c * p->h * p->w, bx);
        weights = bw;
        input = bx;
    }
    for (int i = 0; i < p->batch; ++i) {
        for (int j = 0; j < p->groups; ++j) {
            const float *a = weights + (size_t)j * (nweights / p->groups);
            const float *im = input + (size_t)(i * p->groups + j) * (p->c / p->groups) * p->h * p->w;
            float *c = output + (size_t)(i * p->groups + j) * n * m;
            const float *b = im;
            if (p->size != 1) {
                orc_im2col(im, p->c / p->groups, p->h, p->w, p->size, p->stride, p->pad, col);
                b = col;
            }
            orc_gemm_nn(m, n, k, 1.f, a, k, b, n, c, n);
        }
    }
    orc_bn_bias(output, p, n, biases, scales, rolling_mean, rolling_variance);
    orc_activate_array(output, (long)p->batch * p->n * n, p->activation);
}

/* The integer accumulators of the xnor convolution, with no scale, batchnorm
 * or activation: sign(w) (+1/-1, test "> 0") times sign(x) (+1/-1) through the
 * same im2col (zero padding) and the same gemm_nn.  Every partial sum is an
 * integer of magnitude < 2^24, so the fp32 result is exact.  groups == 1. */
void orc_xnor_accumulate(const orc_conv_t *p, const float *input, const float *weights,
                         float *output, float *workspace)
{
    const int out_h = orc_conv_out_h(p), out_w = orc_conv_out_w(p);
    const int k = p->size * p->size * p->c;
    const int n = out_h * out_w;
    float *col = workspace;
    float *sw = (float *)malloc(sizeof(float) * (size_t)p->n * k);
    float *sx = (float *)malloc(sizeof(float) * (size_t)p->c * p->h * p->w);
    for (long i = 0; i < (long)p->n * k; ++i) sw[i] = (weights[i] > 0) ? 1.f : -1.f;
    memset(output, 0, sizeof(float) * (size_t)p->batch * p->n * n);
    for (int i = 0; i < p->batch; ++i) {
        orc_binarize_input(input + (size_t)i * p->c * p->h * p->w, (long)p->c * p->h * p->w, sx);
        const float *b = sx;
        if (p->size != 1) {
            orc_im2col(sx, p->c, p->h, p->w, p->size, p->stride, p->pad, col);
            b = col;
        }
        orc_gemm_nn(p->n, n, k, 1.f, sw, k, b, n, output + (size_t)i * p->n * n, n);
    }
    free(sw);
    free(sx);
}

/* ------------------------------------------------------------------------- */
/* Connected layer: src/connected_layer.c:151-167.  The output is zeroed, then
 * gemm(0,1,...) = gemm_nt (src/gemm.c:91-106): out[b][o] += sum over i of
 * input[b][i] * weights[o][i], the products summed in a float register in index
 * order and added to the output once; then batchnorm (over the outputs, one
 * value per image: src/batchnorm_layer.c:151-154 with out_h*out_w = 1) or the
 * bias, then the activation.  The input is the previous layer's output in the
 * reference's own order (channel, row, column). */
void orc_connected_forward(int batch, int inputs, int outputs, int batch_normalize, int activation,
                           const float *input, const float *weights, const float *biases,
                           const float *scales, const float *rolling_mean, const float *rolling_variance,
                           float *output)
{
    memset(output, 0, sizeof(float) * (size_t)batch * outputs);
#pragma omp parallel for
    for (int b = 0; b < batch; ++b) {
        for (int o = 0; o < outputs; ++o) {
            float sum = 0;
            for (int i = 0; i < inputs; ++i) sum += 1.f * input[(size_t)b * inputs + i] * weights[(size_t)o * inputs + i];
            output[(size_t)b * outputs + o] += sum;
        }
    }
    orc_conv_t p;
    memset(&p, 0, sizeof(p));
    p.batch = batch; p.n = outputs; p.batch_normalize = batch_normalize;
    orc_bn_bias(output, &p, 1, biases, scales, rolling_mean, rolling_variance);
    orc_activate_array(output, (long)batch * outputs, activation);
}

/* ------------------------------------------------------------------------- */
/* Maxpool: src/maxpool_layer.c:21-52 (geometry) and :79-114 (forward).
 * "pad" is the total padding (parser default size-1, src/parser.c:487); the
 * window starts at -pad/2 (C integer division) and taps outside the image are
 * skipped; out = (in + pad - size)/stride + 1; the first maximum wins ties.
 * indexes may be NULL. */
int orc_maxpool_out(int in, int size, int stride, int pad) { return (in + pad - size) / stride + 1; }

void orc_maxpool_forward(const float *input, int batch, int c, int h, int w,
                         int size, int stride, int pad, float *output, int *indexes)
{
    const int oh = orc_maxpool_out(h, size, stride, pad);
    const int ow = orc_maxpool_out(w, size, stride, pad);
    const int off = -pad / 2;
    for (int b = 0; b < batch; ++b)
        for (int k = 0; k < c; ++k) {
            const size_t plane = (size_t)(b * c + k);
            for (int i = 0; i < oh; ++i)
                for (int j = 0; j < ow; ++j) {
                    float best = -FLT_MAX;
                    int best_i = -1;
                    for (int n = 0; n < size; ++n)
                        for (int m = 0; m < size; ++m) {
                            const int y = off + i * stride + n;
                            const int x = off + j * stride + m;
                            if (y < 0 || y >= h || x < 0 || x >= w) continue;
                            const int index = x + w * (y + h * (int)plane);
                            const float v = input[index];
                            if (v > best) { best = v; best_i = index; }
                        }
                    const size_t o = j + (size_t)ow * (i + (size_t)oh * plane);
                    output[o] = best;
                    if (indexes) indexes[o] = best_i;
                }
        }
}

/* Nearest-neighbour upsample: src/upsample_layer.c:68-76 -> upsample_cpu
 * (src/blas.c:334-349): out[b][c][j][i] = scale * in[b][c][j/s][i/s]. */
void orc_upsample_forward(const float *input, int batch, int c, int h, int w,
                          int stride, float scale, float *output)
{
    const int oh = h * stride, ow = w * stride;
    for (int b = 0; b < batch; ++b)
        for (int k = 0; k < c; ++k) {
            const float *src = input + ((size_t)b * c + k) * h * w;
            float *dst = output + ((size_t)b * c + k) * oh * ow;
            for (int j = 0; j < oh; ++j)
                for (int i = 0; i < ow; ++i)
                    dst[(size_t)j * ow + i] = scale * src[(size_t)(j / stride) * w + i / stride];
        }
}

/* Residual add: src/shortcut_layer.c:62-67 -> shortcut_cpu (src/blas.c:68-92).
 * out starts as a copy of `input` [batch][c2][h2][w2]; `add` is the earlier
 * layer's output [batch][c1][h1][w1].  Over min(w), min(h), min(c):
 * out[i*sample, j*sample, k] = alpha*out + beta*add[i*stride, j*stride, k],
 * stride = w1/w2, sample = w2/w1, both clamped to >= 1.  Then the activation
 * runs over the whole output. */
void orc_shortcut_forward(const float *input, const float *add, int batch,
                          int w1, int h1, int c1, int w2, int h2, int c2,
                          float alpha, float beta, int activation, float *output)
{
    int stride = w1 / w2, sample = w2 / w1;
    if (stride < 1) stride = 1;
    if (sample < 1) sample = 1;
    const int minw = w1 < w2 ? w1 : w2, minh = h1 < h2 ? h1 : h2, minc = c1 < c2 ? c1 : c2;
    const size_t total = (size_t)batch * c2 * h2 * w2;
    memcpy(output, input, total * sizeof(float));
    for (int b = 0; b < batch; ++b)
        for (int k = 0; k < minc; ++k)
            for (int j = 0; j < minh; ++j)
                for (int i = 0; i < minw; ++i) {
                    const size_t oi = i * sample + (size_t)w2 * (j * sample + (size_t)h2 * (k + (size_t)c2 * b));
                    const size_t ai = i * stride + (size_t)w1 * (j * stride + (size_t)h1 * (k + (size_t)c1 * b));
                    output[oi] = alpha * output[oi] + beta * add[ai];
                }
    orc_activate_array(output, (long)total, activation);
}

/* Channel concatenation: src/route_layer.c:74-87.  inputs[i] holds `batch`
 * images of input_sizes[i] floats each; image j of the output is the inputs'
 * image j blocks one after another. */
void orc_route_forward(const float *const *inputs, const int *input_sizes, int n,
                       int batch, float *output)
{
    size_t outputs = 0, offset = 0;
    for (int i = 0; i < n; ++i) outputs += input_sizes[i];
    for (int i = 0; i < n; ++i) {
        for (int j = 0; j < batch; ++j)
            memcpy(output + offset + (size_t)j * outputs, inputs[i] + (size_t)j * input_sizes[i],
                   sizeof(float) * input_sizes[i]);
        offset += input_sizes[i];
    }
}

/* YOLO head, inference branch of the CPU build: src/yolo_layer.c:132-146.
 * The input [batch][n*(5+classes)][h][w] is copied; for each anchor the x,y
 * planes (entries 0,1) and the objectness+class planes (entries 4..4+classes)
 * get the logistic; w,h (entries 2,3) stay raw. */
void orc_yolo_forward(const float *input, int batch, int n, int classes, int h, int w, float *output)
{
    const size_t plane = (size_t)h * w;
    const size_t per_anchor = (size_t)(5 + classes) * plane;
    memcpy(output, input, sizeof(float) * (size_t)batch * n * per_anchor);
    for (int b = 0; b < batch; ++b)
        for (int a = 0; a < n; ++a) {
            float *base = output + ((size_t)b * n + a) * per_anchor;
            orc_activate_array(base, (long)(2 * plane), ORC_LOGISTIC);
            orc_activate_array(base + 4 * plane, (long)((1 + classes) * plane), ORC_LOGISTIC);
        }
}

/* Global average pool: src/avgpool_layer.c:40-55.  Float running sum in
 * index order, then one division by h*w. */
void orc_avgpool_forward(const float *input, int batch, int c, int h, int w, float *output)
{
    for (int b = 0; b < batch; ++b)
        for (int k = 0; k < c; ++k) {
            float acc = 0;
            const float *src = input + ((size_t)b * c + k) * h * w;
            for (int i = 0; i < h * w; ++i) acc += src[i];
            output[(size_t)b * c + k] = acc / (h * w);
        }
}

/* Softmax over each image's `inputs` values split into `groups` equal groups:
 * src/softmax_layer.c:39-50 -> softmax_cpu / softmax (src/blas.c:305-332).
 * e = exp(x/temp - max/temp) in double rounded to float, float running sum. */
void orc_softmax_forward(const float *input, int batch, int inputs, int groups, float temp, float *output)
{
    const int n = inputs / groups;
    for (int b = 0; b < batch; ++b)
        for (int g = 0; g < groups; ++g) {
            const float *x = input + (size_t)b * inputs + (size_t)g * n;
            float *y = output + (size_t)b * inputs + (size_t)g * n;
            float sum = 0, largest = -FLT_MAX;
            for (int i = 0; i < n; ++i) if (x[i] > largest) largest = x[i];
            for (int i = 0; i < n; ++i) {
                float e = (float)exp(x[i] / temp - largest / temp);
                sum += e;
                y[i] = e;
            }
            for (int i = 0; i < n; ++i) y[i] /= sum;
        }
}
