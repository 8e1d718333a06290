// Error text, device queries, tensor validation and the thin extern "C" layer
// over the memory-bound kernels.
#include "common.h"

#include <string.h>

namespace dnb {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}
const char *get_error() { return g_error; }

int sm_count()
{
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cached[dev] = v;
    }
    return cached[dev];
}

int check_current_device(int device, const char *what)
{
    int cur = -1;
    DNB_CUDA(cudaGetDevice(&cur));
    if (cur != device)
        DNB_FAIL(DNB_EINVAL, "%s: created on CUDA device %d but device %d is current; nothing was launched (dnb_set_device(%d) first)", what, device, cur, device);
    return DNB_OK;
}

int check_tensor(const dnb_tensor *t, const char *what)
{
    if (!t) DNB_FAIL(DNB_EINVAL, "%s: null tensor", what);
    if (!t->data) DNB_FAIL(DNB_EINVAL, "%s: null data pointer", what);
    if (t->n < 1 || t->c < 1 || t->h < 1 || t->w < 1) DNB_FAIL(DNB_EINVAL, "%s: extents %dx%dx%dx%d", what, t->n, t->c, t->h, t->w);
    if (t->layout != DNB_NCHW && t->layout != DNB_NHWC) DNB_FAIL(DNB_EINVAL, "%s: layout %d", what, t->layout);
    if (t->dtype != DNB_F32 && t->dtype != DNB_BF16) DNB_FAIL(DNB_EINVAL, "%s: dtype %d", what, t->dtype);
    if (t->layout == DNB_NCHW && t->dtype != DNB_F32) DNB_FAIL(DNB_EINVAL, "%s: NCHW tensors are f32", what);
    if (t->layout == DNB_NHWC) {
        if (t->cpitch < t->c || t->cpitch % 8) DNB_FAIL(DNB_EINVAL, "%s: cpitch %d for %d channels (need a multiple of 8 >= c)", what, t->cpitch, t->c);
        if ((uintptr_t)t->data % 128) DNB_FAIL(DNB_EINVAL, "%s: NHWC data must be 128-byte aligned", what);
    } else if ((uintptr_t)t->data % 16) {
        DNB_FAIL(DNB_EINVAL, "%s: data must be 16-byte aligned", what);
    }
    return DNB_OK;
}

}  // namespace dnb

using namespace dnb;

extern "C" {

const char *dnb_last_error(void) { return get_error(); }
int dnb_version(void) { return 100; }
int dnb_cpitch(int c) { return round_up(c, 8); }

int dnb_set_device(int device)
{
    DNB_CUDA(cudaSetDevice(device));
    return DNB_OK;
}
int dnb_device_count(int *count)
{
    if (!count) DNB_FAIL(DNB_EINVAL, "dnb_device_count: null");
    DNB_CUDA(cudaGetDeviceCount(count));
    return DNB_OK;
}

int dnb_maxpool_forward(const dnb_tensor *x, const dnb_tensor *y, int size, int stride, int padding, void *stream)
{
    return launch_maxpool(x, y, size, stride, padding, (cudaStream_t)stream);
}
int dnb_upsample_forward(const dnb_tensor *x, const dnb_tensor *y, int stride, float scale, void *stream)
{
    return launch_upsample(x, y, stride, scale, (cudaStream_t)stream);
}
int dnb_shortcut_forward(const dnb_tensor *x, const dnb_tensor *add, const dnb_tensor *y, float alpha, float beta,
                         int activation, void *stream)
{
    return launch_shortcut(x, add, y, alpha, beta, activation, (cudaStream_t)stream);
}
int dnb_route_forward(const dnb_tensor *const *inputs, int count, const dnb_tensor *y, void *stream)
{
    return launch_route(inputs, count, y, (cudaStream_t)stream);
}
int dnb_convert(const dnb_tensor *x, const dnb_tensor *y, int round_tf32, void *stream)
{
    return launch_convert(x, y, round_tf32, 0, 0, (cudaStream_t)stream);
}
int dnb_yolo_forward(const dnb_tensor *x, const dnb_tensor *y, int anchors, int classes, void *stream)
{
    if (anchors < 1 || classes < 0) DNB_FAIL(DNB_EINVAL, "yolo: anchors %d classes %d", anchors, classes);
    return launch_convert(x, y, 0, anchors, classes, (cudaStream_t)stream);
}
int dnb_avgpool_forward(const dnb_tensor *x, const dnb_tensor *y, void *stream)
{
    return launch_avgpool(x, y, (cudaStream_t)stream);
}
int dnb_softmax_forward(const dnb_tensor *x, const dnb_tensor *y, int groups, float temperature, void *stream)
{
    return launch_softmax(x, y, groups, temperature, (cudaStream_t)stream);
}

}  // extern "C"
