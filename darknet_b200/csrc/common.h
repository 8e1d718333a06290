// Internal declarations shared by the .cu/.cpp files of libdarknet_b200.
#pragma once
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/darknet_b200.h"

namespace dnb {

// Thread-local error text behind dnb_last_error().
void set_error(const char *fmt, ...);
const char *get_error();

#define DNB_FAIL(code, ...)           \
    do {                              \
        ::dnb::set_error(__VA_ARGS__); \
        return (code);                \
    } while (0)

#define DNB_CUDA(expr)                                                                     \
    do {                                                                                   \
        cudaError_t e__ = (expr);                                                          \
        if (e__ != cudaSuccess)                                                            \
            DNB_FAIL(DNB_ECUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__),   \
                     __FILE__, __LINE__);                                                  \
    } while (0)

#define DNB_TRY(expr)                 \
    do {                              \
        int s__ = (expr);             \
        if (s__ != DNB_OK) return s__; \
    } while (0)

// Launch check: the reference calls check_error(cudaPeekAtLastError()) after
// every launch (src/cuda.c:27-49) and aborts; here the code is returned.
#define DNB_LAUNCH_CHECK(name)                                                        \
    do {                                                                              \
        cudaError_t e__ = cudaPeekAtLastError();                                      \
        if (e__ != cudaSuccess)                                                       \
            DNB_FAIL(DNB_ECUDA, "launch of %s failed: %s", name, cudaGetErrorString(e__)); \
    } while (0)

inline int round_up(int x, int m) { return (x + m - 1) / m * m; }
inline size_t elem_size(int dtype) { return dtype == DNB_BF16 ? 2 : 4; }

// Number of SMs of the current device (cached per device).
int sm_count();

// DNB_EINVAL unless `device` (where a plan or network was created) is the calling thread's current device:
// nothing is launched over another GPU's pointers.
int check_current_device(int device, const char *what);

// Validation helpers (return DNB_OK or set the error).
int check_tensor(const dnb_tensor *t, const char *what);
inline size_t tensor_elems(const dnb_tensor *t)
{
    return t->layout == DNB_NHWC ? (size_t)t->n * t->h * t->w * t->cpitch
                                 : (size_t)t->n * t->c * t->h * t->w;
}

// ---- kernels_mem.cu
// signs: optional int8 channels-last tensor of pitch spitch that receives the output's signs (f32 channels-last tensors)
int launch_maxpool(const dnb_tensor *x, const dnb_tensor *y, int size, int stride, int padding, cudaStream_t s, int8_t *signs = nullptr, int spitch = 0);
int launch_upsample(const dnb_tensor *x, const dnb_tensor *y, int stride, float scale, cudaStream_t s);
int launch_shortcut(const dnb_tensor *x, const dnb_tensor *add, const dnb_tensor *y, float alpha, float beta,
                    int activation, cudaStream_t s);
int launch_route(const dnb_tensor *const *inputs, int count, const dnb_tensor *y, cudaStream_t s);
int launch_convert(const dnb_tensor *x, const dnb_tensor *y, int round_tf32, int yolo_anchors, int yolo_classes,
                   cudaStream_t s);
int launch_avgpool(const dnb_tensor *x, const dnb_tensor *y, cudaStream_t s);
int launch_softmax(const dnb_tensor *x, const dnb_tensor *y, int groups, float temperature, cudaStream_t s);

// ---- conv kernels.  Epilogue parameters shared by all of them.
struct ConvEpilogue {
    const float *scale;   // [n_pad] folded batchnorm scale s' (1 when no batchnorm)
    const float *shift;   // [n_pad] folded shift b'
    int activation;       // dnb_activation
    int round_tf32;       // round f32 NHWC results to TF32-nearest
    // optional fused residual (the [shortcut] layer that follows the convolution):
    // out = act2(alpha * act(conv) + beta * residual), residual channels-last, same extents as the output
    const void *residual;
    int res_cpitch;
    int activation2;
    float alpha, beta;
    int raw_acc;          // int8 (xnor) tensor-core launches: write the int32 sums themselves into the NCHW output
    // fused [yolo] head (tensor-core kernel only): > 0 = entries per anchor (5 + classes); the logistic is applied to
    // every output channel but the w and h entries of each anchor (ch % entries == 2 or 3), after the activation
    int yolo_entries;
};

struct ConvGeom {
    int batch, h, w, c, n, groups, size, stride, pad, out_h, out_w;
};

}  // namespace dnb
