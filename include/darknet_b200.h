/*
 * darknet_b200 - C ABI of the B200 (sm_100a) convolutional forward path.
 *
 * Plain C: opaque handles, raw pointers, ints.  No C++ or torch types cross
 * this boundary.  Every function returns a dnb_status (0 = success); on failure
 * nothing was launched and dnb_last_error() describes why.  The library never
 * falls back to the CPU: without a usable CUDA device the compute entry points
 * fail with DNB_ECUDA.
 *
 * Three levels, bottom up:
 *   1. layer kernels on device tensors (dnb_conv_*, dnb_maxpool_forward, ...):
 *      one call replaces one of the reference's forward_*_layer_gpu functions;
 *   2. a network object that mirrors the reference's parse_network_cfg /
 *      load_weights / network_predict for the layer types on this path;
 *   3. (separate header b200_attach.h, implemented by darknet_b200/shim/b200_attach.c) a shim that re-points the
 *      forward_gpu function pointers of a real Darknet `network`.
 *
 * Each declaration cites the reference interface it stands in for, as
 * path:line within the pjreddie/darknet tree.
 */
#ifndef DARKNET_B200_H
#define DARKNET_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ status */
typedef enum dnb_status {
    DNB_OK = 0,
    DNB_EINVAL = 1,        /* bad argument: shape, pointer, alignment           */
    DNB_EUNSUPPORTED = 2,  /* valid Darknet input this path does not cover       */
    DNB_ECUDA = 3,         /* CUDA runtime/driver error (message has the code)   */
    DNB_EIO = 4,           /* cfg / weights file could not be read               */
    DNB_ETIMEOUT = 5,      /* a bounded device-side wait expired                 */
    DNB_ENOMEM = 6
} dnb_status;

/* Message of the calling thread's last failure ("" if none).  Stands in for the
 * reference's print-and-exit convention (src/cuda.c:27-49 check_error,
 * src/utils.c:253-258 error): here the caller decides. */
const char *dnb_last_error(void);

/* Library ABI version (major*100 + minor). */
int dnb_version(void);

/* src/cuda.c:12-17 cuda_set_device / :19-25 cuda_get_device. */
int dnb_set_device(int device);
int dnb_device_count(int *count);

/* ------------------------------------------------------------------ enums */
/* Same numbering as the reference's ACTIVATION (include/darknet.h:48-50). */
typedef enum dnb_activation {
    DNB_LOGISTIC = 0, DNB_RELU, DNB_RELIE, DNB_LINEAR, DNB_RAMP, DNB_TANH, DNB_PLSE,
    DNB_LEAKY, DNB_ELU, DNB_LOGGY, DNB_STAIR, DNB_HARDTAN, DNB_LHTAN, DNB_SELU
} dnb_activation;

/* Arithmetic of the dense convolutions. */
typedef enum dnb_mode {
    DNB_MODE_TF32 = 0,  /* fp32 storage, TF32 tensor-core products, fp32 accumulate */
    DNB_MODE_BF16 = 1,  /* bf16 storage between layers, fp32 accumulate             */
    DNB_MODE_FP32 = 2   /* fp32 FMA on the CUDA cores (no tensor cores): slow, for
                           narrow layers and as an exact-arithmetic cross-check     */
} dnb_mode;

typedef enum dnb_layout { DNB_NCHW = 0, DNB_NHWC = 1 } dnb_layout;
typedef enum dnb_dtype { DNB_F32 = 0, DNB_BF16 = 1 } dnb_dtype;

/* A device tensor.  Darknet's own tensors are DNB_NCHW / DNB_F32 (one contiguous
 * [c][h][w] block per image).  Between layers this library keeps activations
 * channels-last: element (n,h,w,c) at ((n*h_extent + h)*w_extent + w)*cpitch + c,
 * with cpitch >= c, cpitch a multiple of 8, and the cpitch-c padding channels
 * holding zeros. */
typedef struct dnb_tensor {
    void *data;     /* device pointer, 16-byte aligned (128-byte for NHWC) */
    int layout;     /* dnb_layout */
    int dtype;      /* dnb_dtype  */
    int n, c, h, w; /* logical extents */
    int cpitch;     /* NHWC only: elements from one pixel to the next */
} dnb_tensor;

/* Smallest legal cpitch for c channels. */
int dnb_cpitch(int c);

/* ------------------------------------------------------------------ convolution */
/* Geometry and options of one convolutional layer: the fields of the
 * reference's `layer` that forward_convolutional_layer[_gpu] reads
 * (include/darknet.h:115-422; make_convolutional_layer,
 * src/convolutional_layer.c:176-328).  `pad` is the padding in pixels (the cfg's
 * pad=1 means size/2, src/parser.c:184-187). */
typedef struct dnb_conv_desc {
    int batch, h, w, c;
    int n, groups, size, stride, pad;
    int batch_normalize;
    int activation; /* dnb_activation */
    int xnor;       /* 1: binarise weights and input (l.xnor), popcount path */
} dnb_conv_desc;

typedef struct dnb_conv_plan dnb_conv_plan;

/* Replaces the per-layer setup of make_convolutional_layer
 * (src/convolutional_layer.c:176-328) for the forward path: validates the
 * geometry, picks the kernel, allocates the derived parameter tensors. */
int dnb_conv_plan_create(const dnb_conv_desc *desc, int mode, dnb_conv_plan **plan);
void dnb_conv_plan_destroy(dnb_conv_plan *plan);

/* Host arrays in Darknet's layouts, exactly what load_convolutional_weights
 * reads (src/parser.c:1164-1215): weights [n][c/groups][size][size], biases [n],
 * and for batch_normalize scales/rolling_mean/rolling_variance [n] (else NULL).
 * Replaces push_convolutional_layer (src/convolutional_kernels.cu:286-297) plus
 * the per-forward binarize_weights_gpu (:51-71): folded batchnorm vectors,
 * repacked / rounded / bit-packed weights are built once here. */
int dnb_conv_plan_set_params(dnb_conv_plan *plan, const float *weights, const float *biases,
                             const float *scales, const float *rolling_mean,
                             const float *rolling_variance);

/* Replaces forward_convolutional_layer_gpu (src/convolutional_kernels.cu:73-135)
 * including fill_gpu, im2col_gpu (src/im2col_kernels.cu:48-61), gemm_gpu
 * (src/gemm.c:172-182), forward_batchnorm_layer_gpu's inference branch
 * (src/batchnorm_layer.c:231-233) or add_bias_gpu (src/blas_kernels.cu:69), and
 * activate_array_gpu (src/activation_kernels.cu:196-200): one launch.
 * x: input, NCHW f32 or NHWC (f32 for TF32/FP32/xnor plans, bf16 for BF16 plans).
 * y: output, NCHW f32 or NHWC in the plan's storage type (f32, or bf16 for BF16
 * plans).  y2: optional second copy of the
 * output in the other layout (NULL for none).  A TF32 plan rounds the values of
 * a channels-last f32 output to TF32 (they feed the next layer's tensor-core
 * operand, which would truncate them otherwise); a copy in Darknet's layout
 * written by the same call holds the same rounded values, an NCHW-only output
 * the unrounded ones.  stream: a cudaStream_t (NULL = default stream). */
int dnb_conv_forward(dnb_conv_plan *plan, const dnb_tensor *x, const dnb_tensor *y,
                     const dnb_tensor *y2, void *stream);

/* A convolution and the [shortcut] layer that follows it in one launch:
 *   y = act2(alpha * act(conv(x)) + beta * add)
 * i.e. forward_convolutional_layer_gpu followed by forward_shortcut_layer_gpu
 * (src/shortcut_layer.c:77-82: copy_gpu + shortcut_gpu + activate_array_gpu) without
 * the intermediate tensor.  Tensor-core plans only; x, add and y channels-last in the
 * plan's storage type, add with the extents of y (other shapes: dnb_shortcut_forward).
 * The network object uses it wherever nothing else reads the convolution's own output. */
int dnb_conv_shortcut_forward(dnb_conv_plan *plan, const dnb_tensor *x, const dnb_tensor *add,
                              const dnb_tensor *y, float alpha, float beta, int activation2, void *stream);

/* A convolution and the [yolo] layer that follows it in one launch.  At inference
 * forward_yolo_layer_gpu (src/yolo_layer.c:347-357) copies its input and applies the
 * logistic to the x, y, objectness and class entries of every anchor, i.e. to every
 * channel ch with ch % (classes + 5) not 2 or 3; here the convolution's epilogue does
 * that after the layer's own activation and writes y, the [yolo] layer's output
 * (NCHW f32, anchors * (classes + 5) channels = the plan's filters).  Tensor-core plans
 * only; x channels-last in the plan's storage type.  The network object uses it wherever
 * nothing else reads the convolution's own output. */
int dnb_conv_yolo_forward(dnb_conv_plan *plan, const dnb_tensor *x, const dnb_tensor *y,
                          int anchors, int classes, void *stream);

/* Integer accumulators of an xnor plan, before scale/batchnorm/activation:
 * acc[b][n][oh][ow] (NCHW int32) = sum over in-bounds taps of sign(w)*sign(x).
 * What binarize + im2col + gemm produce in the reference
 * (src/convolutional_layer.c:451-456, :461-475) when mean|w| is factored out;
 * must match it bit for bit. */
int dnb_conv_xnor_accumulate(dnb_conv_plan *plan, const dnb_tensor *x, int32_t *acc, void *stream);

/* The xnor convolution for callers that may not allocate: no plan, no cudaMalloc,
 * cudaFree or allocating library call, on this or any later call.  Meant for hosts
 * whose device memory was handed out once at start-up (a serving loop with a fixed
 * arena, a plug-in inside a process that forbids allocation after initialisation).
 * The caller passes every input and output as device memory it owns:
 *   x       input, NCHW f32 or NHWC (f32 / bf16), extents as in desc
 *   wbits   [n][size*size][ceil(c/32)] words, bit (ch % 32) of word (ch / 32) set
 *           when weights[n][ch][kh][kw] > 0, other bits 0
 *   wmean   [n] mean |w| of each filter
 *   scale, shift  [n] folded batchnorm: out = act(acc * wmean * scale + shift)
 *           (scale 1 and shift = bias for a layer without batchnorm)
 *   y       output, NCHW f32 or NHWC
 * The bit-packed copy of the input, which the plan-based path keeps in memory it
 * allocates, lives here in a fixed 4 MiB array inside the library image (every GPU
 * that loads the library holds it until the process exits), so the layer must
 * satisfy batch*h*w*ceil(c/32) <= 1048576; larger layers are rejected with
 * DNB_EINVAL and need a plan.  The first call on a device looks the array's
 * address up; make that first call outside any stream capture.  All calls share
 * the one array and leave their packed input in it (each call rewrites every word
 * it reads, nothing needs clearing): two calls that overlap on the GPU, on
 * different streams or from different threads, race on it.
 * This entry point has no counterpart in the reference. */
int dnb_conv_xnor_forward_static(const dnb_conv_desc *desc, const dnb_tensor *x, const uint32_t *wbits,
                                 const float *wmean, const float *scale, const float *shift,
                                 const dnb_tensor *y, void *stream);

/* Reads and clears the plan's device status word (synchronises the device copy).
 * DNB_ETIMEOUT if a bounded wait inside the tensor-core kernel expired: the
 * kernel then left early and its output is incomplete.  The reference has no
 * counterpart (its kernels have no waits). */
int dnb_conv_plan_check_status(dnb_conv_plan *plan);

/* Diagnostics of a plan's device-side waits.  wait_limit_cycles: the bound of every
 * wait inside the plan's kernels in SM clock cycles (0 = the default, about one
 * second).  debug_bits: 0, or 32 to make every CTA of the tensor-core kernel withhold
 * one operand load so that a wait runs out; the launch then ends early with its
 * status word set, the context stays usable, and dnb_conv_plan_check_status /
 * dnb_network_collect report DNB_ETIMEOUT.  This is how the time-out path is
 * exercised (host-side injection: nothing faults, traps or hangs); other bits are
 * timing experiments and give wrong results.  The reference has no counterpart:
 * its kernels have no waits (src/convolutional_kernels.cu:73-135). */
int dnb_conv_plan_set_diagnostics(dnb_conv_plan *plan, long long wait_limit_cycles, int debug_bits);

/* Name of the kernel a plan dispatches to ("tc_tf32", "tc_bf16", "direct_fp32",
 * "xnor_popc"); static storage. */
const char *dnb_conv_plan_kernel(const dnb_conv_plan *plan);

/* One line about the plan for logs and tests, written to buf (at most len bytes with the
 * terminator): the kernel name and, for tensor-core plans after their first forward, the
 * tiling ("tc_tf32 pair=1 bn=256 tile=8x2x8 tiles=96 stages=6 ctas_per_sm=1 srb=128").
 * The reference prints a line per layer when it builds the network
 * (src/convolutional_layer.c:325). */
int dnb_conv_plan_describe(const dnb_conv_plan *plan, char *buf, int len);

/* ------------------------------------------------------------------ memory-bound layers */
/* All take tensors of one layout (both NCHW f32, or both NHWC of one dtype). */

/* Replaces forward_maxpool_layer_gpu (src/maxpool_layer_kernels.cu:87-97).
 * `padding` is Darknet's total padding (default size-1, src/parser.c:487);
 * y extents must be (x.h + padding - size)/stride + 1 (src/maxpool_layer.c:30-31).
 * The argmax `indexes` the reference also writes serve only backward and are
 * not produced. */
int dnb_maxpool_forward(const dnb_tensor *x, const dnb_tensor *y, int size, int stride,
                        int padding, void *stream);

/* Replaces forward_upsample_layer_gpu (src/upsample_layer.c:88-96: fill_gpu +
 * upsample_gpu, src/blas_kernels.cu:1007-1035), forward direction only. */
int dnb_upsample_forward(const dnb_tensor *x, const dnb_tensor *y, int stride, float scale,
                         void *stream);

/* Replaces forward_shortcut_layer_gpu (src/shortcut_layer.c:77-82: copy_gpu +
 * shortcut_gpu, src/blas_kernels.cu:711-745, + activate_array_gpu) in one pass:
 * y = act(alpha*x + beta*add) where `add` (the earlier layer's output) may
 * differ from x in width/height/channels as in shortcut_cpu (src/blas.c:68-92). */
int dnb_shortcut_forward(const dnb_tensor *x, const dnb_tensor *add, const dnb_tensor *y,
                         float alpha, float beta, int activation, void *stream);

/* Replaces forward_route_layer_gpu (src/route_layer.c:105-118; one copy_gpu per
 * input per image there): channel concatenation of `count` inputs in one launch
 * per input. */
int dnb_route_forward(const dnb_tensor *const *inputs, int count, const dnb_tensor *y, void *stream);

/* Layout / precision conversion between Darknet's NCHW f32 tensors and the
 * channels-last tensors used between layers.  No counterpart in the reference
 * (it is NCHW throughout).  round_tf32 != 0 rounds f32 results to the nearest
 * TF32 value so that the tensor cores' truncation is exact. */
int dnb_convert(const dnb_tensor *x, const dnb_tensor *y, int round_tf32, void *stream);

/* YOLO head, inference: replaces forward_yolo_layer_gpu's device work
 * (src/yolo_layer.c:347-358: copy_gpu + 2 activate_array_gpu per image per
 * anchor) in one launch.  x NCHW or NHWC; y NCHW f32 [n][anchors*(5+classes)][h][w]
 * with the logistic applied to entries 0,1 and 4..4+classes of every anchor. */
int dnb_yolo_forward(const dnb_tensor *x, const dnb_tensor *y, int anchors, int classes, void *stream);

/* Classifier tail.  Replace forward_avgpool_layer_gpu
 * (src/avgpool_layer_kernels.cu:46-52) and softmax_gpu (src/blas_kernels.cu:1006).
 * y of avgpool has h = w = 1. softmax needs h = w = 1 tensors. */
int dnb_avgpool_forward(const dnb_tensor *x, const dnb_tensor *y, void *stream);
int dnb_softmax_forward(const dnb_tensor *x, const dnb_tensor *y, int groups, float temperature,
                        void *stream);

/* ------------------------------------------------------------------ network */
typedef struct dnb_network dnb_network;

/* parse_network_cfg (src/parser.c:742-889) for the layer types on this path:
 * [net], [convolutional], [maxpool], [upsample], [shortcut], [route], [yolo],
 * [avgpool], [connected], [softmax].  Any other section fails with DNB_EUNSUPPORTED.
 * A [connected] layer (src/connected_layer.c:288-306) runs on the convolution kernels as
 * a 1x1 convolution over the flattened input with the batch folded into the pixel tile.
 * batch_override > 0 replaces the cfg's batch/subdivisions (the reference needs
 * an edited cfg for that, src/parser.c:664).  Allocates every layer's output on
 * the current device. */
int dnb_parse_network_cfg(const char *cfg_path, int mode, int batch_override, dnb_network **net);
/* Same, from cfg text in memory. */
int dnb_parse_network_cfg_text(const char *cfg_text, int mode, int batch_override, dnb_network **net);

/* load_weights (src/parser.c:1308, :1218-1306): reads the .weights file and
 * builds every convolution's and connected layer's derived device tensors.  Both
 * header forms (32- and 64-bit `seen`, :1234-1241), files whose version marks
 * transposed connected-layer matrices (major or minor above 1000, :1244, :1098-1104) and
 * convolutions declared flipped=1 in the cfg (:1206-1208) are read as the reference
 * reads them. */
int dnb_load_weights(dnb_network *net, const char *weights_path);

/* load_weights for a file in which every convolution with xnor=1 is stored in the reference's packed-binary layer
 * format (load_convolutional_weights_binary / save_convolutional_weights_binary, src/parser.c:1134-1162, 926-956:
 * biases and batchnorm vectors as usual, then per filter its mean |w| as a float and one bit per weight, eight to a
 * byte, lowest bit first; set = +mean).  The reference carries the format but leaves its call sites commented out
 * (src/parser.c:961, 1167); it is the natural on-disk form of an xnor network, 32 times smaller.  Filters whose
 * c*size*size is not a multiple of 8 are refused (the reference's size/8 bytes per filter would drop their tail). */
int dnb_load_weights_packed(dnb_network *net, const char *weights_path);

/* load_weights for a host that already holds the parameters in memory: the arrays the reference's
 * load_convolutional_weights fills (src/parser.c:1164-1215) for convolution `layer`, or load_connected_weights
 * (src/parser.c:1098-1120; weights [outputs][inputs]) for a connected layer.  Once every such layer
 * of the network has been given its parameters the network is ready to predict. */
int dnb_network_set_conv_params(dnb_network *net, int layer, const float *weights, const float *biases,
                                const float *scales, const float *rolling_mean, const float *rolling_variance);

/* free_network (src/network.c:720-735). */
void dnb_free_network(dnb_network *net);

/* network_predict (src/network.c:497-508) with HOST buffers: copies `input`
 * (batch*inputs floats, NCHW) to the device, runs forward_network_gpu's loop
 * (src/network.c:762-788) with this library's kernels, copies the output layer
 * (the last layer, as get_network_output_layer picks it, src/network.c:699-706)
 * and every [yolo] layer's output back.  *output points at host memory owned
 * by the network, batch*outputs floats, valid until the next call. */
int dnb_network_predict(dnb_network *net, const float *input, float **output);

/* network_predict split in two so that a caller streaming batches (the loop of
 * validate_detector, examples/detector.c:420-520, or predict_classifier's) hides
 * the host copies: dnb_network_submit enqueues upload, forward and the result
 * copies of one step and returns; dnb_network_collect waits for the OLDEST
 * submitted step and hands out its results as dnb_network_predict does.  At most
 * two steps may be in flight (a third submit returns DNB_EINVAL); the results of
 * a collected step (and dnb_network_yolo_output's pointers) stay valid until the
 * step after the next one is submitted.  `input` should be pinned host memory
 * and must stay untouched until the step is collected.  No counterpart in the
 * reference, whose network_predict blocks on every pull (src/cuda.c:160-165). */
int dnb_network_submit(dnb_network *net, const float *input);
int dnb_network_collect(dnb_network *net, float **output);

/* The device-resident part alone: input already on the device (NCHW f32,
 * batch*inputs floats), no host copies, asynchronous on `stream` (NULL = the
 * legacy default stream). */
int dnb_network_forward(dnb_network *net, const float *device_input, void *stream);

/* Replay dnb_network_forward as a CUDA graph: with `on`, the second call with the same input pointer and
 * (non-NULL) stream is captured and every later one is one graph launch; a different pointer or stream
 * starts over.  For small batches, where the launches of forward_network_gpu's loop (src/network.c:772-785)
 * cost more than the kernels.  No counterpart in the reference. */
int dnb_network_enable_graph(dnb_network *net, int on);

/* Waits for the device, then reads and clears the network's status words:
 * DNB_ETIMEOUT if a bounded wait expired in a convolution since the last check (its
 * outputs are incomplete).  For callers of dnb_network_forward, which returns before
 * its kernels ran; dnb_network_collect / dnb_network_predict report the same for
 * their own step.  check_error(cudaPeekAtLastError()) after each launch is the
 * nearest thing in the reference (src/cuda.c:27-49). */
int dnb_network_check_status(dnb_network *net);

/* dnb_conv_plan_set_diagnostics for convolution `layer` of the network. */
int dnb_network_set_diagnostics(dnb_network *net, int layer, long long wait_limit_cycles, int debug_bits);

/* Geometry queries (net->n, net->batch, net->inputs, net->outputs; layer
 * out_c/out_h/out_w/outputs and type as the section name, e.g. "convolutional"). */
int dnb_network_num_layers(const dnb_network *net);
int dnb_network_batch(const dnb_network *net);
int dnb_network_inputs(const dnb_network *net);
int dnb_network_outputs(const dnb_network *net);
int dnb_network_layer_shape(const dnb_network *net, int layer, int *out_c, int *out_h, int *out_w);
const char *dnb_network_layer_type(const dnb_network *net, int layer);
const char *dnb_network_layer_kernel(const dnb_network *net, int layer);
/* dnb_conv_plan_describe for a convolutional layer, the section name for the others. */
int dnb_network_layer_describe(const dnb_network *net, int layer, char *buf, int len);

/* Copy layer `layer`'s current output to host memory as Darknet lays it out
 * (NCHW f32, batch*outputs floats): what reading l.output after
 * cuda_pull_array (src/cuda.c:160-165) gives in the reference. */
int dnb_network_layer_output(dnb_network *net, int layer, float *host_out);
/* The same into device memory of the caller (what l.output_gpu holds in the reference), asynchronously on
 * `stream`: the hook an attach shim uses to hand results to layers the reference still runs. */
int dnb_network_export_layer(dnb_network *net, int layer, float *device_nchw, void *stream);

/* Images [first, first+count) of that output only: count*outputs floats.  For
 * checking a few images of a large batch without pulling whole layers. */
int dnb_network_layer_output_images(dnb_network *net, int layer, int first, int count, float *host_out);

/* Host pointer to a [yolo] layer's output of the last predict (the reference
 * pulls it inside forward_yolo_layer_gpu, src/yolo_layer.c:360). */
int dnb_network_yolo_output(dnb_network *net, int layer, const float **host_out);

/* Algorithmic FLOPs of one forward of the whole batch, counted as the
 * reference's `ops` command does (examples/darknet.c:81-114). */
double dnb_network_flops(const dnb_network *net);

/* Number of kernel launches one dnb_network_forward issues. */
int dnb_network_launches(const dnb_network *net);

/* dnb_network_forward with a CUDA event recorded between layers; asynchronous.
 * `slot` (0..4096) names an independent set of events, so that several timed
 * forwards can be queued before any is read.  dnb_network_timed_ms waits for
 * the forward recorded in `slot` and returns each layer's device time in
 * milliseconds.  dnb_network_profile = one timed forward on the network's own
 * stream, read back at once.  The reference has only a whole-network
 * wall-clock timer (examples/darknet.c:116-134, the `speed` command). */
int dnb_network_forward_timed(dnb_network *net, const float *device_input, void *stream, int slot);
int dnb_network_timed_ms(dnb_network *net, int slot, float *layer_ms);
int dnb_network_profile(dnb_network *net, const float *device_input, float *layer_ms);

#ifdef __cplusplus
}
#endif
#endif /* DARKNET_B200_H */
