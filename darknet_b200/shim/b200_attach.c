/*
 * Drop-in shim for an unmodified Darknet GPU build: see include/b200_attach.h.
 *
 * Compiled with the Darknet tree's own flags and header:
 *     gcc -DGPU -I<darknet>/include -I<cuda>/include -I<this repo>/include -c b200_attach.c
 * and linked with libdarknet (GPU build) and libdarknet_b200.so.
 *
 * Each replacement has the signature of the pointer it replaces,
 *     void (*forward_gpu)(struct layer, struct network);            include/darknet.h:122
 * and does what the reference's function of that layer type does on the forward path:
 *     forward_convolutional_layer_gpu   src/convolutional_kernels.cu:73-135
 *     forward_maxpool_layer_gpu         src/maxpool_layer_kernels.cu:87-97
 *     forward_upsample_layer_gpu        src/upsample_layer.c:88-96
 *     forward_shortcut_layer_gpu        src/shortcut_layer.c:75-80
 *     forward_route_layer_gpu           src/route_layer.c:105-118
 *     forward_yolo_layer_gpu            src/yolo_layer.c:347-362 (the inference branch: activations, then the pull)
 * Errors follow the reference's convention: print and exit through error() (src/utils.c:253-258).
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <cuda_runtime_api.h>

#include "darknet.h"

#include "b200_attach.h"
#include "darknet_b200.h"

#ifndef GPU
#error "b200_attach.c belongs in a Darknet GPU build: compile it with -DGPU"
#endif

typedef void (*forward_fn)(layer, network);

/* One record per attached network, found again through net.layers (the by-value copies that
 * forward_gpu receives share that pointer with the caller's network). */
typedef struct attached {
    layer *layers;
    int n;
    dnb_conv_plan **plans;      /* per layer, NULL where the layer is not a replaced convolution */
    forward_fn *original;       /* per layer, the pointer that was there before */
    dnb_network *whole;         /* b200_attach_network: this library's own network object, or NULL */
    float **saved_delta;        /* b200_attach_network: the delta_gpu pointers taken out of the layers */
    char *pinned;               /* per layer: l.output was page-locked here (and is released by b200_detach) */
    void **shadow;              /* per layer: channels-last copy of a replaced convolution's output that the next
                                 * replaced convolution reads instead of transposing l.output_gpu again, or NULL */
    int mode;
    struct attached *next;
} attached;

static attached *g_attached = NULL;

static attached *find_attached(const layer *layers)
{
    for (attached *a = g_attached; a; a = a->next)
        if (a->layers == layers) return a;
    return NULL;
}

static void fail(const char *what)
{
    char msg[1024];
    snprintf(msg, sizeof msg, "darknet_b200 %s: %s", what, dnb_last_error());
    error(msg);
}

static dnb_tensor nchw(float *gpu, int n, int c, int h, int w)
{
    dnb_tensor t;
    t.data = gpu; t.layout = DNB_NCHW; t.dtype = DNB_F32;
    t.n = n; t.c = c; t.h = h; t.w = w; t.cpitch = 0;
    return t;
}

static dnb_tensor nhwc(void *gpu, int mode, int n, int c, int h, int w)
{
    dnb_tensor t;
    t.data = gpu; t.layout = DNB_NHWC; t.dtype = mode == DNB_MODE_BF16 ? DNB_BF16 : DNB_F32;
    t.n = n; t.c = c; t.h = h; t.w = w; t.cpitch = (c + 7) / 8 * 8;
    return t;
}

/* Darknet's tensors are NCHW, the tensor-core kernel reads channels-last: a replaced convolution transposes its
 * input into a scratch of its plan first.  Where the layer before it is a replaced convolution too, that layer has
 * written a channels-last copy of its output beside l.output_gpu (the second output of dnb_conv_forward), and this
 * one reads the copy; l.output_gpu is still written for every other reader. */
static void forward_convolutional_layer_b200(layer l, network net)
{
    attached *a = find_attached(net.layers);
    const int i = net.index;
    if (!a || i < 0 || i >= a->n || !a->plans[i]) error("darknet_b200: convolution called on a network that is not attached");
    dnb_tensor x = nchw(net.input_gpu, l.batch, l.c, l.h, l.w);
    if (i > 0 && a->shadow[i - 1] && net.input_gpu == net.layers[i - 1].output_gpu)
        x = nhwc(a->shadow[i - 1], a->mode, l.batch, l.c, l.h, l.w);
    dnb_tensor y = nchw(l.output_gpu, l.batch, l.out_c, l.out_h, l.out_w);
    dnb_tensor y2 = nhwc(a->shadow[i], a->mode, l.batch, l.out_c, l.out_h, l.out_w);
    if (dnb_conv_forward(a->plans[i], &x, &y, a->shadow[i] ? &y2 : NULL, NULL)) fail("convolution");
}

static void forward_maxpool_layer_b200(layer l, network net)
{
    dnb_tensor x = nchw(net.input_gpu, l.batch, l.c, l.h, l.w);
    dnb_tensor y = nchw(l.output_gpu, l.batch, l.out_c, l.out_h, l.out_w);
    if (dnb_maxpool_forward(&x, &y, l.size, l.stride, l.pad, NULL)) fail("maxpool");
}

static void forward_upsample_layer_b200(layer l, network net)
{
    dnb_tensor x = nchw(net.input_gpu, l.batch, l.c, l.h, l.w);
    dnb_tensor y = nchw(l.output_gpu, l.batch, l.out_c, l.out_h, l.out_w);
    if (dnb_upsample_forward(&x, &y, l.stride, l.scale, NULL)) fail("upsample");
}

static void forward_shortcut_layer_b200(layer l, network net)
{
    layer f = net.layers[l.index];
    /* l.w, l.h, l.c describe the `from` tensor, l.out_* this layer's input and output (make_shortcut_layer, src/shortcut_layer.c:9-38) */
    dnb_tensor x = nchw(net.input_gpu, l.batch, l.out_c, l.out_h, l.out_w);
    dnb_tensor add = nchw(f.output_gpu, l.batch, l.c, l.h, l.w);
    dnb_tensor y = nchw(l.output_gpu, l.batch, l.out_c, l.out_h, l.out_w);
    if (dnb_shortcut_forward(&x, &add, &y, l.alpha, l.beta, (int)l.activation, NULL)) fail("shortcut");
}

static void forward_route_layer_b200(layer l, network net)
{
    dnb_tensor in[16];
    const dnb_tensor *ptrs[16];
    for (int i = 0; i < l.n; ++i) {
        layer s = net.layers[l.input_layers[i]];
        in[i] = nchw(s.output_gpu, l.batch, s.out_c, s.out_h, s.out_w);
        ptrs[i] = &in[i];
    }
    dnb_tensor y = nchw(l.output_gpu, l.batch, l.out_c, l.out_h, l.out_w);
    if (dnb_route_forward(ptrs, l.n, &y, NULL)) fail("route");
}

/* forward_yolo_layer_gpu at inference (src/yolo_layer.c:347-362): copy the input, apply the logistic to the x, y,
 * objectness and class entries of every anchor (2 * batch * anchors launches there, one here), pull the result to
 * l.output, where get_yolo_detections reads it (src/yolo_layer.c:316-343). */
static void forward_yolo_layer_b200(layer l, network net)
{
    if (net.train && !l.onlyforward) {   /* the training branch (loss on the host) stays the reference's */
        attached *a = find_attached(net.layers);
        if (!a || net.index < 0 || net.index >= a->n || !a->original[net.index]) error("darknet_b200: yolo layer called on a network that is not attached");
        a->original[net.index](l, net);
        return;
    }
    dnb_tensor x = nchw(net.input_gpu, l.batch, l.c, l.h, l.w);
    dnb_tensor y = nchw(l.output_gpu, l.batch, l.c, l.h, l.w);
    if (dnb_yolo_forward(&x, &y, l.n, l.classes, NULL)) fail("yolo");
    cuda_pull_array(l.output_gpu, l.output, (size_t)l.batch * l.outputs);
}

static int route_is_covered(const network *net, const layer *l)
{
    if (l->n < 1 || l->n > 16) return 0;
    for (int i = 0; i < l->n; ++i) {
        const layer *s = &net->layers[l->input_layers[i]];
        if (s->out_h != l->out_h || s->out_w != l->out_w || !s->output_gpu) return 0;
    }
    return 1;
}

/* Darknet pulls results with a blocking cudaMemcpy into calloc'd host arrays (cuda_pull_array, src/cuda.c:160-165):
 * from pageable memory that runs at a fraction of the link's rate.  The arrays it pulls at inference, every
 * [yolo] layer's l.output and the last layer's, are page-locked in place while the network is attached. */
static void pin_outputs(attached *a, network *net)
{
    a->pinned = calloc((size_t)net->n, 1);
    for (int i = 0; i < net->n; ++i) {
        layer *l = &net->layers[i];
        if ((l->type != YOLO && i != net->n - 1) || !l->output) continue;
        if (cudaHostRegister(l->output, (size_t)l->batch * l->outputs * sizeof(float), cudaHostRegisterDefault) == cudaSuccess) a->pinned[i] = 1;
        else cudaGetLastError();   /* already locked or refused: the pull stays as slow as it was */
    }
}

static void release(attached *a, network *net)
{
    for (int i = 0; i < a->n; ++i) {
        if (net && a->pinned && a->pinned[i]) cudaHostUnregister(net->layers[i].output);
        if (net && a->original[i]) net->layers[i].forward_gpu = a->original[i];
        if (net && a->saved_delta && a->saved_delta[i]) net->layers[i].delta_gpu = a->saved_delta[i];
        if (a->plans[i]) dnb_conv_plan_destroy(a->plans[i]);
        if (a->shadow && a->shadow[i]) cudaFree(a->shadow[i]);
    }
    if (a->whole) dnb_free_network(a->whole);
    free(a->pinned);
    free(a->shadow);
    free(a->saved_delta);
    free(a->plans);
    free(a->original);
    free(a);
}

int b200_attach(network *net, int mode)
{
    if (!net || net->n < 1 || find_attached(net->layers)) return -1;
    attached *a = calloc(1, sizeof *a);
    a->layers = net->layers;
    a->n = net->n;
    a->plans = calloc((size_t)net->n, sizeof *a->plans);
    a->original = calloc((size_t)net->n, sizeof *a->original);
    a->shadow = calloc((size_t)net->n, sizeof *a->shadow);
    a->mode = mode;
    int count = 0;
    for (int i = 0; i < net->n; ++i) {
        layer *l = &net->layers[i];
        forward_fn repl = NULL;
        if (l->type == CONVOLUTIONAL) {
            if (l->binary && !l->xnor) continue;                 /* weight-only binarisation stays with the reference */
            if (l->size == 1 && l->stride > 1) continue;         /* see dnb_conv_plan_create */
            dnb_conv_desc d;
            d.batch = l->batch; d.h = l->h; d.w = l->w; d.c = l->c;
            d.n = l->n; d.groups = l->groups; d.size = l->size; d.stride = l->stride; d.pad = l->pad;
            d.batch_normalize = l->batch_normalize; d.activation = (int)l->activation; d.xnor = l->xnor;
            if (dnb_conv_plan_create(&d, mode, &a->plans[i])) { release(a, net); return -1; }
            /* the host copies load_weights filled (src/parser.c:1164-1215) */
            if (dnb_conv_plan_set_params(a->plans[i], l->weights, l->biases,
                                         l->batch_normalize ? l->scales : NULL,
                                         l->batch_normalize ? l->rolling_mean : NULL,
                                         l->batch_normalize ? l->rolling_variance : NULL)) { release(a, net); return -1; }
            repl = forward_convolutional_layer_b200;
        } else if (l->type == MAXPOOL) {
            repl = forward_maxpool_layer_b200;
        } else if (l->type == UPSAMPLE && !l->reverse) {
            repl = forward_upsample_layer_b200;
        } else if (l->type == SHORTCUT) {
            repl = forward_shortcut_layer_b200;
        } else if (l->type == ROUTE && route_is_covered(net, l)) {
            repl = forward_route_layer_b200;
        } else if (l->type == YOLO && l->c == l->n * (l->classes + 4 + 1) && l->output && l->output_gpu) {
            repl = forward_yolo_layer_b200;
        }
        if (repl) {
            a->original[i] = l->forward_gpu;
            l->forward_gpu = repl;
            ++count;
        }
    }
    /* channels-last copies between consecutive replaced convolutions (tensor-core plans, whose kernels read and write
     * that layout); B200_ATTACH_SHADOWS=0 in the environment keeps every boundary in Darknet's layout only */
    {
        const char *e = getenv("B200_ATTACH_SHADOWS");
        for (int i = 0; i + 1 < net->n && !(e && atoi(e) == 0); ++i) {
            const layer *l = &net->layers[i];
            if (!a->plans[i] || !a->plans[i + 1]) continue;
            const char *k0 = dnb_conv_plan_kernel(a->plans[i]), *k1 = dnb_conv_plan_kernel(a->plans[i + 1]);
            if (strncmp(k0, "tc_", 3) || strncmp(k1, "tc_", 3)) continue;
            const size_t bytes = (size_t)l->batch * l->out_h * l->out_w * ((l->out_c + 7) / 8 * 8) * (mode == DNB_MODE_BF16 ? 2 : 4);
            if (cudaMalloc(&a->shadow[i], bytes) != cudaSuccess) { cudaGetLastError(); a->shadow[i] = NULL; break; }   /* out of memory: the rest stay as they were */
            if (cudaMemset(a->shadow[i], 0, bytes) != cudaSuccess) cudaGetLastError();                                /* padding channels are zero */
        }
    }
    /* inference only from here to b200_detach: forward_network_gpu zero-fills every layer's delta before calling
     * it (src/network.c:775-777), 30 GB per YOLOv3-608 batch of 64; with the pointers set aside it has nothing to clear */
    a->saved_delta = calloc((size_t)net->n, sizeof *a->saved_delta);
    for (int i = 0; i < net->n; ++i) {
        a->saved_delta[i] = net->layers[i].delta_gpu;
        net->layers[i].delta_gpu = NULL;
    }
    pin_outputs(a, net);
    a->next = g_attached;
    g_attached = a;
    return count;
}

/* ------------------------------------------------------------------ whole-network attach
 * The per-layer form above keeps Darknet's tensors (NCHW fp32) at every layer boundary, and Darknet's loop
 * zero-fills every layer's delta before calling it (src/network.c:775-777).  This form hands the whole forward
 * pass to the library's own network object (channels-last between layers, shortcuts fused into convolutions):
 * layer 0's forward_gpu runs all layers and writes Darknet's l.output_gpu only where the reference still looks,
 * i.e. every [yolo] layer (whose host copy the detection code reads) and the last layer (which
 * pull_network_output copies, src/network.c:786); every other forward_gpu becomes a no-op and the delta_gpu
 * pointers are set aside so that the loop has nothing to clear.  Intermediate l.output_gpu buffers are then
 * not written: a host that reads them uses b200_attach instead. */
static const char *const kActivationNames[] = {"logistic", "relu", "relie", "linear", "ramp", "tanh", "plse",
                                               "leaky", "elu", "loggy", "stair", "hardtan", "lhtan", "selu"};

/* The cfg text of the network as the structs describe it (sizes and indices resolved), or NULL when a layer
 * type is outside the convolutional forward path. */
static char *cfg_from_structs(const network *net)
{
    size_t cap = 4096 + (size_t)net->n * 512, len = 0;
    char *t = malloc(cap);
    if (!t) return NULL;
    len += snprintf(t + len, cap - len, "[net]\nbatch=%d\nsubdivisions=1\nheight=%d\nwidth=%d\nchannels=%d\n", net->batch, net->h, net->w, net->c);
    for (int i = 0; i < net->n; ++i) {
        const layer *l = &net->layers[i];
        if (cap - len < 1024) { free(t); return NULL; }
        if ((int)l->activation < 0 || (int)l->activation > 13) { free(t); return NULL; }
        const char *act = kActivationNames[(int)l->activation];
        switch (l->type) {
        case CONVOLUTIONAL:
            if (l->binary && !l->xnor) { free(t); return NULL; }
            len += snprintf(t + len, cap - len, "[convolutional]\nbatch_normalize=%d\nfilters=%d\nsize=%d\nstride=%d\npadding=%d\ngroups=%d\nactivation=%s\nxnor=%d\n",
                            l->batch_normalize, l->n, l->size, l->stride, l->pad, l->groups, act, l->xnor);
            break;
        case MAXPOOL:
            len += snprintf(t + len, cap - len, "[maxpool]\nsize=%d\nstride=%d\npadding=%d\n", l->size, l->stride, l->pad);
            break;
        case UPSAMPLE:
            if (l->reverse) { free(t); return NULL; }
            len += snprintf(t + len, cap - len, "[upsample]\nstride=%d\nscale=%.9g\n", l->stride, l->scale);
            break;
        case SHORTCUT:
            len += snprintf(t + len, cap - len, "[shortcut]\nfrom=%d\nalpha=%.9g\nbeta=%.9g\nactivation=%s\n", l->index, l->alpha, l->beta, act);
            break;
        case ROUTE:
            len += snprintf(t + len, cap - len, "[route]\nlayers=");
            for (int k = 0; k < l->n; ++k) len += snprintf(t + len, cap - len, "%s%d", k ? "," : "", l->input_layers[k]);
            len += snprintf(t + len, cap - len, "\n");
            break;
        case YOLO:
            len += snprintf(t + len, cap - len, "[yolo]\nmask=");
            for (int k = 0; k < l->n; ++k) len += snprintf(t + len, cap - len, "%s%d", k ? "," : "", l->mask ? l->mask[k] : k);
            len += snprintf(t + len, cap - len, "\nnum=%d\nclasses=%d\n", l->total, l->classes);
            break;
        case AVGPOOL:
            len += snprintf(t + len, cap - len, "[avgpool]\n");
            break;
        case SOFTMAX:
            if (l->softmax_tree) { free(t); return NULL; }
            len += snprintf(t + len, cap - len, "[softmax]\ngroups=%d\ntemperature=%.9g\n", l->groups, l->temperature);
            break;
        default:
            free(t);
            return NULL;
        }
    }
    return t;
}

static void forward_whole_network_b200(layer l, network net)
{
    attached *a = find_attached(net.layers);
    if (!a || !a->whole) error("darknet_b200: network called without being attached");
    (void)l;
    if (dnb_network_forward(a->whole, net.input_gpu, NULL)) fail("network");
    for (int i = 0; i < a->n; ++i)
        if (net.layers[i].type == YOLO || i == a->n - 1)
            if (dnb_network_export_layer(a->whole, i, net.layers[i].output_gpu, NULL)) fail("export");
}

static void forward_nothing_b200(layer l, network net) { (void)l; (void)net; }

/* What forward_yolo_layer_gpu leaves behind at inference (src/yolo_layer.c:347-362): the activated tensor in
 * l.output_gpu, already written by layer 0's call, and its host copy in l.output. */
static void forward_yolo_pull_b200(layer l, network net)
{
    (void)net;
    cuda_pull_array(l.output_gpu, l.output, (size_t)l.batch * l.outputs);
}

int b200_attach_network(network *net, int mode)
{
    if (!net || net->n < 1 || find_attached(net->layers)) return -1;
    const size_t count = (size_t)net->n;
    char *cfg = cfg_from_structs(net);
    if (!cfg) return -1;
    dnb_network *whole = NULL;
    int rc = dnb_parse_network_cfg_text(cfg, mode, 0, &whole);
    free(cfg);
    if (rc) return -1;
    for (int i = 0; i < net->n && !rc; ++i) {
        layer *l = &net->layers[i];
        if (l->type != CONVOLUTIONAL) continue;
        rc = dnb_network_set_conv_params(whole, i, l->weights, l->biases, l->batch_normalize ? l->scales : NULL,
                                         l->batch_normalize ? l->rolling_mean : NULL, l->batch_normalize ? l->rolling_variance : NULL);
    }
    if (rc) { dnb_free_network(whole); return -1; }
    attached *a = calloc(1, sizeof *a);
    a->layers = net->layers;
    a->n = net->n;
    a->plans = calloc(count, sizeof *a->plans);
    a->original = calloc(count, sizeof *a->original);
    a->saved_delta = calloc(count, sizeof *a->saved_delta);
    a->shadow = calloc(count, sizeof *a->shadow);
    a->mode = mode;
    a->whole = whole;
    for (int i = 0; i < net->n; ++i) {
        layer *l = &net->layers[i];
        a->original[i] = l->forward_gpu;
        a->saved_delta[i] = l->delta_gpu;
        l->delta_gpu = NULL;
        l->forward_gpu = i == 0 ? forward_whole_network_b200 : (l->type == YOLO ? forward_yolo_pull_b200 : forward_nothing_b200);
    }
    pin_outputs(a, net);
    a->next = g_attached;
    g_attached = a;
    return net->n;
}

void b200_detach(network *net)
{
    if (!net) return;
    attached **pp = &g_attached;
    while (*pp && (*pp)->layers != net->layers) pp = &(*pp)->next;
    if (!*pp) return;
    attached *a = *pp;
    *pp = a->next;
    release(a, net);
}
