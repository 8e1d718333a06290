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
 * Errors follow the reference's convention: print and exit through error() (src/utils.c:253-258).
 */
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

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

static void forward_convolutional_layer_b200(layer l, network net)
{
    attached *a = find_attached(net.layers);
    if (!a || net.index < 0 || net.index >= a->n || !a->plans[net.index]) error("darknet_b200: convolution called on a network that is not attached");
    dnb_tensor x = nchw(net.input_gpu, l.batch, l.c, l.h, l.w);
    dnb_tensor y = nchw(l.output_gpu, l.batch, l.out_c, l.out_h, l.out_w);
    if (dnb_conv_forward(a->plans[net.index], &x, &y, NULL, NULL)) fail("convolution");
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

static int route_is_covered(const network *net, const layer *l)
{
    if (l->n < 1 || l->n > 16) return 0;
    for (int i = 0; i < l->n; ++i) {
        const layer *s = &net->layers[l->input_layers[i]];
        if (s->out_h != l->out_h || s->out_w != l->out_w || !s->output_gpu) return 0;
    }
    return 1;
}

static void release(attached *a, network *net)
{
    for (int i = 0; i < a->n; ++i) {
        if (net && a->original[i]) net->layers[i].forward_gpu = a->original[i];
        if (a->plans[i]) dnb_conv_plan_destroy(a->plans[i]);
    }
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
    a->plans = calloc(net->n, sizeof *a->plans);
    a->original = calloc(net->n, sizeof *a->original);
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
        }
        if (repl) {
            a->original[i] = l->forward_gpu;
            l->forward_gpu = repl;
            ++count;
        }
    }
    a->next = g_attached;
    g_attached = a;
    return count;
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
