/*
 * Thin C harness around the UNMODIFIED reference (pjreddie/darknet): the CPU build, and with -DGPU
 * the reference's own CUDA build (im2col + cuBLAS, recompiled for sm_100a) plus the attach shim.
 *
 * TEST INFRASTRUCTURE ONLY.  Compiled against the reference's own public
 * header (include/darknet.h) and linked with objects built from the
 * reference's own sources where they lie; nothing of the reference is copied
 * here.  It flattens the reference's by-value struct API into plain pointers
 * and ints so that Python (ctypes) can drive parse_network_cfg / load_weights /
 * network_predict and read every layer's output.
 *
 * The product library never links or loads this file.
 */
#include <omp.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "darknet.h"

/* parse_network_cfg (src/parser.c:742) + load_weights (src/parser.c:1308).
 * weights may be NULL or "" to keep the constructor's random initialisation. */
void *ref_load_network(const char *cfg, const char *weights)
{
    network *net = parse_network_cfg((char *)cfg);
    if (weights && weights[0]) load_weights(net, (char *)weights);
    return net;
}

void ref_free_network(void *h) { free_network((network *)h); }

int ref_num_layers(void *h) { return ((network *)h)->n; }
int ref_batch(void *h) { return ((network *)h)->batch; }
int ref_inputs(void *h) { return ((network *)h)->inputs; }
int ref_outputs(void *h) { return ((network *)h)->outputs; }

/* info[0..7] = type, out_c, out_h, out_w, outputs, batch, n, size */
void ref_layer_info(void *h, int i, int *info)
{
    layer *l = &((network *)h)->layers[i];
    info[0] = (int)l->type; info[1] = l->out_c; info[2] = l->out_h; info[3] = l->out_w;
    info[4] = l->outputs;   info[5] = l->batch; info[6] = l->n;     info[7] = l->size;
}

/* Pointer to layer i's host output buffer, outputs*batch floats.  In the GPU build the device copy
 * is pulled first (cuda_pull_array, src/cuda.c:160-165). */
float *ref_layer_output(void *h, int i)
{
    layer *l = &((network *)h)->layers[i];
#ifdef GPU
    if (l->output_gpu && l->output) cuda_pull_array(l->output_gpu, l->output, (size_t)l->outputs * l->batch);
#endif
    return l->output;
}

#ifdef GPU
#include "b200_attach.h"
/* The drop-in under test: re-point the network's forward_gpu pointers at libdarknet_b200. */
int ref_attach_b200(void *h, int mode) { return b200_attach((network *)h, mode); }
int ref_attach_network_b200(void *h, int mode) { return b200_attach_network((network *)h, mode); }
void ref_detach_b200(void *h) { b200_detach((network *)h); }
int ref_is_gpu_build(void) { return 1; }
#else
int ref_is_gpu_build(void) { return 0; }
#endif

/* network_predict (src/network.c:497-508): returns the last layer's output. */
float *ref_network_predict(void *h, float *input) { return network_predict((network *)h, input); }
void ref_save_weights(void *h, char *path) { save_weights((network *)h, path); }

/* The reference's packed-binary layer writer and reader (src/parser.c:926-956, 1134-1162), which its own
 * save_weights / load_weights leave commented out: layer i of the network to / from a file of its own. */
void save_convolutional_weights_binary(layer l, FILE *fp);
void load_convolutional_weights_binary(layer l, FILE *fp);
int ref_save_conv_binary(void *h, int i, const char *path)
{
    network *net = (network *)h;
    FILE *fp = fopen(path, "wb");
    if (!fp || i < 0 || i >= net->n || net->layers[i].type != CONVOLUTIONAL || !net->layers[i].binary_weights) { if (fp) fclose(fp); return -1; }
    save_convolutional_weights_binary(net->layers[i], fp);
    fclose(fp);
    return 0;
}
int ref_load_conv_binary(void *h, int i, const char *path)
{
    network *net = (network *)h;
    FILE *fp = fopen(path, "rb");
    if (!fp || i < 0 || i >= net->n || net->layers[i].type != CONVOLUTIONAL) { if (fp) fclose(fp); return -1; }
    load_convolutional_weights_binary(net->layers[i], fp);
    fclose(fp);
    return 0;
}
float *ref_layer_weights(void *h, int i) { return ((network *)h)->layers[i].weights; }

void ref_set_threads(int n) { omp_set_num_threads(n); }
int ref_max_threads(void) { return omp_get_max_threads(); }

/* Wall-clock seconds of `reps` network_predict calls (reference's own timer,
 * src/utils.c:27-34). */
double ref_time_predict(void *h, float *input, int reps)
{
    double t0 = what_time_is_it_now();
    for (int i = 0; i < reps; ++i) network_predict((network *)h, input);
    return what_time_is_it_now() - t0;
}

/* Direct access to the two primitives the oracle restates, for pinning them
 * one by one: im2col_cpu (src/im2col.c:16) and gemm (src/gemm.c:65). */
void im2col_cpu(float *data_im, int channels, int height, int width, int ksize, int stride, int pad, float *data_col);
void gemm(int TA, int TB, int M, int N, int K, float ALPHA, float *A, int lda, float *B, int ldb, float BETA, float *C, int ldc);
void ref_im2col(float *im, int c, int h, int w, int k, int s, int p, float *col) { im2col_cpu(im, c, h, w, k, s, p, col); }
void ref_gemm_nn(int M, int N, int K, float *A, float *B, float *C) { gemm(0, 0, M, N, K, 1, A, K, B, N, 1, C, N); }
