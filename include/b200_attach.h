/*
 * b200_attach.h -- re-points the forward_gpu function pointers of an UNMODIFIED Darknet `network`
 * (GPU build, -DGPU, no -DCUDNN) at the kernels of libdarknet_b200.
 *
 * Darknet calls l.forward_gpu(l, net) for every layer from forward_network_gpu (src/network.c:772-785),
 * structs by value (include/darknet.h:119-124).  After parse_network_cfg + load_weights a host calls
 * b200_attach(net, mode); from then on network_predict (src/network.c:497-508) runs the convolutional,
 * maxpool, upsample, shortcut and route layers through this library, reading and writing Darknet's own
 * device buffers (net.input_gpu, l.output_gpu: NCHW fp32).  Every other layer type keeps the
 * reference's kernel.  The file that implements this, darknet_b200/shim/b200_attach.c, is compiled inside
 * the Darknet tree (it includes darknet.h, whose struct layout depends on the build flags).
 */
#ifndef B200_ATTACH_H
#define B200_ATTACH_H

#ifdef __cplusplus
extern "C" {
#endif

struct network;

/* mode: a dnb_mode (DNB_MODE_TF32, DNB_MODE_BF16 or DNB_MODE_FP32).  Returns the number of layers whose
 * forward_gpu now points into this library, or -1 with the reason in dnb_last_error().  On failure the
 * network is left as it was.  Layers it does not cover (convolutions with l.binary only, 1x1 with
 * stride > 1, reverse upsample, routes over inputs of unequal size) keep the reference's pointer. */
int b200_attach(struct network *net, int mode);

/* Restores the reference's pointers and frees the plans.  Call before free_network. */
void b200_detach(struct network *net);

#ifdef __cplusplus
}
#endif
#endif
