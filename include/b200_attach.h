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
 *
 * Like Darknet's own network functions these calls are not thread-safe: attach, predict and detach a given
 * network from one thread at a time (the registry of attached networks is a plain list).
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
 * stride > 1, reverse upsample, routes over inputs of unequal size) keep the reference's pointer.
 * Attached networks are for inference: until b200_detach the layers' delta_gpu pointers are set aside (so that
 * forward_network_gpu does not clear 30 GB of gradients per YOLOv3 batch, src/network.c:775-777) and the host
 * arrays Darknet pulls results into are page-locked. */
int b200_attach(struct network *net, int mode);

/* The whole forward pass through this library's own network object (channels-last between layers, shortcut
 * layers fused into convolutions), still behind Darknet's network_predict: layer 0's forward_gpu runs every
 * layer, the other pointers become no-ops, and Darknet's device buffers are written only where the reference
 * still looks: l.output_gpu (and the host copy l.output) of every [yolo] layer, and l.output_gpu of the last
 * layer, which pull_network_output copies (src/network.c:786).  The layers' delta_gpu pointers are set aside
 * until b200_detach so that forward_network_gpu has nothing to clear (src/network.c:775-777).  Returns the
 * number of layers, or -1 when a layer type is outside the convolutional forward path (use b200_attach then)
 * or the library refused the network (dnb_last_error()).  A host that reads intermediate l.output_gpu
 * buffers uses b200_attach instead. */
int b200_attach_network(struct network *net, int mode);

/* Restores the reference's pointers and frees the plans.  Call before free_network. */
void b200_detach(struct network *net);

#ifdef __cplusplus
}
#endif
#endif
