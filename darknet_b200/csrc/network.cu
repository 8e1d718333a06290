// The network object: cfg parsing, weights loading and the forward loop for the
// layer types on the convolutional forward path.  Mirrors the reference's
// parse_network_cfg (src/parser.c:742-889), load_weights (src/parser.c:1218-1308),
// forward_network_gpu (src/network.c:762-788) and network_predict
// (src/network.c:497-508), with activations kept channels-last between layers.
#include <stdlib.h>
#include <string.h>

#include <map>
#include <string>
#include <vector>

#include "common.h"
#include "conv.h"

using namespace dnb;

namespace {

enum LayerKind { L_CONV, L_MAXPOOL, L_UPSAMPLE, L_SHORTCUT, L_ROUTE, L_YOLO, L_AVGPOOL, L_SOFTMAX, L_CONNECTED };
const char *const kKindNames[] = {"convolutional", "maxpool", "upsample", "shortcut", "route", "yolo", "avgpool", "softmax", "connected"};

struct Layer {
    LayerKind kind;
    int c, h, w;                   // input extents
    int out_c, out_h, out_w;
    dnb_tensor out;                // device output: NHWC in the network's storage type (yolo: NCHW f32)
    // convolutional; a connected layer is the 1x1 convolution of a 1x1 map whose channels are the whole input
    // (height x width x channel pitch of the channels-last tensor it reads), the batch folded into the pixel tile
    dnb_conv_desc cd;
    dnb_conv_plan *plan = nullptr;
    bool flipped = false;          // convolutional: the file stores the weight matrix transposed (cfg flipped=1)
    int fc_inputs = 0;             // connected: inputs as the reference counts them (c*h*w of the previous layer)
    int in_cpitch = 0;             // connected: channel pitch of the tensor it reads
    // maxpool / upsample
    int size = 0, stride = 0, padding = 0;
    float scale = 1.f;
    // shortcut / route
    int from = -1;
    float alpha = 1.f, beta = 1.f;
    int activation = DNB_LINEAR;
    std::vector<int> inputs;
    // yolo
    int anchors = 0, classes = 0;
    float *host_out = nullptr;     // pinned; the slot of the step collected last
    float *host_slot[2] = {nullptr, nullptr};   // pinned result buffers of the two steps that may be in flight
    cudaEvent_t done = nullptr;    // compute stream: the layer's output is complete
    cudaEvent_t copied = nullptr;  // copy stream: the device-to-host copy of that output is complete
    bool params_given = false;     // dnb_network_set_conv_params has been called for this convolution
    // softmax
    int groups = 1;
    float temperature = 1.f;
    int launches = 1;
    // a convolution that also performs the [shortcut] layer right after it, and that shortcut layer
    bool fuses_next_shortcut = false, fused_into_prev = false;
    // a convolution that also performs the [yolo] layer right after it (that layer is then fused_into_prev too)
    bool fuses_next_yolo = false;
    // a maxpool layer that also writes the signs of its output, the next (tensor-core xnor) layer's operand
    int8_t *sign_out = nullptr;
    int sign_pitch = 0;
    // the output is a channel range of a later [route] layer's output: its producer writes it in place and the route
    // has nothing to copy for it (the memory belongs to the route layer)
    bool out_is_view = false;
};

typedef std::map<std::string, std::string> Options;

int opt_int(const Options &o, const char *k, int def)
{
    auto it = o.find(k);
    return it == o.end() ? def : atoi(it->second.c_str());
}
float opt_float(const Options &o, const char *k, float def)
{
    auto it = o.find(k);
    return it == o.end() ? def : (float)atof(it->second.c_str());
}
std::string opt_str(const Options &o, const char *k, const char *def)
{
    auto it = o.find(k);
    return it == o.end() ? std::string(def) : it->second;
}

// get_activation (src/activations.c:46-63): unknown names fall back to RELU there; here they are rejected.
int parse_activation(const std::string &s)
{
    static const char *const names[] = {"logistic", "relu", "relie", "linear", "ramp", "tanh", "plse",
                                        "leaky", "elu", "loggy", "stair", "hardtan", "lhtan", "selu"};
    for (int i = 0; i < 14; ++i)
        if (s == names[i]) return i;
    return -1;
}

std::string trim(const std::string &s)
{
    size_t a = s.find_first_not_of(" \t\r\n"), b = s.find_last_not_of(" \t\r\n");
    return a == std::string::npos ? std::string() : s.substr(a, b - a + 1);
}

// read_cfg (src/parser.c:891-924): '[' opens a section, '#' ';' and blank lines are skipped, the rest is key=value.
int split_cfg(const char *text, std::vector<std::pair<std::string, Options>> *sections)
{
    const char *p = text;
    int lineno = 0;
    while (*p) {
        const char *e = strchr(p, '\n');
        std::string line = trim(e ? std::string(p, e - p) : std::string(p));
        p = e ? e + 1 : p + strlen(p);
        ++lineno;
        if (line.empty() || line[0] == '#' || line[0] == ';') continue;
        if (line[0] == '[') {
            size_t r = line.find(']');
            if (r == std::string::npos) DNB_FAIL(DNB_EINVAL, "cfg line %d: unterminated section header", lineno);
            sections->push_back({trim(line.substr(1, r - 1)), Options()});
            continue;
        }
        size_t eq = line.find('=');
        if (eq == std::string::npos || sections->empty()) DNB_FAIL(DNB_EINVAL, "cfg line %d: expected key=value inside a section", lineno);
        sections->back().second[trim(line.substr(0, eq))] = trim(line.substr(eq + 1));
    }
    if (sections->empty()) DNB_FAIL(DNB_EINVAL, "cfg has no sections");
    return DNB_OK;
}

}  // namespace

struct dnb_network {
    int mode = DNB_MODE_TF32;
    int dtype = DNB_F32;             // storage type between layers
    int batch = 0, h = 0, w = 0, c = 0, inputs = 0, outputs = 0;
    std::vector<Layer> layers;
    float *input_dev = nullptr;      // NCHW f32 [batch][inputs]
    dnb_tensor input_nhwc{};         // only when the first layer needs channels-last input
    float *out_dev_nchw = nullptr;   // NCHW f32 staging of the output layer when it is not a yolo layer
    float *out_host = nullptr;       // pinned [batch][outputs]
    float *export_dev = nullptr;     // scratch for dnb_network_layer_output
    size_t export_elems = 0;
    cudaStream_t stream = nullptr;
    cudaStream_t copy_stream = nullptr;   // device-to-host copies of finished [yolo] outputs, overlapping later layers
    cudaStream_t h2d_stream = nullptr;    // host-to-device copy of the next step's images
    float *input_slot[2] = {nullptr, nullptr};     // device images of the two steps that may be in flight ([0] is input_dev)
    float *out_host_slot[2] = {nullptr, nullptr};  // pinned output-layer results ([0] is out_host)
    cudaEvent_t in_ready[2] = {nullptr, nullptr}, fwd_done[2] = {nullptr, nullptr}, copy_done[2] = {nullptr, nullptr};
    unsigned long long submitted = 0, collected = 0;
    int *status_dev = nullptr;            // two time-out status words, one per step that may be in flight; every plan of
                                          // the network is pointed at the word of the step being enqueued
    int *status_host = nullptr;           // pinned copies, read when the step is collected
    int device = 0;
    bool weights_loaded = false;
    int convs_with_params = 0;
    // CUDA-graph replay of the device-resident forward (dnb_network_enable_graph): one instantiated graph per
    // (input pointer, stream) seen last; eager_runs counts forwards with that pair since it changed
    bool graph_enabled = false;
    cudaGraphExec_t graph_exec = nullptr;
    const float *graph_input = nullptr;
    cudaStream_t graph_stream = nullptr;
    int eager_runs = 0;
    std::vector<cudaEvent_t> events;
};

static void drop_graph(dnb_network *net);

static int alloc_activation(dnb_network *net, dnb_tensor *t, int c, int h, int w)
{
    t->layout = DNB_NHWC;
    t->dtype = net->dtype;
    t->n = net->batch; t->c = c; t->h = h; t->w = w;
    t->cpitch = round_up(c, 8);
    const size_t bytes = tensor_elems(t) * elem_size(t->dtype);
    DNB_CUDA(cudaMalloc(&t->data, bytes));
    DNB_CUDA(cudaMemset(t->data, 0, bytes));  // the cpitch - c padding channels stay zero for the lifetime of the network
    return DNB_OK;
}

static int build_network(const char *text, int mode, int batch_override, dnb_network **out)
{
    if (!text || !out) DNB_FAIL(DNB_EINVAL, "parse_network_cfg: null argument");
    *out = nullptr;
    if (mode != DNB_MODE_TF32 && mode != DNB_MODE_BF16 && mode != DNB_MODE_FP32) DNB_FAIL(DNB_EINVAL, "parse_network_cfg: mode %d", mode);
    std::vector<std::pair<std::string, Options>> sections;
    DNB_TRY(split_cfg(text, &sections));
    if (sections[0].first != "net" && sections[0].first != "network") DNB_FAIL(DNB_EINVAL, "cfg: first section must be [net] or [network]");

    dnb_network *net = new dnb_network();
    struct Guard { dnb_network *n; ~Guard() { if (n) dnb_free_network(n); } } guard{net};
    net->mode = mode;
    net->dtype = mode == DNB_MODE_BF16 ? DNB_BF16 : DNB_F32;
    DNB_CUDA(cudaGetDevice(&net->device));
    const Options &no = sections[0].second;
    // parse_net_options (src/parser.c:655-734): batch /= subdivisions
    int subdivs = opt_int(no, "subdivisions", 1);
    if (subdivs < 1) subdivs = 1;
    net->batch = batch_override > 0 ? batch_override : opt_int(no, "batch", 1) / subdivs;
    net->h = opt_int(no, "height", 0); net->w = opt_int(no, "width", 0); net->c = opt_int(no, "channels", 0);
    if (net->batch < 1 || net->h < 1 || net->w < 1 || net->c < 1)
        DNB_FAIL(DNB_EINVAL, "cfg [net]: need positive batch, height, width, channels (got %d, %d, %d, %d)", net->batch, net->h, net->w, net->c);
    net->inputs = net->h * net->w * net->c;

    int c = net->c, h = net->h, w = net->w;
    for (size_t si = 1; si < sections.size(); ++si) {
        const std::string &type = sections[si].first;
        const Options &o = sections[si].second;
        const int index = (int)si - 1;
        Layer L;
        L.c = c; L.h = h; L.w = w;
        if (type == "convolutional" || type == "conv") {
            L.kind = L_CONV;
            const int size = opt_int(o, "size", 1);
            int padding = opt_int(o, "padding", 0);
            if (opt_int(o, "pad", 0)) padding = size / 2;  // src/parser.c:184-187
            const int act = parse_activation(opt_str(o, "activation", "logistic"));
            if (act < 0) DNB_FAIL(DNB_EINVAL, "cfg layer %d: unknown activation '%s'", index, opt_str(o, "activation", "").c_str());
            L.cd = dnb_conv_desc{net->batch, h, w, c, opt_int(o, "filters", 1), opt_int(o, "groups", 1), size,
                                 opt_int(o, "stride", 1), padding, opt_int(o, "batch_normalize", 0), act, opt_int(o, "xnor", 0)};
            L.flipped = opt_int(o, "flipped", 0) != 0;   // parse_convolutional, src/parser.c:199: only the file's weight order differs
            DNB_TRY(dnb_conv_plan_create(&L.cd, mode, &L.plan));
            L.out_c = L.cd.n; L.out_h = L.plan->g.out_h; L.out_w = L.plan->g.out_w;
            L.launches = L.plan->kernel == 3 ? 2 : 1;
        } else if (type == "connected" || type == "conn") {
            // parse_connected (src/parser.c:259-268), make_connected_layer (src/connected_layer.c:14-33)
            L.kind = L_CONNECTED;
            const int act = parse_activation(opt_str(o, "activation", "logistic"));
            if (act < 0) DNB_FAIL(DNB_EINVAL, "cfg layer %d: unknown activation '%s'", index, opt_str(o, "activation", "").c_str());
            const int outputs = opt_int(o, "output", 1);
            if (outputs < 1) DNB_FAIL(DNB_EINVAL, "cfg layer %d: connected output=%d", index, outputs);
            L.fc_inputs = c * h * w;
            L.in_cpitch = round_up(c, 8);
            L.cd = dnb_conv_desc{net->batch, 1, 1, h * w * L.in_cpitch, outputs, 1, 1, 1, 0, opt_int(o, "batch_normalize", 0), act, 0};
            DNB_TRY(dnb_conv_plan_create(&L.cd, mode, &L.plan));
            L.out_c = outputs; L.out_h = 1; L.out_w = 1;
        } else if (type == "maxpool" || type == "max") {
            L.kind = L_MAXPOOL;
            L.stride = opt_int(o, "stride", 1);
            L.size = opt_int(o, "size", L.stride);
            L.padding = opt_int(o, "padding", L.size - 1);  // src/parser.c:485-487
            if (L.stride < 1 || L.size < 1) DNB_FAIL(DNB_EINVAL, "cfg layer %d: maxpool size %d stride %d", index, L.size, L.stride);
            L.out_c = c; L.out_h = (h + L.padding - L.size) / L.stride + 1; L.out_w = (w + L.padding - L.size) / L.stride + 1;
        } else if (type == "upsample") {
            L.kind = L_UPSAMPLE;
            L.stride = opt_int(o, "stride", 2);
            L.scale = opt_float(o, "scale", 1.f);
            if (L.stride < 1) DNB_FAIL(DNB_EUNSUPPORTED, "cfg layer %d: upsample stride %d (reverse form)", index, L.stride);
            L.out_c = c; L.out_h = h * L.stride; L.out_w = w * L.stride;
        } else if (type == "shortcut") {
            L.kind = L_SHORTCUT;
            int from = opt_int(o, "from", 0);
            if (o.find("from") == o.end()) DNB_FAIL(DNB_EINVAL, "cfg layer %d: shortcut without from=", index);
            if (from < 0) from = index + from;
            if (from < 0 || from >= index) DNB_FAIL(DNB_EINVAL, "cfg layer %d: shortcut from=%d out of range", index, from);
            L.from = from;
            L.activation = parse_activation(opt_str(o, "activation", "linear"));
            if (L.activation < 0) DNB_FAIL(DNB_EINVAL, "cfg layer %d: unknown activation", index);
            L.alpha = opt_float(o, "alpha", 1.f); L.beta = opt_float(o, "beta", 1.f);
            L.out_c = c; L.out_h = h; L.out_w = w;
        } else if (type == "route") {
            L.kind = L_ROUTE;
            std::string ls = opt_str(o, "layers", "");
            if (ls.empty()) DNB_FAIL(DNB_EINVAL, "cfg layer %d: route must specify input layers", index);
            size_t pos = 0;
            int csum = 0;
            while (pos <= ls.size()) {
                size_t comma = ls.find(',', pos);
                int id = atoi(ls.substr(pos, comma == std::string::npos ? std::string::npos : comma - pos).c_str());
                if (id < 0) id = index + id;
                if (id < 0 || id >= index) DNB_FAIL(DNB_EINVAL, "cfg layer %d: route input %d out of range", index, id);
                L.inputs.push_back(id);
                csum += net->layers[id].out_c;
                if (comma == std::string::npos) break;
                pos = comma + 1;
            }
            const Layer &first = net->layers[L.inputs[0]];
            for (int id : L.inputs)
                if (net->layers[id].out_h != first.out_h || net->layers[id].out_w != first.out_w)
                    DNB_FAIL(DNB_EUNSUPPORTED, "cfg layer %d: route inputs of unequal width/height", index);
            L.out_c = csum; L.out_h = first.out_h; L.out_w = first.out_w;
            L.launches = (int)L.inputs.size();
        } else if (type == "yolo") {
            L.kind = L_YOLO;
            // parse_yolo (src/parser.c:306-345): n = number of mask entries (or num), classes default 20
            const std::string mask = opt_str(o, "mask", "");
            int n = opt_int(o, "num", 1);
            if (!mask.empty()) { n = 1; for (char ch : mask) if (ch == ',') ++n; }
            L.anchors = n; L.classes = opt_int(o, "classes", 20);
            if (c != n * (L.classes + 5)) DNB_FAIL(DNB_EINVAL, "cfg layer %d: yolo expects %d channels, input has %d", index, n * (L.classes + 5), c);
            L.out_c = c; L.out_h = h; L.out_w = w;
        } else if (type == "avgpool" || type == "avg") {
            L.kind = L_AVGPOOL;
            L.out_c = c; L.out_h = 1; L.out_w = 1;
        } else if (type == "softmax" || type == "soft") {
            L.kind = L_SOFTMAX;
            L.groups = opt_int(o, "groups", 1);
            L.temperature = opt_float(o, "temperature", 1.f);
            if (o.find("tree") != o.end()) DNB_FAIL(DNB_EUNSUPPORTED, "cfg layer %d: softmax tree", index);
            if (h != 1 || w != 1) DNB_FAIL(DNB_EUNSUPPORTED, "cfg layer %d: softmax over a %dx%d map", index, w, h);
            L.out_c = c; L.out_h = 1; L.out_w = 1;
        } else {
            DNB_FAIL(DNB_EUNSUPPORTED, "cfg layer %d: section [%s] is outside the convolutional forward path", index, type.c_str());
        }
        if (L.out_h < 1 || L.out_w < 1) DNB_FAIL(DNB_EINVAL, "cfg layer %d: empty output", index);
        // the previous layer's output must be channels-last for every consumer but none reads a yolo output
        if (index > 0 && net->layers[index - 1].kind == L_YOLO && L.kind != L_ROUTE)
            DNB_FAIL(DNB_EUNSUPPORTED, "cfg layer %d: a [%s] directly after [yolo]", index, type.c_str());
        if (L.kind == L_YOLO) {
            L.out = dnb_tensor{nullptr, DNB_NCHW, DNB_F32, net->batch, L.out_c, L.out_h, L.out_w, 0};
            const size_t bytes = tensor_elems(&L.out) * sizeof(float);
            DNB_CUDA(cudaMalloc(&L.out.data, bytes));
            DNB_CUDA(cudaMallocHost((void **)&L.host_slot[0], bytes));
            L.host_out = L.host_slot[0];
        } else {
            DNB_TRY(alloc_activation(net, &L.out, L.out_c, L.out_h, L.out_w));
        }
        net->layers.push_back(L);
        c = L.out_c; h = L.out_h; w = L.out_w;
    }
    if (net->layers.empty()) DNB_FAIL(DNB_EINVAL, "cfg has no layers");
    for (const Layer &L : net->layers) {
        if (L.kind == L_SHORTCUT && net->layers[L.from].kind == L_YOLO) DNB_FAIL(DNB_EUNSUPPORTED, "cfg: shortcut from a [yolo] layer");
        if (L.kind == L_ROUTE)
            for (int id : L.inputs)
                if (net->layers[id].kind == L_YOLO) DNB_FAIL(DNB_EUNSUPPORTED, "cfg: route from a [yolo] layer");
    }
    // Fuse "convolution, then [shortcut] of equal shape" into the convolution's epilogue when nothing else
    // reads the convolution's own output: one pass over the activations instead of three.
    // DNB_FUSE_SHORTCUT=0 keeps every layer separate (every layer's output stays readable).
    const bool fuse = getenv("DNB_FUSE_SHORTCUT") ? atoi(getenv("DNB_FUSE_SHORTCUT")) != 0 : true;
    for (int i = 0; fuse && i + 1 < (int)net->layers.size(); ++i) {
        Layer &C = net->layers[i], &S = net->layers[i + 1];
        if (C.kind != L_CONV || !C.plan || (C.plan->kernel != 0 && C.plan->kernel != 1) || S.kind != L_SHORTCUT || S.from == i) continue;
        const Layer &F = net->layers[S.from];
        if (F.kind == L_YOLO || F.out_c != S.out_c || F.out_h != S.out_h || F.out_w != S.out_w) continue;
        bool read_elsewhere = false;
        for (int j = i + 2; j < (int)net->layers.size(); ++j) {
            const Layer &L = net->layers[j];
            if (L.kind == L_SHORTCUT && L.from == i) read_elsewhere = true;
            if (L.kind == L_ROUTE)
                for (int id : L.inputs) if (id == i) read_elsewhere = true;
        }
        if (read_elsewhere) continue;
        C.fuses_next_shortcut = true;
        S.fused_into_prev = true;
        S.launches = 0;
        cudaFree(C.out.data);      // never written: the convolution stores straight into the shortcut's output
        C.out.data = nullptr;
    }
    // Fuse "convolution, then [yolo]" when nothing else reads the convolution's output: the epilogue applies the yolo
    // layer's logistic per entry and writes that layer's NCHW output; the channels-last copy of the raw predictions
    // and the pass that transposed it (forward_yolo_layer_gpu, src/yolo_layer.c:347-357) disappear.
    // DNB_FUSE_YOLO=0 keeps the two layers separate.
    const bool fuse_yolo = getenv("DNB_FUSE_YOLO") ? atoi(getenv("DNB_FUSE_YOLO")) != 0 : true;
    for (int i = 0; fuse_yolo && i + 1 < (int)net->layers.size(); ++i) {
        Layer &C = net->layers[i], &Y = net->layers[i + 1];
        if (C.kind != L_CONV || !C.plan || (C.plan->kernel != 0 && C.plan->kernel != 1) || C.plan->stem_tc || Y.kind != L_YOLO) continue;
        if (C.plan->d.activation != DNB_LINEAR || C.plan->g.n % 256 == 0) continue;   // the fused epilogue is built for the linear heads every yolo cfg has (and not for CTA pairs)
        bool read_elsewhere = false;
        for (int j = i + 2; j < (int)net->layers.size(); ++j) {
            const Layer &L = net->layers[j];
            if (L.kind == L_SHORTCUT && L.from == i) read_elsewhere = true;
            if (L.kind == L_ROUTE)
                for (int id : L.inputs) if (id == i) read_elsewhere = true;
        }
        if (read_elsewhere) continue;
        C.fuses_next_yolo = true;
        Y.fused_into_prev = true;
        Y.launches = 0;
        cudaFree(C.out.data);      // never written: the convolution stores straight into the yolo layer's output
        C.out.data = nullptr;
    }
    // Zero-copy [route]: where a route input is produced by a layer whose kernel can write a channel range of a wider
    // channels-last tensor (tensor-core convolutions, with or without a fused shortcut, and upsample), and everything that
    // reads it can read such a range (convolutions, routes, the yolo head, upsample), the input's tensor BECOMES its
    // range of the route's output: forward_route_layer_gpu's copies (src/route_layer.c:105-118) disappear.
    // DNB_ROUTE_ALIAS=0 keeps every layer's own tensor.
    const bool alias = getenv("DNB_ROUTE_ALIAS") ? atoi(getenv("DNB_ROUTE_ALIAS")) != 0 : true;
    for (int r = 0; alias && r < (int)net->layers.size(); ++r) {
        Layer &R = net->layers[r];
        if (R.kind != L_ROUTE) continue;
        const size_t es = elem_size(R.out.dtype);
        int off = 0, copies = 0;
        for (size_t k = 0; k < R.inputs.size(); ++k) {
            const int id = R.inputs[k];
            Layer &P = net->layers[id];
            const int this_off = off;
            off += P.out_c;
            ++copies;
            const bool last_input = k + 1 == R.inputs.size();
            if (P.out_is_view || !P.out.data || P.out.layout != DNB_NHWC) continue;
            if ((size_t)this_off * es % 128 || (!last_input && P.out_c % 8)) continue;
            bool writer_ok = false;
            if (P.kind == L_UPSAMPLE) writer_ok = true;
            if (P.kind == L_CONV && P.plan && (P.plan->kernel == 0 || P.plan->kernel == 1) && !P.plan->stem_tc) writer_ok = true;
            if (P.kind == L_SHORTCUT && P.fused_into_prev) writer_ok = true;   // written by the convolution before it
            if (!writer_ok) continue;
            bool readers_ok = true;
            for (int j = id + 1; j < (int)net->layers.size() && readers_ok; ++j) {
                const Layer &C = net->layers[j];
                const bool reads_as_input = j == id + 1 && C.kind != L_ROUTE && !(C.kind == L_SHORTCUT && C.fused_into_prev);
                if (reads_as_input && !(C.kind == L_CONV && !C.plan->stem_tc) && C.kind != L_YOLO && C.kind != L_UPSAMPLE) readers_ok = false;
                if (C.kind == L_SHORTCUT && C.from == id && !C.fused_into_prev) readers_ok = false;   // the stand-alone kernel wants equal pitches
            }
            if (!readers_ok) continue;
            cudaFree(P.out.data);
            P.out.data = (char *)R.out.data + (size_t)this_off * es;
            P.out.cpitch = R.out.cpitch;
            P.out_is_view = true;
            --copies;
        }
        R.launches = copies;
    }
    // xnor layers in a row: the first one's epilogue writes the second one's int8 operand (conv_plan_link_signs)
    for (int i = 0; i + 1 < (int)net->layers.size(); ++i) {
        Layer &A = net->layers[i], &B = net->layers[i + 1];
        if (B.kind != L_CONV || !B.plan || !A.out.data || A.out.layout != DNB_NHWC) continue;
        if (A.kind == L_CONV && A.plan) {
            if (conv_plan_link_signs(A.plan, B.plan, A.out.data)) B.launches = 1;   // no sign pass of its own
        } else if (A.kind == L_MAXPOOL && A.out.dtype == DNB_F32 && A.out.cpitch == A.out_c) {
            A.sign_out = conv_plan_expect_signs(B.plan, A.out.data, net->batch, A.out_c, A.out_h, A.out_w);
            if (A.sign_out) { A.sign_pitch = A.out_c; B.launches = 1; }
        }
    }
    const Layer &last = net->layers.back();
    net->outputs = last.out_c * last.out_h * last.out_w;
    DNB_CUDA(cudaMalloc((void **)&net->input_dev, (size_t)net->batch * net->inputs * sizeof(float)));
    DNB_CUDA(cudaMallocHost((void **)&net->out_host, (size_t)net->batch * net->outputs * sizeof(float)));
    if (last.kind != L_YOLO) DNB_CUDA(cudaMalloc((void **)&net->out_dev_nchw, (size_t)net->batch * net->outputs * sizeof(float)));
    const Layer &first = net->layers.front();
    const bool first_reads_nchw = first.kind == L_CONV && (first.plan->kernel == 2 || first.plan->kernel == 3);   // a connected first layer reads the channels-last copy
    if (!first_reads_nchw) {
        dnb_tensor *t = &net->input_nhwc;
        DNB_TRY(alloc_activation(net, t, net->c, net->h, net->w));
    }
    DNB_CUDA(cudaStreamCreateWithFlags(&net->stream, cudaStreamNonBlocking));
    DNB_CUDA(cudaStreamCreateWithFlags(&net->copy_stream, cudaStreamNonBlocking));
    DNB_CUDA(cudaStreamCreateWithFlags(&net->h2d_stream, cudaStreamNonBlocking));
    net->input_slot[0] = net->input_dev;
    net->out_host_slot[0] = net->out_host;
    for (int k = 0; k < 2; ++k) {
        DNB_CUDA(cudaEventCreateWithFlags(&net->in_ready[k], cudaEventDisableTiming));
        DNB_CUDA(cudaEventCreateWithFlags(&net->fwd_done[k], cudaEventDisableTiming));
        DNB_CUDA(cudaEventCreateWithFlags(&net->copy_done[k], cudaEventDisableTiming));
    }
    for (Layer &L : net->layers)
        if (L.kind == L_YOLO) {
            DNB_CUDA(cudaEventCreateWithFlags(&L.done, cudaEventDisableTiming));
            DNB_CUDA(cudaEventCreateWithFlags(&L.copied, cudaEventDisableTiming));
        }
    DNB_CUDA(cudaMalloc((void **)&net->status_dev, 2 * sizeof(int)));
    DNB_CUDA(cudaMemset(net->status_dev, 0, 2 * sizeof(int)));
    DNB_CUDA(cudaMallocHost((void **)&net->status_host, 2 * sizeof(int)));
    net->status_host[0] = net->status_host[1] = 0;
    for (Layer &L : net->layers)
        if (L.plan) { L.plan->status = net->status_dev; L.plan->status_shared = true; }
    guard.n = nullptr;
    *out = net;
    return DNB_OK;
}

extern "C" int dnb_parse_network_cfg_text(const char *cfg_text, int mode, int batch_override, dnb_network **net)
{
    return build_network(cfg_text, mode, batch_override, net);
}

extern "C" int dnb_parse_network_cfg(const char *path, int mode, int batch_override, dnb_network **net)
{
    if (!path) DNB_FAIL(DNB_EINVAL, "parse_network_cfg: null path");
    FILE *f = fopen(path, "rb");
    if (!f) DNB_FAIL(DNB_EIO, "Couldn't open file: %s", path);  // file_error, src/utils.c:281-285
    std::string text;
    char buf[4096];
    size_t n;
    while ((n = fread(buf, 1, sizeof(buf), f)) > 0) text.append(buf, n);
    fclose(f);
    return build_network(text.c_str(), mode, batch_override, net);
}

extern "C" void dnb_free_network(dnb_network *net)
{
    if (!net) return;
    for (Layer &L : net->layers) {
        if (L.plan) dnb_conv_plan_destroy(L.plan);
        if (!L.out_is_view) cudaFree(L.out.data);
        for (float *hp : L.host_slot) if (hp) cudaFreeHost(hp);
        if (L.copied) cudaEventDestroy(L.copied);
    }
    cudaFree(net->input_dev); cudaFree(net->input_nhwc.data); cudaFree(net->out_dev_nchw); cudaFree(net->export_dev);
    if (net->out_host) cudaFreeHost(net->out_host);
    if (net->status_host) cudaFreeHost(net->status_host);
    if (net->graph_exec) cudaGraphExecDestroy(net->graph_exec);
    cudaFree(net->status_dev);
    for (cudaEvent_t e : net->events) cudaEventDestroy(e);
    for (Layer &L : net->layers) if (L.done) cudaEventDestroy(L.done);
    if (net->stream) cudaStreamDestroy(net->stream);
    if (net->copy_stream) cudaStreamDestroy(net->copy_stream);
    if (net->h2d_stream) cudaStreamDestroy(net->h2d_stream);
    cudaFree(net->input_slot[1]);
    if (net->out_host_slot[1]) cudaFreeHost(net->out_host_slot[1]);
    for (int k = 0; k < 2; ++k) {
        if (net->in_ready[k]) cudaEventDestroy(net->in_ready[k]);
        if (net->fwd_done[k]) cudaEventDestroy(net->fwd_done[k]);
        if (net->copy_done[k]) cudaEventDestroy(net->copy_done[k]);
    }
    delete net;
}

// A connected layer's matrix, [outputs][inputs] with the inputs in the reference's order (channel, row, column of the
// previous layer's output, src/connected_layer.c:151-160), rearranged for the channels-last tensor the layer reads
// here: input (ch, y, x) sits at ((y * w + x) * cpitch + ch); padding channels get zero weights.
static int set_connected_params(dnb_network *net, Layer &L, int index, const float *weights, const float *biases, const float *scales,
                                const float *mean, const float *var)
{
    const Layer *prev = index > 0 ? &net->layers[index - 1] : nullptr;
    const int c = prev ? prev->out_c : net->c, h = prev ? prev->out_h : net->h, w = prev ? prev->out_w : net->w;
    const int cp = L.in_cpitch, outputs = L.cd.n;
    const size_t k = (size_t)h * w * cp;
    std::vector<float> packed((size_t)outputs * k, 0.f);
    for (int o = 0; o < outputs; ++o)
        for (int ch = 0; ch < c; ++ch)
            for (int y = 0; y < h; ++y)
                for (int x = 0; x < w; ++x)
                    packed[(size_t)o * k + ((size_t)y * w + x) * cp + ch] = weights[(size_t)o * L.fc_inputs + ((size_t)ch * h + y) * w + x];
    return dnb_conv_plan_set_params(L.plan, packed.data(), biases, scales, mean, var);
}

static int load_weights_impl(dnb_network *net, const char *path, bool packed)
{
    if (!net || !path) DNB_FAIL(DNB_EINVAL, "load_weights: null argument");
    FILE *f = fopen(path, "rb");
    if (!f) DNB_FAIL(DNB_EIO, "Couldn't open file: %s", path);
    struct Closer { FILE *f; ~Closer() { fclose(f); } } closer{f};
    int hdr[3];
    if (fread(hdr, sizeof(int), 3, f) != 3) DNB_FAIL(DNB_EIO, "%s: truncated header", path);
    // src/parser.c:1234-1241: a 64-bit `seen` from version 0.2 on, a 32-bit one before
    if ((hdr[0] * 10 + hdr[1]) >= 2 && hdr[0] < 1000 && hdr[1] < 1000) {
        uint64_t seen;
        if (fread(&seen, sizeof(seen), 1, f) != 1) DNB_FAIL(DNB_EIO, "%s: truncated header", path);
    } else {
        int seen;
        if (fread(&seen, sizeof(seen), 1, f) != 1) DNB_FAIL(DNB_EIO, "%s: truncated header", path);
    }
    // File versions above 1000 store connected-layer matrices as [inputs][outputs] (src/parser.c:1244, 1098-1104);
    // convolutional layers are not affected by the version.
    const bool transposed = hdr[0] > 1000 || hdr[1] > 1000;
    int index = 0;
    for (Layer &L : net->layers) {
        if (L.kind == L_CONV) {
            // load_convolutional_weights (src/parser.c:1164-1215): biases, batchnorm vectors, weights
            const dnb_conv_desc &d = L.cd;
            const size_t nw = (size_t)d.n * (d.c / d.groups) * d.size * d.size;
            std::vector<float> biases(d.n), scales, mean, var, weights(nw);
            bool ok = fread(biases.data(), sizeof(float), d.n, f) == (size_t)d.n;
            if (ok && d.batch_normalize) {
                scales.resize(d.n); mean.resize(d.n); var.resize(d.n);
                ok = fread(scales.data(), sizeof(float), d.n, f) == (size_t)d.n &&
                     fread(mean.data(), sizeof(float), d.n, f) == (size_t)d.n &&
                     fread(var.data(), sizeof(float), d.n, f) == (size_t)d.n;
            }
            if (ok && packed && d.xnor) {
                // load_convolutional_weights_binary (src/parser.c:1134-1162): per filter its mean |w| as a float, then one
                // bit per weight (set: +mean, clear: -mean), eight to a byte, lowest bit first.  The reference stores
                // size/8 bytes per filter, so a filter whose c*size*size is not a multiple of 8 would lose its tail.
                const size_t per = nw / d.n;
                if (per % 8) DNB_FAIL(DNB_EUNSUPPORTED, "%s: layer %d has %zu weights per filter; the packed format holds whole bytes of 8 only", path, index, per);
                std::vector<unsigned char> bits(per / 8);
                for (int n = 0; n < d.n && ok; ++n) {
                    float mean = 0;
                    ok = fread(&mean, sizeof(float), 1, f) == 1 && fread(bits.data(), 1, per / 8, f) == per / 8;
                    for (size_t k = 0; ok && k < per; ++k) weights[(size_t)n * per + k] = (bits[k / 8] >> (k % 8)) & 1 ? mean : -mean;
                }
            } else {
                ok = ok && fread(weights.data(), sizeof(float), nw, f) == nw;
            }
            if (!ok) DNB_FAIL(DNB_EIO, "%s: file ends inside layer %d (the reference would silently keep its random initialisation)", path, index);
            if (L.flipped) {
                // transpose_matrix(l.weights, l.c*l.size*l.size, l.n) (src/parser.c:1206-1208, 1085-1096): the file holds
                // c*size*size rows of n values; Darknet's layout is n rows of c*size*size values
                const size_t rows = nw / d.n, cols = d.n;
                std::vector<float> t(nw);
                for (size_t x = 0; x < rows; ++x)
                    for (size_t y = 0; y < cols; ++y) t[y * rows + x] = weights[x * cols + y];
                weights.swap(t);
            }
            DNB_TRY(dnb_conv_plan_set_params(L.plan, weights.data(), biases.data(), d.batch_normalize ? scales.data() : nullptr,
                                             d.batch_normalize ? mean.data() : nullptr, d.batch_normalize ? var.data() : nullptr));
        } else if (L.kind == L_CONNECTED) {
            // load_connected_weights (src/parser.c:1098-1120): biases, weights, then the batchnorm vectors
            const int outputs = L.cd.n, inputs = L.fc_inputs;
            const size_t nw = (size_t)outputs * inputs;
            std::vector<float> biases(outputs), scales, mean, var, weights(nw);
            bool ok = fread(biases.data(), sizeof(float), outputs, f) == (size_t)outputs && fread(weights.data(), sizeof(float), nw, f) == nw;
            if (ok && L.cd.batch_normalize) {
                scales.resize(outputs); mean.resize(outputs); var.resize(outputs);
                ok = fread(scales.data(), sizeof(float), outputs, f) == (size_t)outputs &&
                     fread(mean.data(), sizeof(float), outputs, f) == (size_t)outputs &&
                     fread(var.data(), sizeof(float), outputs, f) == (size_t)outputs;
            }
            if (!ok) DNB_FAIL(DNB_EIO, "%s: file ends inside layer %d", path, index);
            if (transposed) {
                std::vector<float> t(nw);   // transpose_matrix(l.weights, l.inputs, l.outputs)
                for (int x = 0; x < inputs; ++x)
                    for (int y = 0; y < outputs; ++y) t[(size_t)y * inputs + x] = weights[(size_t)x * outputs + y];
                weights.swap(t);
            }
            DNB_TRY(set_connected_params(net, L, index, weights.data(), biases.data(), L.cd.batch_normalize ? scales.data() : nullptr,
                                         L.cd.batch_normalize ? mean.data() : nullptr, L.cd.batch_normalize ? var.data() : nullptr));
        }
        ++index;
    }
    net->weights_loaded = true;
    drop_graph(net);   // a captured forward holds the pointers of the parameter tensors just replaced
    return DNB_OK;
}

extern "C" int dnb_load_weights(dnb_network *net, const char *path) { return load_weights_impl(net, path, false); }

// The same file format with every xnor convolution stored packed (mean |w| and one sign bit per weight).
extern "C" int dnb_load_weights_packed(dnb_network *net, const char *path) { return load_weights_impl(net, path, true); }

// The same derived tensors from host arrays instead of a file: what a host that has already run the
// reference's load_weights holds in l.weights, l.biases, l.scales, l.rolling_mean, l.rolling_variance.
extern "C" int dnb_network_set_conv_params(dnb_network *net, int layer, const float *weights, const float *biases,
                                           const float *scales, const float *rolling_mean, const float *rolling_variance)
{
    if (!net || layer < 0 || layer >= (int)net->layers.size()) DNB_FAIL(DNB_EINVAL, "set_conv_params: bad argument");
    Layer &L = net->layers[layer];
    if (L.kind != L_CONV && L.kind != L_CONNECTED) DNB_FAIL(DNB_EINVAL, "set_conv_params: layer %d has no parameters", layer);
    if (net->submitted != net->collected) DNB_FAIL(DNB_EINVAL, "set_conv_params: a submitted step is still in flight; collect it first");
    if (L.kind == L_CONNECTED) {
        if (!weights || !biases) DNB_FAIL(DNB_EINVAL, "set_conv_params: null argument");
        DNB_TRY(set_connected_params(net, L, layer, weights, biases, scales, rolling_mean, rolling_variance));
    } else {
        DNB_TRY(dnb_conv_plan_set_params(L.plan, weights, biases, scales, rolling_mean, rolling_variance));
    }
    drop_graph(net);   // a captured forward holds the pointers of the parameter tensors just replaced
    if (!L.params_given) { L.params_given = true; ++net->convs_with_params; }
    int convs = 0;
    for (const Layer &K : net->layers) convs += K.kind == L_CONV || K.kind == L_CONNECTED;
    if (net->convs_with_params == convs) net->weights_loaded = true;
    return DNB_OK;
}

// Layer `layer`'s current output in Darknet's layout (NCHW f32) into device memory of the caller, on `stream`.
extern "C" int dnb_network_export_layer(dnb_network *net, int layer, float *device_nchw, void *stream)
{
    if (!net || !device_nchw || layer < 0 || layer >= (int)net->layers.size()) DNB_FAIL(DNB_EINVAL, "export_layer: bad argument");
    Layer &L = net->layers[layer];
    if (!L.out.data) DNB_FAIL(DNB_EUNSUPPORTED, "layer %d is fused into layer %d and has no output of its own", layer, layer + 1);
    cudaStream_t s = (cudaStream_t)stream;
    if (L.out.layout == DNB_NCHW) {
        DNB_CUDA(cudaMemcpyAsync(device_nchw, L.out.data, tensor_elems(&L.out) * sizeof(float), cudaMemcpyDeviceToDevice, s));
        return DNB_OK;
    }
    dnb_tensor o{device_nchw, DNB_NCHW, DNB_F32, net->batch, L.out_c, L.out_h, L.out_w, 0};
    return launch_convert(&L.out, &o, 0, 0, 0, s);
}

// Every convolution launched from here on reports an expired wait in the status word of step slot `slot`.
static void point_status(dnb_network *net, int slot)
{
    for (Layer &L : net->layers)
        if (L.plan) L.plan->status = net->status_dev + slot;
}

static const char *const kTimeoutText =
    "a device-side wait expired in a convolution (code %d: 101 ring slot free, 102 operands landed, 103 accumulator free, "
    "104 accumulator ready, 105 residual tile, 106 shared memory window not 1024-byte aligned); the outputs are incomplete";

// One layer of forward_network_gpu's loop (src/network.c:772-785).
// Transposes the network input into channels-last form when the first layer wants that.
static int prepare_input(dnb_network *net, const float *device_input, cudaStream_t s)
{
    if (!net->input_nhwc.data) return DNB_OK;
    dnb_tensor in{(void *)device_input, DNB_NCHW, DNB_F32, net->batch, net->c, net->h, net->w, 0};
    return launch_convert(&in, &net->input_nhwc, net->mode == DNB_MODE_TF32, 0, 0, s);
}

static int forward_layer(dnb_network *net, int i, const float *device_input, cudaStream_t s)
{
    Layer &L = net->layers[i];
    dnb_tensor in;
    if (i == 0) {
        in = dnb_tensor{(void *)device_input, DNB_NCHW, DNB_F32, net->batch, net->c, net->h, net->w, 0};
        if (net->input_nhwc.data) in = net->input_nhwc;   // filled by prepare_input
    } else {
        in = net->layers[i - 1].out;
    }
    switch (L.kind) {
    case L_CONV:
        if (L.fuses_next_shortcut) {
            Layer &S = net->layers[i + 1];
            return dnb_conv_shortcut_forward(L.plan, &in, &net->layers[S.from].out, &S.out, S.alpha, S.beta, S.activation, s);
        }
        if (L.fuses_next_yolo) {
            Layer &Y = net->layers[i + 1];
            return dnb_conv_yolo_forward(L.plan, &in, &Y.out, Y.anchors, Y.classes, s);
        }
        return dnb_conv_forward(L.plan, &in, &L.out, nullptr, s);
    case L_CONNECTED: {
        // forward_connected_layer_gpu (src/connected_layer.c:288-306): the previous layer's whole channels-last output
        // is one pixel of h*w*cpitch channels per image
        dnb_tensor flat = in;
        flat.h = flat.w = 1;
        flat.c = flat.cpitch = L.cd.c;
        return dnb_conv_forward(L.plan, &flat, &L.out, nullptr, s);
    }
    case L_MAXPOOL: return launch_maxpool(&in, &L.out, L.size, L.stride, L.padding, s, L.sign_out, L.sign_pitch);
    case L_UPSAMPLE: return launch_upsample(&in, &L.out, L.stride, L.scale, s);
    case L_SHORTCUT:
        if (L.fused_into_prev) return DNB_OK;   // done by the convolution before it
        return launch_shortcut(&in, &net->layers[L.from].out, &L.out, L.alpha, L.beta, L.activation, s);
    case L_ROUTE: {
        std::vector<const dnb_tensor *> ins;
        for (int id : L.inputs) ins.push_back(&net->layers[id].out);
        return launch_route(ins.data(), (int)ins.size(), &L.out, s);
    }
    case L_YOLO:
        if (L.fused_into_prev) return DNB_OK;   // done by the convolution before it
        return launch_convert(&in, &L.out, 0, L.anchors, L.classes, s);
    case L_AVGPOOL: return launch_avgpool(&in, &L.out, s);
    case L_SOFTMAX: return launch_softmax(&in, &L.out, L.groups, L.temperature, s);
    }
    return DNB_OK;
}

static int forward_eager(dnb_network *net, const float *device_input, cudaStream_t s)
{
    DNB_TRY(prepare_input(net, device_input, s));
    for (int i = 0; i < (int)net->layers.size(); ++i) DNB_TRY(forward_layer(net, i, device_input, s));
    return DNB_OK;
}

static void drop_graph(dnb_network *net)
{
    if (net->graph_exec) cudaGraphExecDestroy(net->graph_exec);
    net->graph_exec = nullptr;
    net->graph_input = nullptr;
    net->graph_stream = nullptr;
    net->eager_runs = 0;
}

extern "C" int dnb_network_enable_graph(dnb_network *net, int on)
{
    if (!net) DNB_FAIL(DNB_EINVAL, "enable_graph: null network");
    net->graph_enabled = on != 0;
    if (!on) drop_graph(net);
    return DNB_OK;
}

extern "C" int dnb_network_forward(dnb_network *net, const float *device_input, void *stream)
{
    if (!net || !device_input) DNB_FAIL(DNB_EINVAL, "network_forward: null argument");
    if (!net->weights_loaded) DNB_FAIL(DNB_EINVAL, "network_forward: load_weights has not been called");
    if (net->submitted != net->collected) DNB_FAIL(DNB_EINVAL, "network_forward: a submitted step is still in flight (the layers' outputs are shared); collect it first");
    DNB_TRY(check_current_device(net->device, "network_forward"));
    point_status(net, 0);
    cudaStream_t s = (cudaStream_t)stream;  // NULL is the legacy default stream, as everywhere in CUDA
    if (!net->graph_enabled || !s) return forward_eager(net, device_input, s);   // the legacy stream cannot be captured

    // Graph replay: at small batches the 100-odd launches of a forward pass cost more than its kernels.  The
    // first forward with a given (input, stream) runs eagerly (plans build their tensor maps and scratch then),
    // the second is captured, every later one is a single cudaGraphLaunch.
    if (net->graph_exec && net->graph_input == device_input && net->graph_stream == s) {
        DNB_CUDA(cudaGraphLaunch(net->graph_exec, s));
        return DNB_OK;
    }
    if (net->graph_input != device_input || net->graph_stream != s) {
        drop_graph(net);
        net->graph_input = device_input;
        net->graph_stream = s;
    }
    if (net->eager_runs++ == 0) return forward_eager(net, device_input, s);
    cudaGraph_t graph = nullptr;
    DNB_CUDA(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    const int rc = forward_eager(net, device_input, s);
    const cudaError_t ce = cudaStreamEndCapture(s, &graph);
    if (rc != DNB_OK || ce != cudaSuccess || !graph) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        net->graph_enabled = false;          // something on the path cannot be captured: stay eager from here on
        drop_graph(net);
        return forward_eager(net, device_input, s);
    }
    const cudaError_t ie = cudaGraphInstantiate(&net->graph_exec, graph, 0);
    cudaGraphDestroy(graph);
    if (ie != cudaSuccess) {
        cudaGetLastError();
        net->graph_exec = nullptr;
        net->graph_enabled = false;
        return forward_eager(net, device_input, s);
    }
    DNB_CUDA(cudaGraphLaunch(net->graph_exec, s));
    return DNB_OK;
}

extern "C" int dnb_conv_plan_check_status(dnb_conv_plan *p);

// The second set of buffers exists only once two steps are in flight.
static int ensure_second_slot(dnb_network *net)
{
    if (net->input_slot[1]) return DNB_OK;
    DNB_CUDA(cudaMalloc((void **)&net->input_slot[1], (size_t)net->batch * net->inputs * sizeof(float)));
    DNB_CUDA(cudaMallocHost((void **)&net->out_host_slot[1], (size_t)net->batch * net->outputs * sizeof(float)));
    for (Layer &L : net->layers)
        if (L.kind == L_YOLO && !L.host_slot[1]) DNB_CUDA(cudaMallocHost((void **)&L.host_slot[1], tensor_elems(&L.out) * sizeof(float)));
    return DNB_OK;
}

// Enqueues one step: images to the device on the upload stream, forward_network_gpu's loop
// (src/network.c:772-785) on the compute stream, and each [yolo] layer's pull to the host
// (src/yolo_layer.c:360) on the copy stream while the following layers compute.  Up to two steps may be
// in flight, so the copies of one step overlap the layers of the next.
extern "C" int dnb_network_submit(dnb_network *net, const float *input)
{
    if (!net || !input) DNB_FAIL(DNB_EINVAL, "network_submit: null argument");
    if (!net->weights_loaded) DNB_FAIL(DNB_EINVAL, "network_submit: load_weights has not been called");
    if (net->submitted - net->collected >= 2) DNB_FAIL(DNB_EINVAL, "network_submit: two steps are already in flight; collect one first");
    DNB_TRY(check_current_device(net->device, "network_submit"));
    const int slot = (int)(net->submitted & 1);
    if (slot == 1) DNB_TRY(ensure_second_slot(net));
    point_status(net, slot);
    cudaStream_t s = net->stream, cs = net->copy_stream, hs = net->h2d_stream;
    float *in_dev = net->input_slot[slot];
    // the slot's buffers are free: the step that used them last has been collected
    DNB_CUDA(cudaMemcpyAsync(in_dev, input, (size_t)net->batch * net->inputs * sizeof(float), cudaMemcpyHostToDevice, hs));
    DNB_CUDA(cudaEventRecord(net->in_ready[slot], hs));
    DNB_CUDA(cudaStreamWaitEvent(s, net->in_ready[slot], 0));
    DNB_TRY(prepare_input(net, in_dev, s));
    for (int i = 0; i < (int)net->layers.size(); ++i) {
        Layer &L = net->layers[i];
        if (L.kind == L_YOLO && net->submitted > 0) DNB_CUDA(cudaStreamWaitEvent(s, L.copied, 0));   // the previous step's pull has read L.out
        DNB_TRY(forward_layer(net, i, in_dev, s));
        if (L.kind == L_YOLO) {
            DNB_CUDA(cudaEventRecord(L.done, s));
            DNB_CUDA(cudaStreamWaitEvent(cs, L.done, 0));
            DNB_CUDA(cudaMemcpyAsync(L.host_slot[slot], L.out.data, tensor_elems(&L.out) * sizeof(float), cudaMemcpyDeviceToHost, cs));
            DNB_CUDA(cudaEventRecord(L.copied, cs));
        }
    }
    // Every device-to-host copy goes through the copy stream: a copy enqueued on the compute stream would
    // queue behind the large [yolo] pulls on the copy engine and hold back the next step's layers.
    Layer &last = net->layers.back();
    if (last.kind != L_YOLO) {   // the output layer is pulled last (src/network.c:786)
        dnb_tensor o{net->out_dev_nchw, DNB_NCHW, DNB_F32, net->batch, last.out_c, last.out_h, last.out_w, 0};
        if (net->submitted > 0) DNB_CUDA(cudaStreamWaitEvent(s, net->copy_done[slot ^ 1], 0));   // the previous step's pull has read out_dev_nchw
        DNB_TRY(launch_convert(&last.out, &o, 0, 0, 0, s));
    }
    DNB_CUDA(cudaEventRecord(net->fwd_done[slot], s));
    DNB_CUDA(cudaStreamWaitEvent(cs, net->fwd_done[slot], 0));
    if (last.kind != L_YOLO)
        DNB_CUDA(cudaMemcpyAsync(net->out_host_slot[slot], net->out_dev_nchw, (size_t)net->batch * net->outputs * sizeof(float), cudaMemcpyDeviceToHost, cs));
    DNB_CUDA(cudaMemcpyAsync(net->status_host + slot, net->status_dev + slot, sizeof(int), cudaMemcpyDeviceToHost, cs));
    DNB_CUDA(cudaEventRecord(net->copy_done[slot], cs));
    ++net->submitted;
    return DNB_OK;
}

// Waits for the oldest step in flight and hands out its results.
extern "C" int dnb_network_collect(dnb_network *net, float **output)
{
    if (!net || !output) DNB_FAIL(DNB_EINVAL, "network_collect: null argument");
    if (net->submitted == net->collected) DNB_FAIL(DNB_EINVAL, "network_collect: nothing has been submitted");
    const int slot = (int)(net->collected & 1);
    ++net->collected;
    DNB_CUDA(cudaEventSynchronize(net->copy_done[slot]));   // follows fwd_done[slot] and every copy of the step
    for (Layer &L : net->layers) if (L.kind == L_YOLO) L.host_out = L.host_slot[slot];
    if (net->status_host[slot]) {
        // this step's own word: the other step in flight keeps its word and its verdict
        const int code = net->status_host[slot];
        net->status_host[slot] = 0;
        cudaMemsetAsync(net->status_dev + slot, 0, sizeof(int), net->stream);   // before the slot's next step, which follows on this stream
        for (Layer &L : net->layers) conv_plan_reset_after_abort(L.plan, net->stream);
        char text[512];
        snprintf(text, sizeof(text), kTimeoutText, code);
        DNB_FAIL(DNB_ETIMEOUT, "network_predict: %s", text);
    }
    Layer &last = net->layers.back();
    *output = last.kind == L_YOLO ? last.host_out : net->out_host_slot[slot];
    return DNB_OK;
}

// network_predict (src/network.c:497-508): one step, start to finish.
extern "C" int dnb_network_predict(dnb_network *net, const float *input, float **output)
{
    if (!net || !input || !output) DNB_FAIL(DNB_EINVAL, "network_predict: null argument");
    if (net->submitted != net->collected) DNB_FAIL(DNB_EINVAL, "network_predict: a submitted step has not been collected");
    DNB_TRY(dnb_network_submit(net, input));
    return dnb_network_collect(net, output);
}

extern "C" int dnb_network_num_layers(const dnb_network *net) { return net ? (int)net->layers.size() : 0; }
extern "C" int dnb_network_batch(const dnb_network *net) { return net ? net->batch : 0; }
extern "C" int dnb_network_inputs(const dnb_network *net) { return net ? net->inputs : 0; }
extern "C" int dnb_network_outputs(const dnb_network *net) { return net ? net->outputs : 0; }

extern "C" int dnb_network_layer_shape(const dnb_network *net, int i, int *c, int *h, int *w)
{
    if (!net || i < 0 || i >= (int)net->layers.size()) DNB_FAIL(DNB_EINVAL, "layer index %d out of range", i);
    if (c) *c = net->layers[i].out_c;
    if (h) *h = net->layers[i].out_h;
    if (w) *w = net->layers[i].out_w;
    return DNB_OK;
}
extern "C" const char *dnb_network_layer_type(const dnb_network *net, int i)
{
    return (!net || i < 0 || i >= (int)net->layers.size()) ? "" : kKindNames[net->layers[i].kind];
}
extern "C" const char *dnb_network_layer_kernel(const dnb_network *net, int i)
{
    if (!net || i < 0 || i >= (int)net->layers.size()) return "";
    const Layer &L = net->layers[i];
    return L.plan ? dnb_conv_plan_kernel(L.plan) : kKindNames[L.kind];
}

// Images [first, first + count) of layer i's output, NCHW f32, to the host.
extern "C" int dnb_conv_plan_describe(const dnb_conv_plan *p, char *buf, int len);

extern "C" int dnb_network_layer_describe(const dnb_network *net, int i, char *buf, int len)
{
    if (!net || !buf || len < 1 || i < 0 || i >= (int)net->layers.size()) DNB_FAIL(DNB_EINVAL, "layer_describe: bad argument");
    const Layer &L = net->layers[i];
    if (L.plan) return dnb_conv_plan_describe(L.plan, buf, len);
    snprintf(buf, len, "%s", kKindNames[L.kind]);
    return DNB_OK;
}

extern "C" int dnb_network_layer_output_images(dnb_network *net, int i, int first, int count, float *host_out)
{
    if (!net || !host_out || i < 0 || i >= (int)net->layers.size()) DNB_FAIL(DNB_EINVAL, "layer_output: bad argument");
    if (first < 0 || count < 1 || first + count > net->batch) DNB_FAIL(DNB_EINVAL, "layer_output: images %d..%d of a batch of %d", first, first + count - 1, net->batch);
    Layer &L = net->layers[i];
    if (net->submitted != net->collected) DNB_FAIL(DNB_EINVAL, "layer_output: a submitted step is still in flight; collect it first");
    if (!L.out.data)
        DNB_FAIL(DNB_EUNSUPPORTED, "layer %d is fused into layer %d and has no output of its own (DNB_FUSE_SHORTCUT=0 / DNB_FUSE_YOLO=0 keep it)", i, i + 1);
    const size_t per_image = (size_t)L.out_c * L.out_h * L.out_w;
    const size_t elems = (size_t)count * per_image;
    DNB_CUDA(cudaDeviceSynchronize());  // the forward may have run on any stream
    if (L.out.layout == DNB_NCHW) {
        DNB_CUDA(cudaMemcpy(host_out, (const float *)L.out.data + (size_t)first * per_image, elems * sizeof(float), cudaMemcpyDeviceToHost));
        return DNB_OK;
    }
    // a run of whole images of a channels-last tensor is itself a channels-last tensor, if it starts on a 128-byte
    // boundary; where it does not (small maps with odd pitches) the whole layer is converted and the run copied out
    const size_t image_bytes = (size_t)L.out_h * L.out_w * L.out.cpitch * elem_size(L.out.dtype);
    const bool aligned = ((size_t)first * image_bytes) % 128 == 0;
    const int conv_first = aligned ? first : 0, conv_count = aligned ? count : net->batch;
    const size_t conv_elems = (size_t)conv_count * per_image;
    if (conv_elems > net->export_elems) {
        cudaFree(net->export_dev);
        net->export_dev = nullptr; net->export_elems = 0;
        DNB_CUDA(cudaMalloc((void **)&net->export_dev, conv_elems * sizeof(float)));
        net->export_elems = conv_elems;
    }
    dnb_tensor in = L.out;
    in.n = conv_count;
    in.data = (char *)L.out.data + (size_t)conv_first * image_bytes;
    dnb_tensor o{net->export_dev, DNB_NCHW, DNB_F32, conv_count, L.out_c, L.out_h, L.out_w, 0};
    DNB_TRY(launch_convert(&in, &o, 0, 0, 0, net->stream));
    DNB_CUDA(cudaStreamSynchronize(net->stream));
    DNB_CUDA(cudaMemcpy(host_out, net->export_dev + (size_t)(first - conv_first) * per_image, elems * sizeof(float), cudaMemcpyDeviceToHost));
    return DNB_OK;
}

extern "C" int dnb_network_layer_output(dnb_network *net, int i, float *host_out)
{
    if (!net) DNB_FAIL(DNB_EINVAL, "layer_output: bad argument");
    return dnb_network_layer_output_images(net, i, 0, net->batch, host_out);
}

// Waits for the device, then reads and clears both status words: DNB_ETIMEOUT if a bounded wait expired in any
// convolution since the last check.  For callers of the device-resident dnb_network_forward, which returns
// before its kernels have run; dnb_network_collect reports the same for submitted steps.
extern "C" int dnb_network_check_status(dnb_network *net)
{
    if (!net) DNB_FAIL(DNB_EINVAL, "check_status: null network");
    if (net->submitted != net->collected) DNB_FAIL(DNB_EINVAL, "check_status: a submitted step is still in flight; collect it first");
    int v[2] = {0, 0};
    DNB_CUDA(cudaDeviceSynchronize());
    DNB_CUDA(cudaMemcpy(v, net->status_dev, sizeof(v), cudaMemcpyDeviceToHost));
    if (v[0] || v[1]) {
        DNB_CUDA(cudaMemset(net->status_dev, 0, sizeof(v)));
        for (Layer &L : net->layers) conv_plan_reset_after_abort(L.plan);
        char text[512];
        snprintf(text, sizeof(text), kTimeoutText, v[0] ? v[0] : v[1]);
        DNB_FAIL(DNB_ETIMEOUT, "network_forward: %s", text);
    }
    return DNB_OK;
}

extern "C" int dnb_conv_plan_set_diagnostics(dnb_conv_plan *p, long long wait_limit_cycles, int debug_bits);

// dnb_conv_plan_set_diagnostics for convolution `layer` of the network.
extern "C" int dnb_network_set_diagnostics(dnb_network *net, int layer, long long wait_limit_cycles, int debug_bits)
{
    if (!net || layer < 0 || layer >= (int)net->layers.size()) DNB_FAIL(DNB_EINVAL, "set_diagnostics: bad argument");
    Layer &L = net->layers[layer];
    if (L.kind != L_CONV) DNB_FAIL(DNB_EINVAL, "set_diagnostics: layer %d is not convolutional", layer);
    // launches already enqueued carry their own copy of the argument block: only later ones see the change
    drop_graph(net);
    return dnb_conv_plan_set_diagnostics(L.plan, wait_limit_cycles, debug_bits);
}

extern "C" int dnb_network_yolo_output(dnb_network *net, int i, const float **host_out)
{
    if (!net || !host_out || i < 0 || i >= (int)net->layers.size()) DNB_FAIL(DNB_EINVAL, "yolo_output: bad argument");
    if (net->layers[i].kind != L_YOLO) DNB_FAIL(DNB_EINVAL, "layer %d is not a [yolo] layer", i);
    *host_out = net->layers[i].host_out;
    return DNB_OK;
}

// numops (examples/darknet.c:81-114): 2 * n * size^2 * c/groups * out_h * out_w per convolution and image.
extern "C" double dnb_network_flops(const dnb_network *net)
{
    double ops = 0;
    if (!net) return 0;
    for (const Layer &L : net->layers)
        if (L.kind == L_CONV)
            ops += 2.0 * L.cd.n * L.cd.size * L.cd.size * (L.cd.c / L.cd.groups) * L.out_h * L.out_w;
        else if (L.kind == L_CONNECTED)
            ops += 2.0 * L.fc_inputs * L.cd.n;   // examples/darknet.c:91-92
    return ops * net->batch;
}

extern "C" int dnb_network_launches(const dnb_network *net)
{
    int n = 0;
    if (!net) return 0;
    for (const Layer &L : net->layers) n += L.launches;
    if (net->input_nhwc.data) n += 1;
    return n;
}

// Forward with a CUDA event between layers, asynchronous like dnb_network_forward.  `slot` selects an
// independent set of events so that several timed forwards can be in flight before any is read.
extern "C" int dnb_network_forward_timed(dnb_network *net, const float *device_input, void *stream, int slot)
{
    if (!net || !device_input || slot < 0 || slot > 4096) DNB_FAIL(DNB_EINVAL, "network_forward_timed: bad argument");
    if (!net->weights_loaded) DNB_FAIL(DNB_EINVAL, "network_forward_timed: load_weights has not been called");
    if (net->submitted != net->collected) DNB_FAIL(DNB_EINVAL, "network_forward_timed: a submitted step is still in flight; collect it first");
    DNB_TRY(check_current_device(net->device, "network_forward_timed"));
    point_status(net, 0);
    const int n = (int)net->layers.size();
    while ((int)net->events.size() < (slot + 1) * (n + 1)) {
        cudaEvent_t e;
        DNB_CUDA(cudaEventCreate(&e));
        net->events.push_back(e);
    }
    cudaStream_t s = (cudaStream_t)stream;
    cudaEvent_t *ev = &net->events[(size_t)slot * (n + 1)];
    DNB_TRY(prepare_input(net, device_input, s));   // outside the per-layer brackets: layer 0's time is its kernel's
    for (int i = 0; i < n; ++i) {
        DNB_CUDA(cudaEventRecord(ev[i], s));
        DNB_TRY(forward_layer(net, i, device_input, s));
    }
    DNB_CUDA(cudaEventRecord(ev[n], s));
    return DNB_OK;
}

// Per-layer device time of the timed forward in `slot`, milliseconds; waits for that forward to finish.
extern "C" int dnb_network_timed_ms(dnb_network *net, int slot, float *layer_ms)
{
    if (!net || !layer_ms || slot < 0) DNB_FAIL(DNB_EINVAL, "network_timed_ms: bad argument");
    const int n = (int)net->layers.size();
    if ((int)net->events.size() < (slot + 1) * (n + 1)) DNB_FAIL(DNB_EINVAL, "network_timed_ms: slot %d was never recorded", slot);
    cudaEvent_t *ev = &net->events[(size_t)slot * (n + 1)];
    DNB_CUDA(cudaEventSynchronize(ev[n]));
    for (int i = 0; i < n; ++i) DNB_CUDA(cudaEventElapsedTime(&layer_ms[i], ev[i], ev[i + 1]));
    return DNB_OK;
}

extern "C" int dnb_network_profile(dnb_network *net, const float *device_input, float *layer_ms)
{
    DNB_TRY(dnb_network_forward_timed(net, device_input, net->stream, 0));
    return dnb_network_timed_ms(net, 0, layer_ms);
}
