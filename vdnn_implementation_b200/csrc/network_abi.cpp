// extern "C" face of class Network for hosts that are not C++ (section 4 of vdnn_b200.h).
#include <new>

#include "dp_nccl.h"
#include "network.h"

namespace vdnn { extern unsigned long long g_kernel_launches; }

struct vdnn_network { Network* impl; };

#define NET(n) do { if (!(n) || !(n)->impl) return VDNN_ERR_BAD_ARG; } while (0)

extern "C" {

// dry_run is requested by setting device to -1: the schedule is replayed against a bookkeeping-only
// pool and no CUDA call is made.
int vdnn_network_create(vdnn_network** out, const vdnn_network_config* cfg) {
    if (!out || !cfg) return VDNN_ERR_BAD_ARG;
    *out = nullptr;
    vdnn_network_config c = *cfg;
    const bool dry = c.device < 0;
    Network* n = new (std::nothrow) Network(c, dry);
    if (!n) return VDNN_ERR_OUT_OF_MEMORY;
    if (n->status() != VDNN_OK) { const int st = n->status(); delete n; return st; }
    vdnn_network* h = new (std::nothrow) vdnn_network;
    if (!h) { delete n; return VDNN_ERR_OUT_OF_MEMORY; }
    h->impl = n;
    *out = h;
    return VDNN_OK;
}

int vdnn_network_destroy(vdnn_network* net) {
    if (!net) return VDNN_OK;
    delete net->impl;
    delete net;
    return VDNN_OK;
}

int vdnn_network_num_layers(const vdnn_network* net) { return (net && net->impl) ? net->impl->numLayers_() : 0; }

int vdnn_network_layer_spec(const vdnn_network* net, int layer, vdnn_layer_spec* out) {
    NET(net);
    if (!out || layer < 0 || layer >= net->impl->numLayers_()) return VDNN_ERR_BAD_ARG;
    net->impl->layerArray()[layer]->spec(out);
    return VDNN_OK;
}

size_t vdnn_network_input_size(const vdnn_network* net) { return (net && net->impl) ? net->impl->getInputSize() : 0; }
size_t vdnn_network_output_size(const vdnn_network* net) { return (net && net->impl) ? net->impl->getOutputSize() : 0; }

int vdnn_network_set_input(vdnn_network* net, const float* input_h, const float* label_h) { NET(net); return net->impl->setInput(input_h, label_h); }
int vdnn_network_seed_input(vdnn_network* net, uint64_t a, uint64_t b) { NET(net); return net->impl->seedInput(a, b); }
int vdnn_network_forward(vdnn_network* net) { NET(net); return net->impl->forwardPropagation(false); }
int vdnn_network_backward(vdnn_network* net) { NET(net); return net->impl->backwardPropagation(false); }
int vdnn_network_synchronize(vdnn_network* net) { NET(net); return net->impl->synchronize(); }
void* vdnn_network_stream(vdnn_network* net, int which) {
    if (!net || !net->impl) return nullptr;
    vdnnContext& c = net->impl->context();
    switch (which) {
    case 0: return c.stream_compute;
    case 1: return c.stream_d2h;
    case 2: return c.stream_h2d;
    case 3: return c.stream_comm;
    default: return nullptr;
    }
}
int vdnn_network_join(vdnn_network* net) { NET(net); return net->impl->join(); }
unsigned long long vdnn_kernel_launch_count(void) { return vdnn::g_kernel_launches; }
int vdnn_network_loss(vdnn_network* net, double* out2) { NET(net); return net->impl->loss(out2); }

size_t vdnn_network_tensor_size(const vdnn_network* net, int layer, int kind) {
    return (net && net->impl) ? net->impl->tensorSize(layer, kind) : 0;
}
int vdnn_network_read_tensor(vdnn_network* net, int layer, int kind, float* dst_h, size_t count) { NET(net); return net->impl->readTensor(layer, kind, dst_h, count); }
int vdnn_network_write_tensor(vdnn_network* net, int layer, int kind, const float* src_h, size_t count) { NET(net); return net->impl->writeTensor(layer, kind, src_h, count); }

int vdnn_network_trace(vdnn_network* net, vdnn_trace_event* out, int max_events, int* num_events) {
    NET(net);
    const std::vector<vdnn_trace_event>& t = net->impl->context().trace;
    if (num_events) *num_events = static_cast<int>(t.size());
    if (out) for (int i = 0; i < max_events && i < static_cast<int>(t.size()); ++i) out[i] = t[i];
    return VDNN_OK;
}
int vdnn_network_trace_reset(vdnn_network* net) { NET(net); net->impl->context().trace.clear(); return VDNN_OK; }

int vdnn_network_get_stats(vdnn_network* net, vdnn_network_stats* out) { NET(net); return net->impl->getStats(out); }
int vdnn_network_set_profiling(vdnn_network* net, int enabled) { NET(net); return net->impl->setProfiling(enabled != 0); }

int vdnn_network_selected(vdnn_network* net, int* vdnn_type, int* algo_mode) { NET(net); net->impl->selected(vdnn_type, algo_mode); return VDNN_OK; }
int vdnn_network_layer_algos(vdnn_network* net, int layer, int* out3) { NET(net); return net->impl->layerAlgos(layer, out3); }

int vdnn_network_set_offload_order(vdnn_network* net, int forward_order) { NET(net); return net->impl->setOffloadOrder(forward_order != 0); }

int vdnn_set_lean_offload(int on) { Network::setLeanOffloadDefault(on); return VDNN_OK; }
int vdnn_network_lean(const vdnn_network* net) { return (net && net->impl && net->impl->leanOffload()) ? 1 : 0; }

int vdnn_network_timeline(vdnn_network* net, float* out) { NET(net); return net->impl->timeline(out); }

int vdnn_dp_unique_id(char* out128) { return vdnn::dp_unique_id(out128); }
int vdnn_network_enable_dp(vdnn_network* net, int rank, int world, const char* id) { NET(net); return net->impl->enableDataParallel(rank, world, id); }
int vdnn_network_dp_mode(vdnn_network* net) { NET(net); return net->impl->dpMode(); }
int vdnn_network_weight_checksum(vdnn_network* net, uint64_t* out) { NET(net); return net->impl->weightChecksum(out); }

}  // extern "C"
