// Expert parallelism, all-gather form, as ONE host call per step: every launch of every layer and both collectives of a
// layer are queued from C on the caller's stream, so the step costs a few microseconds of host time per launch instead
// of a Python / torch.distributed round trip per operation (measured at two ranks: the Python loop needed as long to
// queue a 48-layer step as the devices needed to run it).
//
// No reference counterpart: the reference is single-device. The pair layout is its expert_start / pair_token /
// pair_weight (native/redmetal_topk.h:182-190), the arithmetic that of the single-device layer (redcuda_moe.cu).
//
// Per layer, with T tokens on every rank and experts sharded as the layer objects say:
//   shared     the rank's own tokens through the shared expert, on a side stream next to everything up to the combine
//   route      router logits (or the caller's drawn logits) -> ids / weights of the rank's own tokens
//   quantise   the rank's token rows into the int8 digits the expert kernels read (once, by their owner, instead of by
//              every rank after the exchange; 3 bytes per value cross the links instead of 4)
//   all-gather digits, row scales, ids and weights of every rank (four ncclAllGather calls in one group: one launch)
//   partial    this shard's experts over the pairs of ALL tokens that select them; the combine sums a token's local
//              pairs and adds the shared-expert part to the rank's own tokens
//   reduce     ncclReduceScatter(sum) of the partial outputs straight into the caller's output rows
// Layers whose expert kernels take fp32 rows (non-IQ2_XXS experts) gather the fp32 rows instead of digits.
// NCCL is loaded at run time (dlopen of libnccl.so.2, which resolves to the copy the process already holds when the
// caller is a torch.distributed program); the library itself has no link dependency on it. world = 1 needs no NCCL.
#include "redcuda_common.cuh"
#include "redcuda_kernels.cuh"
#include "redcuda_moe_mma.cuh"
#include "../../include/redcuda.h"

#include <dlfcn.h>
#include <new>
#include <string.h>

namespace rc {

// the handful of NCCL entry points used, by their public prototypes (nccl.h)
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { ncclInt8 = 0, ncclUint32 = 3, ncclFloat32 = 7, ncclSum = 0 };
struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
};

static NcclApi *nccl_api() {
    static NcclApi api;
    static bool tried = false;
    if (tried) return api.handle ? &api : nullptr;
    tried = true;
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) { set_error("expert parallelism: libnccl.so.2 could not be loaded: %s", dlerror()); return nullptr; }
    api.GetUniqueId = (decltype(api.GetUniqueId))dlsym(h, "ncclGetUniqueId");
    api.CommInitRank = (decltype(api.CommInitRank))dlsym(h, "ncclCommInitRank");
    api.CommDestroy = (decltype(api.CommDestroy))dlsym(h, "ncclCommDestroy");
    api.GroupStart = (decltype(api.GroupStart))dlsym(h, "ncclGroupStart");
    api.GroupEnd = (decltype(api.GroupEnd))dlsym(h, "ncclGroupEnd");
    api.AllGather = (decltype(api.AllGather))dlsym(h, "ncclAllGather");
    api.ReduceScatter = (decltype(api.ReduceScatter))dlsym(h, "ncclReduceScatter");
    api.GetErrorString = (decltype(api.GetErrorString))dlsym(h, "ncclGetErrorString");
    if (!api.GroupStart || !api.GroupEnd || !api.GetUniqueId || !api.CommInitRank || !api.CommDestroy || !api.AllGather || !api.ReduceScatter || !api.GetErrorString) {
        set_error("expert parallelism: libnccl.so.2 lacks an expected entry point");
        return nullptr;
    }
    api.handle = h;
    return &api;
}

#define RC_NCCL(api, expr) do { ncclResult_t r_ = (expr); if (r_ != 0) { rc::set_error("%s failed: %s", #expr, (api)->GetErrorString(r_)); return 0; } } while (0)

bool moe_takes_digits(const redcuda_moe *m);                  // redcuda_moe.cu
int moe_partial_gathered(redcuda_moe *m, uint32_t ntok, const float *x, const int8_t *xq, const float *sx, const uint32_t *ids, const float *w,
                         const float *add, uint32_t add_begin, uint32_t add_count, float *out, cudaStream_t s);

}  // namespace rc

using namespace rc;

struct redcuda_ep {
    int rank = 0, world = 1, device = 0;
    uint32_t tokens = 0, hidden = 0, top_k = 0;
    ncclComm_t comm = nullptr;
    DevMem buf;
    // own tokens: digits, scales, ids, weights, shared-expert part; gathered: the same four plus fp32 rows; partial sums
    int8_t *xq = nullptr, *xq_all = nullptr;
    float *sx = nullptr, *sx_all = nullptr, *w = nullptr, *w_all = nullptr, *x_all = nullptr, *shared = nullptr, *partial = nullptr;
    uint32_t *ids = nullptr, *ids_all = nullptr;
    cudaStream_t side = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
};

extern "C" {

int redcuda_ep_unique_id(void *out128) {
    RC_REQUIRE(out128, "ep unique id: null buffer");
    NcclApi *api = nccl_api();
    if (!api) return 0;
    ncclUniqueId id;
    RC_NCCL(api, api->GetUniqueId(&id));
    memcpy(out128, &id, sizeof(id));
    return 1;
}

void redcuda_ep_destroy(redcuda_ep *ep) {
    if (!ep) return;
    if (ep->side) { cudaStreamSynchronize(ep->side); cudaStreamDestroy(ep->side); }
    if (ep->ev_fork) cudaEventDestroy(ep->ev_fork);
    if (ep->ev_join) cudaEventDestroy(ep->ev_join);
    if (ep->comm) { NcclApi *api = nccl_api(); if (api) api->CommDestroy(ep->comm); }
    delete ep;
}

redcuda_ep *redcuda_ep_create(int rank, int world, const void *unique_id128, uint32_t tokens, uint32_t hidden, uint32_t top_k) {
    if (!require_device()) return nullptr;
    if (world < 1 || rank < 0 || rank >= world || !tokens || !hidden || hidden % 4u || !top_k || top_k > REDCUDA_MAX_TOPK) {
        set_error("ep create: bad rank / world / shape (rank %d of %d, %u tokens, hidden %u, top_k %u; hidden must be a multiple of 4)", rank, world, tokens, hidden, top_k);
        return nullptr;
    }
    redcuda_ep *ep = new (std::nothrow) redcuda_ep();
    if (!ep) { set_error("ep create: out of host memory"); return nullptr; }
    ep->rank = rank; ep->world = world; ep->tokens = tokens; ep->hidden = hidden; ep->top_k = top_k;
    cudaGetDevice(&ep->device);
    auto bail = [&](const char *why) -> redcuda_ep * { if (why) set_error("ep create: %s", why); redcuda_ep_destroy(ep); return nullptr; };
    const size_t T = tokens, W = (size_t)world, H = hidden, K = top_k;
    size_t total = 0;
    auto take = [&](size_t bytes) { const size_t o = total; total = (total + bytes + 255u) / 256u * 256u; return o; };
    const size_t o_xq = take(T * 3u * H), o_sx = take(T * 4u), o_ids = take(T * K * 4u), o_w = take(T * K * 4u), o_sh = take(T * H * 4u),
                 o_xqa = take(W * T * 3u * H), o_sxa = take(W * T * 4u), o_idsa = take(W * T * K * 4u), o_wa = take(W * T * K * 4u), o_xa = take(W * T * H * 4u),
                 o_part = take(W * T * H * 4u);
    if (!ep->buf.alloc(total)) return bail(nullptr);
    uint8_t *B = ep->buf.as<uint8_t>();
    ep->xq = (int8_t *)(B + o_xq); ep->sx = (float *)(B + o_sx); ep->ids = (uint32_t *)(B + o_ids); ep->w = (float *)(B + o_w); ep->shared = (float *)(B + o_sh);
    ep->xq_all = (int8_t *)(B + o_xqa); ep->sx_all = (float *)(B + o_sxa); ep->ids_all = (uint32_t *)(B + o_idsa); ep->w_all = (float *)(B + o_wa);
    ep->x_all = (float *)(B + o_xa); ep->partial = (float *)(B + o_part);
    if (cudaMemset(B, 0, total) != cudaSuccess) return bail("workspace memset failed");
    if (cudaStreamCreateWithFlags(&ep->side, cudaStreamNonBlocking) != cudaSuccess || cudaEventCreateWithFlags(&ep->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&ep->ev_join, cudaEventDisableTiming) != cudaSuccess) return bail("stream / event creation failed");
    if (world > 1) {
        if (!unique_id128) return bail("a unique id from rank 0 (redcuda_ep_unique_id) is required when world > 1");
        NcclApi *api = nccl_api();
        if (!api) { redcuda_ep_destroy(ep); return nullptr; }
        ncclUniqueId id;
        memcpy(&id, unique_id128, sizeof(id));
        const ncclResult_t r = api->CommInitRank(&ep->comm, world, id, rank);
        if (r != 0) { set_error("ep create: ncclCommInitRank failed: %s", api->GetErrorString(r)); ep->comm = nullptr; redcuda_ep_destroy(ep); return nullptr; }
    }
    return ep;
}

int redcuda_ep_layer_forward(redcuda_ep *ep, redcuda_moe *layer, const float *x_dev, const float *logits_in_dev, float *out_dev, void *stream) {
    RC_REQUIRE(ep && layer && x_dev && out_dev, "ep layer: null argument");
    cudaStream_t s = (cudaStream_t)stream;
    const uint32_t T = ep->tokens, H = ep->hidden, k = ep->top_k, W = (uint32_t)ep->world;
    // the shared expert needs neither the router nor the exchange: side stream, joined before the experts' combine
    RC_CUDA(cudaEventRecord(ep->ev_fork, s));
    RC_CUDA(cudaStreamWaitEvent(ep->side, ep->ev_fork, 0));
    if (!redcuda_moe_shared_device(layer, T, x_dev, ep->shared, ep->side)) return 0;
    RC_CUDA(cudaEventRecord(ep->ev_join, ep->side));
    if (!redcuda_moe_route_device(layer, T, x_dev, logits_in_dev, ep->ids, ep->w, s)) return 0;
    const bool digits = moe_takes_digits(layer);
    if (digits && !launch_quant_act(x_dev, H, T, H, ep->xq, ep->sx, s)) return 0;
    if (W == 1u) {
        RC_CUDA(cudaStreamWaitEvent(s, ep->ev_join, 0));
        return moe_partial_gathered(layer, T, x_dev, digits ? ep->xq : nullptr, ep->sx, ep->ids, ep->w, ep->shared, 0u, T, out_dev, s);
    }
    NcclApi *api = nccl_api();
    if (!api) return 0;
    prof_begin("ep_all_gather", s);
    RC_NCCL(api, api->GroupStart());
    if (digits) {
        RC_NCCL(api, api->AllGather(ep->xq, ep->xq_all, (size_t)T * 3u * H, ncclInt8, ep->comm, s));
        RC_NCCL(api, api->AllGather(ep->sx, ep->sx_all, (size_t)T, ncclFloat32, ep->comm, s));
    } else RC_NCCL(api, api->AllGather(x_dev, ep->x_all, (size_t)T * H, ncclFloat32, ep->comm, s));
    RC_NCCL(api, api->AllGather(ep->ids, ep->ids_all, (size_t)T * k, ncclUint32, ep->comm, s));
    RC_NCCL(api, api->AllGather(ep->w, ep->w_all, (size_t)T * k, ncclFloat32, ep->comm, s));
    RC_NCCL(api, api->GroupEnd());
    prof_end(s);
    RC_CUDA(cudaStreamWaitEvent(s, ep->ev_join, 0));
    if (!moe_partial_gathered(layer, W * T, digits ? nullptr : ep->x_all, digits ? ep->xq_all : nullptr, ep->sx_all, ep->ids_all, ep->w_all,
                              ep->shared, (uint32_t)ep->rank * T, T, ep->partial, s)) return 0;
    prof_begin("ep_reduce_scatter", s);
    RC_NCCL(api, api->ReduceScatter(ep->partial, out_dev, (size_t)T * H, ncclFloat32, ncclSum, ep->comm, s));
    prof_end(s);
    return 1;
}

int redcuda_ep_step(redcuda_ep *ep, redcuda_moe *const *layers, uint32_t n_layers, const float *const *x_dev, const float *const *logits_in_dev, float *const *out_dev, void *stream) {
    RC_REQUIRE(ep && layers && n_layers && x_dev && out_dev, "ep step: null or empty argument");
    for (uint32_t l = 0; l < n_layers; ++l)
        if (!redcuda_ep_layer_forward(ep, layers[l], x_dev[l], logits_in_dev ? logits_in_dev[l] : nullptr, out_dev[l], stream)) return 0;
    return 1;
}

}  // extern "C"
