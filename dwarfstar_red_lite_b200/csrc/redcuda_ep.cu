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
//
// Two exchanges. NCCL (the fallback and A/B): the calls above. Peer memory (after redcuda_ep_attach_peers; ranks are
// processes on one node whose exchange areas are mapped into each other with CUDA IPC): the all-gather becomes a push
// (k_ep_push stores the rank's rows into every rank's gather area over NVLink and publishes a sequence number in a flag
// word of every rank; the grouping kernel of the partial step waits for all flags), the reduce-scatter becomes the
// combine itself (k_ep_combine_push stores every token's partial row into the slot its owner keeps for this rank and
// publishes a second flag; k_ep_reduce on the owner waits for all ranks and adds the slots and the shared part). No
// collective kernel remains between the compute kernels. Every wait is bounded (EP_WAIT_NS); a wait that runs out sets
// the sticky status word and a device-local word that makes every later wait return at once, so a step with a missing
// rank ends (with garbage in its outputs and an error at the next synchronisation) instead of hanging.
// Why one buffer per direction is enough: a rank pushes the rows of step n + 1 only after its own reduce of step n, which
// waited for every rank's combine of step n, which ran after that rank's expert kernels had read the rows of step n; the
// slots of step n + 1 are written after the writer's grouping kernel saw the owner's push of step n + 1, which the owner
// queued behind its reduce of step n.
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

bool moe_takes_digits(redcuda_moe *m, uint32_t ntok);          // redcuda_moe.cu
int moe_partial_gathered(redcuda_moe *m, uint32_t ntok, const float *x, const int8_t *xq, const float *sx, const uint32_t *ids, const float *w,
                         const float *add, uint32_t add_begin, uint32_t add_count, float *out, cudaStream_t s, const EpWait *wait, const EpPush *push);

// The rank's own rows into every rank's gather area: up to four segments (digits or fp32 rows, scales, ids, weights), each
// stored at off[i] + rank * bytes[i] of every area; then the gather flag. 16-byte stores where a segment allows them.
struct EpPushArgs { EpPeers peers; const uint8_t *src[4]; size_t off[4]; uint32_t bytes[4]; uint32_t nseg; size_t off_flag; uint32_t seq; uint32_t *ticket; };
__global__ void __launch_bounds__(256) k_ep_push(const __grid_constant__ EpPushArgs A) {
    pdl_prologue();
    const uint32_t gtid = blockIdx.x * 256u + threadIdx.x, gsize = gridDim.x * 256u;
    for (uint32_t sg = 0; sg < A.nseg; ++sg) {
        const uint32_t bytes = A.bytes[sg];
        if (bytes % 16u == 0) {
            const uint4 *src = reinterpret_cast<const uint4 *>(A.src[sg]);
            for (uint32_t i = gtid; i < bytes / 16u; i += gsize) {
                const uint4 v = src[i];
                for (uint32_t p = 0; p < A.peers.world; ++p) reinterpret_cast<uint4 *>(A.peers.base[p] + A.off[sg] + (size_t)A.peers.rank * bytes)[i] = v;
            }
        } else {
            const uint32_t *src = reinterpret_cast<const uint32_t *>(A.src[sg]);
            for (uint32_t i = gtid; i < bytes / 4u; i += gsize) {
                const uint32_t v = src[i];
                for (uint32_t p = 0; p < A.peers.world; ++p) reinterpret_cast<uint32_t *>(A.peers.base[p] + A.off[sg] + (size_t)A.peers.rank * bytes)[i] = v;
            }
        }
    }
    ep_signal_all(A.peers, A.off_flag, A.seq, A.ticket, gridDim.x);
}

// out[t] = (resid[t] +) shared[t] + sum over ranks r of slot[r][t], once every rank's combine has delivered. grid = (hidden / 1024, tokens)
__global__ void __launch_bounds__(256) k_ep_reduce(const float *__restrict__ slots, const float *__restrict__ shared, const float *__restrict__ resid, uint32_t world, uint32_t tokens,
                                                   uint32_t hidden, const EpWait wait, float *__restrict__ out) {
    pdl_prologue();
    ep_wait_all(wait);
    const uint32_t t = blockIdx.y, r = (blockIdx.x * 256u + threadIdx.x) * 4u;
    if (r >= hidden) return;
    float4 acc = *reinterpret_cast<const float4 *>(shared + (size_t)t * hidden + r);
    if (resid) { const float4 v = *reinterpret_cast<const float4 *>(resid + (size_t)t * hidden + r); acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w; }
    for (uint32_t p = 0; p < world; ++p) {
        const float4 v = __ldcg(reinterpret_cast<const float4 *>(slots + ((size_t)p * tokens + t) * hidden + r));      // written by another GPU: read at L2
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    *reinterpret_cast<float4 *>(out + (size_t)t * hidden + r) = acc;
}

// io[i] += resid[i], n4 float4s (the residual of the NCCL and single-rank paths, whose sums end in the caller's buffer)
__global__ void __launch_bounds__(256) k_ep_add_resid(float4 *__restrict__ io, const float4 *__restrict__ resid, uint32_t n4) {
    pdl_prologue();
    const uint32_t i = blockIdx.x * 256u + threadIdx.x;
    if (i >= n4) return;
    float4 a = io[i];
    const float4 b = resid[i];
    a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    io[i] = a;
}

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
    // peer-memory exchange: the area other ranks write into (gathered rows, slots, flags), its mappings, the step counter
    DevMem xch;
    size_t o_xq = 0, o_sx = 0, o_ids = 0, o_w = 0, o_x = 0, o_part = 0, o_gflag = 0, o_rflag = 0;
    uint32_t *dead = nullptr, *ticket = nullptr;
    EpPeers peers{};
    bool attached = false;
    uint32_t seq = 0;
};

static int add_resid(float *io, const float *resid, uint32_t n4, cudaStream_t s) {
    if (!resid) return 1;
    prof_begin("ep_add_resid", s);
    RC_LAUNCH((k_ep_add_resid), (n4 + 255u) / 256u, 256, 0, s, reinterpret_cast<float4 *>(io), reinterpret_cast<const float4 *>(resid), n4);
    prof_end(s);
    RC_LAUNCHED();
    return 1;
}

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
    if (ep->attached)
        for (uint32_t p = 0; p < ep->peers.world; ++p)
            if ((int)p != ep->rank && ep->peers.base[p]) cudaIpcCloseMemHandle(ep->peers.base[p]);
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
    const size_t o_xq = take(T * 3u * H), o_sx = take(T * 4u), o_ids = take(T * K * 4u), o_w = take(T * K * 4u), o_sh = take(T * H * 4u), o_part = take(W * T * H * 4u);
    if (!ep->buf.alloc(total)) return bail(nullptr);
    uint8_t *B = ep->buf.as<uint8_t>();
    ep->xq = (int8_t *)(B + o_xq); ep->sx = (float *)(B + o_sx); ep->ids = (uint32_t *)(B + o_ids); ep->w = (float *)(B + o_w); ep->shared = (float *)(B + o_sh);
    ep->partial = (float *)(B + o_part);
    if (cudaMemset(B, 0, total) != cudaSuccess) return bail("workspace memset failed");
    // the exchange area: what other ranks write (same layout on every rank)
    total = 0;
    ep->o_xq = take(W * T * 3u * H); ep->o_sx = take(W * T * 4u); ep->o_ids = take(W * T * K * 4u); ep->o_w = take(W * T * K * 4u); ep->o_x = take(W * T * H * 4u);
    ep->o_part = take(W * T * H * 4u); ep->o_gflag = take(EP_MAX_WORLD * 128u); ep->o_rflag = take(EP_MAX_WORLD * 128u);
    const size_t o_dead = take(256u);
    if (!ep->xch.alloc(total)) return bail(nullptr);
    uint8_t *X = ep->xch.as<uint8_t>();
    ep->xq_all = (int8_t *)(X + ep->o_xq); ep->sx_all = (float *)(X + ep->o_sx); ep->ids_all = (uint32_t *)(X + ep->o_ids); ep->w_all = (float *)(X + ep->o_w);
    ep->x_all = (float *)(X + ep->o_x); ep->dead = (uint32_t *)(X + o_dead); ep->ticket = ep->dead + 8;
    if (cudaMemset(X, 0, total) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess) return bail("exchange area memset failed");
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

int redcuda_ep_ipc_handle(redcuda_ep *ep, void *out64) {
    RC_REQUIRE(ep && out64, "ep ipc handle: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    RC_CUDA(cudaIpcGetMemHandle(&h, ep->xch.p));
    memcpy(out64, &h, sizeof(h));
    return 1;
}

int redcuda_ep_attach_peers(redcuda_ep *ep, const void *handles) {
    RC_REQUIRE(ep && handles, "ep attach: null argument");
    RC_REQUIRE(!ep->attached, "ep attach: already attached");
    RC_REQUIRE(ep->world >= 2 && ep->world <= (int)EP_MAX_WORLD, "ep attach: the peer-memory exchange serves 2 to %u ranks", EP_MAX_WORLD);
    ep->peers = EpPeers{};
    ep->peers.world = (uint32_t)ep->world; ep->peers.rank = (uint32_t)ep->rank;
    for (int p = 0; p < ep->world; ++p) {
        if (p == ep->rank) { ep->peers.base[p] = ep->xch.as<uint8_t>(); continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, (const uint8_t *)handles + (size_t)p * sizeof(h), sizeof(h));
        void *ptr = nullptr;
        const cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) {
            for (int q = 0; q < p; ++q) if (q != ep->rank && ep->peers.base[q]) cudaIpcCloseMemHandle(ep->peers.base[q]);
            ep->peers = EpPeers{};
            set_error("ep attach: cudaIpcOpenMemHandle for rank %d failed: %s", p, cudaGetErrorString(e));
            return 0;
        }
        ep->peers.base[p] = (uint8_t *)ptr;
    }
    ep->attached = true;
    return 1;
}

// back to the NCCL exchange (a caller uses it when some other rank could not map the areas: all ranks must agree)
int redcuda_ep_detach_peers(redcuda_ep *ep) {
    RC_REQUIRE(ep, "ep detach: null argument");
    if (!ep->attached) return 1;
    RC_CUDA(cudaDeviceSynchronize());
    for (uint32_t p = 0; p < ep->peers.world; ++p)
        if ((int)p != ep->rank && ep->peers.base[p]) cudaIpcCloseMemHandle(ep->peers.base[p]);
    ep->peers = EpPeers{};
    ep->attached = false;
    return 1;
}

int redcuda_ep_layer_forward_n(redcuda_ep *ep, redcuda_moe *layer, uint32_t ntok, const float *x_dev, const float *logits_in_dev, const float *resid_dev, float *out_dev, void *stream) {
    RC_REQUIRE(ep && layer && x_dev && out_dev, "ep layer: null argument");
    RC_REQUIRE(ntok >= 1u && ntok <= ep->tokens, "ep layer: %u tokens outside [1, %u]", ntok, ep->tokens);
    cudaStream_t s = (cudaStream_t)stream;
    const uint32_t T = ntok, H = ep->hidden, k = ep->top_k, W = (uint32_t)ep->world;
    // the shared expert needs neither the router nor the exchange: side stream, joined before the experts' combine
    RC_CUDA(cudaEventRecord(ep->ev_fork, s));
    RC_CUDA(cudaStreamWaitEvent(ep->side, ep->ev_fork, 0));
    if (!redcuda_moe_shared_device(layer, T, x_dev, ep->shared, ep->side)) return 0;
    RC_CUDA(cudaEventRecord(ep->ev_join, ep->side));
    if (!redcuda_moe_route_device(layer, T, x_dev, logits_in_dev, ep->ids, ep->w, s)) return 0;
    const bool digits = moe_takes_digits(layer, W * T);
    if (digits && !launch_quant_act(x_dev, H, T, H, ep->xq, ep->sx, s)) return 0;
    if (W == 1u) {
        RC_CUDA(cudaStreamWaitEvent(s, ep->ev_join, 0));
        if (!moe_partial_gathered(layer, T, x_dev, digits ? ep->xq : nullptr, ep->sx, ep->ids, ep->w, ep->shared, 0u, T, out_dev, s, nullptr, nullptr)) return 0;
        return add_resid(out_dev, resid_dev, T * H / 4u, s);
    }
    if (ep->attached) {
        const uint32_t seq = ++ep->seq;
        EpPushArgs P{};
        P.peers = ep->peers; P.off_flag = ep->o_gflag; P.seq = seq; P.ticket = ep->ticket;
        uint32_t n = 0;
        auto seg = [&](const void *src, size_t off, size_t bytes) { P.src[n] = (const uint8_t *)src; P.off[n] = off; P.bytes[n] = (uint32_t)bytes; ++n; };
        if (digits) { seg(ep->xq, ep->o_xq, (size_t)T * 3u * H); seg(ep->sx, ep->o_sx, (size_t)T * 4u); }
        else seg(x_dev, ep->o_x, (size_t)T * H * 4u);
        seg(ep->ids, ep->o_ids, (size_t)T * k * 4u); seg(ep->w, ep->o_w, (size_t)T * k * 4u);
        P.nseg = n;
        prof_begin("ep_push", s);
        RC_LAUNCH((k_ep_push), 64, 256, 0, s, P);
        prof_end(s);
        RC_LAUNCHED();
        uint8_t *X = ep->xch.as<uint8_t>();
        const EpWait wg{reinterpret_cast<const uint32_t *>(X + ep->o_gflag), W, seq, ep->dead, status_words()};
        const EpWait wr{reinterpret_cast<const uint32_t *>(X + ep->o_rflag), W, seq, ep->dead, status_words()};
        const EpPush pp{ep->peers, ep->o_part, ep->o_rflag, T, seq, ep->ticket + 1};
        if (!moe_partial_gathered(layer, W * T, digits ? nullptr : ep->x_all, digits ? ep->xq_all : nullptr, ep->sx_all, ep->ids_all, ep->w_all,
                                  nullptr, 0u, 0u, nullptr, s, &wg, &pp)) return 0;
        RC_CUDA(cudaStreamWaitEvent(s, ep->ev_join, 0));
        prof_begin("ep_reduce", s);
        RC_LAUNCH((k_ep_reduce), dim3((H / 4u + 255u) / 256u, T), 256, 0, s, reinterpret_cast<const float *>(X + ep->o_part), ep->shared, resid_dev, W, T, H, wr, out_dev);
        prof_end(s);
        RC_LAUNCHED();
        return 1;
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
                              ep->shared, (uint32_t)ep->rank * T, T, ep->partial, s, nullptr, nullptr)) return 0;
    prof_begin("ep_reduce_scatter", s);
    RC_NCCL(api, api->ReduceScatter(ep->partial, out_dev, (size_t)T * H, ncclFloat32, ncclSum, ep->comm, s));
    prof_end(s);
    return add_resid(out_dev, resid_dev, T * H / 4u, s);
}

int redcuda_ep_layer_forward(redcuda_ep *ep, redcuda_moe *layer, const float *x_dev, const float *logits_in_dev, float *out_dev, void *stream) {
    RC_REQUIRE(ep, "ep layer: null argument");
    return redcuda_ep_layer_forward_n(ep, layer, ep->tokens, x_dev, logits_in_dev, nullptr, out_dev, stream);
}

const uint32_t *redcuda_ep_last_ids_device(const redcuda_ep *ep) { return ep ? ep->ids : nullptr; }

int redcuda_ep_step(redcuda_ep *ep, redcuda_moe *const *layers, uint32_t n_layers, const float *const *x_dev, const float *const *logits_in_dev, float *const *out_dev, void *stream) {
    RC_REQUIRE(ep && layers && n_layers && x_dev && out_dev, "ep step: null or empty argument");
    for (uint32_t l = 0; l < n_layers; ++l)
        if (!redcuda_ep_layer_forward(ep, layers[l], x_dev[l], logits_in_dev ? logits_in_dev[l] : nullptr, out_dev[l], stream)) return 0;
    return 1;
}

}  // extern "C"
