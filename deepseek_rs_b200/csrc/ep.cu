// Expert-parallel execution of the routed-expert step behind the C ABI.
//
// The reference is single-GPU (one context, one stream: engine/src/engine.rs:73-74); sharding is new here and is
// defined by "same result as one GPU". Rank r of G owns experts [r * E / G, (r + 1) * E / G) and routes its own tokens
// with the same router kernel as the single-GPU call, so routing is bit-identical. One exchange each way:
//   dispatch  every (token, slot) pair goes to the rank that owns its expert, as the token's Q8_K row (4672 B instead
//             of 16 KB of f32) plus its expert id local to the owner and its router weight;
//   combine   the owner returns the pair's down-projection row (f32 [n_embd]); the source sums a token's k rows in
//             slot order straight from the receive buffer, so the result does not depend on arrival order.
//             By default the combine is FUSED into the owner's down-projection kernel: every rank maps the others'
//             receive buffers (CUDA IPC, exchanged once at set-up) and the grouped GEMM's epilogue stores each finished
//             row straight into its source rank's buffer with plain global stores over NVLink, so the rows travel while
//             the GEMM is still running and no separate transfer follows it. A four-byte all-gather after the kernel is
//             the only synchronisation: when it completes on a rank, every peer's GEMM (which precedes the peer's
//             all-gather in stream order) has finished writing. No TMA and no multicast is involved.
//             DSMOE_EP_NO_P2P=1, or a failed IPC mapping, falls back to grouped ncclSend / ncclRecv of the rows.
// Experts named by dsmoe_ep_set_replicas are held by every rank: their pairs stay on the rank that routed them.
//
// Everything between the router and the slot sum is device work on the caller's stream: the pairs are counted and
// placed by destination rank with the same stable counting sort as the batched single-GPU path, the rows are gathered
// by a kernel, and NCCL moves them (grouped ncclSend / ncclRecv over NVLink). The only host synchronisation of a step
// is the read of the G x G count matrix that sizes the transfers; every rank sees the whole matrix, so a receive
// buffer that would overflow is reported by all ranks alike and no rank is left waiting in a collective.
//
// NCCL is reached through dlsym on the libnccl.so.2 that is already loaded in the process (the one torch brings, when
// the host is Python), so the library never links a second NCCL beside it.
#include <dlfcn.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <vector>

#include "common.cuh"
#include "ep.h"
#include "launch.h"

namespace dsmoe {

// ---- NCCL entry points, resolved at run time -------------------------------------------------------------------
typedef struct { char internal[128]; } nccl_unique_id;  // ncclUniqueId
typedef void *nccl_comm;                                 // ncclComm_t
enum { NCCL_UINT8 = 1, NCCL_INT32 = 2 };                 // ncclDataType_t values used here
struct NcclApi {
    int (*GetUniqueId)(nccl_unique_id *);
    int (*CommInitRank)(nccl_comm *, int, nccl_unique_id, int);
    int (*CommDestroy)(nccl_comm);
    int (*AllGather)(const void *, void *, size_t, int, nccl_comm, cudaStream_t);
    int (*Send)(const void *, size_t, int, int, nccl_comm, cudaStream_t);
    int (*Recv)(void *, size_t, int, int, nccl_comm, cudaStream_t);
    int (*GroupStart)();
    int (*GroupEnd)();
    const char *(*GetErrorString)(int);
    bool ok = false;
};

static const NcclApi *nccl_api()
{
    static NcclApi api;
    static bool looked = false;
    if (looked) return api.ok ? &api : nullptr;
    looked = true;
    void *lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_NOLOAD);  // the copy the process already has, if any
    if (!lib) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!lib) return nullptr;
#define DSMOE_NCCL_SYM(field, name)                                         \
    *reinterpret_cast<void **>(&api.field) = dlsym(lib, name);              \
    if (!api.field) return nullptr;
    DSMOE_NCCL_SYM(GetUniqueId, "ncclGetUniqueId")
    DSMOE_NCCL_SYM(CommInitRank, "ncclCommInitRank")
    DSMOE_NCCL_SYM(CommDestroy, "ncclCommDestroy")
    DSMOE_NCCL_SYM(AllGather, "ncclAllGather")
    DSMOE_NCCL_SYM(Send, "ncclSend")
    DSMOE_NCCL_SYM(Recv, "ncclRecv")
    DSMOE_NCCL_SYM(GroupStart, "ncclGroupStart")
    DSMOE_NCCL_SYM(GroupEnd, "ncclGroupEnd")
    DSMOE_NCCL_SYM(GetErrorString, "ncclGetErrorString")
#undef DSMOE_NCCL_SYM
    api.ok = true;
    return &api;
}

// ---- device side: destination of a pair, counts, stable placement, row gather -------------------------------------
struct EpRoute {
    const int32_t *selected;      // [n_pairs] global expert ids (negative -> expert 0, engine/src/kernels/moe.rs:645-648)
    const int32_t *replica_slot;  // [n_expert]: -1, or the position of the expert in the replica list
    uint32_t n_pairs, per_rank, rank, world;
};

__device__ __forceinline__ void ep_route(const EpRoute &r, uint32_t p, uint32_t *dest, int32_t *local)
{
    int32_t e = r.selected[p];
    if (e < 0) e = 0;
    const int32_t rs = r.replica_slot[e];
    if (rs >= 0) {
        *dest = r.rank;
        *local = (int32_t)r.per_rank + rs;
    } else {
        *dest = (uint32_t)e / r.per_rank;
        *local = e % (int32_t)r.per_rank;
    }
}

// counts[d] = pairs this rank sends to rank d (one CTA per destination). CTA 0 also adds the step's selections to
// the running per-expert histogram from which a host may choose the experts to replicate.
__global__ void __launch_bounds__(256) ep_count_kernel(EpRoute r, int32_t *__restrict__ counts,
                                                        unsigned long long *__restrict__ hist)
{
    __shared__ uint32_t s_warp[8];
    const uint32_t d = blockIdx.x;
    uint32_t c = 0;
    for (uint32_t p = threadIdx.x; p < r.n_pairs; p += 256) {
        uint32_t dest;
        int32_t local;
        ep_route(r, p, &dest, &local);
        c += dest == d;
        if (d == 0 && hist) {
            const int32_t e = r.selected[p];
            atomicAdd(&hist[e < 0 ? 0 : e], 1ull);
        }
    }
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) c += __shfl_xor_sync(FULL, c, m);
    if ((threadIdx.x & 31) == 0) s_warp[threadIdx.x >> 5] = c;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t t = 0;
        for (int w = 0; w < 8; ++w) t += s_warp[w];
        counts[d] = (int32_t)t;
    }
}

// pos[p] = position of pair p in send order (grouped by destination, ascending pair id inside a group), order = its
// inverse. One CTA per destination; same two-pass ballot placement as the batched path's pair grouping.
__global__ void __launch_bounds__(256) ep_place_kernel(EpRoute r, const int32_t *__restrict__ counts,
                                                        int32_t *__restrict__ pos, uint32_t *__restrict__ order)
{
    __shared__ uint32_t s_warp[8];
    const uint32_t d = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t seg = ((r.n_pairs + 7) / 8 + 31) & ~31u, p_lo = min(r.n_pairs, warp * seg), p_hi = min(r.n_pairs, p_lo + seg);
    auto hit_at = [&](uint32_t p) {
        if (p >= p_hi) return false;
        uint32_t dest;
        int32_t local;
        ep_route(r, p, &dest, &local);
        return dest == d;
    };
    uint32_t cnt = 0;
    for (uint32_t p0 = p_lo; p0 < p_hi; p0 += 32) cnt += __popc(__ballot_sync(FULL, hit_at(p0 + lane)));
    if (lane == 0) s_warp[warp] = cnt;
    __syncthreads();
    uint32_t base = 0;
    for (uint32_t i = 0; i < d; ++i) base += (uint32_t)counts[i];
    for (uint32_t w = 0; w < warp; ++w) base += s_warp[w];
    for (uint32_t p0 = p_lo; p0 < p_hi; p0 += 32) {
        const uint32_t p = p0 + lane;
        const bool hit = hit_at(p);
        const uint32_t ballot = __ballot_sync(FULL, hit);
        if (hit) {
            const uint32_t at = base + __popc(ballot & ((1u << lane) - 1u));
            pos[p] = (int32_t)at;
            order[at] = p;
        }
        base += __popc(ballot);
    }
}

// send buffers in send order: the pair's token row of Q8_K blocks (16-byte pieces), its owner-local expert id and its
// router weight. One warp per row.
__global__ void __launch_bounds__(256) ep_gather_kernel(EpRoute r, const uint32_t *__restrict__ order,
                                                         const uint8_t *__restrict__ xq, const float *__restrict__ weights,
                                                         uint32_t k, uint32_t row_bytes, uint8_t *__restrict__ send_xq,
                                                         int32_t *__restrict__ send_sel, float *__restrict__ send_w)
{
    const uint32_t lane = threadIdx.x & 31, i = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (i >= r.n_pairs) return;
    const uint32_t p = order[i];
    const uint4 *src = reinterpret_cast<const uint4 *>(xq + (size_t)(p / k) * row_bytes);
    uint4 *dst = reinterpret_cast<uint4 *>(send_xq + (size_t)i * row_bytes);
    for (uint32_t j = lane; j < row_bytes / 16; j += 32) dst[j] = src[j];
    if (lane == 0) {
        uint32_t dest;
        int32_t local;
        ep_route(r, p, &dest, &local);
        send_sel[i] = local;
        send_w[i] = weights[p];
    }
}

// The same gather with the rows stored straight into the receive buffers of their destination ranks (peer-mapped;
// plain stores over NVLink, never loads): send_end[d] = end of destination d's segment in send order, recv_base[d] =
// first slot of this rank's segment in rank d's receive buffers. One warp per row.
struct EpPeerDst {
    uint8_t *xq[16];
    int32_t *sel[16];
    float *w[16];
    uint32_t send_end[16], recv_base[16];
    uint32_t world;
};
__global__ void __launch_bounds__(256) ep_gather_p2p_kernel(EpRoute r, const uint32_t *__restrict__ order,
                                                             const uint8_t *__restrict__ xq, const float *__restrict__ weights,
                                                             uint32_t k, uint32_t row_bytes, EpPeerDst dst)
{
    const uint32_t lane = threadIdx.x & 31, i = blockIdx.x * 8 + (threadIdx.x >> 5);
    if (i >= r.n_pairs) return;
    uint32_t d = 0, begin = 0;
    while (d + 1 < dst.world && i >= dst.send_end[d]) begin = dst.send_end[d], ++d;
    const size_t slot = (size_t)dst.recv_base[d] + (i - begin);
    const uint32_t p = order[i];
    const uint4 *src = reinterpret_cast<const uint4 *>(xq + (size_t)(p / k) * row_bytes);
    uint4 *out = reinterpret_cast<uint4 *>(dst.xq[d] + slot * row_bytes);
    for (uint32_t j = lane; j < row_bytes / 16; j += 32) out[j] = src[j];
    if (lane == 0) {
        uint32_t dest;
        int32_t local;
        ep_route(r, p, &dest, &local);
        dst.sel[d][slot] = local;
        dst.w[d][slot] = weights[p];
    }
}

// row_ptr[i] for received row i: where its result goes in the buffer of the rank it came from. seg_end[s] = end of
// the rows received from rank s, dst_base[s] = first slot of this rank's segment in rank s's send order.
struct EpRowMap {
    float *peer_back[16];
    uint32_t seg_end[16], dst_base[16];
    uint32_t world, n_embd;
};
__global__ void __launch_bounds__(256) ep_row_ptr_kernel(EpRowMap m, uint32_t n_rows, float **__restrict__ row_ptr)
{
    const uint32_t i = blockIdx.x * 256 + threadIdx.x;
    if (i >= n_rows) return;
    uint32_t s = 0, begin = 0;
    while (s + 1 < m.world && i >= m.seg_end[s]) begin = m.seg_end[s], ++s;
    row_ptr[i] = m.peer_back[s] + (size_t)(m.dst_base[s] + (i - begin)) * m.n_embd;
}

// expert_ffn of the owner-side handle with per-row destinations (api.cu; not part of the C ABI)
}  // namespace dsmoe
extern "C" int dsmoe_expert_ffn_rows(dsmoe_handle *h, cudaStream_t st, uint32_t layer, const uint8_t *xq, const int32_t *selected,
                          const float *weights, uint32_t n_tokens, float *out, float *const *row_ptr);
namespace dsmoe {

// ---- host side ----------------------------------------------------------------------------------------------------
struct EpState {
    const NcclApi *nccl = nullptr;
    nccl_comm comm = nullptr;
    bool own_comm = false;
    int rank = 0, world = 1;
    uint32_t per_rank = 0, max_replicas = 0, recv_cap = 0, max_pairs = 0, row_bytes = 0;
    dsmoe_handle *owner = nullptr;  // n_expert = per_rank + max_replicas, n_expert_used = 1: runs the received rows
    // device
    int32_t *replica_slot = nullptr, *send_counts = nullptr, *count_matrix = nullptr, *pos = nullptr, *send_sel = nullptr,
            *recv_sel = nullptr;
    uint32_t *order = nullptr;
    unsigned long long *hist = nullptr;
    uint8_t *send_xq = nullptr, *recv_xq = nullptr;
    float *send_w = nullptr, *recv_w = nullptr, *rows = nullptr, *back = nullptr;
    // fused combine: the peers' `back` buffers mapped into this process, and per received row its destination
    bool p2p = false;
    float *peer_back[16] = {};
    // fused dispatch: recv_xq, recv_sel and recv_w are carved out of one allocation (recv_blob) whose peers' copies are
    // mapped here, so that the gather kernel stores every row where its owner will read it
    uint8_t *recv_blob = nullptr, *peer_blob[16] = {};
    size_t blob_sel_off = 0, blob_w_off = 0;
    float **row_ptr = nullptr;
    int32_t *token = nullptr;  // [1 + world] ints for the completion all-gather
    // pinned host
    int32_t *h_matrix = nullptr;
    std::vector<int32_t> last_recv;  // rows received from each rank in the most recent step
    char err[384] = {0};
};

static int ep_fail(EpState *s, int code, const char *fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(s->err, sizeof(s->err), fmt, ap);
    va_end(ap);
    return code;
}

const char *ep_last_error(const EpState *s) { return s ? s->err : ""; }

void ep_destroy(EpState *s)
{
    if (!s) return;
    for (int i = 0; i < s->world && i < 16; ++i)
        if (s->p2p && i != s->rank) {
            if (s->peer_back[i]) cudaIpcCloseMemHandle(s->peer_back[i]);
            if (s->peer_blob[i]) cudaIpcCloseMemHandle(s->peer_blob[i]);
        }
    if (s->comm && s->own_comm && s->nccl) s->nccl->CommDestroy(s->comm);
    cudaFree(s->row_ptr), cudaFree(s->token);
    if (s->owner) dsmoe_destroy(s->owner);
    cudaFree(s->replica_slot), cudaFree(s->send_counts), cudaFree(s->count_matrix), cudaFree(s->pos), cudaFree(s->send_sel);
    cudaFree(s->order), cudaFree(s->hist), cudaFree(s->send_xq), cudaFree(s->recv_blob);
    cudaFree(s->send_w), cudaFree(s->rows), cudaFree(s->back);
    if (s->h_matrix) cudaFreeHost(s->h_matrix);
    delete s;
}

int ep_get_unique_id(uint8_t *id128)
{
    const NcclApi *api = nccl_api();
    if (!api) return DSMOE_ERR_NCCL;
    nccl_unique_id id;
    if (api->GetUniqueId(&id) != 0) return DSMOE_ERR_NCCL;
    memcpy(id128, id.internal, 128);
    return DSMOE_OK;
}

int ep_create(const dsmoe_config &cfg, int device, const uint8_t *id128, void *adopt_comm, int rank, int world,
              uint32_t max_replicas, uint32_t recv_capacity_rows, EpState **out, char *err, size_t err_len)
{
    auto fail_early = [&](int code, const char *msg) {
        snprintf(err, err_len, "%s", msg);
        return code;
    };
    *out = nullptr;
    if (world < 1 || rank < 0 || rank >= world || cfg.n_expert % (uint32_t)world) return fail_early(DSMOE_ERR_ARG, "ep_init: bad rank / world, or the experts do not divide evenly over the ranks");
    const uint32_t per = cfg.n_expert / (uint32_t)world;
    if ((per + max_replicas) % 32 || per + max_replicas > 512) return fail_early(DSMOE_ERR_ARG, "ep_init: experts per rank + replicas must be a multiple of 32, at most 512");
    const NcclApi *api = nccl_api();
    if (!api) return fail_early(DSMOE_ERR_NCCL, "ep_init: libnccl.so.2 could not be loaded");
    EpState *s = new (std::nothrow) EpState();
    if (!s) return fail_early(DSMOE_ERR_NOMEM, "ep_init: out of host memory");
    s->nccl = api, s->rank = rank, s->world = world, s->per_rank = per, s->max_replicas = max_replicas;
    s->max_pairs = cfg.max_tokens * cfg.n_expert_used;
    s->recv_cap = recv_capacity_rows ? recv_capacity_rows : 2u * s->max_pairs;
    s->row_bytes = cfg.n_embd / QK_K * Q8K_BYTES;
    if (s->row_bytes % 16) {
        delete s;
        return fail_early(DSMOE_ERR_ARG, "ep_init: the Q8_K row of a token must be a multiple of 16 bytes (n_embd a multiple of 1024)");
    }
    if (adopt_comm) {
        s->comm = adopt_comm;
    } else {
        nccl_unique_id id;
        memcpy(id.internal, id128, 128);
        const int rc = api->CommInitRank(&s->comm, world, id, rank);
        if (rc != 0) {
            snprintf(err, err_len, "ep_init: ncclCommInitRank: %s", api->GetErrorString(rc));
            delete s;
            return DSMOE_ERR_NCCL;
        }
        s->own_comm = true;
    }
    dsmoe_config oc = cfg;
    oc.n_expert = per + max_replicas, oc.n_expert_used = 1, oc.max_tokens = s->recv_cap;
    if (int rc = dsmoe_create(&oc, device, &s->owner)) {
        ep_destroy(s);
        return fail_early(rc, "ep_init: could not create the owner-side handle (receive capacity too large for the device?)");
    }
    const size_t P = s->max_pairs ? s->max_pairs : 1, C = s->recv_cap, W = (size_t)world;
    bool ok = true;
    auto alloc = [&](auto **p, size_t n) { ok = ok && cudaMalloc((void **)p, n * sizeof(**p)) == cudaSuccess; };
    alloc(&s->replica_slot, cfg.n_expert), alloc(&s->send_counts, W), alloc(&s->count_matrix, W * W), alloc(&s->pos, P);
    alloc(&s->order, P), alloc(&s->hist, cfg.n_expert), alloc(&s->send_sel, P);
    alloc(&s->send_xq, P * s->row_bytes), alloc(&s->send_w, P);
    s->blob_sel_off = (C * s->row_bytes + 255) & ~(size_t)255;
    s->blob_w_off = (s->blob_sel_off + C * sizeof(int32_t) + 255) & ~(size_t)255;
    alloc(&s->recv_blob, s->blob_w_off + C * sizeof(float));
    if (ok) {
        s->recv_xq = s->recv_blob;
        s->recv_sel = reinterpret_cast<int32_t *>(s->recv_blob + s->blob_sel_off);
        s->recv_w = reinterpret_cast<float *>(s->recv_blob + s->blob_w_off);
    }
    alloc(&s->rows, C * cfg.n_embd), alloc(&s->back, P * cfg.n_embd);
    ok = ok && cudaMallocHost((void **)&s->h_matrix, W * W * sizeof(int32_t)) == cudaSuccess;
    ok = ok && cudaMemset(s->replica_slot, 0xFF, cfg.n_expert * sizeof(int32_t)) == cudaSuccess;
    ok = ok && cudaMemset(s->hist, 0, cfg.n_expert * sizeof(unsigned long long)) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        ep_destroy(s);
        return fail_early(DSMOE_ERR_NOMEM, "ep_init: device allocation failed");
    }
    s->last_recv.assign(W, 0);
    // Fused combine: exchange CUDA IPC handles of the `back` buffers through the communicator and map the peers'. Any
    // failure leaves p2p off on EVERY rank (the decision is agreed through a second all-gather), and the combine then
    // goes through NCCL.
    {
        const char *no_p2p = getenv("DSMOE_EP_NO_P2P");
        int want = world <= 16 && !(no_p2p && no_p2p[0] == '1') ? 1 : 0;
        uint8_t *d_handles = nullptr;
        int32_t *d_flags = nullptr;
        ok = cudaMalloc((void **)&s->row_ptr, C * sizeof(float *)) == cudaSuccess &&
             cudaMalloc((void **)&s->token, (1 + W) * sizeof(int32_t)) == cudaSuccess &&
             cudaMemset(s->token, 0, (1 + W) * sizeof(int32_t)) == cudaSuccess &&
             cudaMalloc((void **)&d_handles, (W + 1) * sizeof(cudaIpcMemHandle_t)) == cudaSuccess &&
             cudaMalloc((void **)&d_flags, (W + 1) * sizeof(int32_t)) == cudaSuccess;
        // one round per exported buffer: all-gather its handle, open the peers'
        auto exchange = [&](void *mine_ptr, void **peers) {
            std::vector<cudaIpcMemHandle_t> handles(W);
            cudaIpcMemHandle_t mine;
            memset(&mine, 0, sizeof(mine));
            if (ok && want && cudaIpcGetMemHandle(&mine, mine_ptr) != cudaSuccess) want = 0;
            cudaGetLastError();
            if (ok) {
                ok = cudaMemcpy(d_handles + W * sizeof(mine), &mine, sizeof(mine), cudaMemcpyHostToDevice) == cudaSuccess &&
                     api->AllGather(d_handles + W * sizeof(mine), d_handles, sizeof(mine), NCCL_UINT8, s->comm, nullptr) == 0 &&
                     cudaStreamSynchronize(nullptr) == cudaSuccess &&
                     cudaMemcpy(handles.data(), d_handles, W * sizeof(mine), cudaMemcpyDeviceToHost) == cudaSuccess;
            }
            if (ok && want) {
                for (int i = 0; i < world; ++i) {
                    if (i == rank) {
                        peers[i] = mine_ptr;
                    } else if (cudaIpcOpenMemHandle(&peers[i], handles[(size_t)i], cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                        cudaGetLastError();
                        peers[i] = nullptr;
                        want = 0;
                    }
                }
            }
        };
        exchange(s->back, reinterpret_cast<void **>(s->peer_back));
        exchange(s->recv_blob, reinterpret_cast<void **>(s->peer_blob));
        std::vector<int32_t> flags(W, 0);
        if (ok) {
            ok = cudaMemcpy(d_flags + W, &want, sizeof(int32_t), cudaMemcpyHostToDevice) == cudaSuccess &&
                 api->AllGather(d_flags + W, d_flags, 1, NCCL_INT32, s->comm, nullptr) == 0 &&
                 cudaStreamSynchronize(nullptr) == cudaSuccess &&
                 cudaMemcpy(flags.data(), d_flags, W * sizeof(int32_t), cudaMemcpyDeviceToHost) == cudaSuccess;
        }
        cudaFree(d_handles), cudaFree(d_flags);
        if (!ok) {
            cudaGetLastError();
            ep_destroy(s);
            return fail_early(DSMOE_ERR_CUDA, "ep_init: exchange of the peer-buffer handles failed");
        }
        bool all = want != 0;
        for (size_t i = 0; i < W; ++i) all = all && flags[i] != 0;
        if (!all)
            for (int i = 0; i < world; ++i)
                if (i != rank) {
                    if (s->peer_back[i]) cudaIpcCloseMemHandle(s->peer_back[i]), s->peer_back[i] = nullptr;
                    if (s->peer_blob[i]) cudaIpcCloseMemHandle(s->peer_blob[i]), s->peer_blob[i] = nullptr;
                }
        s->p2p = all;
    }
    *out = s;
    return DSMOE_OK;
}

dsmoe_handle *ep_owner(EpState *s) { return s->owner; }
int ep_rank(const EpState *s) { return s->rank; }
int ep_world(const EpState *s) { return s->world; }
int ep_p2p_combine(const EpState *s) { return s->p2p ? 1 : 0; }

int ep_set_replicas(EpState *s, uint32_t n_expert, const int32_t *ids, uint32_t n)
{
    if (n > s->max_replicas) return ep_fail(s, DSMOE_ERR_BOUNDS, "ep_set_replicas: %u replicas, the handle was initialised for %u", n, s->max_replicas);
    std::vector<int32_t> slot(n_expert, -1);
    for (uint32_t i = 0; i < n; ++i) {
        if (ids[i] < 0 || (uint32_t)ids[i] >= n_expert || slot[ids[i]] >= 0) return ep_fail(s, DSMOE_ERR_ARG, "ep_set_replicas: bad or repeated expert id %d", ids[i]);
        slot[ids[i]] = (int32_t)i;
    }
    if (cudaDeviceSynchronize() != cudaSuccess ||
        cudaMemcpy(s->replica_slot, slot.data(), n_expert * sizeof(int32_t), cudaMemcpyHostToDevice) != cudaSuccess)
        return ep_fail(s, DSMOE_ERR_CUDA, "ep_set_replicas: %s", cudaGetErrorString(cudaGetLastError()));
    return DSMOE_OK;
}

int ep_expert_counts(EpState *s, cudaStream_t st, uint32_t n_expert, uint64_t *host_out, int reset)
{
    cudaError_t e = cudaMemcpyAsync(host_out, s->hist, n_expert * sizeof(uint64_t), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess && reset) e = cudaMemsetAsync(s->hist, 0, n_expert * sizeof(uint64_t), st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    return e == cudaSuccess ? DSMOE_OK : ep_fail(s, DSMOE_ERR_CUDA, "ep_expert_counts: %s", cudaGetErrorString(e));
}

int ep_last_recv_rows(const EpState *s, int32_t *per_rank_out)
{
    for (int i = 0; i < s->world; ++i) per_rank_out[i] = s->last_recv[(size_t)i];
    return DSMOE_OK;
}

#define EP_NCCL(call, what)                                                                        \
    do {                                                                                           \
        const int rc_ = (call);                                                                    \
        if (rc_ != 0) return ep_fail(s, DSMOE_ERR_NCCL, "%s: %s", what, s->nccl->GetErrorString(rc_)); \
    } while (0)
#define EP_CUDA(call, what)                                                                        \
    do {                                                                                           \
        const cudaError_t e_ = (call);                                                             \
        if (e_ != cudaSuccess) return ep_fail(s, DSMOE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e_)); \
    } while (0)

// Dispatch, owner compute, combine and slot sum for rows that are already routed and quantised on this rank.
// selected / weights: [n_tokens][k]; xq: Q8_K rows [n_tokens]; out: [n_tokens][n_embd]. Collective: every rank calls it.
int ep_forward(EpState *s, cudaStream_t st, uint32_t layer, const uint8_t *xq, const int32_t *selected, const float *weights,
               uint32_t n_tokens, uint32_t k, uint32_t n_embd, float *out, int *n_launched, cudaEvent_t *marks)
{
    const uint32_t P = n_tokens * k, W = (uint32_t)s->world;
    if (P > s->max_pairs) return ep_fail(s, DSMOE_ERR_BOUNDS, "moe_forward_ep: %u pairs, the handle was created for %u", P, s->max_pairs);
    auto mark = [&](int i) {
        if (marks) cudaEventRecord(marks[i], st);
    };
    const EpRoute r = {selected, s->replica_slot, P, s->per_rank, (uint32_t)s->rank, W};
    mark(0);
    // 1. counts by destination, gathered from every rank; placement and row gather run while the matrix travels
    ep_count_kernel<<<W, 256, 0, st>>>(r, s->send_counts, s->hist);
    EP_NCCL(s->nccl->AllGather(s->send_counts, s->count_matrix, W, NCCL_INT32, s->comm, st), "count exchange");
    EP_CUDA(cudaMemcpyAsync(s->h_matrix, s->count_matrix, (size_t)W * W * sizeof(int32_t), cudaMemcpyDeviceToHost, st), "count read");
    if (P) {
        ep_place_kernel<<<W, 256, 0, st>>>(r, s->send_counts, s->pos, s->order);
        if (!s->p2p)
            ep_gather_kernel<<<(P + 7) / 8, 256, 0, st>>>(r, s->order, xq, weights, k, s->row_bytes, s->send_xq, s->send_sel, s->send_w);
    }
    EP_CUDA(cudaGetLastError(), "plan launch");
    *n_launched += P ? (s->p2p ? 2 : 3) : 1;
    EP_CUDA(cudaStreamSynchronize(st), "count read");
    mark(1);
    // 2. sizes; every rank evaluates every rank's receive total, so an overflow is reported by all of them alike
    const int32_t *M = s->h_matrix;  // M[src * W + dst]
    for (uint32_t d = 0; d < W; ++d) {
        uint64_t total = 0;
        for (uint32_t src = 0; src < W; ++src) total += (uint32_t)M[src * W + d];
        if (total > s->recv_cap)
            return ep_fail(s, DSMOE_ERR_BOUNDS, "moe_forward_ep: rank %u would receive %llu rows, its buffer holds %u (raise recv_capacity_rows or replicate the hot experts)",
                           d, (unsigned long long)total, s->recv_cap);
    }
    std::vector<size_t> soff(W + 1, 0), roff(W + 1, 0);
    for (uint32_t i = 0; i < W; ++i) {
        soff[i + 1] = soff[i] + (uint32_t)M[(uint32_t)s->rank * W + i];
        roff[i + 1] = roff[i] + (uint32_t)M[i * W + (uint32_t)s->rank];
        s->last_recv[i] = M[i * W + (uint32_t)s->rank];
    }
    const size_t R = roff[W];
    // 3. dispatch
    if (s->p2p) {
        // fused with the gather: every row is stored where its owner reads it. A rank's completion all-gather follows
        // its gather in stream order, so when it completes here every peer has finished storing into this rank's
        // buffers. (The buffers are free: the step before ended with an all-gather that followed every rank's GEMM.)
        if (P) {
            EpPeerDst dst = {};
            dst.world = W;
            for (uint32_t d = 0; d < W; ++d) {
                dst.xq[d] = s->peer_blob[d];
                dst.sel[d] = reinterpret_cast<int32_t *>(s->peer_blob[d] + s->blob_sel_off);
                dst.w[d] = reinterpret_cast<float *>(s->peer_blob[d] + s->blob_w_off);
                dst.send_end[d] = (uint32_t)soff[d + 1];
                uint32_t base = 0;
                for (uint32_t src = 0; src < (uint32_t)s->rank; ++src) base += (uint32_t)M[src * W + d];
                dst.recv_base[d] = base;
            }
            ep_gather_p2p_kernel<<<(P + 7) / 8, 256, 0, st>>>(r, s->order, xq, weights, k, s->row_bytes, dst);
            EP_CUDA(cudaGetLastError(), "dispatch launch");
            *n_launched += 1;
        }
        EP_NCCL(s->nccl->AllGather(s->token, s->token + 1, 1, NCCL_INT32, s->comm, st), "dispatch completion");
    } else {
    EP_NCCL(s->nccl->GroupStart(), "dispatch");
    for (uint32_t peer = 0; peer < W; ++peer) {
        const size_t sc = soff[peer + 1] - soff[peer], rc = roff[peer + 1] - roff[peer];
        if (sc) {
            EP_NCCL(s->nccl->Send(s->send_xq + soff[peer] * s->row_bytes, sc * s->row_bytes, NCCL_UINT8, (int)peer, s->comm, st), "dispatch send");
            EP_NCCL(s->nccl->Send(s->send_sel + soff[peer], sc, NCCL_INT32, (int)peer, s->comm, st), "dispatch send");
            EP_NCCL(s->nccl->Send(s->send_w + soff[peer], sc * 4, NCCL_UINT8, (int)peer, s->comm, st), "dispatch send");
        }
        if (rc) {
            EP_NCCL(s->nccl->Recv(s->recv_xq + roff[peer] * s->row_bytes, rc * s->row_bytes, NCCL_UINT8, (int)peer, s->comm, st), "dispatch recv");
            EP_NCCL(s->nccl->Recv(s->recv_sel + roff[peer], rc, NCCL_INT32, (int)peer, s->comm, st), "dispatch recv");
            EP_NCCL(s->nccl->Recv(s->recv_w + roff[peer], rc * 4, NCCL_UINT8, (int)peer, s->comm, st), "dispatch recv");
        }
    }
    EP_NCCL(s->nccl->GroupEnd(), "dispatch");
    }
    mark(2);
    // 4. the owner's compute: every received row is one (token, slot) pair of one local expert
    if (R && s->p2p) {
        // fused combine: the down projection's epilogue stores every row where its source rank will sum it
        EpRowMap m = {};
        m.world = W, m.n_embd = n_embd;
        for (uint32_t src = 0; src < W; ++src) {
            m.peer_back[src] = s->peer_back[src];
            m.seg_end[src] = (uint32_t)roff[src + 1];
            uint32_t base = 0;
            for (uint32_t d = 0; d < (uint32_t)s->rank; ++d) base += (uint32_t)M[src * W + d];
            m.dst_base[src] = base;
        }
        ep_row_ptr_kernel<<<((uint32_t)R + 255) / 256, 256, 0, st>>>(m, (uint32_t)R, s->row_ptr);
        const uint64_t before = dsmoe_launch_count(s->owner);
        const int rc = dsmoe_expert_ffn_rows(s->owner, st, layer, s->recv_xq, s->recv_sel, s->recv_w, (uint32_t)R, s->rows, s->row_ptr);
        if (rc != DSMOE_OK) return ep_fail(s, rc, "moe_forward_ep: owner compute: %s", dsmoe_last_error(s->owner));
        *n_launched += 1 + (int)(dsmoe_launch_count(s->owner) - before);
    } else if (R) {
        const uint64_t before = dsmoe_launch_count(s->owner);
        const int rc = dsmoe_expert_ffn(s->owner, st, layer, s->recv_xq, s->recv_sel, s->recv_w, (uint32_t)R, s->rows);
        if (rc != DSMOE_OK) return ep_fail(s, rc, "moe_forward_ep: owner compute: %s", dsmoe_last_error(s->owner));
        *n_launched += (int)(dsmoe_launch_count(s->owner) - before);
    }
    mark(3);
    if (s->p2p) {
        // completion: a rank's all-gather follows its GEMM in stream order, so when this one completes here every peer
        // has finished storing into this rank's buffer
        EP_NCCL(s->nccl->AllGather(s->token, s->token + 1, 1, NCCL_INT32, s->comm, st), "combine completion");
        mark(4);
        if (P) {
            launch_moe_sum(st, s->back, s->pos, out, n_embd, k, n_tokens);
            EP_CUDA(cudaGetLastError(), "slot sum");
            *n_launched += 1;
        }
        mark(5);
        return DSMOE_OK;
    }
    // 5. combine: the rows travel back along the same splits and land in send order
    EP_NCCL(s->nccl->GroupStart(), "combine");
    for (uint32_t peer = 0; peer < W; ++peer) {
        const size_t sc = soff[peer + 1] - soff[peer], rc = roff[peer + 1] - roff[peer];
        if (rc) EP_NCCL(s->nccl->Send(s->rows + roff[peer] * n_embd, rc * n_embd * 4, NCCL_UINT8, (int)peer, s->comm, st), "combine send");
        if (sc) EP_NCCL(s->nccl->Recv(s->back + soff[peer] * n_embd, sc * n_embd * 4, NCCL_UINT8, (int)peer, s->comm, st), "combine recv");
    }
    EP_NCCL(s->nccl->GroupEnd(), "combine");
    mark(4);
    // 6. slots summed in slot order, each row read where it landed
    if (P) {
        launch_moe_sum(st, s->back, s->pos, out, n_embd, k, n_tokens);
        EP_CUDA(cudaGetLastError(), "slot sum");
        *n_launched += 1;
    }
    mark(5);
    return DSMOE_OK;
}

}  // namespace dsmoe
