// Peer groups: mailbox allocation and exchange of CUDA IPC handles between the ranks of a node.
#include "common.cuh"
#include "peer.cuh"

#include <cstring>

using namespace acro_b200_detail;

struct acro_b200_peer_group
{
    int world = 0, rank = 0, device = -1;
    bool connected = false;
    unsigned long long seq = 0;
    void *own = nullptr;                           // this rank's mailbox (cudaMalloc)
    void *peer[ACRO_B200_MAX_PEERS] = {nullptr};   // mapped mailboxes (own entry = own)
};

namespace acro_b200_detail
{
PeerView next_peer_view(acro_b200_peer_group *g, int64_t exchanges)
{
    PeerView v;
    v.world = g->world;
    v.rank = g->rank;
    v.seq = g->seq + 1;
    g->seq += static_cast<unsigned long long>(exchanges < 1 ? 1 : exchanges);
    for (int p = 0; p < ACRO_B200_MAX_PEERS; ++p)
    {
        char *base = static_cast<char *>(p < g->world ? g->peer[p] : nullptr);
        v.data[p] = reinterpret_cast<double *>(base);
        v.flag[p] = base ? reinterpret_cast<unsigned long long *>(base + peer_data_doubles(g->world) * sizeof(double)) : nullptr;
    }
    return v;
}
}

namespace
{

constexpr int kAllreduceThreads = 1024;

// dst[i] (op)= sum over the ranks of src[i], i < n.  One CTA walks the entries in exchanges of at most
// kPeerSlot: it stores its own values into every rank's mailbox (plain remote stores), publishes the
// exchange's sequence number, waits (bounded, polling its own memory) for the other ranks and adds
// the world contributions in rank order, so every rank ends with the same bits.  src == dst is allowed
// (each entry is read and written by the same thread).  When a wait gives up the flag is raised and
// the remaining exchanges are skipped: the result is invalid and nothing hangs.
__global__ void __launch_bounds__(kAllreduceThreads)
peer_allreduce_kernel(double *dst, const double *src, int64_t n, int op, PeerView pv, int *wait_flag)
{
    __shared__ int gave_up;
    const int t = threadIdx.x;
    if (n <= kPeerWordEntries)
    {
        // short results travel as self-marking words, the form of the reduction kernel's fused exchange: the ranks
        // of one call may have planned different families, and the choice here depends on the result's size alone
        const double total = exchange_words(pv, t, static_cast<int>(n), t < n ? src[t] : 0.0, wait_flag);
        if (t < n)
        {
            if (op == ACRO_B200_OP_ASSIGN) dst[t] = total;
            else if (op == ACRO_B200_OP_ADD) dst[t] += total;
            else dst[t] -= total;
        }
        return;
    }
    if (t == 0) gave_up = 0;
    __syncthreads();
    for (int64_t base = 0; base < n; base += kPeerSlot, ++pv.seq)
    {
        const int len = static_cast<int>(n - base < kPeerSlot ? n - base : kPeerSlot);
        const int par = static_cast<int>(pv.seq & 1ull);
        const size_t slot = (static_cast<size_t>(par) * pv.world + pv.rank) * kPeerSlot;
        for (int i = t; i < len; i += kAllreduceThreads)
        {
            const double v = src[base + i];
            for (int p = 0; p < pv.world; ++p) pv.data[p][slot + i] = v;
        }
        __threadfence_system();     // also orders the previous exchange's mailbox reads before this publication
        __syncthreads();
        if (t < pv.world)
        {
            volatile unsigned long long *remote = pv.flag[t] + static_cast<size_t>(par) * pv.world + pv.rank;
            *remote = pv.seq;
            volatile unsigned long long *own = pv.flag[pv.rank] + static_cast<size_t>(par) * pv.world + t;
            bool arrived = false;
            for (unsigned int tries = 0; tries < (1u << 21); ++tries)   // about a second
            {
                if (*own >= pv.seq) { arrived = true; break; }
                __nanosleep(64);
            }
            if (!arrived)
            {
                atomicExch(wait_flag, 1);
                gave_up = 1;
            }
            __threadfence_system();
        }
        __syncthreads();
        if (gave_up != 0) return;
        const volatile double *box = pv.data[pv.rank] + static_cast<size_t>(par) * pv.world * kPeerSlot;
        for (int i = t; i < len; i += kAllreduceThreads)
        {
            double total = 0.0;
            for (int r = 0; r < pv.world; ++r) total += box[static_cast<size_t>(r) * kPeerSlot + i];
            if (op == ACRO_B200_OP_ASSIGN) dst[base + i] = total;
            else if (op == ACRO_B200_OP_ADD) dst[base + i] += total;
            else dst[base + i] -= total;
        }
    }
}

}

extern "C" {

int acro_b200_peer_allreduce(double *dst, const double *src, int64_t n, int op, acro_b200_peer_group *group, void *stream)
{
    if (dst == nullptr || src == nullptr || group == nullptr) return fail_invalid("acro_b200_peer_allreduce: null argument");
    if (n < 1 || op < 0 || op > 2) return fail_invalid("acro_b200_peer_allreduce: bad count or operator");
    if (!group->connected) return fail_invalid("acro_b200_peer_allreduce: the peer group is not connected");
    int *wait_flag = wait_flag_device_ptr();
    if (wait_flag == nullptr) return fail_cuda(cudaErrorUnknown, "acro_b200_peer_allreduce (status flag)");
    const int64_t exchanges = (n + kPeerSlot - 1) / kPeerSlot;
    const PeerView pv = next_peer_view(group, exchanges);
    peer_allreduce_kernel<<<1, kAllreduceThreads, 0, as_stream(stream)>>>(dst, src, n, op, pv, wait_flag);
    return launch_status("acro_b200_peer_allreduce");
}

int acro_b200_peer_group_create(int world, int rank, acro_b200_peer_group **out, unsigned char *handle_out)
{
    if (out == nullptr || handle_out == nullptr) return fail_invalid("acro_b200_peer_group_create: null argument");
    if (world < 1 || world > ACRO_B200_MAX_PEERS || rank < 0 || rank >= world) return fail_invalid("acro_b200_peer_group_create: bad world size or rank");
    static_assert(sizeof(cudaIpcMemHandle_t) <= ACRO_B200_IPC_HANDLE_BYTES, "IPC handle does not fit");
    acro_b200_peer_group *g = new acro_b200_peer_group;
    g->world = world;
    g->rank = rank;
    cudaError_t status = cudaGetDevice(&g->device);
    if (status == cudaSuccess) status = cudaMalloc(&g->own, peer_mailbox_bytes(world));
    if (status == cudaSuccess) status = cudaMemset(g->own, 0, peer_mailbox_bytes(world));
    std::memset(handle_out, 0, ACRO_B200_IPC_HANDLE_BYTES);
    if (status == cudaSuccess && world > 1)
    {
        cudaIpcMemHandle_t h;
        status = cudaIpcGetMemHandle(&h, g->own);
        if (status == cudaSuccess) std::memcpy(handle_out, &h, sizeof h);
    }
    if (status != cudaSuccess)
    {
        if (g->own) cudaFree(g->own);
        delete g;
        return fail_cuda(status, "acro_b200_peer_group_create");
    }
    g->peer[rank] = g->own;
    g->connected = (world == 1);
    *out = g;
    return ACRO_B200_OK;
}

int acro_b200_peer_group_connect(acro_b200_peer_group *g, const unsigned char *all_handles)
{
    if (g == nullptr || all_handles == nullptr) return fail_invalid("acro_b200_peer_group_connect: null argument");
    if (g->connected) return ACRO_B200_OK;
    for (int p = 0; p < g->world; ++p)
    {
        if (p == g->rank) continue;
        cudaIpcMemHandle_t h;
        std::memcpy(&h, all_handles + static_cast<size_t>(p) * ACRO_B200_IPC_HANDLE_BYTES, sizeof h);
        cudaError_t status = cudaIpcOpenMemHandle(&g->peer[p], h, cudaIpcMemLazyEnablePeerAccess);
        if (status != cudaSuccess) return fail_cuda(status, "acro_b200_peer_group_connect (cudaIpcOpenMemHandle)");
    }
    g->connected = true;
    return ACRO_B200_OK;
}

int acro_b200_peer_group_destroy(acro_b200_peer_group *g)
{
    if (g == nullptr) return ACRO_B200_OK;
    for (int p = 0; p < g->world; ++p)
    {
        if (p != g->rank && g->peer[p] != nullptr) cudaIpcCloseMemHandle(g->peer[p]);
    }
    if (g->own) cudaFree(g->own);
    delete g;
    return ACRO_B200_OK;
}

int acro_b200_peer_group_world(const acro_b200_peer_group *g) { return g ? g->world : ACRO_B200_EINVAL; }
int acro_b200_peer_group_is_connected(const acro_b200_peer_group *g) { return g ? (g->connected ? 1 : 0) : ACRO_B200_EINVAL; }

}
