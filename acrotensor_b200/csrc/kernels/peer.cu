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
PeerView next_peer_view(acro_b200_peer_group *g)
{
    PeerView v;
    v.world = g->world;
    v.rank = g->rank;
    v.seq = ++g->seq;
    for (int p = 0; p < ACRO_B200_MAX_PEERS; ++p)
    {
        char *base = static_cast<char *>(p < g->world ? g->peer[p] : nullptr);
        v.data[p] = reinterpret_cast<double *>(base);
        v.flag[p] = base ? reinterpret_cast<unsigned long long *>(base + peer_data_doubles(g->world) * sizeof(double)) : nullptr;
    }
    return v;
}
}

extern "C" {

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
