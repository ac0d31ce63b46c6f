// Shared-entry exchange for a sharded FlatIndexedSumGather.
//
// When the range of an IndexMapping (element-local entries) is cut into one slab per rank, a
// rank's sum-gather only holds the contributions of its own slab.  Entries of the domain
// (global degrees of freedom) reached from several ranks' slabs must be summed over those
// ranks.  Each rank owns an inbox in its own device memory, exported to the other ranks of the
// node (CUDA IPC, NVLink peer mappings):
//     data [2][stride]  doubles, one segment per sending rank, each listing the entries shared
//                       with that rank in ascending domain order
//     flag [2][world]   uint64 sequence number of the sender's last complete write
// send:    reads this rank's partial value of every shared entry and stores it into the inbox
//          segment of every rank sharing it (plain remote stores); the CTA that finishes last
//          publishes the call's sequence number to those ranks.
// combine: waits (bounded, polling its own memory) for the sequence numbers of the ranks it
//          shares entries with, then replaces every shared entry by the sum of all sharing
//          ranks' partial values in ascending rank order, so all of them hold identical bits.
// Two parity halves make back-to-back calls safe: a rank cannot send call k+2 before every
// neighbour has published call k+1, which each does only after it combined call k.
// No loads from peer memory, no atomics on peer memory, no multicast.
#include "common.cuh"

#include <cstring>
#include <vector>

using namespace acro_b200_detail;

namespace
{

constexpr int kThreads = 256;

struct HaloView   // passed to kernels by value
{
    int world, rank;
    unsigned int neighbours;                  // bit p: rank p shares entries with this rank
    unsigned long long seq;                   // sequence number of this call (>= 1)
    long long n_shared;
    const int *shared_idx;                    // [n_shared] domain position, ascending
    const int *entry_off;                     // [n_shared + 1] CSR over the sharing ranks of each entry
    const int *entry_peer;                    // sharing rank (ascending within an entry, never this rank)
    const int *entry_send;                    // slot in that rank's inbox half
    const int *entry_recv;                    // slot in this rank's inbox half holding that rank's value
    double *inbox[ACRO_B200_MAX_PEERS];
    unsigned long long *flag[ACRO_B200_MAX_PEERS];
    long long stride[ACRO_B200_MAX_PEERS];    // doubles per parity half of rank p's inbox
    unsigned int *ticket;
    int *wait_flag;
};

__global__ void __launch_bounds__(kThreads)
halo_send_kernel(const HaloView v, const double *__restrict__ values)
{
    __shared__ bool is_last;
    const int par = static_cast<int>(v.seq & 1ull);
    const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long k = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; k < v.n_shared; k += step)
    {
        const double x = values[v.shared_idx[k]];
        for (int e = v.entry_off[k]; e < v.entry_off[k + 1]; ++e)
        {
            const int p = v.entry_peer[e];
            v.inbox[p][par * v.stride[p] + v.entry_send[e]] = x;      // remote store over the peer mapping
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) is_last = (atomicAdd(v.ticket, 1u) == gridDim.x - 1);
    __syncthreads();
    if (!is_last) return;
    __threadfence_system();
    if (threadIdx.x < v.world && ((v.neighbours >> threadIdx.x) & 1u))
    {
        volatile unsigned long long *remote = v.flag[threadIdx.x] + static_cast<size_t>(par) * v.world + v.rank;
        *remote = v.seq;
    }
    if (threadIdx.x == 0) *v.ticket = 0u;
}

__global__ void __launch_bounds__(kThreads)
halo_combine_kernel(const HaloView v, double *__restrict__ values)
{
    const int par = static_cast<int>(v.seq & 1ull);
    if (threadIdx.x < v.world && ((v.neighbours >> threadIdx.x) & 1u))
    {
        volatile unsigned long long *own = v.flag[v.rank] + static_cast<size_t>(par) * v.world + threadIdx.x;
        bool arrived = false;
        for (unsigned int tries = 0; tries < (1u << 21); ++tries)   // about a second
        {
            if (*own >= v.seq) { arrived = true; break; }
            __nanosleep(64);
        }
        if (!arrived) atomicExch(v.wait_flag, 1);
        __threadfence_system();
    }
    __syncthreads();
    const double *box = v.inbox[v.rank] + par * v.stride[v.rank];
    const long long step = static_cast<long long>(gridDim.x) * blockDim.x;
    for (long long k = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; k < v.n_shared; k += step)
    {
        const int d = v.shared_idx[k];
        const double mine = values[d];
        double total = 0.0;
        bool placed = false;
        for (int e = v.entry_off[k]; e < v.entry_off[k + 1]; ++e)
        {
            if (!placed && v.entry_peer[e] > v.rank)
            {
                total = __dadd_rn(total, mine);
                placed = true;
            }
            total = __dadd_rn(total, __ldcg(box + v.entry_recv[e]));   // written by a peer: read at L2
        }
        if (!placed) total = __dadd_rn(total, mine);
        values[d] = total;
    }
}

inline bool bit_of(const unsigned char *bitmap, int64_t d) { return (bitmap[d >> 3] >> (d & 7)) & 1u; }

}

struct acro_b200_halo
{
    int world = 0, rank = 0, device = -1;
    int64_t domain = 0;
    bool on_device = false, connected = false, opened_by_ipc = false;
    unsigned long long seq = 0;
    unsigned int neighbours = 0;
    // the plan (host copies)
    std::vector<int> shared_idx, entry_off, entry_peer, entry_send, entry_recv;
    long long stride[ACRO_B200_MAX_PEERS] = {0};       // doubles per parity half of every rank's inbox
    // device side
    int *d_plan = nullptr;                             // the five arrays above, back to back
    unsigned int *d_ticket = nullptr;
    void *own = nullptr;
    void *peer[ACRO_B200_MAX_PEERS] = {nullptr};
};

namespace
{

size_t mailbox_bytes(const acro_b200_halo *h, int p)
{
    return 2u * static_cast<size_t>(h->stride[p]) * sizeof(double) + 2u * static_cast<size_t>(h->world) * sizeof(unsigned long long);
}

HaloView view_of(acro_b200_halo *h, bool advance)
{
    HaloView v;
    std::memset(&v, 0, sizeof v);
    v.world = h->world;
    v.rank = h->rank;
    v.neighbours = h->neighbours;
    if (advance) ++h->seq;
    v.seq = h->seq;
    v.n_shared = static_cast<long long>(h->shared_idx.size());
    const size_t ns = h->shared_idx.size(), ne = h->entry_peer.size();
    v.shared_idx = h->d_plan;
    v.entry_off = h->d_plan + ns;
    v.entry_peer = h->d_plan + ns + (ns + 1);
    v.entry_send = h->d_plan + ns + (ns + 1) + ne;
    v.entry_recv = h->d_plan + ns + (ns + 1) + 2 * ne;
    for (int p = 0; p < h->world; ++p)
    {
        char *base = static_cast<char *>(h->peer[p]);
        v.inbox[p] = reinterpret_cast<double *>(base);
        v.flag[p] = base ? reinterpret_cast<unsigned long long *>(base + 2u * static_cast<size_t>(h->stride[p]) * sizeof(double)) : nullptr;
        v.stride[p] = h->stride[p];
    }
    v.ticket = h->d_ticket;
    v.wait_flag = wait_flag_device_ptr();
    return v;
}

int grid_for(long long n)
{
    long long blocks = (n + kThreads - 1) / kThreads;
    const long long cap = static_cast<long long>(sm_count() > 0 ? sm_count() : 1) * 8;
    if (blocks > cap) blocks = cap;
    return static_cast<int>(blocks > 0 ? blocks : 1);
}

int check_ready(const acro_b200_halo *h, const double *values, const char *who)
{
    if (h == nullptr || values == nullptr) return fail_invalid(std::string(who) + ": null argument");
    if (!h->on_device) return fail_invalid(std::string(who) + ": this exchange was created as a host-side plan only");
    if (!h->connected) return fail_invalid(std::string(who) + ": the ranks' inboxes are not connected yet");
    return ACRO_B200_OK;
}

}

extern "C" {

int acro_b200_halo_mark_touched(const int *map, int64_t range_size, int64_t domain_size, unsigned char *bitmap)
{
    if (map == nullptr || bitmap == nullptr || range_size < 0 || domain_size < 1) return fail_invalid("acro_b200_halo_mark_touched: bad arguments");
    std::memset(bitmap, 0, static_cast<size_t>((domain_size + 7) / 8));
    for (int64_t i = 0; i < range_size; ++i)
    {
        const int64_t d = map[i];
        if (d < 0 || d >= domain_size) return fail_invalid("acro_b200_halo_mark_touched: map value outside the domain");
        bitmap[d >> 3] = static_cast<unsigned char>(bitmap[d >> 3] | (1u << (d & 7)));
    }
    return ACRO_B200_OK;
}

int acro_b200_halo_create(int world, int rank, int64_t domain_size, const unsigned char *all_bitmaps, int on_device,
                          acro_b200_halo **out, unsigned char *handle_out)
{
    if (out == nullptr || all_bitmaps == nullptr) return fail_invalid("acro_b200_halo_create: null argument");
    if (world < 1 || world > ACRO_B200_MAX_PEERS || rank < 0 || rank >= world) return fail_invalid("acro_b200_halo_create: bad world size or rank");
    if (domain_size < 1 || domain_size > INT32_MAX) return fail_invalid("acro_b200_halo_create: domain size must be in 1..2^31-1");
    if (on_device && handle_out == nullptr) return fail_invalid("acro_b200_halo_create: null handle buffer");
    const size_t bytes = static_cast<size_t>((domain_size + 7) / 8);
    std::vector<const unsigned char *> bits(world);
    for (int p = 0; p < world; ++p) bits[p] = all_bitmaps + static_cast<size_t>(p) * bytes;

    // |S(a,b)| = number of domain entries reached by both a and b: fixes every rank's inbox layout
    std::vector<long long> pair(static_cast<size_t>(world) * world, 0);
    for (int a = 0; a < world; ++a)
    {
        for (int b = a + 1; b < world; ++b)
        {
            long long n = 0;
            for (size_t i = 0; i < bytes; ++i) n += __builtin_popcount(static_cast<unsigned int>(bits[a][i] & bits[b][i]));
            pair[a * world + b] = pair[b * world + a] = n;
        }
    }
    // segment of sender b inside rank a's inbox half
    std::vector<long long> seg(static_cast<size_t>(world) * world, 0);
    acro_b200_halo *h = new acro_b200_halo;
    h->world = world;
    h->rank = rank;
    h->domain = domain_size;
    for (int a = 0; a < world; ++a)
    {
        long long total = 0;
        for (int b = 0; b < world; ++b)
        {
            seg[a * world + b] = total;
            if (b != a) total += pair[a * world + b];
        }
        if (total >= INT32_MAX)
        {
            delete h;
            return fail_unsupported("acro_b200_halo_create: more than 2^31 shared entries on one rank");
        }
        h->stride[a] = ((total + 31) / 32) * 32 + 32;
    }
    for (int p = 0; p < world; ++p)
    {
        if (p != rank && pair[rank * world + p] > 0) h->neighbours |= 1u << p;
    }

    // this rank's shared entries, ascending, with their slots on both sides
    std::vector<long long> pos(world, 0);        // entries of S(rank,p) seen so far
    h->entry_off.push_back(0);
    for (int64_t d = 0; d < domain_size; ++d)
    {
        if (!bit_of(bits[rank], d)) continue;
        bool shared = false;
        for (int p = 0; p < world; ++p)
        {
            if (p == rank || !bit_of(bits[p], d)) continue;
            shared = true;
            h->entry_peer.push_back(p);
            h->entry_send.push_back(static_cast<int>(seg[p * world + rank] + pos[p]));
            h->entry_recv.push_back(static_cast<int>(seg[rank * world + p] + pos[p]));
            ++pos[p];
        }
        if (shared)
        {
            h->shared_idx.push_back(static_cast<int>(d));
            h->entry_off.push_back(static_cast<int>(h->entry_peer.size()));
        }
    }

    if (handle_out != nullptr) std::memset(handle_out, 0, ACRO_B200_IPC_HANDLE_BYTES);
    if (on_device)
    {
        static_assert(sizeof(cudaIpcMemHandle_t) <= ACRO_B200_IPC_HANDLE_BYTES, "IPC handle does not fit");
        std::vector<int> plan;
        plan.insert(plan.end(), h->shared_idx.begin(), h->shared_idx.end());
        plan.insert(plan.end(), h->entry_off.begin(), h->entry_off.end());
        plan.insert(plan.end(), h->entry_peer.begin(), h->entry_peer.end());
        plan.insert(plan.end(), h->entry_send.begin(), h->entry_send.end());
        plan.insert(plan.end(), h->entry_recv.begin(), h->entry_recv.end());
        cudaError_t status = cudaGetDevice(&h->device);
        if (status == cudaSuccess) status = cudaMalloc(&h->d_plan, plan.size() * sizeof(int));
        if (status == cudaSuccess) status = cudaMemcpy(h->d_plan, plan.data(), plan.size() * sizeof(int), cudaMemcpyHostToDevice);
        if (status == cudaSuccess) status = cudaMalloc(&h->d_ticket, 256);
        if (status == cudaSuccess) status = cudaMemset(h->d_ticket, 0, 256);
        if (status == cudaSuccess) status = cudaMalloc(&h->own, mailbox_bytes(h, rank));
        if (status == cudaSuccess) status = cudaMemset(h->own, 0, mailbox_bytes(h, rank));
        if (status == cudaSuccess && world > 1)
        {
            cudaIpcMemHandle_t ipc;
            status = cudaIpcGetMemHandle(&ipc, h->own);
            if (status == cudaSuccess) std::memcpy(handle_out, &ipc, sizeof ipc);
        }
        if (status != cudaSuccess)
        {
            if (h->d_plan) cudaFree(h->d_plan);
            if (h->d_ticket) cudaFree(h->d_ticket);
            if (h->own) cudaFree(h->own);
            delete h;
            return fail_cuda(status, "acro_b200_halo_create");
        }
        h->on_device = true;
        h->peer[rank] = h->own;
        h->connected = (world == 1);
    }
    *out = h;
    return ACRO_B200_OK;
}

int acro_b200_halo_counts(const acro_b200_halo *h, int64_t *shared_entries, int64_t *sharing_pairs, int64_t *inbox_doubles)
{
    if (h == nullptr) return fail_invalid("acro_b200_halo_counts: null argument");
    if (shared_entries) *shared_entries = static_cast<int64_t>(h->shared_idx.size());
    if (sharing_pairs) *sharing_pairs = static_cast<int64_t>(h->entry_peer.size());
    if (inbox_doubles) *inbox_doubles = h->stride[h->rank];
    return ACRO_B200_OK;
}

int acro_b200_halo_copy_plan(const acro_b200_halo *h, int *shared_idx, int *entry_off, int *entry_peer, int *entry_send, int *entry_recv)
{
    if (h == nullptr || shared_idx == nullptr || entry_off == nullptr || entry_peer == nullptr || entry_send == nullptr || entry_recv == nullptr)
        return fail_invalid("acro_b200_halo_copy_plan: null argument");
    std::memcpy(shared_idx, h->shared_idx.data(), h->shared_idx.size() * sizeof(int));
    std::memcpy(entry_off, h->entry_off.data(), h->entry_off.size() * sizeof(int));
    std::memcpy(entry_peer, h->entry_peer.data(), h->entry_peer.size() * sizeof(int));
    std::memcpy(entry_send, h->entry_send.data(), h->entry_send.size() * sizeof(int));
    std::memcpy(entry_recv, h->entry_recv.data(), h->entry_recv.size() * sizeof(int));
    return ACRO_B200_OK;
}

int acro_b200_halo_connect(acro_b200_halo *h, const unsigned char *all_handles)
{
    if (h == nullptr || all_handles == nullptr) return fail_invalid("acro_b200_halo_connect: null argument");
    if (!h->on_device) return fail_invalid("acro_b200_halo_connect: this exchange was created as a host-side plan only");
    if (h->connected) return ACRO_B200_OK;
    for (int p = 0; p < h->world; ++p)
    {
        if (p == h->rank) continue;
        cudaIpcMemHandle_t ipc;
        std::memcpy(&ipc, all_handles + static_cast<size_t>(p) * ACRO_B200_IPC_HANDLE_BYTES, sizeof ipc);
        cudaError_t status = cudaIpcOpenMemHandle(&h->peer[p], ipc, cudaIpcMemLazyEnablePeerAccess);
        if (status != cudaSuccess) return fail_cuda(status, "acro_b200_halo_connect (cudaIpcOpenMemHandle)");
    }
    h->opened_by_ipc = true;
    h->connected = true;
    return ACRO_B200_OK;
}

void *acro_b200_halo_inbox(const acro_b200_halo *h) { return h ? h->own : nullptr; }

int acro_b200_halo_connect_pointers(acro_b200_halo *h, void *const *inboxes)
{
    if (h == nullptr || inboxes == nullptr) return fail_invalid("acro_b200_halo_connect_pointers: null argument");
    if (!h->on_device) return fail_invalid("acro_b200_halo_connect_pointers: this exchange was created as a host-side plan only");
    if (h->connected) return ACRO_B200_OK;
    for (int p = 0; p < h->world; ++p)
    {
        if (p == h->rank) continue;
        if (inboxes[p] == nullptr) return fail_invalid("acro_b200_halo_connect_pointers: null inbox pointer");
        h->peer[p] = inboxes[p];
    }
    h->connected = true;
    return ACRO_B200_OK;
}

int acro_b200_halo_send(acro_b200_halo *h, const double *values, void *stream)
{
    const int ready = check_ready(h, values, "acro_b200_halo_send");
    if (ready != ACRO_B200_OK) return ready;
    const HaloView v = view_of(h, true);
    if (v.n_shared == 0) return ACRO_B200_OK;
    if (v.wait_flag == nullptr || sm_count() <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_halo_send");
    halo_send_kernel<<<grid_for(v.n_shared), kThreads, 0, as_stream(stream)>>>(v, values);
    return launch_status("acro_b200_halo_send");
}

int acro_b200_halo_combine(acro_b200_halo *h, double *values, void *stream)
{
    const int ready = check_ready(h, values, "acro_b200_halo_combine");
    if (ready != ACRO_B200_OK) return ready;
    if (h->seq == 0) return fail_invalid("acro_b200_halo_combine: no matching acro_b200_halo_send");
    const HaloView v = view_of(h, false);
    if (v.n_shared == 0) return ACRO_B200_OK;
    if (v.wait_flag == nullptr || sm_count() <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_halo_combine");
    halo_combine_kernel<<<grid_for(v.n_shared), kThreads, 0, as_stream(stream)>>>(v, values);
    return launch_status("acro_b200_halo_combine");
}

int acro_b200_halo_exchange_sum(acro_b200_halo *h, double *values, void *stream)
{
    const int sent = acro_b200_halo_send(h, values, stream);
    return sent != ACRO_B200_OK ? sent : acro_b200_halo_combine(h, values, stream);
}

int acro_b200_halo_destroy(acro_b200_halo *h)
{
    if (h == nullptr) return ACRO_B200_OK;
    if (h->opened_by_ipc)
    {
        for (int p = 0; p < h->world; ++p)
        {
            if (p != h->rank && h->peer[p] != nullptr) cudaIpcCloseMemHandle(h->peer[p]);
        }
    }
    if (h->d_plan) cudaFree(h->d_plan);
    if (h->d_ticket) cudaFree(h->d_ticket);
    if (h->own) cudaFree(h->own);
    delete h;
    return ACRO_B200_OK;
}

}
