// reduce_batch: out[f] (op)= sum_n A[n*F + f] * w[n].
//
// A is read once as a flat stream of double2 words.  A tile is 2*T doubles, with the
// thread count T a multiple of F, so a thread's two lanes keep fixed columns (f) for
// the whole kernel and only the row advances.  Per-thread partial sums are combined
// per column in a fixed order inside the CTA, then across CTAs by whichever CTA
// finishes last (ticket counter), again in a fixed order: results do not depend on
// scheduling.
//
// Algorithmic HBM traffic: 8*F bytes of A and 8 bytes of w per row.
#include "common.cuh"
#include "peer.cuh"

#include <mutex>

using namespace acro_b200_detail;

namespace
{

constexpr int kMaxThreads = 512;
constexpr int kMaxGrid = 2048;
constexpr int kUnroll = 4;
constexpr size_t kCounterBytes = 256;   // keeps the partial sums 256-byte aligned

// Built-in scratch of the allocation-free entry point: room for rows of up to
// kNoAllocMaxF entries (256 + 2048*32*8 = 524,544 bytes, held by every GPU that loads
// the library until the process exits).
constexpr int kNoAllocMaxF = 32;
constexpr size_t kNoAllocBytes = kCounterBytes + static_cast<size_t>(kMaxGrid) * kNoAllocMaxF * sizeof(double);
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

__host__ __device__ inline int threads_for(int F) { return (kMaxThreads / F) * F; }

struct ReduceArgs
{
    const double *A;
    const double *w;
    double *out;
    int64_t rows;
    int F;
    int op;
    unsigned int *counter;
    double *partials;   // [gridDim.x][F]
    int *wait_flag;     // raised when the bounded wait on the peers gives up
};

template <bool WEIGHTED, bool VECTOR, bool PEERS>
__global__ void __launch_bounds__(kMaxThreads)
reduce_batch_kernel(const ReduceArgs a, const PeerView pv)
{
    extern __shared__ double lanes[];   // 2*T per-lane sums, reused by the final combine
    __shared__ bool is_last;

    const int F = a.F;
    const int T = blockDim.x;
    const int t = threadIdx.x;
    const int64_t tile_doubles = 2 * static_cast<int64_t>(T);
    const int64_t tile_rows = tile_doubles / F;
    const int64_t full_tiles = a.rows / tile_rows;

    // Columns and row offsets of this thread's two lanes inside a tile.
    const int e0 = 2 * t, e1 = 2 * t + 1;
    const int r0 = e0 / F, r1 = e1 / F;
    double acc0 = 0.0, acc1 = 0.0;

    // Main loop: kUnroll independent tiles in flight per thread.  The last, incomplete group takes the same
    // path with the missing tiles read as zeros (adding them changes nothing), so that its loads are in
    // flight together as well instead of one after the other.
    for (int64_t tile = blockIdx.x; tile < full_tiles; tile += static_cast<int64_t>(kUnroll) * gridDim.x)
    {
        double2 v[kUnroll];
        double w0[kUnroll], w1[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
        {
            const int64_t tl = tile + static_cast<int64_t>(u) * gridDim.x;
            v[u] = make_double2(0.0, 0.0);
            w0[u] = w1[u] = 0.0;
            if (tl < full_tiles)
            {
                const double *src = a.A + tl * tile_doubles + e0;
                if (VECTOR) v[u] = __ldcs(reinterpret_cast<const double2 *>(src));
                else { v[u].x = __ldcs(src); v[u].y = __ldcs(src + 1); }
                if (WEIGHTED)
                {
                    const int64_t row = tl * tile_rows;
                    w0[u] = __ldg(a.w + row + r0);
                    w1[u] = __ldg(a.w + row + r1);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < kUnroll; ++u)
        {
            if (WEIGHTED) { acc0 = fma(v[u].x, w0[u], acc0); acc1 = fma(v[u].y, w1[u], acc1); }
            else { acc0 += v[u].x; acc1 += v[u].y; }
        }
    }
    // Ragged tail (fewer rows than a tile): handled by the CTA whose turn it would be.
    if (static_cast<int64_t>(blockIdx.x) == full_tiles % gridDim.x)
    {
        const int64_t row_base = full_tiles * tile_rows;
        const int64_t left = a.rows - row_base;
        if (r0 < left)
        {
            const double x = a.A[(row_base + r0) * F + (e0 - r0 * F)];
            acc0 = WEIGHTED ? fma(x, a.w[row_base + r0], acc0) : acc0 + x;
        }
        if (r1 < left)
        {
            const double x = a.A[(row_base + r1) * F + (e1 - r1 * F)];
            acc1 = WEIGHTED ? fma(x, a.w[row_base + r1], acc1) : acc1 + x;
        }
    }

    // CTA combine: lane e belongs to column e % F; column sums in ascending lane order.
    lanes[e0] = acc0;
    lanes[e1] = acc1;
    __syncthreads();
    if (t < F)
    {
        double s = 0.0;
        for (int e = t; e < 2 * T; e += F) s += lanes[e];
        a.partials[static_cast<int64_t>(blockIdx.x) * F + t] = s;
    }

    // Ticket: the CTA that arrives last combines all partial sums.
    __threadfence();
    __syncthreads();
    if (t == 0)
    {
        const unsigned int ticket = atomicAdd(a.counter, 1u);
        is_last = (ticket == gridDim.x - 1);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();

    // Thread (column c = t % F, slot j = t / F) adds partials of CTAs j, j+J, ...; then
    // column c adds its J slot sums in ascending order.
    const int J = T / F;
    const int c = t % F, j = t / F;
    double s = 0.0;
    for (int g = j; g < static_cast<int>(gridDim.x); g += J) s += __ldcg(a.partials + static_cast<int64_t>(g) * F + c);
    lanes[j * F + c] = s;
    __syncthreads();
    double total = 0.0;
    if (t < F)
    {
        for (int jj = 0; jj < J; ++jj) total += lanes[jj * F + t];
    }
    if (PEERS) total = exchange_words(pv, t, F, total, a.wait_flag);
    if (t < F)
    {
        if (a.op == ACRO_B200_OP_ASSIGN) a.out[t] = total;
        else if (a.op == ACRO_B200_OP_ADD) a.out[t] += total;
        else a.out[t] -= total;
    }
    if (t == 0) *a.counter = 0u;   // leave the scratch ready for the next call
}

}

extern "C" {

size_t acro_b200_reduce_batch_scratch_bytes(int F)
{
    if (F < 1) return 0;
    return kCounterBytes + static_cast<size_t>(kMaxGrid) * static_cast<size_t>(F) * sizeof(double);
}

int acro_b200_reduce_batch_supported(int64_t rows, int F)
{
    return (F >= 1 && F <= kMaxThreads / 2 && rows >= 256) ? 1 : 0;
}

static int launch_reduce(const double *A, const double *w, double *out, int64_t rows, int F, int op, double *scratch,
                         size_t scratch_bytes, acro_b200_peer_group *group, void *stream)
{
    if (A == nullptr || out == nullptr || scratch == nullptr) return fail_invalid("acro_b200_reduce_batch: null argument");
    // The ticket counter must be zero when the kernel starts, and the kernel leaves it zero.  A caller
    // that zeroed it once may say so and save the clear in front of every launch.
    const bool counter_is_zero = (op & ACRO_B200_SCRATCH_READY) != 0;
    op &= ~ACRO_B200_SCRATCH_READY;
    if (rows < 1 || op < 0 || op > 2) return fail_invalid("acro_b200_reduce_batch: bad rows or operator");
    if (F < 1 || F > kMaxThreads / 2) return fail_unsupported("acro_b200_reduce_batch: row length must be 1..256");
    if (scratch_bytes < acro_b200_reduce_batch_scratch_bytes(F)) return fail_invalid("acro_b200_reduce_batch: scratch buffer too small");
    if ((reinterpret_cast<uintptr_t>(scratch) & 255u) != 0) return fail_invalid("acro_b200_reduce_batch: scratch must be 256-byte aligned");
    const int sms = sm_count();
    if (sms <= 0) return fail_cuda(cudaErrorNoDevice, "acro_b200_reduce_batch");

    const int T = threads_for(F);
    const int64_t tile_rows = 2 * static_cast<int64_t>(T) / F;
    const int64_t tiles = (rows + tile_rows - 1) / tile_rows;

    ReduceArgs args;
    args.A = A;
    args.w = w;
    args.out = out;
    args.rows = rows;
    args.F = F;
    args.op = op;
    args.counter = reinterpret_cast<unsigned int *>(scratch);
    args.partials = reinterpret_cast<double *>(reinterpret_cast<char *>(scratch) + kCounterBytes);
    args.wait_flag = nullptr;
    PeerView pv;
    pv.world = 0;
    if (group != nullptr)
    {
        if (acro_b200_peer_group_is_connected(group) != 1) return fail_invalid("acro_b200_reduce_batch_allreduce: the peer group is not connected");
        if (F > kPeerWordEntries) return fail_unsupported("acro_b200_reduce_batch_allreduce: row length exceeds the mailbox slot");
        args.wait_flag = wait_flag_device_ptr();
        if (args.wait_flag == nullptr) return fail_cuda(cudaErrorUnknown, "acro_b200_reduce_batch_allreduce (status flag)");
        pv = next_peer_view(group);
    }

    cudaStream_t s = as_stream(stream);
    if (!counter_is_zero)
    {
        cudaError_t status = cudaMemsetAsync(args.counter, 0, kCounterBytes, s);
        if (status != cudaSuccess) return fail_cuda(status, "acro_b200_reduce_batch (counter reset)");
    }
    const size_t smem = 2 * static_cast<size_t>(T) * sizeof(double);
    const bool vec = aligned16(A);
    typedef void (*kernel_t)(const ReduceArgs, const PeerView);
    const kernel_t kernel = group != nullptr
                                ? (w != nullptr ? (vec ? reduce_batch_kernel<true, true, true> : reduce_batch_kernel<true, false, true>)
                                                : (vec ? reduce_batch_kernel<false, true, true> : reduce_batch_kernel<false, false, true>))
                                : (w != nullptr ? (vec ? reduce_batch_kernel<true, true, false> : reduce_batch_kernel<true, false, false>)
                                                : (vec ? reduce_batch_kernel<false, true, false> : reduce_batch_kernel<false, false, false>));
    // One CTA per slot the SMs offer this kernel (registers allow two or three CTAs of this size per SM): every CTA
    // is resident from the start and walks its share of the tiles, so there is no second wave of CTAs half-way through.
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, T, smem) != cudaSuccess || per_sm < 1) per_sm = 1;
    int64_t grid = static_cast<int64_t>(sms) * per_sm;
    if (grid > tiles) grid = tiles;
    if (grid > kMaxGrid) grid = kMaxGrid;
    if (grid < 1) grid = 1;
    kernel<<<static_cast<int>(grid), T, smem, s>>>(args, pv);
    return launch_status(group != nullptr ? "acro_b200_reduce_batch_allreduce" : "acro_b200_reduce_batch");
}

int acro_b200_reduce_batch(const double *A, const double *w, double *out, int64_t rows, int F, int op,
                           double *scratch, size_t scratch_bytes, void *stream)
{
    return launch_reduce(A, w, out, rows, F, op, scratch, scratch_bytes, nullptr, stream);
}

// The reduction fused with the all-reduce over the ranks of a peer group: every rank streams
// its own slab of rows, and the last CTA of each rank exchanges the F column totals with the
// other ranks through their mailboxes (remote stores over NVLink, one bounded wait on local
// memory) before it writes the result.  One kernel, no separate collective launch; all ranks
// obtain bit-identical results.  Every rank of the group must make the same sequence of
// calls; a rank that never calls makes the others give up after about a second with
// ACRO_B200_ETIMEOUT reported by acro_b200_device_status().
int acro_b200_reduce_batch_allreduce(const double *A, const double *w, double *out, int64_t rows, int F, int op,
                                     double *scratch, size_t scratch_bytes, acro_b200_peer_group *group, void *stream)
{
    if (group == nullptr) return fail_invalid("acro_b200_reduce_batch_allreduce: null peer group");
    return launch_reduce(A, w, out, rows, F, op, scratch, scratch_bytes, group, stream);
}

int acro_b200_reduce_batch_noalloc_max_f(void) { return kNoAllocMaxF; }

// Same reduction as acro_b200_reduce_batch, for callers that must not allocate device
// memory: the partial sums and the ticket counter live in g_noalloc_scratch.
//
// In host code the name g_noalloc_scratch is only a host-side handle of the symbol, not a
// device address, so the address is looked up with cudaGetSymbolAddress, once per device
// and with that device current, the first time this function runs on the device.  That
// first call should therefore happen before any stream capture begins.  Later calls only
// read the cached address.  A call of acro_b200_set_context makes the next call on every
// device a first call again (the address is per context), with the same rule about capture.
//
// The function itself calls no cudaMalloc / cudaFree and no allocating library routine.
// All calls on one GPU share the one scratch array, which still holds the previous call's
// partial sums: the ticket counter is cleared on the stream before every launch, the
// partial sums are fully rewritten before they are read.  Two calls that overlap on the
// same GPU (different streams, or different host threads without ordering) race on it.
int acro_b200_reduce_batch_noalloc(const double *A, const double *w, double *out, int64_t rows, int F, int op, void *stream)
{
    if (F < 1 || F > kNoAllocMaxF)
    {
        return fail_unsupported("acro_b200_reduce_batch_noalloc: row length " + std::to_string(F) +
                                " exceeds the built-in scratch (at most " + std::to_string(kNoAllocMaxF) +
                                " entries per row); use acro_b200_reduce_batch with caller-provided scratch");
    }
    constexpr int kMaxDevices = 64;
    static std::mutex lock;
    static double *scratch_of_device[kMaxDevices] = {nullptr};
    static unsigned long long epoch_of_device[kMaxDevices] = {0};
    int dev = -1;
    cudaError_t status = cudaGetDevice(&dev);
    if (status != cudaSuccess) return fail_cuda(status, "acro_b200_reduce_batch_noalloc (cudaGetDevice)");
    if (dev < 0 || dev >= kMaxDevices) return fail_invalid("acro_b200_reduce_batch_noalloc: device ordinal out of range");
    double *scratch = nullptr;
    {
        std::lock_guard<std::mutex> guard(lock);
        // The symbol has one address per CUDA context: after acro_b200_set_context the address
        // found earlier belongs to the context that was current then, so it is looked up again.
        const unsigned long long epoch = context_epoch();
        if (scratch_of_device[dev] == nullptr || epoch_of_device[dev] != epoch)
        {
            void *ptr = nullptr;
            status = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
            if (status != cudaSuccess) return fail_cuda(status, "acro_b200_reduce_batch_noalloc (cudaGetSymbolAddress)");
            scratch_of_device[dev] = static_cast<double *>(ptr);
            epoch_of_device[dev] = epoch;
        }
        scratch = scratch_of_device[dev];
    }
    return acro_b200_reduce_batch(A, w, out, rows, F, op, scratch, kNoAllocBytes, stream);
}

}
