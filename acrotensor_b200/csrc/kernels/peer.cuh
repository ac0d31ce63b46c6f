// A peer group: the ranks (one process per GPU) that share a contracted batch index, and the
// device "mailbox" each of them exposes to the others over NVLink peer mappings.
//
// Mailbox of a rank (lives in that rank's own device memory):
//     data [2][world][kPeerSlot] doubles   partial results, indexed by call parity and sender
//     flag [2][world]            uint64    sequence number of the sender's last complete write
//     word [2][world][kPeerWords] uint64   short results that carry their own arrival mark (below)
// A sender writes its partial into every rank's mailbox (plain remote stores), fences, then
// publishes the call's sequence number; a receiver polls only its OWN memory.  Two parity
// slots are enough: a rank cannot start call k+2 before every rank has published call k+1,
// which each does only after it finished reading call k.
//
// Results of at most 256 entries (the reduction kernel's fused exchange, and the stand-alone
// all-reduce for results of that size, so that the two are interchangeable) use the `word` area
// instead and need no fence: a double travels as two 8-byte words, each holding one half of its
// bits below the low 32 bits of the call's sequence number.  An 8-byte store arrives whole, so a
// word whose upper half has reached the call's number holds that call's data; the receiver polls
// the words themselves.  The fenced form costs two NVLink round trips per call (data, fence, flag,
// and the reader's fence), this one a single one-way trip.
#ifndef ACRO_B200_KERNELS_PEER_CUH
#define ACRO_B200_KERNELS_PEER_CUH

#include <cstdint>

#include "acro_b200.h"

namespace acro_b200_detail
{

// Doubles one rank can deposit per exchange (32 KB): a 64 x 64 result travels in one exchange; longer
// results take several, one sequence number each.
constexpr int kPeerSlot = 4096;
// 8-byte words per (call parity, sender) of the fence-free area: two per entry, rows of at most 256 entries.
constexpr int kPeerWordEntries = 256;
constexpr int kPeerWords = 2 * kPeerWordEntries;

struct PeerView   // passed to kernels by value
{
    int world;
    int rank;
    unsigned long long seq;                       // sequence number of this call (>= 1)
    double *data[ACRO_B200_MAX_PEERS];            // mailbox data of every rank (own one is local)
    unsigned long long *flag[ACRO_B200_MAX_PEERS];
};

__host__ __device__ inline size_t peer_data_doubles(int world) { return 2u * static_cast<size_t>(world) * kPeerSlot; }
__host__ __device__ inline size_t peer_mailbox_bytes(int world)
{
    return peer_data_doubles(world) * sizeof(double) + 2u * static_cast<size_t>(world) * sizeof(unsigned long long)
           + 2u * static_cast<size_t>(world) * kPeerWords * sizeof(unsigned long long);
}

// The fence-free word area of rank p's mailbox (16-byte aligned: it follows 16 * world bytes of flags).
__host__ __device__ inline unsigned long long *peer_words(const PeerView &v, int p) { return v.flag[p] + 2u * static_cast<size_t>(v.world); }

#ifdef __CUDACC__
__device__ __forceinline__ void store_word_pair(unsigned long long *p, unsigned long long a, unsigned long long b)
{
    asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void load_word_pair(const unsigned long long *p, unsigned long long &a, unsigned long long &b)
{
    asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
// true when the word was written by call `mark` or a later one (sequence numbers compared modulo 2^32)
__device__ __forceinline__ bool word_arrived(unsigned long long w, unsigned int mark)
{
    return static_cast<int>(static_cast<unsigned int>(w >> 32) - mark) >= 0;
}

// Sum of this rank's total with the totals of all peer ranks, exchanged through the word area of the
// mailboxes (above: every 8-byte word carries half a double and the call's number, so there is
// no fence and no separate flag).  Called by all threads of one CTA; `mine` is column t's total
// on this rank (t < F <= kPeerWordEntries).  Every (column, sender) pair is polled by a thread of its
// own, then every rank adds the world totals in rank order, so all ranks obtain the same bits.  The
// wait is bounded; when it runs out a flag is raised for the host and the (then meaningless) result
// is still written, so nothing hangs.  A word from a later call also ends the wait: a rank that comes
// late finds its peers' slots already reused, gets a meaningless sum for the calls the peers gave up
// on, and meets them again at the first call they have not started yet.
__device__ __forceinline__ double exchange_words(const PeerView &pv, int t, int F, double mine, int *wait_flag)
{
    const int par = static_cast<int>(pv.seq & 1ull);
    const unsigned int mark = static_cast<unsigned int>(pv.seq);
    if (t < F)
    {
        const unsigned long long bits = static_cast<unsigned long long>(__double_as_longlong(mine));
        const unsigned long long lo = (static_cast<unsigned long long>(mark) << 32) | (bits & 0xffffffffull);
        const unsigned long long hi = (static_cast<unsigned long long>(mark) << 32) | (bits >> 32);
        const size_t at = (static_cast<size_t>(par) * pv.world + pv.rank) * kPeerWords + 2 * static_cast<size_t>(t);
        for (int p = 0; p < pv.world; ++p) store_word_pair(peer_words(pv, p) + at, lo, hi);   // remote stores over the peer mapping
    }
    const unsigned long long *box = peer_words(pv, pv.rank) + static_cast<size_t>(par) * pv.world * kPeerWords;
    bool gave_up = false;
    for (int i = t; i < F * pv.world; i += static_cast<int>(blockDim.x))
    {
        const int r = i / F, c = i - r * F;
        const unsigned long long *src = box + static_cast<size_t>(r) * kPeerWords + 2 * c;
        bool arrived = false;
        for (unsigned int tries = 0; tries < (1u << 21); ++tries)   // about half a second
        {
            unsigned long long lo, hi;
            load_word_pair(src, lo, hi);
            if (word_arrived(lo, mark) && word_arrived(hi, mark)) { arrived = true; break; }
            __nanosleep(64);
        }
        if (!arrived) gave_up = true;
    }
    if (gave_up) atomicExch(wait_flag, 1);
    __syncthreads();
    double total = 0.0;
    if (t < F)
    {
        for (int r = 0; r < pv.world; ++r)
        {
            unsigned long long lo, hi;
            load_word_pair(box + static_cast<size_t>(r) * kPeerWords + 2 * t, lo, hi);
            total += __longlong_as_double(static_cast<long long>((hi << 32) | (lo & 0xffffffffull)));
        }
    }
    return total;
}
#endif

// Advances the group's call counter by `exchanges` (>= 1) and returns the view of the first of them
// (its seq member; the following exchanges use seq + 1, seq + 2, ...).
PeerView next_peer_view(acro_b200_peer_group *group, int64_t exchanges = 1);

}

#endif
