// A peer group: the ranks (one process per GPU) that share a contracted batch index, and the
// device "mailbox" each of them exposes to the others over NVLink peer mappings.
//
// Mailbox of a rank (lives in that rank's own device memory):
//     data [2][world][kPeerSlot] doubles   partial results, indexed by call parity and sender
//     flag [2][world]            uint64    sequence number of the sender's last complete write
// A sender writes its partial into every rank's mailbox (plain remote stores), fences, then
// publishes the call's sequence number; a receiver polls only its OWN memory.  Two parity
// slots are enough: a rank cannot start call k+2 before every rank has published call k+1,
// which each does only after it finished reading call k.
#ifndef ACRO_B200_KERNELS_PEER_CUH
#define ACRO_B200_KERNELS_PEER_CUH

#include <cstdint>

#include "acro_b200.h"

namespace acro_b200_detail
{

// Doubles one rank can deposit per exchange (32 KB): a 64 x 64 result travels in one exchange; longer
// results take several, one sequence number each.
constexpr int kPeerSlot = 4096;

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
    return peer_data_doubles(world) * sizeof(double) + 2u * static_cast<size_t>(world) * sizeof(unsigned long long);
}

// Advances the group's call counter by `exchanges` (>= 1) and returns the view of the first of them
// (its seq member; the following exchanges use seq + 1, seq + 2, ...).
PeerView next_peer_view(acro_b200_peer_group *group, int64_t exchanges = 1);

}

#endif
