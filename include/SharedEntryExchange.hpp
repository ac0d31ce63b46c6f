// acro::SharedEntryExchange — sums the domain entries of a sharded IndexMapping that several
// ranks reach (one process per GPU of one node).  No counterpart in LLNL/acrotensor, which is
// single-GPU; it completes TensorEngine::FlatIndexedSumGather (kernel/TensorEngine.hpp:84) when
// the range of the mapping is cut into one slab per rank.
//
//   all_gather(bytes) must return the same-sized byte strings of every rank in rank order
//   (MPI_Allgather, torch.distributed ...).  It is called twice: with the bitmap of the domain
//   entries this rank's map reaches, then with the CUDA IPC handle of this rank's inbox.
//
//   acro::SharedEntryExchange X(M, world, rank, all_gather);
//   TE.FlatIndexedSumGather(Aout, Ain, M, X);      // local sum, then the sum over the sharing ranks
#ifndef ACRO_B200_SHARED_ENTRY_EXCHANGE_HPP
#define ACRO_B200_SHARED_ENTRY_EXCHANGE_HPP

#include <functional>
#include <string>
#include <vector>

#include "Error.hpp"
#include "IndexMapping.hpp"
#include "acro_b200.h"

namespace acro
{

class SharedEntryExchange
{
    public:
    typedef std::vector<unsigned char> Bytes;
    typedef std::function<std::vector<Bytes>(const Bytes &)> AllGather;

    SharedEntryExchange(IndexMapping &M, int world, int rank, AllGather all_gather) : Handle(nullptr)
    {
        const std::int64_t domain = M.GetDomainSize();
        Bytes mine(static_cast<size_t>((domain + 7) / 8));
        Check(acro_b200_halo_mark_touched(&M[0], M.GetRangeSize(), domain, mine.data()));
        Bytes handle(ACRO_B200_IPC_HANDLE_BYTES);
        Check(acro_b200_halo_create(world, rank, domain, Flatten(all_gather(mine), world, mine.size()).data(), 1, &Handle, handle.data()));
        if (world > 1) Check(acro_b200_halo_connect(Handle, Flatten(all_gather(handle), world, handle.size()).data()));
    }
    ~SharedEntryExchange() { acro_b200_halo_destroy(Handle); }
    SharedEntryExchange(const SharedEntryExchange &) = delete;
    SharedEntryExchange &operator=(const SharedEntryExchange &) = delete;

    // Number of domain entries this rank shares with at least one other rank.
    std::int64_t GetNumShared()
    {
        std::int64_t n = 0;
        Check(acro_b200_halo_counts(Handle, &n, nullptr, nullptr));
        return n;
    }

    operator void *() { return Handle; }
    acro_b200_halo *GetHandle() { return Handle; }

    private:
    static void Check(int status)
    {
        if (status != ACRO_B200_OK) throw_error(std::string("SharedEntryExchange:  ") + acro_b200_last_error());
    }
    static Bytes Flatten(const std::vector<Bytes> &parts, int world, size_t each)
    {
        ACROBATIC_ASSERT(static_cast<int>(parts.size()) == world, "all_gather must return one byte string per rank.");
        Bytes flat;
        for (const Bytes &p : parts)
        {
            ACROBATIC_ASSERT(p.size() == each, "all_gather returned byte strings of different sizes.");
            flat.insert(flat.end(), p.begin(), p.end());
        }
        return flat;
    }
    acro_b200_halo *Handle;
};

}

#endif
