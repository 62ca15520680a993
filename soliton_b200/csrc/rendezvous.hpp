// Host-side rendezvous of the ranks of one box through a shared-memory file.
//
// Takes the place of the NCCL bootstrap the reference uses (ncclGetUniqueId / ncclCommInitRank,
// core/cuda/kernels.cu:761-771): rank 0 creates a file (under /dev/shm when present) and puts its path into the
// 128-byte id that Soliton's Python publishes to the other ranks (python/soliton/distributed.py:21-32); every rank
// maps the file. Through it the ranks exchange, with plain loads and stores and monotonic counters:
//   - once: device facts and the IPC handle of each rank's workspace;
//   - per collective: which device allocations hold the rank's gradients (a table of export slots with IPC
//     handles plus a table of (export, offset, elements) per segment), and the fact that the rank has arrived.
//     An export slot goes through: published -> freed by its owner -> let go by every peer (acks) -> reusable.
// Nothing here touches CUDA: handles are opaque 64-byte blobs, which is what lets CPU-only tests drive the
// protocol with several processes. Every wait is bounded and returns an error instead of hanging.
#pragma once
#include <atomic>
#include <cstddef>
#include <cstdint>

namespace slb {

constexpr int kRdvMaxWorld = 8;
constexpr int kRdvMaxSegs = 4096;
constexpr int kRdvMaxExports = 8192;
constexpr int kIdBytes = 128;  // NCCL_UNIQUE_ID_BYTES, the size Soliton's Python allocates for the id

struct RdvExport {              // one device allocation a rank lets its peers map
    unsigned char handle[64];
    uint64_t size;
    std::atomic<uint32_t> freed;  // set by the owner when it wants the allocation back
    std::atomic<uint32_t> acks;   // bit r: rank r has seen `freed` and holds no mapping of this allocation any more
    uint32_t generation;          // counts the allocations this slot has described
    uint32_t pad;
};

struct RdvSegment {             // where one segment's gradient lives on the publishing rank
    uint32_t export_id;
    uint32_t generation;        // of that export slot when the table was written
    uint64_t offset;            // bytes from the allocation's base
    int64_t n;                  // elements
};

struct RdvRank {
    std::atomic<uint32_t> stage;        // init / teardown handshake
    std::atomic<uint32_t> failed;       // this rank gave up; peers stop waiting for it
    int32_t ordinal, sm_count, pid, pad;
    unsigned char ws_handle[64];
    uint64_t ws_offset;
    std::atomic<uint64_t> arrive;       // collectives entered so far
    uint64_t version_at[2];             // table version used for collective k, at [k & 1]
    uint32_t nseg_at[2];
    std::atomic<uint32_t> n_exports;    // slots in use so far (high-water mark; freed slots below it are reused)
    std::atomic<uint32_t> free_epoch;   // bumped by every mark_freed: peers rescan the slots only when it moved
    RdvExport exports[kRdvMaxExports];
    RdvSegment table[2][kRdvMaxSegs];   // contents of table version v at [v & 1]
};

struct RdvShared {
    uint64_t magic;
    uint32_t world;
    uint32_t pad;
    RdvRank rank[kRdvMaxWorld];
};

class Rendezvous {
public:
    // Rank 0: creates the shared file and writes the id the other ranks open it with. 0 on success.
    static int create_id(char out[kIdBytes]);

    int open(const char id[kIdBytes], int rank, int world, double timeout_s);
    void close();
    // Rank 0, once every rank has mapped the file: remove its name. The mapping stays valid for all of them, and
    // nothing is left behind in the file system if the job dies later.
    void unlink_now();
    bool is_open() const { return shm_ != nullptr; }

    int rank() const { return rank_; }
    int world() const { return world_; }
    RdvRank& self() { return shm_->rank[rank_]; }
    RdvRank& peer(int r) { return shm_->rank[r]; }

    // Handshake: announce stage s and wait until every rank has reached it. 0, or -1 on timeout / peer failure.
    int stage_barrier(uint32_t s, double timeout_s);

    // Publishes an allocation in a slot of this rank's export table -- a slot whose previous allocation every peer
    // has let go of, else a new one -- and returns the slot, or -1 when all kRdvMaxExports slots are live.
    int add_export(const unsigned char handle[64], uint64_t size);
    uint32_t generation_of(uint32_t export_id) { return self().exports[export_id].generation; }
    // Owner: asks the peers to let go of the allocation in that slot.
    void mark_freed(uint32_t export_id);
    // Owner: true once every peer has acknowledged; the slot then returns to the free list.
    bool released_by_all(uint32_t export_id);
    void recycle(uint32_t export_id);
    // Peer: acknowledges that this rank holds no mapping of rank r's slot any more.
    void ack_freed(int r, uint32_t export_id);

    // Collective k (1, 2, ...): publish this rank's table (only copied when it differs from the previous one),
    // announce arrival, wait for every rank. 0, or -1 on timeout / peer failure / disagreement on nseg.
    int arrive(uint64_t k, const RdvSegment* table, uint32_t nseg, double timeout_s);
    // After arrive(k): the table rank r published for collective k. *version tells whether it changed.
    const RdvSegment* table_of(int r, uint64_t k, uint32_t* nseg, uint64_t* version);

    void fail();  // tell the peers this rank is leaving with an error

private:
    RdvShared* shm_ = nullptr;
    int rank_ = 0, world_ = 1;
    bool owner_ = false;
    char path_[kIdBytes] = {0};
    uint64_t my_version_ = 0;
    uint32_t free_slots_[kRdvMaxExports];   // owner side: slots ready for reuse (a stack)
    uint32_t n_free_slots_ = 0;
};

}  // namespace slb
