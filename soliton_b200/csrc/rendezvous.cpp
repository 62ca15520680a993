// Shared-memory rendezvous (see rendezvous.hpp).
#include "rendezvous.hpp"

#include <fcntl.h>
#include <sched.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>

namespace slb {

static constexpr uint64_t kMagic = 0x534c42325f524456ULL;  // "SLB2_RDV"
static constexpr char kIdTag[8] = {'S', 'L', 'B', '2', 'S', 'H', 'M', 0};

static double mono() {
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec + 1e-9 * ts.tv_nsec;
}

static void backoff(int& spins) {
    if (++spins < 2000) {
        sched_yield();
    } else {
        timespec ts{0, 50000};
        nanosleep(&ts, nullptr);
    }
}

int Rendezvous::create_id(char out[kIdBytes]) {
    memset(out, 0, kIdBytes);
    const char* dir = getenv("SOLITON_B200_SHM_DIR");
    struct stat sb;
    if (!dir) dir = (stat("/dev/shm", &sb) == 0 && S_ISDIR(sb.st_mode)) ? "/dev/shm" : "/tmp";
    unsigned long long token = 0;
    int rnd = ::open("/dev/urandom", O_RDONLY);
    if (rnd >= 0) {
        if (read(rnd, &token, sizeof token) != (ssize_t)sizeof token) token = 0;
        ::close(rnd);
    }
    token ^= (unsigned long long)getpid() << 32 ^ (unsigned long long)(mono() * 1e9);
    memcpy(out, kIdTag, 8);
    const int len = snprintf(out + 8, kIdBytes - 8, "%s/soliton_b200_%016llx", dir, token);
    if (len <= 0 || len >= kIdBytes - 8) return -1;
    const int fd = ::open(out + 8, O_CREAT | O_EXCL | O_RDWR, 0600);
    if (fd < 0) return -1;
    const int rc = ftruncate(fd, sizeof(RdvShared));  // zero-filled: all counters start at 0
    ::close(fd);
    if (rc != 0) {
        unlink(out + 8);
        return -1;
    }
    return 0;
}

int Rendezvous::open(const char id[kIdBytes], int rank, int world, double timeout_s) {
    if (shm_ || world < 1 || world > kRdvMaxWorld || rank < 0 || rank >= world) return -1;
    if (memcmp(id, kIdTag, 8) != 0 || id[kIdBytes - 1] != 0) return -1;
    memcpy(path_, id + 8, kIdBytes - 8);
    const double t0 = mono();
    int fd = -1, spins = 0;
    for (;;) {
        fd = ::open(path_, O_RDWR);
        struct stat sb;
        if (fd >= 0 && fstat(fd, &sb) == 0 && (size_t)sb.st_size >= sizeof(RdvShared)) break;
        if (fd >= 0) ::close(fd), fd = -1;
        if (mono() - t0 > timeout_s) return -1;
        backoff(spins);
    }
    void* m = mmap(nullptr, sizeof(RdvShared), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED) return -1;
    shm_ = static_cast<RdvShared*>(m);
    rank_ = rank, world_ = world, owner_ = rank == 0, my_version_ = 0, n_free_slots_ = 0;
    if (rank == 0) {
        shm_->world = (uint32_t)world;
        std::atomic_thread_fence(std::memory_order_release);
        shm_->magic = kMagic;
    }
    return 0;
}

void Rendezvous::close() {
    if (!shm_) return;
    munmap(shm_, sizeof(RdvShared));
    shm_ = nullptr;
    if (owner_) unlink(path_);
}

void Rendezvous::unlink_now() {
    if (shm_ && owner_) unlink(path_);
}

void Rendezvous::fail() {
    if (shm_) self().failed.store(1, std::memory_order_release);
}

int Rendezvous::stage_barrier(uint32_t s, double timeout_s) {
    self().stage.store(s, std::memory_order_release);
    const double t0 = mono();
    for (int r = 0; r < world_; r++) {
        int spins = 0;
        while (peer(r).stage.load(std::memory_order_acquire) < s) {
            if (peer(r).failed.load(std::memory_order_acquire) || mono() - t0 > timeout_s) return -1;
            backoff(spins);
        }
    }
    return 0;
}

int Rendezvous::add_export(const unsigned char handle[64], uint64_t size) {
    RdvRank& me = self();
    uint32_t id;
    if (n_free_slots_ > 0) {
        id = free_slots_[--n_free_slots_];
    } else {
        id = me.n_exports.load(std::memory_order_relaxed);
        if (id >= (uint32_t)kRdvMaxExports) return -1;
    }
    RdvExport& x = me.exports[id];
    memcpy(x.handle, handle, 64);
    x.size = size;
    x.generation++;
    x.acks.store(0, std::memory_order_relaxed);
    x.freed.store(0, std::memory_order_release);
    if (id >= me.n_exports.load(std::memory_order_relaxed)) me.n_exports.store(id + 1, std::memory_order_release);
    return (int)id;
}

void Rendezvous::mark_freed(uint32_t export_id) {
    if (!shm_ || export_id >= (uint32_t)kRdvMaxExports) return;
    self().exports[export_id].freed.store(1, std::memory_order_release);
    self().free_epoch.fetch_add(1, std::memory_order_release);
}

bool Rendezvous::released_by_all(uint32_t export_id) {
    if (!shm_ || export_id >= (uint32_t)kRdvMaxExports) return true;
    const uint32_t everyone = ((1u << world_) - 1) & ~(1u << rank_);
    return (self().exports[export_id].acks.load(std::memory_order_acquire) & everyone) == everyone;
}

void Rendezvous::recycle(uint32_t export_id) {
    if (shm_ && export_id < (uint32_t)kRdvMaxExports && n_free_slots_ < (uint32_t)kRdvMaxExports)
        free_slots_[n_free_slots_++] = export_id;
}

void Rendezvous::ack_freed(int r, uint32_t export_id) {
    if (shm_ && export_id < (uint32_t)kRdvMaxExports)
        peer(r).exports[export_id].acks.fetch_or(1u << rank_, std::memory_order_acq_rel);
}

int Rendezvous::arrive(uint64_t k, const RdvSegment* table, uint32_t nseg, double timeout_s) {
    if (nseg > (uint32_t)kRdvMaxSegs) return -1;
    RdvRank& me = self();
    // Publish a new version only when the table changed. Version v lives in slot v & 1; the slot a reader of
    // collective k may still be looking at is never the one written here, because a rank can be at most one
    // collective ahead of the slowest rank (it waits for everybody below).
    bool changed = my_version_ == 0;
    if (!changed) {
        const uint32_t prev = me.nseg_at[(k - 1) & 1];
        changed = prev != nseg || memcmp(me.table[my_version_ & 1], table, nseg * sizeof(RdvSegment)) != 0;
    }
    if (changed) {
        my_version_++;
        memcpy(me.table[my_version_ & 1], table, nseg * sizeof(RdvSegment));
    }
    me.version_at[k & 1] = my_version_;
    me.nseg_at[k & 1] = nseg;
    me.arrive.store(k, std::memory_order_release);
    const double t0 = mono();
    for (int r = 0; r < world_; r++) {
        int spins = 0;
        while (peer(r).arrive.load(std::memory_order_acquire) < k) {
            if (peer(r).failed.load(std::memory_order_acquire) || mono() - t0 > timeout_s) return -1;
            backoff(spins);
        }
        if (peer(r).nseg_at[k & 1] != nseg) return -1;  // the ranks disagree about this collective
    }
    return 0;
}

const RdvSegment* Rendezvous::table_of(int r, uint64_t k, uint32_t* nseg, uint64_t* version) {
    RdvRank& p = peer(r);
    *nseg = p.nseg_at[k & 1];
    *version = p.version_at[k & 1];
    return p.table[*version & 1];
}

}  // namespace slb
