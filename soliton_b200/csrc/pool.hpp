// Deterministic caching allocator: one pool per device kind (cpu, meta, cuda).
//
// Policy-equivalent to Soliton's core/soliton/alloc.d (Pool, alloc.d:26-223): the same size classes, the same
// exact-size block cache, the same FNV-1a trace hash over (kind, rounded size) events, the same reserve limit with
// one flush-and-retry, the same trace recording and arena replay. Because the policy depends only on the sequence
// of requested sizes, the meta pool (fake addresses, no memory) reports the byte counts the cuda pool will see.
// The cache hands blocks out in the reference's order too (the first block of the exact size, whose place the last
// cached block then takes, alloc.d:145-151), so that the sequence of addresses a run sees is the reference's. The cuda
// pool additionally keeps a registry of the raw blocks it owns, so that the data-parallel engine can export them to
// peer processes.
#pragma once
#include <cstddef>
#include <cstdint>
#include <map>
#include <unordered_map>
#include <vector>

namespace slb {

enum Dev : int { DEV_CPU = 0, DEV_META = 1, DEV_CUDA = 2, DEV_COUNT = 3 };

// Raw memory source of the cuda pool, installed by the CUDA side of the library (so this file needs no CUDA).
struct RawBackend {
    void* (*alloc)(size_t) = nullptr;
    void (*free)(void*) = nullptr;
    void (*on_free)(void* base) = nullptr;  // called before a raw cuda block is returned to the driver
};

class Pool {
public:
    explicit Pool(int dev) : dev_(dev) {}

    // alloc.d:54-60: 512-byte classes below 1 MiB, 2 MiB classes from there on; a zero request counts as 1 byte.
    static size_t round_size(size_t n) {
        constexpr size_t small = 512, large = size_t(2) << 20;
        if (n == 0) n = 1;
        return n < (size_t(1) << 20) ? (n + small - 1) / small * small : (n + large - 1) / large * large;
    }

    void* alloc(size_t n);             // alloc.d:128-174
    void release(void* p, size_t n);   // alloc.d:176-200
    void empty_cache();                // alloc.d:215-223

    // statistics (api.d:143-164)
    void stats(int64_t out[7]) const;
    void reset_stats();
    void set_limit(int64_t bytes) { limit_ = bytes; }

    // trace recording (api.d:168-215, alloc.d:113-126)
    void record_start();
    void record_stop() { recording_ = false; }
    void record_mark();
    int64_t record_count() const { return (int64_t)rec_size_.size(); }
    int64_t record_body() const { return marks_.empty() ? 0 : marks_.back(); }
    void record_get(int64_t* size, int64_t* start, int64_t* end) const;

    // arena replay (api.d:217-260, alloc.d:98-111, 202-213)
    int arena_install(const int64_t* offsets, const int64_t* sizes, int64_t count, int64_t body, int64_t bytes);
    bool diverged() const { return diverged_; }
    void arena_off();

    // Registry of raw cuda blocks (base -> size), for the peer-export table. Empty for cpu and meta.
    bool find_raw(const void* p, void** base, size_t* size) const;

    static RawBackend cuda_backend;

private:
    void* raw_alloc(size_t n);
    void raw_free(void* p);
    void* arena_alloc(size_t n);
    void release_arena();
    void mix(uint64_t kind, size_t n) {
        hash_ = (hash_ ^ kind) * 1099511628211ULL;
        hash_ = (hash_ ^ (uint64_t)n) * 1099511628211ULL;
    }
    void count_alloc(size_t n) {
        allocated_ += (int64_t)n;
        n_alloc_++;
        if (allocated_ > peak_allocated_) peak_allocated_ = allocated_;
    }

    static constexpr uint64_t kHashSeed = 1469598103934665603ULL;
    static constexpr size_t kMaxMarks = 64;

    int dev_;
    struct Cached {
        size_t size;
        void* ptr;
    };
    std::vector<Cached> cache_;   // in release order, holes filled from the back (alloc.d:145-151, 199)
    int64_t allocated_ = 0, reserved_ = 0, peak_allocated_ = 0, peak_reserved_ = 0, n_alloc_ = 0, n_raw_ = 0;
    int64_t limit_ = 0;
    uint64_t hash_ = kHashSeed;
    size_t meta_next_ = 4096;

    bool recording_ = false;
    std::vector<int64_t> rec_size_, rec_start_, rec_end_, marks_;

    char* arena_ = nullptr;
    int64_t arena_bytes_ = 0;
    const int64_t* plan_offset_ = nullptr;
    const int64_t* plan_size_ = nullptr;
    size_t plan_count_ = 0, plan_cursor_ = 0, plan_body_ = 0;
    bool arena_mode_ = false, diverged_ = false;

    std::map<uintptr_t, size_t> raw_blocks_;
};

Pool& pool(int dev);
inline bool valid_dev(int dev) { return dev >= 0 && dev < DEV_COUNT; }

}  // namespace slb
