// Deterministic caching allocator (see pool.hpp). Follows the policy of core/soliton/alloc.d step by step; each
// member cites the lines it answers to.
#include "pool.hpp"

#include <cstdlib>

namespace slb {

RawBackend Pool::cuda_backend;

Pool& pool(int dev) {
    static Pool pools[DEV_COUNT] = {Pool(DEV_CPU), Pool(DEV_META), Pool(DEV_CUDA)};  // alloc.d:225
    return pools[dev];
}

// alloc.d:68-86. The limit is checked against bytes already reserved, so hitting it looks like a device OOM.
void* Pool::raw_alloc(size_t n) {
    if (limit_ && reserved_ + (int64_t)n > limit_) return nullptr;
    switch (dev_) {
        case DEV_CPU: {
            void* p = nullptr;
            return posix_memalign(&p, 64, n) == 0 ? p : nullptr;
        }
        case DEV_META: {
            void* p = reinterpret_cast<void*>(meta_next_);  // a fake address; nothing ever dereferences it
            meta_next_ += n;
            return p;
        }
        default: {
            void* p = cuda_backend.alloc ? cuda_backend.alloc(n) : nullptr;
            if (p) raw_blocks_[reinterpret_cast<uintptr_t>(p)] = n;
            return p;
        }
    }
}

// alloc.d:88-94
void Pool::raw_free(void* p) {
    if (dev_ == DEV_CPU) {
        std::free(p);
    } else if (dev_ == DEV_CUDA) {
        raw_blocks_.erase(reinterpret_cast<uintptr_t>(p));
        if (cuda_backend.on_free) cuda_backend.on_free(p);
        if (cuda_backend.free) cuda_backend.free(p);
    }
}

bool Pool::find_raw(const void* p, void** base, size_t* size) const {
    const auto a = reinterpret_cast<uintptr_t>(p);
    auto it = raw_blocks_.upper_bound(a);
    if (it == raw_blocks_.begin()) return false;
    --it;
    if (a >= it->first + it->second) return false;
    *base = reinterpret_cast<void*>(it->first);
    *size = it->second;
    return true;
}

// alloc.d:98-111: the k-th allocation of a replayed run gets the k-th planned offset; any other size means the
// run left its plan, which fails (null) instead of handing out the wrong bytes.
void* Pool::arena_alloc(size_t n) {
    if (plan_cursor_ >= plan_count_ || plan_size_[plan_cursor_] != (int64_t)n) {
        diverged_ = true;
        return nullptr;
    }
    void* p = arena_ + plan_offset_[plan_cursor_++];
    count_alloc(n);
    return p;
}

// alloc.d:128-174
void* Pool::alloc(size_t n) {
    n = round_size(n);
    mix(1, n);
    if (arena_mode_) return arena_alloc(n);
    if (recording_) {
        // alloc.d:134-143: every allocation is its own block with a lifetime; the cache is bypassed so that
        // lifetimes never merge. The record index travels in the fake pointer so release() can close it.
        const size_t idx = rec_size_.size();
        rec_size_.push_back((int64_t)n);
        rec_start_.push_back((int64_t)idx);
        rec_end_.push_back(-1);
        count_alloc(n);
        return reinterpret_cast<void*>(4096 + idx * 64);
    }
    void* p = nullptr;
    for (size_t i = 0; i < cache_.size(); i++) {  // alloc.d:145-151: first exact fit; the last entry takes its place
        if (cache_[i].size == n) {
            p = cache_[i].ptr;
            cache_[i] = cache_.back();
            cache_.pop_back();
            break;
        }
    }
    if (!p) {
        p = raw_alloc(n);
        if (!p) {
            empty_cache();  // alloc.d:158-162: one flush-and-retry, exactly as a real allocator under pressure
            p = raw_alloc(n);
        }
        if (!p) return nullptr;
        reserved_ += (int64_t)n;
        n_raw_++;
        if (reserved_ > peak_reserved_) peak_reserved_ = reserved_;
    }
    count_alloc(n);
    return p;
}

// alloc.d:176-200
void Pool::release(void* p, size_t n) {
    n = round_size(n);
    mix(2, n);
    allocated_ -= (int64_t)n;
    if (arena_ && (char*)p >= arena_ && (char*)p < arena_ + arena_bytes_) {
        // An arena-backed block never enters the cache: the cache outlives the arena.
        if (!arena_mode_ && allocated_ == 0) release_arena();
        return;
    }
    if (recording_) {
        const size_t idx = (reinterpret_cast<size_t>(p) - 4096) / 64;
        if (idx < rec_size_.size()) rec_end_[idx] = (int64_t)rec_size_.size();
        return;
    }
    cache_.push_back(Cached{n, p});
}

// alloc.d:204-213
void Pool::release_arena() {
    if (!arena_) return;
    raw_free(arena_);
    reserved_ -= arena_bytes_;
    arena_ = nullptr;
    arena_bytes_ = 0;
}

// alloc.d:215-223
void Pool::empty_cache() {
    for (const Cached& b : cache_) {
        raw_free(b.ptr);
        reserved_ -= (int64_t)b.size;
    }
    cache_.clear();
}

// api.d:143-154: allocated, reserved, peak_allocated, peak_reserved, n_alloc, n_raw, trace_hash
void Pool::stats(int64_t o[7]) const {
    o[0] = allocated_, o[1] = reserved_, o[2] = peak_allocated_, o[3] = peak_reserved_;
    o[4] = n_alloc_, o[5] = n_raw_, o[6] = (int64_t)hash_;
}

// api.d:156-164
void Pool::reset_stats() {
    peak_allocated_ = allocated_;
    peak_reserved_ = reserved_;
    n_alloc_ = n_raw_ = 0;
    hash_ = kHashSeed;
}

// api.d:168-173
void Pool::record_start() {
    rec_size_.clear(), rec_start_.clear(), rec_end_.clear(), marks_.clear();
    recording_ = true;
}

// api.d:180-192: while recording a mark is a step boundary; while replaying it rewinds to the repeating body.
void Pool::record_mark() {
    if (recording_ && marks_.size() < kMaxMarks)
        marks_.push_back((int64_t)rec_size_.size());
    else if (arena_mode_)
        plan_cursor_ = plan_body_;
}

// api.d:205-215
void Pool::record_get(int64_t* size, int64_t* start, int64_t* end) const {
    for (size_t i = 0; i < rec_size_.size(); i++) size[i] = rec_size_[i], start[i] = rec_start_[i], end[i] = rec_end_[i];
}

// api.d:217-238. The plan arrays stay owned by the caller (python/soliton/arena.py:88-93 keeps them alive).
int Pool::arena_install(const int64_t* offsets, const int64_t* sizes, int64_t count, int64_t body, int64_t bytes) {
    empty_cache();
    void* a = raw_alloc((size_t)bytes);
    if (!a) return -2;
    arena_ = (char*)a;
    arena_bytes_ = bytes;
    plan_offset_ = offsets, plan_size_ = sizes;
    plan_count_ = (size_t)count, plan_body_ = (size_t)body, plan_cursor_ = 0;
    arena_mode_ = true, diverged_ = false;
    reserved_ += bytes;
    if (reserved_ > peak_reserved_) peak_reserved_ = reserved_;
    return 0;
}

// api.d:246-254
void Pool::arena_off() {
    if (!arena_mode_) return;
    arena_mode_ = false;
    if (allocated_ == 0) release_arena();
}

}  // namespace slb
