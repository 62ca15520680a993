// Host side of the data-parallel optimizer path (see dp_engine.hpp).
#include "dp_engine.hpp"

#include <cuda_runtime.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>

#include "dp_launch.h"
#include "pool.hpp"

namespace slb {

// The reference reserves a 32 MiB cuBLAS workspace from the pool when a device is initialised, on meta as on cuda
// (core/soliton/api.d:129,262-274). This library runs no GEMM, but it keeps the reservation so that its pool
// statistics line up with the reference's; the data-parallel workspace follows it the same way.
constexpr size_t kBlasWorkspace = size_t(32) << 20;
// Blocks per SM of collective launches. A constant rather than the occupancy of the kernel variant at hand:
// block b of one rank pairs with block b of its peers, so all ranks must agree on the count whatever variant
// each of them launches.
constexpr int kCollectiveBlocksPerSm = 2;

Engine& Engine::get() {
    static Engine e;
    return e;
}

static void* cuda_raw_alloc(size_t n) {
    void* p = nullptr;
    if (cudaMalloc(&p, n) != cudaSuccess) {
        cudaGetLastError();  // an out-of-memory answer is reported through the null pointer, not as a sticky error
        return Engine::retry_after_deferred_frees(n);
    }
    return p;
}
// A block that peers have mapped goes back to the driver only after they have let go of it; see collect_released.
static void cuda_raw_free(void* p) {
    if (!Engine::take_deferred_free(p)) cudaFree(p);
}

static bool aligned_vec(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31) == 0; }  // 256-bit accesses
static bool aligned4(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3) == 0; }

static void* driver_entry(const char* name) {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &f, cudaEnableDefault, &q) != cudaSuccess || !f) {
        cudaGetLastError();
        return nullptr;
    }
    return f;
}

// Base and size of the device allocation that contains p: the pool's own registry first, the driver otherwise
// (memory that did not come from sl_alloc).
static bool find_allocation(const void* p, void** base, size_t* size, bool* from_pool) {
    if (pool(DEV_CUDA).find_raw(p, base, size)) {
        *from_pool = true;
        return true;
    }
    *from_pool = false;
    typedef int (*range_fn)(unsigned long long*, size_t*, unsigned long long);
    static range_fn fn = reinterpret_cast<range_fn>(driver_entry("cuMemGetAddressRange"));
    if (!fn) return false;
    unsigned long long b = 0;
    size_t s = 0;
    if (fn(&b, &s, (unsigned long long)reinterpret_cast<uintptr_t>(p)) != 0) return false;
    *base = reinterpret_cast<void*>((uintptr_t)b);
    *size = s;
    return true;
}

// The driver's id of the allocation at p: unique per allocation for the life of the process, so a free followed by
// an allocation at the same address shows. 0 when it cannot be read.
static unsigned long long buffer_id_of(const void* p) {
    typedef int (*attr_fn)(void*, int, unsigned long long);
    static attr_fn fn = reinterpret_cast<attr_fn>(driver_entry("cuPointerGetAttribute"));
    unsigned long long id = 0;
    constexpr int kAttributeBufferId = 9;  // CU_POINTER_ATTRIBUTE_BUFFER_ID
    if (!fn || fn(&id, kAttributeBufferId, (unsigned long long)reinterpret_cast<uintptr_t>(p)) != 0) return 0;
    return id;
}

// ---------------------------------------------------------------- lanes

int Lanes::init() {
    if (ready_) return 0;
    for (int i = 0; i < COUNT; i++)
        if (cudaStreamCreateWithFlags(&streams_[i], cudaStreamNonBlocking) != cudaSuccess) return -1;
    for (int i = 0; i < COUNT; i++) open_[i].ev = nullptr;
    ready_ = true;
    return 0;
}

static void coalesce(std::vector<Range>& v) {
    std::sort(v.begin(), v.end());
    size_t out = 0;
    for (size_t i = 0; i < v.size(); i++) {
        if (v[i].hi <= v[i].lo) continue;
        if (out > 0 && v[i].lo <= v[out - 1].hi) {
            if (v[i].hi > v[out - 1].hi) v[out - 1].hi = v[i].hi;
        } else {
            v[out++] = v[i];
        }
    }
    v.resize(out);
}

// Both lists sorted by lo and free of overlaps inside themselves.
bool Lanes::overlaps(const std::vector<Range>& a, const std::vector<Range>& b) {
    size_t i = 0, j = 0;
    while (i < a.size() && j < b.size()) {
        if (a[i].hi <= b[j].lo)
            i++;
        else if (b[j].hi <= a[i].lo)
            j++;
        else
            return true;
    }
    return false;
}

cudaEvent_t Lanes::take_event() {
    if (!spare_.empty()) {
        cudaEvent_t e = spare_.back();
        spare_.pop_back();
        return e;
    }
    cudaEvent_t e = nullptr;
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    return e;
}

void Lanes::retire_finished() {
    size_t out = 0;
    for (size_t i = 0; i < pieces_.size(); i++) {
        if (cudaEventQuery(pieces_[i].ev) == cudaSuccess) {
            spare_.push_back(pieces_[i].ev);
        } else {
            if (out != i) pieces_[out] = std::move(pieces_[i]);
            out++;
        }
    }
    pieces_.resize(out);
    cudaGetLastError();  // cudaErrorNotReady from the queries is not an error
}

int Lanes::begin(int lane, cudaStream_t st, std::vector<Range>& reads, std::vector<Range>& writes) {
    coalesce(reads), coalesce(writes);
    if (pieces_.size() > 96) retire_finished();
    const Piece* latest[COUNT] = {nullptr, nullptr, nullptr};
    for (const Piece& p : pieces_) {
        if (p.lane == lane) continue;  // the same stream: ordered anyway
        if (latest[p.lane] && latest[p.lane]->seq > p.seq) continue;
        if (overlaps(writes, p.writes) || overlaps(writes, p.reads) || overlaps(reads, p.writes)) latest[p.lane] = &p;
    }
    for (int l = 0; l < COUNT; l++) {
        if (!latest[l] || latest[l]->seq <= waited_[lane][l]) continue;
        if (cudaStreamWaitEvent(st, latest[l]->ev, 0) != cudaSuccess) return -1;
        waited_[lane][l] = latest[l]->seq;
    }
    open_[lane].lane = lane;
    open_[lane].reads.swap(reads);
    open_[lane].writes.swap(writes);
    return 0;
}

int Lanes::end(int lane, cudaStream_t st) {
    Piece p;
    p.lane = lane, p.seq = ++seq_, p.ev = take_event();
    p.reads.swap(open_[lane].reads), p.writes.swap(open_[lane].writes);
    if (!p.ev || cudaEventRecord(p.ev, st) != cudaSuccess) return -1;
    pieces_.push_back(std::move(p));
    return 0;
}

// p == nullptr: everything.
int Lanes::legacy_touches(const void* p, size_t bytes, bool write) {
    if (pieces_.empty()) return 0;
    std::vector<Range> r(1);
    r[0].lo = p ? reinterpret_cast<uintptr_t>(p) : 0;
    r[0].hi = p ? r[0].lo + bytes : ~(uintptr_t)0;
    const Piece* latest[COUNT] = {nullptr, nullptr, nullptr};
    for (const Piece& q : pieces_) {
        if (latest[q.lane] && latest[q.lane]->seq > q.seq) continue;
        if (overlaps(r, q.writes) || (write && overlaps(r, q.reads))) latest[q.lane] = &q;
    }
    for (int l = 0; l < COUNT; l++) {
        if (!latest[l] || latest[l]->seq <= waited_[COUNT][l]) continue;
        if (cudaStreamWaitEvent(0, latest[l]->ev, 0) != cudaSuccess) return -1;
        waited_[COUNT][l] = latest[l]->seq;
    }
    return 0;
}

void Lanes::forget() {
    for (Piece& p : pieces_) spare_.push_back(p.ev);
    pieces_.clear();
}

int Lanes::wait_copies() {
    if (!ready_) return 0;
    const bool ok = cudaStreamSynchronize(streams_[UP]) == cudaSuccess && cudaStreamSynchronize(streams_[DOWN]) == cudaSuccess;
    retire_finished();
    return ok ? 0 : -1;
}

// ---------------------------------------------------------------- device

int Engine::device_count() {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n;
}

int Engine::bind_device(int ordinal) {
    if (cudaSetDevice(ordinal) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    ordinal_ = ordinal;
    if (cudaDeviceGetAttribute(&sm_count_, cudaDevAttrMultiProcessorCount, ordinal) != cudaSuccess) return -1;
    Pool::cuda_backend.alloc = cuda_raw_alloc;
    Pool::cuda_backend.free = cuda_raw_free;
    Pool::cuda_backend.on_free = on_raw_free;
    if (!status_host_) {
        if (cudaHostAlloc((void**)&status_host_, kMaxWorld * sizeof(int), cudaHostAllocMapped) != cudaSuccess) return -1;
        memset(status_host_, 0, kMaxWorld * sizeof(int));
        if (cudaHostGetDevicePointer((void**)&status_dev_, status_host_, 0) != cudaSuccess) return -1;
    }
    return 0;
}

int Engine::adopt_workspace(void* p, size_t n) {
    if (!p || n < kWorkspaceBytes) return -1;
    if (!status_host_) {
        int ordinal = 0;
        if (cudaGetDevice(&ordinal) != cudaSuccess || bind_device(ordinal) != 0) return -1;
    }
    if (ws_) sync();
    ws_ = static_cast<char*>(p);
    if (cudaMemset(ws_, 0, kCtlBytes) != cudaSuccess) return -1;
    resident_.clear(), resident_used_ = 0;
    fused_.valid = false;
    return 0;
}

int Engine::init_device(int dev, int ordinal) {
    if (dev == DEV_CPU) return 0;
    if (!valid_dev(dev)) return -1;
    if (dev == DEV_CUDA && bind_device(ordinal) != 0) return -1;
    void* blas = pool(dev).alloc(kBlasWorkspace);
    if (!blas) return -2;  // api.d:110 OOM code
    if (dev == DEV_CUDA) blas_ws_ = blas;
    void* ws = pool(dev).alloc(kWorkspaceBytes);
    if (!ws) return -2;
    if (dev == DEV_CUDA && adopt_workspace(ws, kWorkspaceBytes) != 0) return -1;
    return 0;
}

void Engine::clear_error() {
    err_ = 0;
    if (status_host_) memset(status_host_, 0, kMaxWorld * sizeof(int));
    cudaGetLastError();
}

void Engine::sync() {
    flush();
    if (cudaDeviceSynchronize() != cudaSuccess) set_error(ERR_SYNC);
    lanes_.forget();
    check();
}

int Engine::check() {
    if (!err_ && status_host_ && status_host_[0]) err_ = status_host_[0];
    if (!err_ && cudaPeekAtLastError() != cudaSuccess) err_ = ERR_LAUNCH;
    return err_;
}

void engine_flush_pending() {
    Engine& e = Engine::get();
    if (e.cuda_ready()) {
        e.flush();
        // the static step runs on the legacy stream: after anything a lane still does (callers of that entry point
        // do not know which tensors a lane holds, so it waits for all of them)
        e.copy_blocking(nullptr, nullptr, 0, -1);
    }
}
void engine_count_launch() { Engine::get().launches++; }

// ---------------------------------------------------------------- step builder

int Engine::hyper_index(const HyperKey& k) {
    for (size_t i = 0; i < hypers_.size(); i++)
        if (hypers_[i] == k) return (int)i;
    if (hypers_.size() >= (size_t)kMaxHyper) return -1;
    hypers_.push_back(k);
    return (int)hypers_.size() - 1;
}

void Engine::adamw(float* p, const float* g, float* m, float* v, int64_t n, float lr, float b1, float b2, float eps,
                   float wd, int step) {
    if (!cuda_ready()) return set_error(ERR_NO_WORKSPACE);
    if (n <= 0) return;
    if (!p || !g || !m || !v || !aligned4(p) || !aligned4(g) || !aligned4(m) || !aligned4(v)) return set_error(ERR_BAD_ARG);
    const HyperKey key{lr, b1, b2, eps, step};
    float gscale = 1.0f;  // an in-place scale of this gradient that is still deferred rides along with the update
    {
        auto sc = pending_scale_.find(const_cast<float*>(g));
        if (sc != pending_scale_.end()) {
            if (sc->second.first == n && !reduce_pending_) {
                gscale = sc->second.second;
                pending_scale_.erase(sc);
                sumsq_cache_.erase(std::make_pair(g, n));  // the launch rewrites this gradient
            } else {
                flush_scales();
            }
        }
    }
    if (reduce_pending_) {
        auto it = by_grad_.find(g);
        if (it != by_grad_.end() && !items_[it->second].p && items_[it->second].n == n) {
            const int hi = hyper_index(key);
            if (hi >= 0) {
                StepItem& s = items_[it->second];
                s.p = p, s.m = m, s.v = v, s.wd = wd, s.hyper = hi;
                if (++attached_ == (int)items_.size() || opt.eager) flush_step();
                return;
            }
        }
        flush_step();  // this update is not part of the pending all-reduce: finish that first
    }
    if (in_group_) return set_error(ERR_BAD_ARG);  // an optimizer step inside an open group has no defined order
    if (params_in_batch_.count(p) || items_.size() >= (size_t)kMaxSegs) flush_step();
    int hi = hyper_index(key);
    if (hi < 0) {
        flush_step();
        hi = hyper_index(key);
    }
    StepItem s;
    s.g = const_cast<float*>(g), s.p = p, s.m = m, s.v = v, s.n = n, s.wd = wd, s.hyper = hi, s.gscale = gscale;
    items_.push_back(s);
    params_in_batch_.insert(p);
    if (opt.eager) flush_step();
}

int Engine::group(int start) {
    if (!cuda_ready() || !rdv_.is_open()) return -1;
    if (start) {
        flush();
        in_group_ = true;
        return 0;
    }
    if (!in_group_) return -1;
    in_group_ = false;
    if (items_.empty()) return 0;
    if (world_ == 1) {  // the mean over one rank is the gradient itself
        items_.clear(), by_grad_.clear();
        return 0;
    }
    if (exchange() != 0) {
        items_.clear(), by_grad_.clear();
        return -1;
    }
    reduce_pending_ = true;
    attached_ = 0;
    sumsq_plan_.clear();  // a clip of this step asks for the sum of squares of exactly these gradients
    for (const StepItem& it : items_) sumsq_plan_.push_back(TensorRef{it.g, it.n});
    if (opt.eager) flush_step();
    return 0;
}

int Engine::allreduce_mean(float* g, int64_t n) {
    if (!cuda_ready() || !rdv_.is_open()) return -1;
    if (n < 0 || (n > 0 && (!g || !aligned4(g)))) return -1;
    if (!in_group_) {  // a bare call is a group of one
        if (group(1) != 0) return -1;
        const int rc = allreduce_mean(g, n);
        return group(0) != 0 ? -1 : rc;
    }
    if (n == 0) return 0;
    if (items_.size() >= (size_t)kMaxSegs || by_grad_.count(g)) return -1;
    StepItem s;
    s.g = g, s.n = n;
    by_grad_[g] = (int)items_.size();
    items_.push_back(s);
    return 0;
}

void Engine::flush_step() {
    if (in_group_) return;  // an open group has nothing that may be launched yet
    if (!items_.empty()) {
        const int rc = launch_items(items_, hypers_, reduce_pending_);
        if (rc) set_error(rc);
    }
    items_.clear(), hypers_.clear(), by_grad_.clear(), params_in_batch_.clear();
    reduce_pending_ = false;
    attached_ = 0;
}

// Everything deferred goes out: the pending step, in-place scales that no AdamW call picked up. What was learned
// about this clip's sumsq calls becomes the plan for the next one; cached sums die, memory may change from here on.
void Engine::flush() {
    flush_step();
    flush_scales();
    if (!sumsq_learn_.empty()) {
        sumsq_history_.insert(sumsq_history_.begin(), std::vector<TensorRef>());
        sumsq_history_.front().swap(sumsq_learn_);
        if (sumsq_history_.size() > 3) sumsq_history_.pop_back();
    }
    sumsq_cache_.clear();
    fused_.valid = false;
}

void Engine::flush_scales() {
    for (auto& kv : pending_scale_) {
        lanes_.legacy_touches(kv.first, (size_t)kv.second.first * 4, true);
        if (launch_scale(kv.first, kv.first, kv.second.first, kv.second.second, 0)) set_error(ERR_LAUNCH);
        launches++, legacy_epoch_++;
    }
    pending_scale_.clear();
}

static void fill_hyper(Hyper& h, const HyperKey& k) {
    // core/cuda/kernels.cu:253: 1.0 - pow(b, step) with both arguments promoted to double
    h.bc1 = 1.0 - std::pow((double)k.b1, (double)k.step);
    h.bc2 = 1.0 - std::pow((double)k.b2, (double)k.step);
    h.rbc1 = 1.0 / h.bc1, h.rbc2 = 1.0 / h.bc2;
    h.lr = k.lr, h.b1 = k.b1, h.b2 = k.b2, h.eps = k.eps;
    h.c1 = 1 - k.b1, h.c2 = 1 - k.b2;
}

// Builds the segment table of a step. Returns the tile total or -1.
static int64_t build_table(const std::vector<StepItem>& items, int world, int rank, const std::vector<float*>* peer_g,
                           std::vector<Seg>& segs, std::vector<int>& prefix, bool* any_adam) {
    const size_t nseg = items.size();
    segs.assign(nseg, Seg{});
    prefix.assign(nseg + 1, 0);
    int64_t tiles = 0;
    *any_adam = false;
    for (size_t s = 0; s < nseg; s++) {
        const StepItem& it = items[s];
        Seg& d = segs[s];
        d.p = it.p, d.m = it.m, d.v = it.v, d.n = it.n, d.wd = it.wd, d.hyper = it.hyper, d.gscale = it.gscale;
        bool vec = aligned_vec(it.g) && (!it.p || (aligned_vec(it.p) && aligned_vec(it.m) && aligned_vec(it.v)));
        for (int r = 0; r < world; r++) {
            d.g[r] = (world == 1 || r == rank) ? it.g : peer_g[r][s];
            vec = vec && aligned_vec(d.g[r]);
        }
        d.vec = vec ? 1 : 0;
        if (it.p) *any_adam = true;
        prefix[s] = (int)tiles;
        tiles += (it.n + kTile - 1) / kTile;
        if (tiles > 0x7fffffff) return -1;
    }
    prefix[nseg] = (int)tiles;
    return tiles;
}

// Capacity of one (parity, source rank) staging slot: the staging area holds 2 x world of them. Whole tiles, so
// that every slot starts 16-byte aligned whatever the world size.
static int stage_slot_floats(int world) {
    const size_t raw = kStageBytes / 4 / (2 * (size_t)(world > 1 ? world : 1));
    return (int)(raw / kTile * kTile);
}

static int min_chunk(int T, int world) {
    int best = T;
    for (int c = 0; c < world; c++) {
        const int len = (int)((int64_t)T * (c + 1) / world) - (int)((int64_t)T * c / world);
        if (len < best) best = len;
    }
    return best;
}

// A step's tables live in the workspace's table area, one image each: [rank context][tile prefix][segments]. A
// training loop repeats the same few steps (one per bucket), so an image is uploaded when it is first seen and found
// again by content afterwards; when the area is full everything is dropped and uploaded anew. Uploads and the
// launches that read the tables are on the same stream, so an image is never overwritten under a running kernel.
const RankCtx* Engine::resident_tables(const RankCtx& ctx, const std::vector<Seg>& segs, const std::vector<int>& prefix,
                                       cudaStream_t st) {
    const size_t prefix_bytes = (prefix.size() * sizeof(int) + 15) & ~size_t(15);
    const size_t bytes = sizeof(RankCtx) + prefix_bytes + segs.size() * sizeof(Seg);
    if (bytes > kTableBytes) return nullptr;
    std::vector<unsigned char> image(bytes, 0);
    memcpy(image.data(), &ctx, sizeof ctx);  // its two table pointers are still null: the key does not depend on the place
    memcpy(image.data() + sizeof(RankCtx), prefix.data(), prefix.size() * sizeof(int));
    memcpy(image.data() + sizeof(RankCtx) + prefix_bytes, segs.data(), segs.size() * sizeof(Seg));
    static cudaStream_t last_stream = nullptr;
    if (st != last_stream) {  // launches moved to another stream: the old one may still read what is resident
        if (!resident_.empty()) cudaStreamSynchronize(last_stream);
        resident_.clear(), resident_used_ = 0;
        last_stream = st;
    }
    for (const Resident& r : resident_)
        if (r.image.size() == bytes && memcmp(r.image.data(), image.data(), bytes) == 0)
            return reinterpret_cast<const RankCtx*>(ws_ + kTableOff + r.offset);
    if (resident_used_ + bytes > kTableBytes || resident_.size() >= 64) resident_.clear(), resident_used_ = 0;
    Resident r;
    r.offset = resident_used_;
    char* at = ws_ + kTableOff + r.offset;
    std::vector<unsigned char> placed = image;
    RankCtx* pc = reinterpret_cast<RankCtx*>(placed.data());
    pc->tile_prefix = reinterpret_cast<const int*>(at + sizeof(RankCtx));
    pc->segs = reinterpret_cast<const Seg*>(at + sizeof(RankCtx) + prefix_bytes);
    if (cudaMemcpyAsync(at, placed.data(), bytes, cudaMemcpyHostToDevice, st) != cudaSuccess) return nullptr;
    r.image.swap(image);
    resident_.push_back(std::move(r));
    resident_used_ += (bytes + 255) & ~size_t(255);
    return reinterpret_cast<const RankCtx*>(at);
}

int Engine::launch_items(std::vector<StepItem>& items, const std::vector<HyperKey>& hypers, bool collective) {
    const int W = collective ? world_ : 1;
    const int me = collective ? rank_ : 0;
    std::vector<Seg> segs;
    std::vector<int> prefix;
    bool adam = false;
    const int64_t T = build_table(items, W, me, peer_g_, segs, prefix, &adam);
    if (T < 0) return ERR_BAD_ARG;
    const int nseg = (int)items.size();

    const int slot_floats = stage_slot_floats(W);
    bool oneshot = false;
    if (W > 1) {
        const bool fits = T * kTile <= slot_floats;
        const bool small = opt.oneshot_max_bytes < 0 || T * kTile * 4 <= opt.oneshot_max_bytes;
        oneshot = fits && (opt.mode == 1 || (opt.mode == 0 && small));
    }
    const int kind = oneshot ? KERNEL_ONESHOT : KERNEL_PLAIN;
    const size_t smem = (size_t)(nseg + 1) * sizeof(int);
    int per_sm;
    if (W > 1) {
        per_sm = kCollectiveBlocksPerSm;
        if (opt.blocks_per_sm > 0 && opt.blocks_per_sm < per_sm) per_sm = opt.blocks_per_sm;
        if (step_occupancy(W, adam, kind, smem) < per_sm) return ERR_LAUNCH;
    } else {
        per_sm = step_occupancy(W, adam, kind, smem);
        if (opt.blocks_per_sm > 0 && opt.blocks_per_sm < per_sm) per_sm = opt.blocks_per_sm;
        if (per_sm < 1) return ERR_LAUNCH;
    }
    int cap = per_sm * sm_count_;
    if (cap > kFlagBlocks) cap = kFlagBlocks;
    const int work = (W == 1 || oneshot) ? (int)T : min_chunk((int)T, W);
    const int G = work < 1 ? 1 : (work < cap ? work : cap);

    // Which stream, and what has to come first on it.
    if (opt.overlap && lanes_.init() != 0) return ERR_LAUNCH;
    const cudaStream_t st = lanes_.stream(Lanes::STEP, opt.overlap != 0);
    const bool tracked = lanes_.ready();  // from the first use of another stream on, every launch leaves an event
    if (!tracked) legacy_epoch_++;
    if (tracked) {
        std::vector<Range> reads, writes;
        for (const StepItem& it : items) {
            const uintptr_t g = reinterpret_cast<uintptr_t>(it.g), bytes = (uintptr_t)it.n * 4;
            (W > 1 || it.gscale != 1.0f ? writes : reads).push_back(Range{g, g + bytes});
            if (it.p) {
                for (float* q : {it.p, it.m, it.v}) writes.push_back(Range{reinterpret_cast<uintptr_t>(q), reinterpret_cast<uintptr_t>(q) + bytes});
            }
        }
        if (lanes_.begin(Lanes::STEP, st, reads, writes) != 0) return ERR_LAUNCH;
        if (after_legacy(Lanes::STEP, st) != 0) return ERR_LAUNCH;
    }

    RankCtx ctx{};
    ctx.nseg = nseg, ctx.rank = me, ctx.world = W;
    for (int r = 0; r < W; r++) {
        char* base = (W == 1 || r == me) ? ws_ : peer_ws_[r];
        ctx.flags[r] = reinterpret_cast<unsigned*>(base + kFlagOff);
        ctx.stage[r] = reinterpret_cast<float*>(base + kCtlBytes);
    }
    ctx.status = status_dev_;
    ctx.stamps = (opt.stamps && W > 1) ? reinterpret_cast<unsigned long long*>(ws_ + kStampOff) : nullptr;
    const RankCtx* d_ctx = resident_tables(ctx, segs, prefix, st);
    if (!d_ctx) return ERR_LAUNCH;

    LaunchArgs a{};
    a.ctxs = d_ctx;
    a.blocks_per_rank = G;
    a.seq = W > 1 ? ++seq_ : 0;
    a.parity = oneshot ? (oneshots_++ & 1) : 0;
    a.stage_slot_floats = slot_floats;
    a.timeout_ns = opt.timeout_ns;
    a.inv_world = 1.0f / (float)W;
    a.sumsq_on = (W > 1 && !adam && !oneshot && T <= kMaxPieceTiles) ? 1 : 0;
    a.cyclic = opt.cyclic;
    for (size_t i = 0; i < hypers.size() && i < (size_t)kMaxHyper; i++) fill_hyper(a.hp[i], hypers[i]);
    last_mode = W == 1 ? 0 : (oneshot ? 1 : 2);
    last_blocks = G;
    launches++;
    const int rc = launch_step(W, adam, kind, false, G, smem, a, st);
    if (tracked && lanes_.end(Lanes::STEP, st) != 0) return ERR_LAUNCH;
    if (W > 1) fused_.valid = false;  // any collective launch reuses the staging area
    if (rc == 0 && a.sumsq_on) {
        fused_.valid = true, fused_.world = W, fused_.blocks = G, fused_.prefix = prefix;
        fused_.tensors.clear();
        for (const StepItem& it : items) fused_.tensors.push_back(TensorRef{it.g, it.n});
    }
    return rc == 0 ? 0 : ERR_LAUNCH;
}

// ---------------------------------------------------------------- process group

// Life cycle of gradient memory that peers map (CUDA IPC). The owner publishes an allocation in a slot of its
// export table; peers open the handle when a gradient table first names the slot. When the owner's allocator gives
// the block back, the owner marks the slot freed and KEEPS the allocation: returning it to the driver while a peer
// still has it open is undefined. At their next collective the peers close their mappings of freed slots and
// acknowledge; once every peer has, the owner calls cudaFree and the slot can describe another allocation.
// Memory that is not the pool's cannot be kept alive this way: it is recognised again by the driver's buffer id,
// and its owner must keep it allocated until the collective after the last one that used it has begun.

void Engine::on_raw_free(void* base) {
    Engine& e = get();
    e.sumsq_plan_.clear(), e.sumsq_learn_.clear(), e.sumsq_history_.clear();  // remembered addresses may die with this block
    auto it = e.export_ids_.find(base);
    if (it == e.export_ids_.end()) return;
    if (e.rdv_.is_open()) {
        e.rdv_.mark_freed((uint32_t)it->second.id);
        e.pending_free_.push_back(PendingFree{base, (uint32_t)it->second.id});
        e.deferred_.insert(base);
    }
    e.export_ids_.erase(it);
}

bool Engine::take_deferred_free(void* base) { return get().deferred_.count(base) != 0; }

void* Engine::retry_after_deferred_frees(size_t n) {
    Engine& e = get();
    if (e.pending_free_.empty()) return nullptr;
    e.collect_released(false);
    void* p = nullptr;
    if (cudaMalloc(&p, n) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return p;
}

void Engine::collect_released(bool force) {
    size_t out = 0;
    for (size_t i = 0; i < pending_free_.size(); i++) {
        const PendingFree f = pending_free_[i];
        if (force || rdv_.released_by_all(f.id)) {
            if (f.base) {
                deferred_.erase(f.base);
                cudaFree(f.base);
            }
            if (!force) rdv_.recycle(f.id);
        } else {
            pending_free_[out++] = f;
        }
    }
    pending_free_.resize(out);
}

int Engine::export_id_for(void* base, size_t size, bool from_pool) {
    auto it = export_ids_.find(base);
    if (it != export_ids_.end()) {
        if (from_pool) return it->second.id;  // the pool tells when its blocks die (on_raw_free)
        if (it->second.buffer_id != 0 && it->second.buffer_id == buffer_id_of(base) && it->second.size == size) return it->second.id;
        // another allocation now sits at this address: retire the slot of the one that is gone
        rdv_.mark_freed((uint32_t)it->second.id);
        pending_free_.push_back(PendingFree{nullptr, (uint32_t)it->second.id});
        export_ids_.erase(it);
    }
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, base) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    static_assert(sizeof(h) == 64, "IPC handle size");
    const int id = rdv_.add_export(reinterpret_cast<unsigned char*>(&h), size);
    if (id >= 0) export_ids_[base] = Exported{id, from_pool, from_pool ? 0ull : buffer_id_of(base), size};
    return id;
}

int Engine::dist_unique_id(char* out) { return out ? Rendezvous::create_id(out) : -1; }

int Engine::dist_init(int rank, int world, const char* id) {
    if (!cuda_ready() || rdv_.is_open() || !id) return -1;
    sync();
    if (rdv_.open(id, rank, world, opt.host_timeout_s) != 0) return -1;
    rank_ = rank, world_ = world, seq_ = 0, collectives_ = 0, oneshots_ = 0;
    resident_.clear(), resident_used_ = 0;
    for (int r = 0; r < kMaxWorld; r++) peer_ws_[r] = nullptr, peer_version_[r] = 0, peer_free_epoch_[r] = 0, peer_g_[r].clear();
    bool ok = cudaMemset(ws_ + kFlagOff, 0, kFlagBytes) == cudaSuccess && cudaDeviceSynchronize() == cudaSuccess;
    RdvRank& me = rdv_.self();
    me.ordinal = ordinal_, me.sm_count = sm_count_, me.pid = (int)getpid();
    if (ok && world > 1) {
        void* base = nullptr;
        size_t size = 0;
        bool from_pool = false;
        cudaIpcMemHandle_t h;
        ok = find_allocation(ws_, &base, &size, &from_pool) && cudaIpcGetMemHandle(&h, base) == cudaSuccess;
        if (ok) {
            memcpy(me.ws_handle, &h, 64);
            me.ws_offset = (uint64_t)(ws_ - static_cast<char*>(base));
        }
    }
    if (!ok) rdv_.fail();
    ok = ok && rdv_.stage_barrier(1, opt.host_timeout_s) == 0;
    peer_ws_[rank] = ws_;
    for (int r = 0; ok && r < world; r++) {
        if (r == rank) continue;
        RdvRank& p = rdv_.peer(r);
        int can = 0;
        ok = p.sm_count == sm_count_ && cudaDeviceCanAccessPeer(&can, ordinal_, p.ordinal) == cudaSuccess && can;
        if (!ok) break;
        cudaIpcMemHandle_t h;
        memcpy(&h, p.ws_handle, 64);
        void* base = nullptr;
        ok = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess) == cudaSuccess;
        if (ok) peer_ws_[r] = static_cast<char*>(base) + p.ws_offset;
    }
    if (!ok) rdv_.fail();
    ok = ok && rdv_.stage_barrier(2, opt.host_timeout_s) == 0;
    if (ok) rdv_.unlink_now();  // everybody has the file mapped: its name is not needed any more
    if (!ok) {
        cudaGetLastError();
        close_peer_maps();
        rdv_.close();
        rank_ = 0, world_ = 1;
        return -1;
    }
    return 0;
}

void Engine::close_peer_maps() {
    for (int r = 0; r < kMaxWorld; r++) {
        for (auto& kv : peer_open_[r]) cudaIpcCloseMemHandle(kv.second.base);
        peer_open_[r].clear();
        peer_g_[r].clear();
        peer_version_[r] = 0;
        if (r != rank_ && peer_ws_[r]) cudaIpcCloseMemHandle(peer_ws_[r] - rdv_.peer(r).ws_offset);
        peer_ws_[r] = nullptr;
    }
    cudaGetLastError();
}

void Engine::dist_destroy() {
    if (!rdv_.is_open()) return;
    in_group_ = false;
    sync();
    rdv_.stage_barrier(3, 10.0);  // every rank's kernels are done before any mapping goes away
    close_peer_maps();
    rdv_.stage_barrier(4, 10.0);  // every rank has closed its mappings before any exported block goes to the driver
    collect_released(true);
    export_ids_.clear();
    rdv_.close();
    rank_ = 0, world_ = 1;
    resident_.clear(), resident_used_ = 0;
    fused_.valid = false;
}

// Closes this rank's mappings of the allocations rank r wants back, and tells r.
void Engine::let_go_of_freed(int r) {
    RdvRank& pr = rdv_.peer(r);
    const uint32_t epoch = pr.free_epoch.load(std::memory_order_acquire);
    if (epoch == peer_free_epoch_[r]) return;
    peer_free_epoch_[r] = epoch;
    const uint32_t mine = 1u << rank_;
    const uint32_t n = pr.n_exports.load(std::memory_order_acquire);
    bool closed_any = false;
    for (uint32_t id = 0; id < n; id++) {
        if (!pr.exports[id].freed.load(std::memory_order_acquire)) continue;
        if (pr.exports[id].acks.load(std::memory_order_acquire) & mine) continue;
        auto it = peer_open_[r].find(id);
        if (it != peer_open_[r].end()) {
            cudaIpcCloseMemHandle(it->second.base);
            peer_open_[r].erase(it);
            closed_any = true;
        }
        rdv_.ack_freed(r, id);
    }
    if (closed_any) peer_version_[r] = 0, peer_g_[r].clear();  // pointers into closed mappings must not survive
    cudaGetLastError();
}

int Engine::exchange() {
    const uint32_t nseg = (uint32_t)items_.size();
    my_table_.resize(nseg);
    for (uint32_t s = 0; s < nseg; s++) {
        void* base = nullptr;
        size_t size = 0;
        bool from_pool = false;
        if (!find_allocation(items_[s].g, &base, &size, &from_pool)) return -1;
        const uint64_t off = (uint64_t)(reinterpret_cast<char*>(items_[s].g) - static_cast<char*>(base));
        if (off + (uint64_t)items_[s].n * 4 > size) return -1;
        const int id = export_id_for(base, size, from_pool);
        if (id < 0) return -1;
        my_table_[s].export_id = (uint32_t)id, my_table_[s].generation = rdv_.generation_of((uint32_t)id);
        my_table_[s].offset = off, my_table_[s].n = items_[s].n;
    }
    const uint64_t k = ++collectives_;
    if (rdv_.arrive(k, my_table_.data(), nseg, opt.host_timeout_s) != 0) {
        rdv_.fail();
        return -1;
    }
    for (int r = 0; r < world_; r++) {
        if (r == rank_) continue;
        let_go_of_freed(r);
        uint32_t n2 = 0;
        uint64_t ver = 0;
        const RdvSegment* t = rdv_.table_of(r, k, &n2, &ver);
        for (uint32_t s = 0; s < nseg; s++)
            if (t[s].n != items_[s].n) return -1;  // the ranks disagree about the tensors of this step
        if (ver == peer_version_[r] && peer_g_[r].size() == nseg) continue;
        RdvRank& pr = rdv_.peer(r);
        peer_g_[r].assign(nseg, nullptr);
        for (uint32_t s = 0; s < nseg; s++) {
            const uint32_t id = t[s].export_id;
            if (id >= pr.n_exports.load(std::memory_order_acquire)) return -1;
            auto it = peer_open_[r].find(id);
            if (it != peer_open_[r].end() && it->second.generation != t[s].generation) {  // the slot describes another allocation now
                cudaIpcCloseMemHandle(it->second.base);
                peer_open_[r].erase(it);
                it = peer_open_[r].end();
            }
            void* base = nullptr;
            if (it != peer_open_[r].end()) {
                base = it->second.base;
            } else {
                cudaIpcMemHandle_t h;
                memcpy(&h, pr.exports[id].handle, 64);
                if (cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                    cudaGetLastError();
                    return -1;
                }
                peer_open_[r][id] = PeerMap{base, t[s].generation};
            }
            if (t[s].offset + (uint64_t)t[s].n * 4 > pr.exports[id].size) return -1;
            peer_g_[r][s] = reinterpret_cast<float*>(static_cast<char*>(base) + t[s].offset);
        }
        peer_version_[r] = ver;
    }
    if (!pending_free_.empty()) collect_released(false);
    return 0;
}

// ---------------------------------------------------------------- copies and streams beside the path

void Engine::copy_blocking(void* dst, const void* src, size_t n, int kind) {
    flush();
    if (kind < 0) {  // no copy: only the ordering against the lanes, for everything
        lanes_.legacy_touches(nullptr, 0, true);
        return;
    }
    if (kind == cudaMemcpyHostToDevice || kind == cudaMemcpyDeviceToDevice) lanes_.legacy_touches(dst, n, true);
    if (kind == cudaMemcpyDeviceToHost || kind == cudaMemcpyDeviceToDevice) lanes_.legacy_touches(src, n, false);
    if (cudaMemcpy(dst, src, n, (cudaMemcpyKind)kind) != cudaSuccess) set_error(ERR_SYNC);
    if (kind != cudaMemcpyDeviceToHost) legacy_epoch_++;  // an upload from pageable memory may return before its DMA ends
}

void Engine::before_release(const void* p, size_t n) {
    flush();
    lanes_.legacy_touches(p, n, true);
}

// Work on the legacy stream is not remembered piece by piece. With the "overlap" option the caller keeps launching
// there (backward), so every piece of lane work waits for the legacy stream as it is at that moment. Without it, only
// what this library itself has put on the legacy stream since the lane last looked can matter (fills, scales, sums,
// blocking uploads whose DMA may still run); a lane that has seen it all does not wait again. Kernels a caller
// launches on the legacy stream by other means are not covered without "overlap".
int Engine::after_legacy(int lane, cudaStream_t st) {
    if (st == (cudaStream_t)0) return 0;
    if (!opt.overlap && lane_seen_epoch_[lane] == legacy_epoch_) return 0;
    lane_seen_epoch_[lane] = legacy_epoch_;
    if (!legacy_ev_ && cudaEventCreateWithFlags(&legacy_ev_, cudaEventDisableTiming) != cudaSuccess) return -1;
    return cudaEventRecord(legacy_ev_, 0) == cudaSuccess && cudaStreamWaitEvent(st, legacy_ev_, 0) == cudaSuccess ? 0 : -1;
}

int Engine::from_host_async(int k, void* const* dst, const void* const* src, const size_t* bytes) {
    if (!cuda_ready() || k < 0 || (k > 0 && (!dst || !src || !bytes))) return -1;
    flush();
    if (lanes_.init() != 0) return -1;
    const cudaStream_t st = lanes_.stream(Lanes::UP, true);
    std::vector<Range> reads, writes;
    for (int i = 0; i < k; i++) writes.push_back(Range{reinterpret_cast<uintptr_t>(dst[i]), reinterpret_cast<uintptr_t>(dst[i]) + bytes[i]});
    if (lanes_.begin(Lanes::UP, st, reads, writes) != 0 || after_legacy(Lanes::UP, st) != 0) return -1;
    bool ok = true;
    for (int i = 0; i < k && ok; i++)
        ok = bytes[i] == 0 || cudaMemcpyAsync(dst[i], src[i], bytes[i], cudaMemcpyHostToDevice, st) == cudaSuccess;
    return lanes_.end(Lanes::UP, st) == 0 && ok ? 0 : -1;
}

int Engine::to_host_async(int k, void* const* dst, const void* const* src, const size_t* bytes) {
    if (!cuda_ready() || k < 0 || (k > 0 && (!dst || !src || !bytes))) return -1;
    flush();
    if (lanes_.init() != 0) return -1;
    const cudaStream_t st = lanes_.stream(Lanes::DOWN, true);
    std::vector<Range> reads, writes;
    for (int i = 0; i < k; i++) reads.push_back(Range{reinterpret_cast<uintptr_t>(src[i]), reinterpret_cast<uintptr_t>(src[i]) + bytes[i]});
    if (lanes_.begin(Lanes::DOWN, st, reads, writes) != 0 || after_legacy(Lanes::DOWN, st) != 0) return -1;
    bool ok = true;
    for (int i = 0; i < k && ok; i++)
        ok = bytes[i] == 0 || cudaMemcpyAsync(dst[i], src[i], bytes[i], cudaMemcpyDeviceToHost, st) == cudaSuccess;
    return lanes_.end(Lanes::DOWN, st) == 0 && ok ? 0 : -1;
}

int Engine::wait_copies() {
    flush();
    const int rc = lanes_.wait_copies();
    check();
    return rc;
}

int Engine::read_stamps(unsigned long long* out) {
    if (!cuda_ready() || !out) return -1;
    sync();
    return cudaMemcpy(out, ws_ + kStampOff, kStamps * sizeof(unsigned long long), cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : -1;
}

// ---------------------------------------------------------------- next to the path

void Engine::scale(const float* x, float* y, int64_t n, float alpha) {
    if (!cuda_ready()) return set_error(ERR_NO_WORKSPACE);
    if (n > 0 && (!x || !y)) return set_error(ERR_BAD_ARG);
    if (n <= 0) return;
    if (x == y && !opt.eager) {
        // In place (gradient clipping): remembered, and applied by the AdamW launch that consumes this gradient, or
        // by a plain scale launch at the next point where anything could look at the memory.
        flush_step();
        if (pending_scale_.count(y)) flush_scales();
        sumsq_cache_.clear();
        pending_scale_[y] = std::make_pair(n, alpha);
        return;
    }
    flush();
    lanes_.legacy_touches(x, (size_t)n * 4, false), lanes_.legacy_touches(y, (size_t)n * 4, true);
    if (launch_scale(x, y, n, alpha, 0)) set_error(ERR_LAUNCH);
    launches++, legacy_epoch_++;
}
void Engine::axpy(const float* x, float* y, int64_t n, float alpha) {
    if (!cuda_ready()) return set_error(ERR_NO_WORKSPACE);
    flush();
    if (n > 0 && (!x || !y)) return set_error(ERR_BAD_ARG);
    if (n > 0) lanes_.legacy_touches(x, (size_t)n * 4, false), lanes_.legacy_touches(y, (size_t)n * 4, true);
    if (launch_axpy(x, y, n, alpha, 0)) set_error(ERR_LAUNCH);
    launches += n > 0, legacy_epoch_++;
}
void Engine::fill(float* p, int64_t n, float v) {
    if (!cuda_ready()) return set_error(ERR_NO_WORKSPACE);
    flush();
    if (n > 0 && !p) return set_error(ERR_BAD_ARG);
    if (n > 0) lanes_.legacy_touches(p, (size_t)n * 4, true);
    if (launch_fill(p, n, v, 0)) set_error(ERR_LAUNCH);
    launches += n > 0, legacy_epoch_++;
}

// One launch for the sum of squares of every tensor in `plan`; results land in sumsq_cache_.
bool Engine::sumsq_batch(const std::vector<TensorRef>& plan) {
    std::vector<SumsqSlice> slices;
    for (const TensorRef& t : plan)
        for (int64_t off = 0; off < t.n; off += kSumsqSlice)
            slices.push_back(SumsqSlice{t.x + off, t.n - off < kSumsqSlice ? t.n - off : (int64_t)kSumsqSlice});
    if (slices.empty() || slices.size() > (size_t)kMaxSumsqSlices) return false;
    SumsqSlice* d_slices = reinterpret_cast<SumsqSlice*>(ws_ + kSliceTableOff);
    double* d_part = reinterpret_cast<double*>(ws_ + kSlicePartialOff);
    if (slices.size() != dev_slices_.size() || memcmp(slices.data(), dev_slices_.data(), slices.size() * sizeof(SumsqSlice)) != 0) {
        if (cudaMemcpyAsync(d_slices, slices.data(), slices.size() * sizeof(SumsqSlice), cudaMemcpyHostToDevice, 0) != cudaSuccess) return false;
        dev_slices_ = slices;
    }
    if (launch_sumsq_slices((int)slices.size(), d_slices, d_part, sm_count_ * 8, 0)) {
        set_error(ERR_LAUNCH);
        return false;
    }
    launches++;
    std::vector<double> h(slices.size());
    if (cudaMemcpy(h.data(), d_part, h.size() * sizeof(double), cudaMemcpyDeviceToHost) != cudaSuccess) {
        set_error(ERR_SYNC);
        return false;
    }
    size_t i = 0;
    for (const TensorRef& t : plan) {
        double sum = 0;
        for (int64_t off = 0; off < t.n; off += kSumsqSlice) sum += h[i++];  // slice order: reproducible
        sumsq_cache_[std::make_pair(t.x, t.n)] = sum;
    }
    return true;
}

void combine_pieces(const double* table, const std::vector<int>& prefix, int world, int blocks, double* out) {
    const int nseg = (int)prefix.size() - 1;
    const int T = prefix[nseg];
    std::vector<int> starts;
    for (int c = 0; c < world; c++) {
        const int cb = (int)((int64_t)T * c / world), L = (int)((int64_t)T * (c + 1) / world) - cb;
        for (int b = 0; b < blocks; b++) {
            const int r0 = cb + (int)((int64_t)L * b / blocks), r1 = cb + (int)((int64_t)L * (b + 1) / blocks);
            if (r1 > r0) starts.push_back(r0);
        }
    }
    for (int s = 0; s < nseg; s++)
        if (prefix[s + 1] > prefix[s]) starts.push_back(prefix[s]);
    std::sort(starts.begin(), starts.end());
    starts.erase(std::unique(starts.begin(), starts.end()), starts.end());
    for (int s = 0; s < nseg; s++) out[s] = 0;
    int s = 0;
    for (int t : starts) {  // ascending: a tensor's pieces are added in tile order
        while (s + 1 < nseg && prefix[s + 1] <= t) s++;
        out[s] += table[t];
    }
}

// The two-shot mean that just ran left, in the staging area, the sum of squares of every piece of the mean. Reads
// them and fills the cache with the sums of all tensors of that launch.
bool Engine::harvest_fused_sumsq() {
    if (!fused_.valid) return false;
    fused_.valid = false;
    const int nseg = (int)fused_.tensors.size();
    const int T = fused_.prefix[nseg];
    std::vector<double> table((size_t)T);
    lanes_.legacy_touches(nullptr, 0, true);
    if (cudaMemcpy(table.data(), ws_ + kCtlBytes, table.size() * sizeof(double), cudaMemcpyDeviceToHost) != cudaSuccess) {
        set_error(ERR_SYNC);
        return false;
    }
    std::vector<double> sums((size_t)nseg);
    combine_pieces(table.data(), fused_.prefix, fused_.world, fused_.blocks, sums.data());
    for (int s = 0; s < nseg; s++) sumsq_cache_[std::make_pair(fused_.tensors[s].x, fused_.tensors[s].n)] = sums[s];
    return true;
}

// Sum of squares of a tensor (the reference: cublasSdot, core/cuda/kernels.cu:219-224, blocking). Fixed slices and
// a fixed combination order make the value reproducible run to run; double partials make it at least as accurate
// as the float dot it stands in for. Soliton's clip asks tensor by tensor (python/soliton/optim.py:34). When the
// gradients were just averaged by a two-shot launch, that launch has already summed the squares of the mean it
// produced, and all questions are answered from what it left behind. Otherwise the first question is answered by
// summing every tensor the clip is expected to ask about -- the gradients of the group that was just reduced, else
// the tensors of the previous clips -- in one launch, the rest from that launch.
double Engine::sumsq(const float* x, int64_t n) {
    if (!cuda_ready()) {
        set_error(ERR_NO_WORKSPACE);
        return NAN;
    }
    flush_step();
    if (!pending_scale_.empty()) {
        flush_scales();
        sumsq_cache_.clear();
        fused_.valid = false;
    }
    if (n <= 0) return 0.0;
    if (!x) {
        set_error(ERR_BAD_ARG);
        return NAN;
    }
    sumsq_learn_.push_back(TensorRef{x, n});
    if (fused_.valid) harvest_fused_sumsq();
    auto hit = sumsq_cache_.find(std::make_pair(x, n));
    if (hit != sumsq_cache_.end()) return hit->second;
    lanes_.legacy_touches(nullptr, 0, false);
    // Known from the group that was just reduced or from one of the last few clips? Then sum everything those lists
    // name (their union: equal-sized blocks can swap places from step to step, which shows up as the same address
    // with another length). A stale entry costs a little arithmetic; its sum is that of the memory as it is now.
    bool known = false;
    std::vector<TensorRef> plan;
    auto add_list = [&](const std::vector<TensorRef>& list) {
        for (const TensorRef& t : list) {
            known = known || (t.x == x && t.n == n);
            bool dup = false;
            for (const TensorRef& q : plan) dup = dup || (q.x == t.x && q.n == t.n);
            void* base;
            size_t size;
            // only tensors inside the pool's own blocks: readable until a raw block is freed, which clears the lists
            if (!dup && pool(DEV_CUDA).find_raw(t.x, &base, &size) &&
                reinterpret_cast<const char*>(t.x + t.n) <= static_cast<char*>(base) + size)
                plan.push_back(t);
        }
    };
    if (!opt.eager) {
        add_list(sumsq_plan_);
        for (const auto& list : sumsq_history_) add_list(list);
    }
    if (known) {
        bool mine = false;
        for (const TensorRef& t : plan) mine = mine || (t.x == x && t.n == n);
        if (mine && sumsq_batch(plan)) {
            auto got = sumsq_cache_.find(std::make_pair(x, n));
            if (got != sumsq_cache_.end()) return got->second;
        }
    }
    if (!sumsq_batch(std::vector<TensorRef>{TensorRef{x, n}})) {
        // more slices than the table holds: the single-tensor kernel with its fixed 1024 partials
        double* d = reinterpret_cast<double*>(ws_ + kPartialOff);
        if (launch_sumsq_partials(x, n, d, kSumsqBlocks, 0)) set_error(ERR_LAUNCH);
        launches++;
        double h[kSumsqBlocks];
        if (cudaMemcpy(h, d, sizeof h, cudaMemcpyDeviceToHost) != cudaSuccess) {
            set_error(ERR_SYNC);
            return NAN;
        }
        double s = 0;
        for (int i = 0; i < kSumsqBlocks; i++) s += h[i];
        return s;
    }
    return sumsq_cache_[std::make_pair(x, n)];
}

// ---------------------------------------------------------------- single-GPU emulation of several ranks

// Per virtual rank: flag words, tile prefix, segment table, staging area.
constexpr size_t kSimCtx = 65536;
constexpr size_t kSimFlagOff = 0;
constexpr size_t kSimPrefixOff = kFlagBytes;
constexpr size_t kSimSegOff = kSimPrefixOff + 32768;
constexpr size_t kSimStageOff = size_t(1) << 20;
constexpr size_t kSimRankBytes = kSimStageOff + kStageBytes;
static_assert(kSimSegOff + size_t(kMaxSegs) * sizeof(Seg) <= kSimStageOff, "emulation layout");

int Engine::sim_step(int world, int nseg, const int64_t* n, float* const* p, float* const* g, float* const* m,
                     float* const* v, const float* wd, float lr, float b1, float b2, float eps, int step, int adam,
                     int mode, int blocks_per_rank, unsigned long long timeout_ns, unsigned active_mask,
                     int* status_out, double* sumsq_out) {
    if (!cuda_ready()) return -1;
    if (world < 1 || world > kMaxWorld || nseg < 1 || nseg > kMaxSegs) return -1;
    sync();
    if (!sim_ws_) {
        sim_ws_ = static_cast<char*>(pool(DEV_CUDA).alloc(kSimCtx + kMaxWorld * kSimRankBytes));
        if (!sim_ws_) return -2;
        if (cudaMemset(sim_ws_, 0, kSimCtx) != cudaSuccess) return -1;
        for (int r = 0; r < kMaxWorld; r++)
            if (cudaMemset(sim_ws_ + kSimCtx + r * kSimRankBytes, 0, kSimStageOff) != cudaSuccess) return -1;
    }
    auto rank_base = [&](int r) { return sim_ws_ + kSimCtx + (size_t)r * kSimRankBytes; };

    std::vector<RankCtx> ctxs;
    std::vector<Seg> segs;
    std::vector<int> prefix;
    std::vector<float*> peer_g[kMaxWorld];
    int64_t T = 0;
    for (int r = 0; r < world; r++) {
        peer_g[r].resize(nseg);
        for (int s = 0; s < nseg; s++) peer_g[r][s] = g[r * nseg + s];
    }
    for (int r = 0; r < world; r++) {
        if (!(active_mask >> r & 1)) continue;
        std::vector<StepItem> items(nseg);
        for (int s = 0; s < nseg; s++) {
            StepItem& it = items[s];
            it.g = g[r * nseg + s], it.n = n[s], it.wd = wd ? wd[s] : 0.f, it.hyper = 0;
            if (adam) it.p = p[r * nseg + s], it.m = m[r * nseg + s], it.v = v[r * nseg + s];
        }
        bool any = false;
        T = build_table(items, world, r, peer_g, segs, prefix, &any);
        if (T < 0) return -1;
        char* rb = rank_base(r);
        if (cudaMemcpyAsync(rb + kSimSegOff, segs.data(), segs.size() * sizeof(Seg), cudaMemcpyHostToDevice, 0) != cudaSuccess) return -1;
        if (cudaMemcpyAsync(rb + kSimPrefixOff, prefix.data(), prefix.size() * sizeof(int), cudaMemcpyHostToDevice, 0) != cudaSuccess) return -1;
        RankCtx c{};
        c.segs = reinterpret_cast<Seg*>(rb + kSimSegOff), c.tile_prefix = reinterpret_cast<int*>(rb + kSimPrefixOff);
        c.nseg = nseg, c.rank = r, c.world = world;
        for (int q = 0; q < world; q++) {
            c.flags[q] = reinterpret_cast<unsigned*>(rank_base(q) + kSimFlagOff);
            c.stage[q] = reinterpret_cast<float*>(rank_base(q) + kSimStageOff);
        }
        c.status = status_dev_ + r;
        status_host_[r] = 0;
        ctxs.push_back(c);
    }
    if (ctxs.empty()) return -1;
    if (cudaMemcpyAsync(sim_ws_, ctxs.data(), ctxs.size() * sizeof(RankCtx), cudaMemcpyHostToDevice, 0) != cudaSuccess) return -1;

    const int slot_floats = stage_slot_floats(world);
    const bool fits = T * kTile <= slot_floats;
    bool oneshot = world > 1 && fits && (mode == 1 || (mode == 0 && T * kTile * 4 <= (opt.oneshot_max_bytes < 0 ? INT64_MAX : opt.oneshot_max_bytes)));
    if (mode == 1 && !oneshot) return -4;  // asked for one-shot, but the step does not fit the staging slots
    const int kind = oneshot ? KERNEL_ONESHOT : KERNEL_PLAIN;
    const size_t smem = (size_t)(nseg + 1) * sizeof(int);
    const int occ = step_occupancy(world, adam != 0, kind, smem);
    const int cap = occ * sm_count_ / (int)ctxs.size();
    if (cap < 1) return -3;
    const int work = (world == 1 || oneshot) ? (int)T : min_chunk((int)T, world);
    int G = blocks_per_rank > 0 ? blocks_per_rank : (work < 1 ? 1 : work);
    if (G > cap) G = cap;
    if (G > kFlagBlocks) G = kFlagBlocks;

    LaunchArgs a{};
    a.ctxs = reinterpret_cast<const RankCtx*>(sim_ws_);
    a.blocks_per_rank = G;
    a.seq = ++sim_seq_;
    a.parity = oneshot ? (sim_oneshots_++ & 1) : 0;
    a.stage_slot_floats = slot_floats;
    a.timeout_ns = timeout_ns ? timeout_ns : opt.timeout_ns;
    a.inv_world = 1.0f / (float)world;
    a.sumsq_on = (world > 1 && !adam && !oneshot && T <= kMaxPieceTiles) ? 1 : 0;
    fill_hyper(a.hp[0], HyperKey{lr, b1, b2, eps, step});
    last_mode = world == 1 ? 0 : (oneshot ? 1 : 2);
    last_blocks = G;
    launches++;
    if (launch_step(world, adam != 0, kind, true, G * (int)ctxs.size(), smem, a, 0) != 0) {
        cudaGetLastError();
        return -5;
    }
    if (cudaDeviceSynchronize() != cudaSuccess) return -6;
    if (status_out)
        for (int r = 0; r < world; r++) status_out[r] = status_host_[r];
    for (int r = 0; r < kMaxWorld; r++) status_host_[r] = 0;  // emulated ranks do not feed the sticky error
    if (sumsq_out) {
        if (!a.sumsq_on) return -7;
        std::vector<double> table((size_t)T);
        for (int r = 0; r < world; r++) {
            if (!(active_mask >> r & 1)) continue;
            if (cudaMemcpy(table.data(), rank_base(r) + kSimStageOff, table.size() * sizeof(double), cudaMemcpyDeviceToHost) != cudaSuccess) return -6;
            combine_pieces(table.data(), prefix, world, G, sumsq_out + (size_t)r * nseg);
        }
    }
    return 0;
}

}  // namespace slb
