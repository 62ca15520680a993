// Host side of the data-parallel optimizer path (see dp_engine.hpp).
#include "dp_engine.hpp"

#include <cuda_runtime.h>
#include <unistd.h>

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
        return nullptr;
    }
    return p;
}
static void cuda_raw_free(void* p) { cudaFree(p); }

static bool aligned_vec(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31) == 0; }  // 256-bit accesses
static bool aligned4(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 3) == 0; }

// Base and size of the device allocation that contains p: the pool's own registry first, the driver otherwise
// (memory that did not come from sl_alloc).
static bool find_allocation(const void* p, void** base, size_t* size) {
    if (pool(DEV_CUDA).find_raw(p, base, size)) return true;
    typedef int (*range_fn)(unsigned long long*, size_t*, unsigned long long);
    static range_fn fn = nullptr;
    if (!fn) {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &q) != cudaSuccess || !f) {
            cudaGetLastError();
            return false;
        }
        fn = reinterpret_cast<range_fn>(f);
    }
    unsigned long long b = 0;
    size_t s = 0;
    if (fn(&b, &s, (unsigned long long)reinterpret_cast<uintptr_t>(p)) != 0) return false;
    *base = reinterpret_cast<void*>((uintptr_t)b);
    *size = s;
    return true;
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
    flush();
    ws_ = static_cast<char*>(p);
    if (cudaMemset(ws_, 0, kCtlBytes) != cudaSuccess) return -1;
    dev_segs_.clear(), dev_prefix_.clear();
    dev_ctx_valid_ = false;
    return 0;
}

int Engine::init_device(int dev, int ordinal) {
    if (dev == DEV_CPU) return 0;
    if (!valid_dev(dev)) return -1;
    if (dev == DEV_CUDA && bind_device(ordinal) != 0) return -1;
    if (!pool(dev).alloc(kBlasWorkspace)) return -2;  // api.d:110 OOM code
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
    check();
}

int Engine::check() {
    if (!err_ && status_host_ && status_host_[0]) err_ = status_host_[0];
    if (!err_ && cudaPeekAtLastError() != cudaSuccess) err_ = ERR_LAUNCH;
    return err_;
}

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
}

void Engine::flush_scales() {
    for (auto& kv : pending_scale_) {
        if (launch_scale(kv.first, kv.first, kv.second.first, kv.second.second, 0)) set_error(ERR_LAUNCH);
        launches++;
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

// The kernel for steps too large for one-shot. Both candidates compute the same bits; the choice is by measured
// time on 8xB200 with the GPT-2 124M parameter set: since the register-staged kernel (k_twoshot) moves 256 bits per
// access it is ahead of the shared-memory ring (k_step) at every world size (1 rank: 0.573 vs 0.61 ms; 2 ranks:
// 0.877 vs 0.929 ms; 4 ranks: 1.234 vs 1.52 ms), so the ring only runs when the "pipeline" option asks for it.
static int large_step_kernel(int option, int world) {
    (void)world;
    return option > 0 ? KERNEL_STEP : KERNEL_PLAIN;
}

static int min_chunk(int T, int world) {
    int best = T;
    for (int c = 0; c < world; c++) {
        const int len = (int)((int64_t)T * (c + 1) / world) - (int)((int64_t)T * c / world);
        if (len < best) best = len;
    }
    return best;
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
    const int kind = oneshot ? KERNEL_ONESHOT : large_step_kernel(opt.pipeline, W);
    int stages = 0;
    const size_t smem = kind == KERNEL_STEP ? step_smem(W, adam, nseg, &stages) : (size_t)(nseg + 1) * sizeof(int);
    if (smem == 0) return ERR_LAUNCH;
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

    // Tables travel to the device only when they changed; a training loop repeats the same one every step.
    Seg* d_segs = reinterpret_cast<Seg*>(ws_ + kSegOff);
    int* d_prefix = reinterpret_cast<int*>(ws_ + kTilePrefixOff);
    if (segs.size() != dev_segs_.size() || memcmp(segs.data(), dev_segs_.data(), segs.size() * sizeof(Seg)) != 0) {
        if (cudaMemcpyAsync(d_segs, segs.data(), segs.size() * sizeof(Seg), cudaMemcpyHostToDevice, 0) != cudaSuccess) return ERR_LAUNCH;
        dev_segs_ = segs;
    }
    if (prefix != dev_prefix_) {
        if (cudaMemcpyAsync(d_prefix, prefix.data(), prefix.size() * sizeof(int), cudaMemcpyHostToDevice, 0) != cudaSuccess) return ERR_LAUNCH;
        dev_prefix_ = prefix;
    }
    RankCtx ctx{};
    ctx.segs = d_segs, ctx.tile_prefix = d_prefix, ctx.nseg = nseg, ctx.rank = me, ctx.world = W;
    for (int r = 0; r < W; r++) {
        char* base = (W == 1 || r == me) ? ws_ : peer_ws_[r];
        ctx.flags[r] = reinterpret_cast<unsigned*>(base + kFlagOff);
        ctx.stage[r] = reinterpret_cast<float*>(base + kCtlBytes);
    }
    ctx.status = status_dev_;
    if (!dev_ctx_valid_ || memcmp(&ctx, &dev_ctx_, sizeof ctx) != 0) {
        if (cudaMemcpyAsync(ws_ + kCtxOff, &ctx, sizeof ctx, cudaMemcpyHostToDevice, 0) != cudaSuccess) return ERR_LAUNCH;
        dev_ctx_ = ctx;
        dev_ctx_valid_ = true;
    }

    LaunchArgs a{};
    a.ctxs = reinterpret_cast<const RankCtx*>(ws_ + kCtxOff);
    a.blocks_per_rank = G;
    a.seq = W > 1 ? ++seq_ : 0;
    a.parity = oneshot ? (oneshots_++ & 1) : 0;
    a.stage_slot_floats = slot_floats;
    a.timeout_ns = opt.timeout_ns;
    a.inv_world = 1.0f / (float)W;
    a.stages = stages;
    a.cyclic = opt.cyclic;
    for (size_t i = 0; i < hypers.size() && i < (size_t)kMaxHyper; i++) fill_hyper(a.hp[i], hypers[i]);
    last_mode = W == 1 ? 0 : (oneshot ? 1 : 2);
    last_blocks = G;
    launches++;
    return launch_step(W, adam, kind, false, G, smem, a, 0) == 0 ? 0 : ERR_LAUNCH;
}

// ---------------------------------------------------------------- process group

void Engine::on_raw_free(void* base) {
    Engine& e = get();
    e.sumsq_plan_.clear(), e.sumsq_learn_.clear(), e.sumsq_history_.clear();  // remembered addresses may die with this block
    auto it = e.export_ids_.find(base);
    if (it == e.export_ids_.end()) return;
    e.rdv_.mark_freed((uint32_t)it->second);
    e.export_ids_.erase(it);
}

int Engine::export_id_for(void* base, size_t size) {
    auto it = export_ids_.find(base);
    if (it != export_ids_.end()) return it->second;
    cudaIpcMemHandle_t h;
    if (cudaIpcGetMemHandle(&h, base) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    static_assert(sizeof(h) == 64, "IPC handle size");
    const int id = rdv_.add_export(reinterpret_cast<unsigned char*>(&h), size);
    if (id >= 0) export_ids_[base] = id;
    return id;
}

int Engine::dist_unique_id(char* out) { return out ? Rendezvous::create_id(out) : -1; }

int Engine::dist_init(int rank, int world, const char* id) {
    if (!cuda_ready() || rdv_.is_open() || !id) return -1;
    flush();
    if (rdv_.open(id, rank, world, opt.host_timeout_s) != 0) return -1;
    rank_ = rank, world_ = world, seq_ = 0, collectives_ = 0, oneshots_ = 0;
    dev_ctx_valid_ = false;
    for (int r = 0; r < kMaxWorld; r++) peer_ws_[r] = nullptr, peer_version_[r] = 0, peer_g_[r].clear();
    bool ok = cudaMemset(ws_ + kFlagOff, 0, kFlagBytes) == cudaSuccess && cudaDeviceSynchronize() == cudaSuccess;
    RdvRank& me = rdv_.self();
    me.ordinal = ordinal_, me.sm_count = sm_count_, me.pid = (int)getpid();
    if (ok && world > 1) {
        void* base = nullptr;
        size_t size = 0;
        cudaIpcMemHandle_t h;
        ok = find_allocation(ws_, &base, &size) && cudaIpcGetMemHandle(&h, base) == cudaSuccess;
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
        for (auto& kv : peer_open_[r]) cudaIpcCloseMemHandle(kv.second);
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
    flush();
    cudaDeviceSynchronize();
    rdv_.stage_barrier(3, 10.0);  // every rank's kernels are done before any mapping goes away
    close_peer_maps();
    export_ids_.clear();
    rdv_.close();
    rank_ = 0, world_ = 1;
    dev_ctx_valid_ = false;
    dev_segs_.clear();
}

int Engine::exchange() {
    const uint32_t nseg = (uint32_t)items_.size();
    my_table_.resize(nseg);
    for (uint32_t s = 0; s < nseg; s++) {
        void* base = nullptr;
        size_t size = 0;
        if (!find_allocation(items_[s].g, &base, &size)) return -1;
        const uint64_t off = (uint64_t)(reinterpret_cast<char*>(items_[s].g) - static_cast<char*>(base));
        if (off + (uint64_t)items_[s].n * 4 > size) return -1;
        const int id = export_id_for(base, size);
        if (id < 0) return -1;
        my_table_[s].export_id = (uint32_t)id, my_table_[s].pad = 0, my_table_[s].offset = off, my_table_[s].n = items_[s].n;
    }
    const uint64_t k = ++collectives_;
    if (rdv_.arrive(k, my_table_.data(), nseg, opt.host_timeout_s) != 0) {
        rdv_.fail();
        return -1;
    }
    for (int r = 0; r < world_; r++) {
        if (r == rank_) continue;
        uint32_t n2 = 0;
        uint64_t ver = 0;
        const RdvSegment* t = rdv_.table_of(r, k, &n2, &ver);
        for (uint32_t s = 0; s < nseg; s++)
            if (t[s].n != items_[s].n) return -1;  // the ranks disagree about the tensors of this step
        if (ver == peer_version_[r] && peer_g_[r].size() == nseg) continue;
        RdvRank& pr = rdv_.peer(r);
        for (auto it = peer_open_[r].begin(); it != peer_open_[r].end();) {  // drop mappings of freed allocations
            if (pr.exports[it->first].freed.load(std::memory_order_acquire)) {
                cudaIpcCloseMemHandle(it->second);
                it = peer_open_[r].erase(it);
            } else {
                ++it;
            }
        }
        peer_g_[r].assign(nseg, nullptr);
        for (uint32_t s = 0; s < nseg; s++) {
            const uint32_t id = t[s].export_id;
            if (id >= pr.n_exports.load(std::memory_order_acquire)) return -1;
            auto it = peer_open_[r].find(id);
            void* base = nullptr;
            if (it != peer_open_[r].end()) {
                base = it->second;
            } else {
                cudaIpcMemHandle_t h;
                memcpy(&h, pr.exports[id].handle, 64);
                if (cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) {
                    cudaGetLastError();
                    return -1;
                }
                peer_open_[r][id] = base;
            }
            if (t[s].offset + (uint64_t)t[s].n * 4 > pr.exports[id].size) return -1;
            peer_g_[r][s] = reinterpret_cast<float*>(static_cast<char*>(base) + t[s].offset);
        }
        peer_version_[r] = ver;
    }
    return 0;
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
    if (launch_scale(x, y, n, alpha, 0)) set_error(ERR_LAUNCH);
    launches++;
}
void Engine::axpy(const float* x, float* y, int64_t n, float alpha) {
    if (!cuda_ready()) return set_error(ERR_NO_WORKSPACE);
    flush();
    if (n > 0 && (!x || !y)) return set_error(ERR_BAD_ARG);
    if (launch_axpy(x, y, n, alpha, 0)) set_error(ERR_LAUNCH);
    launches += n > 0;
}
void Engine::fill(float* p, int64_t n, float v) {
    if (!cuda_ready()) return set_error(ERR_NO_WORKSPACE);
    flush();
    if (n > 0 && !p) return set_error(ERR_BAD_ARG);
    if (launch_fill(p, n, v, 0)) set_error(ERR_LAUNCH);
    launches += n > 0;
}

// Sum of squares of a tensor (the reference: cublasSdot, core/cuda/kernels.cu:219-224, blocking). Fixed block
// slices and a fixed combination order make the value reproducible run to run; double partials make it at least
// as accurate as the float dot it stands in for.
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

// Sum of squares of a tensor (the reference: cublasSdot, core/cuda/kernels.cu:219-224, blocking). Fixed slices and
// a fixed combination order make the value reproducible run to run; double partials make it at least as accurate
// as the float dot it stands in for. Soliton's clip asks tensor by tensor (python/soliton/optim.py:34); the first
// question is answered by summing every tensor the clip is expected to ask about -- the gradients of the group
// that was just reduced, else the tensors of the previous clip -- in one launch, the rest from that launch.
double Engine::sumsq(const float* x, int64_t n) {
    if (!cuda_ready()) {
        set_error(ERR_NO_WORKSPACE);
        return NAN;
    }
    flush_step();
    if (!pending_scale_.empty()) {
        flush_scales();
        sumsq_cache_.clear();
    }
    if (n <= 0) return 0.0;
    if (!x) {
        set_error(ERR_BAD_ARG);
        return NAN;
    }
    sumsq_learn_.push_back(TensorRef{x, n});
    auto hit = sumsq_cache_.find(std::make_pair(x, n));
    if (hit != sumsq_cache_.end()) return hit->second;
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
                     int* status_out) {
    if (!cuda_ready()) return -1;
    if (world < 1 || world > kMaxWorld || nseg < 1 || nseg > kMaxSegs) return -1;
    flush();
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
    const int kind = oneshot ? KERNEL_ONESHOT : large_step_kernel(opt.pipeline, world);
    int stages = 0;
    const size_t smem = kind == KERNEL_STEP ? step_smem(world, adam != 0, nseg, &stages) : (size_t)(nseg + 1) * sizeof(int);
    if (smem == 0) return -3;
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
    a.stages = stages;
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
    return 0;
}

}  // namespace slb
