// The C ABI of libsoliton_b200.so (declared in include/soliton_b200.h): routing by device kind, as
// core/soliton/api.d does it. meta does the allocator traffic and nothing else; cuda goes to the engine; cpu is
// served for memory and data movement only -- compute on cpu raises sticky error 13, this library has no host
// kernels to fall back to.
#include <cuda_runtime.h>

#include <cmath>
#include <cstring>
#include <vector>

#include "../../include/soliton_b200.h"
#include "dp_engine.hpp"
#include "foreign_path.h"
#include "pool.hpp"

using namespace slb;

static Engine& E() { return Engine::get(); }
static inline const SlbForeignPath* foreign(int dev) {
    return dev == DEV_CUDA && slb_foreign_path ? slb_foreign_path() : nullptr;
}
static inline void before_memory_op(int dev) {
    if (dev == DEV_CUDA) E().flush();  // nothing pending may outlive memory it points into
}
static inline void before_release(int dev, const void* p, size_t n) {
    if (dev == DEV_CUDA && E().cuda_ready()) E().before_release(p, n);  // nor may work in flight on another stream
}

extern "C" int slb_foreign_check(void) __attribute__((weak));

extern "C" {

// ---- memory

void* sl_alloc(int dev, size_t n) { return valid_dev(dev) ? pool(dev).alloc(n) : nullptr; }

void sl_free(int dev, void* p, size_t n) {
    if (!valid_dev(dev)) return;
    before_release(dev, p, n);
    pool(dev).release(p, n);
}

void sl_stats(int dev, int64_t* out7) {
    if (valid_dev(dev)) pool(dev).stats(out7);
}
void sl_reset_stats(int dev) {
    if (valid_dev(dev)) pool(dev).reset_stats();
}
void sl_empty_cache(int dev) {
    if (!valid_dev(dev)) return;
    before_memory_op(dev);
    pool(dev).empty_cache();
}
void sl_set_limit(int dev, int64_t bytes) {
    if (valid_dev(dev)) pool(dev).set_limit(bytes);
}
void sl_record_start(int dev) {
    if (valid_dev(dev)) pool(dev).record_start();
}
void sl_record_stop(int dev) {
    if (valid_dev(dev)) pool(dev).record_stop();
}
void sl_record_mark(int dev) {
    if (valid_dev(dev)) pool(dev).record_mark();
}
int64_t sl_record_count(int dev) { return valid_dev(dev) ? pool(dev).record_count() : 0; }
int64_t sl_record_body(int dev) { return valid_dev(dev) ? pool(dev).record_body() : 0; }
void sl_record_get(int dev, int64_t* size, int64_t* start, int64_t* end) {
    if (valid_dev(dev)) pool(dev).record_get(size, start, end);
}
int sl_arena_install(int dev, const int64_t* offsets, const int64_t* sizes, int64_t count, int64_t body,
                     int64_t arena_bytes) {
    if (!valid_dev(dev)) return -1;
    before_memory_op(dev);
    return pool(dev).arena_install(offsets, sizes, count, body, arena_bytes);
}
int sl_arena_diverged(int dev) { return valid_dev(dev) && pool(dev).diverged() ? 1 : 0; }
void sl_arena_off(int dev) {
    if (!valid_dev(dev)) return;
    before_memory_op(dev);
    pool(dev).arena_off();
}

// ---- device

int sl_init_device(int dev, int ordinal) { return E().init_device(dev, ordinal); }
int sl_cuda_count(void) { return E().device_count(); }
int sl_check(int dev) {
    int e = E().check();
    // a build that serves the rest of Soliton's ABI from another backend folds that backend's sticky error in here
    if (!e && dev == DEV_CUDA && slb_foreign_check) e = slb_foreign_check();
    return dev == DEV_CUDA || e == ERR_NO_CPU_COMPUTE ? e : 0;
}
void sl_sync(int dev) {
    if (dev == DEV_CUDA) E().sync();
}
void sl_mem_info(size_t* free_bytes, size_t* total_bytes) {
    if (cudaMemGetInfo(free_bytes, total_bytes) != cudaSuccess) {
        cudaGetLastError();
        *free_bytes = *total_bytes = 0;
    }
}

// ---- data movement

static void copy_any(int dev, void* dst, const void* src, size_t n, cudaMemcpyKind kind) {
    if (n == 0) return;
    if (dev == DEV_CPU) {
        memcpy(dst, src, n);
    } else if (dev == DEV_CUDA) {
        E().copy_blocking(dst, src, n, (int)kind);
    }
}
void sl_from_host(int dev, void* dst, const void* src, size_t n) { copy_any(dev, dst, src, n, cudaMemcpyHostToDevice); }
void sl_to_host(int dev, void* dst, const void* src, size_t n) { copy_any(dev, dst, src, n, cudaMemcpyDeviceToHost); }
void sl_copy(int dev, void* dst, const void* src, size_t n) { copy_any(dev, dst, src, n, cudaMemcpyDeviceToDevice); }

void sl_fill(int dev, float* p, int64_t n, float v) {
    if (dev == DEV_CPU) {
        for (int64_t i = 0; i < n; i++) p[i] = v;  // initialisation of host buffers, not a compute kernel
    } else if (dev == DEV_CUDA) {
        E().fill(p, n, v);
    }
}

// ---- the path

void sl_adamw(int dev, float* p, const float* g, float* m, float* v, int64_t n, float lr, float b1, float b2,
              float eps, float wd, int step) {
    if (const SlbForeignPath* f = foreign(dev)) return f->adamw(p, g, m, v, n, lr, b1, b2, eps, wd, step);
    if (dev == DEV_CUDA)
        E().adamw(p, g, m, v, n, lr, b1, b2, eps, wd, step);
    else if (dev == DEV_CPU)
        E().set_error(ERR_NO_CPU_COMPUTE);
}
int sl_dist_unique_id(char* out128) {
    if (const SlbForeignPath* f = foreign(DEV_CUDA)) return f->dist_unique_id(out128);
    return E().dist_unique_id(out128);
}
int sl_dist_init(int rank, int world, const char* id128) {
    if (const SlbForeignPath* f = foreign(DEV_CUDA)) return f->dist_init(rank, world, id128);
    return E().dist_init(rank, world, id128);
}
int sl_dist_group(int dev, int start) {
    if (const SlbForeignPath* f = foreign(dev)) return f->dist_group(start);
    return dev == DEV_CUDA ? E().group(start) : 0;
}
int sl_dist_allreduce_mean(int dev, float* p, int64_t n) {
    if (const SlbForeignPath* f = foreign(dev)) return f->dist_allreduce_mean(p, n);
    return dev == DEV_CUDA ? E().allreduce_mean(p, n) : 0;
}
void sl_dist_destroy(void) {
    if (const SlbForeignPath* f = foreign(DEV_CUDA)) return f->dist_destroy();
    E().dist_destroy();
}

// ---- next to the path

void sl_axpy(int dev, const float* x, float* y, int64_t n, float alpha) {
    if (const SlbForeignPath* f = foreign(dev)) return f->axpy(x, y, n, alpha);
    if (dev == DEV_CUDA)
        E().axpy(x, y, n, alpha);
    else if (dev == DEV_CPU)
        E().set_error(ERR_NO_CPU_COMPUTE);
}
void sl_scale(int dev, const float* x, float* y, int64_t n, float alpha) {
    if (const SlbForeignPath* f = foreign(dev)) return f->scale(x, y, n, alpha);
    if (dev == DEV_CUDA)
        E().scale(x, y, n, alpha);
    else if (dev == DEV_CPU)
        E().set_error(ERR_NO_CPU_COMPUTE);
}
double sl_sumsq(int dev, const float* x, int64_t n) {
    if (const SlbForeignPath* f = foreign(dev)) return f->sumsq(x, n);
    if (dev == DEV_CUDA) return E().sumsq(x, n);
    if (dev == DEV_CPU) E().set_error(ERR_NO_CPU_COMPUTE);
    return NAN;
}

// ---- backend level

void sl_cuda_adamw(float* p, const float* g, float* m, float* v, int64_t n, float lr, float b1, float b2, float eps,
                   float wd, int step) {
    E().adamw(p, g, m, v, n, lr, b1, b2, eps, wd, step);
}
int sl_cuda_nccl_unique_id(char* out128) { return E().dist_unique_id(out128); }
int sl_cuda_nccl_init(int rank, int world, const char* id128) { return E().dist_init(rank, world, id128); }
int sl_cuda_nccl_group(int start) { return E().group(start); }
int sl_cuda_nccl_allreduce_mean(float* p, int64_t n) { return E().allreduce_mean(p, n); }
void sl_cuda_nccl_destroy(void) { E().dist_destroy(); }
int sl_cuda_dp_set_workspace(void* p, size_t n) { return E().adopt_workspace(p, n); }
void sl_cuda_axpy(const float* x, float* y, int64_t n, float alpha) { E().axpy(x, y, n, alpha); }
void sl_cuda_scale(const float* x, float* y, int64_t n, float alpha) { E().scale(x, y, n, alpha); }
double sl_cuda_sumsq(const float* x, int64_t n) { return E().sumsq(x, n); }

// ---- additions

size_t slb_workspace_bytes(void) { return kWorkspaceBytes; }

int slb_set_option(const char* name, int64_t value) {
    Options& o = E().opt;
    if (!name) return -1;
    if (!strcmp(name, "eager")) o.eager = (int)value;
    else if (!strcmp(name, "mode")) o.mode = (int)value;
    else if (!strcmp(name, "blocks_per_sm")) o.blocks_per_sm = (int)value;
    else if (!strcmp(name, "stamps")) o.stamps = (int)value;
    else if (!strcmp(name, "overlap")) {
        if (E().cuda_ready()) E().sync();  // launches change stream: nothing may be in flight across the switch
        o.overlap = (int)value;
    }
    else if (!strcmp(name, "cyclic")) o.cyclic = (int)value;
    else if (!strcmp(name, "timeout_ms")) o.timeout_ns = (unsigned long long)value * 1000000ull;
    else if (!strcmp(name, "host_timeout_ms")) o.host_timeout_s = (double)value / 1000.0;
    else if (!strcmp(name, "oneshot_max_bytes")) o.oneshot_max_bytes = value;
    else return -1;
    return 0;
}

int64_t slb_get_counter(const char* name) {
    if (!name) return -1;
    if (!strcmp(name, "launches")) return (int64_t)E().launches;
    if (!strcmp(name, "last_mode")) return E().last_mode;
    if (!strcmp(name, "last_blocks")) return E().last_blocks;
    if (!strcmp(name, "world")) return E().world();
    if (!strcmp(name, "sm_count")) return E().sm_count();
    if (!strcmp(name, "pending_frees")) return E().pending_frees();
    return -1;
}

void slb_flush(void) { E().flush(); }

int slb_from_host_async(int k, void* const* dst, const void* const* src, const size_t* bytes) {
    return E().from_host_async(k, dst, src, bytes);
}
int slb_to_host_async(int k, void* const* dst, const void* const* src, const size_t* bytes) {
    return E().to_host_async(k, dst, src, bytes);
}
int slb_wait_copies(void) { return E().wait_copies(); }
int slb_read_stamps(uint64_t* out5) { return E().read_stamps(reinterpret_cast<unsigned long long*>(out5)); }
void slb_clear_error(void) { E().clear_error(); }

int64_t slb_tile_count(const int64_t* n, int nseg) {
    int64_t t = 0;
    for (int s = 0; s < nseg; s++) t += (n[s] + kTile - 1) / kTile;
    return t;
}

void slb_run_range(int64_t tiles, int world, int chunk, int blocks, int block, int64_t* begin, int64_t* end) {
    int64_t cb = 0, ce = tiles;
    if (chunk >= 0) cb = tiles * chunk / world, ce = tiles * (chunk + 1) / world;
    const int64_t len = ce - cb;
    *begin = cb + len * block / blocks;
    *end = cb + len * (block + 1) / blocks;
}

int slb_sim_step(int world, int nseg, const int64_t* n, float* const* p, float* const* g, float* const* m,
                 float* const* v, const float* wd, float lr, float b1, float b2, float eps, int step, int adam,
                 int mode, int blocks_per_rank, int64_t timeout_ms, unsigned active_mask, int* status_out,
                 double* sumsq_out) {
    return E().sim_step(world, nseg, n, p, g, m, v, wd, lr, b1, b2, eps, step, adam, mode, blocks_per_rank,
                        (unsigned long long)timeout_ms * 1000000ull, active_mask, status_out, sumsq_out);
}

int slb_rdv_create_id(char* out128) { return Rendezvous::create_id(out128); }

int slb_rdv_selftest(const char* id128, int rank, int world, int rounds) {
    Rendezvous r;
    const double wait_s = E().opt.host_timeout_s;
    if (r.open(id128, rank, world, wait_s) != 0) return -1;
    int rc = 0;
    if (r.stage_barrier(1, wait_s) != 0) rc = -2;
    if (rc == 0) r.unlink_now();
    // Round k: rank q publishes nseg = 3 + (k / 2) % 2 segments {export q, offset 1000 q + 16 (k / 2) + s, n = 7 s + 1},
    // so tables change every second round and the unchanged rounds must not bump the version.
    uint64_t last_version[kRdvMaxWorld] = {0};
    for (int k = 1; rc == 0 && k <= rounds; k++) {
        const uint32_t nseg = 3 + (k / 2) % 2;
        std::vector<RdvSegment> t(nseg);
        for (uint32_t s = 0; s < nseg; s++) t[s] = RdvSegment{(uint32_t)rank, 1, (uint64_t)(1000 * rank + 16 * (k / 2) + s), (int64_t)(7 * s + 1)};
        if (r.arrive((uint64_t)k, t.data(), nseg, wait_s) != 0) {
            rc = -3;
            break;
        }
        for (int q = 0; q < world; q++) {
            uint32_t n2 = 0;
            uint64_t ver = 0;
            const RdvSegment* pt = r.table_of(q, (uint64_t)k, &n2, &ver);
            if (n2 != nseg) rc = -4;
            for (uint32_t s = 0; rc == 0 && s < nseg; s++)
                if (pt[s].export_id != (uint32_t)q || pt[s].offset != (uint64_t)(1000 * q + 16 * (k / 2) + s) || pt[s].n != (int64_t)(7 * s + 1)) rc = -5;
            const bool should_change = k == 1 || (k % 2 == 0);
            if (rc == 0 && should_change != (ver != last_version[q])) rc = -6;
            last_version[q] = ver;
        }
    }
    if (rc != 0) r.fail();
    if (r.stage_barrier(2, wait_s) != 0 && rc == 0) rc = -7;
    r.close();
    return rc;
}

// Export slot life cycle without CUDA: every cycle each rank publishes `per_cycle` fake allocations, the peers check
// what they read, the owner asks for them back, the peers acknowledge, the owner recycles the slots. More
// allocations pass through than the table has slots.
int slb_rdv_slot_selftest(const char* id128, int rank, int world, int cycles, int per_cycle) {
    Rendezvous r;
    const double wait_s = E().opt.host_timeout_s;
    if (per_cycle < 1 || per_cycle > 256 || r.open(id128, rank, world, wait_s) != 0) return -1;
    int rc = r.stage_barrier(1, wait_s) != 0 ? -2 : 0;
    if (rc == 0) r.unlink_now();
    uint64_t k = 0;
    std::vector<int> mine((size_t)per_cycle);
    std::vector<RdvSegment> t((size_t)per_cycle);
    for (int c = 0; rc == 0 && c < cycles; c++) {
        for (int i = 0; i < per_cycle; i++) {
            unsigned char h[64];
            for (int b = 0; b < 64; b++) h[b] = (unsigned char)(rank * 31 + c * 7 + i * 3 + b);
            mine[i] = r.add_export(h, (uint64_t)(1000 + c));
            if (mine[i] < 0) return -3;  // ran out of slots: recycling does not work
            t[i] = RdvSegment{(uint32_t)mine[i], r.generation_of((uint32_t)mine[i]), (uint64_t)i, 1};
        }
        if (r.arrive(++k, t.data(), (uint32_t)per_cycle, wait_s) != 0) rc = -4;
        for (int q = 0; rc == 0 && q < world; q++) {
            uint32_t n2 = 0;
            uint64_t ver = 0;
            const RdvSegment* pt = r.table_of(q, k, &n2, &ver);
            for (int i = 0; rc == 0 && i < per_cycle; i++) {
                const RdvExport& x = r.peer(q).exports[pt[i].export_id];
                if (x.generation != pt[i].generation || x.size != (uint64_t)(1000 + c) ||
                    x.handle[5] != (unsigned char)(q * 31 + c * 7 + i * 3 + 5))
                    rc = -5;
            }
        }
        for (int i = 0; i < per_cycle; i++) r.mark_freed((uint32_t)mine[i]);
        if (rc == 0 && r.arrive(++k, t.data(), (uint32_t)per_cycle, wait_s) != 0) rc = -6;
        for (int q = 0; rc == 0 && q < world; q++) {
            if (q == rank) continue;
            uint32_t n2 = 0;
            uint64_t ver = 0;
            const RdvSegment* pt = r.table_of(q, k, &n2, &ver);
            for (int i = 0; i < per_cycle; i++) {
                if (!r.peer(q).exports[pt[i].export_id].freed.load()) rc = -7;
                r.ack_freed(q, pt[i].export_id);
            }
        }
        if (rc == 0 && r.arrive(++k, t.data(), (uint32_t)per_cycle, wait_s) != 0) rc = -8;
        for (int i = 0; rc == 0 && i < per_cycle; i++) {
            if (!r.released_by_all((uint32_t)mine[i])) rc = -9;
            r.recycle((uint32_t)mine[i]);
        }
    }
    const uint32_t used = r.self().n_exports.load();
    if (rc == 0 && used > (uint32_t)per_cycle) rc = -10;  // slots were reused, not appended
    if (rc != 0) r.fail();
    if (r.stage_barrier(2, wait_s) != 0 && rc == 0) rc = -11;
    r.close();
    return rc;
}

int slb_device_pci_bus_id(int ordinal, char* out, int len) {
    if (!out || len < 16 || cudaDeviceGetPCIBusId(out, len, ordinal) != cudaSuccess) {
        cudaGetLastError();
        return -1;
    }
    return 0;
}

void* slb_pinned_alloc(size_t n) {
    void* p = nullptr;
    if (cudaHostAlloc(&p, n ? n : 1, cudaHostAllocPortable) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return p;
}
void* slb_pinned_alloc_wc(size_t n) {
    void* p = nullptr;
    if (cudaHostAlloc(&p, n ? n : 1, cudaHostAllocPortable | cudaHostAllocWriteCombined) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return p;
}
void slb_pinned_free(void* p) {
    if (p) cudaFreeHost(p);
}

}  // extern "C"
