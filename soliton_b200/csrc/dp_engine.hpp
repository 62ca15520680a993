// Host side of the data-parallel optimizer path: device set-up, the deferred step builder that turns Soliton's
// per-tensor calls into one launch, peer mapping of gradient memory, the streams the path may run on beside the
// legacy stream, and the single-GPU emulation of several ranks.
//
// Soliton's Python delivers a step as separate calls (python/soliton/distributed.py:42-53, optim.py:17-24):
//     sl_dist_group(1); sl_dist_allreduce_mean(g_i) x K; sl_dist_group(0); sl_adamw(p_i, g_i, m_i, v_i, ...) x K
// The engine keeps those symbols and their observable results but launches once: group-end records the gradients
// and meets the peers on the host; each sl_adamw whose gradient is one of them is attached to it; when the last
// one is attached the fused all-reduce + scale + AdamW kernel goes out. Anything else that could observe or free
// memory in between (sl_sync, sl_to_host, sl_scale, sl_sumsq, sl_free, ...) first flushes what is pending, in
// which case gradients that have no AdamW call yet are only averaged. Without a process group, consecutive
// sl_adamw calls are batched the same way into one multi-tensor launch.
//
// A caller that closes a group per bucket of tensors (gradients become final in reverse layer order,
// python/soliton/tensor.py:427-471) gets one fused launch per bucket, as soon as the bucket's last sl_adamw has
// arrived. With the "overlap" option these launches go to a stream of their own, beside whatever the caller still has
// running on the legacy stream (the rest of backward), and asynchronous host copies run on two more streams
// (slb_from_host_async, slb_to_host_async). Ordering between the streams is by address range: every piece of work
// on one of these streams is remembered with the memory it reads and writes and an event, and anything that touches
// an overlapping range later, on whichever stream, waits for that event first (Lanes, below).
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <map>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "dp_types.h"
#include "rendezvous.hpp"

namespace slb {

struct Options {
    int eager = 0;                          // 1: launch at every call instead of deferring
    int mode = 0;                           // 0: pick one-shot / two-shot by size; 1: one-shot; 2: two-shot
    int blocks_per_sm = 0;                  // 0: as many as are resident
    int cyclic = 4;                         // single-rank step: blocks take groups of this many tiles round robin, so
                                            // that resident blocks walk each tensor side by side; 0: one contiguous run
    int stamps = 0;                         // collective launches record device times at their phase borders
    int overlap = 0;                        // 1: path launches go to a stream of their own instead of the legacy stream
    unsigned long long timeout_ns = 10ull * 1000 * 1000 * 1000;  // bound of every device-side flag wait
    double host_timeout_s = 120.0;          // bound of every host-side wait on a peer
    long long oneshot_max_bytes = -1;       // -1: whatever fits the staging slots
};

struct StepItem {               // one tensor of a pending step
    float *g = nullptr, *p = nullptr, *m = nullptr, *v = nullptr;
    int64_t n = 0;
    float wd = 0;
    int hyper = 0;
    float gscale = 1.0f;        // in-place gradient scale folded into the update (clipping)
};

struct HyperKey {
    float lr, b1, b2, eps;
    int step;
    bool operator==(const HyperKey& o) const {
        return lr == o.lr && b1 == o.b1 && b2 == o.b2 && eps == o.eps && step == o.step;
    }
};

struct Range {                  // [lo, hi) of device addresses
    uintptr_t lo, hi;
    bool operator<(const Range& o) const { return lo < o.lo; }
};

// The streams the path uses and the ordering between them. Lane 0 carries the path's kernels (the legacy stream, or
// the step stream with the "overlap" option), lane 1 host-to-device copies, lane 2 device-to-host copies. A piece
// of work is `begin`-ed with the ranges it will read and write -- its stream then waits for every earlier piece, on
// another lane, that conflicts -- issued by the caller, and `end`-ed, which records the event later work waits on.
// The legacy stream itself is not a lane: work the caller puts there is ordered against the lanes by
// `legacy_touches`, which makes the legacy stream wait for conflicting pieces.
class Lanes {
public:
    enum : int { STEP = 0, UP = 1, DOWN = 2, COUNT = 3 };
    int init();                                     // creates the streams; 0 or -1
    cudaStream_t stream(int lane, bool overlap) const { return lane == STEP && !overlap ? (cudaStream_t)0 : streams_[lane]; }
    int begin(int lane, cudaStream_t st, std::vector<Range>& reads, std::vector<Range>& writes);
    int end(int lane, cudaStream_t st);
    int legacy_touches(const void* p, size_t bytes, bool write);
    bool idle() const { return pieces_.empty(); }
    void forget();                                  // after the device has been synchronised: nothing is in flight
    int wait_copies();                              // host waits for lanes UP and DOWN
    bool ready() const { return ready_; }

private:
    struct Piece {
        int lane;
        uint64_t seq;
        cudaEvent_t ev;
        std::vector<Range> reads, writes;           // sorted by lo
    };
    static bool overlaps(const std::vector<Range>& a, const std::vector<Range>& b);
    cudaEvent_t take_event();
    void retire_finished();
    bool ready_ = false;
    cudaStream_t streams_[COUNT] = {nullptr, nullptr, nullptr};
    std::vector<Piece> pieces_;
    std::vector<cudaEvent_t> spare_;
    Piece open_[COUNT];                             // between begin and end
    uint64_t seq_ = 0;
    uint64_t waited_[COUNT + 1][COUNT] = {{0}};     // [waiting lane or COUNT = legacy][lane waited for] -> latest seq
};

class Engine {
public:
    static Engine& get();

    // --- device
    int init_device(int dev, int ordinal);          // core/soliton/api.d:262-274
    int device_count();
    void sync();
    int check();
    void set_error(int code) { if (!err_) err_ = code; }
    void clear_error();
    int sm_count() const { return sm_count_; }
    // Backend-level set-up for a host core that owns the allocator: binds the current device and takes `n` bytes
    // at `p` (at least kWorkspaceBytes, from that core's pool) as the path's workspace. 0 or -1.
    int adopt_workspace(void* p, size_t n);
    bool cuda_ready() const { return ws_ != nullptr; }
    char* workspace() const { return ws_; }
    int ordinal() const { return ordinal_; }
    // The 32 MiB the reference reserves for cuBLAS at device initialisation (core/soliton/api.d:129,268-272): this
    // library has no use for it, a backend that serves the rest of the ABI does.
    void* blas_workspace() const { return blas_ws_; }
    size_t blas_workspace_bytes() const { return blas_ws_ ? size_t(32) << 20 : 0; }

    // --- the path
    void adamw(float* p, const float* g, float* m, float* v, int64_t n, float lr, float b1, float b2, float eps,
               float wd, int step);                 // api.d:539-543
    int group(int start);                           // api.d:582-585
    int allreduce_mean(float* g, int64_t n);        // api.d:587-590
    int dist_unique_id(char* out);                  // api.d:572-575
    int dist_init(int rank, int world, const char* id);  // api.d:577-580
    void dist_destroy();                            // api.d:592-595
    void flush();                                   // launch whatever is pending: the step, deferred scales
    void flush_step();                              // only the pending step (all-reduce and/or AdamW batch)

    // --- next to the path
    void scale(const float* x, float* y, int64_t n, float alpha);
    void axpy(const float* x, float* y, int64_t n, float alpha);
    void fill(float* p, int64_t n, float v);
    double sumsq(const float* x, int64_t n);
    // Blocking copy on the legacy stream, ordered after whatever the lanes still do with that memory.
    void copy_blocking(void* dst, const void* src, size_t n, int kind);
    // Memory is about to go back to the allocator: the legacy stream waits for lane work that still uses it.
    void before_release(const void* p, size_t n);

    // --- copies beside the path (pinned host memory), k buffers per call; 0 or -1
    int from_host_async(int k, void* const* dst, const void* const* src, const size_t* bytes);
    int to_host_async(int k, void* const* dst, const void* const* src, const size_t* bytes);
    int wait_copies();

    // --- device times of the last collective launch with the "stamps" option (kStamps values); 0 or -1
    int read_stamps(unsigned long long* out);

    // --- single-GPU emulation of `world` ranks in one cooperative launch (tests). Pointer arrays are indexed
    // [rank * nseg + segment]; active_mask selects which ranks' blocks exist. Returns 0 or a negative code;
    // status_out[r] receives rank r's device status word. With sumsq_out (world x nseg doubles) and adam = 0 in
    // two-shot mode, the per-tensor sums of squares of the mean as every rank's piece table gives them.
    int sim_step(int world, int nseg, const int64_t* n, float* const* p, float* const* g, float* const* m,
                 float* const* v, const float* wd, float lr, float b1, float b2, float eps, int step, int adam,
                 int mode, int blocks_per_rank, unsigned long long timeout_ns, unsigned active_mask, int* status_out,
                 double* sumsq_out);

    // Export slots of this rank that wait for the peers to let go (tests).
    int pending_frees() const { return (int)pending_free_.size(); }
    static bool take_deferred_free(void* base);     // the pool's raw free asks: is this block's cudaFree deferred?
    static void* retry_after_deferred_frees(size_t n);

    Options opt;
    uint64_t launches = 0;      // kernels of this library launched so far
    int world() const { return world_; }
    int last_mode = 0, last_blocks = 0;

private:
    struct TensorRef {
        const float* x;
        int64_t n;
    };
    int bind_device(int ordinal);
    int launch_items(std::vector<StepItem>& items, const std::vector<HyperKey>& hypers, bool collective);
    int exchange();             // host meeting at group end: publish my gradient table, map the peers'
    int hyper_index(const HyperKey& k);
    static void on_raw_free(void* base);
    int export_id_for(void* base, size_t size, bool from_pool);
    void close_peer_maps();
    void let_go_of_freed(int r);        // peer side of the export slot life cycle
    void collect_released(bool force);  // owner side: cudaFree blocks every peer has let go of
    // Device copy of a step's tables (rank context, tile prefix, segments): uploaded once, found again by content.
    const RankCtx* resident_tables(const RankCtx& ctx, const std::vector<Seg>& segs, const std::vector<int>& prefix,
                                   cudaStream_t st);
    bool harvest_fused_sumsq();
    int after_legacy(int lane, cudaStream_t st);

    int err_ = 0;
    int ordinal_ = 0, sm_count_ = 0;
    char* ws_ = nullptr;
    void* blas_ws_ = nullptr;
    int* status_host_ = nullptr;    // kMaxWorld ints, host-mapped; [0] is the real rank's
    int* status_dev_ = nullptr;
    Lanes lanes_;
    cudaEvent_t legacy_ev_ = nullptr;
    uint64_t legacy_epoch_ = 1, lane_seen_epoch_[Lanes::COUNT] = {0, 0, 0};

    // pending step
    bool in_group_ = false, reduce_pending_ = false;
    std::vector<StepItem> items_;
    std::vector<HyperKey> hypers_;
    std::unordered_map<const float*, int> by_grad_;
    std::unordered_set<const float*> params_in_batch_;
    int attached_ = 0;

    // tables resident in the workspace
    struct Resident {
        std::vector<unsigned char> image;   // ctx + prefix + segs as uploaded
        size_t offset;                      // of the image inside the table area
    };
    std::vector<Resident> resident_;
    size_t resident_used_ = 0;

    // process group
    Rendezvous rdv_;
    int rank_ = 0, world_ = 1;
    unsigned seq_ = 0;
    uint64_t collectives_ = 0;
    int oneshots_ = 0;
    char* peer_ws_[kMaxWorld] = {nullptr};
    struct Exported {
        int id;
        bool from_pool;
        unsigned long long buffer_id;       // driver's id of the allocation (memory that is not the pool's)
        size_t size;
    };
    std::unordered_map<void*, Exported> export_ids_;                    // allocation base -> slot in my export table
    struct PendingFree {
        void* base;                         // null: memory that is not ours to free
        uint32_t id;
    };
    std::vector<PendingFree> pending_free_;
    std::unordered_set<void*> deferred_;                                // bases whose cudaFree waits in pending_free_
    struct PeerMap {
        void* base;
        uint32_t generation;
    };
    std::unordered_map<uint32_t, PeerMap> peer_open_[kMaxWorld];        // export slot of rank r -> mapping here
    uint32_t peer_free_epoch_[kMaxWorld] = {0};
    uint64_t peer_version_[kMaxWorld] = {0};
    std::vector<float*> peer_g_[kMaxWorld];                             // per segment, rank r's gradient as mapped here
    std::vector<RdvSegment> my_table_;

    // Gradient clipping next to the path (python/soliton/optim.py:31-39): the per-tensor sumsq calls of one clip are
    // answered from one batched launch -- or, after a two-shot gradient mean, from the pieces that launch left in
    // the staging area -- and the in-place scales that follow are folded into the AdamW launch.
    void flush_scales();
    bool sumsq_batch(const std::vector<TensorRef>& plan);
    std::vector<TensorRef> sumsq_plan_, sumsq_learn_;   // gradients of the last reduced group / tensors seen in this clip
    std::vector<std::vector<TensorRef>> sumsq_history_; // tensor lists of the last few clips, newest first (the pool
                                                        // hands equal-sized blocks out in an order that can alternate)
    std::map<std::pair<const float*, int64_t>, double> sumsq_cache_;   // (address, elements) -> sum, until memory may change
    std::unordered_map<float*, std::pair<int64_t, float>> pending_scale_;
    std::vector<SumsqSlice> dev_slices_;
    struct FusedSumsq {                     // what the last two-shot mean without an optimizer left behind
        bool valid = false;
        int world = 1, blocks = 1;
        std::vector<int> prefix;
        std::vector<TensorRef> tensors;
    } fused_;

    // emulation
    char* sim_ws_ = nullptr;
    unsigned sim_seq_ = 0;
    int sim_oneshots_ = 0;
};

// Sum-of-squares pieces of a two-shot launch: tensor s gets the table entries at its piece starts, in tile order.
// A piece starts where a block's run starts and where a segment starts. out[s] for s < nseg.
void combine_pieces(const double* table, const std::vector<int>& prefix, int world, int blocks, double* out);

}  // namespace slb
