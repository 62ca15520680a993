// Host side of the data-parallel optimizer path: device set-up, the deferred step builder that turns Soliton's
// per-tensor calls into one launch, peer mapping of gradient memory, and the single-GPU emulation of several ranks.
//
// Soliton's Python delivers a step as separate calls (python/soliton/distributed.py:42-53, optim.py:17-24):
//     sl_dist_group(1); sl_dist_allreduce_mean(g_i) x K; sl_dist_group(0); sl_adamw(p_i, g_i, m_i, v_i, ...) x K
// The engine keeps those symbols and their observable results but launches once: group-end records the gradients
// and meets the peers on the host; each sl_adamw whose gradient is one of them is attached to it; when the last
// one is attached the fused all-reduce + scale + AdamW kernel goes out. Anything else that could observe or free
// memory in between (sl_sync, sl_to_host, sl_scale, sl_sumsq, sl_free, ...) first flushes what is pending, in
// which case gradients that have no AdamW call yet are only averaged. Without a process group, consecutive
// sl_adamw calls are batched the same way into one multi-tensor launch.
#pragma once
#include <cstdint>
#include <map>
#include <unordered_map>
#include <unordered_set>
#include <vector>

#include "dp_types.h"
#include "rendezvous.hpp"

namespace slb {

struct Options {
    int eager = 0;                          // 1: launch at every call instead of deferring (debugging aid)
    int mode = 0;                           // 0: pick one-shot / two-shot by size; 1: one-shot; 2: two-shot
    int blocks_per_sm = 0;                  // 0: as many as are resident
    int cyclic = 4;                         // single-rank step: blocks take groups of this many tiles round robin, so
                                            // that resident blocks walk each tensor side by side (measured: 0.566 ms
                                            // against 0.578 ms with one contiguous run per block, option value 0)
    int pipeline = -1;                      // which large-step kernel: 1 k_step (shared-memory ring), 0 k_twoshot
                                            // (register-staged), -1 the faster of the two as measured per world size
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

    // --- single-GPU emulation of `world` ranks in one cooperative launch (tests). Pointer arrays are indexed
    // [rank * nseg + segment]; active_mask selects which ranks' blocks exist. Returns 0 or a negative code;
    // status_out[r] receives rank r's device status word.
    int sim_step(int world, int nseg, const int64_t* n, float* const* p, float* const* g, float* const* m,
                 float* const* v, const float* wd, float lr, float b1, float b2, float eps, int step, int adam,
                 int mode, int blocks_per_rank, unsigned long long timeout_ns, unsigned active_mask, int* status_out);

    Options opt;
    uint64_t launches = 0;      // kernels of this library launched so far
    int world() const { return world_; }
    int last_mode = 0, last_blocks = 0;

private:
    int bind_device(int ordinal);
    int launch_items(std::vector<StepItem>& items, const std::vector<HyperKey>& hypers, bool collective);
    int exchange();             // host meeting at group end: publish my gradient table, map the peers'
    int hyper_index(const HyperKey& k);
    static void on_raw_free(void* base);
    int export_id_for(void* base, size_t size);
    void close_peer_maps();

    int err_ = 0;
    int ordinal_ = 0, sm_count_ = 0;
    char* ws_ = nullptr;
    int* status_host_ = nullptr;    // kMaxWorld ints, host-mapped; [0] is the real rank's
    int* status_dev_ = nullptr;

    // pending step
    bool in_group_ = false, reduce_pending_ = false;
    std::vector<StepItem> items_;
    std::vector<HyperKey> hypers_;
    std::unordered_map<const float*, int> by_grad_;
    std::unordered_set<const float*> params_in_batch_;
    int attached_ = 0;

    // what the device currently holds
    std::vector<Seg> dev_segs_;
    std::vector<int> dev_prefix_;
    RankCtx dev_ctx_{};
    bool dev_ctx_valid_ = false;

    // process group
    Rendezvous rdv_;
    int rank_ = 0, world_ = 1;
    unsigned seq_ = 0;
    uint64_t collectives_ = 0;
    int oneshots_ = 0;
    char* peer_ws_[kMaxWorld] = {nullptr};
    std::unordered_map<void*, int> export_ids_;                         // allocation base -> id in my export log
    std::unordered_map<uint32_t, void*> peer_open_[kMaxWorld];          // export id of rank r -> mapped base
    uint64_t peer_version_[kMaxWorld] = {0};
    std::vector<float*> peer_g_[kMaxWorld];                             // per segment, rank r's gradient as mapped here
    std::vector<RdvSegment> my_table_;

    // Gradient clipping next to the path (python/soliton/optim.py:31-39): the per-tensor sumsq calls of one clip are
    // answered from one batched launch, and the in-place scales that follow are folded into the AdamW launch.
    struct TensorRef {
        const float* x;
        int64_t n;
    };
    void flush_scales();
    bool sumsq_batch(const std::vector<TensorRef>& plan);
    std::vector<TensorRef> sumsq_plan_, sumsq_learn_;   // gradients of the last reduced group / tensors seen in this clip
    std::vector<std::vector<TensorRef>> sumsq_history_; // tensor lists of the last few clips, newest first (the pool
                                                        // hands equal-sized blocks out in an order that can alternate)
    std::map<std::pair<const float*, int64_t>, double> sumsq_cache_;   // (address, elements) -> sum, until memory may change
    std::unordered_map<float*, std::pair<int64_t, float>> pending_scale_;
    std::vector<SumsqSlice> dev_slices_;

    // emulation
    char* sim_ws_ = nullptr;
    unsigned sim_seq_ = 0;
    int sim_oneshots_ = 0;
};

}  // namespace slb
