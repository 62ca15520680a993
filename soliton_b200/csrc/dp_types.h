// Structures shared by the host step builder and the device kernels of the data-parallel optimizer path.
//
// Vocabulary. A *segment* is one parameter tensor of the step (its gradient on every rank, and this rank's
// parameter and AdamW moments). The step's segments, each padded up to whole *tiles* of kTile floats, form one
// virtual sequence of tiles. For the two-shot exchange the sequence is cut into `world` contiguous *chunks*,
// chunk c owned by rank c; inside a chunk (or, for one-shot and single-rank steps, inside the whole sequence)
// every thread block works on one contiguous *run* of tiles. All of these cuts are pure functions of the segment
// sizes, the world size and the block count, so every rank computes the same partition without talking.
#pragma once
#include <cstdint>

namespace slb {

constexpr int kMaxWorld = 8;        // ranks of one NVSwitch box
constexpr int kThreads = 256;       // threads per block
constexpr int kTile = 8 * kThreads; // floats per tile: 2048 (8 KiB per tensor stream), one 256-bit access per thread
constexpr int kMaxSegs = 4096;      // segments per step
constexpr int kMaxHyper = 8;        // distinct hyperparameter sets per step
constexpr int kFlagBlocks = 1024;   // upper bound on blocks per rank that take part in flag barriers
constexpr int kFlagRows = 3;        // start, reduced, done

// Workspace the path reserves once per device from the deterministic allocator (identically on meta):
// [control: rank contexts, flag words, segment table, tile prefix][one-shot staging].
constexpr size_t kCtlBytes = size_t(2) << 20;
constexpr size_t kStageBytes = size_t(16) << 20;
constexpr size_t kWorkspaceBytes = kCtlBytes + kStageBytes;  // 18 MiB
// Offsets inside the control area.
constexpr size_t kCtxOff = 0;                                   // kMaxWorld rank contexts (emulation uses all)
constexpr size_t kStampOff = 4096;                              // kStamps device timestamps of the last collective launch
constexpr int kStamps = 5;                                      // start, peers present, own chunk reduced, gathered, peers done
constexpr size_t kFlagOff = 8192;                               // kFlagRows x kFlagBlocks x kMaxWorld x 4 B
constexpr size_t kFlagBytes = size_t(kFlagRows) * kFlagBlocks * kMaxWorld * 4;
constexpr size_t kTableOff = kFlagOff + kFlagBytes;              // resident step tables: rank context, tile prefix, segments
constexpr size_t kTableBytes = size_t(768) << 10;                // holds at least one table of kMaxSegs segments
constexpr size_t kPartialOff = kTableOff + kTableBytes;          // kSumsqBlocks doubles (sum-of-squares partials)
constexpr int kSumsqBlocks = 1024;
// Batched sum of squares over many tensors: tensors are cut into slices of kSumsqSlice floats, one partial each.
constexpr int kSumsqSlice = 65536;
constexpr int kMaxSumsqSlices = 16384;
constexpr size_t kSliceTableOff = kPartialOff + size_t(kSumsqBlocks) * 8;          // kMaxSumsqSlices x {ptr, n}
constexpr size_t kSlicePartialOff = kSliceTableOff + size_t(kMaxSumsqSlices) * 16;  // kMaxSumsqSlices doubles
static_assert(kSlicePartialOff + size_t(kMaxSumsqSlices) * 8 <= kCtlBytes, "control area layout");
static_assert(kStampOff + kStamps * 8 <= kFlagOff, "control area layout");
constexpr int64_t kMaxPieceTiles = (int64_t)(kStageBytes / 8);  // sum-of-squares pieces live in the staging area, by tile

struct SumsqSlice {      // one slice of one tensor
    const float* x;
    int64_t n;
};

struct Hyper {  // one AdamW hyperparameter set of a step (core/cuda/kernels.cu:251-254 computes bc1, bc2 on the host)
    double bc1, bc2;        // 1 - b1^step, 1 - b2^step, in double
    double rbc1, rbc2;      // their correctly rounded reciprocals
    float lr, b1, b2, eps;
    float c1, c2;           // the floats (1 - b1), (1 - b2)
};

struct alignas(16) Seg {
    float* p;               // this rank's parameter, first moment, second moment; all null for a bare all-reduce
    float* m;
    float* v;
    float* g[kMaxWorld];    // rank r's gradient of this tensor as addressable from this rank; g[rank] is local
    int64_t n;              // elements
    float wd;               // weight decay of this tensor (python/soliton/optim.py:23)
    int hyper;              // index into the launch's Hyper sets
    int vec;                // 1 when every pointer above is 32-byte aligned (256-bit path), else scalar path
    float gscale;           // factor applied to the gradient before the update and stored back with it (gradient
                            // clipping, python/soliton/optim.py:35-38); 1 = gradient used and left as it is
};
static_assert(sizeof(Seg) == 112, "segment layout");

// What one rank needs to run a launch. Lives in device memory so that one kernel can also run several virtual
// ranks side by side on one GPU (single-GPU emulation of the multi-rank protocol, used by the tests).
struct alignas(16) RankCtx {
    const Seg* segs;
    const int* tile_prefix;         // nseg + 1 entries: first tile of each segment, then the total
    int nseg;
    int rank;
    int world;
    int pad;
    unsigned* flags[kMaxWorld];     // flag area of every rank as addressable from this rank; flags[rank] is local
    float* stage[kMaxWorld];        // one-shot staging area of every rank, likewise; two-shot launches without an
                                    // optimizer use it as the table of sum-of-squares pieces (doubles, by first tile)
    int* status;                    // first error of this rank's kernels (0 = none); host-mapped
    unsigned long long* stamps;     // kStamps device times of block 0, or null
};
static_assert(sizeof(RankCtx) == 176, "rank context layout");

enum Status : int {
    ST_OK = 0,
    ST_TIMEOUT_START = 21,   // a peer never announced its gradients
    ST_TIMEOUT_REDUCED = 22, // a peer never announced its reduced chunk / its staged gradients
    ST_TIMEOUT_DONE = 23,    // a peer never announced that it finished reading
};

struct LaunchArgs {
    const RankCtx* ctxs;            // one per virtual rank; the real multi-process path has exactly one
    int blocks_per_rank;
    unsigned seq;                   // launch sequence number, equal on all ranks; flag words are monotonic in it
    int parity;                     // which half of the staging area this one-shot launch uses
    int stage_slot_floats;          // capacity of one (parity, source rank) staging slot
    unsigned long long timeout_ns;  // bound of every flag wait
    float inv_world;
    int sumsq_on;                   // two-shot without an optimizer: write the sum-of-squares pieces of the mean
    int cyclic;                     // single-rank k_twoshot: > 0 = block-cyclic tile order in groups of this many tiles
    Hyper hp[kMaxHyper];
};

// Sticky error codes surfaced by sl_check. 1..11 are the reference's (core/cuda/kernels.cu:21-34,101-108);
// the rest are this library's.
enum Err : int {
    ERR_LAUNCH = 2,
    ERR_SYNC = 3,
    ERR_BAD_ARG = 12,        // misuse of an entry point (null/odd pointer, negative size, too many segments)
    ERR_NO_CPU_COMPUTE = 13, // a compute op was asked to run on the cpu device: this library has no host kernels
    ERR_NO_WORKSPACE = 14,   // the device was not initialised through sl_init_device
    ERR_PEER = 20,           // 21..23: a bounded wait on a peer ran out (see Status)
};

}  // namespace slb
