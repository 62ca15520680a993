// sm_100a kernels of the data-parallel optimizer path: gradient mean over ranks + AdamW, in one launch.
//
// Replaces, for this path, the reference's ncclAllReduce(ncclAvg) (core/cuda/kernels.cu:773-775) followed by one
// k_adamw launch per tensor (core/cuda/kernels.cu:242-254).
//
// The path is bandwidth-bound (28 algorithmic HBM bytes per parameter, no contraction), so the kernels are built
// around memory traffic: 256-bit coalesced accesses, every thread issuing all loads of a tile before it touches
// the data, streaming cache hints for local tensors, one launch for all tensors of a step, and grids sized to the
// number of blocks that are resident at once. Peer gradients are read and written directly through
// NVSwitch-mapped pointers; no library collective runs.
//
//   k_twoshot<W,ADAM>  reduce-scatter + all-gather. Rank c owns chunk c of the tile sequence: it pulls that chunk
//                      from every rank, sums in rank order 0..W-1, multiplies by 1/W, stores the mean into its own
//                      gradient and (ADAM) updates its own p, m, v on the spot. Then it pulls every other chunk's
//                      mean from its owner, stores it into its local gradient and updates p, m, v there.
//                      With W == 1 this is the plain multi-tensor AdamW step.
//                      Without an optimizer (ADAM = false) the owner also accumulates the sum of squares of the
//                      mean it produces, piece by piece, for the gradient clip that follows such a launch.
//                      A tile's loads are all issued when the tile is reached. Running the peer loads several tiles
//                      ahead (a register ring; a shared-memory ring filled by cp.async) was built and measured on
//                      2, 4 and 8 GPUs: no faster at best, so it is not here. The fabric, not the depth of
//                      outstanding loads, bounds the exchange.
//   k_oneshot<W,ADAM>  for small steps: every rank pushes its gradients into a staging slot on every peer, one
//                      barrier, then every rank reduces all W copies locally in the same rank order.
//
// All of them produce the same bits: the sum is ((g0 + g1) + g2) + ... in float, then one multiply by 1/W, whoever
// computes it; so weights stay bit-identical across ranks and across the one-shot/two-shot choice.
//
// Synchronisation is per block index: block b of a rank only ever depends on block b of its peers, because the
// run of tiles block b works on inside a chunk is the same on every rank. Flag words are monotonic in the launch
// sequence number, written with st.release.sys and polled with ld.acquire.sys; every poll loop is bounded by
// LaunchArgs::timeout_ns, after which the block records a status code, skips its remaining data work, still posts
// its own flags (so peers do not wait on it in turn) and returns normally.
#include <cuda_runtime.h>

#include <cmath>
#include <cstring>

#include "dp_launch.h"
#include "dp_types.h"

namespace slb {

enum Mode : int { REDUCE_OWN = 0, GATHER = 1, PUSH = 2, REDUCE_STAGED = 3 };
enum Barrier : int { B_START = 0, B_REDUCED = 1, B_DONE = 2 };  // rows of the flag area

// ---------------------------------------------------------------- memory primitives

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// Gradient data that another GPU may have written during this launch (or that lives on another GPU): strong
// system-scope loads, which never hit a stale L1 line. Ordered after the acquiring flag poll by program order.
__device__ __forceinline__ float ld_sys1(const float* p) {
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
    return v;
}
// 256-bit accesses (sm_100): eight floats per thread and instruction, half as many memory instructions and requests
// for the same bytes.
struct alignas(32) float8 {
    float4 lo, hi;
};
__device__ __forceinline__ float8 ld_sys8(const float* p) {
    float8 v;
    asm volatile("ld.relaxed.sys.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(v.lo.x), "=f"(v.lo.y), "=f"(v.lo.z), "=f"(v.lo.w), "=f"(v.hi.x), "=f"(v.hi.y), "=f"(v.hi.z), "=f"(v.hi.w)
                 : "l"(p)
                 : "memory");
    return v;
}
// Local tensors that are read once and written once per step: streaming (evict-first) accesses.
__device__ __forceinline__ float8 ld_stream8(const float* p) {
    float8 v;
    asm volatile("ld.global.cs.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(v.lo.x), "=f"(v.lo.y), "=f"(v.lo.z), "=f"(v.lo.w), "=f"(v.hi.x), "=f"(v.hi.y), "=f"(v.hi.z), "=f"(v.hi.w)
                 : "l"(p)
                 : "memory");
    return v;
}
__device__ __forceinline__ void st_stream8(float* p, const float8& v) {
    asm volatile("st.global.cs.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(v.lo.x), "f"(v.lo.y), "f"(v.lo.z),
                 "f"(v.lo.w), "f"(v.hi.x), "f"(v.hi.y), "f"(v.hi.z), "f"(v.hi.w)
                 : "memory");
}
__device__ __forceinline__ void st_plain8(float* p, const float8& v) {
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(v.lo.x), "f"(v.lo.y), "f"(v.lo.z),
                 "f"(v.lo.w), "f"(v.hi.x), "f"(v.hi.y), "f"(v.hi.z), "f"(v.hi.w)
                 : "memory");
}

// ---------------------------------------------------------------- AdamW arithmetic

// Branch-free double-precision building blocks. CUDA's own IEEE division and square root carry a range check with
// a slow path, and that branch keeps the compiler from interleaving the eight independent elements a thread holds.
// The operands here are floats promoted to double and bias corrections in (0, 1], far from the exponent limits,
// so the checked range is not needed. Each routine ends in FMA residual corrections that make the result the
// correctly rounded one (Markstein's construction); the GPU tests compare every bit with IEEE division / sqrt.
// Operands must be finite: adamw_elem deals with an overflowed second moment before it gets here.
__device__ __forceinline__ double rcp_seed(double d) {
    double y;
    asm("rcp.approx.ftz.f64 %0, %1;" : "=d"(y) : "d"(d));
    return y;
}
__device__ __forceinline__ double rsqrt_seed(double x) {
    double y;
    asm("rsqrt.approx.ftz.f64 %0, %1;" : "=d"(y) : "d"(x));
    return y;
}
// a / b with y = RN(1 / b) supplied (b is a launch constant; the host rounds its reciprocal correctly).
__device__ __forceinline__ double div_by_const(double a, double b, double y) {
    double q = __dmul_rn(a, y);
    double r = __fma_rn(-b, q, a);
    q = __fma_rn(r, y, q);      // faithful
    r = __fma_rn(-b, q, a);
    return __fma_rn(r, y, q);   // correctly rounded
}
__device__ __forceinline__ double div_exact(double a, double d) {
    double y = rcp_seed(d);                     // ~20 bits
    double e = __fma_rn(-d, y, 1.0);
    y = __fma_rn(y, e, y);                      // ~40 bits
    e = __fma_rn(-d, y, 1.0);
    y = __fma_rn(y, e, y);                      // full precision, within an ulp
    e = __fma_rn(-d, y, 1.0);
    y = __fma_rn(y, e, y);                      // RN(1 / d)
    return div_by_const(a, d, y);
}
__device__ __forceinline__ double sqrt_exact(double x) {
    const double y = rsqrt_seed(x);             // ~20 bits of 1 / sqrt(x)
    double g = __dmul_rn(x, y), h = __dmul_rn(0.5, y);
    double r = __fma_rn(-g, h, 0.5);
    g = __fma_rn(g, r, g), h = __fma_rn(h, r, h);
    r = __fma_rn(-g, h, 0.5);
    g = __fma_rn(g, r, g), h = __fma_rn(h, r, h);
    double rem = __fma_rn(-g, g, x);
    g = __fma_rn(rem, h, g);
    rem = __fma_rn(-g, g, x);
    g = __fma_rn(rem, h, g);
    return x == 0.0 ? 0.0 : g;                  // the seed of 0 is inf; sqrt(0) is 0
}

// One element of the reference update (core/cuda/kernels.cu:242-250) with every rounding written out, so that the
// result does not depend on how a compiler contracts the expression: m and v in float with the products feeding
// an FMA, bias-corrected moments and the quotient in correctly rounded double, wd * p rounded in float before it
// is promoted, one final rounding of p to float.
// A gradient beyond about 1.8e19 overflows the float second moment to +inf. IEEE arithmetic then gives
// sqrt(inf) = inf and m / (inf + eps) = a zero with the sign of m (NaN when m is infinite too), where the Newton
// steps above would give NaN. That one case is decided on the float v and patched in with selects: the quotient
// becomes -0 (the neutral element of addition, signs included) and the signed zero, or NaN, of m * 0 is added to
// wd * p in float, which is exact.
__device__ __forceinline__ void adamw_elem(float& p, float g, float& m, float& v, const Hyper& h, float wd) {
    m = __fmaf_rn(h.b1, m, __fmul_rn(h.c1, g));
    v = __fmaf_rn(h.b2, v, __fmul_rn(__fmul_rn(h.c2, g), g));
    const bool overflowed = v == __int_as_float(0x7f800000);
    const float wdp = __fmul_rn(wd, p);
    const double decay = (double)(overflowed ? __fadd_rn(__fmul_rn(m, 0.0f), wdp) : wdp);
    const double mh = div_by_const((double)m, h.bc1, h.rbc1);
    const double vh = div_by_const((double)v, h.bc2, h.rbc2);
    double q = div_exact(mh, __dadd_rn(sqrt_exact(vh), (double)h.eps));
    q = overflowed ? -0.0 : q;
    p = __double2float_rn(__fma_rn(-(double)h.lr, __dadd_rn(q, decay), (double)p));
}
__device__ __forceinline__ void adamw_vec(float4& p, const float4& g, float4& m, float4& v, const Hyper& h, float wd) {
    adamw_elem(p.x, g.x, m.x, v.x, h, wd);
    adamw_elem(p.y, g.y, m.y, v.y, h, wd);
    adamw_elem(p.z, g.z, m.z, v.z, h, wd);
    adamw_elem(p.w, g.w, m.w, v.w, h, wd);
}
__device__ __forceinline__ float4 add4(const float4& a, const float4& b) {
    return make_float4(__fadd_rn(a.x, b.x), __fadd_rn(a.y, b.y), __fadd_rn(a.z, b.z), __fadd_rn(a.w, b.w));
}
__device__ __forceinline__ float4 mul4(const float4& a, float s) {
    return make_float4(__fmul_rn(a.x, s), __fmul_rn(a.y, s), __fmul_rn(a.z, s), __fmul_rn(a.w, s));
}
__device__ __forceinline__ float8 add8(const float8& a, const float8& b) {
    float8 r;
    r.lo = add4(a.lo, b.lo), r.hi = add4(a.hi, b.hi);
    return r;
}
__device__ __forceinline__ float8 mul8(const float8& a, float s) {
    float8 r;
    r.lo = mul4(a.lo, s), r.hi = mul4(a.hi, s);
    return r;
}
// acc += x^2 over the eight floats of v, in element order, in double (one FMA each).
__device__ __forceinline__ double sumsq8(double acc, const float8& v) {
    acc = __fma_rn((double)v.lo.x, (double)v.lo.x, acc);
    acc = __fma_rn((double)v.lo.y, (double)v.lo.y, acc);
    acc = __fma_rn((double)v.lo.z, (double)v.lo.z, acc);
    acc = __fma_rn((double)v.lo.w, (double)v.lo.w, acc);
    acc = __fma_rn((double)v.hi.x, (double)v.hi.x, acc);
    acc = __fma_rn((double)v.hi.y, (double)v.hi.y, acc);
    acc = __fma_rn((double)v.hi.z, (double)v.hi.z, acc);
    acc = __fma_rn((double)v.hi.w, (double)v.hi.w, acc);
    return acc;
}

// ---------------------------------------------------------------- segment lookup

// The segment a block is currently inside, held in registers; refilled only when a tile leaves its range. The
// peers' gradient pointers stay in the table: one warp-uniform, cached 8-byte load whenever one is needed.
struct SegView {
    float *p, *m, *v;
    float* gme;    // this rank's gradient
    float* gsrc;   // GATHER: the owner's gradient
    const Seg* sg;
    int64_t n;
    float wd, gscale;
    int hyper, vec;
    int first_tile, end_tile;  // [first, end) of this segment in the tile sequence
};

// Largest s with prefix[s] <= t (segments without elements share their successor's prefix and are skipped).
__device__ __forceinline__ int find_seg(const int* prefix, int nseg, int t) {
    int lo = 0, hi = nseg;  // invariant: prefix[lo] <= t < prefix[hi]
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (prefix[mid] <= t)
            lo = mid;
        else
            hi = mid;
    }
    return lo;
}

// Rank r's gradient of a segment, as mapped on this rank. The table does not change while a kernel runs.
__device__ __forceinline__ float* peer_grad(const Seg* sg, int r) {
    return reinterpret_cast<float*>(__ldg(reinterpret_cast<const unsigned long long*>(&sg->g[r])));
}

__device__ __forceinline__ void load_seg(SegView& s, const RankCtx& c, const int* prefix, int t, int me, int src) {
    const int i = find_seg(prefix, c.nseg, t);
    const Seg* sg = c.segs + i;
    s.sg = sg;
    s.p = sg->p, s.m = sg->m, s.v = sg->v;
    s.gme = peer_grad(sg, me);
    s.gsrc = peer_grad(sg, src);
    s.n = sg->n, s.wd = sg->wd, s.gscale = sg->gscale, s.hyper = sg->hyper, s.vec = sg->vec;
    s.first_tile = prefix[i], s.end_tile = prefix[i + 1];
}

// ---------------------------------------------------------------- one tile, every load issued up front

// Processes tile t of the sequence in the given mode. `stage` (one-shot only) is the base of the staging half in
// use on this rank; peers' halves come from c.stage[r] + stage_off. `ssq` collects the squares of the mean this
// tile produces (REDUCE_OWN of several ranks without an optimizer); untouched otherwise.
template <int W, bool ADAM, int MODE>
__device__ __forceinline__ void do_tile(const SegView& s, const LaunchArgs& a, const RankCtx& c, int t, int me,
                                        const float* stage, size_t stage_off, double& ssq) {
    constexpr bool SUMSQ = W > 1 && !ADAM && MODE == REDUCE_OWN;
    const int tid = threadIdx.x;
    const int64_t base = (int64_t)(t - s.first_tile) * kTile;
    const int64_t left = s.n - base;
    const int cnt = left < kTile ? (int)left : kTile;
    const int slot = a.stage_slot_floats;
    const Hyper& h = a.hp[s.hyper];
    const bool adam = ADAM && s.p != nullptr;
    if (s.vec && cnt == kTile) {
        // one 256-bit access per stream and thread; every load of the tile is issued before the first use
        static_assert(kTile == 8 * kThreads, "one float8 per thread and stream");
        const int e = tid * 8;
        const int64_t off = base + e;
        float8 gv[W], pv, mv, vv;
        if (MODE == REDUCE_OWN) {
            if (W == 1) {
                gv[0] = ld_stream8(s.gme + off);
            } else {
#pragma unroll
                for (int r = 0; r < W; r++) gv[r] = ld_sys8(peer_grad(s.sg, r) + off);
            }
        } else if (MODE == GATHER) {
            gv[0] = ld_sys8(s.gsrc + off);
        } else if (MODE == REDUCE_STAGED) {
#pragma unroll
            for (int r = 0; r < W; r++)
                gv[r] = r == me ? ld_sys8(s.gme + off) : ld_sys8(stage + (size_t)r * slot + (size_t)t * kTile + e);
        } else {
            gv[0] = ld_stream8(s.gme + off);
        }
        if (MODE != PUSH && adam) {
            pv = ld_stream8(s.p + off);
            mv = ld_stream8(s.m + off);
            vv = ld_stream8(s.v + off);
        }
        if (MODE == PUSH) {
#pragma unroll
            for (int r = 0; r < W; r++)
                if (r != me) st_plain8(c.stage[r] + stage_off + (size_t)me * slot + (size_t)t * kTile + e, gv[0]);
        } else {
            float8 avg = gv[0];
            if (MODE != GATHER && W > 1) {
#pragma unroll
                for (int r = 1; r < W; r++) avg = add8(avg, gv[r]);
                avg = mul8(avg, a.inv_world);
            }
            if (W == 1 && s.gscale != 1.0f) {  // clipped gradient: y = alpha * x in float, kept in place
                avg = mul8(avg, s.gscale);
                st_stream8(s.gme + off, avg);
            }
            if (W > 1) st_stream8(s.gme + off, avg);
            if (SUMSQ) ssq = sumsq8(ssq, avg);
            if (adam) {
                adamw_vec(pv.lo, avg.lo, mv.lo, vv.lo, h, s.wd);
                adamw_vec(pv.hi, avg.hi, mv.hi, vv.hi, h, s.wd);
                st_stream8(s.p + off, pv);
                st_stream8(s.m + off, mv);
                st_stream8(s.v + off, vv);
            }
        }
    } else {
        // partial tiles (a segment's tail, tensors smaller than a tile) and unaligned tensors: one float at a time
        for (int e = tid; e < cnt; e += kThreads) {
            const int64_t off = base + e;
            if (MODE == PUSH) {
                const float x = s.gme[off];
#pragma unroll
                for (int r = 0; r < W; r++)
                    if (r != me) c.stage[r][stage_off + (size_t)me * slot + (size_t)t * kTile + e] = x;
                continue;
            }
            float avg;
            if (MODE == GATHER) {
                avg = ld_sys1(s.gsrc + off);
            } else if (W == 1) {
                avg = s.gme[off];
            } else {
                float x[W];
#pragma unroll
                for (int r = 0; r < W; r++) {
                    if (MODE == REDUCE_OWN)
                        x[r] = ld_sys1(peer_grad(s.sg, r) + off);
                    else
                        x[r] = r == me ? ld_sys1(s.gme + off) : ld_sys1(stage + (size_t)r * slot + (size_t)t * kTile + e);
                }
                avg = x[0];
#pragma unroll
                for (int r = 1; r < W; r++) avg = __fadd_rn(avg, x[r]);
                avg = __fmul_rn(avg, a.inv_world);
            }
            if (W == 1 && s.gscale != 1.0f) {
                avg = __fmul_rn(s.gscale, avg);
                s.gme[off] = avg;
            }
            if (W > 1) s.gme[off] = avg;
            if (SUMSQ) ssq = __fma_rn((double)avg, (double)avg, ssq);
            if (adam) {
                float p = s.p[off], m = s.m[off], v = s.v[off];
                adamw_elem(p, avg, m, v, h, s.wd);
                s.p[off] = p, s.m[off] = m, s.v[off] = v;
            }
        }
    }
}

// A contiguous run of tiles in one mode, tile by tile (single-rank steps and both halves of one-shot).
template <int W, bool ADAM, int MODE>
__device__ __forceinline__ void do_run(const LaunchArgs& a, const RankCtx& c, const int* prefix, int t0, int t1, int me,
                                       int src, const float* stage, size_t stage_off) {
    SegView s;
    s.first_tile = 0, s.end_tile = 0;
    double unused = 0;
    for (int t = t0; t < t1; t++) {
        if (t >= s.end_tile || t < s.first_tile) load_seg(s, c, prefix, t, me, src);
        do_tile<W, ADAM, MODE>(s, a, c, t, me, stage, stage_off, unused);
    }
}

// ---------------------------------------------------------------- the two halves of two-shot

// The sum of squares of the mean a block produced since `first`: per thread in element order, then a fixed tree.
struct Piece {
    double acc;
    int first;
};
// Closes the open piece: the block's sum goes to entry `first` of every rank's partial table (the staging area,
// which two-shot launches do not use otherwise). The host adds a tensor's pieces in tile order. All threads call.
template <int W>
__device__ __forceinline__ void flush_piece(const RankCtx& c, Piece& pc, double* s_red) {
    double acc = pc.acc;
    for (int o = 16; o; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
    __syncthreads();  // the previous piece's s_red has been read
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0;
        for (int w = 0; w < kThreads / 32; w++) t += s_red[w];
        s_red[kThreads / 32] = t;
    }
    __syncthreads();
    // thread r tells rank r; the same thread later posts the flag that publishes this store to that rank
    if (threadIdx.x < W) reinterpret_cast<double*>(c.stage[threadIdx.x])[pc.first] = s_red[kThreads / 32];
    pc.acc = 0;
}

// Reduce half: the run [t0, t1) of this rank's own chunk. Mean in rank order, stored into the own gradient, and
// the update of the own p, m, v (ADAM) or the sum of squares of the mean (no optimizer) on the spot. A piece of
// the sum of squares ends where the segment changes and where the run ends.
template <int W, bool ADAM>
__device__ __forceinline__ void reduce_run(const LaunchArgs& a, const RankCtx& c, const int* prefix, int t0, int t1, int me,
                                           double* s_red) {
    const bool pieces = !ADAM && a.sumsq_on;
    SegView s;
    s.first_tile = 0, s.end_tile = 0;
    Piece pc;
    pc.acc = 0, pc.first = t0;
    for (int t = t0; t < t1; t++) {
        if (t >= s.end_tile || t < s.first_tile) {
            if (pieces && t > pc.first) flush_piece<W>(c, pc, s_red);
            load_seg(s, c, prefix, t, me, me);
            pc.first = t;
        }
        do_tile<W, ADAM, REDUCE_OWN>(s, a, c, t, me, nullptr, 0, pc.acc);
    }
    if (pieces && t1 > pc.first) flush_piece<W>(c, pc, s_red);
}

// ---------------------------------------------------------------- flag barriers

__device__ __forceinline__ size_t flag_index(int barrier, int block, int src) {
    return ((size_t)barrier * kFlagBlocks + block) * kMaxWorld + src;
}

// Tell every peer that this block of this rank reached `barrier` in launch `seq`.
template <int W>
__device__ __forceinline__ void post(const RankCtx& c, int barrier, int block, int me, unsigned seq) {
    __syncthreads();  // all of the block's stores come before the release below
    const int r = threadIdx.x;
    if (r < W && r != me) {
        __threadfence_system();
        st_release_sys(c.flags[r] + flag_index(barrier, block, me), seq);
    }
}

// Wait (bounded) until rank `src` posted `barrier` for this block index. src < 0 waits for every peer.
template <int W>
__device__ __forceinline__ void await(const RankCtx& c, const LaunchArgs& a, int barrier, int block, int me, int src,
                                      int code, int* s_abort) {
    const int r = threadIdx.x;
    if (r < W && r != me && (src < 0 || r == src)) {
        const unsigned* f = c.flags[me] + flag_index(barrier, block, r);
        const unsigned long long t0 = global_ns();
        while ((int)(ld_acquire_sys(f) - a.seq) < 0) {
            if (global_ns() - t0 > a.timeout_ns) {
                atomicCAS(c.status, 0, code);
                *s_abort = 1;
                break;
            }
            __nanosleep(32);
        }
    }
    __syncthreads();
}

__device__ __forceinline__ int cut(int total, int part, int parts) { return (int)((int64_t)total * part / parts); }

// Device time of block 0 at the borders of a launch's phases (start, peers present, own chunk reduced, all chunks
// gathered, peers done), for the host to read afterwards. Off when the rank context carries no stamp area.
__device__ __forceinline__ void stamp(const RankCtx& c, int block, int i) {
    if (c.stamps != nullptr && block == 0 && threadIdx.x == 0) c.stamps[i] = global_ns();
}

// ---------------------------------------------------------------- kernels

// Resident blocks per SM the single-rank kernel is compiled for (80 registers per thread).
constexpr int kLocalBlocksPerSm = 3;
template <int W, bool ADAM>
__global__ void __launch_bounds__(kThreads, W == 1 ? kLocalBlocksPerSm : 2) k_twoshot(const __grid_constant__ LaunchArgs a) {
    extern __shared__ int s_prefix[];
    __shared__ int s_abort;
    __shared__ double s_red[kThreads / 32 + 1];
    const int G = a.blocks_per_rank;
    const int b = blockIdx.x % G;
    const RankCtx& c = a.ctxs[blockIdx.x / G];
    const int me = c.rank, nseg = c.nseg;
    for (int i = threadIdx.x; i <= nseg; i += kThreads) s_prefix[i] = c.tile_prefix[i];
    if (threadIdx.x == 0) s_abort = 0;
    __syncthreads();
    const int T = s_prefix[nseg];

    if constexpr (W == 1) {
        if (a.cyclic > 0) {
            // block-cyclic order: block b takes groups b, b + G, ... of `cyclic` consecutive tiles, so that the
            // resident blocks walk through each tensor stream side by side instead of in G far-apart places
            const int C = a.cyclic, groups = (T + C - 1) / C;
            SegView s;
            s.first_tile = 0, s.end_tile = 0;
            double unused = 0;
            for (int j = b; j < groups; j += G) {
                const int t1 = (j + 1) * C < T ? (j + 1) * C : T;
                for (int t = j * C; t < t1; t++) {
                    if (t >= s.end_tile || t < s.first_tile) load_seg(s, c, s_prefix, t, me, me);
                    do_tile<W, ADAM, REDUCE_OWN>(s, a, c, t, me, nullptr, 0, unused);
                }
            }
        } else {
            do_run<W, ADAM, REDUCE_OWN>(a, c, s_prefix, cut(T, b, G), cut(T, b + 1, G), me, me, nullptr, 0);
        }
    } else {
        stamp(c, b, 0);
        post<W>(c, B_START, b, me, a.seq);
        await<W>(c, a, B_START, b, me, -1, ST_TIMEOUT_START, &s_abort);
        stamp(c, b, 1);
        {   // own chunk: reduce, scale, update
            const int cb = cut(T, me, W), ce = cut(T, me + 1, W), L = ce - cb;
            if (!s_abort) reduce_run<W, ADAM>(a, c, s_prefix, cb + cut(L, b, G), cb + cut(L, b + 1, G), me, s_red);
        }
        stamp(c, b, 2);
        post<W>(c, B_REDUCED, b, me, a.seq);
        for (int k = 1; k < W; k++) {  // other chunks, starting after the own one so that owners are hit evenly
            const int src = (me + k) % W;
            await<W>(c, a, B_REDUCED, b, me, src, ST_TIMEOUT_REDUCED, &s_abort);
            const int cb = cut(T, src, W), ce = cut(T, src + 1, W), L = ce - cb;
            if (!s_abort) do_run<W, ADAM, GATHER>(a, c, s_prefix, cb + cut(L, b, G), cb + cut(L, b + 1, G), me, src, nullptr, 0);
        }
        stamp(c, b, 3);
        // nobody may reuse or free gradient memory that a peer is still reading
        post<W>(c, B_DONE, b, me, a.seq);
        await<W>(c, a, B_DONE, b, me, -1, ST_TIMEOUT_DONE, &s_abort);
        stamp(c, b, 4);
    }
}

template <int W, bool ADAM>
__global__ void __launch_bounds__(kThreads, 2) k_oneshot(const __grid_constant__ LaunchArgs a) {
    extern __shared__ int s_prefix[];
    __shared__ int s_abort;
    const int G = a.blocks_per_rank;
    const int b = blockIdx.x % G;
    const RankCtx& c = a.ctxs[blockIdx.x / G];
    const int me = c.rank, nseg = c.nseg;
    for (int i = threadIdx.x; i <= nseg; i += kThreads) s_prefix[i] = c.tile_prefix[i];
    if (threadIdx.x == 0) s_abort = 0;
    __syncthreads();
    const int T = s_prefix[nseg];
    const int t0 = cut(T, b, G), t1 = cut(T, b + 1, G);
    // Staging is double-buffered by launch parity: a peer that already runs the next one-shot launch writes the
    // other half, and it cannot be two launches ahead because it waits for this rank's flag in between.
    const size_t stage_off = (size_t)a.parity * W * a.stage_slot_floats;
    do_run<W, ADAM, PUSH>(a, c, s_prefix, t0, t1, me, me, nullptr, stage_off);
    post<W>(c, B_REDUCED, b, me, a.seq);
    await<W>(c, a, B_REDUCED, b, me, -1, ST_TIMEOUT_REDUCED, &s_abort);
    if (!s_abort) do_run<W, ADAM, REDUCE_STAGED>(a, c, s_prefix, t0, t1, me, me, c.stage[me] + stage_off, stage_off);
}

// ---------------------------------------------------------------- small elementwise kernels next to the path

// y = alpha * x (core/cuda/kernels.cu:208-212), y += alpha * x (sl_cuda_axpy), p = value (k_fill, :127-131).
__global__ void __launch_bounds__(kThreads) k_scale(int64_t n, const float* x, float* y, float alpha) {
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kThreads)
        y[i] = __fmul_rn(alpha, x[i]);
}
__global__ void __launch_bounds__(kThreads) k_axpy(int64_t n, const float* x, float* y, float alpha) {
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kThreads)
        y[i] = __fmaf_rn(alpha, x[i], y[i]);
}
__global__ void __launch_bounds__(kThreads) k_fill(int64_t n, float* p, float value) {
    for (int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kThreads)
        p[i] = value;
}

// Sum of squares, deterministic: block b owns the fixed slice [n*b/B, n*(b+1)/B), a thread accumulates its strided
// elements in double, warps combine by shuffle in a fixed tree, warp results are added in warp order.
__global__ void __launch_bounds__(kThreads) k_sumsq(int64_t n, const float* x, double* partials) {
    __shared__ double s_warp[kThreads / 32];
    const int64_t lo = n / gridDim.x * blockIdx.x + (n % gridDim.x) * blockIdx.x / gridDim.x;
    const int64_t hi = n / gridDim.x * (blockIdx.x + 1) + (n % gridDim.x) * (blockIdx.x + 1) / gridDim.x;
    double acc = 0;
    for (int64_t i = lo + threadIdx.x; i < hi; i += kThreads) {
        const double v = (double)x[i];
        acc = __fma_rn(v, v, acc);
    }
    for (int o = 16; o; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31) == 0) s_warp[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        double t = 0;
        for (int w = 0; w < kThreads / 32; w++) t += s_warp[w];
        partials[blockIdx.x] = t;
    }
}

// Sum of squares of many tensors in one launch: slice i (at most kSumsqSlice floats of one tensor) is summed by one
// block in the same fixed order as k_sumsq, blocks take slices round robin; the host adds a tensor's partials in
// slice order. Nothing depends on scheduling.
__global__ void __launch_bounds__(kThreads) k_sumsq_slices(int nslices, const SumsqSlice* slices, double* partials) {
    __shared__ double s_warp[kThreads / 32];
    for (int i = blockIdx.x; i < nslices; i += gridDim.x) {
        const float* x = slices[i].x;
        const int64_t n = slices[i].n;
        double acc = 0;
        for (int64_t e = threadIdx.x; e < n; e += kThreads) {
            const double v = (double)x[e];
            acc = __fma_rn(v, v, acc);
        }
        for (int o = 16; o; o >>= 1) acc += __shfl_down_sync(0xffffffffu, acc, o);
        __syncthreads();  // the previous slice's s_warp has been read
        if ((threadIdx.x & 31) == 0) s_warp[threadIdx.x >> 5] = acc;
        __syncthreads();
        if (threadIdx.x == 0) {
            double t = 0;
            for (int w = 0; w < kThreads / 32; w++) t += s_warp[w];
            partials[i] = t;
        }
    }
}

// ---------------------------------------------------------------- launch

template <int W, bool ADAM>
static void (*kernel_of(int kind))(const LaunchArgs) {
    return kind == KERNEL_ONESHOT ? k_oneshot<W, ADAM> : k_twoshot<W, ADAM>;
}

template <int W, bool ADAM>
static cudaError_t launch_w(int kind, bool cooperative, int grid, size_t smem, const LaunchArgs& a, cudaStream_t st) {
    void (*kern)(const LaunchArgs) = kernel_of<W, ADAM>(kind);
    if (cooperative) {
        void* params[] = {const_cast<LaunchArgs*>(&a)};
        return cudaLaunchCooperativeKernel((const void*)kern, dim3(grid), dim3(kThreads), params, smem, st);
    }
    kern<<<grid, kThreads, smem, st>>>(a);
    return cudaPeekAtLastError();
}

template <int W, bool ADAM>
static int occupancy_w(int kind, size_t smem) {
    int n = 0;
    void (*kern)(const LaunchArgs) = kernel_of<W, ADAM>(kind);
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, (const void*)kern, kThreads, smem) != cudaSuccess) return 0;
    return n;
}

#define SLB_DISPATCH(W_, fn, ...)                                        \
    switch (W_) {                                                        \
        case 1: return adam ? fn<1, true>(__VA_ARGS__) : fn<1, false>(__VA_ARGS__); \
        case 2: return adam ? fn<2, true>(__VA_ARGS__) : fn<2, false>(__VA_ARGS__); \
        case 3: return adam ? fn<3, true>(__VA_ARGS__) : fn<3, false>(__VA_ARGS__); \
        case 4: return adam ? fn<4, true>(__VA_ARGS__) : fn<4, false>(__VA_ARGS__); \
        case 5: return adam ? fn<5, true>(__VA_ARGS__) : fn<5, false>(__VA_ARGS__); \
        case 6: return adam ? fn<6, true>(__VA_ARGS__) : fn<6, false>(__VA_ARGS__); \
        case 7: return adam ? fn<7, true>(__VA_ARGS__) : fn<7, false>(__VA_ARGS__); \
        case 8: return adam ? fn<8, true>(__VA_ARGS__) : fn<8, false>(__VA_ARGS__); \
    }

int launch_step(int world, bool adam, int kind, bool cooperative, int grid, size_t smem, const LaunchArgs& a, cudaStream_t st) {
    SLB_DISPATCH(world, launch_w, kind, cooperative, grid, smem, a, st)
    return (int)cudaErrorInvalidValue;
}

int step_occupancy(int world, bool adam, int kind, size_t smem) {
    SLB_DISPATCH(world, occupancy_w, kind, smem)
    return 0;
}

static int flat_grid(int64_t n) {
    int64_t g = (n + kThreads - 1) / kThreads;
    return (int)(g < 1 ? 1 : g > 148 * 8 ? 148 * 8 : g);
}
int launch_scale(const float* x, float* y, int64_t n, float alpha, cudaStream_t st) {
    if (n <= 0) return 0;
    k_scale<<<flat_grid(n), kThreads, 0, st>>>(n, x, y, alpha);
    return (int)cudaPeekAtLastError();
}
int launch_axpy(const float* x, float* y, int64_t n, float alpha, cudaStream_t st) {
    if (n <= 0) return 0;
    k_axpy<<<flat_grid(n), kThreads, 0, st>>>(n, x, y, alpha);
    return (int)cudaPeekAtLastError();
}
int launch_fill(float* p, int64_t n, float value, cudaStream_t st) {
    if (n <= 0) return 0;
    k_fill<<<flat_grid(n), kThreads, 0, st>>>(n, p, value);
    return (int)cudaPeekAtLastError();
}

int launch_sumsq_slices(int nslices, const SumsqSlice* slices, double* partials, int blocks, cudaStream_t st) {
    if (nslices <= 0) return 0;
    k_sumsq_slices<<<blocks < nslices ? blocks : nslices, kThreads, 0, st>>>(nslices, slices, partials);
    return (int)cudaPeekAtLastError();
}
int launch_sumsq_partials(const float* x, int64_t n, double* partials, int blocks, cudaStream_t st) {
    k_sumsq<<<blocks, kThreads, 0, st>>>(n, x, partials);
    return (int)cudaPeekAtLastError();
}

}  // namespace slb

// ---------------------------------------------------------------- a fused AdamW step that allocates nothing

namespace slb {

// Some callers cannot let this library take device memory on their behalf. The case this was written for is a host
// runtime that owns the whole device heap and plans it ahead of time -- Soliton's core does: every device byte goes
// through its pool so that a dry run predicts the peak exactly, and an allocation made behind its back would make
// that prediction wrong. Such a caller may also not have handed the library a workspace (sl_init_device or
// sl_cuda_dp_set_workspace), which every other entry point of the path needs for its segment table.
//
// slb_adamw_step_static is the multi-tensor AdamW step (the k_twoshot<1, true> kernel, same arithmetic, same bits)
// with that table in a fixed array that is part of the library image instead: kStaticMaxSegs tensors per call at
// most, 59,904 bytes of device memory per GPU that loads the library, held until the process exits. The entry
// point calls no cudaMalloc / cudaFree and nothing that allocates on its behalf; the table image is built in a
// static host buffer and copied over with one cudaMemcpyAsync on the legacy default stream, ahead of the launch.
//
// The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that device
// current) and remembers it; make that first call outside any stream capture. All calls share the one array, which
// keeps the previous call's table: every call overwrites the part it uses, including the status word that must start
// at zero, so stale contents are harmless -- but two calls whose kernels overlap on the GPU (launched from different
// threads or processes' streams that are not ordered with the legacy stream) would race on it. Calls from one thread
// are ordered by the stream and safe.
constexpr int kStaticMaxSegs = 512;
constexpr size_t kStaticStatusOff = 192;   // behind the RankCtx (176 bytes)
constexpr size_t kStaticPrefixOff = 256;   // (kStaticMaxSegs + 1) ints
constexpr size_t kStaticSegOff = 2560;
constexpr size_t kStaticBytes = kStaticSegOff + size_t(kStaticMaxSegs) * sizeof(Seg);
static_assert(sizeof(RankCtx) <= kStaticStatusOff, "static scratch layout");
static_assert(kStaticPrefixOff + (kStaticMaxSegs + 1) * sizeof(int) <= kStaticSegOff, "static scratch layout");

static __device__ __align__(256) unsigned char g_static_step_scratch[kStaticBytes];

// Device address of the array on the current device, looked up once per device. In host code the array's name is
// only a handle for this lookup, never a pointer a kernel could use.
static unsigned char* static_scratch_address() {
    constexpr int kMaxDevices = 64;
    static unsigned char* cached[kMaxDevices] = {nullptr};
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
    if (!cached[dev]) {
        void* ptr = nullptr;
        if (cudaGetSymbolAddress(&ptr, g_static_step_scratch) != cudaSuccess || !ptr) {
            cudaGetLastError();
            return nullptr;
        }
        cached[dev] = static_cast<unsigned char*>(ptr);
    }
    return cached[dev];
}

}  // namespace slb

// 0 on success; -1 bad argument; -2 more tensors (or tiles) than the fixed table holds; -3 a CUDA call failed.
extern "C" int slb_adamw_step_static(int nseg, float* const* p, const float* const* g, float* const* m, float* const* v,
                                     const int64_t* n, const float* wd, float lr, float b1, float b2, float eps,
                                     int step) {
    using namespace slb;
    if (nseg < 1 || !p || !g || !m || !v || !n || step < 1) return -1;
    if (nseg > kStaticMaxSegs) return -2;
    // Work the engine has recorded but not launched yet (a gradient mean, an in-place clip scale, batched sl_adamw
    // calls) comes first in stream order, as it came first in call order. Launches planned work only: no allocation.
    engine_flush_pending();
    unsigned char* dev = static_scratch_address();
    if (!dev) return -3;

    static unsigned char image[kStaticBytes];  // host copy of the part of the array this call uses
    RankCtx* ctx = reinterpret_cast<RankCtx*>(image);
    int* prefix = reinterpret_cast<int*>(image + kStaticPrefixOff);
    Seg* segs = reinterpret_cast<Seg*>(image + kStaticSegOff);
    memset(image, 0, kStaticSegOff);  // context, status word (must start at zero), prefix
    int64_t tiles = 0;
    for (int s = 0; s < nseg; s++) {
        if (n[s] < 0) return -1;
        const uintptr_t bits = reinterpret_cast<uintptr_t>(p[s]) | reinterpret_cast<uintptr_t>(g[s]) |
                               reinterpret_cast<uintptr_t>(m[s]) | reinterpret_cast<uintptr_t>(v[s]);
        if (n[s] > 0 && (!p[s] || !g[s] || !m[s] || !v[s] || (bits & 3))) return -1;
        Seg& d = segs[s];
        memset(&d, 0, sizeof d);
        d.p = p[s], d.m = m[s], d.v = v[s], d.g[0] = const_cast<float*>(g[s]);
        d.n = n[s], d.wd = wd ? wd[s] : 0.0f, d.hyper = 0, d.vec = (bits & 31) == 0, d.gscale = 1.0f;
        prefix[s] = (int)tiles;
        tiles += (n[s] + kTile - 1) / kTile;
        if (tiles > 0x7fffffff) return -2;
    }
    prefix[nseg] = (int)tiles;
    if (tiles == 0) return 0;
    ctx->segs = reinterpret_cast<const Seg*>(dev + kStaticSegOff);
    ctx->tile_prefix = reinterpret_cast<const int*>(dev + kStaticPrefixOff);
    ctx->nseg = nseg, ctx->rank = 0, ctx->world = 1;
    ctx->flags[0] = nullptr, ctx->stage[0] = nullptr, ctx->stamps = nullptr;
    ctx->status = reinterpret_cast<int*>(dev + kStaticStatusOff);
    const size_t used = kStaticSegOff + (size_t)nseg * sizeof(Seg);
    if (cudaMemcpyAsync(dev, image, used, cudaMemcpyHostToDevice, 0) != cudaSuccess) {
        cudaGetLastError();
        return -3;
    }

    int device = 0, sms = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess)
        return -3;
    const size_t smem = (size_t)(nseg + 1) * sizeof(int);
    const int per_sm = step_occupancy(1, true, KERNEL_PLAIN, smem);
    if (per_sm < 1 || sms < 1) return -3;
    const int64_t cap = (int64_t)per_sm * sms;
    LaunchArgs a{};
    a.ctxs = reinterpret_cast<const RankCtx*>(dev);
    a.blocks_per_rank = (int)(tiles < cap ? tiles : cap);
    a.inv_world = 1.0f;
    Hyper& h = a.hp[0];
    h.bc1 = 1.0 - pow((double)b1, (double)step), h.bc2 = 1.0 - pow((double)b2, (double)step);
    h.rbc1 = 1.0 / h.bc1, h.rbc2 = 1.0 / h.bc2;
    h.lr = lr, h.b1 = b1, h.b2 = b2, h.eps = eps, h.c1 = 1 - b1, h.c2 = 1 - b2;
    a.cyclic = 0;
    if (launch_step(1, true, KERNEL_PLAIN, false, a.blocks_per_rank, smem, a, 0) != 0) return -3;
    engine_count_launch();
    return 0;
}

