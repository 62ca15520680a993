// Cross entropy over rows of logits (fused softmax + negative log likelihood), forward and backward.
//
// Same backend-level names and signatures as the reference's CUDA file (core/cuda/kernels.cu:488-534). Both
// directions are bandwidth-bound: GPT-2's logits are 8,192 rows of 50,257 floats, 1.65 GB. The reference walks a row
// with 256 threads and scalar loads three times (maximum, sum of exponentials, gradient). Here a block of 512 threads
// reads the row ONCE for both statistics (a running maximum with the sum rescaled when it moves), in 128-bit loads
// from the first 16-byte boundary of the row -- rows of an odd length start at every alignment -- and the backward
// pass keeps the row in shared memory (a row is 201 KB; L2 does not hold the rows in flight next to the gradient
// being written: measured, a second global read costs 0.94 of a second DRAM read) while it writes the gradient, the
// target's `- g` folded into the store that owns it. Longer rows are read twice. The mean of the row losses is summed
// on the device in double precision in a fixed order, so that the blocking copy to the host is 8 bytes instead of
// one float per row.
//
// Algorithmic traffic: forward 4 B per logit, backward 8 B per logit (read, write).
#include <cooperative_groups.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <vector>

#include "../../include/soliton_b200.h"
#include "dp_engine.hpp"

namespace slb_xent {

constexpr int kThreads = 512;

// Running (maximum, sum of exp(x - maximum)). A maximum of -inf carries a sum of 0.
struct Stat {
    float m, z;
};
__device__ __forceinline__ void take(Stat& s, float4 x) {
    const float cm = fmaxf(fmaxf(x.x, x.y), fmaxf(x.z, x.w));
    if (cm > s.m) {
        s.z *= __expf(s.m - cm);  // first time: 0 * exp(-inf) = 0
        s.m = cm;
    }
    s.z += (__expf(x.x - s.m) + __expf(x.y - s.m)) + (__expf(x.z - s.m) + __expf(x.w - s.m));
}
__device__ __forceinline__ void take(Stat& s, float x) {
    if (x > s.m) {
        s.z *= __expf(s.m - x);
        s.m = x;
    }
    s.z += __expf(x - s.m);
}
__device__ __forceinline__ Stat merge(Stat a, Stat b) {
    const float m = fmaxf(a.m, b.m);
    if (m == -INFINITY) return Stat{m, 0.0f};
    return Stat{m, a.z * __expf(a.m - m) + b.z * __expf(b.m - m)};
}

// How a row splits into a scalar head up to the first 16-byte boundary, 128-bit words, and a scalar tail.
struct Span {
    int head;
    int64_t words, tail0;
};
__device__ __forceinline__ Span span_of(const float* row, int64_t v) {
    Span s;
    const int64_t h = (4 - (int)((reinterpret_cast<uintptr_t>(row) >> 2) & 3)) & 3;
    s.head = (int)(h < v ? h : v);
    s.words = (v - s.head) >> 2;
    s.tail0 = s.head + 4 * s.words;
    return s;
}

// Maximum and sum of exponentials of one row, on every thread of the block. One pass over the row; with STASH the
// 128-bit words go into shared memory first, word i by the thread that reads it back.
template <int THREADS, bool STASH>
__device__ __forceinline__ Stat row_stat(const float* __restrict__ row, int64_t v, const Span sp, float4* stash) {
    constexpr int WARPS = THREADS / 32;
    __shared__ Stat part[WARPS];
    __shared__ Stat total;
    Stat s{-INFINITY, 0.0f};
    const float4* w = reinterpret_cast<const float4*>(row + sp.head);
    if constexpr (STASH) {
        // every word of the row is requested before the first one is waited for: asynchronous 16-byte copies from
        // global into shared memory, no registers in between, the whole row in flight per SM
        for (int64_t i = threadIdx.x; i < sp.words; i += THREADS) {
            const unsigned dst = (unsigned)__cvta_generic_to_shared(stash + i);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(w + i) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");  // a thread reads back only the words it asked for
        for (int64_t i = threadIdx.x; i < sp.words; i += THREADS) take(s, stash[i]);
    } else {
        int64_t i = threadIdx.x;
        for (; i + 3 * THREADS < sp.words; i += 4 * THREADS) {
            const float4 a = w[i], b = w[i + THREADS], c = w[i + 2 * THREADS], d = w[i + 3 * THREADS];
            take(s, a), take(s, b), take(s, c), take(s, d);
        }
        for (; i < sp.words; i += THREADS) take(s, w[i]);
    }
    if ((int)threadIdx.x < sp.head) take(s, row[threadIdx.x]);
    if (sp.tail0 + threadIdx.x < v) take(s, row[sp.tail0 + threadIdx.x]);
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        Stat other;
        other.m = __shfl_xor_sync(0xffffffffu, s.m, o);
        other.z = __shfl_xor_sync(0xffffffffu, s.z, o);
        s = merge(s, other);
    }
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        Stat t = part[0];
        for (int k = 1; k < WARPS; k++) t = merge(t, part[k]);  // warp order: the same bits every run
        total = t;
    }
    __syncthreads();
    return total;
}

// rowloss[r] = log(sum exp) + max - logit of the target (core/cuda/kernels.cu:490-501)
__global__ void __launch_bounds__(kThreads) k_xent_rows(const float* __restrict__ logits, const int* __restrict__ t,
                                                        float* __restrict__ rowloss, int64_t v) {
    const int64_t r = blockIdx.x;
    const float* row = logits + r * v;
    const Stat s = row_stat<kThreads, false>(row, v, span_of(row, v), nullptr);
    if (threadIdx.x == 0) rowloss[r] = logf(s.z) + s.m - row[t[r]];
}

// The sum of n row losses in double precision, thread-strided partials and a tree in shared memory: a fixed order.
// The mean overwrites the first 8 bytes of the row losses.
__global__ void __launch_bounds__(1024) k_xent_mean(float* rowloss, int64_t n) {
    __shared__ double part[1024];
    double s = 0;
    for (int64_t i = threadIdx.x; i < n; i += 1024) s += (double)rowloss[i];
    part[threadIdx.x] = s;
    __syncthreads();
    for (int o = 512; o; o >>= 1) {
        if ((int)threadIdx.x < o) part[threadIdx.x] += part[threadIdx.x + o];
        __syncthreads();
    }
    if (threadIdx.x == 0) *reinterpret_cast<double*>(rowloss) = part[0] / (double)n;
}

// dl[r][j] = exp(logit - max) * g / sum, minus g at the target (core/cuda/kernels.cu:514-530)
__global__ void __launch_bounds__(kThreads) k_xent_bwd_rows(const float* __restrict__ logits, const int* __restrict__ t,
                                                            float* __restrict__ dl, int64_t v, float g) {
    const int64_t r = blockIdx.x;
    const float* row = logits + r * v;
    float* out = dl + r * v;
    const Span sp = span_of(row, v);
    const Stat s = row_stat<kThreads, false>(row, v, sp, nullptr);
    const float scale = g / s.z, m = s.m;
    const int64_t target = t[r];
    if ((reinterpret_cast<uintptr_t>(out + sp.head) & 15) == 0) {
        const float4* w = reinterpret_cast<const float4*>(row + sp.head);
        float4* o = reinterpret_cast<float4*>(out + sp.head);
        const int64_t tw = target >= sp.head && target < sp.tail0 ? (target - sp.head) >> 2 : -1;  // the word of the target
        const int tk = (int)((target - sp.head) & 3);
#pragma unroll 4
        for (int64_t i = threadIdx.x; i < sp.words; i += kThreads) {
            const float4 x = w[i];
            float4 y = make_float4(__expf(x.x - m) * scale, __expf(x.y - m) * scale, __expf(x.z - m) * scale, __expf(x.w - m) * scale);
            if (i == tw) {
                if (tk == 0) y.x -= g; else if (tk == 1) y.y -= g; else if (tk == 2) y.z -= g; else y.w -= g;
            }
            __stcs(o + i, y);  // 1.65 GB of gradient: streamed past L2's resident lines
        }
        if ((int)threadIdx.x < sp.head) out[threadIdx.x] = __expf(row[threadIdx.x] - m) * scale - (threadIdx.x == target ? g : 0.0f);
        const int64_t j = sp.tail0 + threadIdx.x;
        if (j < v) out[j] = __expf(row[j] - m) * scale - (j == target ? g : 0.0f);
    } else {  // the gradient's row sits at another alignment than the logits': scalar stores
        for (int64_t j = threadIdx.x; j < v; j += kThreads) out[j] = __expf(row[j] - m) * scale - (j == target ? g : 0.0f);
    }
}

// The same with the row kept on chip between the two passes, so that DRAM sees one read and one write of it. A
// row (201 KB for GPT-2's 50,257 logits) is split over a thread-block cluster of C blocks: each block copies its part
// into shared memory with asynchronous 16-byte copies (every word requested before the first is waited for), forms
// the statistics of its part, hands them to every block of the cluster through distributed shared memory, and after
// one cluster barrier all blocks merge the C parts in rank order -- the same bits in every block. With a part of a
// row per block an SM holds parts of several rows in different phases, so reads, arithmetic and writes overlap. Only
// for gradients whose rows sit at the same 16-byte phase as the logits' (the caller checks).
template <int C, int THREADS>
__global__ void __launch_bounds__(THREADS) k_xent_bwd_rows_cluster(const float* __restrict__ logits, const int* __restrict__ t,
                                                                   float* __restrict__ dl, int64_t v, float g) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    extern __shared__ float4 stash[];
    __shared__ Stat part[THREADS / 32];
    __shared__ Stat all[C];
    const unsigned k = cluster.block_rank();
    const int64_t r = blockIdx.x / C;
    const float* row = logits + r * v;
    float* out = dl + r * v;
    const Span sp = span_of(row, v);
    const int64_t w0 = sp.words * k / C, nw = sp.words * (k + 1) / C - w0;
    const float4* w = reinterpret_cast<const float4*>(row + sp.head) + w0;
    for (int64_t i = threadIdx.x; i < nw; i += THREADS) {
        const unsigned dst = (unsigned)__cvta_generic_to_shared(stash + i);
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(w + i) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    cluster.sync();  // every block of the cluster is running before any of them writes into another's shared memory
    asm volatile("cp.async.wait_group 0;" ::: "memory");  // a thread reads back only the words it asked for
    Stat s{-INFINITY, 0.0f};
    for (int64_t i = threadIdx.x; i < nw; i += THREADS) take(s, stash[i]);
    if (k == 0 && (int)threadIdx.x < sp.head) take(s, row[threadIdx.x]);
    if (k == C - 1 && sp.tail0 + threadIdx.x < v) take(s, row[sp.tail0 + threadIdx.x]);
#pragma unroll
    for (int o = 16; o; o >>= 1) {
        Stat other;
        other.m = __shfl_xor_sync(0xffffffffu, s.m, o);
        other.z = __shfl_xor_sync(0xffffffffu, s.z, o);
        s = merge(s, other);
    }
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        Stat mine = part[0];
        for (int q = 1; q < THREADS / 32; q++) mine = merge(mine, part[q]);
        for (int c = 0; c < C; c++) *cluster.map_shared_rank(&all[k], c) = mine;
    }
    cluster.sync();  // every block has every part; nothing remote is touched after this
    s = all[0];
#pragma unroll
    for (int c = 1; c < C; c++) s = merge(s, all[c]);
    const float scale = g / s.z, m = s.m;
    const int64_t target = t[r];
    float4* o = reinterpret_cast<float4*>(out + sp.head) + w0;
    const int64_t tw = target >= sp.head && target < sp.tail0 ? ((target - sp.head) >> 2) - w0 : -1;  // the word of the target
    const int tk = (int)((target - sp.head) & 3);
#pragma unroll 4
    for (int64_t i = threadIdx.x; i < nw; i += THREADS) {
        const float4 x = stash[i];
        float4 y = make_float4(__expf(x.x - m) * scale, __expf(x.y - m) * scale, __expf(x.z - m) * scale, __expf(x.w - m) * scale);
        if (i == tw) {
            if (tk == 0) y.x -= g; else if (tk == 1) y.y -= g; else if (tk == 2) y.z -= g; else y.w -= g;
        }
        __stcs(o + i, y);
    }
    if (k == 0 && (int)threadIdx.x < sp.head) out[threadIdx.x] = __expf(row[threadIdx.x] - m) * scale - (threadIdx.x == target ? g : 0.0f);
    const int64_t j = sp.tail0 + threadIdx.x;
    if (k == C - 1 && j < v) out[j] = __expf(row[j] - m) * scale - (j == target ? g : 0.0f);
}
constexpr size_t kMaxStashBytes = 100 * 1024;  // per block: two blocks per SM at the least

template <int C, int THREADS>
static cudaError_t launch_cluster(const float* logits, const int* t, float* dl, int64_t n, int64_t v, float g) {
    const size_t stash = (size_t)(v / 4 / C + 2) * sizeof(float4);
    static const cudaError_t allowed = cudaFuncSetAttribute((const void*)k_xent_bwd_rows_cluster<C, THREADS>,
                                                            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxStashBytes);
    if (allowed != cudaSuccess || stash > kMaxStashBytes) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(n * C));
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = stash;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = C, attr.val.clusterDim.y = 1, attr.val.clusterDim.z = 1;
    cfg.attrs = &attr, cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, k_xent_bwd_rows_cluster<C, THREADS>, logits, t, dl, v, g);
}

static void report(cudaError_t e, int code) {
    if (e != cudaSuccess) slb::Engine::get().set_error(code);
}

}  // namespace slb_xent

using namespace slb_xent;

extern "C" double sl_cuda_cross_entropy(const float* logits, const int* t, int64_t n, int64_t v, float* rowloss) {
    if (n <= 0 || v <= 0) return std::nan("");  // the reference divides 0 by 0 here
    k_xent_rows<<<(unsigned)n, kThreads>>>(logits, t, rowloss, v);
    report(cudaPeekAtLastError(), slb::ERR_LAUNCH);
    if (n >= 2 && (reinterpret_cast<uintptr_t>(rowloss) & 7) == 0) {
        k_xent_mean<<<1, 1024>>>(rowloss, n);
        report(cudaPeekAtLastError(), slb::ERR_LAUNCH);
        double mean = std::nan("");
        report(cudaMemcpy(&mean, rowloss, sizeof(double), cudaMemcpyDeviceToHost), slb::ERR_SYNC);
        return mean;
    }
    std::vector<float> host((size_t)n);
    report(cudaMemcpy(host.data(), rowloss, (size_t)n * sizeof(float), cudaMemcpyDeviceToHost), slb::ERR_SYNC);
    double s = 0;
    for (float x : host) s += x;
    return s / (double)n;
}

extern "C" void sl_cuda_cross_entropy_bwd(const float* logits, const int* t, float* dl, int64_t n, int64_t v, float dloss) {
    if (n <= 0 || v <= 0) return;
    const float g = dloss / (float)n;
    // Rows of logits and of the gradient start at the same 16-byte phase when the two bases do (row r of both is
    // r * v floats in); then a row that fits is kept in shared memory between its two passes.
    const bool same_phase = ((reinterpret_cast<uintptr_t>(logits) ^ reinterpret_cast<uintptr_t>(dl)) & 15) == 0;
    if (same_phase && v >= 4096 && n * 8 < (int64_t)1 << 31) {
        // clusters of 4 (measured: 2 is no faster than reading twice, 8 equals 4); of 8 for rows up to twice as long
        cudaError_t e = launch_cluster<4, 256>(logits, t, dl, n, v, g);
        if (e != cudaSuccess) (void)cudaGetLastError(), e = launch_cluster<8, 256>(logits, t, dl, n, v, g);
        if (e == cudaSuccess) return;
        (void)cudaGetLastError();  // too long a row for a cluster's shared memory: the two-read kernel takes it
    }
    k_xent_bwd_rows<<<(unsigned)n, kThreads>>>(logits, t, dl, v, g);
    report(cudaPeekAtLastError(), slb::ERR_LAUNCH);
}
