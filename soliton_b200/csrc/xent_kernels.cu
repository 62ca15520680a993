// Cross entropy over rows of logits (fused softmax + negative log likelihood), forward and backward.
//
// Same backend-level names and signatures as the reference's CUDA file (core/cuda/kernels.cu:488-534). Both
// directions are bandwidth-bound: GPT-2's logits are 8,192 rows of 50,257 floats, 1.65 GB. The reference walks a row
// with 256 threads and scalar loads three times (maximum, sum of exponentials, gradient). Here a block of 512 threads
// reads the row ONCE for both statistics (a running maximum with the sum rescaled when it moves), in 128-bit loads
// from the first 16-byte boundary of the row -- rows of an odd length start at every alignment -- and the backward
// pass reads it a second time out of L2 (a row is 201 KB) while it writes the gradient, the target's `- g` folded into
// the store that owns it. The mean of the row losses is summed on the device in double precision in a fixed order, so
// that the blocking copy to the host is 8 bytes instead of one float per row.
//
// Algorithmic traffic: forward 4 B per logit, backward 8 B per logit (read, write).
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <vector>

#include "../../include/soliton_b200.h"
#include "dp_engine.hpp"

namespace slb_xent {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;

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

// Maximum and sum of exponentials of one row, on every thread of the block. One pass over the row.
__device__ __forceinline__ Stat row_stat(const float* __restrict__ row, int64_t v, const Span sp) {
    __shared__ Stat part[kWarps];
    __shared__ Stat total;
    Stat s{-INFINITY, 0.0f};
    const float4* w = reinterpret_cast<const float4*>(row + sp.head);
    int64_t i = threadIdx.x;
    for (; i + 3 * kThreads < sp.words; i += 4 * kThreads) {
        const float4 a = w[i], b = w[i + kThreads], c = w[i + 2 * kThreads], d = w[i + 3 * kThreads];
        take(s, a), take(s, b), take(s, c), take(s, d);
    }
    for (; i < sp.words; i += kThreads) take(s, w[i]);
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
        for (int k = 1; k < kWarps; k++) t = merge(t, part[k]);  // warp order: the same bits every run
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
    const Stat s = row_stat(row, v, span_of(row, v));
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
    const Stat s = row_stat(row, v, sp);
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
            o[i] = y;
        }
        if ((int)threadIdx.x < sp.head) out[threadIdx.x] = __expf(row[threadIdx.x] - m) * scale - (threadIdx.x == target ? g : 0.0f);
        const int64_t j = sp.tail0 + threadIdx.x;
        if (j < v) out[j] = __expf(row[j] - m) * scale - (j == target ? g : 0.0f);
    } else {  // the gradient's row sits at another alignment than the logits': scalar stores
        for (int64_t j = threadIdx.x; j < v; j += kThreads) out[j] = __expf(row[j] - m) * scale - (j == target ? g : 0.0f);
    }
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
    k_xent_bwd_rows<<<(unsigned)n, kThreads>>>(logits, t, dl, v, dloss / (float)n);
    report(cudaPeekAtLastError(), slb::ERR_LAUNCH);
}
