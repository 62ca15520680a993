// More bandwidth-bound pieces of a Soliton training step: broadcasting binary ops, GELU, the embedding's backward.
//
// Same backend-level names and signatures as the reference's CUDA file (core/cuda/kernels.cu:139-181, 226-240,
// 459-487), and the same bits: each output element is the same fp32 expression of the same inputs (binary, GELU),
// or the same rows added in the same order (embedding).
//
// Binary ops. A GPT-2 step runs 49 of them, nearly all "suffix" cases: residual adds (both inputs shaped like the
// output) and bias adds (one input is the output's trailing dimension). The reference gives each element a thread
// and two 64-bit remainders; here a thread takes 128 bits of the output and one 32-bit remainder per input that
// actually repeats. Other stride patterns decompose the index per element, as they must.
//
// Embedding backward. The reference sorts the token ids, then lets ONE THREAD per run of equal ids add up that run's
// rows of dy, 768 floats one after the other, each thread striding through memory on its own. Here a block takes a
// run and its threads the columns, so rows are read and written in full lines; runs are still added in sorted order
// (the sort is stable, so in token order), which keeps the sums bit-identical to the reference's.
#include <cuda_runtime.h>

#include <cstdint>
#include <cub/cub.cuh>

#include "../../include/soliton_b200.h"
#include "dp_engine.hpp"

namespace slb_elt {

constexpr int kThreads = 256;
constexpr int kMaxDims = 8;  // as the reference's Strided (core/cuda/kernels.cu:71-74)

__device__ __forceinline__ float apply(int op, float x, float y) {
    return op == 0 ? x + y : op == 1 ? x - y : op == 2 ? __fmul_rn(x, y) : x / y;
}
__device__ __forceinline__ float4 apply4(int op, float4 x, float4 y) {
    return make_float4(apply(op, x.x, y.x), apply(op, x.y, y.y), apply(op, x.z, y.z), apply(op, x.w, y.w));
}

// o[i] = a[i mod na] op b[i mod nb] in 128-bit words; n4, na4, nb4 count words and fit 32 bits.
__global__ void __launch_bounds__(kThreads) k_binary_suffix4(unsigned n4, int op, const float4* __restrict__ a,
                                                             const float4* __restrict__ b, float4* __restrict__ o,
                                                             unsigned na4, unsigned nb4) {
    const unsigned i = blockIdx.x * kThreads + threadIdx.x;
    if (i >= n4) return;
    const float4 x = a[na4 == n4 ? i : i % na4], y = b[nb4 == n4 ? i : i % nb4];
    o[i] = apply4(op, x, y);
}
// The same element by element: odd sizes or alignments.
__global__ void __launch_bounds__(kThreads) k_binary_suffix1(int64_t n, int op, const float* __restrict__ a,
                                                             const float* __restrict__ b, float* __restrict__ o, int64_t na,
                                                             int64_t nb) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i < n) o[i] = apply(op, a[i % na], b[i % nb]);
}

struct Dims {
    int nd;
    int64_t shape[kMaxDims], sa[kMaxDims], sb[kMaxDims];
};
// Any strides (0 where an input broadcasts): the output index is taken apart dimension by dimension.
__global__ void __launch_bounds__(kThreads) k_binary_strided(int64_t n, int op, const float* __restrict__ a,
                                                             const float* __restrict__ b, float* __restrict__ o, Dims d) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n) return;
    int64_t rest = i, ia = 0, ib = 0;
    for (int k = d.nd - 1; k >= 0; k--) {
        const int64_t q = rest / d.shape[k], r = rest - q * d.shape[k];
        ia += r * d.sa[k], ib += r * d.sb[k];
        rest = q;
    }
    o[i] = apply(op, a[ia], b[ib]);
}

// Elements of an input that is the output's trailing dimensions laid out densely and repeated over the leading
// ones (the whole output, a bias, a scalar); -1 for anything else.
static int64_t repeating_suffix(int nd, const int64_t* shape, const int64_t* stride) {
    int64_t dense = 1;
    int d = nd - 1;
    for (; d >= 0 && stride[d] == dense; d--) dense *= shape[d];
    for (; d >= 0; d--)
        if (stride[d] != 0 && shape[d] != 1) return -1;
    return dense;
}

// ---------------------------------------------------------------- GELU

// The exact GELU, x * Phi(x) with Phi through erf, and its derivative Phi(x) + x * phi(x)
// (core/cuda/kernels.cu:226-240), four elements per thread.
__device__ __forceinline__ float gelu(float x) { return 0.5f * x * (1.0f + erff(x * 0.70710678f)); }
__device__ __forceinline__ float gelu_grad(float x, float dy) {
    const float cdf = 0.5f * (1.0f + erff(x * 0.70710678f));
    const float pdf = expf(-0.5f * x * x) * 0.39894228f;
    return dy * (cdf + x * pdf);
}
__global__ void __launch_bounds__(kThreads) k_gelu4(int64_t n4, const float4* __restrict__ x, float4* __restrict__ y) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n4) return;
    const float4 v = x[i];
    y[i] = make_float4(gelu(v.x), gelu(v.y), gelu(v.z), gelu(v.w));
}
__global__ void __launch_bounds__(kThreads) k_gelu1(int64_t n, const float* __restrict__ x, float* __restrict__ y) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i < n) y[i] = gelu(x[i]);
}
__global__ void __launch_bounds__(kThreads) k_gelu_bwd4(int64_t n4, const float4* __restrict__ x, const float4* __restrict__ dy,
                                                        float4* __restrict__ dx) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i >= n4) return;
    const float4 v = x[i], g = dy[i];
    dx[i] = make_float4(gelu_grad(v.x, g.x), gelu_grad(v.y, g.y), gelu_grad(v.z, g.z), gelu_grad(v.w, g.w));
}
__global__ void __launch_bounds__(kThreads) k_gelu_bwd1(int64_t n, const float* __restrict__ x, const float* __restrict__ dy,
                                                        float* __restrict__ dx) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i < n) dx[i] = gelu_grad(x[i], dy[i]);
}

// ---------------------------------------------------------------- embedding backward

__global__ void __launch_bounds__(kThreads) k_fill4(float4* __restrict__ p, int64_t n4, float4 v) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i < n4) p[i] = v;
}
__global__ void __launch_bounds__(kThreads) k_fill1(float* __restrict__ p, int64_t n, float v) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i < n) p[i] = v;
}
__global__ void __launch_bounds__(kThreads) k_iota(int* __restrict__ p, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (i < n) p[i] = (int)i;
}
// Block i of n: if sorted position i starts a run of equal ids, add the run's rows of dy into that id's row of dw,
// threads over the columns, rows in sorted order. dw was zero-filled, and x + 0 = x: sums start from the first row.
__global__ void __launch_bounds__(kThreads) k_embedding_bwd_runs(int64_t n, const float* __restrict__ dy,
                                                                 const int* __restrict__ keys, const int* __restrict__ perm,
                                                                 float* __restrict__ dw, int64_t c) {
    const int64_t i = blockIdx.x;
    const int id = keys[i];
    if (i > 0 && keys[i - 1] == id) return;
    int64_t end = i + 1;
    while (end < n && keys[end] == id) end++;
    float* row = dw + (int64_t)id * c;
    for (int64_t q = threadIdx.x; q < c; q += kThreads) {
        float sum = 0.0f;
        for (int64_t j = i; j < end; j++) sum += dy[(int64_t)perm[j] * c + q];
        row[q] = sum;
    }
}

static void report(cudaError_t e, int code) {
    if (e != cudaSuccess) slb::Engine::get().set_error(code);
}
static unsigned blocks_for(int64_t n) { return (unsigned)((n + kThreads - 1) / kThreads); }
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace slb_elt

using namespace slb_elt;

// Which kernel sl_cuda_binary picks for these shapes and strides, without launching anything: 2 = 128-bit suffix
// kernel, 1 = element-wise suffix kernel, 0 = general strides, -1 = refused; out[0], out[1] = the repeat lengths of a
// and b (-1 where an input is no repeating suffix). Pointers are taken as 16-byte aligned.
extern "C" int slb_binary_plan(int nd, const int64_t* shape, const int64_t* sa, const int64_t* sb, int64_t* out) {
    if (nd < 0 || nd > kMaxDims) return -1;
    int64_t n = 1;
    for (int d = 0; d < nd; d++) n *= shape[d];
    const int64_t na = repeating_suffix(nd, shape, sa), nb = repeating_suffix(nd, shape, sb);
    if (out) out[0] = na, out[1] = nb;
    if (!(na > 0 && nb > 0)) return 0;
    return n % 4 == 0 && na % 4 == 0 && nb % 4 == 0 && n / 4 < ((int64_t)1 << 32) - kThreads ? 2 : 1;
}

extern "C" void sl_cuda_binary(int op, const float* a, const float* b, float* o, int nd, const int64_t* shape,
                               const int64_t* sa, const int64_t* sb) {
    if (nd < 0 || nd > kMaxDims || op < 0 || op > 3) return report(cudaErrorInvalidValue, slb::ERR_BAD_ARG);
    int64_t n = 1;
    for (int d = 0; d < nd; d++) n *= shape[d];
    if (n <= 0) return;
    int64_t rep[2];
    const int plan = slb_binary_plan(nd, shape, sa, sb, rep);
    const int64_t na = rep[0], nb = rep[1];
    if (plan > 0) {
        if (plan == 2 && aligned16(a) && aligned16(b) && aligned16(o))
            k_binary_suffix4<<<blocks_for(n / 4), kThreads>>>((unsigned)(n / 4), op, reinterpret_cast<const float4*>(a),
                                                             reinterpret_cast<const float4*>(b), reinterpret_cast<float4*>(o),
                                                             (unsigned)(na / 4), (unsigned)(nb / 4));
        else
            k_binary_suffix1<<<blocks_for(n), kThreads>>>(n, op, a, b, o, na, nb);
    } else {
        Dims d{};
        d.nd = nd;
        for (int k = 0; k < nd; k++) d.shape[k] = shape[k], d.sa[k] = sa[k], d.sb[k] = sb[k];
        k_binary_strided<<<blocks_for(n), kThreads>>>(n, op, a, b, o, d);
    }
    report(cudaPeekAtLastError(), slb::ERR_LAUNCH);
}

extern "C" void sl_cuda_gelu(const float* x, float* y, int64_t n) {
    if (n <= 0) return;
    if (n % 4 == 0 && aligned16(x) && aligned16(y))
        k_gelu4<<<blocks_for(n / 4), kThreads>>>(n / 4, reinterpret_cast<const float4*>(x), reinterpret_cast<float4*>(y));
    else
        k_gelu1<<<blocks_for(n), kThreads>>>(n, x, y);
    report(cudaPeekAtLastError(), slb::ERR_LAUNCH);
}

extern "C" void sl_cuda_gelu_bwd(const float* x, const float* dy, float* dx, int64_t n) {
    if (n <= 0) return;
    if (n % 4 == 0 && aligned16(x) && aligned16(dy) && aligned16(dx))
        k_gelu_bwd4<<<blocks_for(n / 4), kThreads>>>(n / 4, reinterpret_cast<const float4*>(x), reinterpret_cast<const float4*>(dy),
                                                    reinterpret_cast<float4*>(dx));
    else
        k_gelu_bwd1<<<blocks_for(n), kThreads>>>(n, x, dy, dx);
    report(cudaPeekAtLastError(), slb::ERR_LAUNCH);
}

extern "C" size_t sl_cuda_sort_temp_bytes(int64_t n) {
    size_t bytes = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, bytes, (const int*)nullptr, (int*)nullptr, (const int*)nullptr, (int*)nullptr, (int)n);
    return bytes;
}

extern "C" void sl_cuda_embedding_bwd(const float* dy, const int* idx, float* dw, int64_t vocab, int64_t n, int64_t c, int* keys,
                                      int* perm, int* perm_out, void* temp, size_t temp_bytes) {
    if (vocab <= 0 || c <= 0) return;
    const int64_t total = vocab * c;
    if (total % 4 == 0 && aligned16(dw)) k_fill4<<<blocks_for(total / 4), kThreads>>>(reinterpret_cast<float4*>(dw), total / 4, make_float4(0, 0, 0, 0));
    else k_fill1<<<blocks_for(total), kThreads>>>(dw, total, 0.0f);
    report(cudaPeekAtLastError(), slb::ERR_LAUNCH);
    if (n <= 0) return;
    size_t need = temp_bytes;
    if (sl_cuda_sort_temp_bytes(n) > temp_bytes) return slb::Engine::get().set_error(8);  // the reference's code for this
    k_iota<<<blocks_for(n), kThreads>>>(perm, n);
    if (cub::DeviceRadixSort::SortPairs(temp, need, idx, keys, perm, perm_out, (int)n) != cudaSuccess) return slb::Engine::get().set_error(6);
    k_embedding_bwd_runs<<<(unsigned)n, kThreads>>>(n, dy, keys, perm_out, dw, c);
    report(cudaPeekAtLastError(), slb::ERR_LAUNCH);
}
