// sm_100a kernels for the compute side of a Soliton training step, first of them: layer normalisation.
//
// Same backend-level names and signatures as the reference's CUDA file (core/cuda/kernels.cu:409-449), so that a
// Soliton build can link them in place; the scratch arguments its host core passes are accepted as they are.
//
// The reference normalises forward with one block per row and scalar loads, and runs the backward pass as eight
// elementwise launches and four cuBLAS matrix-vector products over scratch copies of the activation (thirteen
// passes over an outer x c matrix). Both directions are bandwidth-bound and have no contraction worth a tensor core,
// so here each is ONE pass: a warp owns a row, holds it in registers (256-bit loads, c / 256 of them per lane and
// tensor), reduces with shuffles, and writes the result once. The column sums of the backward pass (dw, db) are
// accumulated per lane over the rows a warp walks, combined per block in shared memory in warp order, written as one
// partial per block into the caller's scratch matrix, and added up over the blocks in a fixed order by a second, tiny
// launch: no atomics, the same bits on every run.
//
// Algorithmic traffic: forward 8 B per element (read x, write y), backward 12 B per element (read dy and x, write dx).
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/soliton_b200.h"
#include "dp_engine.hpp"

namespace slb_step {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxVecC = 1024;  // widest row the register path takes (four 256-bit loads per lane and tensor)

struct alignas(32) f8 {
    float v[8];
};
__device__ __forceinline__ f8 ld8(const float* p) {
    f8 r;
    asm volatile("ld.global.cs.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7])
                 : "l"(p)
                 : "memory");
    return r;
}
__device__ __forceinline__ f8 ld8_keep(const float* p) {  // parameters: read by every row, worth a cache line
    f8 r;
    asm volatile("ld.global.nc.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(r.v[0]), "=f"(r.v[1]), "=f"(r.v[2]), "=f"(r.v[3]), "=f"(r.v[4]), "=f"(r.v[5]), "=f"(r.v[6]), "=f"(r.v[7])
                 : "l"(p));
    return r;
}
__device__ __forceinline__ void st8(float* p, const f8& r) {
    asm volatile("st.global.cs.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(r.v[0]), "f"(r.v[1]), "f"(r.v[2]),
                 "f"(r.v[3]), "f"(r.v[4]), "f"(r.v[5]), "f"(r.v[6]), "f"(r.v[7])
                 : "memory");
}
// Sum over the warp, the same value (and the same bits) in every lane: a butterfly has one fixed shape.
__device__ __forceinline__ float warp_all_sum(float v) {
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// The reference's arithmetic per element (core/cuda/kernels.cu:395-407, as nvcc contracts it): mean = sum / c,
// invstd = rsqrtf(max(sum of squares / c - mean^2, 0) + eps), y = fma((x - mean) * invstd, w, b).
__device__ __forceinline__ void row_stats(float s, float sq, int64_t c, float eps, float& mean, float& invstd) {
    mean = s / (float)c;
    invstd = rsqrtf(fmaxf(sq / (float)c - mean * mean, 0.0f) + eps);
}

// ---------------------------------------------------------------- forward

// K = c / 256: 256-bit loads per lane and tensor. A warp walks rows warp, warp + total warps, ...
template <int K>
__global__ void __launch_bounds__(kThreads) k_ln_fwd_vec(const float* __restrict__ x, const float* __restrict__ w,
                                                         const float* __restrict__ b, float* __restrict__ y,
                                                         float* __restrict__ mean, float* __restrict__ invstd, int64_t outer,
                                                         float eps) {
    constexpr int64_t c = 256 * K;
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5), warps = (int64_t)gridDim.x * kWarps;
    f8 wv[K], bv[K];
#pragma unroll
    for (int k = 0; k < K; k++) wv[k] = ld8_keep(w + k * 256 + lane * 8), bv[k] = ld8_keep(b + k * 256 + lane * 8);
    for (int64_t r = warp; r < outer; r += warps) {
        f8 xv[K];
#pragma unroll
        for (int k = 0; k < K; k++) xv[k] = ld8(x + r * c + k * 256 + lane * 8);
        float s = 0, sq = 0;
#pragma unroll
        for (int k = 0; k < K; k++)
#pragma unroll
            for (int e = 0; e < 8; e++) s += xv[k].v[e], sq = __fmaf_rn(xv[k].v[e], xv[k].v[e], sq);
        s = warp_all_sum(s), sq = warp_all_sum(sq);
        float m, is;
        row_stats(s, sq, c, eps, m, is);
        if (lane == 0) mean[r] = m, invstd[r] = is;
#pragma unroll
        for (int k = 0; k < K; k++) {
            f8 o;
#pragma unroll
            for (int e = 0; e < 8; e++) o.v[e] = __fmaf_rn(__fmul_rn(__fsub_rn(xv[k].v[e], m), is), wv[k].v[e], bv[k].v[e]);
            st8(y + r * c + k * 256 + lane * 8, o);
        }
    }
}

// Any c, any alignment: a warp per row, two passes over the row (the second one finds it in cache).
__global__ void __launch_bounds__(kThreads) k_ln_fwd_any(const float* __restrict__ x, const float* __restrict__ w,
                                                         const float* __restrict__ b, float* __restrict__ y,
                                                         float* __restrict__ mean, float* __restrict__ invstd, int64_t outer,
                                                         int64_t c, float eps) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5), warps = (int64_t)gridDim.x * kWarps;
    for (int64_t r = warp; r < outer; r += warps) {
        const float* X = x + r * c;
        float s = 0, sq = 0;
        for (int64_t j = lane; j < c; j += 32) s += X[j], sq = __fmaf_rn(X[j], X[j], sq);
        s = warp_all_sum(s), sq = warp_all_sum(sq);
        float m, is;
        row_stats(s, sq, c, eps, m, is);
        if (lane == 0) mean[r] = m, invstd[r] = is;
        for (int64_t j = lane; j < c; j += 32) y[r * c + j] = __fmaf_rn(__fmul_rn(__fsub_rn(X[j], m), is), w[j], b[j]);
    }
}

// ---------------------------------------------------------------- backward

// g = dy * w; xhat = (x - mean) * invstd; dx = invstd * (g - mean_row(g) - xhat * mean_row(g * xhat))
// (core/cuda/kernels.cu:436-449); dw = sum over rows of dy * xhat, db = sum over rows of dy.
// partial: gridDim.x x 2 x c floats (the caller's scratch matrix), block b's column sums of dw then db.
template <int K>
__global__ void __launch_bounds__(kThreads, K <= 3 ? 2 : 1) k_ln_bwd_vec(const float* __restrict__ dy, const float* __restrict__ x,
                                                         const float* __restrict__ w, const float* __restrict__ mean,
                                                         const float* __restrict__ invstd, float* __restrict__ dx,
                                                         float* __restrict__ partial, int64_t outer) {
    constexpr int64_t c = 256 * K;
    __shared__ float s_cols[kWarps][c];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t warp = (int64_t)blockIdx.x * kWarps + wid, warps = (int64_t)gridDim.x * kWarps;
    f8 dw[K], db[K];  // the row's w is fetched again for every row (it stays in L1): registers are for the accumulators
#pragma unroll
    for (int k = 0; k < K; k++)
#pragma unroll
        for (int e = 0; e < 8; e++) dw[k].v[e] = 0, db[k].v[e] = 0;
    const float inv_c = 1.0f / (float)c;
    for (int64_t r = warp; r < outer; r += warps) {
        f8 gv[K], xh[K];
#pragma unroll
        for (int k = 0; k < K; k++) gv[k] = ld8(dy + r * c + k * 256 + lane * 8), xh[k] = ld8(x + r * c + k * 256 + lane * 8);
        const float m = mean[r], is = invstd[r];
        float sg = 0, sgx = 0;
#pragma unroll
        for (int k = 0; k < K; k++) {
            const f8 wk = ld8_keep(w + k * 256 + lane * 8);
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const float d = gv[k].v[e];
                const float h = __fmul_rn(__fsub_rn(xh[k].v[e], m), is);
                db[k].v[e] += d;
                dw[k].v[e] = __fmaf_rn(d, h, dw[k].v[e]);
                const float g = __fmul_rn(d, wk.v[e]);
                sg += g, sgx = __fmaf_rn(g, h, sgx);
                gv[k].v[e] = g, xh[k].v[e] = h;
            }
        }
        sg = warp_all_sum(sg) * inv_c, sgx = warp_all_sum(sgx) * inv_c;
#pragma unroll
        for (int k = 0; k < K; k++) {
            f8 o;
#pragma unroll
            for (int e = 0; e < 8; e++) o.v[e] = __fmul_rn(is, __fsub_rn(__fsub_rn(gv[k].v[e], sg), __fmul_rn(xh[k].v[e], sgx)));
            st8(dx + r * c + k * 256 + lane * 8, o);
        }
    }
    // the block's column sums: warps in warp order, first dw, then db
    for (int pass = 0; pass < 2; pass++) {
        __syncthreads();
#pragma unroll
        for (int k = 0; k < K; k++)
#pragma unroll
            for (int e = 0; e < 8; e++) s_cols[wid][k * 256 + lane * 8 + e] = pass == 0 ? dw[k].v[e] : db[k].v[e];
        __syncthreads();
        for (int j = threadIdx.x; j < c; j += kThreads) {
            float t = 0;
#pragma unroll
            for (int q = 0; q < kWarps; q++) t += s_cols[q][j];
            partial[((int64_t)blockIdx.x * 2 + pass) * c + j] = t;
        }
    }
}

// dw[j], db[j] = the partials of the blocks. A block owns 32 columns (of dw and db laid side by side); each of its
// eight warps adds up every eighth block's partial, and the eight sums meet in shared memory in warp order: a fixed
// order, so the same bits every run, with eight times the loads in flight of one thread per column.
__global__ void __launch_bounds__(kThreads) k_ln_bwd_finish(const float* __restrict__ partial, int blocks, int64_t c,
                                                            float* __restrict__ dw, float* __restrict__ db) {
    __shared__ float part[kWarps][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t j = (int64_t)blockIdx.x * 32 + lane;  // c is a multiple of 256 here: a block never straddles dw and db
    const int pass = j >= c;
    const int64_t col = j - pass * c;
    float t = 0;
    if (j < 2 * c)
        for (int b = warp; b < blocks; b += kWarps) t += partial[((int64_t)b * 2 + pass) * c + col];
    part[warp][lane] = t;
    __syncthreads();
    if (warp == 0 && j < 2 * c) {
        float sum = part[0][lane];
#pragma unroll
        for (int k = 1; k < kWarps; k++) sum += part[k][lane];
        (pass ? db : dw)[col] = sum;
    }
}

// Any c: a warp per row for dx, then a thread per column for dw and db, rows in order.
__global__ void __launch_bounds__(kThreads) k_ln_dx_any(const float* __restrict__ dy, const float* __restrict__ x,
                                                        const float* __restrict__ w, const float* __restrict__ mean,
                                                        const float* __restrict__ invstd, float* __restrict__ dx,
                                                        int64_t outer, int64_t c) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (int64_t)blockIdx.x * kWarps + (threadIdx.x >> 5), warps = (int64_t)gridDim.x * kWarps;
    const float inv_c = 1.0f / (float)c;
    for (int64_t r = warp; r < outer; r += warps) {
        const float m = mean[r], is = invstd[r];
        float sg = 0, sgx = 0;
        for (int64_t j = lane; j < c; j += 32) {
            const float g = __fmul_rn(dy[r * c + j], w[j]), h = __fmul_rn(__fsub_rn(x[r * c + j], m), is);
            sg += g, sgx = __fmaf_rn(g, h, sgx);
        }
        sg = warp_all_sum(sg) * inv_c, sgx = warp_all_sum(sgx) * inv_c;
        for (int64_t j = lane; j < c; j += 32) {
            const float g = __fmul_rn(dy[r * c + j], w[j]), h = __fmul_rn(__fsub_rn(x[r * c + j], m), is);
            dx[r * c + j] = __fmul_rn(is, __fsub_rn(__fsub_rn(g, sg), __fmul_rn(h, sgx)));
        }
    }
}
__global__ void __launch_bounds__(kThreads) k_ln_cols_any(const float* __restrict__ dy, const float* __restrict__ x,
                                                          const float* __restrict__ mean, const float* __restrict__ invstd,
                                                          float* __restrict__ dw, float* __restrict__ db, int64_t outer,
                                                          int64_t c) {
    const int64_t j = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (j >= c) return;
    float a = 0, s = 0;
    for (int64_t r = 0; r < outer; r++) {
        const float d = dy[r * c + j];
        a = __fmaf_rn(d, __fmul_rn(__fsub_rn(x[r * c + j], mean[r]), invstd[r]), a);
        s += d;
    }
    dw[j] = a, db[j] = s;
}

static bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31) == 0; }
static int sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) n = 148;
    }
    return n;
}
// Blocks for `outer` rows at a warp per row: enough warps for every row, at most four blocks per SM.
static int row_grid(int64_t outer) {
    const int64_t need = (outer + kWarps - 1) / kWarps, cap = 4 * (int64_t)sm_count();
    return (int)(need < 1 ? 1 : need < cap ? need : cap);
}

}  // namespace slb_step

using namespace slb_step;

// Launch failures surface through the library's sticky error (sl_check), as every void entry point's do.
static void report(cudaError_t e) {
    if (e != cudaSuccess) slb::Engine::get().set_error(slb::ERR_LAUNCH);
}

extern "C" void sl_cuda_layernorm(const float* x, const float* w, const float* b, float* y, float* mean, float* invstd,
                                 int64_t outer, int64_t c, float eps, float* ones) {
    (void)ones;  // scratch of the reference's host core; not needed
    if (outer <= 0 || c <= 0) return;
    const bool vec = c % 256 == 0 && c <= kMaxVecC && aligned32(x) && aligned32(w) && aligned32(b) && aligned32(y);
    const int grid = row_grid(outer);
    if (vec) {
        switch (c / 256) {
            case 1: k_ln_fwd_vec<1><<<grid, kThreads>>>(x, w, b, y, mean, invstd, outer, eps); break;
            case 2: k_ln_fwd_vec<2><<<grid, kThreads>>>(x, w, b, y, mean, invstd, outer, eps); break;
            case 3: k_ln_fwd_vec<3><<<grid, kThreads>>>(x, w, b, y, mean, invstd, outer, eps); break;
            default: k_ln_fwd_vec<4><<<grid, kThreads>>>(x, w, b, y, mean, invstd, outer, eps); break;
        }
    } else {
        k_ln_fwd_any<<<grid, kThreads>>>(x, w, b, y, mean, invstd, outer, c, eps);
    }
    report(cudaPeekAtLastError());
}

extern "C" void sl_cuda_layernorm_bwd(const float* dy, const float* x, const float* w, const float* mean,
                                     const float* invstd, float* dx, float* dw, float* db, int64_t outer, int64_t c,
                                     float* tmp, float* sg, float* sgx, float* ones_c, float* ones_rows) {
    (void)sg, (void)sgx, (void)ones_c, (void)ones_rows;  // scratch of the reference's host core; only tmp is used
    if (outer <= 0 || c <= 0) return;
    int grid = row_grid(outer);
    if (grid > 2 * sm_count()) grid = 2 * sm_count();  // the register path holds three tensors per row: two blocks per SM
    // the per-block column sums need 2 x c floats per block inside tmp (outer x c floats)
    const bool vec = c % 256 == 0 && c <= kMaxVecC && tmp != nullptr && 2 * (int64_t)grid <= outer && aligned32(dy) &&
                     aligned32(x) && aligned32(w) && aligned32(dx);
    if (vec) {
        switch (c / 256) {
            case 1: k_ln_bwd_vec<1><<<grid, kThreads>>>(dy, x, w, mean, invstd, dx, tmp, outer); break;
            case 2: k_ln_bwd_vec<2><<<grid, kThreads>>>(dy, x, w, mean, invstd, dx, tmp, outer); break;
            case 3: k_ln_bwd_vec<3><<<grid, kThreads>>>(dy, x, w, mean, invstd, dx, tmp, outer); break;
            default: k_ln_bwd_vec<4><<<grid, kThreads>>>(dy, x, w, mean, invstd, dx, tmp, outer); break;
        }
        k_ln_bwd_finish<<<(unsigned)((2 * c + 31) / 32), kThreads>>>(tmp, grid, c, dw, db);
    } else {
        k_ln_dx_any<<<row_grid(outer), kThreads>>>(dy, x, w, mean, invstd, dx, outer, c);
        k_ln_cols_any<<<(unsigned)((c + kThreads - 1) / kThreads), kThreads>>>(dy, x, mean, invstd, dw, db, outer, c);
    }
    report(cudaPeekAtLastError());
}
