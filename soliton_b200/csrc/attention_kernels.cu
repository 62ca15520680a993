// Fused causal attention, forward and backward, head size 64, in both precisions of the reference's matmuls.
//
// Same backend-level names and scratch arguments as the reference's CUDA file (core/cuda/kernels.cu:536-692). The
// reference tiles at 256 and keeps every score tile in HBM between cuBLAS batched GEMMs and a dozen elementwise
// launches per tile pair; with TF32 enabled that is about 37 % of a GPT-2 124M training step. Here a block owns 64
// query rows (forward, dQ) or 64 key rows (dK, dV), walks the other side in tiles of 64, and keeps scores,
// probabilities and accumulators in registers; only Q, K, V, dO come from memory, only O, L and the gradients go back.
// Products run on the tensor cores (warp-level mma, m16n8k8, TF32 operands, fp32 accumulation) in one of two ways,
// chosen like the reference's matmul mode (sl_cuda_attention_set_tf32, next to sl_cuda_set_tf32):
//   TF32 (template X3 = false): operands rounded to TF32 once, as cuBLAS does in the reference's TF32 mode;
//   fp32 class (X3 = true, the default): operands stay fp32 in shared memory and are split as they are read into
//     a TF32 head and a TF32 remainder, x = hi + lo to about 2^-22; a product is lo*hi + hi*lo + hi*hi, smallest
//     terms first. Three tensor-core products instead of one, an error of about 2^-21 per operand pair.
// Backward is two kernels -- one accumulates dQ over the key tiles, one dK and dV over the query tiles -- so that no
// atomic is needed and every gradient has one fixed summation order: the same bits every run.
//
// What bounds the TF32 kernels is shared-memory bandwidth, not the tensor pipe (40-43 % busy): a warp-level product
// takes two 32-bit shared loads per lane for its B operand. This is the legacy tensor path; tcgen05 with operands
// delivered by TMA and accumulators in tensor memory is the way past that ceiling and is not what this file does.
//
// Layouts (core/cuda/kernels.cu:538-540, 614-692): qkv and dqkv packed (B, T, 3, H, 64); out and dout (B, T, H, 64);
// L (B, H, T) = row maximum + log of the softmax denominator of the scaled, masked scores.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>

#include "../../include/soliton_b200.h"
#include "dp_engine.hpp"

namespace slb_attn {

constexpr int HS = 64;       // head size
constexpr int BT = 64;       // rows per tile, both sides
constexpr int kThreads = 128;
constexpr int S_NK = 68;     // row stride of a tile read as B[k][n] = tile[n][k]: lanes (n = g, k = t) hit 32 banks
constexpr int S_KN = 72;     // row stride of a tile read as B[k][n] = tile[k][n]: lanes (k = t, n = g) hit 32 banks
constexpr int S_P = 68;      // per-warp staging of a 16 x 64 probability block, read back as an A operand

// Round to TF32 (10 mantissa bits), nearest with ties away from zero like cvt.rna.tf32.f32, in two integer
// operations: half a TF32 unit is added to the magnitude and the 13 low bits are cleared.
__device__ __forceinline__ uint32_t tf32(float x) { return (__float_as_uint(x) + 0x1000u) & 0xffffe000u; }
// D(16x8) += A(16x8, row) * B(8x8, col). Lane l: g = l / 4, t = l % 4. A: a0 (g, t) a1 (g+8, t) a2 (g, t+4) a3 (g+8, t+4);
// B: b0 (k = t, n = g) b1 (k = t+4, n = g); D: d0 (g, 2t) d1 (g, 2t+1) d2 (g+8, 2t) d3 (g+8, 2t+1).
__device__ __forceinline__ void mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float ex2(float x) {  // 2^x, flushing; ex2(-inf) = 0
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
constexpr float kLog2e = 1.4426950408889634f;
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

// One operand in the two pieces of the split-precision products: x = hi + lo to about 2^-22, both TF32.
__device__ __forceinline__ void split(float x, uint32_t& hi, uint32_t& lo) {
    hi = tf32(x);
    lo = tf32(x - __uint_as_float(hi));
}

// A 64 x 64 tile of one head (rows row0 .., row stride ld floats) into shared memory with row stride `stride`:
// rounded to TF32, or as it is when the products are split (X3). All eight 128-bit loads of a thread are issued
// before the first store, so that they are in flight together.
template <bool X3>
__device__ __forceinline__ void load_tile(float* dst, int stride, const float* __restrict__ src, int64_t ld, int row0) {
    constexpr int kPer = BT * (HS / 4) / kThreads;  // 8
    float4 v[kPer];
#pragma unroll
    for (int u = 0; u < kPer; u++) {
        const int i = threadIdx.x + u * kThreads;
        v[u] = __ldg(reinterpret_cast<const float4*>(src + (int64_t)(row0 + (i >> 4)) * ld + (i & 15) * 4));
    }
#pragma unroll
    for (int u = 0; u < kPer; u++) {
        const int i = threadIdx.x + u * kThreads;
        float* d = dst + (i >> 4) * stride + (i & 15) * 4;
        if constexpr (X3) *reinterpret_cast<float4*>(d) = v[u];
        else *reinterpret_cast<uint4*>(d) = make_uint4(tf32(v[u].x), tf32(v[u].y), tf32(v[u].z), tf32(v[u].w));
    }
}
// The same tile into two places with two strides: a tile that is read both as B[k][n] = tile[n][k] and as
// B[k][n] = tile[k][n] has no single stride that keeps both reads free of bank conflicts.
template <bool X3>
__device__ __forceinline__ void load_tile2(float* dst, int stride, float* dst2, int stride2, const float* __restrict__ src,
                                           int64_t ld, int row0) {
    constexpr int kPer = BT * (HS / 4) / kThreads;  // 8
    float4 v[kPer];
#pragma unroll
    for (int u = 0; u < kPer; u++) {
        const int i = threadIdx.x + u * kThreads;
        v[u] = __ldg(reinterpret_cast<const float4*>(src + (int64_t)(row0 + (i >> 4)) * ld + (i & 15) * 4));
    }
#pragma unroll
    for (int u = 0; u < kPer; u++) {
        const int i = threadIdx.x + u * kThreads;
        float4 w = v[u];
        if constexpr (!X3) w = make_float4(__uint_as_float(tf32(w.x)), __uint_as_float(tf32(w.y)), __uint_as_float(tf32(w.z)), __uint_as_float(tf32(w.w)));
        *reinterpret_cast<float4*>(dst + (i >> 4) * stride + (i & 15) * 4) = w;
        *reinterpret_cast<float4*>(dst2 + (i >> 4) * stride2 + (i & 15) * 4) = w;
    }
}
// The A operand of 16 rows (row0 + g, row0 + g + 8) x 64 columns straight from memory: 8 k-steps of 8 columns.
__device__ __forceinline__ void load_a(uint32_t (&a)[8][4], const float* src, int64_t ld, int row0, int g, int t) {
    const float* r0 = src + (int64_t)(row0 + g) * ld;
    const float* r1 = src + (int64_t)(row0 + g + 8) * ld;
#pragma unroll
    for (int ks = 0; ks < 8; ks++) {
        a[ks][0] = tf32(r0[ks * 8 + t]), a[ks][1] = tf32(r1[ks * 8 + t]);
        a[ks][2] = tf32(r0[ks * 8 + t + 4]), a[ks][3] = tf32(r1[ks * 8 + t + 4]);
    }
}
// The B operand of k-step ks and column block nt out of a 64 x 64 tile in shared memory with row stride sb:
// TRANS ? B[k][n] = tile[n][k] : B[k][n] = tile[k][n].
template <bool TRANS>
__device__ __forceinline__ void b_index(int ks, int nt, int sb, int g, int t, int& i0, int& i1) {
    if constexpr (TRANS) i0 = (nt * 8 + g) * sb + ks * 8 + t, i1 = i0 + 4;
    else i0 = (ks * 8 + t) * sb + nt * 8 + g, i1 = i0 + 4 * sb;
}
// acc(16 x 64) += A * B, A (16 x 64) in registers as TF32, B from a tile of TF32 values.
template <bool TRANS>
__device__ __forceinline__ void gemm_ra(float (&acc)[8][4], const uint32_t (&a)[8][4], const float* tile, int sb, int g, int t) {
    const uint32_t* u = reinterpret_cast<const uint32_t*>(tile);
#pragma unroll
    for (int ks = 0; ks < 8; ks++)
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            int i0, i1;
            b_index<TRANS>(ks, nt, sb, g, t, i0, i1);
            mma(acc[nt], a[ks], u[i0], u[i1]);
        }
}
// acc(16 x 64) += A * B, A (rows g and g + 8 of `a`, row stride sa) and B both from shared memory. Without X3 both
// hold TF32 values: one product. With X3 both hold fp32 values, split as they are read: lo x hi + hi x lo + hi x hi,
// smallest terms first -- an fp32-class product out of three TF32 ones.
template <bool X3, bool TRANS>
__device__ __forceinline__ void gemm_sa(float (&acc)[8][4], const float* a, int sa, const float* tile, int sb, int g, int t) {
#pragma unroll
    for (int ks = 0; ks < 8; ks++) {
        const float a0 = a[g * sa + ks * 8 + t], a1 = a[(g + 8) * sa + ks * 8 + t];
        const float a2 = a[g * sa + ks * 8 + t + 4], a3 = a[(g + 8) * sa + ks * 8 + t + 4];
        uint32_t ah[4], al[4];
        if constexpr (X3) {
            split(a0, ah[0], al[0]), split(a1, ah[1], al[1]), split(a2, ah[2], al[2]), split(a3, ah[3], al[3]);
        } else {
            ah[0] = __float_as_uint(a0), ah[1] = __float_as_uint(a1), ah[2] = __float_as_uint(a2), ah[3] = __float_as_uint(a3);
        }
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            int i0, i1;
            b_index<TRANS>(ks, nt, sb, g, t, i0, i1);
            if constexpr (X3) {
                uint32_t h0, l0, h1, l1;
                split(tile[i0], h0, l0), split(tile[i1], h1, l1);
                mma(acc[nt], al, h0, h1);
                mma(acc[nt], ah, l0, l1);
                mma(acc[nt], ah, h0, h1);
            } else {
                mma(acc[nt], ah, __float_as_uint(tile[i0]), __float_as_uint(tile[i1]));
            }
        }
    }
}
// A 16 x 64 block in accumulator layout into this warp's staging area: as TF32, or as it is for split products.
template <bool X3>
__device__ __forceinline__ void stage(float* p, const float (&v)[8][4], int g, int t) {
#pragma unroll
    for (int nt = 0; nt < 8; nt++) {
        float2 lo = make_float2(v[nt][0], v[nt][1]), hi = make_float2(v[nt][2], v[nt][3]);
        if constexpr (!X3) {
            lo = make_float2(__uint_as_float(tf32(lo.x)), __uint_as_float(tf32(lo.y)));
            hi = make_float2(__uint_as_float(tf32(hi.x)), __uint_as_float(tf32(hi.y)));
        }
        *reinterpret_cast<float2*>(p + g * S_P + nt * 8 + 2 * t) = lo;
        *reinterpret_cast<float2*>(p + (g + 8) * S_P + nt * 8 + 2 * t) = hi;
    }
}
__device__ __forceinline__ void zero(float (&v)[8][4]) {
#pragma unroll
    for (int nt = 0; nt < 8; nt++) v[nt][0] = v[nt][1] = v[nt][2] = v[nt][3] = 0;
}

// ---------------------------------------------------------------- forward

// grid (T / 64, B * H). out = softmax(scale * Q K^T, causal) V; L = scale * row max + log(row sum).
// X3: fp32-class products (operands split in two TF32 pieces); otherwise plain TF32 products.
template <bool X3>
__global__ void __launch_bounds__(kThreads) k_attn_fwd(const float* __restrict__ qkv, float* __restrict__ out,
                                                       float* __restrict__ L, int T, int H, float scale) {
    extern __shared__ float smem[];
    float* sK = smem;
    float* sV = sK + BT * S_NK;
    float* sP = sV + BT * S_KN;
    float* sQ = sP + 4 * 16 * S_P;              // X3 only: the block's queries, unrounded
    const int qt = gridDim.x - 1 - blockIdx.x;  // the long rows of the causal triangle first
    const int bh = blockIdx.y, b = bh / H, h = bh % H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int64_t ld = (int64_t)3 * H * HS;
    const float* q = qkv + (int64_t)b * T * ld + h * HS;
    const float* k = q + H * HS;
    const float* v = k + H * HS;
    const int row0 = qt * BT + warp * 16;
    float* myP = sP + warp * 16 * S_P;

    uint32_t qa[X3 ? 1 : 8][4];
    if constexpr (X3) load_tile<true>(sQ, S_NK, q, ld, qt * BT);  // visible after the barriers of the first tile
    else load_a(qa, q, ld, row0, g, t);
    float o[8][4];
    zero(o);
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0, l1 = 0;  // maxima of the unscaled products
    const float sl2 = scale * kLog2e;

    for (int j = 0; j <= qt; j++) {
        __syncthreads();  // every warp is done with the previous tile
        load_tile<X3>(sK, S_NK, k, ld, j * BT);
        load_tile<X3>(sV, S_KN, v, ld, j * BT);
        __syncthreads();
        float s[8][4];
        zero(s);
        if constexpr (X3) gemm_sa<true, true>(s, sQ + warp * 16 * S_NK, S_NK, sK, S_NK, g, t);
        else gemm_ra<true>(s, qa, sK, S_NK, g, t);
        if (j == qt) {  // the diagonal tile: keys after the query are masked
#pragma unroll
            for (int nt = 0; nt < 8; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (nt * 8 + 2 * t + (e & 1) > warp * 16 + g + (e >> 1) * 8) s[nt][e] = -INFINITY;
        }
        // running maxima of the raw products; scale > 0 is folded into the exponent: exp(scale * (s - m)) = 2^(sl2 * s - sl2 * m)
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; nt++) mx0 = fmaxf(mx0, fmaxf(s[nt][0], s[nt][1])), mx1 = fmaxf(mx1, fmaxf(s[nt][2], s[nt][3]));
        mx0 = quad_max(mx0), mx1 = quad_max(mx1);
        const float n0 = fmaxf(m0, mx0), n1 = fmaxf(m1, mx1);  // finite: every row sees its own column at the latest
        const float c0 = ex2((m0 - n0) * sl2), c1 = ex2((m1 - n1) * sl2);  // 0 the first time (m = -inf)
        const float b0 = n0 * sl2, b1 = n1 * sl2;
        m0 = n0, m1 = n1;
        float r0 = 0, r1 = 0;
#pragma unroll
        for (int nt = 0; nt < 8; nt++) {
            if constexpr (X3) {  // the difference first: exact for the entries near the maximum, which carry the sum
                s[nt][0] = ex2((s[nt][0] - n0) * sl2), s[nt][1] = ex2((s[nt][1] - n0) * sl2);
                s[nt][2] = ex2((s[nt][2] - n1) * sl2), s[nt][3] = ex2((s[nt][3] - n1) * sl2);
            } else {
                s[nt][0] = ex2(__fmaf_rn(s[nt][0], sl2, -b0)), s[nt][1] = ex2(__fmaf_rn(s[nt][1], sl2, -b0));
                s[nt][2] = ex2(__fmaf_rn(s[nt][2], sl2, -b1)), s[nt][3] = ex2(__fmaf_rn(s[nt][3], sl2, -b1));
            }
            r0 += s[nt][0] + s[nt][1], r1 += s[nt][2] + s[nt][3];
            o[nt][0] *= c0, o[nt][1] *= c0, o[nt][2] *= c1, o[nt][3] *= c1;
        }
        l0 = l0 * c0 + r0, l1 = l1 * c1 + r1;  // per-lane part of the row sum; the four lanes of a row meet at the end
        stage<X3>(myP, s, g, t);
        __syncwarp();
        gemm_sa<X3, false>(o, myP, S_P, sV, S_KN, g, t);
        __syncwarp();
    }
    l0 = quad_sum(l0), l1 = quad_sum(l1);
    const float i0 = 1.0f / l0, i1 = 1.0f / l1;
    float* o0 = out + ((int64_t)(b * T + row0 + g) * H + h) * HS;
    float* o1 = out + ((int64_t)(b * T + row0 + g + 8) * H + h) * HS;
#pragma unroll
    for (int nt = 0; nt < 8; nt++) {
        *reinterpret_cast<float2*>(o0 + nt * 8 + 2 * t) = make_float2(o[nt][0] * i0, o[nt][1] * i0);
        *reinterpret_cast<float2*>(o1 + nt * 8 + 2 * t) = make_float2(o[nt][2] * i1, o[nt][3] * i1);
    }
    if (t == 0) {
        L[(int64_t)bh * T + row0 + g] = m0 * scale + logf(l0);
        L[(int64_t)bh * T + row0 + g + 8] = m1 * scale + logf(l1);
    }
}

// ---------------------------------------------------------------- backward

// D[bh][q] = sum over d of dout * out (core/cuda/kernels.cu:664-666). One warp per row.
__global__ void __launch_bounds__(kThreads) k_attn_rowdot(const float* __restrict__ out, const float* __restrict__ dout,
                                                          float* __restrict__ D, int B, int T, int H) {
    const int64_t row = (int64_t)blockIdx.x * (kThreads / 32) + (threadIdx.x >> 5);  // over (b, t, h)
    if (row >= (int64_t)B * T * H) return;
    const int lane = threadIdx.x & 31;
    const float2 a = *reinterpret_cast<const float2*>(out + row * HS + lane * 2);
    const float2 d = *reinterpret_cast<const float2*>(dout + row * HS + lane * 2);
    float s = a.x * d.x + a.y * d.y;
    for (int o = 16; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) {
        const int h = (int)(row % H);
        const int64_t bt = row / H;
        D[((bt / T) * H + h) * T + bt % T] = s;
    }
}

// grid (T / 64, B * H): dQ of 64 query rows, key tiles 0 .. own. P = exp(scale S - L); dS = P (dP - D) scale.
template <bool X3>
__global__ void __launch_bounds__(kThreads) k_attn_bwd_dq(const float* __restrict__ qkv, const float* __restrict__ dout,
                                                          const float* __restrict__ L, const float* __restrict__ D,
                                                          float* __restrict__ dqkv, int T, int H, float scale) {
    extern __shared__ float smem[];
    float* sK = smem;               // stride S_NK: read as K^T for S = Q K^T
    float* sV = sK + BT * S_NK;     // stride S_NK: read as V^T for dP = dO V^T
    // TF32: the same keys again with stride S_KN, read as K for dQ += dS K free of bank conflicts. The split-product
    // kernel is bound by its products and short of shared memory: it reads sK both ways.
    float* sK2 = X3 ? sK : sV + BT * S_NK;
    constexpr int S_K2 = X3 ? S_NK : S_KN;
    float* sP = sV + BT * S_NK + (X3 ? 0 : BT * S_KN);
    float* sQ = sP + 4 * 16 * S_P;  // X3 only: the block's queries and output gradients, unrounded
    float* sO = sQ + BT * S_NK;
    const int qt = gridDim.x - 1 - blockIdx.x;
    const int bh = blockIdx.y, b = bh / H, h = bh % H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int64_t ld = (int64_t)3 * H * HS, ldo = (int64_t)H * HS;
    const float* q = qkv + (int64_t)b * T * ld + h * HS;
    const float* k = q + H * HS;
    const float* v = k + H * HS;
    const float* dO = dout + (int64_t)b * T * ldo + h * HS;
    const int row0 = qt * BT + warp * 16;
    float* myP = sP + warp * 16 * S_P;

    uint32_t qa[X3 ? 1 : 8][4], da[X3 ? 1 : 8][4];
    if constexpr (X3) {
        load_tile<true>(sQ, S_NK, q, ld, qt * BT);  // visible after the barriers of the first tile
        load_tile<true>(sO, S_NK, dO, ldo, qt * BT);
    } else {
        load_a(qa, q, ld, row0, g, t);
        load_a(da, dO, ldo, row0, g, t);
    }
    const float sl2 = scale * kLog2e;  // exp(scale * s - L) = 2^(sl2 * s - log2(e) * L)
    const float L0 = L[(int64_t)bh * T + row0 + g] * kLog2e, L1 = L[(int64_t)bh * T + row0 + g + 8] * kLog2e;
    const float D0 = D[(int64_t)bh * T + row0 + g], D1 = D[(int64_t)bh * T + row0 + g + 8];
    float dq[8][4];
    zero(dq);

    for (int j = 0; j <= qt; j++) {
        __syncthreads();
        if constexpr (X3) load_tile<true>(sK, S_NK, k, ld, j * BT);
        else load_tile2<false>(sK, S_NK, sK2, S_KN, k, ld, j * BT);
        load_tile<X3>(sV, S_NK, v, ld, j * BT);
        __syncthreads();
        float s[8][4], dp[8][4];
        zero(s), zero(dp);
        if constexpr (X3) {
            gemm_sa<true, true>(s, sQ + warp * 16 * S_NK, S_NK, sK, S_NK, g, t);
            gemm_sa<true, true>(dp, sO + warp * 16 * S_NK, S_NK, sV, S_NK, g, t);
        } else {
            gemm_ra<true>(s, qa, sK, S_NK, g, t);
            gemm_ra<true>(dp, da, sV, S_NK, g, t);
        }
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) s[nt][e] = ex2(__fmaf_rn(s[nt][e], sl2, -(e < 2 ? L0 : L1)));  // P
        if (j == qt) {  // the diagonal tile: keys after the query have probability 0
#pragma unroll
            for (int nt = 0; nt < 8; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (nt * 8 + 2 * t + (e & 1) > warp * 16 + g + (e >> 1) * 8) s[nt][e] = 0.0f;
        }
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) s[nt][e] = s[nt][e] * (dp[nt][e] - (e < 2 ? D0 : D1)) * scale;  // dS
        stage<X3>(myP, s, g, t);
        __syncwarp();
        gemm_sa<X3, false>(dq, myP, S_P, sK2, S_K2, g, t);
        __syncwarp();
    }
    float* g0 = dqkv + (int64_t)(b * T + row0 + g) * ld + h * HS;
    float* g1 = dqkv + (int64_t)(b * T + row0 + g + 8) * ld + h * HS;
#pragma unroll
    for (int nt = 0; nt < 8; nt++) {
        *reinterpret_cast<float2*>(g0 + nt * 8 + 2 * t) = make_float2(dq[nt][0], dq[nt][1]);
        *reinterpret_cast<float2*>(g1 + nt * 8 + 2 * t) = make_float2(dq[nt][2], dq[nt][3]);
    }
}

// grid (T / 64, B * H): dK and dV of 64 key rows, query tiles own .. last. Works on the transposed problem: rows are
// keys, columns queries. P^T = exp(scale K Q^T - L[q]); dV += P^T dO; dP^T = V dO^T; dS^T = P^T (dP^T - D[q]) scale;
// dK += dS^T Q.
template <bool X3>
__global__ void __launch_bounds__(kThreads) k_attn_bwd_dkv(const float* __restrict__ qkv, const float* __restrict__ dout,
                                                           const float* __restrict__ L, const float* __restrict__ D,
                                                           float* __restrict__ dqkv, int T, int H, float scale) {
    extern __shared__ float smem[];
    float* sQ = smem;               // stride S_NK: read as Q^T for S^T = K Q^T
    float* sO = sQ + BT * S_NK;     // dO, stride S_NK: read as dO^T for dP^T = V dO^T
    // TF32: the same two tiles again with stride S_KN, read as Q for dK += dS^T Q and as dO for dV += P^T dO free of
    // bank conflicts. The split-product kernel is bound by its products and short of shared memory: one copy, both ways.
    float* sQ2 = X3 ? sQ : sO + BT * S_NK;
    float* sO2 = X3 ? sO : sQ2 + BT * S_KN;
    constexpr int S_2 = X3 ? S_NK : S_KN;
    float* sP = sO + BT * S_NK + (X3 ? 0 : 2 * BT * S_KN);
    float* sL = sP + 4 * 16 * S_P;  // L and D of the 64 queries of the tile
    float* sD = sL + BT;
    float* sK = sD + BT;            // X3 only: the block's keys and values, unrounded
    float* sV = sK + BT * S_NK;
    const int kt = blockIdx.x;      // key tile 0 has the most query tiles: blocks are issued in that order
    const int bh = blockIdx.y, b = bh / H, h = bh % H;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int64_t ld = (int64_t)3 * H * HS, ldo = (int64_t)H * HS;
    const float* q = qkv + (int64_t)b * T * ld + h * HS;
    const float* k = q + H * HS;
    const float* v = k + H * HS;
    const float* dO = dout + (int64_t)b * T * ldo + h * HS;
    const int row0 = kt * BT + warp * 16;  // key rows of this warp
    float* myP = sP + warp * 16 * S_P;

    const float sl2 = scale * kLog2e;
    uint32_t ka[X3 ? 1 : 8][4], va[X3 ? 1 : 8][4];
    if constexpr (X3) {
        load_tile<true>(sK, S_NK, k, ld, kt * BT);  // visible after the barriers of the first tile
        load_tile<true>(sV, S_NK, v, ld, kt * BT);
    } else {
        load_a(ka, k, ld, row0, g, t);
        load_a(va, v, ld, row0, g, t);
    }
    float dk[8][4], dv[8][4];
    zero(dk), zero(dv);

    const int tiles = T / BT;
    for (int i = kt; i < tiles; i++) {
        __syncthreads();
        if constexpr (X3) {
            load_tile<true>(sQ, S_NK, q, ld, i * BT);
            load_tile<true>(sO, S_NK, dO, ldo, i * BT);
        } else {
            load_tile2<false>(sQ, S_NK, sQ2, S_KN, q, ld, i * BT);
            load_tile2<false>(sO, S_NK, sO2, S_KN, dO, ldo, i * BT);
        }
        if (threadIdx.x < BT) {
            sL[threadIdx.x] = L[(int64_t)bh * T + i * BT + threadIdx.x] * kLog2e;
            sD[threadIdx.x] = D[(int64_t)bh * T + i * BT + threadIdx.x];
        }
        __syncthreads();
        float s[8][4], dp[8][4];
        zero(s), zero(dp);
        if constexpr (X3) {
            gemm_sa<true, true>(s, sK + warp * 16 * S_NK, S_NK, sQ, S_NK, g, t);    // S^T: rows keys, columns queries
            gemm_sa<true, true>(dp, sV + warp * 16 * S_NK, S_NK, sO, S_NK, g, t);   // dP^T
        } else {
            gemm_ra<true>(s, ka, sQ, S_NK, g, t);
            gemm_ra<true>(dp, va, sO, S_NK, g, t);
        }
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) s[nt][e] = ex2(__fmaf_rn(s[nt][e], sl2, -sL[nt * 8 + 2 * t + (e & 1)]));  // P^T
        if (i == kt) {  // the diagonal tile: keys after the query have probability 0
#pragma unroll
            for (int nt = 0; nt < 8; nt++)
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (warp * 16 + g + (e >> 1) * 8 > nt * 8 + 2 * t + (e & 1)) s[nt][e] = 0.0f;
        }
#pragma unroll
        for (int nt = 0; nt < 8; nt++)
#pragma unroll
            for (int e = 0; e < 4; e++) dp[nt][e] = s[nt][e] * (dp[nt][e] - sD[nt * 8 + 2 * t + (e & 1)]) * scale;  // dS^T
        stage<X3>(myP, s, g, t);
        __syncwarp();
        gemm_sa<X3, false>(dv, myP, S_P, sO2, S_2, g, t);
        __syncwarp();
        stage<X3>(myP, dp, g, t);
        __syncwarp();
        gemm_sa<X3, false>(dk, myP, S_P, sQ2, S_2, g, t);
        __syncwarp();
    }
    float* k0 = dqkv + (int64_t)(b * T + row0 + g) * ld + (H + h) * HS;
    float* k1 = dqkv + (int64_t)(b * T + row0 + g + 8) * ld + (H + h) * HS;
#pragma unroll
    for (int nt = 0; nt < 8; nt++) {
        *reinterpret_cast<float2*>(k0 + nt * 8 + 2 * t) = make_float2(dk[nt][0], dk[nt][1]);
        *reinterpret_cast<float2*>(k1 + nt * 8 + 2 * t) = make_float2(dk[nt][2], dk[nt][3]);
        *reinterpret_cast<float2*>(k0 + H * HS + nt * 8 + 2 * t) = make_float2(dv[nt][0], dv[nt][1]);
        *reinterpret_cast<float2*>(k1 + H * HS + nt * 8 + 2 * t) = make_float2(dv[nt][2], dv[nt][3]);
    }
}

// Shared memory per block; the split-product kernels also keep their own side's tile(s) there.
constexpr size_t fwd_smem(bool x3) { return (size_t)(BT * S_NK + BT * S_KN + 4 * 16 * S_P + (x3 ? BT * S_NK : 0)) * sizeof(float); }
constexpr size_t dq_smem(bool x3) { return (size_t)(2 * BT * S_NK + 4 * 16 * S_P + (x3 ? 2 * BT * S_NK : BT * S_KN)) * sizeof(float); }
constexpr size_t dkv_smem(bool x3) { return (size_t)(2 * BT * S_NK + 4 * 16 * S_P + 2 * BT + (x3 ? 2 * BT * S_NK : 2 * BT * S_KN)) * sizeof(float); }

static bool allow(const void* kernel, size_t smem) {
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess;
}
static void report(cudaError_t e) {
    if (e != cudaSuccess) slb::Engine::get().set_error(slb::ERR_LAUNCH);
}
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
static bool g_tf32 = false;  // sl_cuda_attention_set_tf32

template <bool X3>
static void forward(const float* qkv, float* out, float* L, int64_t B, int64_t T, int64_t H, float scale) {
    static const bool ok = allow((const void*)k_attn_fwd<X3>, fwd_smem(X3));
    if (!ok) return report(cudaErrorInvalidValue);
    k_attn_fwd<X3><<<dim3((unsigned)(T / BT), (unsigned)(B * H)), kThreads, fwd_smem(X3)>>>(qkv, out, L, (int)T, (int)H, scale);
    report(cudaPeekAtLastError());
}
template <bool X3>
static void backward(const float* qkv, const float* L, const float* dout, const float* rowdot, float* dqkv, int64_t B, int64_t T,
                     int64_t H, float scale) {
    static const bool ok = allow((const void*)k_attn_bwd_dq<X3>, dq_smem(X3)) && allow((const void*)k_attn_bwd_dkv<X3>, dkv_smem(X3));
    if (!ok) return report(cudaErrorInvalidValue);
    const dim3 grid((unsigned)(T / BT), (unsigned)(B * H));
    k_attn_bwd_dq<X3><<<grid, kThreads, dq_smem(X3)>>>(qkv, dout, L, rowdot, dqkv, (int)T, (int)H, scale);
    k_attn_bwd_dkv<X3><<<grid, kThreads, dkv_smem(X3)>>>(qkv, dout, L, rowdot, dqkv, (int)T, (int)H, scale);
    report(cudaPeekAtLastError());
}

}  // namespace slb_attn

using namespace slb_attn;

extern "C" int sl_cuda_attention_supported(int64_t T, int64_t hs) { return hs == HS && T >= BT && T % BT == 0 ? 1 : 0; }

extern "C" void sl_cuda_attention_set_tf32(int on) { g_tf32 = on != 0; }

extern "C" void sl_cuda_attention(const float* qkv, float* out, float* L, int64_t B, int64_t T, int64_t H, int64_t hs,
                                  float scale, int64_t tile, float* s, float* acc, float* m, float* l, float* c,
                                  float* rowbuf, float* ones, void* ptrs) {
    (void)tile, (void)s, (void)acc, (void)m, (void)l, (void)c, (void)rowbuf, (void)ones, (void)ptrs;  // the reference's scratch: unused
    if (B <= 0 || H <= 0) return;
    if (!sl_cuda_attention_supported(T, hs) || !aligned16(qkv) || !aligned16(out)) return report(cudaErrorInvalidValue);
    if (g_tf32) forward<false>(qkv, out, L, B, T, H, scale);
    else forward<true>(qkv, out, L, B, T, H, scale);
}

extern "C" void sl_cuda_attention_bwd(const float* qkv, const float* out, const float* L, const float* dout, float* dqkv,
                                      int64_t B, int64_t T, int64_t H, int64_t hs, float scale, int64_t tile, float* s,
                                      float* dp, float* doc, float* oc, float* lrow, float* D, float* rowbuf, float* ones,
                                      void* ptrs) {
    (void)tile, (void)s, (void)dp, (void)doc, (void)lrow, (void)D, (void)rowbuf, (void)ones, (void)ptrs;
    if (B <= 0 || H <= 0) return;
    if (!sl_cuda_attention_supported(T, hs) || !aligned16(qkv) || !aligned16(dout) || !aligned16(dqkv) || !oc)
        return report(cudaErrorInvalidValue);
    // `oc` (B * H * tile * 64 floats of the reference's scratch, tile >= 64) holds the B * H * T row dots
    float* rowdot = oc;
    const int64_t rows = B * T * H;
    k_attn_rowdot<<<(unsigned)((rows + kThreads / 32 - 1) / (kThreads / 32)), kThreads>>>(out, dout, rowdot, (int)B, (int)T, (int)H);
    report(cudaPeekAtLastError());
    if (g_tf32) backward<false>(qkv, L, dout, rowdot, dqkv, B, T, H, scale);
    else backward<true>(qkv, L, dout, rowdot, dqkv, B, T, H, scale);
}
