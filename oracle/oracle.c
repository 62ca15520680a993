/*
 * TEST INFRASTRUCTURE ONLY -- never linked into, imported by or called from the product library.
 *
 * CPU restatement of the arithmetic on Soliton's data-parallel optimizer path: the host kernels of
 * core/soliton/cpu.d (axpy, scale, sumsq, adamw) plus the gradient mean the path computes across ranks.
 * Only the tests, the smoke check and the CPU-baseline leg of the benchmark may load this file's library.
 *
 * Parity status: PINNED. The restatement is checked (tests/test_oracle.py) against torch.optim.AdamW on CPU
 * with the reference's own recipe (tests/test_ops.py:121-134, rtol 1e-5 / atol 1e-6), and on a GPU
 * (tests/test_gpu_reference.py) bit for bit against the reference's own k_adamw (core/cuda/kernels.cu:242-254)
 * compiled unmodified into oracle/_ref/. The cross-rank summation order of NCCL (the reference's all-reduce,
 * core/cuda/kernels.cu:773-775) is a third-party detail the reference does not pin; the order used here is the
 * fixed rank order the product guarantees: ((g0 + g1) + g2) + ... then one multiply by 1/world.
 *
 * Build: gcc -O3 -ffp-contract=off -shared -fPIC (see oracle/build.py). Contraction is off so that every
 * fused multiply-add below is one that is written out with fmaf()/fma().
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <time.h>

/* core/soliton/cpu.d:85-89  y[i] += alpha * x[i] */
void oracle_axpy(const float* x, float* y, int64_t n, float alpha) {
    for (int64_t i = 0; i < n; i++) y[i] += alpha * x[i];
}

/* core/soliton/cpu.d:97-101  y[i] = alpha * x[i] */
void oracle_scale(const float* x, float* y, int64_t n, float alpha) {
    for (int64_t i = 0; i < n; i++) y[i] = alpha * x[i];
}

/* core/soliton/cpu.d:103-109  double accumulator over float squares, index order */
double oracle_sumsq(const float* x, int64_t n) {
    double s = 0;
    for (int64_t i = 0; i < n; i++) s += (double)x[i] * x[i];
    return s;
}

/*
 * core/soliton/cpu.d:362-373. m and v are updated in float (left-associated, "(1 - b1)" is a float), the
 * bias corrections are doubles from pow(double,double), "wd * p" is rounded in float before it is promoted,
 * and the rest of the parameter update runs in double and is rounded to float once.
 * No contraction: LDC does not fuse a*b+c without fast-math flags.
 */
void oracle_adamw(float* p, const float* g, float* m, float* v, int64_t n, float lr, float b1, float b2,
                  float eps, float wd, int step) {
    const double bc1 = 1.0 - pow((double)b1, (double)step), bc2 = 1.0 - pow((double)b2, (double)step);
    for (int64_t i = 0; i < n; i++) {
        m[i] = b1 * m[i] + (1 - b1) * g[i];
        v[i] = b2 * v[i] + (1 - b2) * g[i] * g[i];
        const double mh = m[i] / bc1, vh = v[i] / bc2;
        p[i] = (float)(p[i] - lr * (mh / (sqrt(vh) + eps) + wd * p[i]));
    }
}

/*
 * core/cuda/kernels.cu:242-254 (k_adamw and its host wrapper): the same formula as compiled by nvcc with its
 * default contraction (-fmad=true). The products feeding each sum become FMAs: m = fma(b1, m, (1-b1)*g),
 * v = fma(b2, v, ((1-b2)*g)*g), and in double p - lr*x = fma(-lr, x, p). The host computes
 * bc = 1.0 - pow(b, step) with both arguments promoted to double. Differs from oracle_adamw only from the
 * second step on (when m, v are non-zero) and then by at most one float ulp in m and v.
 */
void oracle_adamw_fma(float* p, const float* g, float* m, float* v, int64_t n, float lr, float b1, float b2,
                      float eps, float wd, int step) {
    const double bc1 = 1.0 - pow((double)b1, (double)step), bc2 = 1.0 - pow((double)b2, (double)step);
    const float c1 = 1 - b1, c2 = 1 - b2;
    for (int64_t i = 0; i < n; i++) {
        const float gi = g[i];
        m[i] = fmaf(b1, m[i], c1 * gi);
        v[i] = fmaf(b2, v[i], (c2 * gi) * gi);
        const double mh = m[i] / bc1, vh = v[i] / bc2;
        const double x = mh / (sqrt(vh) + (double)eps) + (double)(wd * p[i]);
        p[i] = (float)fma(-(double)lr, x, (double)p[i]);
    }
}

/*
 * Mean of `world` per-rank gradients in the product's fixed order: sum ranks 0..world-1 left to right in
 * float, then multiply once by the float 1/world. The reference has no host all-reduce
 * (core/soliton/api.d:587-590 returns 0 off CUDA); composed from its axpy and scale this is
 * acc = g0; axpy(g_r, acc, 1) for r >= 1; scale(acc, out, 1/world).
 */
void oracle_mean_ranks(const float* const* g, int world, int64_t n, float* out) {
    const float inv = 1.0f / (float)world;
    for (int64_t i = 0; i < n; i++) {
        float s = g[0][i];
        for (int r = 1; r < world; r++) s += g[r][i];
        out[i] = s * inv;
    }
}

/* One rank's whole host step for one tensor: mean of the ranks' gradients into gavg, then AdamW. */
void oracle_dp_step(float* p, float* m, float* v, float* gavg, const float* const* g, int world, int64_t n,
                    float lr, float b1, float b2, float eps, float wd, int step, int fma_shape) {
    oracle_mean_ranks(g, world, n, gavg);
    if (fma_shape)
        oracle_adamw_fma(p, gavg, m, v, n, lr, b1, b2, eps, wd, step);
    else
        oracle_adamw(p, gavg, m, v, n, lr, b1, b2, eps, wd, step);
}

/*
 * Gradient clipping as python/soliton/optim.py:31-39 does it on the host device: the norm is the square root
 * of the sum over tensors of sumsq, and the scale max_norm / (norm + 1e-6) is applied in place when the norm
 * exceeds max_norm. Returns the pre-clip norm.
 */
double oracle_clip(float* const* g, const int64_t* n, int ntensors, double max_norm) {
    double tot = 0;
    for (int t = 0; t < ntensors; t++) tot += oracle_sumsq(g[t], n[t]);
    const double norm = sqrt(tot);
    if (norm > max_norm) {
        const float s = (float)(max_norm / (norm + 1e-6));
        for (int t = 0; t < ntensors; t++) oracle_scale(g[t], g[t], n[t], s);
    }
    return norm;
}


/*
 * Sum of squares the way the two-shot gradient mean accumulates it for the clip that follows
 * (python/soliton/optim.py:31-39 asks for it tensor by tensor; the reference answers with cublasSdot,
 * core/cuda/kernels.cu:219-224, whose summation order is not pinned). A "piece" is the part of one tensor that one
 * thread block reduces in one go: tiles [tile_a, tile_b) of the tensor, 2048 floats each, the last one of a tensor
 * possibly shorter. 256 threads each keep one double: in a whole tile of a 32-byte aligned tensor (vec != 0)
 * thread t squares elements 8t .. 8t+7 in order, in any other tile elements t, t+256, ...; every square enters with
 * one fused multiply-add. At the end of the piece the 32 lanes of a warp combine in a halving tree (lane l adds
 * lane l + 16, then + 8, ...), and the eight warp results are added in warp order.
 */
double oracle_sumsq_piece(const float* x, int64_t n, int64_t tile_a, int64_t tile_b, int vec) {
    enum { TILE = 2048, THREADS = 256 };
    double acc[THREADS];
    for (int t = 0; t < THREADS; t++) acc[t] = 0.0;
    for (int64_t k = tile_a; k < tile_b; k++) {
        const int64_t base = k * TILE;
        const int64_t cnt = n - base < TILE ? n - base : TILE;
        if (vec && cnt == TILE) {
            for (int t = 0; t < THREADS; t++)
                for (int j = 0; j < 8; j++) {
                    const double v = (double)x[base + 8 * t + j];
                    acc[t] = fma(v, v, acc[t]);
                }
        } else {
            for (int t = 0; t < THREADS; t++)
                for (int64_t e = t; e < cnt; e += THREADS) {
                    const double v = (double)x[base + e];
                    acc[t] = fma(v, v, acc[t]);
                }
        }
    }
    double total = 0.0;
    for (int w = 0; w < THREADS / 32; w++) {
        double lane[32];
        for (int l = 0; l < 32; l++) lane[l] = acc[32 * w + l];
        for (int o = 16; o; o >>= 1)
            for (int l = 0; l < o; l++) lane[l] = lane[l] + lane[l + o];
        total += lane[0];
    }
    return total;
}

/* ---- timing harness for the CPU baseline: `threads` host ranks each run the whole per-rank path ---- */

typedef struct {
    float *p, *m, *v, *acc;
    const float* const* g;
    int world, reps;
    int64_t n;
    double seconds;
} bench_arg;

static double now_s(void) {
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec + 1e-9 * ts.tv_nsec;
}

static void* bench_rank(void* a_) {
    bench_arg* a = (bench_arg*)a_;
    const double t0 = now_s();
    for (int r = 0; r < a->reps; r++) {
        /* the host composition of the reference's kernels: copy, axpy per further rank, scale, adamw */
        memcpy(a->acc, a->g[0], (size_t)a->n * sizeof(float));
        for (int q = 1; q < a->world; q++) oracle_axpy(a->g[q], a->acc, a->n, 1.0f);
        if (a->world > 1) oracle_scale(a->acc, a->acc, a->n, 1.0f / (float)a->world);
        oracle_adamw(a->p, a->acc, a->m, a->v, a->n, 3e-4f, 0.9f, 0.999f, 1e-8f, 0.1f, r + 1);
    }
    a->seconds = now_s() - t0;
    return NULL;
}

/*
 * Runs `reps` host steps over n parameters on each of `threads` threads (one thread stands for one rank's
 * host process; the reference's CPU kernels are single-threaded loops). g holds `world` gradient buffers that
 * all threads read; every thread owns its p, m, v. Returns the slowest thread's seconds, or -1 on failure.
 */
double oracle_bench(const float* p0, const float* const* g, int world, int64_t n, int reps, int threads) {
    if (threads < 1 || threads > 64) return -1;
    bench_arg args[64];
    pthread_t tid[64];
    for (int t = 0; t < threads; t++) {
        bench_arg* a = &args[t];
        a->p = (float*)malloc((size_t)n * 4);
        a->m = (float*)malloc((size_t)n * 4);
        a->v = (float*)malloc((size_t)n * 4);
        a->acc = (float*)malloc((size_t)n * 4);
        if (!a->p || !a->m || !a->v || !a->acc) return -1;
        memcpy(a->p, p0, (size_t)n * 4);
        /* every page is touched before the clock starts: the steady state of a training loop, not its first step */
        memset(a->m, 0, (size_t)n * 4), memset(a->v, 0, (size_t)n * 4), memset(a->acc, 0, (size_t)n * 4);
        a->g = g, a->world = world, a->n = n, a->reps = reps, a->seconds = 0;
    }
    for (int t = 0; t < threads; t++)
        if (pthread_create(&tid[t], NULL, bench_rank, &args[t])) return -1;
    double worst = 0;
    for (int t = 0; t < threads; t++) {
        pthread_join(tid[t], NULL);
        if (args[t].seconds > worst) worst = args[t].seconds;
        free(args[t].p), free(args[t].m), free(args[t].v), free(args[t].acc);
    }
    return worst;
}
