// The rest of Soliton's C ABI, so that the UNMODIFIED Soliton Python package (python/soliton/_C.py:11-70 resolves all
// 55 `sl_*` names when it is imported) can run whole training steps on top of libsoliton_b200: the 33 entry points of
// the optimizer path and its surroundings come from this repository's library; the 22 defined here -- everything
// forward and backward needs -- go to the reference's own CUDA backend, core/cuda/kernels.cu compiled unmodified into
// a shared object (oracle/_ref/), loaded at run time.
//
// This file takes the place of the op section of Soliton's D core (core/soliton/api.d:262-569), which cannot be
// built here (no D compiler). What it has to keep is the allocator traffic: every scratch buffer of an op is taken
// from the deterministic pool in the order api.d takes it, on meta as on cuda, and released in reverse order when
// the op returns, because the meta dry run predicts the cuda run's peak bytes only if both replay the same trace.
// Each entry cites the api.d lines whose scratch sequence it restates. There are no host kernels: ops on the cpu
// device raise sticky error 13 like the rest of the library.
//
// Test and benchmark infrastructure, not part of the product library: it exists so that full data-parallel training
// steps (the callers on either side of the optimizer path) can be measured and checked end to end.
#include <dlfcn.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "../include/soliton_b200.h"
#include "../soliton_b200/csrc/dp_engine.hpp"
#include "../soliton_b200/csrc/foreign_path.h"
#include "../soliton_b200/csrc/pool.hpp"

using namespace slb;

namespace {

// ---- the reference backend, bound by name

struct Backend {
    void* so = nullptr;
    int (*set_device)(int) = nullptr;
    int (*check)() = nullptr;
    void (*set_workspace)(void*, size_t) = nullptr;
    void (*set_tf32)(int) = nullptr;
    void (*binary)(int, const float*, const float*, float*, int, const int64_t*, const int64_t*, const int64_t*) = nullptr;
    void (*strided_copy)(const float*, int64_t, float*, int, const int64_t*, const int64_t*) = nullptr;
    void (*reduce_sum)(const float*, float*, int64_t, int, const int64_t*, const int64_t*, float*) = nullptr;
    void (*add_scalar)(float*, int64_t, float) = nullptr;
    void (*matmul)(const float*, const float*, float*, int64_t, int64_t, int64_t, int64_t, int, int) = nullptr;
    void (*softmax)(const float*, float*, int64_t, int64_t, int64_t, float*, float*, float*, float*) = nullptr;
    void (*softmax_bwd)(const float*, const float*, float*, int64_t, int64_t, float*, float*) = nullptr;
    void (*gelu)(const float*, float*, int64_t) = nullptr;
    void (*gelu_bwd)(const float*, const float*, float*, int64_t) = nullptr;
    void (*layernorm)(const float*, const float*, const float*, float*, float*, float*, int64_t, int64_t, float, float*) = nullptr;
    void (*layernorm_bwd)(const float*, const float*, const float*, const float*, const float*, float*, float*, float*,
                          int64_t, int64_t, float*, float*, float*, float*, float*) = nullptr;
    void (*embedding)(const float*, const int*, float*, int64_t, int64_t) = nullptr;
    void (*embedding_bwd)(const float*, const int*, float*, int64_t, int64_t, int64_t, int*, int*, int*, void*, size_t) = nullptr;
    double (*cross_entropy)(const float*, const int*, int64_t, int64_t, float*) = nullptr;
    void (*cross_entropy_bwd)(const float*, const int*, float*, int64_t, int64_t, float) = nullptr;
    void (*attention)(const float*, float*, float*, int64_t, int64_t, int64_t, int64_t, float, int64_t, float*, float*,
                      float*, float*, float*, float*, float*, void*) = nullptr;
    void (*attention_bwd)(const float*, const float*, const float*, const float*, float*, int64_t, int64_t, int64_t,
                          int64_t, float, int64_t, float*, float*, float*, float*, float*, float*, float*, float*, void*) = nullptr;
    // the reference's own data-parallel path and the small ops around it (core/cuda/kernels.cu:200-224,242-254,756-779)
    SlbForeignPath dp{};
    int (*nccl_unique_id)(char*) = nullptr;
    int (*jit)(const char*, const char*, void**) = nullptr;
    void (*jit_launch)(void*, int64_t, void**) = nullptr;
    void (*jit_free)(void*) = nullptr;
    const char* (*jit_log)() = nullptr;
    bool ok = false;
};

template <class F>
bool bind(void* so, const char* name, F& out) {
    out = reinterpret_cast<F>(dlsym(so, name));
    if (!out) fprintf(stderr, "fullstep: the reference backend lacks %s\n", name);
    return out != nullptr;
}

// Loaded at the first op on cuda: the library next to this one, or SOLITON_REF_BACKEND. RTLD_LOCAL keeps its
// sl_cuda_adamw / sl_cuda_nccl_* apart from this library's own.
Backend& backend() {
    static Backend b;
    static bool loaded = false, device_done = false;
    if (!loaded) {
        loaded = true;
        const char* path = getenv("SOLITON_REF_BACKEND");
        char beside[4096];
        if (!path) {
            Dl_info info;
            if (dladdr(reinterpret_cast<void*>(&backend), &info) && info.dli_fname) {
                snprintf(beside, sizeof beside, "%s", info.dli_fname);
                char* slash = strrchr(beside, '/');
                if (slash) {
                    snprintf(slash + 1, sizeof beside - (size_t)(slash + 1 - beside), "libsoliton_ref_cuda.so");
                    path = beside;
                }
            }
        }
        b.so = path ? dlopen(path, RTLD_NOW | RTLD_LOCAL) : nullptr;
        if (!b.so) {
            fprintf(stderr, "fullstep: cannot load the reference backend (%s)\n", dlerror());
            return b;
        }
        const bool all = bind(b.so, "sl_cuda_set_device", b.set_device) & bind(b.so, "sl_cuda_check", b.check) &
                         bind(b.so, "sl_cuda_set_workspace", b.set_workspace) & bind(b.so, "sl_cuda_set_tf32", b.set_tf32) &
                         bind(b.so, "sl_cuda_binary", b.binary) & bind(b.so, "sl_cuda_strided_copy", b.strided_copy) &
                         bind(b.so, "sl_cuda_reduce_sum", b.reduce_sum) & bind(b.so, "sl_cuda_add_scalar", b.add_scalar) &
                         bind(b.so, "sl_cuda_matmul", b.matmul) & bind(b.so, "sl_cuda_softmax", b.softmax) &
                         bind(b.so, "sl_cuda_softmax_bwd", b.softmax_bwd) & bind(b.so, "sl_cuda_gelu", b.gelu) &
                         bind(b.so, "sl_cuda_gelu_bwd", b.gelu_bwd) & bind(b.so, "sl_cuda_layernorm", b.layernorm) &
                         bind(b.so, "sl_cuda_layernorm_bwd", b.layernorm_bwd) & bind(b.so, "sl_cuda_embedding", b.embedding) &
                         bind(b.so, "sl_cuda_embedding_bwd", b.embedding_bwd) &
                         bind(b.so, "sl_cuda_cross_entropy", b.cross_entropy) &
                         bind(b.so, "sl_cuda_cross_entropy_bwd", b.cross_entropy_bwd) &
                         bind(b.so, "sl_cuda_attention", b.attention) & bind(b.so, "sl_cuda_attention_bwd", b.attention_bwd) &
                         bind(b.so, "sl_cuda_jit", b.jit) & bind(b.so, "sl_cuda_jit_launch", b.jit_launch) &
                         bind(b.so, "sl_cuda_jit_free", b.jit_free) & bind(b.so, "sl_cuda_jit_log", b.jit_log) &
                         bind(b.so, "sl_cuda_adamw", b.dp.adamw) & bind(b.so, "sl_cuda_nccl_unique_id", b.dp.dist_unique_id) &
                         bind(b.so, "sl_cuda_nccl_init", b.dp.dist_init) & bind(b.so, "sl_cuda_nccl_group", b.dp.dist_group) &
                         bind(b.so, "sl_cuda_nccl_allreduce_mean", b.dp.dist_allreduce_mean) &
                         bind(b.so, "sl_cuda_nccl_destroy", b.dp.dist_destroy) & bind(b.so, "sl_cuda_sumsq", b.dp.sumsq) &
                         bind(b.so, "sl_cuda_scale", b.dp.scale) & bind(b.so, "sl_cuda_axpy", b.dp.axpy);
        if (!all) {
            dlclose(b.so);
            b.so = nullptr;
        }
    }
    if (b.so && !device_done && Engine::get().cuda_ready()) {
        // core/soliton/api.d:262-274: the device is selected and the cuBLAS workspace, which sl_init_device took
        // from the pool, is handed to the backend
        device_done = true;
        Engine& e = Engine::get();
        if (b.set_device(e.ordinal()) == 0) {
            b.set_workspace(e.blas_workspace(), e.blas_workspace_bytes());
            b.ok = true;
        }
    }
    return b;
}

// What every op does first: on cuda, whatever the optimizer path has recorded goes out (an op may read parameters a
// deferred update is about to write); on cpu there is nothing to run.
enum Route { SKIP, RUN };
Route route(int dev) {
    if (dev == DEV_CUDA) {
        Engine& e = Engine::get();
        if (!e.cuda_ready()) {
            e.set_error(ERR_NO_WORKSPACE);
            return SKIP;
        }
        e.flush();
        if (!backend().ok) {
            e.set_error(ERR_LAUNCH);
            return SKIP;
        }
        return RUN;
    }
    if (dev == DEV_CPU) Engine::get().set_error(ERR_NO_CPU_COMPUTE);
    return SKIP;  // meta: allocator traffic only
}

// Scratch buffers of one op: taken from the pool in call order, given back in reverse order (api.d:78-108).
class Scratch {
public:
    explicit Scratch(int dev) : pool_(pool(dev)) {}
    ~Scratch() {
        for (int i = count_ - 1; i >= 0; i--)
            if (ptr_[i]) pool_.release(ptr_[i], size_[i]);
    }
    void* bytes(size_t n) {
        void* p = pool_.alloc(n);
        ok = ok && p != nullptr;
        ptr_[count_] = p, size_[count_++] = n;
        return p;
    }
    float* floats(int64_t n) { return static_cast<float*>(bytes((size_t)n * sizeof(float))); }
    bool ok = true;

private:
    Pool& pool_;
    void* ptr_[16];
    size_t size_[16];
    int count_ = 0;
};

constexpr int kOutOfMemory = -2;  // api.d:110

int64_t chunks_for(int64_t dim) {  // api.d:113-119: about sqrt(dim) chunks for row maxima
    int64_t c = 1;
    while (c * c < dim) c++;
    return c;
}
size_t sort_temp_bytes(int64_t n) { return (size_t)n * 16 + (size_t(1) << 20); }  // api.d:124-127
int64_t attention_tile(int64_t T) { return T % 256 == 0 ? 256 : T; }             // core/cuda/kernels.cu:612

// SOLITON_FULLSTEP_ATTN=reference: attention from the reference backend instead of this library's fused kernels
// (which follow sl_set_tf32 like the reference's: fp32-class products by default, TF32 ones when enabled).
bool fused_attention(int64_t B, int64_t T, int64_t H, int64_t hs, int64_t tile) {
    static const bool refused = [] {
        const char* v = getenv("SOLITON_FULLSTEP_ATTN");
        return v && strcmp(v, "reference") == 0;
    }();
    return !refused && sl_cuda_attention_supported(T, hs) && B * H * T <= B * H * tile * hs;
}
// SOLITON_FULLSTEP_ELT=reference: binary ops, GELU and the embedding's backward from the reference backend instead of
// this library's kernels.
bool reference_elementwise() {
    static const bool wanted = [] {
        const char* v = getenv("SOLITON_FULLSTEP_ELT");
        return v && strcmp(v, "reference") == 0;
    }();
    return wanted;
}
// SOLITON_FULLSTEP_XENT=reference: cross entropy from the reference backend instead of this library's kernels.
bool reference_xent() {
    static const bool wanted = [] {
        const char* v = getenv("SOLITON_FULLSTEP_XENT");
        return v && strcmp(v, "reference") == 0;
    }();
    return wanted;
}
}  // namespace

extern "C" {

// api.d:292-297
void sl_set_tf32(int dev, int on) {
    if (route(dev) == RUN) {
        backend().set_tf32(on);
        sl_cuda_attention_set_tf32(on);
    }
}

// api.d:335-346
void sl_binary(int dev, int op, const float* a, const float* b, float* o, int nd, const int64_t* shape, const int64_t* sa,
               const int64_t* sb) {
    if (route(dev) == RUN) (reference_elementwise() ? backend().binary : sl_cuda_binary)(op, a, b, o, nd, shape, sa, sb);
}
void sl_strided_copy(int dev, const float* src, int64_t base, float* o, int nd, const int64_t* shape, const int64_t* ss) {
    if (route(dev) == RUN) backend().strided_copy(src, base, o, nd, shape, ss);
}

// api.d:348-362: ones vector of (elements / outputs) floats
int sl_reduce_sum(int dev, const float* src, float* dst, int64_t ndst, int nd, const int64_t* shape, const int64_t* sd) {
    if (!valid_dev(dev)) return -1;
    int64_t n = 1;
    for (int d = 0; d < nd; d++) n *= shape[d];
    Scratch s(dev);
    float* ones = s.floats(n / (ndst > 0 ? ndst : 1));
    if (!s.ok) return kOutOfMemory;
    if (route(dev) == RUN) backend().reduce_sum(src, dst, ndst, nd, shape, sd, ones);
    return 0;
}

// api.d:374-377
void sl_add_scalar(int dev, float* p, int64_t n, float c) {
    if (route(dev) == RUN) backend().add_scalar(p, n, c);
}

// api.d:384-388
void sl_matmul(int dev, const float* a, const float* b, float* o, int64_t bt, int64_t n, int64_t k, int64_t m, int ta, int tb) {
    if (route(dev) == RUN) backend().matmul(a, b, o, bt, n, k, m, ta, tb);
}

// api.d:390-402: chunk maxima, row maxima, row sums, ones
int sl_softmax(int dev, const float* x, float* y, int64_t outer, int64_t dim) {
    if (!valid_dev(dev)) return -1;
    const int64_t chunks = chunks_for(dim);
    Scratch s(dev);
    float* cmax = s.floats(outer * chunks);
    float* rmax = s.floats(outer);
    float* rsum = s.floats(outer);
    float* ones = s.floats(dim);
    if (!s.ok) return kOutOfMemory;
    if (route(dev) == RUN) backend().softmax(x, y, outer, dim, chunks, cmax, rmax, rsum, ones);
    return 0;
}

// api.d:404-415: row dots, ones
int sl_softmax_bwd(int dev, const float* y, const float* dy, float* dx, int64_t outer, int64_t dim) {
    if (!valid_dev(dev)) return -1;
    Scratch s(dev);
    float* dot = s.floats(outer);
    float* ones = s.floats(dim);
    if (!s.ok) return kOutOfMemory;
    if (route(dev) == RUN) backend().softmax_bwd(y, dy, dx, outer, dim, dot, ones);
    return 0;
}

// api.d:417-425
void sl_gelu(int dev, const float* x, float* y, int64_t n) {
    if (route(dev) == RUN) (reference_elementwise() ? backend().gelu : sl_cuda_gelu)(x, y, n);
}
void sl_gelu_bwd(int dev, const float* x, const float* dy, float* dx, int64_t n) {
    if (route(dev) == RUN) (reference_elementwise() ? backend().gelu_bwd : sl_cuda_gelu_bwd)(x, dy, dx, n);
}

// SOLITON_FULLSTEP_LN=reference: layer normalisation from the reference backend instead of this library's kernels.
static bool reference_layernorm() {
    static const bool wanted = [] {
        const char* v = getenv("SOLITON_FULLSTEP_LN");
        return v && strcmp(v, "reference") == 0;
    }();
    return wanted;
}

// api.d:427-439: ones of c floats
int sl_layernorm(int dev, const float* x, const float* w, const float* b, float* y, float* mean, float* invstd,
                 int64_t outer, int64_t c, float eps) {
    if (!valid_dev(dev)) return -1;
    Scratch s(dev);
    float* ones = s.floats(c);
    if (!s.ok) return kOutOfMemory;
    if (route(dev) == RUN) {
        if (reference_layernorm())
            backend().layernorm(x, w, b, y, mean, invstd, outer, c, eps, ones);
        else
            sl_cuda_layernorm(x, w, b, y, mean, invstd, outer, c, eps, ones);
    }
    return 0;
}

// api.d:441-455: tmp (outer x c), sg, sgx (outer each), ones of c, ones of outer
int sl_layernorm_bwd(int dev, const float* dy, const float* x, const float* w, const float* mean, const float* invstd,
                     float* dx, float* dw, float* db, int64_t outer, int64_t c) {
    if (!valid_dev(dev)) return -1;
    Scratch s(dev);
    float* tmp = s.floats(outer * c);
    float* sg = s.floats(outer);
    float* sgx = s.floats(outer);
    float* ones_c = s.floats(c);
    float* ones_rows = s.floats(outer);
    if (!s.ok) return kOutOfMemory;
    if (route(dev) == RUN) {
        if (reference_layernorm())
            backend().layernorm_bwd(dy, x, w, mean, invstd, dx, dw, db, outer, c, tmp, sg, sgx, ones_c, ones_rows);
        else
            sl_cuda_layernorm_bwd(dy, x, w, mean, invstd, dx, dw, db, outer, c, tmp, sg, sgx, ones_c, ones_rows);
    }
    return 0;
}

// api.d:457-460
void sl_embedding(int dev, const float* w, const int* idx, float* o, int64_t n, int64_t c) {
    if (route(dev) == RUN) backend().embedding(w, idx, o, n, c);
}

// api.d:462-478: sort keys, permutation in and out (n ints each), sort scratch
int sl_embedding_bwd(int dev, const float* dy, const int* idx, float* dw, int64_t vocab, int64_t n, int64_t c) {
    if (!valid_dev(dev)) return -1;
    const size_t temp_bytes = sort_temp_bytes(n);
    Scratch s(dev);
    int* keys = static_cast<int*>(s.bytes((size_t)n * sizeof(int)));
    int* perm = static_cast<int*>(s.bytes((size_t)n * sizeof(int)));
    int* perm_out = static_cast<int*>(s.bytes((size_t)n * sizeof(int)));
    void* temp = s.bytes(temp_bytes);
    if (!s.ok) return kOutOfMemory;
    if (route(dev) == RUN)
        (reference_elementwise() ? backend().embedding_bwd : sl_cuda_embedding_bwd)(dy, idx, dw, vocab, n, c, keys, perm, perm_out, temp, temp_bytes);
    return 0;
}

// api.d:480-491: row losses; the mean loss comes back (NaN on meta)
double sl_cross_entropy(int dev, const float* logits, const int* t, int64_t n, int64_t v, int* err) {
    if (!valid_dev(dev)) {
        *err = -1;
        return NAN;
    }
    Scratch s(dev);
    float* rowloss = s.floats(n);
    *err = s.ok ? 0 : kOutOfMemory;
    if (!s.ok) return NAN;
    if (route(dev) != RUN) return NAN;
    return reference_xent() ? backend().cross_entropy(logits, t, n, v, rowloss) : sl_cuda_cross_entropy(logits, t, n, v, rowloss);
}

// api.d:493-499: no scratch
int sl_cross_entropy_bwd(int dev, const float* logits, const int* t, float* dl, int64_t n, int64_t v, float dloss) {
    if (route(dev) == RUN) (reference_xent() ? backend().cross_entropy_bwd : sl_cuda_cross_entropy_bwd)(logits, t, dl, n, v, dloss);
    return 0;
}

// api.d:501-519: score tile, accumulator, running max / sum / correction, row buffer, ones, pointer table
int sl_attention(int dev, const float* qkv, float* o, float* L, int64_t B, int64_t T, int64_t H, int64_t hs, float scale) {
    if (!valid_dev(dev)) return -1;
    const int64_t tile = attention_tile(T), bh = B * H, rows = bh * tile;
    Scratch s(dev);
    float* sc = s.floats(rows * tile);
    float* acc = s.floats(rows * hs);
    float* m = s.floats(rows);
    float* l = s.floats(rows);
    float* c = s.floats(rows);
    float* rowbuf = s.floats(rows * (chunks_for(tile) + 1));
    float* ones = s.floats(tile > hs ? tile : hs);
    void* ptrs = s.bytes((size_t)(5 * bh) * sizeof(void*));
    if (!s.ok) return kOutOfMemory;
    if (route(dev) == RUN)
        (fused_attention(B, T, H, hs, tile) ? sl_cuda_attention : backend().attention)(qkv, o, L, B, T, H, hs, scale, tile, sc, acc, m, l, c,
                                                                                     rowbuf, ones, ptrs);
    return 0;
}

// api.d:521-541: two score tiles, two head-size tiles, row logsumexp and D, row buffer, ones, pointer table
int sl_attention_bwd(int dev, const float* qkv, const float* o, const float* L, const float* dout, float* dqkv, int64_t B,
                     int64_t T, int64_t H, int64_t hs, float scale) {
    if (!valid_dev(dev)) return -1;
    const int64_t tile = attention_tile(T), bh = B * H, rows = bh * tile;
    Scratch s(dev);
    float* sc = s.floats(rows * tile);
    float* dp = s.floats(rows * tile);
    float* doc = s.floats(rows * hs);
    float* oc = s.floats(rows * hs);
    float* lrow = s.floats(rows);
    float* dd = s.floats(rows);
    float* rowbuf = s.floats(rows * (chunks_for(tile) + 1));
    float* ones = s.floats(tile > hs ? tile : hs);
    void* ptrs = s.bytes((size_t)(9 * bh) * sizeof(void*));
    if (!s.ok) return kOutOfMemory;
    if (route(dev) == RUN)
        (fused_attention(B, T, H, hs, tile) ? sl_cuda_attention_bwd : backend().attention_bwd)(qkv, o, L, dout, dqkv, B, T, H, hs, scale, tile,
                                                                                             sc, dp, doc, oc, lrow, dd, rowbuf, ones, ptrs);
    return 0;
}

// api.d:545-567: runtime-compiled fused elementwise kernels, cuda only
int sl_jit(int dev, const char* src, const char* name, void** handle) {
    if (dev != DEV_CUDA) return 0;
    return route(dev) == RUN ? backend().jit(src, name, handle) : -1;
}
void sl_jit_launch(int dev, void* handle, int64_t n, void** args) {
    if (dev == DEV_CUDA && route(dev) == RUN) backend().jit_launch(handle, n, args);
}
void sl_jit_free(int dev, void* handle) {
    if (dev == DEV_CUDA && backend().ok) backend().jit_free(handle);
}
const char* sl_jit_log(void) { return backend().ok ? backend().jit_log() : ""; }

// SOLITON_FULLSTEP_DP=reference: the path's entry points go to the reference's own NCCL + k_adamw instead of this
// library's kernels (see csrc/foreign_path.h). Everything else -- allocator, forward, backward -- stays as it is.
const SlbForeignPath* slb_foreign_path(void) {
    static const bool wanted = [] {
        const char* v = getenv("SOLITON_FULLSTEP_DP");
        return v && strcmp(v, "reference") == 0;
    }();
    if (!wanted) return nullptr;
    Backend& b = backend();
    return b.ok ? &b.dp : nullptr;
}

// The backend's own sticky error (core/cuda/kernels.cu:21,101-105), for the library's sl_check to fold in.
int slb_foreign_check(void) {
    Backend& b = backend();
    return b.ok ? b.check() : 0;
}

}  // extern "C"
