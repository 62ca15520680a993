/*
 * soliton_b200 -- C ABI of libsoliton_b200.so
 *
 * A B200-native replacement for one path of Soliton (vishesh9131/soliton): the data-parallel gradient mean
 * (NCCL ncclAvg in the reference), the 1/world scaling and the AdamW update, fused into one family of sm_100a
 * kernels that exchange gradients through NVSwitch peer loads and stores.
 *
 * Three groups of entry points:
 *   1. `sl_*`       -- the functions Soliton's Python binds through ctypes (python/soliton/_C.py:11-67) that lie on
 *                      the path or that the path's callers need around it (allocator, device, data movement).
 *                      Same names, argument meaning, return codes and error channel as core/soliton/api.d.
 *   2. `sl_cuda_*`  -- the backend functions Soliton's D core declares (core/soliton/api.d:10-65) and its CUDA file
 *                      defines for this path. A Soliton build links these in place of the originals.
 *   3. `slb_*`      -- additions without a counterpart in the reference (options, counters, test hooks).
 *
 * Conventions (core/soliton/alloc.d:12, python/soliton/tensor.py:22-23): dev 0 = cpu, 1 = meta, 2 = cuda.
 * On meta every function does the same allocator traffic as on cuda and no device work. Compute entry points
 * called with dev = 0 set sticky error 13: this library has no host kernels. All device work is enqueued on the
 * legacy default stream, as in the reference; nothing throws; one thread per process.
 * Sticky error codes read by sl_check: 1..11 as in core/cuda/kernels.cu:21-34,101-108 (2 launch, 3 sync);
 * 12 bad argument, 13 compute on cpu, 14 device not initialised through sl_init_device,
 * 21/22/23 a bounded device-side wait on a peer rank ran out (start / reduced / done barrier).
 */
#ifndef SOLITON_B200_H
#define SOLITON_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ 1. sl_*: memory (the allocator contract) */

/* core/soliton/api.d:133-136 (Pool.alloc, core/soliton/alloc.d:128-174). NULL when out of memory / diverged. */
void* sl_alloc(int dev, size_t n);
/* core/soliton/api.d:138-141 (Pool.release, alloc.d:176-200). n is the unrounded size given to sl_alloc. */
void sl_free(int dev, void* p, size_t n);
/* core/soliton/api.d:144-154. out: allocated, reserved, peak_allocated, peak_reserved, n_alloc, n_raw, trace_hash */
void sl_stats(int dev, int64_t* out7);
/* core/soliton/api.d:156-164 */
void sl_reset_stats(int dev);
/* core/soliton/api.d:165-168 */
void sl_empty_cache(int dev);
/* core/soliton/api.d:256-260. 0 = unlimited. */
void sl_set_limit(int dev, int64_t bytes);
/* core/soliton/api.d:172-215: trace recording for the arena planner */
void sl_record_start(int dev);
void sl_record_stop(int dev);
void sl_record_mark(int dev);
int64_t sl_record_count(int dev);
int64_t sl_record_body(int dev);
void sl_record_get(int dev, int64_t* size, int64_t* start, int64_t* end);
/* core/soliton/api.d:217-238. The two arrays stay owned by the caller and must outlive the install. 0 or -2. */
int sl_arena_install(int dev, const int64_t* offsets, const int64_t* sizes, int64_t count, int64_t body,
                     int64_t arena_bytes);
/* core/soliton/api.d:241-244 */
int sl_arena_diverged(int dev);
/* core/soliton/api.d:246-254 */
void sl_arena_off(int dev);

/* ------------------------------------------------------------------ sl_*: device */

/* core/soliton/api.d:262-274. cpu: 0. meta and cuda: reserves, from the pool, the reference's 32 MiB BLAS
 * workspace and then this library's 18 MiB data-parallel workspace (flag words, segment tables, one-shot
 * staging) -- the only scratch the path ever uses, taken once and in this fixed order on both devices, so a meta
 * dry run predicts the cuda pool exactly. 0, -1 (no such device) or -2 (out of memory). */
int sl_init_device(int dev, int ordinal);
/* core/soliton/api.d:276-279 */
int sl_cuda_count(void);
/* core/soliton/api.d:281-284. Sticky error code, 0 when none. */
int sl_check(int dev);
/* core/soliton/api.d:286-290. Launches whatever step is pending, then waits for the device. */
void sl_sync(int dev);
/* core/soliton/api.d:299-302 */
void sl_mem_info(size_t* free_bytes, size_t* total_bytes);

/* ------------------------------------------------------------------ sl_*: data movement (blocking, as the reference) */

/* core/soliton/api.d:313-326 */
void sl_from_host(int dev, void* dst, const void* src, size_t n);
void sl_to_host(int dev, void* dst, const void* src, size_t n);
void sl_copy(int dev, void* dst, const void* src, size_t n);
/* core/soliton/api.d:330-333 */
void sl_fill(int dev, float* p, int64_t n, float v);

/* ------------------------------------------------------------------ sl_*: the path */

/* core/soliton/api.d:539-543 -> core/cuda/kernels.cu:242-254. One AdamW update of p, m, v (n floats each) with
 * gradient g. On cuda the call is recorded and launched together with its neighbours (see sl_dist_group). */
void sl_adamw(int dev, float* p, const float* g, float* m, float* v, int64_t n, float lr, float b1, float b2,
              float eps, float wd, int step);
/* core/soliton/api.d:572-575 -> core/cuda/kernels.cu:761-766. Rank 0: fills 128 bytes that name the group. */
int sl_dist_unique_id(char* out128);
/* core/soliton/api.d:577-580 -> core/cuda/kernels.cu:767-771. After sl_init_device(2, ordinal). 0 or -1. */
int sl_dist_init(int rank, int world, const char* id128);
/* core/soliton/api.d:582-585 -> core/cuda/kernels.cu:772. start=1 opens a group, start=0 closes it; closing
 * meets the peers on the host (bounded) and arms one fused launch for all gradients of the group. 0 or -1. */
int sl_dist_group(int dev, int start);
/* core/soliton/api.d:587-590 -> core/cuda/kernels.cu:773-775. In place mean over ranks of n floats at p. 0 or -1. */
int sl_dist_allreduce_mean(int dev, float* p, int64_t n);
/* core/soliton/api.d:592-595 -> core/cuda/kernels.cu:776-779 */
void sl_dist_destroy(void);

/* ------------------------------------------------------------------ sl_*: next to the path (gradient clipping, accumulation) */

/* core/soliton/api.d:364-372 (python/soliton/optim.py:31-39 uses sumsq + scale; tensor.py:451-462 uses axpy) */
void sl_axpy(int dev, const float* x, float* y, int64_t n, float alpha);
void sl_scale(int dev, const float* x, float* y, int64_t n, float alpha);
/* core/soliton/api.d:379-382. Blocking. NaN on meta. */
double sl_sumsq(int dev, const float* x, int64_t n);

/* ------------------------------------------------------------------ 2. sl_cuda_*: backend level */

/* core/soliton/api.d:47-48 -> core/cuda/kernels.cu:251-254 */
void sl_cuda_adamw(float* p, const float* g, float* m, float* v, int64_t n, float lr, float b1, float b2, float eps,
                   float wd, int step);
/* core/soliton/api.d:58-62 -> core/cuda/kernels.cu:761-779 */
int sl_cuda_nccl_unique_id(char* out128);
int sl_cuda_nccl_init(int rank, int world, const char* id128);
int sl_cuda_nccl_group(int start);
int sl_cuda_nccl_allreduce_mean(float* p, int64_t n);
void sl_cuda_nccl_destroy(void);
/* core/soliton/api.d:26-29 -> core/cuda/kernels.cu:200,212,219-224: the small ops the trainer runs between the
 * gradient mean and the step (gradient accumulation, clipping). Linking these as well lets the clip ride along with
 * the path: the sums of squares come out of the gradient mean's launch, in-place scales are applied by the AdamW
 * launch. sl_cuda_sumsq blocks, like the reference's. */
void sl_cuda_axpy(const float* x, float* y, int64_t n, float alpha);
void sl_cuda_scale(const float* x, float* y, int64_t n, float alpha);
double sl_cuda_sumsq(const float* x, int64_t n);
/* core/soliton/api.d:37-41 -> core/cuda/kernels.cu:409-449: layer normalisation over rows of c floats, forward
 * (y, and the row's mean and 1/std for the backward pass) and backward (dx, and dw, db summed over the rows). One pass
 * over the activations in each direction. The scratch pointers are the ones the reference's host core passes: only
 * `tmp` (outer x c floats) is used, for the per-block column sums; `ones`, `sg`, `sgx`, `ones_c`, `ones_rows` may be
 * NULL. Asynchronous on the legacy stream; a launch failure sets the sticky error 2. */
void sl_cuda_layernorm(const float* x, const float* w, const float* b, float* y, float* mean, float* invstd, int64_t outer,
                       int64_t c, float eps, float* ones);
void sl_cuda_layernorm_bwd(const float* dy, const float* x, const float* w, const float* mean, const float* invstd,
                           float* dx, float* dw, float* db, int64_t outer, int64_t c, float* tmp, float* sg, float* sgx,
                           float* ones_c, float* ones_rows);
/* core/soliton/api.d:51-55 -> core/cuda/kernels.cu:536-692: causal attention over packed qkv (B, T, 3, H, hs) -> out
 * (B, T, H, hs) and L (B, H, T) = row maximum + log of the softmax denominator; backward writes all of dqkv. Fused
 * kernels that keep scores and probabilities on chip; products on the tensor cores with fp32 accumulation. Like the
 * reference's matmuls they have two precisions: fp32-class by default (every operand split into two TF32 pieces,
 * three products each), plain TF32 operands after sl_cuda_attention_set_tf32(1) -- call it wherever
 * sl_cuda_set_tf32 (core/cuda/kernels.cu:117-122) is called. Only hs = 64 and T a multiple of 64
 * (sl_cuda_attention_supported); other shapes set the sticky error 2 and do nothing. Of the reference's scratch
 * arguments only `oc` is used (backward: B * H * T floats of row dots; the reference sizes it B * H * tile * hs); the
 * others may be NULL. Results do not vary from run to run: no atomics, one fixed summation order. */
void sl_cuda_attention_set_tf32(int on);
int sl_cuda_attention_supported(int64_t T, int64_t hs);
void sl_cuda_attention(const float* qkv, float* out, float* L, int64_t B, int64_t T, int64_t H, int64_t hs, float scale,
                       int64_t tile, float* s, float* acc, float* m, float* l, float* c, float* rowbuf, float* ones, void* ptrs);
void sl_cuda_attention_bwd(const float* qkv, const float* out, const float* L, const float* dout, float* dqkv, int64_t B,
                           int64_t T, int64_t H, int64_t hs, float scale, int64_t tile, float* s, float* dp, float* doc,
                           float* oc, float* lrow, float* D, float* rowbuf, float* ones, void* ptrs);
/* core/soliton/api.d:46-47 -> core/cuda/kernels.cu:488-534: cross entropy of n rows of v logits against integer
 * targets: the mean loss (blocking: the value comes back to the host), and the gradient dl = (softmax - onehot) *
 * dloss / n. One pass over the logits forward, one read and one write backward. `rowloss` (n floats) is the
 * reference's scratch; when it is 8-byte aligned the mean is formed on the device in double precision and
 * overwrites its first 8 bytes. */
double sl_cuda_cross_entropy(const float* logits, const int* t, int64_t n, int64_t v, float* rowloss);
void sl_cuda_cross_entropy_bwd(const float* logits, const int* t, float* dl, int64_t n, int64_t v, float dloss);
/* core/soliton/api.d:23-24,44-45 -> core/cuda/kernels.cu:139-181,459-487: out = a op b (op 0 add, 1 subtract,
 * 2 multiply, 3 divide) over an output of up to 8 dimensions, the inputs given by their strides in elements (0 where
 * they broadcast); and the embedding's backward: dw (vocab x c) = for every id the sum of the rows of dy (n x c)
 * whose token has that id, rows added in token order. `keys`, `perm`, `perm_out` (n ints each) and `temp`
 * (sl_cuda_sort_temp_bytes(n) bytes at the least, else sticky error 8) are the caller's scratch. Both give the
 * reference's bits. */
void sl_cuda_binary(int op, const float* a, const float* b, float* o, int nd, const int64_t* shape, const int64_t* sa,
                    const int64_t* sb);
size_t sl_cuda_sort_temp_bytes(int64_t n);
/* Host only, for tests: which kernel sl_cuda_binary picks (2 = 128-bit suffix, 1 = element-wise suffix, 0 = general
 * strides, -1 = refused) and, in out[0..1], how many elements of a and of b repeat (-1: not a repeating suffix). The
 * classification is the reference's suffix_numel (core/cuda/kernels.cu:154-169). */
int slb_binary_plan(int nd, const int64_t* shape, const int64_t* sa, const int64_t* sb, int64_t* out);
/* core/soliton/api.d:36-37 -> core/cuda/kernels.cu:226-240: y = x * Phi(x) (the exact GELU, through erf) and its
 * backward dx = dy * (Phi(x) + x * phi(x)), four elements per thread; the reference's bits. */
void sl_cuda_gelu(const float* x, float* y, int64_t n);
void sl_cuda_gelu_bwd(const float* x, const float* dy, float* dx, int64_t n);
void sl_cuda_embedding_bwd(const float* dy, const int* idx, float* dw, int64_t vocab, int64_t n, int64_t c, int* keys, int* perm,
                           int* perm_out, void* temp, size_t temp_bytes);
/* No counterpart in the reference; modelled on sl_cuda_set_workspace (core/cuda/kernels.cu:115). A host core that
 * owns the allocator hands the path its workspace (slb_workspace_bytes() bytes from its pool) once per device. */
int sl_cuda_dp_set_workspace(void* p, size_t n);

/* ------------------------------------------------------------------ 3. slb_*: no counterpart in the reference */

size_t slb_workspace_bytes(void);
/* Options: "eager" (0/1: launch at every call instead of deferring -- with it a Soliton build needs no slb_flush
 * hooks at all), "mode" (0 auto, 1 one-shot, 2 two-shot), "blocks_per_sm", "cyclic" (single-rank steps: blocks take
 * groups of this many tiles round robin; 0 = one contiguous run per block; default 4), "stamps" (collective launches
 * record device times at their phase borders, see slb_read_stamps), "overlap" (1: the path's launches go to a stream
 * of their own beside the legacy stream, ordered against it by events; default 0), "timeout_ms" (device waits),
 * "host_timeout_ms", "oneshot_max_bytes" (-1: whatever fits the staging slots). Must be set alike on all ranks.
 * Returns 0, or -1 for an unknown name. */
int slb_set_option(const char* name, int64_t value);
/* Counters: "launches" (kernels of this library launched so far), "last_mode" (0 local, 1 one-shot, 2 two-shot),
 * "last_blocks", "world", "sm_count", "pending_frees" (exported allocations this rank has released and still holds
 * until every peer has closed its mapping). -1 for an unknown name. */
int64_t slb_get_counter(const char* name);
/* Launches whatever step is pending without waiting for the device (sl_sync does the same and then waits). */
void slb_flush(void);
/* Copies beside the path, for callers that feed the step bucket by bucket (python/soliton/tensor.py:427-471 makes
 * gradients final in reverse layer order): k buffers per call between PINNED host memory and device memory, on
 * streams of their own (one per direction). Ordering is by address: an upload waits for launched work that still
 * reads or writes its destination, a launch waits for uploads into its tensors and for downloads that still read
 * them, a download waits for the launch that writes its source. Blocking entry points (sl_to_host, sl_sync, ...)
 * wait as well. slb_wait_copies blocks the host until both copy streams are idle. 0 or -1. */
int slb_from_host_async(int k, void* const* dst, const void* const* src, const size_t* bytes);
int slb_to_host_async(int k, void* const* dst, const void* const* src, const size_t* bytes);
int slb_wait_copies(void);
/* With option "stamps": device times (globaltimer, ns) that block 0 of the last collective launch took at its phase
 * borders: start, every peer present, own chunk reduced, all chunks gathered, every peer done. Waits for the
 * device. 0 or -1. */
int slb_read_stamps(uint64_t* out5);
/* Clears the sticky error (after a test provoked one on purpose). */
void slb_clear_error(void);
/* The partition the kernels use: tiles of the step, and the tile range [*begin, *end) that block `block` of
 * `blocks` works on inside chunk `chunk` of `world` (chunk = -1: inside the whole sequence). */
int64_t slb_tile_count(const int64_t* n, int nseg);
void slb_run_range(int64_t tiles, int world, int chunk, int blocks, int block, int64_t* begin, int64_t* end);
/* No counterpart in the reference. The fused multi-tensor AdamW step of sl_adamw for callers that must not see this
 * library allocate device memory and have given it no workspace -- a host core that owns and plans the whole device
 * heap, as Soliton's does. The segment table lives in a fixed 59,904-byte device array inside the library image, so
 * at most 512 tensors per call; the call makes no cudaMalloc / cudaFree. Arrays are host arrays of nseg entries
 * (device pointers, element counts, per-tensor weight decay; wd may be NULL for none). Work goes to the legacy
 * default stream. The first call on a device looks up the array's address: make it outside stream capture. All calls
 * share the array; calls whose kernels could overlap on the GPU race. 0 ok, -1 bad argument, -2 more than 512
 * tensors, -3 a CUDA call failed. */
int slb_adamw_step_static(int nseg, float* const* p, const float* const* g, float* const* m, float* const* v,
                          const int64_t* n, const float* wd, float lr, float b1, float b2, float eps, int step);
/* Test hook: `world` ranks emulated on one GPU by one cooperative launch (blocks of all ranks resident together).
 * Pointer arrays are indexed [rank * nseg + segment]; p/m/v may be NULL when adam = 0. mode: 0 auto, 1 one-shot,
 * 2 two-shot. active_mask: bit r set = rank r takes part (a missing rank makes the others' waits run out).
 * status_out[world] receives each rank's device status (0, or 21/22/23). sumsq_out (NULL, or world x nseg doubles;
 * two-shot without an optimizer only): per rank and tensor, the sum of squares of the mean as the launch's piece
 * table on that rank gives it. Returns 0 or a negative code. */
int slb_sim_step(int world, int nseg, const int64_t* n, float* const* p, float* const* g, float* const* m,
                 float* const* v, const float* wd, float lr, float b1, float b2, float eps, int step, int adam,
                 int mode, int blocks_per_rank, int64_t timeout_ms, unsigned active_mask, int* status_out,
                 double* sumsq_out);
/* Test hook: runs the host rendezvous protocol (no CUDA) as rank `rank` of `world` for `rounds` collectives with
 * synthetic tables and checks what it reads from the peers. 0 when everything matched. */
int slb_rdv_selftest(const char* id128, int rank, int world, int rounds);
int slb_rdv_create_id(char* out128);
/* Test hook: the life cycle of export slots (published, freed by the owner, let go by every peer, reused) driven
 * by `world` processes without CUDA, `cycles` x `per_cycle` fake allocations per rank. 0 when everything matched
 * and no more than per_cycle slots were ever in use. */
int slb_rdv_slot_selftest(const char* id128, int rank, int world, int cycles, int per_cycle);
/* Measurement, no counterpart in the reference: what the NVLink fabric of this box delivers when `ngpus` GPUs move
 * `bytes` per pair at once, driven from this one process. mode 0: copy engines (cudaMemcpyPeerAsync); 1: a kernel on
 * the receiver pulling with 256-bit loads; 2: a kernel on the sender pushing with 256-bit stores. both_directions 0:
 * the lower half of the GPUs receives from the upper half (every link one way only); 1: every GPU exchanges with
 * every other (every link both ways at once, as in an all-reduce). gbs_per_gpu[ngpus] (and ms_per_gpu, may be NULL)
 * receive, for every GPU that issued work, GB/s received (modes 0, 1) or sent (mode 2) and its device time.
 * 0, -1 bad argument, -2 fewer GPUs than asked, -3 a CUDA call failed or peer access is not available. */
int slb_fabric_probe(int ngpus, size_t bytes, int mode, int both_directions, int repeats, double* gbs_per_gpu,
                     double* ms_per_gpu);
/* PCI address of a device ("0000:1b:00.0"), for callers that want to place their host buffers on the NUMA node the
 * GPU hangs on (/sys/bus/pci/devices/<address>/numa_node). 0 or -1. */
int slb_device_pci_bus_id(int ordinal, char* out, int len);
/* Page-locked host memory for slb_from_host_async / slb_to_host_async (cudaHostAlloc). NULL on failure. */
void* slb_pinned_alloc(size_t n);
/* The same, write-combined: for buffers the host only ever writes (upload sources); reading them on the host is slow. */
void* slb_pinned_alloc_wc(size_t n);
void slb_pinned_free(void* p);

#ifdef __cplusplus
}
#endif
#endif /* SOLITON_B200_H */
