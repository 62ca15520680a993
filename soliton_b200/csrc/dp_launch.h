// Host-callable launchers of the kernels in dp_kernels.cu.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

#include "dp_types.h"

namespace slb {

enum KernelKind : int {
    KERNEL_PLAIN = 0,    // k_twoshot: reduce-scatter + all-gather by peer loads; with one rank the plain AdamW step
    KERNEL_ONESHOT = 1,  // k_oneshot: small steps, push to staging + local reduce
};

// Launches one kernel of the family for `world` ranks. `grid` = blocks_per_rank x (virtual ranks in this launch);
// `cooperative` asks the driver to guarantee that all blocks are resident at once (required when several virtual
// ranks, which wait on one another, share one GPU). Returns a cudaError_t value.
int launch_step(int world, bool adam, int kind, bool cooperative, int grid, size_t smem, const LaunchArgs& a, cudaStream_t st);
// Resident blocks per SM of that kernel variant.
int step_occupancy(int world, bool adam, int kind, size_t smem);
// The engine's side of an entry point that launches on its own: first everything the engine has recorded and not yet
// launched goes out (nothing happens while no device is initialised), afterwards the launch is counted.
void engine_flush_pending();
void engine_count_launch();

int launch_scale(const float* x, float* y, int64_t n, float alpha, cudaStream_t st);
int launch_axpy(const float* x, float* y, int64_t n, float alpha, cudaStream_t st);
int launch_fill(float* p, int64_t n, float value, cudaStream_t st);
// Fixed-shape sum of squares: `blocks` double partials into `partials` (block b sums a fixed contiguous slice,
// threads and warps combine in a fixed tree), so the result does not depend on scheduling.
// Sum of squares of nslices tensor slices, one double partial per slice.
int launch_sumsq_slices(int nslices, const SumsqSlice* slices, double* partials, int blocks, cudaStream_t st);
int launch_sumsq_partials(const float* x, int64_t n, double* partials, int blocks, cudaStream_t st);

}  // namespace slb
