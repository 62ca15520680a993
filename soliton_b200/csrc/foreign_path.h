// A second implementation of the path's entry points, selectable at run time by a build that links one in.
//
// The product library defines none: slb_foreign_path is a weak symbol that stays null, and every entry point runs this
// library's own code. The build that serves whole Soliton training steps (fullstep/) defines it so that the same
// process can also be run on the REFERENCE's own data-parallel path -- ncclAllReduce(avg) and k_adamw from
// core/cuda/kernels.cu -- for comparisons: same caller, same allocator, same forward and backward; only the path
// differs.
#pragma once
#include <cstdint>

extern "C" {
struct SlbForeignPath {
    void (*adamw)(float* p, const float* g, float* m, float* v, int64_t n, float lr, float b1, float b2, float eps, float wd, int step);
    int (*dist_unique_id)(char* out128);
    int (*dist_init)(int rank, int world, const char* id128);
    int (*dist_group)(int start);
    int (*dist_allreduce_mean)(float* p, int64_t n);
    void (*dist_destroy)(void);
    double (*sumsq)(const float* x, int64_t n);
    void (*scale)(const float* x, float* y, int64_t n, float alpha);
    void (*axpy)(const float* x, float* y, int64_t n, float alpha);
};
// Null, or the implementation to use instead of this library's for the calls above (cuda device only).
const SlbForeignPath* slb_foreign_path(void) __attribute__((weak));
}
