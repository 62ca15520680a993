// Measures what the NVLink fabric of one box delivers, as the ceiling the collective kernels are judged against.
//
// One process drives all GPUs. Every receiving GPU takes `bytes` from each of its sources at the same time, by one of
//   mode 0  the copy engines (cudaMemcpyPeerAsync, one stream per pair),
//   mode 1  a kernel on the receiver that pulls with 256-bit loads (four per thread in flight) and stores locally,
//   mode 2  a kernel on the sender that loads locally and pushes with 256-bit stores,
// in one of two patterns:
//   one direction   the lower half of the GPUs receives, the upper half sends: every link carries data one way only;
//   both directions every GPU receives from every other GPU: every link carries data both ways at once, which is
//                   what an all-reduce does to it.
// Timed on the devices with events (all streams of a GPU are gated by one start event and joined into one stop
// event); the figure per GPU is bytes received (mode 0, 1) or sent (mode 2) over its own elapsed time.
#include <cuda_runtime.h>

#include <cstdint>
#include <vector>

#include "../../include/soliton_b200.h"

namespace {

constexpr int kMaxGpus = 8;
constexpr int kProbeThreads = 256;

struct alignas(32) f8 {
    float4 lo, hi;
};
__device__ __forceinline__ f8 ld8(const float* p) {
    f8 v;
    asm volatile("ld.relaxed.sys.global.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(v.lo.x), "=f"(v.lo.y), "=f"(v.lo.z), "=f"(v.lo.w), "=f"(v.hi.x), "=f"(v.hi.y), "=f"(v.hi.z), "=f"(v.hi.w)
                 : "l"(p)
                 : "memory");
    return v;
}
__device__ __forceinline__ void st8(float* p, const f8& v) {
    asm volatile("st.global.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "f"(v.lo.x), "f"(v.lo.y), "f"(v.lo.z),
                 "f"(v.lo.w), "f"(v.hi.x), "f"(v.hi.y), "f"(v.hi.z), "f"(v.hi.w)
                 : "memory");
}

struct Pairs {
    const float* src[kMaxGpus];
    float* dst[kMaxGpus];
    int n;
};

// Copies `floats` floats of every pair, the pairs interleaved tile by tile so that all of them are in flight
// together. A tile is 4 x 2048 floats: each thread issues four 32-byte loads before its first store.
__global__ void __launch_bounds__(kProbeThreads, 2) k_probe(const __grid_constant__ Pairs p, size_t floats) {
    constexpr size_t kTileFloats = 4 * 8 * kProbeThreads;
    const size_t tiles = floats / kTileFloats;
    for (size_t t = blockIdx.x; t < tiles * p.n; t += gridDim.x) {
        const int pair = (int)(t % p.n);
        const size_t off = (t / p.n) * kTileFloats + (size_t)threadIdx.x * 8;
        const float* s = p.src[pair] + off;
        float* d = p.dst[pair] + off;
        f8 v[4];
#pragma unroll
        for (int j = 0; j < 4; j++) v[j] = ld8(s + (size_t)j * 8 * kProbeThreads);
#pragma unroll
        for (int j = 0; j < 4; j++) st8(d + (size_t)j * 8 * kProbeThreads, v[j]);
    }
}

}  // namespace

extern "C" int slb_fabric_probe(int ngpus, size_t bytes, int mode, int both_directions, int repeats, double* gbs_per_gpu,
                                double* ms_per_gpu) {
    if (ngpus < 2 || ngpus > kMaxGpus || mode < 0 || mode > 2 || repeats < 1 || !gbs_per_gpu) return -1;
    int have = 0;
    if (cudaGetDeviceCount(&have) != cudaSuccess || have < ngpus) return -2;
    bytes = bytes / (4 * 8 * kProbeThreads * 4) * (4 * 8 * kProbeThreads * 4);  // whole probe tiles
    if (bytes == 0) return -1;
    int before = 0;
    cudaGetDevice(&before);

    std::vector<char*> sendbuf(ngpus, nullptr), recvbuf(ngpus, nullptr);
    std::vector<std::vector<cudaStream_t>> streams(ngpus);
    std::vector<cudaStream_t> gate(ngpus, nullptr);
    std::vector<cudaEvent_t> start(ngpus, nullptr), stop(ngpus, nullptr);
    std::vector<std::vector<cudaEvent_t>> done(ngpus);
    bool ok = true;
    for (int d = 0; d < ngpus && ok; d++) {
        ok = cudaSetDevice(d) == cudaSuccess;
        for (int q = 0; q < ngpus && ok; q++) {
            if (q == d) continue;
            int can = 0;
            ok = cudaDeviceCanAccessPeer(&can, d, q) == cudaSuccess && can;
            if (ok) {
                const cudaError_t e = cudaDeviceEnablePeerAccess(q, 0);
                if (e == cudaErrorPeerAccessAlreadyEnabled) cudaGetLastError();
                else ok = e == cudaSuccess;
            }
        }
        ok = ok && cudaMalloc((void**)&sendbuf[d], bytes * ngpus) == cudaSuccess &&
             cudaMalloc((void**)&recvbuf[d], bytes * ngpus) == cudaSuccess &&
             cudaMemset(sendbuf[d], 1, bytes * ngpus) == cudaSuccess && cudaMemset(recvbuf[d], 0, bytes * ngpus) == cudaSuccess;
        ok = ok && cudaStreamCreateWithFlags(&gate[d], cudaStreamNonBlocking) == cudaSuccess &&
             cudaEventCreate(&start[d]) == cudaSuccess && cudaEventCreate(&stop[d]) == cudaSuccess;
        streams[d].assign(ngpus, nullptr), done[d].assign(ngpus, nullptr);
        for (int q = 0; q < ngpus && ok; q++)
            ok = cudaStreamCreateWithFlags(&streams[d][q], cudaStreamNonBlocking) == cudaSuccess &&
                 cudaEventCreateWithFlags(&done[d][q], cudaEventDisableTiming) == cudaSuccess;
    }
    for (int d = 0; d < ngpus && ok; d++) ok = cudaSetDevice(d) == cudaSuccess && cudaDeviceSynchronize() == cudaSuccess;

    // who moves data to whom: active[d] lists the partners of GPU d, the GPU that issues the work
    auto receives = [&](int d) { return both_directions || d < ngpus / 2; };
    auto sends = [&](int d) { return both_directions || d >= ngpus / 2; };
    std::vector<int> issuers;
    for (int pass = 0; pass < 2 && ok; pass++) {  // pass 0 warms up (first-touch of peer mappings), pass 1 is timed
        const int reps = pass == 0 ? 1 : repeats;
        issuers.clear();
        for (int d = 0; d < ngpus && ok; d++) {
            const bool issuer = mode == 2 ? sends(d) : receives(d);
            if (!issuer) continue;
            issuers.push_back(d);
            ok = cudaSetDevice(d) == cudaSuccess && cudaEventRecord(start[d], gate[d]) == cudaSuccess;
            Pairs p{};
            for (int q = 0; q < ngpus; q++) {
                if (q == d) continue;
                if (mode == 2 ? !receives(q) : !sends(q)) continue;
                // receiver d keeps what q sent in slot q of its receive buffer; sender q reads slot d of its send buffer
                if (mode == 2) p.src[p.n] = reinterpret_cast<float*>(sendbuf[d] + bytes * q), p.dst[p.n] = reinterpret_cast<float*>(recvbuf[q] + bytes * d);
                else p.src[p.n] = reinterpret_cast<float*>(sendbuf[q] + bytes * d), p.dst[p.n] = reinterpret_cast<float*>(recvbuf[d] + bytes * q);
                p.n++;
            }
            if (mode == 0) {
                int k = 0;
                for (int q = 0; q < ngpus && ok; q++) {
                    if (q == d || !sends(q)) continue;
                    cudaStream_t s = streams[d][q];
                    ok = cudaStreamWaitEvent(s, start[d], 0) == cudaSuccess;
                    for (int r = 0; r < reps && ok; r++)
                        ok = cudaMemcpyPeerAsync(p.dst[k], d, p.src[k], q, bytes, s) == cudaSuccess;
                    ok = ok && cudaEventRecord(done[d][q], s) == cudaSuccess && cudaStreamWaitEvent(gate[d], done[d][q], 0) == cudaSuccess;
                    k++;
                }
            } else {
                int sms = 0;
                ok = ok && cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d) == cudaSuccess;
                for (int r = 0; r < reps && ok; r++) {
                    k_probe<<<2 * sms, kProbeThreads, 0, gate[d]>>>(p, bytes / 4);
                    ok = cudaPeekAtLastError() == cudaSuccess;
                }
            }
            ok = ok && cudaEventRecord(stop[d], gate[d]) == cudaSuccess;
        }
        for (int d : issuers) ok = ok && cudaSetDevice(d) == cudaSuccess && cudaDeviceSynchronize() == cudaSuccess;
    }
    for (int d = 0; d < ngpus; d++) gbs_per_gpu[d] = 0, ms_per_gpu ? ms_per_gpu[d] = 0 : 0;
    for (int d : issuers) {
        float ms = 0;
        if (!ok || cudaSetDevice(d) != cudaSuccess || cudaEventElapsedTime(&ms, start[d], stop[d]) != cudaSuccess || ms <= 0) {
            ok = false;
            break;
        }
        int partners = 0;
        for (int q = 0; q < ngpus; q++)
            if (q != d && (mode == 2 ? receives(q) : sends(q))) partners++;
        gbs_per_gpu[d] = (double)bytes * partners * repeats / (ms * 1e-3) / 1e9;
        if (ms_per_gpu) ms_per_gpu[d] = ms;
    }
    for (int d = 0; d < ngpus; d++) {
        if (cudaSetDevice(d) != cudaSuccess) continue;
        cudaDeviceSynchronize();
        if (sendbuf[d]) cudaFree(sendbuf[d]);
        if (recvbuf[d]) cudaFree(recvbuf[d]);
        for (cudaStream_t s : streams[d]) if (s) cudaStreamDestroy(s);
        for (cudaEvent_t e : done[d]) if (e) cudaEventDestroy(e);
        if (gate[d]) cudaStreamDestroy(gate[d]);
        if (start[d]) cudaEventDestroy(start[d]);
        if (stop[d]) cudaEventDestroy(stop[d]);
    }
    cudaSetDevice(before);
    cudaGetLastError();
    return ok ? 0 : -3;
}
