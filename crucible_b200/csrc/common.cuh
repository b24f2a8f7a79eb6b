// Shared helpers for the kernels of this package: element conversion between
// float and bfloat16, reductions, and the launch-status convention.  Every
// exported launcher returns a cudaError_t as int (0 = success) and never
// synchronises; the caller passes the stream to launch on.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define CB_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes shared with the Python wrappers
#define CB_F32 0
#define CB_BF16 1

// launcher-level refusals (not CUDA errors); Python turns them into messages
#define CB_ERR_UNSUPPORTED 100001

__device__ __forceinline__ float cb_to_float(float v) { return v; }
__device__ __forceinline__ float cb_to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T cb_from_float(float v);
template <> __device__ __forceinline__ float cb_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 cb_from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float cb_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float cb_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; `scratch` holds 32 floats.  The
// order of the additions is fixed by the block size alone.
__device__ __forceinline__ float cb_block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = cb_warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    const int nwarps = (blockDim.x + 31) >> 5;
    float total = 0.f;
    for (int w = 0; w < nwarps; ++w) total += scratch[w];
    return total;
}

// The first launch failure since the last call (launches record it), else the
// runtime's last error.
static thread_local int cb_launch_failure = 0;
static inline int cb_last_error() {
    const int rc = cb_launch_failure;
    cb_launch_failure = 0;
    return rc ? rc : (int)cudaGetLastError();
}

// ---- programmatic dependent launch ------------------------------------------------
// Every kernel of this package is launched with the programmatic-stream-
// serialization attribute: it may become resident while the kernel before it in
// the stream is still running, and must call cb_pdl_wait() before it reads
// anything an earlier kernel wrote (the wait returns once all earlier kernels
// have completed and their writes are visible).  What a kernel does before the
// wait -- index arithmetic, barrier and tensor-memory set-up, loads of weights,
// which no kernel writes -- overlaps the tail of its predecessor.  Each kernel
// calls cb_pdl_trigger() so that its successor may be scheduled early: kernels that hold
// tensor memory only after they have allocated it and passed their own wait (a successor
// that started earlier could take the tensor memory of an SM first and then wait for this
// kernel, which waits for that tensor memory), the others at their start or once their own
// loads are on their way.  Which kernels get the attribute was measured on B200 inside captured graphs,
// source file by source file (CB_PDL_BIT, defined before this header is included, is the
// file's bit): the tensor-core products for more than 32 rows gain most (their barriers,
// tensor memory and descriptors are set up under the kernel before: 1.09 -> 1.02 ms per
// 2,048-token prefill, 0.93 -> 0.88 ms per batch-64 decode step); the prompt attention a
// little; the split decode attention gains once it lets its own successor start only after
// its query rows are staged (0.42 -> 0.41 ms at batch 8, 0.85 -> 0.84 ms at batch 64); norms and the like gain in small
// launches and lose in large ones (CB_PDL_MAX_BLOCKS); the few-row products lose if they
// let their successor start at once (0.41 -> 0.44 ms: its loads of weights get in the way of
// the loads this kernel waits for) and gain if they do so once their own rows are staged
// (0.41 -> 0.385 ms at batch 8, 0.37 -> 0.35 ms at batch 1), for up to 16 rows.  Hence the
// default below.  CRUCIBLE_PDL in the environment overrides it: a
// number is taken as the files' bits, "all" sets every bit.  Without the attribute the
// two device calls are no-ops.
__device__ __forceinline__ void cb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void cb_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

#include <cstdlib>
#include <cstring>
#include <utility>
#ifndef CB_PDL_BIT
#define CB_PDL_BIT 31
#endif
#ifndef CB_PDL_MAX_BLOCKS
#define CB_PDL_MAX_BLOCKS 0          // 0: launches of any size
#endif
// bits: 0 gemm_tcgen05, 1 attention_tcgen05, 2 attention_decode_tcgen05, 3 elementwise, 4 decode_small,
// 5 gemm_skinny_tcgen05
#define CB_PDL_DEFAULT_MASK 0x3Ful
static inline bool cb_pdl_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("CRUCIBLE_PDL");
        unsigned long mask = CB_PDL_DEFAULT_MASK;
        if (v && std::strcmp(v, "all") == 0) mask = ~0ul;
        else if (v && v[0]) mask = std::strtoul(v, nullptr, 0);
        return ((mask >> CB_PDL_BIT) & 1ul) != 0;
    }();
    return on;
}

// cluster_z > 1: the blocks (x, y, 0..cluster_z-1) form a thread-block cluster.
// allow_early: the launcher's own word on the programmatic launch (false: never).
template <typename... KArgs, typename... Args>
static inline int cb_launch_ex(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                               cudaStream_t stream, int cluster_z, bool allow_early, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    const size_t blocks = (size_t)grid.x * grid.y * grid.z;
    if (allow_early && cb_pdl_enabled() && (CB_PDL_MAX_BLOCKS == 0 || blocks <= CB_PDL_MAX_BLOCKS)) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_z > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = 1;
        attr[n].val.clusterDim.y = 1;
        attr[n].val.clusterDim.z = (unsigned)cluster_z;
        ++n;
    }
    cfg.attrs = attr;
    cfg.numAttrs = n;
    const int rc = (int)cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
    if (rc != 0 && cb_launch_failure == 0) cb_launch_failure = rc;
    return rc;
}

template <typename... KArgs, typename... Args>
static inline int cb_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                    cudaStream_t stream, int cluster_z, Args&&... args) {
    return cb_launch_ex(kernel, grid, block, smem, stream, cluster_z, true, std::forward<Args>(args)...);
}

template <typename... KArgs, typename... Args>
static inline int cb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                            cudaStream_t stream, Args&&... args) {
    return cb_launch_ex(kernel, grid, block, smem, stream, 1, true, std::forward<Args>(args)...);
}
