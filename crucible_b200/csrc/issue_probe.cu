// What it costs one thread to send work to the tensor cores and to the TMA unit on this GPU:
// two probes whose figures the tensor-core kernels' loops were shaped by (a narrow tile's step
// of K is what its MMA thread can send, not what the tensor cores or the memory can do).
//
//   cb_probe_mma_send: one thread sends `count` tcgen05.mma of M x N x 16 (bf16, operands
//     resident in shared memory, one accumulator) back to back, commits and waits; returns
//     cycles per MMA.  With `tight` the descriptors are loop-invariant registers; without, each
//     MMA computes its accumulate flag and its descriptors as a straightforward loop would.
//   cb_probe_tma_send: one thread sends `count` 2-D boxes of `rows` x 128 bytes (128-byte
//     swizzle) from a matrix in global memory to shared memory, one barrier armed once for
//     all bytes; returns cycles per box for the sending loop and until all have landed.
//   Measured on B200: 54 cycles per MMA for tiles up to 64 columns (64 at 128, 128 at 256: there
//   the tensor cores' own time), 60 cycles per box of up to 64 rows, 97 for 128 rows.
//
// One block, a few microseconds; every wait is bounded and tensor memory is freed on all
// paths (tc_common.cuh).  status: device int, stays 0 unless a wait ran out.
#include "common.cuh"
#include "tc_common.cuh"

namespace {

struct ProbeSmem {
    alignas(1024) uint8_t a[128 * 128];       // 128 rows x 64 bf16, content irrelevant
    alignas(1024) uint8_t b[256 * 128];
    alignas(1024) uint8_t ring[4][128 * 128]; // landing place of the boxes
    uint64_t bar;
    uint32_t tmem;
    int abort_flag;
};

template <int M, int N>
__global__ void __launch_bounds__(128) mma_send_kernel(int count, int tight, long long* out, int* status) {
    extern __shared__ uint8_t raw[];
    ProbeSmem& s = *reinterpret_cast<ProbeSmem*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
    const int tid = threadIdx.x;
    for (int i = tid; i < (int)sizeof(s.a) / 4; i += 128) reinterpret_cast<uint32_t*>(s.a)[i] = 0x3c003c00u;
    for (int i = tid; i < (int)sizeof(s.b) / 4; i += 128) reinterpret_cast<uint32_t*>(s.b)[i] = 0x3c003c00u;
    if (tid == 0) {
        tc::mbar_init(&s.bar, 1);
        s.abort_flag = 0;
        tc::fence_barrier_init();
    }
    tc::fence_proxy_async();
    __syncthreads();
    if (tid < 32) {
        tc::tmem_alloc(&s.tmem, 256);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem = s.tmem;
    if (tid == 0) {
        const uint64_t a0 = tc::smem_desc_sw128(tc::smem_u32(s.a)), b0 = tc::smem_desc_sw128(tc::smem_u32(s.b));
        constexpr uint32_t idesc = tc::instr_desc_bf16(M, N);
        const long long t0 = clock64();
        if (tight) {
            const uint64_t a1 = a0 + 2, a2 = a0 + 4, a3 = a0 + 6, b1 = b0 + 2, b2 = b0 + 4, b3 = b0 + 6;
            tc::umma_bf16(tmem, a0, b0, idesc, 0u);
            for (int i = 1; i < count; i += 4) {
                tc::umma_bf16_add(tmem, a1, b1, idesc);
                tc::umma_bf16_add(tmem, a2, b2, idesc);
                tc::umma_bf16_add(tmem, a3, b3, idesc);
                tc::umma_bf16_add(tmem, a0, b0, idesc);
            }
        } else {
            for (int i = 0; i < count; ++i)
                tc::umma_bf16(tmem, a0 + 2 * (i & 3), b0 + 2 * (i & 3), idesc, i > 0 ? 1u : 0u);
        }
        tc::umma_commit(&s.bar);
        const bool ok = tc::mbar_wait(&s.bar, 0, &s.abort_flag);
        const long long t1 = clock64();
        if (!ok) tc::give_up(&s.abort_flag, status, tc::ST_MMA_TIMEOUT);
        out[0] = t1 - t0;
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (tid < 32) {
        tc::tc_fence_after_sync();
        tc::tmem_dealloc(tmem, 256);
    }
}

template <int ROWS>
__global__ void __launch_bounds__(128) tma_send_kernel(const __grid_constant__ CUtensorMap map, int count,
                                                       int k_cols, long long* out, int* status) {
    extern __shared__ uint8_t raw[];
    ProbeSmem& s = *reinterpret_cast<ProbeSmem*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~uintptr_t(1023));
    if (threadIdx.x == 0) {
        tc::mbar_init(&s.bar, 1);
        s.abort_flag = 0;
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&map);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        tc::mbar_expect_tx(&s.bar, (uint32_t)count * ROWS * 128);
        int x = 0;
        const long long t0 = clock64();
        for (int i = 0; i < count; ++i) {
            tc::tma_load_2d(s.ring[i & 3], &map, &s.bar, x, 0);
            x += 64;
            if (x + 64 > k_cols) x = 0;
        }
        const long long t1 = clock64();
        const bool ok = tc::mbar_wait(&s.bar, 0, &s.abort_flag);
        const long long t2 = clock64();
        if (!ok) tc::give_up(&s.abort_flag, status, tc::ST_PRODUCER_TIMEOUT);
        out[0] = t1 - t0;
        out[1] = t2 - t0;
    }
}

}  // namespace

// out: one device int64 (cycles for all `count` MMAs, commit and wait included).
// m: 64 or 128; n: 64, 128 or 256; count: 1 + a multiple of 4, at most 4097.
CB_EXPORT int cb_probe_mma_send(int m, int n, int count, int tight, long long* out, int* status, void* stream) {
    if (count < 1 || count > 4097 || (count - 1) % 4) return CB_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    const int smem = (int)sizeof(ProbeSmem) + 1024;
#define CB_PROBE_CASE(MM, NN)                                                                              \
    if (m == MM && n == NN) {                                                                              \
        cudaError_t e = cudaFuncSetAttribute(mma_send_kernel<MM, NN>,                                      \
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);           \
        if (e != cudaSuccess) return (int)e;                                                               \
        mma_send_kernel<MM, NN><<<1, 128, smem, st>>>(count, tight, out, status);                          \
        return cb_last_error();                                                                            \
    }
    CB_PROBE_CASE(128, 64)
    CB_PROBE_CASE(128, 128)
    CB_PROBE_CASE(128, 256)
    CB_PROBE_CASE(64, 64)
#undef CB_PROBE_CASE
    return CB_ERR_UNSUPPORTED;
}

// matrix: bf16 [rows_total, k_cols] row-major in device memory, k_cols a multiple of 64, at
// least 128 rows.  rows: 16, 64 or 128 (the box's height); count * rows * 128 < 2^20.
// out: two device int64: cycles of the sending loop, cycles until every box has landed.
CB_EXPORT int cb_probe_tma_send(const void* matrix, int rows_total, int k_cols, int rows, int count,
                                long long* out, int* status, void* stream) {
    if (count < 1 || (long long)count * rows * 128 >= (1 << 20) || k_cols < 64 || (k_cols & 63) || rows_total < 128 ||
        ((uintptr_t)matrix & 15))
        return CB_ERR_UNSUPPORTED;
    CUtensorMap map;
    if (!tc::make_map_2d(&map, matrix, (uint64_t)rows_total, (uint64_t)k_cols, (uint64_t)k_cols, (uint32_t)rows))
        return CB_ERR_UNSUPPORTED;
    cudaStream_t st = (cudaStream_t)stream;
    const int smem = (int)sizeof(ProbeSmem) + 1024;
#define CB_PROBE_CASE(RR)                                                                                  \
    if (rows == RR) {                                                                                      \
        cudaError_t e = cudaFuncSetAttribute(tma_send_kernel<RR>,                                          \
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);           \
        if (e != cudaSuccess) return (int)e;                                                               \
        tma_send_kernel<RR><<<1, 128, smem, st>>>(map, count, k_cols, out, status);                        \
        return cb_last_error();                                                                            \
    }
    CB_PROBE_CASE(16)
    CB_PROBE_CASE(64)
    CB_PROBE_CASE(128)
#undef CB_PROBE_CASE
    return CB_ERR_UNSUPPORTED;
}
