// Building blocks for the sm_100a tensor-core kernels: mbarrier waits with an
// iteration limit, TMA tile loads, tcgen05 (5th-generation tensor core)
// descriptors, MMA issue, commit, and tensor-memory loads, as inline PTX; and
// the host-side encoder of TMA tensor maps.
//
// Waiting discipline: no wait in these kernels is unbounded.  A wait that runs
// out records a code in the kernel's status word, raises the block's abort
// flag, and every role leaves its loop; the block then waits (bounded) for its
// own copies in flight, frees its tensor memory and returns.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tc {

constexpr uint32_t WAIT_LIMIT = 1u << 22;

// status codes written to the status word (0 = fine)
constexpr int ST_PRODUCER_TIMEOUT = 1;
constexpr int ST_MMA_TIMEOUT = 2;
constexpr int ST_EPILOGUE_TIMEOUT = 3;
constexpr int ST_PROBE_TIMEOUT = 4;     // the wait probe of the tests (see cb_tc_wait_probe)

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Whether the barrier's phase of that parity is over; never suspends the thread (try_wait
// may, for a time of the hardware's choosing: wrong for a thread that polls several barriers).
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false if the limit ran out or the block is aborting.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          uint32_t limit = WAIT_LIMIT) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    return false;
}

// The same on a barrier given by its shared-memory address (for loops that reach a
// stage's barrier as a constant offset from the first).
__device__ __forceinline__ bool mbar_try_wait_at(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool mbar_wait_at(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                             uint32_t limit = WAIT_LIMIT) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait_at(bar, parity)) return true;
        if ((i & 1023u) == 1023u && *abort_flag) return false;
    }
    return false;
}

__device__ __forceinline__ void give_up(volatile int* abort_flag, int* status, int code) {
    *abort_flag = 1;
    if (status) atomicCAS(status, 0, code);
}

// 2-D tiled TMA load global -> shared, completion on an mbarrier.  x is the
// innermost (contiguous) coordinate; x * element size must be a multiple of 16.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar,
                                            int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"((uint64_t)map), "r"(smem_u32(bar)), "r"(c0), "r"(c1),
        "r"(c2), "r"(c3)
        : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"((uint64_t)map) : "memory");
}

// ---- tensor memory -----------------------------------------------------------

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(smem_result)),
                 "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// Shared-memory operand descriptor for a K-major tile whose rows are 128 bytes
// (64 bf16) with the 128-byte swizzle, as TMA writes it: rows 128 B apart,
// groups of 8 rows 1024 B apart; the tile base must be 1024-byte aligned.
// Bits: [0,14) address >> 4; [16,30) leading byte offset >> 4 (1: unused for
// swizzled K-major); [32,46) stride byte offset >> 4 (64 = 1024 B);
// [46,48) version 1 (sm_100); [61,64) layout 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)64 << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// Instruction descriptor for kind::f16 with bf16 A and B (both K-major) and an
// fp32 accumulator: [4,6) D format 1 = f32; [7,10) A format 1 = bf16; [10,13)
// B format 1 = bf16; bit 15 / 16 A / B major 0 = K; [17,23) N >> 3; [24,29) M >> 4.
__host__ __device__ constexpr uint32_t instr_desc_bf16(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) |
           ((uint32_t)(m >> 4) << 24);
}

// The same with B stored MN-major (its N index contiguous in shared memory, as a
// [keys, head_dim] tile of values is for P . V): bit 16 set.
__host__ __device__ constexpr uint32_t instr_desc_bf16_b_mn(int m, int n) {
    return instr_desc_bf16(m, n) | (1u << 16);
}

// D[tmem] (+)= A[smem] * B[smem]^T; issued by one thread.
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                          uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// The same, always accumulating: no predicate to compute.
__device__ __forceinline__ void umma_bf16_add(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                              uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.eq.b32 p, 1, 1;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc)
        : "memory");
}

// An operand descriptor from its two words: the low one carries the tile's address (in
// 16-byte units, so a tile 16 * n bytes further is the low word + n, as long as the sum
// stays below the 14 bits of the field, which every shared-memory address does), the high
// one is the same for all tiles of one layout.
__device__ __forceinline__ uint64_t desc_of(uint32_t lo, uint32_t hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
    return d;
}

// The mbarrier gets one arrival when every MMA issued so far by this thread has
// finished (its reads of shared memory and writes of tensor memory included).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void umma_commit_at(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// 32 lanes x 32 columns of 32-bit tensor memory: thread t of the warp receives
// columns [col, col + 32) of lane (lane_base + t).  A warp may only touch the
// lane quarter (warp index % 4).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// The reverse: thread t of the warp writes columns [col, col + 32) of its lane.
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
          "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
          "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void tmem_st_32x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
          "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
          "r"(r[14]), "r"(r[15])
        : "memory");
}

// ---- thread-block clusters: barrier over all threads of the cluster, a peer's shared memory ----
// Every thread of every block of the cluster has to come here (the barrier has no
// time limit of its own, so nothing may skip it: waits before it are bounded).
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// the address, in the cluster's shared window, of this block's shared address `local` in block `rank`
__device__ __forceinline__ uint32_t cluster_map(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
__device__ __forceinline__ float4 cluster_ld_f4(uint32_t addr) {
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
    return v;
}

__device__ __forceinline__ void tmem_st_wait() {
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

}  // namespace tc

// ---- host side: TMA tensor maps -------------------------------------------------
#include <map>
#include <mutex>
#include <tuple>

namespace tc {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

// A bf16 matrix [rows, cols] with `ld` elements between rows, read in boxes of
// [box_rows, 64] elements with the 128-byte swizzle; out-of-range elements read 0.
inline bool make_map_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                        uint64_t ld, uint32_t box_rows) {
    typedef std::tuple<const void*, uint64_t, uint64_t, uint64_t, uint32_t> Key;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    Key key(base, rows, cols, ld, box_rows);
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {64, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 8192) cache.clear();
    cache[key] = *out;
    return true;
}

// A bf16 matrix written in boxes of `box_cols` columns (at most 128 bytes) of `box_rows` rows
// that lie unswizzled in shared memory, row after row.
inline bool make_plain_box_map_2d(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols,
                                  uint64_t ld, uint32_t box_cols, uint32_t box_rows) {
    typedef std::tuple<const void*, uint64_t, uint64_t, uint64_t, uint32_t, uint32_t> Key;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    Key key(base, rows, cols, ld, box_cols, box_rows);
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box,
                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 8192) cache.clear();
    cache[key] = *out;
    return true;
}

// K or V pages [n_pages][n_kv_heads][page_tokens][head_dim] bf16 as a 4-D tensor, read in boxes
// of 64 features of `box_pages` consecutive pages of one KV head (128-byte swizzle): a tile of keys whose pages
// follow one another in the pool comes in with one copy instead of one per page.
inline bool make_map_pages(CUtensorMap* out, const void* base, uint64_t n_pages, uint64_t n_kv_heads,
                           uint32_t page_tokens, uint32_t head_dim, uint32_t box_pages) {
    typedef std::tuple<const void*, uint64_t, uint64_t, uint32_t, uint32_t, uint32_t> Key;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    Key key(base, n_pages, n_kv_heads, page_tokens, head_dim, box_pages);
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t row = (cuuint64_t)head_dim * 2;          // bytes of one token's features
    cuuint64_t dims[4] = {head_dim, page_tokens, n_kv_heads, n_pages};
    cuuint64_t strides[3] = {row, page_tokens * row, n_kv_heads * page_tokens * row};
    cuuint32_t box[4] = {64, page_tokens, 1, box_pages};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides,
                    box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 8192) cache.clear();
    cache[key] = *out;
    return true;
}

// An output matrix [rows, cols] (bf16 or fp32) with `ld` elements between rows,
// written in boxes of [box_rows, 128 bytes] with the 128-byte swizzle.
inline bool make_out_map_2d(CUtensorMap* out, const void* base, bool f32, uint64_t rows,
                            uint64_t cols, uint64_t ld, uint32_t box_rows) {
    typedef std::tuple<const void*, bool, uint64_t, uint64_t, uint64_t, uint32_t> Key;
    static std::map<Key, CUtensorMap> cache;
    static std::mutex mu;
    Key key(base, f32, rows, cols, ld, box_rows);
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
        *out = it->second;
        return true;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const uint64_t esize = f32 ? 4 : 2;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * esize};
    cuuint32_t box[2] = {(cuuint32_t)(128 / esize), box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(out, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                    const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return false;
    if (cache.size() > 8192) cache.clear();
    cache[key] = *out;
    return true;
}

// 2-D tiled TMA store shared -> global of one box; elements outside the tensor are
// not written.  x * element size must be a multiple of 16; never negative.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"((uint64_t)map), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}

// The same box added to global memory (fp32 add at the memory side).
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"((uint64_t)map), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
                 : "memory");
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// waits until every committed store of this thread has been written
// waits until the stores sent so far have read their shared memory (it may be written again)
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// silu(g) = g / (1 + e^-g) = g (1 + tanh(g / 2)) / 2 in fp32 with the hardware's tanh (relative
// error about 2^-11; the result is then rounded to bfloat16, 2^-9).  One trip to the
// special-function unit per element, where the exponential and the reciprocal were two, and that
// unit is what an epilogue of 128 elements a thread waits for (a warp's `ex2` takes it 5.5
// cycles); the IEEE division costs a hundred dependent cycles per element.
__device__ __forceinline__ float silu_fast(float g) {
    float t;
    const float h = 0.5f * g;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
    return fmaf(h, t, h);
}

}  // namespace tc
