// Token selection on the device: greedy (argmax) and temperature sampling over
// the top-k candidates, one block per logits row.
//
// Rules, from the reference's sampler (engine/src/sampling.rs):
//  * greedy: `best = 0; for i: if v[i] > v[best]: best = i` (:141-149): the highest
//    logit, ties to the lowest index; a NaN never displaces anything, and a NaN at
//    index 0 is never displaced (nothing compares greater than it), so such a row
//    gives 0;
//  * sampled: candidates are the k best in canonical order (logit descending,
//    token id ascending; :161-163) found by radix selection on a 64-bit key
//    (value key << 32 | ~id; :178-202); weights exp((v - max) / T) in fp32,
//    non-finite -> 0; sum and walk in fp64; threshold = u * sum; the first
//    candidate whose running sum reaches it wins (:243-283).  u is one uniform
//    number per sampled token, drawn by the host from the request's own
//    generator, so a request's sequence does not depend on its neighbours.
//  * temperature <= 0 means greedy and uses no randomness (:290-298).
#define CB_PDL_BIT 6      // this file's bit in CRUCIBLE_PDL
#include "common.cuh"
#include "no_alloc_argmax.h"

namespace {

constexpr int SAMPLE_THREADS = 1024;
constexpr int MAX_TOP_K = 1024;

// Order-preserving map from a logit to an unsigned key: NaN lowest (0), -0.0 as
// +0.0 (sampling.rs:178-186).
__device__ __forceinline__ uint32_t value_key(float v) {
    uint32_t u = __float_as_uint(v);
    if (u == 0x80000000u) u = 0u;
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0u;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ unsigned long long sort_key(float v, int id) {
    return ((unsigned long long)value_key(v) << 32) | (unsigned long long)(0xffffffffu - (uint32_t)id);
}

// If `scatter_index` is given, the chosen id of row r is also written to
// scatter_out[scatter_index[r]]: the engine keeps each request's latest token
// on the device that way, so that the next step can read it without the host.
__device__ __forceinline__ void publish(int row, int id, int* out_ids, const int* scatter_index,
                                        int* scatter_out) {
    out_ids[row] = id;
    if (scatter_index != nullptr) scatter_out[scatter_index[row]] = id;
}

// The step's status word rides to the host with the chosen ids: one thread of the
// launch copies it behind them, so that the host, which reads the ids anyway, learns
// of a kernel that gave up a bounded wait without a transfer or a wait of its own.
__device__ __forceinline__ void relay_status(const int* status_src, int* status_dst) {
    if (status_src != nullptr && status_dst != nullptr) *status_dst = *status_src;
}

__device__ void block_argmax(const float* row, int vocab, int* out_id, float* s_val, int* s_idx) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float x = row[i];
        if (x > bv || (x == bv && i < bi)) { bv = x; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { s_val[warp] = bv; s_idx[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        const int nw = (blockDim.x + 31) >> 5;
        for (int w = 1; w < nw; ++w)
            if (s_val[w] > bv || (s_val[w] == bv && s_idx[w] < bi)) { bv = s_val[w]; bi = s_idx[w]; }
        // every logit NaN: token 0; a NaN at index 0 is never displaced
        *out_id = (bi == 0x7fffffff || row[0] != row[0]) ? 0 : bi;
    }
    __syncthreads();
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, int vocab, const float* __restrict__ temperature,
                   const int* __restrict__ top_k, const float* __restrict__ uniform,
                   int* __restrict__ out_ids, const int* __restrict__ scatter_index,
                   int* __restrict__ scatter_out, const int* __restrict__ status_src,
                   int* __restrict__ status_dst) {
    cb_pdl_trigger();
    cb_pdl_wait();
    if (blockIdx.x == 0 && threadIdx.x == 0) relay_status(status_src, status_dst);
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ unsigned int hist[256];
    __shared__ unsigned long long cand[MAX_TOP_K];
    __shared__ unsigned long long prefix_sh;
    __shared__ int remaining_sh;
    __shared__ unsigned int n_cand;

    const int row_i = blockIdx.x;
    const float* row = logits + (size_t)row_i * vocab;
    const float temp = temperature ? temperature[row_i] : 0.f;
    if (!(temp > 0.f)) {
        __shared__ int greedy_id;
        block_argmax(row, vocab, &greedy_id, s_val, s_idx);
        if (threadIdx.x == 0) publish(row_i, greedy_id, out_ids, scatter_index, scatter_out);
        return;
    }
    int k = top_k[row_i];
    k = k < 1 ? 1 : (k > vocab ? vocab : k);
    if (k > MAX_TOP_K) k = MAX_TOP_K;          // the launcher refuses larger k

    // Radix selection of the k-th largest 64-bit key, 8 bits per pass from the top.
    if (threadIdx.x == 0) { prefix_sh = 0ull; remaining_sh = k; }
    __syncthreads();
    for (int pass = 0; pass < 8; ++pass) {
        const int shift = 56 - 8 * pass;
        for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0u;
        __syncthreads();
        const unsigned long long prefix = prefix_sh;
        const unsigned long long mask = pass == 0 ? 0ull : (~0ull << (shift + 8));
        for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
            const unsigned long long key = sort_key(row[i], i);
            if ((key & mask) == prefix) atomicAdd(&hist[(unsigned)(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            int rem = remaining_sh;
            int d = 255;
            for (; d > 0; --d) {
                if ((int)hist[d] >= rem) break;
                rem -= (int)hist[d];
            }
            prefix_sh = prefix | ((unsigned long long)d << shift);
            remaining_sh = rem;
        }
        __syncthreads();
    }
    const unsigned long long kth = prefix_sh;   // exactly k keys are >= kth (keys are unique)

    if (threadIdx.x == 0) n_cand = 0u;
    for (int i = threadIdx.x; i < MAX_TOP_K; i += blockDim.x) cand[i] = 0ull;
    __syncthreads();
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const unsigned long long key = sort_key(row[i], i);
        if (key >= kth) {
            const unsigned int slot = atomicAdd(&n_cand, 1u);
            if (slot < MAX_TOP_K) cand[slot] = key;
        }
    }
    __syncthreads();
    // Bitonic sort, descending, over the smallest power of two >= k.
    int n = 1;
    while (n < k) n <<= 1;
    for (int size = 2; size <= n; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            for (int i = threadIdx.x; i < n; i += blockDim.x) {
                const int j = i ^ stride;
                if (j > i) {
                    const bool desc = (i & size) == 0;
                    const unsigned long long a = cand[i], b = cand[j];
                    if (desc ? a < b : a > b) { cand[i] = b; cand[j] = a; }
                }
            }
            __syncthreads();
        }
    }
    if (threadIdx.x == 0) {
        const int best = (int)(0xffffffffu - (uint32_t)(cand[0] & 0xffffffffull));
        float vmax = -INFINITY;
        for (int i = 0; i < k; ++i) {
            const int id = (int)(0xffffffffu - (uint32_t)(cand[i] & 0xffffffffull));
            const float v = row[id];
            if (v > vmax) vmax = v;
        }
        double sum = 0.0;
        for (int i = 0; i < k; ++i) {
            const int id = (int)(0xffffffffu - (uint32_t)(cand[i] & 0xffffffffull));
            const float w = expf((row[id] - vmax) / temp);
            sum += isfinite(w) ? (double)w : 0.0;
        }
        int chosen = best;
        if (sum > 0.0) {
            const double threshold = (double)uniform[row_i] * sum;
            double acc = 0.0;
            chosen = (int)(0xffffffffu - (uint32_t)(cand[k - 1] & 0xffffffffull));
            for (int i = 0; i < k; ++i) {
                const int id = (int)(0xffffffffu - (uint32_t)(cand[i] & 0xffffffffull));
                const float w = expf((row[id] - vmax) / temp);
                acc += isfinite(w) ? (double)w : 0.0;
                if (acc >= threshold) { chosen = id; break; }
            }
        }
        publish(row_i, chosen, out_ids, scatter_index, scatter_out);
    }
}

__global__ void __launch_bounds__(256)
argmax_rows_kernel(const float* __restrict__ logits, int vocab, int* __restrict__ out_ids,
                   const int* __restrict__ scatter_index, int* __restrict__ scatter_out,
                   const int* __restrict__ status_src, int* __restrict__ status_dst) {
    cb_pdl_trigger();
    cb_pdl_wait();
    if (blockIdx.x == 0 && threadIdx.x == 0) relay_status(status_src, status_dst);
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ int id;
    block_argmax(logits + (size_t)blockIdx.x * vocab, vocab, &id, s_val, s_idx);
    if (threadIdx.x == 0) publish(blockIdx.x, id, out_ids, scatter_index, scatter_out);
}

// Two-stage argmax for wide rows: stage one reduces a slice of the row per
// block and writes (value, index) to scratch; stage two reduces the slices.
// The winner is the same as the one-block kernel's: highest value, lowest
// index among equals, NaN never.
constexpr int ARGMAX_SLICES = 32;

__global__ void __launch_bounds__(256)
argmax_slices_kernel(const float* __restrict__ logits, int vocab, float* __restrict__ part_val,
                     int* __restrict__ part_idx) {
    cb_pdl_trigger();
    cb_pdl_wait();
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    const int row = blockIdx.y, slice = blockIdx.x;
    const int per = (vocab + ARGMAX_SLICES - 1) / ARGMAX_SLICES;
    const int lo = slice * per, hi = min(vocab, lo + per);
    const float* r = logits + (size_t)row * vocab;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float x = r[i];
        if (x > bv || (x == bv && i < bi)) { bv = x; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { s_val[warp] = bv; s_idx[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (s_val[w] > bv || (s_val[w] == bv && s_idx[w] < bi)) { bv = s_val[w]; bi = s_idx[w]; }
        // a NaN at index 0 is never displaced: it enters the second stage as the
        // highest value at the lowest index, which wins there against everything
        if (slice == 0 && r[0] != r[0]) { bv = INFINITY; bi = 0; }
        part_val[row * ARGMAX_SLICES + slice] = bv;
        part_idx[row * ARGMAX_SLICES + slice] = bi;
    }
}

// Both stages in one launch: every block leaves its slice's winner and arrives at the row's
// counter (an atomic; no block waits for another); the block that arrives last reduces the
// row's slices, publishes the id and puts the counter back to zero for the next launch.
// The winner is the one the two kernels find: the same values meet in the same comparison.
__global__ void __launch_bounds__(256)
argmax_fused_kernel(const float* __restrict__ logits, int vocab, float* __restrict__ part_val,
                    int* __restrict__ part_idx, int* __restrict__ counters,
                    int* __restrict__ out_ids, const int* __restrict__ scatter_index,
                    int* __restrict__ scatter_out, const int* __restrict__ status_src,
                    int* __restrict__ status_dst) {
    cb_pdl_trigger();
    cb_pdl_wait();
    __shared__ float s_val[32];
    __shared__ int s_idx[32];
    __shared__ int is_last;
    const int row = blockIdx.y, slice = blockIdx.x;
    const int per = (vocab + ARGMAX_SLICES - 1) / ARGMAX_SLICES;
    const int lo = slice * per, hi = min(vocab, lo + per);
    const float* r = logits + (size_t)row * vocab;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = lo + threadIdx.x; i < hi; i += blockDim.x) {
        const float x = r[i];
        if (x > bv || (x == bv && i < bi)) { bv = x; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { s_val[warp] = bv; s_idx[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (s_val[w] > bv || (s_val[w] == bv && s_idx[w] < bi)) { bv = s_val[w]; bi = s_idx[w]; }
        if (slice == 0 && r[0] != r[0]) { bv = INFINITY; bi = 0; }      // (as in argmax_slices_kernel)
        part_val[row * ARGMAX_SLICES + slice] = bv;
        part_idx[row * ARGMAX_SLICES + slice] = bi;
        __threadfence();
        is_last = atomicAdd(&counters[row], 1) == ARGMAX_SLICES - 1;
    }
    __syncthreads();
    if (!is_last || warp != 0) return;
    __threadfence();
    bv = __ldcg(part_val + row * ARGMAX_SLICES + lane);
    bi = __ldcg(part_idx + row * ARGMAX_SLICES + lane);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) {
        publish(row, bi == 0x7fffffff ? 0 : bi, out_ids, scatter_index, scatter_out);
        counters[row] = 0;
        if (row == 0) relay_status(status_src, status_dst);
    }
}

__global__ void argmax_final_kernel(const float* __restrict__ part_val,
                                    const int* __restrict__ part_idx, int* __restrict__ out_ids,
                                    const int* __restrict__ scatter_index,
                                    int* __restrict__ scatter_out,
                                    const int* __restrict__ status_src,
                                    int* __restrict__ status_dst) {
    cb_pdl_trigger();
    cb_pdl_wait();
    if (blockIdx.x == 0 && threadIdx.x == 0) relay_status(status_src, status_dst);
    const int row = blockIdx.x, lane = threadIdx.x;
    float bv = part_val[row * ARGMAX_SLICES + lane];
    int bi = part_idx[row * ARGMAX_SLICES + lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) publish(row, bi == 0x7fffffff ? 0 : bi, out_ids, scatter_index, scatter_out);
}

}  // namespace

// scratch: n_rows * 32 floats followed by n_rows * 32 ints (cb_argmax_scratch_bytes),
// or null: then one block per row does the whole row.
// counters: null, or n_rows ints that are zero before the call and zero again after it:
// both stages then run as one launch.
// status_src, status_dst (both or neither): *status_dst = *status_src, by the launch
// that writes the ids.
CB_EXPORT int cb_argmax_rows(const float* logits, int n_rows, int vocab, int* out_ids,
                             void* scratch, const int* scatter_index, int* scatter_out,
                             const int* status_src, int* status_dst, void* stream, int* counters) {
    if (n_rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (scratch == nullptr || vocab < 4096) {
        cb_launch(argmax_rows_kernel, dim3(n_rows), dim3(256), 0, s, logits, vocab, out_ids,
                  scatter_index, scatter_out, status_src, status_dst);
        return cb_last_error();
    }
    float* part_val = (float*)scratch;
    int* part_idx = (int*)(part_val + (size_t)n_rows * ARGMAX_SLICES);
    if (counters != nullptr) {
        cb_launch(argmax_fused_kernel, dim3(ARGMAX_SLICES, n_rows), dim3(256), 0, s, logits, vocab, part_val,
                  part_idx, counters, out_ids, scatter_index, scatter_out, status_src, status_dst);
        return cb_last_error();
    }
    cb_launch(argmax_slices_kernel, dim3(ARGMAX_SLICES, n_rows), dim3(256), 0, s, logits, vocab, part_val,
                                                                     part_idx);
    cb_launch(argmax_final_kernel, dim3(n_rows), dim3(32), 0, s, (const float*)part_val,
              (const int*)part_idx, out_ids, scatter_index, scatter_out, status_src, status_dst);
    return cb_last_error();
}

CB_EXPORT long cb_argmax_scratch_bytes(int n_rows) { return (long)n_rows * ARGMAX_SLICES * 8; }

// temperature[row] <= 0: greedy.  max_top_k is the largest k among the rows;
// the launcher refuses k above the kernel's candidate capacity.
CB_EXPORT int cb_sample_rows(const float* logits, int n_rows, int vocab, const float* temperature,
                             const int* top_k, const float* uniform, int max_top_k, int* out_ids,
                             const int* scatter_index, int* scatter_out, const int* status_src,
                             int* status_dst, void* stream) {
    if (n_rows <= 0) return 0;
    if (max_top_k > MAX_TOP_K) return CB_ERR_UNSUPPORTED;
    cb_launch(sample_rows_kernel, dim3(n_rows), dim3(SAMPLE_THREADS), 0, (cudaStream_t)stream,
              logits, vocab, temperature, top_k, uniform, out_ids, scatter_index, scatter_out,
              status_src, status_dst);
    return cb_last_error();
}

CB_EXPORT int cb_sample_max_top_k() { return MAX_TOP_K; }

// ---------------------------------------------------------------------------
// The same two-stage argmax with its scratch inside the library, for callers
// that cannot allocate (see no_alloc_argmax.h).  The array's name is a host-side
// stand-in in host code, not a device address: the address is looked up once per
// device with cudaGetSymbolAddress and that pointer is what the kernels get.
// ---------------------------------------------------------------------------
static __device__ __align__(256) unsigned char
    cb_argmax_static_scratch[CB_ARGMAX_STATIC_MAX_ROWS * ARGMAX_SLICES * 8];

CB_EXPORT int cb_argmax_rows_static(const float* logits, int n_rows, int vocab, int* out_ids,
                                    void* stream) {
    if (n_rows <= 0) return 0;
    if (n_rows > CB_ARGMAX_STATIC_MAX_ROWS) return CB_ERR_STATIC_TOO_LARGE;
    constexpr int MAX_DEVICES = 64;
    static void* scratch_of_device[MAX_DEVICES] = {};
    int device = 0;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess) return (int)e;
    if (device < 0 || device >= MAX_DEVICES) return (int)cudaErrorInvalidDevice;
    if (scratch_of_device[device] == nullptr) {
        // set-up, once per device, with that device current
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, cb_argmax_static_scratch);
        if (e != cudaSuccess) return (int)e;
        scratch_of_device[device] = ptr;
    }
    float* part_val = (float*)scratch_of_device[device];
    int* part_idx = (int*)(part_val + (size_t)n_rows * ARGMAX_SLICES);
    cudaStream_t s = (cudaStream_t)stream;
    cb_launch(argmax_slices_kernel, dim3(ARGMAX_SLICES, n_rows), dim3(256), 0, s, logits, vocab,
              part_val, part_idx);
    cb_launch(argmax_final_kernel, dim3(n_rows), dim3(32), 0, s, (const float*)part_val,
              (const int*)part_idx, out_ids, (const int*)nullptr, (int*)nullptr,
              (const int*)nullptr, (int*)nullptr);
    return cb_last_error();
}
