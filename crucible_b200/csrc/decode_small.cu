// Matrix products for steps of at most 8 rows (a few decoded tokens), fused
// with what stands before and after them.  Such a step only streams the
// weights once; what decides its time is the length of each kernel's chain of
// dependent memory round trips and the number of kernels.  So these run on CUDA
// cores with plain 16-byte loads (no descriptor fetch, no barrier, no tensor-
// memory allocation in the chain) and each replaces two or three launches:
//
//   NORM_IN   the input is the fp32 residual stream; RMSNorm (fp32 statistics
//             and gain) is applied while it is staged in shared memory, so the
//             normalised row never goes to global memory and is not rounded;
//   epilogues ACCUM_F32    out[m, n] += dot               (output projections)
//             STORE_F32    out[m, n]  = dot               (logits)
//             SWIGLU_BF16  out[m, i]  = silu(g_i) * u_i   (gate and up rows paired)
//             ROPE_APPEND  rows (j, j + hd/2) of a head paired: q rotated and
//                          stored, k rotated into the request's cache page,
//                          v copied into it.
// One warp computes two rows of W against all rows of the step; every dot
// product is one fp32 sum whose order depends on K alone.
//
// Sizes: at most 8 rows; K a multiple of 8 with 16-byte aligned weight rows;
// ROPE_APPEND needs the whole head rotated (rotary_dim == head_dim).  Anything
// else is refused and the caller runs the general kernels.
// Reference counterparts: `gemv_f32_warp` (engine/kernels/kernels.cu:549),
// `mlp_swiglu_f32` (:637), `rope_rows_f32` (:1677), `cache_store_rows_paged_f32`
// (:1713).
#include "common.cuh"

namespace {

enum SmallEpilogue { ACCUM_F32 = 0, STORE_F32 = 1, SWIGLU_BF16 = 2, ROPE_APPEND = 3 };

struct SmallParams {
    const float* x;               // NORM_IN: fp32 [M, K]
    const __nv_bfloat16* a;       // else: bf16 [M, lda]
    int lda;
    const float* gain;
    float eps;
    const __nv_bfloat16* w;       // [rows, K], ldw elements between rows
    int ldw;
    int M, K, N;                  // N: output columns (SWIGLU: the intermediate width)
    int n_tasks;
    void* out;                    // ACCUM/STORE: fp32 [M, ldc]; SWIGLU: bf16 [M, ldc]; ROPE: bf16 q [M, ldc]
    int ldc;
    // ROPE_APPEND
    const float* cos_t;
    const float* sin_t;
    const int* positions;
    const int* row_request;
    const int* block_table;
    int table_stride;
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;
    int n_heads, n_kv_heads, head_dim, page_tokens, write_cache;
};

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 t = __bfloat1622float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

template <int MB, bool NORM_IN, int EPI, int CH>
__global__ void __launch_bounds__(128) small_linear_kernel(const SmallParams p) {
    cb_pdl_trigger();
    extern __shared__ __align__(16) float xs[];          // [M][K]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    const int K = p.K;
    const int task = blockIdx.x * n_warps + warp;
    const bool valid = task < p.n_tasks;
    // ---- the two rows of W this warp owns ----------------------------------------------
    int r0 = 0, r1 = 0;
    bool has1 = true;
    if (valid) {
        if (EPI == SWIGLU_BF16) {
            r0 = task;
            r1 = p.N + task;
        } else if (EPI == ROPE_APPEND) {
            const int half = p.head_dim >> 1;
            const int head = task / half, j = task - head * half;
            r0 = head * p.head_dim + j;
            r1 = r0 + half;
        } else {
            r0 = 2 * task;
            r1 = r0 + 1;
            has1 = r1 < p.N;
        }
    }
    const __nv_bfloat16* w0 = p.w + (size_t)r0 * p.ldw;
    const __nv_bfloat16* w1 = p.w + (size_t)(has1 ? r1 : r0) * p.ldw;
    const int n_chunks = (K + 255) >> 8;                 // 256 elements per warp and chunk
    // The first batch of weight loads goes out before anything else: it depends on
    // nothing, and the staging of the step's rows below hides under its latency.
    uint4 v0[CH], v1[CH];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int k = (c * 32 + lane) * 8;
        if (valid && c < n_chunks && k < K) {
            v0[c] = __ldg(reinterpret_cast<const uint4*>(w0 + k));
            v1[c] = __ldg(reinterpret_cast<const uint4*>(w1 + k));
        } else {
            v0[c] = v1[c] = make_uint4(0, 0, 0, 0);
        }
    }
    // the weights above are written by no kernel; everything below reads what earlier
    // kernels of the stream produced
    cb_pdl_wait();
    float old0 = 0.f, old1 = 0.f;                        // ACCUM: the residual values, fetched early
    if (EPI == ACCUM_F32 && valid && lane < p.M) {
        const float* out = (const float*)p.out + (size_t)lane * p.ldc;
        old0 = out[r0];
        if (has1) old1 = out[r1];
    }
    // ---- stage the step's rows in shared memory (normalised if asked) -------------------
    // 16-byte loads, unrolled so that a row's loads are in flight together: these few
    // round trips are the whole prologue of the kernel.
    if (NORM_IN) {
        const int n4 = K >> 2;
        const float4* g4 = reinterpret_cast<const float4*>(p.gain);
        for (int m = warp; m < p.M; m += n_warps) {
            const float4* row4 = reinterpret_cast<const float4*>(p.x + (size_t)m * K);
            float ss = 0.f;
#pragma unroll 8
            for (int j = lane; j < n4; j += 32) {
                const float4 v = row4[j];
                ss = fmaf(v.x, v.x, ss);
                ss = fmaf(v.y, v.y, ss);
                ss = fmaf(v.z, v.z, ss);
                ss = fmaf(v.w, v.w, ss);
            }
            ss = cb_warp_sum(ss);
            const float r = 1.0f / sqrtf(ss / (float)K + p.eps);
            float4* dst4 = reinterpret_cast<float4*>(xs + m * K);
#pragma unroll 8
            for (int j = lane; j < n4; j += 32) {
                const float4 v = row4[j];
                const float4 g = g4[j];
                dst4[j] = make_float4(v.x * r * g.x, v.y * r * g.y, v.z * r * g.z, v.w * r * g.w);
            }
        }
    } else {
        const int n8 = K >> 3;
        const int total = p.M * n8;
#pragma unroll 4
        for (int i = threadIdx.x; i < total; i += blockDim.x) {
            const int m = i / n8, c = i - m * n8;
            const uint4 v = *reinterpret_cast<const uint4*>(p.a + (size_t)m * p.lda + c * 8);
            float f[8];
            unpack8(v, f);
            float4* dst4 = reinterpret_cast<float4*>(xs + m * K + c * 8);
            dst4[0] = make_float4(f[0], f[1], f[2], f[3]);
            dst4[1] = make_float4(f[4], f[5], f[6], f[7]);
        }
    }
    __syncthreads();
    if (!valid) return;
    float acc0[MB], acc1[MB];
#pragma unroll
    for (int m = 0; m < MB; ++m) acc0[m] = acc1[m] = 0.f;
    for (int c0 = 0; c0 < n_chunks; c0 += CH) {
        if (c0 > 0) {
#pragma unroll
            for (int c = 0; c < CH; ++c) {
                const int k = ((c0 + c) * 32 + lane) * 8;
                if (c0 + c < n_chunks && k < K) {
                    v0[c] = __ldg(reinterpret_cast<const uint4*>(w0 + k));
                    v1[c] = __ldg(reinterpret_cast<const uint4*>(w1 + k));
                } else {
                    v0[c] = v1[c] = make_uint4(0, 0, 0, 0);
                }
            }
        }
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const int k = ((c0 + c) * 32 + lane) * 8;
            if (c0 + c < n_chunks && k < K) {
                float f0[8], f1[8];
                unpack8(v0[c], f0);
                unpack8(v1[c], f1);
#pragma unroll
                for (int m = 0; m < MB; ++m) {
                    if (m < p.M) {
                        const float4 xa = *reinterpret_cast<const float4*>(xs + m * K + k);
                        const float4 xb = *reinterpret_cast<const float4*>(xs + m * K + k + 4);
                        acc0[m] = fmaf(f0[0], xa.x, acc0[m]); acc1[m] = fmaf(f1[0], xa.x, acc1[m]);
                        acc0[m] = fmaf(f0[1], xa.y, acc0[m]); acc1[m] = fmaf(f1[1], xa.y, acc1[m]);
                        acc0[m] = fmaf(f0[2], xa.z, acc0[m]); acc1[m] = fmaf(f1[2], xa.z, acc1[m]);
                        acc0[m] = fmaf(f0[3], xa.w, acc0[m]); acc1[m] = fmaf(f1[3], xa.w, acc1[m]);
                        acc0[m] = fmaf(f0[4], xb.x, acc0[m]); acc1[m] = fmaf(f1[4], xb.x, acc1[m]);
                        acc0[m] = fmaf(f0[5], xb.y, acc0[m]); acc1[m] = fmaf(f1[5], xb.y, acc1[m]);
                        acc0[m] = fmaf(f0[6], xb.z, acc0[m]); acc1[m] = fmaf(f1[6], xb.z, acc1[m]);
                        acc0[m] = fmaf(f0[7], xb.w, acc0[m]); acc1[m] = fmaf(f1[7], xb.w, acc1[m]);
                    }
                }
            }
        }
    }
    // ---- reduce over the warp; lane m keeps row m's two sums -------------------------
    float d0 = 0.f, d1 = 0.f;
#pragma unroll
    for (int m = 0; m < MB; ++m) {
        const float s0 = cb_warp_sum(acc0[m]);
        const float s1 = cb_warp_sum(acc1[m]);
        if (lane == m) { d0 = s0; d1 = s1; }
    }
    if (lane >= p.M) return;
    const int m = lane;
    if (EPI == ACCUM_F32 || EPI == STORE_F32) {
        float* out = (float*)p.out + (size_t)m * p.ldc;
        if (EPI == ACCUM_F32) {
            out[r0] = old0 + d0;
            if (has1) out[r1] = old1 + d1;
        } else {
            out[r0] = d0;
            if (has1) out[r1] = d1;
        }
    } else if (EPI == SWIGLU_BF16) {
        ((__nv_bfloat16*)p.out)[(size_t)m * p.ldc + task] =
            __float2bfloat16_rn(d0 / (1.0f + expf(-d0)) * d1);
    } else {
        const int half = p.head_dim >> 1;
        const int head = task / half, j = task - head * half;
        const int pos = p.positions[m];
        if (head < p.n_heads + p.n_kv_heads) {           // q or k: rotate
            const float c = p.cos_t[(size_t)pos * half + j], s = p.sin_t[(size_t)pos * half + j];
            const float y0 = d0 * c - d1 * s, y1 = d0 * s + d1 * c;
            d0 = y0;
            d1 = y1;
        }
        if (head < p.n_heads) {
            __nv_bfloat16* q = (__nv_bfloat16*)p.out + (size_t)m * p.ldc + (size_t)head * p.head_dim;
            q[j] = __float2bfloat16_rn(d0);
            q[j + half] = __float2bfloat16_rn(d1);
        } else if (p.write_cache) {
            const int page = p.block_table[(size_t)p.row_request[m] * p.table_stride + pos / p.page_tokens];
            const bool is_k = head < p.n_heads + p.n_kv_heads;
            const int kvh = is_k ? head - p.n_heads : head - p.n_heads - p.n_kv_heads;
            __nv_bfloat16* dst = (is_k ? p.k_cache : p.v_cache) +
                (((size_t)page * p.page_tokens + pos % p.page_tokens) * p.n_kv_heads + kvh) * p.head_dim;
            dst[j] = __float2bfloat16_rn(d0);
            dst[j + half] = __float2bfloat16_rn(d1);
        }
    }
}

template <int MB, bool NORM_IN, int EPI, int CH>
int launch_ch(const SmallParams& p, cudaStream_t s) {
    // two warps per block while the tasks are few, so that enough blocks pull on memory
    const int warps = p.n_tasks < 148 * 4 ? 2 : 4;
    const int smem = p.M * p.K * 4;
    static int configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(small_linear_kernel<MB, NORM_IN, EPI, CH>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    const int blocks = (p.n_tasks + warps - 1) / warps;
    cb_launch(small_linear_kernel<MB, NORM_IN, EPI, CH>, dim3(blocks), dim3(warps * 32), smem, s, p);
    return cb_last_error();
}

// Weight loads kept in flight per lane: 4 chunks of 256 elements cover K <= 1024
// in one batch, 8 cover K <= 2048.
template <int MB, bool NORM_IN, int EPI>
int launch(const SmallParams& p, cudaStream_t s) {
    if (p.K <= 1024) return launch_ch<MB, NORM_IN, EPI, 4>(p, s);
    return launch_ch<MB, NORM_IN, EPI, 8>(p, s);
}

template <bool NORM_IN, int EPI>
int launch_rows(const SmallParams& p, cudaStream_t s) {
    if (p.M <= 1) return launch<1, NORM_IN, EPI>(p, s);
    if (p.M <= 2) return launch<2, NORM_IN, EPI>(p, s);
    if (p.M <= 4) return launch<4, NORM_IN, EPI>(p, s);
    return launch<8, NORM_IN, EPI>(p, s);
}

bool sizes_ok(const float* x, const float* gain, const void* a, int lda, int M, int K, int ldw,
              const void* w) {
    if (x ? (((uintptr_t)x & 15) || ((uintptr_t)gain & 15)) : (((uintptr_t)a & 15) || (lda & 7)))
        return false;
    return M >= 1 && M <= 8 && K > 0 && (K & 7) == 0 && (ldw & 7) == 0 && ((uintptr_t)w & 15) == 0 &&
           (size_t)M * K * 4 <= 200 * 1024;
}

}  // namespace

// out[M, N] (+)= act . W^T.  x != null: act = rmsnorm(x, gain, eps) (fp32 [M, K]);
// else act = a (bf16 [M, lda]).  accumulate: add into out (fp32).
CB_EXPORT int cb_small_linear(const float* x, const float* gain, float eps, const void* a, int lda,
                              const void* w, int ldw, float* out, int ldc, int M, int N, int K,
                              int accumulate, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (!sizes_ok(x, gain, a, lda, M, K, ldw, w)) return CB_ERR_UNSUPPORTED;
    SmallParams p = {};
    p.x = x; p.gain = gain; p.eps = eps; p.a = (const __nv_bfloat16*)a; p.lda = lda;
    p.w = (const __nv_bfloat16*)w; p.ldw = ldw; p.M = M; p.K = K; p.N = N;
    p.n_tasks = (N + 1) / 2; p.out = out; p.ldc = ldc;
    cudaStream_t s = (cudaStream_t)stream;
    if (x) return accumulate ? launch_rows<true, ACCUM_F32>(p, s) : launch_rows<true, STORE_F32>(p, s);
    return accumulate ? launch_rows<false, ACCUM_F32>(p, s) : launch_rows<false, STORE_F32>(p, s);
}

// out[M, inter] (bf16) = silu(act Wg^T) * (act Wu^T), W = [Wg; Wu] ([2 inter, K]).
CB_EXPORT int cb_small_swiglu(const float* x, const float* gain, float eps, const void* a, int lda,
                              const void* w, int ldw, void* out, int ldc, int M, int inter, int K,
                              void* stream) {
    if (M <= 0 || inter <= 0) return 0;
    if (!sizes_ok(x, gain, a, lda, M, K, ldw, w)) return CB_ERR_UNSUPPORTED;
    SmallParams p = {};
    p.x = x; p.gain = gain; p.eps = eps; p.a = (const __nv_bfloat16*)a; p.lda = lda;
    p.w = (const __nv_bfloat16*)w; p.ldw = ldw; p.M = M; p.K = K; p.N = inter;
    p.n_tasks = inter; p.out = out; p.ldc = ldc;
    cudaStream_t s = (cudaStream_t)stream;
    return x ? launch_rows<true, SWIGLU_BF16>(p, s) : launch_rows<false, SWIGLU_BF16>(p, s);
}

// The query/key/value projection of an attention layer for a few rows: W =
// [Wq; Wk; Wv]; q is rotated and written (bf16) to q_out[M, ldq]; k (rotated)
// and v go to the rows' cache pages (unless write_cache == 0).
CB_EXPORT int cb_small_qkv_rope_append(const float* x, const float* gain, float eps, const void* a,
                                       int lda, const void* w, int ldw, void* q_out, int ldq,
                                       const float* cos_t, const float* sin_t, int rotary_dim,
                                       const int* positions, const int* row_request,
                                       const int* block_table, int table_stride, void* k_cache,
                                       void* v_cache, int M, int K, int n_heads, int n_kv_heads,
                                       int head_dim, int page_tokens, int write_cache,
                                       void* stream) {
    if (M <= 0) return 0;
    if (!sizes_ok(x, gain, a, lda, M, K, ldw, w) || rotary_dim != head_dim || (head_dim & 1)) return CB_ERR_UNSUPPORTED;
    SmallParams p = {};
    p.x = x; p.gain = gain; p.eps = eps; p.a = (const __nv_bfloat16*)a; p.lda = lda;
    p.w = (const __nv_bfloat16*)w; p.ldw = ldw; p.M = M; p.K = K;
    p.N = (n_heads + 2 * n_kv_heads) * head_dim;
    const int heads = write_cache ? n_heads + 2 * n_kv_heads : n_heads;
    p.n_tasks = heads * (head_dim / 2);
    p.out = q_out; p.ldc = ldq;
    p.cos_t = cos_t; p.sin_t = sin_t; p.positions = positions; p.row_request = row_request;
    p.block_table = block_table; p.table_stride = table_stride;
    p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim;
    p.page_tokens = page_tokens; p.write_cache = write_cache;
    cudaStream_t s = (cudaStream_t)stream;
    return x ? launch_rows<true, ROPE_APPEND>(p, s) : launch_rows<false, ROPE_APPEND>(p, s);
}
