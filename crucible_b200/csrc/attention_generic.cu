// Paged causal attention, the plain form: one warp per (token row, query head),
// keys visited one by one in ascending position with a running maximum, all in
// fp32.  It serves prompts, portions of prompts and decoded tokens alike: a row
// at position p of request r reads keys lo..p of that request through its block
// table (lo = 0, or p - window + 1).  The result for a row depends only on that
// row's query and its keys, never on the rest of the batch.
//
// This is the attention of the 32-bit path, and the refuge of the bfloat16 path
// for head sizes or options its tensor-core kernels refuse.
// Reference counterparts: `attention_decode_paged_f32`
// (engine/kernels/kernels.cu:1741-1839) and `attention_prefill_paged_impl`
// (:1844-1925): scores scaled by hd^-1/2, max, exp(s - max), sum, one division.
#define CB_PDL_BIT 8      // this file's bit in CRUCIBLE_PDL
#include "common.cuh"

namespace {

constexpr int MAX_PER_LANE = 8;   // head_dim <= 256

template <typename T>
__global__ void attention_generic_kernel(
    const T* __restrict__ qkv, int qkv_stride, T* __restrict__ out, int out_stride,
    const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    const int* __restrict__ positions, const int* __restrict__ row_request,
    const int* __restrict__ block_table, int table_stride, int n_rows, int n_heads,
    int n_kv_heads, int head_dim, int page_tokens, float scale, int window) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int warps_per_block = blockDim.x >> 5;
    const int unit = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
    if (unit >= n_rows * n_heads) return;
    const int lane = threadIdx.x & 31;
    const int t = unit / n_heads, h = unit - t * n_heads;
    const int kvh = h / (n_heads / n_kv_heads);
    const int pos = positions[t];
    const int r = row_request[t];
    const int* table = block_table + (size_t)r * table_stride;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;

    float q[MAX_PER_LANE], acc[MAX_PER_LANE];
    const T* qrow = qkv + (size_t)t * qkv_stride + (size_t)h * head_dim;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int f = lane + 32 * i;
        q[i] = f < head_dim ? cb_to_float(qrow[f]) : 0.f;
        acc[i] = 0.f;
    }
    float m = -INFINITY, l = 0.f;
    for (int j = lo; j <= pos; ++j) {
        const int page = table[j / page_tokens];
        const size_t base =
            (((size_t)page * n_kv_heads + kvh) * page_tokens + (j % page_tokens)) * head_dim;
        float part = 0.f;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int f = lane + 32 * i;
            if (f < head_dim) part = fmaf(q[i], cb_to_float(k_cache[base + f]), part);
        }
        const float s = cb_warp_sum(part) * scale;
        const float m_new = fmaxf(m, s);
        const float corr = expf(m - m_new);     // exp(-inf) = 0 at the first key
        const float p = expf(s - m_new);
        l = l * corr + p;
#pragma unroll
        for (int i = 0; i < MAX_PER_LANE; ++i) {
            const int f = lane + 32 * i;
            if (f < head_dim) acc[i] = fmaf(p, cb_to_float(v_cache[base + f]), acc[i] * corr);
        }
        m = m_new;
    }
    const float inv = 1.0f / l;
    T* orow = out + (size_t)t * out_stride + (size_t)h * head_dim;
#pragma unroll
    for (int i = 0; i < MAX_PER_LANE; ++i) {
        const int f = lane + 32 * i;
        if (f < head_dim) orow[f] = cb_from_float<T>(acc[i] * inv);
    }
}

}  // namespace

CB_EXPORT int cb_attention_generic(const void* qkv, int qkv_stride, void* out, int out_stride,
                                   const void* k_cache, const void* v_cache, int dtype,
                                   const int* positions, const int* row_request,
                                   const int* block_table, int table_stride, int n_rows,
                                   int n_heads, int n_kv_heads, int head_dim, int page_tokens,
                                   float scale, int window, void* stream) {
    if (n_rows <= 0) return 0;
    if (head_dim > 32 * MAX_PER_LANE || n_heads % n_kv_heads != 0) return CB_ERR_UNSUPPORTED;
    const int warps = 4;
    const long units = (long)n_rows * n_heads;
    const int blocks = (int)((units + warps - 1) / warps);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == CB_F32)
        cb_launch(attention_generic_kernel<float>, dim3(blocks), dim3(warps * 32), 0, s, 
            (const float*)qkv, qkv_stride, (float*)out, out_stride, (const float*)k_cache,
            (const float*)v_cache, positions, row_request, block_table, table_stride, n_rows,
            n_heads, n_kv_heads, head_dim, page_tokens, scale, window);
    else
        cb_launch(attention_generic_kernel<__nv_bfloat16>, dim3(blocks), dim3(warps * 32), 0, s, 
            (const __nv_bfloat16*)qkv, qkv_stride, (__nv_bfloat16*)out, out_stride,
            (const __nv_bfloat16*)k_cache, (const __nv_bfloat16*)v_cache, positions, row_request,
            block_table, table_stride, n_rows, n_heads, n_kv_heads, head_dim, page_tokens, scale,
            window);
    return cb_last_error();
}
