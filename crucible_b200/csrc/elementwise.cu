// Row-wise kernels: embedding gather, RMSNorm, SwiGLU activation, row gather,
// and rotary encoding fused with the write of keys and values into the paged
// cache.  All arithmetic is fp32; T is the storage type of activations
// (float for the 32-bit engine, __nv_bfloat16 for the bfloat16 engine).
#define CB_PDL_BIT 3      // this file's bit in CRUCIBLE_PDL
#define CB_PDL_MAX_BLOCKS 148
#include "common.cuh"

// ---------------------------------------------------------------------------
// embedding: out[t, :] = float(table[ids[t], :]).  A negative id -(s + 1) means
// "the token the engine last chose for state slot s", read from device_tokens[s]:
// a decoded token then never has to visit the host before it is run.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                                  float* __restrict__ out, int width, int vocab,
                                  const int* __restrict__ device_tokens) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int t = blockIdx.x;
    int id = ids[t];
    if (id < 0 && device_tokens != nullptr) id = device_tokens[-id - 1];
    // ids are validated on the host; an id outside the table still must not
    // read outside it
    id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
    const T* row = table + (size_t)id * width;
    float* dst = out + (size_t)t * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = cb_to_float(row[i]);
}

CB_EXPORT int cb_embed_rows(const void* table, int table_dtype, const int* ids, float* out,
                            int n_rows, int width, int vocab, const int* device_tokens,
                            void* stream) {
    if (n_rows <= 0) return 0;
    const int threads = width >= 256 ? 256 : 64;
    if (table_dtype == CB_F32)
        cb_launch(embed_rows_kernel<float>, dim3(n_rows), dim3(threads), 0, (cudaStream_t)stream, 
            (const float*)table, ids, out, width, vocab, device_tokens);
    else
        cb_launch(embed_rows_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, (cudaStream_t)stream, 
            (const __nv_bfloat16*)table, ids, out, width, vocab, device_tokens);
    return cb_last_error();
}

// ---------------------------------------------------------------------------
// RMSNorm: y = x * (1/sqrt(mean(x^2) + eps)) * gain     (x fp32, gain fp32)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                               T* __restrict__ out, int width, float eps) {
    cb_pdl_trigger();
    cb_pdl_wait();
    __shared__ float scratch[32];
    const float* row = x + (size_t)blockIdx.x * width;
    T* dst = out + (size_t)blockIdx.x * width;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        const float v = row[i];
        ss = fmaf(v, v, ss);
    }
    const float total = cb_block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(total / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        dst[i] = cb_from_float<T>(row[i] * r * gain[i]);
}

// The same for widths that are multiples of 4: float4 loads, the row kept in
// registers between the two passes (up to 4 vectors per thread).
template <typename T>
__global__ void rmsnorm_vec4_kernel(const float* __restrict__ x, const float* __restrict__ gain,
                                    T* __restrict__ out, int width, float eps) {
    cb_pdl_trigger();
    cb_pdl_wait();
    __shared__ float scratch[32];
    const int n4 = width >> 2;
    const float4* row = reinterpret_cast<const float4*>(x + (size_t)blockIdx.x * width);
    const float4* g4 = reinterpret_cast<const float4*>(gain);
    float4 v[4];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        v[j] = i < n4 ? row[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        ss = fmaf(v[j].x, v[j].x, ss);
        ss = fmaf(v[j].y, v[j].y, ss);
        ss = fmaf(v[j].z, v[j].z, ss);
        ss = fmaf(v[j].w, v[j].w, ss);
    }
    const float total = cb_block_sum(ss, scratch);
    const float r = 1.0f / sqrtf(total / (float)width + eps);
    T* dst = out + (size_t)blockIdx.x * width;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < n4) {
            const float4 g = g4[i];
            dst[4 * i + 0] = cb_from_float<T>(v[j].x * r * g.x);
            dst[4 * i + 1] = cb_from_float<T>(v[j].y * r * g.y);
            dst[4 * i + 2] = cb_from_float<T>(v[j].z * r * g.z);
            dst[4 * i + 3] = cb_from_float<T>(v[j].w * r * g.w);
        }
    }
}

// One warp per row (widths up to 32 * 4 * V floats): the row stays in registers between
// the two passes, no block barrier, several rows per block; the result leaves in 8- or
// 16-byte stores.  For many rows this keeps far more bytes in flight than a block per row.
template <typename T, int V>
__global__ void __launch_bounds__(128) rmsnorm_warp_kernel(const float* __restrict__ x,
                                                           const float* __restrict__ gain,
                                                           T* __restrict__ out, int n_rows, int width,
                                                           float eps) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= n_rows) return;
    const int n4 = width >> 2;
    const float4* row = reinterpret_cast<const float4*>(x + (size_t)r * width);
    const float4* g4 = reinterpret_cast<const float4*>(gain);
    float4 v[V];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < V; ++j) {
        const int i = lane + 32 * j;
        v[j] = i < n4 ? row[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
#pragma unroll
    for (int j = 0; j < V; ++j) {
        ss = fmaf(v[j].x, v[j].x, ss);
        ss = fmaf(v[j].y, v[j].y, ss);
        ss = fmaf(v[j].z, v[j].z, ss);
        ss = fmaf(v[j].w, v[j].w, ss);
    }
    ss = cb_warp_sum(ss);
    const float rs = 1.0f / sqrtf(ss / (float)width + eps);
    T* dst = out + (size_t)r * width;
#pragma unroll
    for (int j = 0; j < V; ++j) {
        const int i = lane + 32 * j;
        if (i < n4) {
            const float4 g = __ldg(g4 + i);
            const float y0 = v[j].x * rs * g.x, y1 = v[j].y * rs * g.y;
            const float y2 = v[j].z * rs * g.z, y3 = v[j].w * rs * g.w;
            if (sizeof(T) == 2) {
                __nv_bfloat162 a = __floats2bfloat162_rn(y0, y1), b = __floats2bfloat162_rn(y2, y3);
                uint2 w;
                w.x = *reinterpret_cast<uint32_t*>(&a);
                w.y = *reinterpret_cast<uint32_t*>(&b);
                reinterpret_cast<uint2*>(dst)[i] = w;
            } else {
                reinterpret_cast<float4*>(dst)[i] = make_float4(y0, y1, y2, y3);
            }
        }
    }
}

template <typename T>
static void launch_rmsnorm_warp(const float* x, const float* gain, T* out, int n_rows, int width,
                                float eps, cudaStream_t s) {
    const int blocks = (n_rows + 3) / 4;
    if ((width >> 2) <= 32 * 8)
        cb_launch(rmsnorm_warp_kernel<T, 8>, dim3(blocks), dim3(128), 0, s, x, gain, out, n_rows, width, eps);
    else
        cb_launch(rmsnorm_warp_kernel<T, 32>, dim3(blocks), dim3(128), 0, s, x, gain, out, n_rows, width, eps);
}

CB_EXPORT int cb_rmsnorm(const float* x, const float* gain, void* out, int out_dtype,
                         int n_rows, int width, float eps, void* stream) {
    if (n_rows <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = (width & 3) == 0 && width <= 4 * 4 * 1024 && ((uintptr_t)x & 15) == 0 &&
                     ((uintptr_t)gain & 15) == 0;
    // Many rows with a bfloat16 result: a warp per row; the output's rows must allow the
    // vector stores.  A float32 result (the 32-bit engine) never takes this form: the warp
    // kernel adds a row's squares in another order than the block kernels below, and the
    // 32-bit path's sums must be the same whatever the number of rows in the step, so that
    // a token's values do not depend on how its prompt was cut.  Below, the kernel and its
    // block size are functions of the width and of the pointers' alignment alone.
    const bool out_vec = ((uintptr_t)out & 7) == 0;
    if (vec && out_vec && out_dtype != CB_F32 && n_rows >= 64 && (width >> 2) <= 32 * 32) {
        launch_rmsnorm_warp<__nv_bfloat16>(x, gain, (__nv_bfloat16*)out, n_rows, width, eps, s);
        return cb_last_error();
    }
    if (vec) {
        int threads = ((width >> 2) + 31) / 32 * 32;
        if (threads > 1024) threads = ((width >> 2) + 4 * 32 - 1) / (4 * 32) * 32;
        if (threads < 32) threads = 32;
        if (out_dtype == CB_F32)
            cb_launch(rmsnorm_vec4_kernel<float>, dim3(n_rows), dim3(threads), 0, s, x, gain, (float*)out, width, eps);
        else
            cb_launch(rmsnorm_vec4_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, s, 
                x, gain, (__nv_bfloat16*)out, width, eps);
        return cb_last_error();
    }
    const int threads = width >= 1024 ? 256 : 128;
    if (out_dtype == CB_F32)
        cb_launch(rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), 0, s, x, gain, (float*)out, width, eps);
    else
        cb_launch(rmsnorm_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, s, x, gain, (__nv_bfloat16*)out,
                                                                 width, eps);
    return cb_last_error();
}

// ---------------------------------------------------------------------------
// SwiGLU activation on a fused [T, 2I] gate|up buffer: h = g / (1 + exp(-g)) * u
// ---------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gate_up, T* __restrict__ out,
                              int inter, size_t total) {
    cb_pdl_trigger();
    cb_pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const size_t t = i / inter;
        const int c = (int)(i - t * inter);
        const float g = cb_to_float(gate_up[t * 2 * inter + c]);
        const float u = cb_to_float(gate_up[t * 2 * inter + inter + c]);
        out[i] = cb_from_float<T>(g / (1.0f + expf(-g)) * u);
    }
}

CB_EXPORT int cb_swiglu(const void* gate_up, void* out, int dtype, int n_rows, int inter,
                        void* stream) {
    const size_t total = (size_t)n_rows * inter;
    if (total == 0) return 0;
    const int threads = 256;
    size_t blocks = (total + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (dtype == CB_F32)
        cb_launch(swiglu_kernel<float>, dim3((int)blocks), dim3(threads), 0, (cudaStream_t)stream, 
            (const float*)gate_up, (float*)out, inter, total);
    else
        cb_launch(swiglu_kernel<__nv_bfloat16>, dim3((int)blocks), dim3(threads), 0, (cudaStream_t)stream, 
            (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total);
    return cb_last_error();
}

// ---------------------------------------------------------------------------
// gather of fp32 rows: out[i, :] = x[rows[i], :]
// ---------------------------------------------------------------------------
__global__ void gather_rows_kernel(const float* __restrict__ x, const int* __restrict__ rows,
                                   float* __restrict__ out, int width) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const float* src = x + (size_t)rows[blockIdx.x] * width;
    float* dst = out + (size_t)blockIdx.x * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = src[i];
}

CB_EXPORT int cb_gather_rows(const float* x, const int* rows, float* out, int n_rows, int width,
                             void* stream) {
    if (n_rows <= 0) return 0;
    cb_launch(gather_rows_kernel, dim3(n_rows), dim3(128), 0, (cudaStream_t)stream, x, rows, out, width);
    return cb_last_error();
}

// ---------------------------------------------------------------------------
// Rotary encoding of q and k (half-split pairing) fused with the cache write.
// qkv: [T, (Hq + 2 Hkv) * hd]; q is rotated in place; rotated k and plain v go
// to the token's page: cache[page][kv_head][slot][feature].
// One block per (token, head); heads 0..Hq-1 are q, then Hkv k heads, then
// Hkv v heads.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_append_kernel(T* __restrict__ qkv, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, int rotary_dim,
                                      const int* __restrict__ positions,
                                      const int* __restrict__ row_request,
                                      const int* __restrict__ block_table, int table_stride,
                                      T* __restrict__ k_cache, T* __restrict__ v_cache,
                                      int n_heads, int n_kv_heads, int head_dim,
                                      int page_tokens, int write_cache) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int t = blockIdx.x;
    const int row_width = (n_heads + 2 * n_kv_heads) * head_dim;
    T* row = qkv + (size_t)t * row_width;
    const int pos = positions[t];
    const int half = rotary_dim >> 1;
    const int pass = head_dim - rotary_dim;          // features that are not rotated
    // cache[page][kv_head][slot][feature]: the token's row of KV head h starts at
    // cache_base + h * head_stride
    size_t cache_base = 0;
    const size_t head_stride = (size_t)page_tokens * head_dim;
    if (write_cache) {
        const int r = row_request[t];
        const int page = block_table[(size_t)r * table_stride + pos / page_tokens];
        cache_base = (size_t)page * n_kv_heads * head_stride + (size_t)(pos % page_tokens) * head_dim;
    }
    const float* c_row = cos_t + (size_t)pos * half;
    const float* s_row = sin_t + (size_t)pos * half;
    // rotated pairs of q and k heads
    const int n_rot_heads = n_heads + (write_cache ? n_kv_heads : 0);
    for (int i = threadIdx.x; i < n_rot_heads * half; i += blockDim.x) {
        const int h = i / half, j = i - h * half;
        T* src = row + (size_t)h * head_dim;
        const float c = c_row[j], s = s_row[j];
        const float x1 = cb_to_float(src[j]);
        const float x2 = cb_to_float(src[j + half]);
        T* dst = h < n_heads ? src : k_cache + cache_base + (size_t)(h - n_heads) * head_stride;
        dst[j] = cb_from_float<T>(x1 * c - x2 * s);
        dst[j + half] = cb_from_float<T>(x1 * s + x2 * c);
    }
    if (!write_cache) return;
    // unrotated tail of the k heads, and the v heads
    if (pass > 0) {
        for (int i = threadIdx.x; i < n_kv_heads * pass; i += blockDim.x) {
            const int h = i / pass, j = rotary_dim + (i - h * pass);
            k_cache[cache_base + (size_t)h * head_stride + j] = row[(size_t)(n_heads + h) * head_dim + j];
        }
    }
    const T* v_src = row + (size_t)(n_heads + n_kv_heads) * head_dim;
    for (int i = threadIdx.x; i < n_kv_heads * head_dim; i += blockDim.x) {
        const int h = i / head_dim;
        v_cache[cache_base + (size_t)h * head_stride + (i - h * head_dim)] = v_src[i];
    }
}

// The same for bfloat16 rows whose head size, rotated half and unrotated tail are
// multiples of 8: a thread takes 8 features (16 bytes) of a head - for rotated
// features the 8 of the first half and their 8 partners - so a token's row is
// read and written once in 16-byte pieces.  Items are spread over the grid
// whatever the number of tokens.
__global__ void rope_kv_append_vec8_kernel(__nv_bfloat16* __restrict__ qkv,
                                           const float* __restrict__ cos_t,
                                           const float* __restrict__ sin_t, int rotary_dim,
                                           const int* __restrict__ positions,
                                           const int* __restrict__ row_request,
                                           const int* __restrict__ block_table, int table_stride,
                                           __nv_bfloat16* __restrict__ k_cache,
                                           __nv_bfloat16* __restrict__ v_cache, int n_rows,
                                           int n_heads, int n_kv_heads, int head_dim,
                                           int page_tokens, int write_cache) {
    cb_pdl_trigger();
    cb_pdl_wait();
    const int half = rotary_dim >> 1;
    const int pass = head_dim - rotary_dim;
    const int n_rot_heads = n_heads + (write_cache ? n_kv_heads : 0);
    const int rot_items = n_rot_heads * (half >> 3);
    const int tail_items = write_cache ? n_kv_heads * (pass >> 3) : 0;
    const int v_items = write_cache ? n_kv_heads * (head_dim >> 3) : 0;
    const int per_token = rot_items + tail_items + v_items;
    const int row_width = (n_heads + 2 * n_kv_heads) * head_dim;
    const size_t head_stride = (size_t)page_tokens * head_dim;
    const long total = (long)n_rows * per_token;
    for (long idx = (long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (long)gridDim.x * blockDim.x) {
        const int t = (int)(idx / per_token);
        int item = (int)(idx - (long)t * per_token);
        __nv_bfloat16* row = qkv + (size_t)t * row_width;
        const int pos = positions[t];
        size_t cache_base = 0;
        if (write_cache) {
            const int page = block_table[(size_t)row_request[t] * table_stride + pos / page_tokens];
            cache_base = (size_t)page * n_kv_heads * head_stride + (size_t)(pos % page_tokens) * head_dim;
        }
        if (item < rot_items) {
            const int per_head = half >> 3;
            const int h = item / per_head, j = (item - h * per_head) << 3;
            const __nv_bfloat16* src = row + (size_t)h * head_dim;
            const uint4 lo = *reinterpret_cast<const uint4*>(src + j);
            const uint4 hi = *reinterpret_cast<const uint4*>(src + j + half);
            const float4 c0 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + j);
            const float4 c1 = *reinterpret_cast<const float4*>(cos_t + (size_t)pos * half + j + 4);
            const float4 s0 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + j);
            const float4 s1 = *reinterpret_cast<const float4*>(sin_t + (size_t)pos * half + j + 4);
            const float c[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
            const float sn[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            const __nv_bfloat16* x1 = reinterpret_cast<const __nv_bfloat16*>(&lo);
            const __nv_bfloat16* x2 = reinterpret_cast<const __nv_bfloat16*>(&hi);
            uint4 out_lo, out_hi;
            __nv_bfloat16* y1 = reinterpret_cast<__nv_bfloat16*>(&out_lo);
            __nv_bfloat16* y2 = reinterpret_cast<__nv_bfloat16*>(&out_hi);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float a = __bfloat162float(x1[i]), b = __bfloat162float(x2[i]);
                y1[i] = __float2bfloat16_rn(a * c[i] - b * sn[i]);
                y2[i] = __float2bfloat16_rn(a * sn[i] + b * c[i]);
            }
            __nv_bfloat16* dst = h < n_heads ? row + (size_t)h * head_dim
                                             : k_cache + cache_base + (size_t)(h - n_heads) * head_stride;
            *reinterpret_cast<uint4*>(dst + j) = out_lo;
            *reinterpret_cast<uint4*>(dst + j + half) = out_hi;
            continue;
        }
        item -= rot_items;
        if (item < tail_items) {
            const int per_head = pass >> 3;
            const int h = item / per_head, j = rotary_dim + ((item - h * per_head) << 3);
            *reinterpret_cast<uint4*>(k_cache + cache_base + (size_t)h * head_stride + j) =
                *reinterpret_cast<const uint4*>(row + (size_t)(n_heads + h) * head_dim + j);
            continue;
        }
        item -= tail_items;
        const int per_head = head_dim >> 3;
        const int h = item / per_head, j = (item - h * per_head) << 3;
        *reinterpret_cast<uint4*>(v_cache + cache_base + (size_t)h * head_stride + j) =
            *reinterpret_cast<const uint4*>(row + (size_t)(n_heads + n_kv_heads + h) * head_dim + j);
    }
}

CB_EXPORT int cb_rope_kv_append(void* qkv, int dtype, const float* cos_t, const float* sin_t,
                                int rotary_dim, const int* positions, const int* row_request,
                                const int* block_table, int table_stride, void* k_cache,
                                void* v_cache, int n_rows, int n_heads, int n_kv_heads,
                                int head_dim, int page_tokens, int write_cache, void* stream) {
    if (n_rows <= 0) return 0;
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1)) return CB_ERR_UNSUPPORTED;
    const int work = (n_heads + n_kv_heads) * (rotary_dim / 2);
    int threads = (work + 31) / 32 * 32;
    if (threads > 512) threads = 512;
    if (threads < 64) threads = 64;
    if (dtype != CB_F32 && (head_dim & 7) == 0 && (rotary_dim & 15) == 0 &&
        ((uintptr_t)qkv & 15) == 0 && ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0 &&
        (rotary_dim == 0 || (((uintptr_t)cos_t | (uintptr_t)sin_t) & 15) == 0)) {
        const int half8 = rotary_dim >> 4;
        const long per_token = (long)(n_heads + (write_cache ? n_kv_heads : 0)) * half8 +
                               (write_cache ? (long)n_kv_heads * (((head_dim - rotary_dim) >> 3) + (head_dim >> 3)) : 0);
        const long total = (long)n_rows * per_token;
        if (total == 0) return 0;
        long blocks = (total + 255) / 256;
        if (blocks > 148 * 8) blocks = 148 * 8;
        cb_launch(rope_kv_append_vec8_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream,
                  (__nv_bfloat16*)qkv, cos_t, sin_t, rotary_dim, positions, row_request, block_table,
                  table_stride, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, n_rows, n_heads,
                  n_kv_heads, head_dim, page_tokens, write_cache);
        return cb_last_error();
    }
    if (dtype == CB_F32)
        cb_launch(rope_kv_append_kernel<float>, dim3(n_rows), dim3(threads), 0, (cudaStream_t)stream, 
            (float*)qkv, cos_t, sin_t, rotary_dim, positions, row_request, block_table,
            table_stride, (float*)k_cache, (float*)v_cache, n_heads, n_kv_heads, head_dim,
            page_tokens, write_cache);
    else
        cb_launch(rope_kv_append_kernel<__nv_bfloat16>, dim3(n_rows), dim3(threads), 0, (cudaStream_t)stream, 
            (__nv_bfloat16*)qkv, cos_t, sin_t, rotary_dim, positions, row_request, block_table,
            table_stride, (__nv_bfloat16*)k_cache, (__nv_bfloat16*)v_cache, n_heads, n_kv_heads,
            head_dim, page_tokens, write_cache);
    return cb_last_error();
}

CB_EXPORT const char* cb_error_string(int code) {
    if (code == CB_ERR_UNSUPPORTED) return "sizes or options this kernel does not take";
    return cudaGetErrorString((cudaError_t)code);
}
