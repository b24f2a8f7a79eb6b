// Matrix products for steps of at most 8 rows (a few decoded tokens), fused
// with what stands before and after them.  Such a step only streams the
// weights once; what decides its time is the length of each kernel's chain of
// dependent memory round trips and the number of kernels.  So these kernels
// read the weights with plain 16-byte loads that are issued before anything
// else (no descriptor fetch, no barrier, no tensor-memory allocation in the
// chain), multiply on the tensor cores with mma.sync m16n8k16 (16 rows of W
// against the step's up to 8 rows, fp32 accumulation), and each replaces two or
// three launches:
//
//   NORM_IN   the input is the fp32 residual stream; RMSNorm (fp32 statistics
//             and gain) is applied while it is staged in shared memory, so the
//             normalised rows never go to global memory;
//   epilogues ACCUM_F32    out[m, n] += dot               (output projections)
//             STORE_F32    out[m, n]  = dot               (logits)
//             SWIGLU_BF16  out[m, i]  = silu(g_i) * u_i   (gate and up rows paired)
//             ROPE_APPEND  rows (j, j + hd/2) of a head paired: q rotated and
//                          stored, k rotated into the request's cache page,
//                          v copied into it.
// A block owns 16 rows of W: 8 "first" rows and their 8 partners (the next 8
// rows, the matching up rows, or the other half of the rotary pairs), so that
// both members of a pair end in the same thread.  Its four warps split K in
// blocks of 32 elements and their partial sums are added in warp order, so a
// dot product's summation order depends on K alone.
//
// Within a block of 32 elements along K, thread t of a quad loads elements
// [8t, 8t + 8) of its two W rows and of its row of the step with one 16-byte
// load each, and feeds them to two MMAs as "k = 2t, 2t+1, 2t+8, 2t+9": the same
// permutation of k on both operands, which a dot product does not see.
//
// Sizes: at most 32 rows (in groups of 8: each weight fragment then meets one, two or four
// pairs of MMAs); K a multiple of
// 8 with 16-byte aligned weight rows;
// ROPE_APPEND needs the whole head rotated (rotary_dim == head_dim).  Anything
// else is refused and the caller runs the general kernels.
// Reference counterparts: `gemv_batch_i8_b*` (engine/kernels/kernels.cu:1598),
// `mlp_swiglu_f32` (:637), `rope_rows_f32` (:1677), `cache_store_rows_paged_f32`
// (:1713).
#define CB_PDL_BIT 4      // this file's bit in CRUCIBLE_PDL
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
    int n_tiles;
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
    int trigger_early;            // let the kernel after this one start as soon as this one's weights are asked for
                                  // (the q/k/v product: measured on B200 at batch 1 / 8, 2,048-token contexts,
                                  // 0.291 -> 0.286 / 0.345 -> 0.330 ms per step; for the other products 0 to
                                  // 0.03 ms slower: their successors' weight loads get in the way)
};

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

constexpr int BATCH = 8;          // blocks of 32 elements a warp keeps in flight per row

// DEEP: K spans more than one batch of weight loads per warp; the next batch is then in
// flight while the current one is multiplied (costs registers, so short K keeps the plain form).
// WARPS: 4, or 8 for long K (each warp's share of K is then short enough for one batch).
// MT: groups of 8 rows of the step (1, 2 or 4: up to 8, 16 or 32 rows); each weight fragment
// then meets MT pairs of MMAs, and the rows are staged one group after the other.
template <bool NORM_IN, int EPI, bool DEEP, int WARPS, int MT>
__global__ void __launch_bounds__(WARPS * 32) small_linear_kernel(const SmallParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int K = p.K;
    const int pitch = K + 32;                             // bf16 elements; staggers the rows over the banks
    __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(smem_raw);                    // [8 * MT][pitch]
    float* red = reinterpret_cast<float*>(smem_raw + (size_t)8 * MT * pitch * 2);      // [WARPS][MT][32][4]
    const int tile = blockIdx.x;
    // ---- this thread's two rows of W: first row g of the tile, and its partner ------------
    int rf, rs;
    bool ok_f, ok_s;
    if (EPI == SWIGLU_BF16) {
        rf = tile * 8 + g;
        ok_f = ok_s = rf < p.N;
        rs = p.N + rf;
    } else if (EPI == ROPE_APPEND) {
        const int half = p.head_dim >> 1;
        const int pair = tile * 8 + g;
        const int head = pair / half, j = pair - head * half;
        const int heads = p.write_cache ? p.n_heads + 2 * p.n_kv_heads : p.n_heads;
        ok_f = ok_s = head < heads;
        rf = head * p.head_dim + j;
        rs = rf + half;
    } else {
        rf = tile * 16 + g;
        rs = rf + 8;
        ok_f = rf < p.N;
        ok_s = rs < p.N;
    }
    const __nv_bfloat16* wf = p.w + (size_t)(ok_f ? rf : 0) * p.ldw + t * 8;
    const __nv_bfloat16* ws = p.w + (size_t)(ok_s ? rs : 0) * p.ldw + t * 8;
    const int k_blocks = (K + 31) >> 5;
    // The first batch of weight loads goes out before anything else: it depends on
    // nothing, and the staging of the step's rows below hides under its latency.
    uint4 vf[BATCH], vs[BATCH];
#pragma unroll
    for (int i = 0; i < BATCH; ++i) {
        const int kb = warp + i * WARPS;
        const bool in = kb < k_blocks && kb * 32 + t * 8 < K;
        vf[i] = in ? __ldg(reinterpret_cast<const uint4*>(wf + kb * 32)) : make_uint4(0, 0, 0, 0);
        vs[i] = in ? __ldg(reinterpret_cast<const uint4*>(ws + kb * 32)) : make_uint4(0, 0, 0, 0);
    }
    // The kernel after the q/k/v product is the attention over the cache: it may start at
    // once, so that its blocks are resident and their barriers, tensor memory, metadata and
    // block-table lookups are done by the time this kernel ends.
    if (p.trigger_early) cb_pdl_trigger();
    // the weights above are written by no kernel; everything below reads what earlier
    // kernels of the stream produced
    cb_pdl_wait();
    // What the epilogue will need from memory is asked for now, before the staging, so
    // that every round trip of this kernel's prologue is in flight at the same time.
    // ACCUM: the residual values this block will add to.
    float old[MT][4];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
        old[nt][0] = old[nt][1] = old[nt][2] = old[nt][3] = 0.f;
        if (EPI == ACCUM_F32 && warp == 0) {
            const float* out = (const float*)p.out;
            const int m0 = nt * 8 + 2 * t, m1 = m0 + 1;
            if (m0 < p.M && ok_f) old[nt][0] = out[(size_t)m0 * p.ldc + rf];
            if (m1 < p.M && ok_f) old[nt][1] = out[(size_t)m1 * p.ldc + rf];
            if (m0 < p.M && ok_s) old[nt][2] = out[(size_t)m0 * p.ldc + rs];
            if (m1 < p.M && ok_s) old[nt][3] = out[(size_t)m1 * p.ldc + rs];
        }
    }
    // ROPE_APPEND: positions, rotation factors and cache pages of the two step rows this
    // thread will finish.
    int pos2[2 * MT], page2[2 * MT];
    float cs2[2 * MT], sn2[2 * MT];
#pragma unroll
    for (int e = 0; e < 2 * MT; ++e) {
        pos2[e] = page2[e] = 0;
        cs2[e] = 1.f;
        sn2[e] = 0.f;
    }
    if (EPI == ROPE_APPEND && warp == 0 && ok_f) {
        const int half = p.head_dim >> 1;
        const int pair = tile * 8 + g;
        const int head = pair / half, j = pair - head * half;
#pragma unroll
        for (int e = 0; e < 2 * MT; ++e) {
            const int m = (e >> 1) * 8 + 2 * t + (e & 1);
            if (m < p.M) {
                pos2[e] = p.positions[m];
                if (head >= p.n_heads)
                    page2[e] = p.block_table[(size_t)p.row_request[m] * p.table_stride +
                                             pos2[e] / p.page_tokens];
                if (head < p.n_heads + p.n_kv_heads) {
                    cs2[e] = p.cos_t[(size_t)pos2[e] * half + j];
                    sn2[e] = p.sin_t[(size_t)pos2[e] * half + j];
                }
            }
        }
    }
    // ---- stage the step's rows in shared memory as bf16 (normalised if asked) -------------
    if (NORM_IN) {
        // each of four warps normalises rows `warp` and `warp + 4` side by side (of eight
        // warps each takes one row); for widths up to
        // 1024 both rows and the gain stay in registers between the two passes, so the
        // whole staging is one round trip
        const int n4 = K >> 2;
        const float4* g4 = reinterpret_cast<const float4*>(p.gain);
        // one group of 8 rows after the other
#pragma unroll 1
        for (int grp = 0; grp < MT; ++grp) {
            const int ma = grp * 8 + warp, mb = ma + WARPS;
            const bool has_a = ma < p.M, has_b = WARPS == 4 && mb < p.M;
            const float4* row_a = reinterpret_cast<const float4*>(p.x + (size_t)(has_a ? ma : 0) * K);
            const float4* row_b = reinterpret_cast<const float4*>(p.x + (size_t)(has_b ? mb : 0) * K);
            uint2* dst_a = reinterpret_cast<uint2*>(xs + (size_t)ma * pitch);
            uint2* dst_b = reinterpret_cast<uint2*>(xs + (size_t)mb * pitch);
            constexpr int J = 8;
            const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
            if (n4 <= 32 * J) {
                float4 va[J], vb[J], gn[J];
    #pragma unroll
                for (int j = 0; j < J; ++j) {
                    const int i = lane + 32 * j;
                    const bool in = i < n4;
                    va[j] = (in && has_a) ? row_a[i] : zero4;
                    vb[j] = (in && has_b) ? row_b[i] : zero4;
                    gn[j] = in ? g4[i] : zero4;
                }
                float ss_a = 0.f, ss_b = 0.f;
    #pragma unroll
                for (int j = 0; j < J; ++j) {
                    ss_a = fmaf(va[j].x, va[j].x, ss_a); ss_a = fmaf(va[j].y, va[j].y, ss_a);
                    ss_a = fmaf(va[j].z, va[j].z, ss_a); ss_a = fmaf(va[j].w, va[j].w, ss_a);
                    ss_b = fmaf(vb[j].x, vb[j].x, ss_b); ss_b = fmaf(vb[j].y, vb[j].y, ss_b);
                    ss_b = fmaf(vb[j].z, vb[j].z, ss_b); ss_b = fmaf(vb[j].w, vb[j].w, ss_b);
                }
                ss_a = cb_warp_sum(ss_a);
                ss_b = cb_warp_sum(ss_b);
                const float r_a = 1.0f / sqrtf(ss_a / (float)K + p.eps);
                const float r_b = 1.0f / sqrtf(ss_b / (float)K + p.eps);
    #pragma unroll
                for (int j = 0; j < J; ++j) {
                    const int i = lane + 32 * j;
                    if (i < n4) {
                        dst_a[i] = make_uint2(pack2(va[j].x * r_a * gn[j].x, va[j].y * r_a * gn[j].y),
                                              pack2(va[j].z * r_a * gn[j].z, va[j].w * r_a * gn[j].w));
                        if (WARPS == 4)                     // with eight warps a warp has one row
                            dst_b[i] = make_uint2(pack2(vb[j].x * r_b * gn[j].x, vb[j].y * r_b * gn[j].y),
                                                  pack2(vb[j].z * r_b * gn[j].z, vb[j].w * r_b * gn[j].w));
                    }
                }
            } else {
                float ss_a = 0.f, ss_b = 0.f;
                if (has_a) {
    #pragma unroll 4
                    for (int j = lane; j < n4; j += 32) {
                        const float4 va = row_a[j];
                        const float4 vb = has_b ? row_b[j] : zero4;
                        ss_a = fmaf(va.x, va.x, ss_a); ss_a = fmaf(va.y, va.y, ss_a);
                        ss_a = fmaf(va.z, va.z, ss_a); ss_a = fmaf(va.w, va.w, ss_a);
                        ss_b = fmaf(vb.x, vb.x, ss_b); ss_b = fmaf(vb.y, vb.y, ss_b);
                        ss_b = fmaf(vb.z, vb.z, ss_b); ss_b = fmaf(vb.w, vb.w, ss_b);
                    }
                }
                ss_a = cb_warp_sum(ss_a);
                ss_b = cb_warp_sum(ss_b);
                const float r_a = 1.0f / sqrtf(ss_a / (float)K + p.eps);
                const float r_b = 1.0f / sqrtf(ss_b / (float)K + p.eps);
    #pragma unroll 4
                for (int j = lane; j < n4; j += 32) {
                    uint2 oa = make_uint2(0, 0), ob = make_uint2(0, 0);
                    if (has_a) {
                        const float4 gn = g4[j];
                        const float4 va = row_a[j];
                        oa = make_uint2(pack2(va.x * r_a * gn.x, va.y * r_a * gn.y),
                                        pack2(va.z * r_a * gn.z, va.w * r_a * gn.w));
                        if (has_b) {
                            const float4 vb = row_b[j];
                            ob = make_uint2(pack2(vb.x * r_b * gn.x, vb.y * r_b * gn.y),
                                            pack2(vb.z * r_b * gn.z, vb.w * r_b * gn.w));
                        }
                    }
                    dst_a[j] = oa;
                    if (WARPS == 4) dst_b[j] = ob;
                }
            }
        }
    } else {
        // bf16 rows go to shared memory as they are: asynchronous 16-byte copies, all in
        // flight at once; rows past the step's last are zero-filled
        const int n8 = K >> 3;
        for (int i = threadIdx.x; i < 8 * MT * n8; i += blockDim.x) {
            const int m = i / n8, c = i - m * n8;
            const bool in = m < p.M;
            const __nv_bfloat16* src = p.a + (size_t)(in ? m : 0) * p.lda + c * 8;
            const uint32_t dst = (uint32_t)__cvta_generic_to_shared(xs + (size_t)m * pitch + c * 8);
            const int bytes = in ? 16 : 0;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src),
                         "r"(bytes) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    // the step's rows are staged and this block's weights are on their way: the kernel after
    // this one may start and ask for its own
    if (!p.trigger_early) cb_pdl_trigger();
    // ---- multiply: this warp's blocks of K -------------------------------------------------
    float c[MT][4];
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) c[nt][0] = c[nt][1] = c[nt][2] = c[nt][3] = 0.f;
    const __nv_bfloat16* xrow = xs + (size_t)g * pitch + t * 8;
    for (int kb0 = 0; kb0 < k_blocks; kb0 += BATCH * WARPS) {
        const bool more = DEEP && kb0 + BATCH * WARPS < k_blocks;    // block-uniform
        uint4 nf[DEEP ? BATCH : 1], ns[DEEP ? BATCH : 1];
        if (DEEP) {
            if (more) {
#pragma unroll
                for (int i = 0; i < BATCH; ++i) {
                    const int kb = kb0 + BATCH * WARPS + warp + i * WARPS;
                    const bool in = kb < k_blocks && kb * 32 + t * 8 < K;
                    nf[i] = in ? __ldg(reinterpret_cast<const uint4*>(wf + kb * 32)) : make_uint4(0, 0, 0, 0);
                    ns[i] = in ? __ldg(reinterpret_cast<const uint4*>(ws + kb * 32)) : make_uint4(0, 0, 0, 0);
                }
            }
        } else if (kb0 > 0) {
#pragma unroll
            for (int i = 0; i < BATCH; ++i) {
                const int kb = kb0 + warp + i * WARPS;
                const bool in = kb < k_blocks && kb * 32 + t * 8 < K;
                vf[i] = in ? __ldg(reinterpret_cast<const uint4*>(wf + kb * 32)) : make_uint4(0, 0, 0, 0);
                vs[i] = in ? __ldg(reinterpret_cast<const uint4*>(ws + kb * 32)) : make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int i = 0; i < BATCH; ++i) {
            const int kb = kb0 + warp + i * WARPS;
            if (kb < k_blocks) {                          // warp-uniform
#pragma unroll
                for (int nt = 0; nt < MT; ++nt) {
                    uint4 xb = make_uint4(0, 0, 0, 0);
                    if (kb * 32 + t * 8 < K)
                        xb = *reinterpret_cast<const uint4*>(xrow + (size_t)nt * 8 * pitch + kb * 32);
                    mma_bf16(c[nt], vf[i].x, vs[i].x, vf[i].y, vs[i].y, xb.x, xb.y);
                    mma_bf16(c[nt], vf[i].z, vs[i].z, vf[i].w, vs[i].w, xb.z, xb.w);
                }
            }
        }
        if (DEEP && more) {
#pragma unroll
            for (int i = 0; i < BATCH; ++i) {
                vf[i] = nf[i];
                vs[i] = ns[i];
            }
        }
    }
    // ---- add the warps' partial sums in warp order; warp 0 finishes ------------------------
#pragma unroll
    for (int nt = 0; nt < MT; ++nt)
        reinterpret_cast<float4*>(red)[(warp * MT + nt) * 32 + lane] =
            make_float4(c[nt][0], c[nt][1], c[nt][2], c[nt][3]);
    __syncthreads();
    if (warp != 0) return;
#pragma unroll
    for (int nt = 0; nt < MT; ++nt) {
        float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float4 v = reinterpret_cast<const float4*>(red)[(w * MT + nt) * 32 + lane];
            d[0] += v.x; d[1] += v.y; d[2] += v.z; d[3] += v.w;
        }
        // d[0], d[1]: first row x step rows 8 nt + 2t, + 1;  d[2], d[3]: partner row x the same
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const int m = nt * 8 + 2 * t + e;
            if (m >= p.M) continue;
            const float df = d[e], ds = d[2 + e];
            if (EPI == ACCUM_F32 || EPI == STORE_F32) {
                float* out = (float*)p.out + (size_t)m * p.ldc;
                if (ok_f) out[rf] = EPI == ACCUM_F32 ? old[nt][e] + df : df;
                if (ok_s) out[rs] = EPI == ACCUM_F32 ? old[nt][2 + e] + ds : ds;
            } else if (EPI == SWIGLU_BF16) {
                if (ok_f)
                    ((__nv_bfloat16*)p.out)[(size_t)m * p.ldc + rf] =
                        __float2bfloat16_rn(df / (1.0f + expf(-df)) * ds);
            } else if (ok_f) {
                const int half = p.head_dim >> 1;
                const int pair = tile * 8 + g;
                const int head = pair / half, j = pair - head * half;
                const int pos = pos2[2 * nt + e];
                const float y0 = df * cs2[2 * nt + e] - ds * sn2[2 * nt + e];   // v heads keep cos 1, sin 0
                const float y1 = df * sn2[2 * nt + e] + ds * cs2[2 * nt + e];
                if (head < p.n_heads) {
                    __nv_bfloat16* q = (__nv_bfloat16*)p.out + (size_t)m * p.ldc + (size_t)head * p.head_dim;
                    q[j] = __float2bfloat16_rn(y0);
                    q[j + half] = __float2bfloat16_rn(y1);
                } else {
                    const bool is_k = head < p.n_heads + p.n_kv_heads;
                    const int kvh = is_k ? head - p.n_heads : head - p.n_heads - p.n_kv_heads;
                    __nv_bfloat16* dst = (is_k ? p.k_cache : p.v_cache) +
                        (((size_t)page2[2 * nt + e] * p.n_kv_heads + kvh) * p.page_tokens + pos % p.page_tokens) *
                            p.head_dim;
                    dst[j] = __float2bfloat16_rn(y0);
                    dst[j + half] = __float2bfloat16_rn(y1);
                }
            }
        }
    }
}

template <bool NORM_IN, int EPI, bool DEEP, int WARPS, int MT>
int launch_rows_as(const SmallParams& p, cudaStream_t s) {
    const int smem = 8 * MT * (p.K + 32) * 2 + WARPS * MT * 32 * 16;
    static int configured = 0;
    if (smem > 48 * 1024 && smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(small_linear_kernel<NORM_IN, EPI, DEEP, WARPS, MT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    // started under the kernel before it for up to 16 rows (measured: beyond, it loses)
    cb_launch_ex(small_linear_kernel<NORM_IN, EPI, DEEP, WARPS, MT>, dim3(p.n_tiles), dim3(WARPS * 32), smem,
                 s, 1, MT <= 2, p);
    return cb_last_error();
}

template <bool NORM_IN, int EPI, int MT>
int launch_rows_mt(const SmallParams& p, cudaStream_t s) {
    // A warp takes one batch of 8 blocks of 32 elements at a time.  K up to 1024: four warps,
    // one batch each.  Up to 2048: eight warps, still one batch each (the chain of round trips
    // stays as short).  Beyond: eight warps with two batches in flight.
    if (p.K <= BATCH * 4 * 32) return launch_rows_as<NORM_IN, EPI, false, 4, MT>(p, s);
    if (p.K <= BATCH * 8 * 32) return launch_rows_as<NORM_IN, EPI, false, 8, MT>(p, s);
    return launch_rows_as<NORM_IN, EPI, true, 8, MT>(p, s);
}

// More than 8 rows: in two or four groups of 8.
template <bool NORM_IN, int EPI>
int launch_rows(const SmallParams& p, cudaStream_t s) {
    if (p.M <= 8) return launch_rows_mt<NORM_IN, EPI, 1>(p, s);
    if (p.M <= 16) return launch_rows_mt<NORM_IN, EPI, 2>(p, s);
    return launch_rows_mt<NORM_IN, EPI, 4>(p, s);
}

bool sizes_ok(const float* x, const float* gain, const void* a, int lda, int M, int K, int ldw,
              const void* w) {
    if (x ? (((uintptr_t)x & 15) || ((uintptr_t)gain & 15)) : (((uintptr_t)a & 15) || (lda & 7)))
        return false;
    const int groups = M <= 8 ? 1 : (M <= 16 ? 2 : 4);
    return M >= 1 && M <= 32 && K > 0 && (K & 7) == 0 && (ldw & 7) == 0 &&
           ((uintptr_t)w & 15) == 0 && (size_t)8 * groups * (K + 32) * 2 <= 200 * 1024;
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
    p.n_tiles = (N + 15) / 16; p.out = out; p.ldc = ldc;
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
    p.n_tiles = (inter + 7) / 8; p.out = out; p.ldc = ldc;
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
    p.n_tiles = (heads * (head_dim / 2) + 7) / 8;
    p.out = q_out; p.ldc = ldq;
    p.cos_t = cos_t; p.sin_t = sin_t; p.positions = positions; p.row_request = row_request;
    p.block_table = block_table; p.table_stride = table_stride;
    p.k_cache = (__nv_bfloat16*)k_cache; p.v_cache = (__nv_bfloat16*)v_cache;
    p.n_heads = n_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim;
    p.page_tokens = page_tokens; p.write_cache = write_cache;
    p.trigger_early = 1;
    cudaStream_t s = (cudaStream_t)stream;
    return x ? launch_rows<true, ROPE_APPEND>(p, s) : launch_rows<false, ROPE_APPEND>(p, s);
}
