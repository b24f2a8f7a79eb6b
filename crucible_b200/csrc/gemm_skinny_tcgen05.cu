// C[M,N] = A[M,K] . W[N,K]^T for few rows (M <= 64: decoded tokens), bfloat16 on
// tcgen05 with the operands swapped: 128 rows of W are the M side of the MMA
// and the (zero-padded) rows of A are its N side (16, 32 or 64), so no tensor
// work is spent on padding 128 activation rows.  Such a product only streams
// W once, so what matters is how many blocks pull on memory at a time: the K
// range is split over `splits` blocks per 128-row tile of W.  Every block
// writes its partial tile to scratch; the block that arrives last at the tile's
// counter (an atomic, no block ever waits for another) sums the partials in
// ascending split order -- so the result does not depend on which block was
// last -- and applies the epilogue:
//   STORE_BF16, STORE_F32, ACCUM_F32 (fp32 residual add), SWIGLU_BF16 (the tile
//   holds 64 gate rows and the 64 matching up rows of W = [Wg; Wu]).
// With splits == 1 nothing goes through scratch.
//
// Scratch: floats [n_tiles][splits][MT][128] and ints [n_tiles] that are zero
// before the launch and zero again after it.
// Sizes: any N, M <= 64; K and the row strides multiples of 8, bases 16-byte
// aligned (TMA); otherwise refused.
// Reference counterpart: the batched GEMV family `gemv_batch_i8_b*`
// (engine/kernels/kernels.cu:1598-1607): read W once for all rows.
#define CB_PDL_BIT 5      // this file's bit in CRUCIBLE_PDL
#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int WM = 128;                // rows of W per block
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES_SHARED = 4;        // 72-96 KB a block: up to three blocks share an SM
constexpr int STAGES_ALONE = 8;         // 144-192 KB: a block that has its SM to itself

enum Epilogue { STORE_BF16 = 0, STORE_F32 = 1, ACCUM_F32 = 2, SWIGLU_BF16 = 3 };

template <int MT, int STAGES>
struct SkinnyStorage {
    alignas(1024) uint8_t w[STAGES][WM * BK * 2];
    alignas(1024) uint8_t a[STAGES][MT * BK * 2];
    alignas(8) uint64_t full_bar[STAGES];
    uint64_t empty_bar[STAGES];
    uint64_t tmem_full_bar;
    uint32_t tmem_base;
    int abort_flag;
    int is_last;
};

template <int MT>
__device__ __forceinline__ void load_acc(uint32_t taddr, float (&v)[MT]) {
    if constexpr (MT == 16) {
        uint32_t r[16];
        tc::tmem_ld_32x16(taddr, r);
        tc::tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
    } else {
#pragma unroll
        for (int c = 0; c < MT; c += 32) {
            uint32_t r[32];
            tc::tmem_ld_32x32(taddr + c, r);
            tc::tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[c + i] = __uint_as_float(r[i]);
        }
    }
}

template <int MT, int EPI, int STAGES>
__global__ void __launch_bounds__(192)
gemm_skinny_kernel(const __grid_constant__ CUtensorMap map_w,
                   const __grid_constant__ CUtensorMap map_a, void* __restrict__ c_ptr, int M,
                   int N, int K, int ldc, int inter, int splits, float* __restrict__ partial,
                   int* __restrict__ counters, int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    using Storage = SkinnyStorage<MT, STAGES>;
    Storage& s = *reinterpret_cast<Storage*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tile = blockIdx.x, split = blockIdx.y;
    const int k_blocks = (K + BK - 1) / BK;
    const int per = (k_blocks + splits - 1) / splits;
    const int kb0 = split * per;
    const int kb1 = min(k_blocks, kb0 + per);
    const int n_kb = max(0, kb1 - kb0);
    volatile int* abort_flag = &s.abort_flag;
    constexpr uint32_t TMEM_COLS = MT < 32 ? 32 : MT;
    constexpr uint32_t STAGE_BYTES = (WM + MT) * BK * 2;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            tc::mbar_init(&s.full_bar[i], 1);
            tc::mbar_init(&s.empty_bar[i], 1);
        }
        tc::mbar_init(&s.tmem_full_bar, 1);
        s.abort_flag = 0;
        s.is_last = 0;
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&map_w);
        tc::prefetch_tensormap(&map_a);
    }
    if (warp == 1) {
        tc::tmem_alloc(&s.tmem_base, TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_acc = s.tmem_base;
    auto load_w = [&](int i, int st) {
        const int kx = (kb0 + i) * BK;
        if (EPI == SWIGLU_BF16) {
            tc::tma_load_2d(s.w[st], &map_w, &s.full_bar[st], kx, tile * (WM / 2));
            tc::tma_load_2d(s.w[st] + (WM / 2) * BK * 2, &map_w, &s.full_bar[st], kx,
                            inter + tile * (WM / 2));
        } else {
            tc::tma_load_2d(s.w[st], &map_w, &s.full_bar[st], kx, tile * WM);
        }
    };
    // Barriers, tensor memory and descriptors are ready.  The first stages' tiles of W go out
    // now (a weight matrix, which no kernel of the stream writes); the step's rows are the
    // output of the kernels before this one and wait for them.
    const int w_ahead = n_kb < STAGES ? n_kb : STAGES;
    if (warp == 0 && lane == 0) {
        for (int i = 0; i < w_ahead; ++i) {
            tc::mbar_expect_tx(&s.full_bar[i], STAGE_BYTES);
            load_w(i, i);
        }
    }
    cb_pdl_wait();
    cb_pdl_trigger();

    if (warp == 0) {
        if (lane == 0) {
            // (the stage and its parity are carried along: a division by a run-time value
            // costs a lone thread about as much as two boxes)
            int armed = w_ahead, st = 0;
            uint32_t parity = 1;                // of the stage's last round, once there was one
            for (int i = 0; i < n_kb; ++i) {
                if (i >= STAGES && !tc::mbar_wait(&s.empty_bar[st], parity, abort_flag)) {
                    tc::give_up(abort_flag, status, tc::ST_PRODUCER_TIMEOUT);
                    break;
                }
                if (i >= w_ahead) {
                    tc::mbar_expect_tx(&s.full_bar[st], STAGE_BYTES);
                    load_w(i, st);
                }
                tc::tma_load_2d(s.a[st], &map_a, &s.full_bar[st], (kb0 + i) * BK, 0);
                if (i + 1 > armed) armed = i + 1;
                if (++st == STAGES) st = 0, parity ^= 1;
            }
            if (*abort_flag) {
                const int first = armed > STAGES ? armed - STAGES : 0;
                for (int i = first; i < armed; ++i)
                    for (uint32_t t = 0; t < tc::WAIT_LIMIT; ++t)
                        if (tc::mbar_try_wait(&s.full_bar[i % STAGES], (i / STAGES) & 1)) break;
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // One thread, whose own instructions are what a step of K takes with tiles this
            // narrow (a block that has its SM to itself streams what this loop can hand on);
            // so the ring is walked by an unrolled loop in which a stage's barriers and
            // descriptors are constants away from those of stage 0.
            constexpr uint32_t idesc = tc::instr_desc_bf16(WM, MT);
            constexpr uint32_t W_STEP = sizeof(s.w[0]) >> 4, A_STEP = sizeof(s.a[0]) >> 4;
            const uint64_t desc0 = tc::smem_desc_sw128(tc::smem_u32(s.w[0]));
            const uint32_t desc_hi = (uint32_t)(desc0 >> 32);
            const uint32_t w_lo = (uint32_t)desc0;
            const uint32_t a_lo = (uint32_t)tc::smem_desc_sw128(tc::smem_u32(s.a[0]));
            const uint32_t full0 = tc::smem_u32(&s.full_bar[0]), empty0 = tc::smem_u32(&s.empty_bar[0]);
            bool ok = true;
            uint32_t phase = 0;
            for (int i0 = 0; i0 < n_kb && ok; i0 += STAGES, phase ^= 1) {
#pragma unroll
                for (int st = 0; st < STAGES; ++st) {
                    if (i0 + st >= n_kb) break;
                    if (!tc::mbar_wait_at(full0 + 8 * st, phase, abort_flag)) {
                        tc::give_up(abort_flag, status, tc::ST_MMA_TIMEOUT);
                        ok = false;
                        break;
                    }
                    tc::tc_fence_after_sync();
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t w_desc = tc::desc_of(w_lo + st * W_STEP + 2 * k, desc_hi);
                        const uint64_t a_desc = tc::desc_of(a_lo + st * A_STEP + 2 * k, desc_hi);
                        if (st == 0 && k == 0)
                            tc::umma_bf16(tmem_acc, w_desc, a_desc, idesc, i0 > 0 ? 1u : 0u);
                        else
                            tc::umma_bf16_add(tmem_acc, w_desc, a_desc, idesc);
                    }
                    tc::umma_commit_at(empty0 + 8 * st);
                }
            }
            if (ok && n_kb > 0) tc::umma_commit(&s.tmem_full_bar);
        }
    }

    // ---- epilogue: warps 2..5 own the four lane quarters of the accumulator --------
    const bool epi_warp = warp >= 2;
    const int quarter = warp & 3;
    const int w_row = quarter * 32 + lane;              // row of the W tile = accumulator lane
    float acc[MT];
#pragma unroll
    for (int i = 0; i < MT; ++i) acc[i] = 0.f;
    // ACCUM_F32: the values to add to are asked for now, while the products run (every
    // block asks: which one writes is not known yet, and a tile's values are 8 KB from the L2)
    constexpr bool EARLY = EPI == ACCUM_F32 && MT <= 32;      // (64 values more would cost a block per SM)
    float add_to[EARLY ? MT : 1];
    if (EARLY && epi_warp && tile * WM + w_row < N) {
        const float* src = (const float*)c_ptr + tile * WM + w_row;
#pragma unroll
        for (int m = 0; m < MT; ++m) add_to[m] = m < M ? __ldcg(src + (size_t)m * ldc) : 0.f;
    }
    bool ok = true;
    if (epi_warp && n_kb > 0) {
        ok = tc::mbar_wait(&s.tmem_full_bar, 0, abort_flag);
        if (!ok && !*abort_flag) tc::give_up(abort_flag, status, tc::ST_EPILOGUE_TIMEOUT);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tc::tc_fence_after_sync();
            load_acc<MT>(tmem_acc + ((uint32_t)(quarter * 32) << 16), acc);
        }
    }
    if (splits > 1) {
        // every block leaves its partial; the last to arrive sums them all
        float* mine = partial + ((size_t)tile * splits + split) * MT * WM;
        if (epi_warp) {
#pragma unroll
            for (int m = 0; m < MT; ++m)
                if (m < M) mine[m * WM + w_row] = acc[m];
        }
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            const int prev = atomicAdd(&counters[tile], 1);
            s.is_last = prev == splits - 1;
        }
        __syncthreads();
        if (s.is_last && epi_warp) {
            __threadfence();
            const float* base = partial + (size_t)tile * splits * MT * WM;
#pragma unroll
            for (int m = 0; m < MT; ++m) acc[m] = 0.f;
            // summed in ascending order of the splits whichever block came last; the loads of
            // four splits are on their way at a time (a trip to the L2 each, otherwise)
            constexpr int AT_ONCE = MT <= 16 ? 4 : (MT <= 32 ? 2 : 1);
            for (int sp0 = 0; sp0 < splits; sp0 += AT_ONCE) {
                float part[AT_ONCE][MT];
#pragma unroll
                for (int u = 0; u < AT_ONCE; ++u) {
                    const float* src = base + (size_t)(sp0 + u) * MT * WM + w_row;
#pragma unroll
                    for (int m = 0; m < MT; ++m)
                        part[u][m] = (sp0 + u < splits && m < M) ? __ldcg(src + m * WM) : 0.f;
                }
#pragma unroll
                for (int u = 0; u < AT_ONCE; ++u)
#pragma unroll
                    for (int m = 0; m < MT; ++m) acc[m] += part[u][m];
            }
        }
        if (s.is_last && threadIdx.x == 0) counters[tile] = 0;    // ready for the next launch
    }
    const bool writer = (splits == 1 || s.is_last) && ok && !*abort_flag;
    if (EPI == SWIGLU_BF16) {
        // lanes 0..63 of the tile are gate rows, 64..127 the matching up rows
        float* xch = reinterpret_cast<float*>(s.w[0]);         // [64][MT], the stages are idle now
        __syncthreads();
        if (writer && epi_warp && w_row >= WM / 2) {
#pragma unroll
            for (int m = 0; m < MT; ++m) xch[(w_row - WM / 2) * MT + m] = acc[m];
        }
        __syncthreads();
        if (writer && epi_warp && w_row < WM / 2) {
            const int col = tile * (WM / 2) + w_row;
            if (col < inter) {
                __nv_bfloat16* C = (__nv_bfloat16*)c_ptr;
#pragma unroll
                for (int m = 0; m < MT; ++m) {
                    if (m < M) {
                        const float g = acc[m], u = xch[w_row * MT + m];
                        C[(size_t)m * ldc + col] = __float2bfloat16_rn(tc::silu_fast(g) * u);
                    }
                }
            }
        }
    } else if (writer && epi_warp) {
        const int col = tile * WM + w_row;
        if (col < N) {
            if (EARLY) {
#pragma unroll
                for (int m = 0; m < MT; ++m) acc[m] += add_to[m];
            } else if (EPI == ACCUM_F32) {
                const float* src = (const float*)c_ptr + col;
#pragma unroll
                for (int m = 0; m < MT; ++m)
                    if (m < M) acc[m] += __ldcg(src + (size_t)m * ldc);
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                if (m < M) {
                    if (EPI == STORE_BF16)
                        ((__nv_bfloat16*)c_ptr)[(size_t)m * ldc + col] = __float2bfloat16_rn(acc[m]);
                    else
                        ((float*)c_ptr)[(size_t)m * ldc + col] = acc[m];
                }
            }
        }
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::tc_fence_after_sync();
        tc::tmem_dealloc(tmem_acc, TMEM_COLS);
    }
}

template <int MT, int EPI, int STAGES>
int launch_stages(const CUtensorMap& mw, const CUtensorMap& ma, void* C, int M, int N, int K, int ldc,
                  int inter, int n_tiles, int splits, float* partial, int* counters, int* status,
                  cudaStream_t stream) {
    const int smem = (int)sizeof(SkinnyStorage<MT, STAGES>) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(gemm_skinny_kernel<MT, EPI, STAGES>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cb_launch(gemm_skinny_kernel<MT, EPI, STAGES>, dim3(n_tiles, splits), dim3(192), smem, stream,
        mw, ma, C, M, N, K, ldc, inter, splits, partial, counters, status);
    return cb_last_error();
}

// A block keeps STAGES tiles of W on their way, and what one block streams is that many
// bytes per trip to memory and back (about 1.2 us with the hand-over between the threads): 53
// GB/s with four stages.  A launch of at most one block per SM gets eight.
template <int MT, int EPI>
int launch(const CUtensorMap& mw, const CUtensorMap& ma, void* C, int M, int N, int K, int ldc,
           int inter, int n_tiles, int splits, float* partial, int* counters, int* status,
           cudaStream_t stream) {
    static int n_sms = 0;
    if (n_sms == 0) {
        int dev = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&n_sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            n_sms = 1;
    }
    const int k_blocks = (K + BK - 1) / BK;
    if ((long)n_tiles * splits <= n_sms && k_blocks > STAGES_SHARED * splits)
        return launch_stages<MT, EPI, STAGES_ALONE>(mw, ma, C, M, N, K, ldc, inter, n_tiles, splits, partial,
                                                    counters, status, stream);
    return launch_stages<MT, EPI, STAGES_SHARED>(mw, ma, C, M, N, K, ldc, inter, n_tiles, splits, partial,
                                                 counters, status, stream);
}

template <int MT>
int launch_epi(int epi, const CUtensorMap& mw, const CUtensorMap& ma, void* C, int M, int N, int K,
               int ldc, int inter, int n_tiles, int splits, float* partial, int* counters,
               int* status, cudaStream_t s) {
    switch (epi) {
        case STORE_BF16: return launch<MT, STORE_BF16>(mw, ma, C, M, N, K, ldc, inter, n_tiles, splits, partial, counters, status, s);
        case STORE_F32: return launch<MT, STORE_F32>(mw, ma, C, M, N, K, ldc, inter, n_tiles, splits, partial, counters, status, s);
        case ACCUM_F32: return launch<MT, ACCUM_F32>(mw, ma, C, M, N, K, ldc, inter, n_tiles, splits, partial, counters, status, s);
        case SWIGLU_BF16: return launch<MT, SWIGLU_BF16>(mw, ma, C, M, N, K, ldc, inter, n_tiles, splits, partial, counters, status, s);
    }
    return CB_ERR_UNSUPPORTED;
}

inline int padded_rows(int m) { return m <= 16 ? 16 : (m <= 32 ? 32 : 64); }

}  // namespace

// Tiles of 128 rows of W for this product (for SWIGLU_BF16, N = inter and W has 2N rows).
CB_EXPORT int cb_gemm_skinny_tiles(int N, int epi) {
    return epi == SWIGLU_BF16 ? (N + WM / 2 - 1) / (WM / 2) : (N + WM - 1) / WM;
}

// Bytes of scratch for partial tiles (the counters, one int per tile, are separate).
CB_EXPORT long cb_gemm_skinny_partial_bytes(int M, int N, int epi, int splits) {
    if (splits <= 1) return 0;
    return (long)cb_gemm_skinny_tiles(N, epi) * splits * padded_rows(M) * WM * 4;
}

CB_EXPORT int cb_gemm_skinny(const void* A, const void* W, void* C, int M, int N, int K, int lda,
                             int ldw, int ldc, int epi, int splits, float* partial, int* counters,
                             int* status, void* stream) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 64 || K <= 0 || (K & 7) || (lda & 7) || (ldw & 7) || ((uintptr_t)A & 15) ||
        ((uintptr_t)W & 15))
        return CB_ERR_UNSUPPORTED;
    const int k_blocks = (K + BK - 1) / BK;
    if (splits < 1) splits = 1;
    if (splits > k_blocks) splits = k_blocks;
    // no split may be empty: the last block must find every partial written
    while (splits > 1 && (splits - 1) * ((k_blocks + splits - 1) / splits) >= k_blocks) --splits;
    if (splits > 1 && (partial == nullptr || counters == nullptr)) return CB_ERR_UNSUPPORTED;
    const int mt = padded_rows(M);
    const int w_rows = epi == SWIGLU_BF16 ? 2 * N : N;
    const int box_rows = epi == SWIGLU_BF16 ? WM / 2 : WM;
    CUtensorMap mw, ma;
    if (!tc::make_map_2d(&mw, W, (uint64_t)w_rows, (uint64_t)K, (uint64_t)ldw, box_rows))
        return CB_ERR_UNSUPPORTED;
    if (!tc::make_map_2d(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, mt)) return CB_ERR_UNSUPPORTED;
    const int inter = epi == SWIGLU_BF16 ? N : 0;
    const int n_tiles = cb_gemm_skinny_tiles(N, epi);
    cudaStream_t s = (cudaStream_t)stream;
    switch (mt) {
        case 16: return launch_epi<16>(epi, mw, ma, C, M, N, K, ldc, inter, n_tiles, splits, partial, counters, status, s);
        case 32: return launch_epi<32>(epi, mw, ma, C, M, N, K, ldc, inter, n_tiles, splits, partial, counters, status, s);
        case 64: return launch_epi<64>(epi, mw, ma, C, M, N, K, ldc, inter, n_tiles, splits, partial, counters, status, s);
    }
    return CB_ERR_UNSUPPORTED;
}
