// C[M,N] = A[M,K] . W[N,K]^T in bfloat16 on the 5th-generation tensor cores:
// TMA brings 128 x 64 tiles of A and BN x 64 tiles of W into shared memory
// (128-byte swizzle), one thread issues tcgen05.mma (M = 128, N = BN, K = 16)
// into an fp32 accumulator in tensor memory, and four warps read it back with
// tcgen05.ld for the epilogue.  Roles: warp 0 loads, warp 1 owns tensor memory
// and issues the MMAs, warps 2-5 do the epilogue.  One output tile per block.
//
// Epilogues (fused where it saves memory traffic):
//   STORE_BF16  C bf16 = acc
//   STORE_F32   C fp32 = acc                      (logits)
//   ACCUM_F32   C fp32 += acc                     (residual add in 32 bits)
//   SWIGLU_BF16 W = [Wg; Wu] ([2I, K]); the tile holds BN/2 gate rows and the
//               BN/2 matching up rows; C[M, I] bf16 = silu(g) * u in fp32
//
// Many tiles and a long K (prompts at the larger layer sizes): 148 blocks of 128 x 256 ask
// the L2 for more operand bytes than it delivers (384 rows of operands per 128 x 256 of
// output).  MH = 2 gives a block two accumulators, 256 x 256 of output from 512 rows of
// operands: the W tile in shared memory meets two A tiles.  Three stages of 64 KB then, and
// all 512 columns of tensor memory; the output leaves through shared memory and TMA, half
// after half.
//
// Few tiles and a long K (a step of 33 to a few hundred rows): the blocks (x, y, 0..S-1)
// form a cluster that splits K.  Each multiplies its share into its own accumulator; the
// others then leave theirs in their shared memory, and block 0 of the cluster adds them
// to its own in the order of the shares (over distributed shared memory, so the order
// of the sum is fixed), writes the sums back to tensor memory and runs the epilogue.
//
// Sizes: any M, N; K a multiple of 8 (a TMA row stride must be a multiple of
// 16 bytes) with lda, ldw multiples of 8 and 16-byte aligned bases; tails in
// M, N and K are zero-filled by TMA and masked at the store.  Anything else is
// refused by the launcher (the caller then runs the CUDA-core product).
//
// Reference counterpart: `gemm_f32_wmma` (engine/kernels/kernels.cu:2420-2520),
// fp16 wmma tiles 16x64 / 64x64.
#define CB_PDL_BIT 0      // this file's bit in CRUCIBLE_PDL
#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int BM = 128;
constexpr int BK = 64;                 // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;

enum Epilogue { STORE_BF16 = 0, STORE_F32 = 1, ACCUM_F32 = 2, SWIGLU_BF16 = 3, ROPE_APPEND = 4 };

// ROPE_APPEND: W = [Wq; Wk; Wv]; a tile covers whole heads.  The q heads are rotated
// and stored (bf16) to C[M, ldc]; the k heads are rotated and the v heads copied into
// the rows' cache pages [page][kv_head][slot][head_dim].
struct RopeArgs {
    const float* cos_t;           // [positions][head_dim / 2]
    const float* sin_t;
    const int* positions;         // per row
    const int* row_request;
    const int* block_table;
    int table_stride;
    __nv_bfloat16* k_cache;
    __nv_bfloat16* v_cache;
    int n_heads, n_kv_heads, head_dim, page_tokens, write_cache;
};

// What a product knows of the RMS norm on either side of it.
//   After it (ACCUM_F32 as the rows' last write before a norm): with `gain` set the epilogue
//   also leaves bf16(x * gain) of the summed rows x in `scaled` and the tile's share of every
//   row's sum of squares in `sumsq_out` [tiles along N][M] (summed in the order of the
//   columns).  The tile of C comes into shared memory by TMA while the products run, so the
//   thread that holds a row's accumulators also has the values they are added to; C itself
//   still gets its sums by TMA adds, `scaled` leaves by TMA stores of 32-column boxes (a single
//   tile of rows: in 64-byte pieces of the threads' own rows).
//   Tiles up to 128 columns, N a multiple of 32.
//   Before it (any epilogue): with `sumsq_in` set the rows of A are bf16(x * gain) of rows
//   not yet divided by their root mean square; the epilogue sums a row's `parts` shares in
//   their order and multiplies the row's accumulators by 1 / sqrt(sum / width + eps), which
//   is the same product as with normalised rows up to the rounding of A.
struct NormArgs {
    const float* gain;
    __nv_bfloat16* scaled;
    float* sumsq_out;
    int ld_scaled;
    const float* sumsq_in;
    int parts;
    float width, eps;
};

template <int BN, int STAGES, int MH>
struct SharedStorage {
    alignas(1024) uint8_t a[STAGES][MH * BM * BK * 2];
    alignas(1024) uint8_t b[STAGES][BN * BK * 2];
    alignas(8) uint64_t full_bar[STAGES];
    uint64_t empty_bar[STAGES];
    uint64_t tmem_full_bar;
    uint64_t c_bar;             // a norm after the product: the tile of C has landed
    alignas(16) float gain[128];   // ... and the norm's gain for the tile's columns
    long row_base[BM];          // ROPE_APPEND: a row's first element in a cache page / head_dim, or -1
    uint32_t tmem_base;
    int abort_flag;
};

// NORM: what the product has to do with the norm around it, fixed when it is compiled so that
// the other forms carry none of its code (an epilogue runs once per block, its instructions
// come from memory, and a tenth more of them cost every product 0.4 us): NORM_NONE, NORM_PRE
// (the rows of A are ahead of their norm, `sumsq_in`), NORM_EMIT (`gain`: leave the next
// norm's input).
enum NormForm { NORM_NONE = 0, NORM_PRE = 1, NORM_EMIT = 2 };

template <int BN, int STAGES, int EPI, int MH, int NORM>
__global__ void __launch_bounds__(192, (STAGES <= 3 && MH == 1) ? 2 : 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a,
                    const __grid_constant__ CUtensorMap map_w,
                    const __grid_constant__ CUtensorMap map_c,
                    const __grid_constant__ CUtensorMap map_s, int tma_out,
                    void* __restrict__ c_ptr, int M, int N, int K, int ldc, int inter,
                    int k_splits, int* __restrict__ status, const RopeArgs ra, const NormArgs na) {
    extern __shared__ uint8_t smem_raw[];
    using Storage = SharedStorage<BN, STAGES, MH>;
    Storage& s = *reinterpret_cast<Storage*>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * BM * MH;
    const int n_tile = blockIdx.x;
    // this block's share of K: blocks of 64 elements [kb_first, kb_first + k_blocks)
    const uint32_t split = k_splits > 1 ? tc::cluster_rank() : 0u;
    const int k_blocks_all = (K + BK - 1) / BK;
    const int per_split = (k_blocks_all + k_splits - 1) / k_splits;
    const int kb_first = (int)split * per_split;
    const int k_blocks = min(per_split, k_blocks_all - kb_first);      // the launcher keeps it positive
    volatile int* abort_flag = &s.abort_flag;
    // tensor-memory columns are allocated in powers of two
    constexpr uint32_t TMEM_COLS = MH * BN <= 32 ? 32 : (MH * BN <= 64 ? 64 : (MH * BN <= 128 ? 128 : (MH * BN <= 256 ? 256 : 512)));
    constexpr uint32_t STAGE_BYTES = (MH * BM + BN) * BK * 2;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            tc::mbar_init(&s.full_bar[i], 1);
            tc::mbar_init(&s.empty_bar[i], 1);
        }
        tc::mbar_init(&s.tmem_full_bar, 1);
        tc::mbar_init(&s.c_bar, 1);
        s.abort_flag = 0;
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&map_a);
        tc::prefetch_tensormap(&map_w);
        if (tma_out) tc::prefetch_tensormap(&map_c);
        if (NORM == NORM_EMIT && M > BM) tc::prefetch_tensormap(&map_s);
    }
    if (warp == 1) {
        tc::tmem_alloc(&s.tmem_base, TMEM_COLS);
        tc::tmem_relinquish();
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    const uint32_t tmem_acc = s.tmem_base;
    constexpr bool PRE = NORM == NORM_PRE;
    auto load_w = [&](int kb, int st) {
        if (EPI == SWIGLU_BF16) {
            const int half = BN / 2;
            tc::tma_load_2d(s.b[st], &map_w, &s.full_bar[st], (kb_first + kb) * BK, n_tile * half);
            tc::tma_load_2d(s.b[st] + half * BK * 2, &map_w, &s.full_bar[st], (kb_first + kb) * BK,
                            inter + n_tile * half);
        } else {
            tc::tma_load_2d(s.b[st], &map_w, &s.full_bar[st], (kb_first + kb) * BK, n_tile * BN);
        }
    };
    // Barriers, tensor memory and descriptors are ready.  The first stages' tiles of W go out
    // now: W is a weight matrix, which no kernel of the stream writes, so these copies need
    // not wait for the kernels before this one; A is their output and does.
    const int w_ahead = k_blocks < STAGES ? k_blocks : STAGES;
    if (warp == 0 && lane == 0) {
        for (int kb = 0; kb < w_ahead; ++kb) {
            tc::mbar_expect_tx(&s.full_bar[kb], STAGE_BYTES);
            load_w(kb, kb);
        }
    }
    cb_pdl_wait();
    cb_pdl_trigger();

    // A norm after the product: the tile of C (32-column boxes in the 128-byte swizzle) comes
    // into its own piece of shared memory behind the stages, asked for by an epilogue thread
    // that has nothing else to do yet.  Only the block that runs the epilogue asks.
    const bool emit = NORM == NORM_EMIT && EPI == ACCUM_F32 && MH == 1 && BN <= 128 && split == 0;
    uint8_t* const c_tile = reinterpret_cast<uint8_t*>(&s) + ((sizeof(Storage) + 1023) & ~(size_t)1023);
    if (emit && warp >= 2) {
        // (read in the epilogue, behind a barrier of these four warps)
        const int i = threadIdx.x - 64;
        if (i < BN) s.gain[i] = n_tile * BN + i < N ? __ldg(na.gain + n_tile * BN + i) : 0.f;
    }
    if (emit && warp == 2 && lane == 0) {
        int boxes = 0;
        for (int c = 0; c < BN / 32; ++c) boxes += n_tile * BN + c * 32 < N;
        tc::mbar_expect_tx(&s.c_bar, (uint32_t)boxes * BM * 128);
        for (int c = 0; c < BN / 32; ++c)
            if (n_tile * BN + c * 32 < N)
                tc::tma_load_2d(c_tile + c * (BM * 128), &map_c, &s.c_bar, n_tile * BN + c * 32, m0);
    }

    if (warp == 0) {
        // ---- producer: one thread feeds the ring of stages -------------------
        if (lane == 0) {
            // (sending a box costs this thread about 60 cycles whatever the box's size, a division
            // by a run-time value a hundred, a dependent integer instruction about 5, so
            // the loop around it carries the stage and its parity along instead of dividing)
            int armed = w_ahead, st = 0;
            uint32_t parity = 1;                // of the stage's last round, once there was one
            for (int kb = 0; kb < k_blocks; ++kb) {
                if (kb >= STAGES && !tc::mbar_wait(&s.empty_bar[st], parity, abort_flag)) {
                    tc::give_up(abort_flag, status, tc::ST_PRODUCER_TIMEOUT);
                    break;
                }
                if (kb >= w_ahead) {
                    tc::mbar_expect_tx(&s.full_bar[st], STAGE_BYTES);
                    load_w(kb, st);
                }
#pragma unroll
                for (int mh = 0; mh < MH; ++mh)
                    tc::tma_load_2d(s.a[st] + mh * (BM * BK * 2), &map_a, &s.full_bar[st], (kb_first + kb) * BK,
                                    m0 + mh * BM);
                if (kb + 1 > armed) armed = kb + 1;
                if (++st == STAGES) st = 0, parity ^= 1;
            }
            if (*abort_flag) {
                // let our own copies land before the block's shared memory goes away
                const int first = armed > STAGES ? armed - STAGES : 0;
                for (int kb = first; kb < armed; ++kb) {
                    const int st = kb % STAGES;
                    for (uint32_t i = 0; i < tc::WAIT_LIMIT; ++i)
                        if (tc::mbar_try_wait(&s.full_bar[st], (kb / STAGES) & 1)) break;
                }
            }
        }
        if (k_splits > 1) {                 // the two barriers of the epilogue warps
            __syncwarp();
            tc::cluster_sync_all();
            tc::cluster_sync_all();
        }
    } else if (warp == 1) {
        // ---- MMA issuer --------------------------------------------------------
        // One thread, and for tiles up to 128 columns wide its own instructions are what a
        // step of K takes: sending a tcgen05.mma costs the thread about 54 cycles (the tensor
        // cores need 32 to 64 for 64 to 128 columns), a commit about 60, and every dependent
        // integer instruction of a lone thread about 5.  So the ring is walked by an unrolled
        // loop: a stage's barriers and operand descriptors are constants away from those of
        // stage 0 (the descriptor's low word carries the address in 16-byte units, its high
        // word is the same for every tile), and only the first MMA of the first stage asks
        // whether it accumulates.
        if (lane == 0) {
            constexpr uint32_t idesc = tc::instr_desc_bf16(BM, BN);
            constexpr uint32_t A_STEP = sizeof(s.a[0]) >> 4, B_STEP = sizeof(s.b[0]) >> 4;
            constexpr uint32_t A_HALF = (BM * BK * 2) >> 4;
            const uint64_t desc0 = tc::smem_desc_sw128(tc::smem_u32(s.a[0]));
            const uint32_t desc_hi = (uint32_t)(desc0 >> 32);
            const uint32_t a_lo = (uint32_t)desc0;
            const uint32_t b_lo = (uint32_t)tc::smem_desc_sw128(tc::smem_u32(s.b[0]));
            const uint32_t full0 = tc::smem_u32(&s.full_bar[0]), empty0 = tc::smem_u32(&s.empty_bar[0]);
            bool ok = true;
            uint32_t phase = 0;
            for (int kb0 = 0; kb0 < k_blocks && ok; kb0 += STAGES, phase ^= 1) {
#pragma unroll
                for (int st = 0; st < STAGES; ++st) {
                    if (kb0 + st >= k_blocks) break;
                    if (!tc::mbar_wait_at(full0 + 8 * st, phase, abort_flag)) {
                        tc::give_up(abort_flag, status, tc::ST_MMA_TIMEOUT);
                        ok = false;
                        break;
                    }
                    tc::tc_fence_after_sync();
#pragma unroll
                    for (int mh = 0; mh < MH; ++mh) {
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            // advancing 16 elements along K = 32 bytes = 2 descriptor units
                            const uint64_t a_desc = tc::desc_of(a_lo + st * A_STEP + mh * A_HALF + 2 * k, desc_hi);
                            const uint64_t b_desc = tc::desc_of(b_lo + st * B_STEP + 2 * k, desc_hi);
                            if (st == 0 && k == 0)
                                tc::umma_bf16(tmem_acc + mh * BN, a_desc, b_desc, idesc, kb0 > 0 ? 1u : 0u);
                            else
                                tc::umma_bf16_add(tmem_acc + mh * BN, a_desc, b_desc, idesc);
                        }
                    }
                    tc::umma_commit_at(empty0 + 8 * st);     // stage free once these MMAs are done
                }
            }
            if (ok) tc::umma_commit(&s.tmem_full_bar);   // accumulator complete
        }
        if (k_splits > 1) {
            __syncwarp();
            tc::cluster_sync_all();
            tc::cluster_sync_all();
        }
    } else {
        // ---- epilogue: warps 2..5, lane quarter = warp % 4 -----------------------
        const int quarter = warp & 3;
        const int row = m0 + quarter * 32 + lane;
        // ACCUM_F32: the values to add to are asked for now, while the products run; the
        // thread's whole row of the tile stays in registers (tiles up to 128 wide)
        constexpr bool EARLY = EPI == ACCUM_F32 && BN <= 128 && MH == 1;
        constexpr int NQ = EARLY ? BN / 4 : 1;
        float4 early[NQ];
        if (EARLY && !tma_out) {
            const bool vec = (ldc & 3) == 0 && row < M;
#pragma unroll
            for (int q = 0; q < NQ; ++q) {
                const int col = n_tile * BN + (q >> 3) * 32;          // the chunk of 32 columns
                early[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (vec && col + 32 <= N)
                    early[q] = __ldcg(reinterpret_cast<const float4*>((const float*)c_ptr +
                                                                      (size_t)row * ldc + col) + (q & 7));
            }
        }
        // ROPE_APPEND: the row's position and its place in the cache pages, asked for while
        // the products run; every epilogue thread publishes its row's place.  For head size 64
        // also its 32 rotation factors, kept in registers for every head.  (Per 128 rows: a
        // block with two accumulators does this again for its second half.)
        // rows not yet divided by their root mean square: the row's factor, from the shares of
        // its sum of squares (asked for while the products run)
        auto row_factor = [&](int at_row) -> float {
            if (!PRE || at_row >= M) return 1.f;
            float ss = 0.f;
#pragma unroll 4
            for (int t = 0; t < na.parts; ++t) ss += __ldcg(na.sumsq_in + (size_t)t * M + at_row);
            return 1.0f / sqrtf(ss / na.width + na.eps);
        };
        float rf[MH];
#pragma unroll
        for (int mh = 0; mh < MH; ++mh) rf[mh] = row_factor(row + mh * BM);
        int row_pos = 0;
        float4 cs_reg[8], sn_reg[8];
        auto rope_rows = [&](int at_row) {
            long base = -1;
            row_pos = 0;
            if (at_row < M) {
                row_pos = ra.positions[at_row];
                if (ra.write_cache) {
                    const int page = ra.block_table[(size_t)ra.row_request[at_row] * ra.table_stride +
                                                    row_pos / ra.page_tokens];
                    base = (long)page * ra.n_kv_heads * ra.page_tokens + row_pos % ra.page_tokens;
                }
            }
            s.row_base[quarter * 32 + lane] = base;
            if (ra.head_dim == 64) {
                const float4* cp = reinterpret_cast<const float4*>(ra.cos_t + (size_t)row_pos * 32);
                const float4* sp = reinterpret_cast<const float4*>(ra.sin_t + (size_t)row_pos * 32);
#pragma unroll
                for (int q4 = 0; q4 < 8; ++q4) {
                    cs_reg[q4] = __ldg(cp + q4);
                    sn_reg[q4] = __ldg(sp + q4);
                }
            }
        };
        if (EPI == ROPE_APPEND) rope_rows(row);
        bool ok = tc::mbar_wait(&s.tmem_full_bar, 0, abort_flag);
        if (!ok && !*abort_flag) tc::give_up(abort_flag, status, tc::ST_EPILOGUE_TIMEOUT);
        ok = __all_sync(0xffffffffu, ok);
        const uint32_t lane_addr = tmem_acc + ((uint32_t)(quarter * 32) << 16);
        if (k_splits > 1) {
            // Shares of K: a block other than the cluster's first leaves its accumulator in
            // its shared memory (the ring of stages is free by now) as [4 columns][row], so
            // that neighbouring threads touch neighbouring 16 bytes; the first block adds
            // the shares in their order and puts the sums back into tensor memory.
            float4* part = reinterpret_cast<float4*>(s.a[0]);
            const int r = quarter * 32 + lane;
            if (split != 0 && ok) {
                tc::tc_fence_after_sync();
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t v[32];
                    tc::tmem_ld_32x32(lane_addr + c0, v);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int q = 0; q < 8; ++q)
                        part[((c0 >> 2) + q) * BM + r] =
                            make_float4(__uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                                        __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
                }
            }
            tc::cluster_sync_all();
            if (split == 0 && ok) {
                // 16 columns at a time, and the loads from up to four other blocks go out together
                // (a round trip over the cluster's network per four blocks, not per block)
                tc::tc_fence_after_sync();
                const uint32_t mine = tc::smem_u32(part);
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    uint32_t v[16];
                    tc::tmem_ld_32x16(lane_addr + c0, v);
                    tc::tmem_ld_wait();
#pragma unroll 1
                    for (int sp0 = 1; sp0 < k_splits; sp0 += 4) {          // four blocks' loads at a time
                        float4 o[4][4];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (sp0 + i < k_splits) {
                                const uint32_t theirs = tc::cluster_map(mine, (uint32_t)(sp0 + i)) +
                                                        (uint32_t)(((c0 >> 2) * BM + r) * 16);
#pragma unroll
                                for (int q = 0; q < 4; ++q)
                                    o[i][q] = tc::cluster_ld_f4(theirs + (uint32_t)(q * BM * 16));
                            }
                        }
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            if (sp0 + i < k_splits) {
#pragma unroll
                                for (int q = 0; q < 4; ++q) {
                                    v[4 * q] = __float_as_uint(__uint_as_float(v[4 * q]) + o[i][q].x);
                                    v[4 * q + 1] = __float_as_uint(__uint_as_float(v[4 * q + 1]) + o[i][q].y);
                                    v[4 * q + 2] = __float_as_uint(__uint_as_float(v[4 * q + 2]) + o[i][q].z);
                                    v[4 * q + 3] = __float_as_uint(__uint_as_float(v[4 * q + 3]) + o[i][q].w);
                                }
                            }
                        }
                    }
                    tc::tmem_st_32x16(lane_addr + c0, v);
                }
                tc::tmem_st_wait();
            }
            tc::cluster_sync_all();          // the others' shared memory may go now
            if (split != 0) ok = false;      // the first block alone has the epilogue
        }
        if (ok) {
            tc::tc_fence_after_sync();
            if (EPI == ROPE_APPEND) {
                // A thread owns one token's row of the tile: whole heads of head_dim columns,
                // taken in pairs of 32-column chunks (j, j + head_dim / 2), rotated in
                // registers and staged in shared memory as [128 rows][128 bytes] per 64
                // columns (the ring of stages is free by now).  A q head then leaves by TMA;
                // a k or v head is copied to the rows' cache pages by all threads, a row's
                // 128 bytes as eight 16-byte pieces of neighbouring lanes.
                const int hd = ra.head_dim, half = hd >> 1;
                const int r = quarter * 32 + lane;
                const int heads_all = ra.n_heads + 2 * ra.n_kv_heads;
                const int chunks = hd >> 6;                         // 64-column chunks per head
                uint8_t* ring = s.a[0];
#pragma unroll 1
                for (int mh = 0; mh < MH; ++mh) {                   // one accumulator after the other
                if (mh > 0) {
                    // the staging buffers and the rows' places are used again: the first half's
                    // stores and copies must be done with them
                    if (warp == 2 && lane == 0) tc::tma_store_wait_read();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    rope_rows(row + mh * BM);
                }
                const uint32_t lane_addr_h = lane_addr + mh * BN;
                const int m0_h = m0 + mh * BM;
                const float f = mh == 0 ? rf[0] : rf[MH - 1];
                const float* cs_row = ra.cos_t + (size_t)row_pos * half;
                const float* sn_row = ra.sin_t + (size_t)row_pos * half;
#pragma unroll 1
                for (int hc = 0; hc < BN; hc += hd) {
                    const int head = (n_tile * BN + hc) / hd;
                    if (head >= heads_all) break;
                    const bool is_q = head < ra.n_heads, is_k = !is_q && head < ra.n_heads + ra.n_kv_heads;
                    uint8_t* buf = ring + (hc >> 6) * (BM * 128);
#pragma unroll 1
                    for (int c = 0; c < half; c += 32) {
                        uint32_t lo[32], hi[32];
                        tc::tmem_ld_32x32(lane_addr_h + hc + c, lo);
                        tc::tmem_ld_32x32(lane_addr_h + hc + half + c, hi);
                        tc::tmem_ld_wait();
                        if (PRE) {
#pragma unroll
                            for (int i = 0; i < 32; ++i) {
                                lo[i] = __float_as_uint(__uint_as_float(lo[i]) * f);
                                hi[i] = __float_as_uint(__uint_as_float(hi[i]) * f);
                            }
                        }
                        if (is_q || is_k) {
#pragma unroll
                            for (int q4 = 0; q4 < 8; ++q4) {
                                const float4 cs = hd == 64 ? cs_reg[q4]
                                                           : __ldg(reinterpret_cast<const float4*>(cs_row + c) + q4);
                                const float4 sn = hd == 64 ? sn_reg[q4]
                                                           : __ldg(reinterpret_cast<const float4*>(sn_row + c) + q4);
                                const float cc[4] = {cs.x, cs.y, cs.z, cs.w};
                                const float ss[4] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const float x1 = __uint_as_float(lo[4 * q4 + i]);
                                    const float x2 = __uint_as_float(hi[4 * q4 + i]);
                                    lo[4 * q4 + i] = __float_as_uint(x1 * cc[i] - x2 * ss[i]);
                                    hi[4 * q4 + i] = __float_as_uint(x1 * ss[i] + x2 * cc[i]);
                                }
                            }
                        }
                        // columns c.. and half + c.. of the head: which 64-column chunk, which pieces
                        uint8_t* lo_row = buf + (c >> 6) * (BM * 128) + r * 128;
                        uint8_t* hi_row = buf + ((half + c) >> 6) * (BM * 128) + r * 128;
                        const int lo_piece = (c & 63) >> 3, hi_piece = ((half + c) & 63) >> 3;
#pragma unroll
                        for (int q8 = 0; q8 < 4; ++q8) {
                            uint32_t pl[4], ph[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(lo[q8 * 8 + 2 * j]),
                                                                          __uint_as_float(lo[q8 * 8 + 2 * j + 1]));
                                __nv_bfloat162 b2 = __floats2bfloat162_rn(__uint_as_float(hi[q8 * 8 + 2 * j]),
                                                                          __uint_as_float(hi[q8 * 8 + 2 * j + 1]));
                                pl[j] = *reinterpret_cast<uint32_t*>(&a2);
                                ph[j] = *reinterpret_cast<uint32_t*>(&b2);
                            }
                            *reinterpret_cast<uint4*>(lo_row + (((lo_piece + q8) ^ (r & 7)) << 4)) =
                                make_uint4(pl[0], pl[1], pl[2], pl[3]);
                            *reinterpret_cast<uint4*>(hi_row + (((hi_piece + q8) ^ (r & 7)) << 4)) =
                                make_uint4(ph[0], ph[1], ph[2], ph[3]);
                        }
                    }
                    tc::fence_proxy_async();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (is_q) {
                        if (warp == 2 && lane == 0) {
                            for (int ch = 0; ch < chunks; ++ch)
                                tc::tma_store_2d(&map_c, buf + ch * (BM * 128), head * hd + ch * 64, m0_h);
                            tc::tma_store_commit();
                        }
                    } else if (ra.write_cache) {
                        const int kvh = is_k ? head - ra.n_heads : head - ra.n_heads - ra.n_kv_heads;
                        __nv_bfloat16* cache = is_k ? ra.k_cache : ra.v_cache;
                        for (int i = r; i < BM * 8 * chunks; i += 128) {
                            const int ch = i / (BM * 8), rr = (i >> 3) & (BM - 1), piece = i & 7;
                            const long base = s.row_base[rr];
                            if (base < 0) continue;
                            const uint4 v = *reinterpret_cast<const uint4*>(
                                buf + ch * (BM * 128) + rr * 128 + ((piece ^ (rr & 7)) << 4));
                            *reinterpret_cast<uint4*>(cache + ((size_t)base + (size_t)kvh * ra.page_tokens) * hd +
                                                      ch * 64 + piece * 8) = v;
                        }
                    }
                }
                }
                if (warp == 2 && lane == 0) tc::tma_store_wait_all();
            } else if (tma_out) {
                // Through shared memory and out by TMA: the ring of stages is free by now.
                // Chunks of [128 rows][128 bytes] in the 128-byte swizzle; a thread writes
                // its row's eight 16-byte pieces, then one thread sends the box: a store, or
                // for ACCUM_F32 an fp32 add at the memory side (no read of C at all).
                const int r = quarter * 32 + lane;
                uint8_t* ring = s.a[0];
                constexpr int OUT_COLS = EPI == SWIGLU_BF16 ? BN / 2 : BN;     // columns of C per tile
                constexpr int CHUNK = (EPI == STORE_F32 || EPI == ACCUM_F32) ? 32 : 64;
                const int n_out = EPI == SWIGLU_BF16 ? inter : N;
                float ss4[4] = {0.f, 0.f, 0.f, 0.f};
                uint8_t* const sbuf = ring + (BN / 32) * (BM * 128);     // behind the staged chunks of C
                static_assert(NORM != NORM_EMIT || EPI != ACCUM_F32 || BN > 128 || MH > 1 ||
                                  (BN / 32) * (BM * 192) <= (int)(sizeof(s.a) + sizeof(s.b)),
                              "the staged chunks of C and of the scaled rows must fit in the ring of stages");
                const bool direct = M <= BM;
                if (emit) {
                    asm volatile("bar.sync 1, 128;" ::: "memory");          // the gain is in shared memory
                    if (!tc::mbar_wait(&s.c_bar, 0, abort_flag)) tc::give_up(abort_flag, status, tc::ST_EPILOGUE_TIMEOUT);
                }
#pragma unroll 1
                for (int mh = 0; mh < MH; ++mh) {                   // one accumulator after the other
                const uint32_t lane_addr_h = lane_addr + mh * BN;
                const float f = mh == 0 ? rf[0] : rf[MH - 1];
                if (mh > 0) {
                    // the staging buffers are used again: the first half's stores must have read them
                    if (warp == 2 && lane == 0) tc::tma_store_wait_read();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                }
#pragma unroll 1
                for (int c = 0; c < OUT_COLS / CHUNK; ++c) {
                    uint8_t* buf = ring + c * (BM * 128);
                    uint8_t* mine = buf + r * 128;
                    if (EPI == STORE_F32 || EPI == ACCUM_F32) {
                        uint32_t v[32];
                        tc::tmem_ld_32x32(lane_addr_h + c * 32, v);
                        // a norm after the product: the chunk's values of C and the gain come out
                        // of shared memory while the accumulators come out of tensor memory
                        constexpr bool EMIT = NORM == NORM_EMIT && EPI == ACCUM_F32 && MH == 1;
                        const bool emit_chunk = EMIT && emit && n_tile * BN + c * 32 < N;
                        float4 o[EMIT ? 8 : 1], g[EMIT ? 8 : 1];
                        if (EMIT && emit_chunk) {
                            const uint8_t* old_row = c_tile + c * (BM * 128) + r * 128;
                            const float4* g4 = reinterpret_cast<const float4*>(s.gain + (c * 32 & 127));
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                o[q] = *reinterpret_cast<const float4*>(old_row + ((q ^ (r & 7)) << 4));
                                g[q] = g4[q];
                            }
                        }
                        tc::tmem_ld_wait();
                        if (PRE) {
#pragma unroll
                            for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * f);
                        }
#pragma unroll
                        for (int q = 0; q < 8; ++q)
                            *reinterpret_cast<uint4*>(mine + ((q ^ (r & 7)) << 4)) =
                                make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                        if (EMIT && emit_chunk) {
                            // The sums as the TMA add will leave them in C (the same two fp32
                            // operands), their squares in four interleaved chains, and bf16(x * gain):
                            // for a single tile of rows in 64-byte pieces of the thread's own row
                            // straight to memory (a TMA store more per chunk and the wait for it
                            // cost 0.3 us more there), for many rows staged behind the chunks of C
                            // as [128 rows][64 bytes], unswizzled, and sent as a box.
                            uint8_t* staged = sbuf + c * (BM * 64) + r * 64;
                            uint8_t* s_row = direct ? reinterpret_cast<uint8_t*>(na.scaled + (size_t)row * na.ld_scaled +
                                                                                 n_tile * BN + c * 32)
                                                    : staged;
                            uint32_t pk[4];
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                const float x0 = o[q].x + __uint_as_float(v[4 * q]);
                                const float x1 = o[q].y + __uint_as_float(v[4 * q + 1]);
                                const float x2 = o[q].z + __uint_as_float(v[4 * q + 2]);
                                const float x3 = o[q].w + __uint_as_float(v[4 * q + 3]);
                                ss4[0] = fmaf(x0, x0, ss4[0]);
                                ss4[1] = fmaf(x1, x1, ss4[1]);
                                ss4[2] = fmaf(x2, x2, ss4[2]);
                                ss4[3] = fmaf(x3, x3, ss4[3]);
                                __nv_bfloat162 a2 = __floats2bfloat162_rn(x0 * g[q].x, x1 * g[q].y);
                                __nv_bfloat162 b2 = __floats2bfloat162_rn(x2 * g[q].z, x3 * g[q].w);
                                pk[2 * (q & 1)] = *reinterpret_cast<uint32_t*>(&a2);
                                pk[2 * (q & 1) + 1] = *reinterpret_cast<uint32_t*>(&b2);
                                if ((q & 1) && (!direct || row < M))
                                    *reinterpret_cast<uint4*>(s_row + (q >> 1) * 16) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                            }
                        }
                    } else {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            uint32_t v[32];
                            tc::tmem_ld_32x32(lane_addr_h + c * 64 + h * 32, v);
                            if (EPI == SWIGLU_BF16) {
                                uint32_t u[32];
                                tc::tmem_ld_32x32(lane_addr_h + BN / 2 + c * 64 + h * 32, u);
                                tc::tmem_ld_wait();
#pragma unroll
                                for (int j = 0; j < 32; ++j)
                                    v[j] = __float_as_uint(tc::silu_fast(__uint_as_float(v[j]) * f) *
                                                           (__uint_as_float(u[j]) * f));
                            } else {
                                tc::tmem_ld_wait();
                                if (PRE) {
#pragma unroll
                                    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * f);
                                }
                            }
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                uint32_t pk[4];
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    __nv_bfloat162 b2 = __floats2bfloat162_rn(
                                        __uint_as_float(v[q * 8 + 2 * j]), __uint_as_float(v[q * 8 + 2 * j + 1]));
                                    pk[j] = *reinterpret_cast<uint32_t*>(&b2);
                                }
                                *reinterpret_cast<uint4*>(mine + (((h * 4 + q) ^ (r & 7)) << 4)) =
                                    make_uint4(pk[0], pk[1], pk[2], pk[3]);
                            }
                        }
                    }
                    tc::fence_proxy_async();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (warp == 2 && lane == 0) {
                        const int x = n_tile * OUT_COLS + c * CHUNK;
                        if (x < n_out) {
                            if (EPI == ACCUM_F32) tc::tma_reduce_add_2d(&map_c, buf, x, m0 + mh * BM);
                            else tc::tma_store_2d(&map_c, buf, x, m0 + mh * BM);

                            if (NORM == NORM_EMIT && EPI == ACCUM_F32 && MH == 1 && emit && !direct)
                                tc::tma_store_2d(&map_s, sbuf + c * (BM * 64), x, m0);
                            tc::tma_store_commit();
                        }
                    }
                }
                }
                if (NORM == NORM_EMIT && EPI == ACCUM_F32 && MH == 1 && emit && row < M)
                    na.sumsq_out[(size_t)n_tile * M + row] = (ss4[0] + ss4[1]) + (ss4[2] + ss4[3]);
                if (warp == 2 && lane == 0) tc::tma_store_wait_all();
            } else if (EPI == SWIGLU_BF16) {
                constexpr int HALF = BN / 2;
                __nv_bfloat16* C = (__nv_bfloat16*)c_ptr;
#pragma unroll 1
                for (int c0 = 0; c0 < HALF; c0 += 16) {
                    uint32_t g[16], u[16];
                    tc::tmem_ld_32x16(lane_addr + c0, g);
                    tc::tmem_ld_32x16(lane_addr + HALF + c0, u);
                    tc::tmem_ld_wait();
                    const int col0 = n_tile * HALF + c0;
                    if (row < M) {
                        __nv_bfloat16* dst = C + (size_t)row * ldc + col0;
                        if (col0 + 16 <= inter && ((ldc & 7) == 0)) {
                            uint32_t packed[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) {
                                const float g0 = __uint_as_float(g[2 * j]) * rf[0];
                                const float g1 = __uint_as_float(g[2 * j + 1]) * rf[0];
                                const float h0 = tc::silu_fast(g0) * (__uint_as_float(u[2 * j]) * rf[0]);
                                const float h1 = tc::silu_fast(g1) * (__uint_as_float(u[2 * j + 1]) * rf[0]);
                                __nv_bfloat162 v = __floats2bfloat162_rn(h0, h1);
                                packed[j] = *reinterpret_cast<uint32_t*>(&v);
                            }
                            uint4* d4 = reinterpret_cast<uint4*>(dst);
                            d4[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                            d4[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                if (col0 + j < inter) {
                                    const float gv = __uint_as_float(g[j]) * rf[0];
                                    dst[j] = __float2bfloat16_rn(tc::silu_fast(gv) *
                                                                 (__uint_as_float(u[j]) * rf[0]));
                                }
                            }
                        }
                    }
                }
            } else if (EARLY) {
#pragma unroll
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t r[32];
                    tc::tmem_ld_32x32(lane_addr + c0, r);
                    tc::tmem_ld_wait();
                    const int col0 = n_tile * BN + c0;
                    if (row >= M || col0 >= N) continue;
                    float* dst = (float*)c_ptr + (size_t)row * ldc + col0;
                    if (col0 + 32 <= N && (ldc & 3) == 0) {
                        float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
                        for (int q = 0; q < 8; ++q) {
                            const float4 o = early[(c0 >> 2) + q];
                            d4[q] = make_float4(o.x + __uint_as_float(r[4 * q]) * rf[0],
                                                o.y + __uint_as_float(r[4 * q + 1]) * rf[0],
                                                o.z + __uint_as_float(r[4 * q + 2]) * rf[0],
                                                o.w + __uint_as_float(r[4 * q + 3]) * rf[0]);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (col0 + j < N) dst[j] += __uint_as_float(r[j]) * rf[0];
                    }
                }
            } else {
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 32) {
                    uint32_t r[32];
                    tc::tmem_ld_32x32(lane_addr + c0, r);
                    tc::tmem_ld_wait();
                    const int col0 = n_tile * BN + c0;
                    if (row >= M || col0 >= N) continue;
                    if (PRE) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * rf[0]);
                    }
                    const bool full = col0 + 32 <= N;
                    if (EPI == STORE_BF16) {
                        __nv_bfloat16* dst = (__nv_bfloat16*)c_ptr + (size_t)row * ldc + col0;
                        if (full && (ldc & 7) == 0) {
                            uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
                            for (int q = 0; q < 4; ++q) {
                                uint32_t p[4];
#pragma unroll
                                for (int j = 0; j < 4; ++j) {
                                    __nv_bfloat162 v = __floats2bfloat162_rn(
                                        __uint_as_float(r[q * 8 + 2 * j]),
                                        __uint_as_float(r[q * 8 + 2 * j + 1]));
                                    p[j] = *reinterpret_cast<uint32_t*>(&v);
                                }
                                d4[q] = make_uint4(p[0], p[1], p[2], p[3]);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (col0 + j < N) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
                        }
                    } else {
                        float* dst = (float*)c_ptr + (size_t)row * ldc + col0;
                        if (full && (ldc & 3) == 0) {
                            float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
                            for (int q = 0; q < 8; ++q) {
                                float4 v = make_float4(__uint_as_float(r[4 * q]), __uint_as_float(r[4 * q + 1]),
                                                       __uint_as_float(r[4 * q + 2]), __uint_as_float(r[4 * q + 3]));
                                if (EPI == ACCUM_F32) {
                                    const float4 o = d4[q];
                                    v.x += o.x; v.y += o.y; v.z += o.z; v.w += o.w;
                                }
                                d4[q] = v;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; ++j) {
                                if (col0 + j < N) {
                                    const float v = __uint_as_float(r[j]);
                                    dst[j] = EPI == ACCUM_F32 ? dst[j] + v : v;
                                }
                            }
                        }
                    }
                }
            }
        }
    }
    if (emit && warp == 2 && lane == 0 && *abort_flag) {
        // the tile of C may still be on its way into this block's shared memory
        for (uint32_t i = 0; i < tc::WAIT_LIMIT; ++i)
            if (tc::mbar_try_wait(&s.c_bar, 0)) break;
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::tc_fence_after_sync();
        tc::tmem_dealloc(tmem_acc, TMEM_COLS);
    }
}

template <int BN, int STAGES, int EPI, int MH, int NORM>
int launch_norm(const CUtensorMap& ma, const CUtensorMap& mw, void* C, int M, int N, int K, int ldc,
                int inter, int k_splits, int* status, cudaStream_t stream, const RopeArgs& ra, const NormArgs& na) {
    if (MH > 1 && k_splits > 1) return CB_ERR_UNSUPPORTED;
    // a norm after the product: only the epilogue that has the summed rows in registers leaves it
    const bool emit = na.gain != nullptr;
    using Storage = SharedStorage<BN, STAGES, MH>;
    const size_t smem_plain = sizeof(Storage) + 1024;
    const size_t smem_emit = ((sizeof(Storage) + 1023) & ~(size_t)1023) + (size_t)BM * BN * 4 + 1024;
    if (emit && (EPI != ACCUM_F32 || BN > 128 || MH != 1 || (N & 31) || (ldc & 3) || (na.ld_scaled & 7) ||
                 ((uintptr_t)na.scaled & 15) || ((uintptr_t)na.gain & 15) || ((uintptr_t)C & 15) ||
                 na.scaled == nullptr || na.sumsq_out == nullptr || smem_emit > 227 * 1024))
        return CB_ERR_UNSUPPORTED;
    if (na.sumsq_in != nullptr && (na.parts < 1 || !(na.width > 0.f))) return CB_ERR_UNSUPPORTED;
    // shares of K: at most 8 blocks in a cluster, every share at least one block of 64
    // elements, and a block's accumulator (128 x BN fp32) has to fit in the ring of stages
    if (k_splits < 1) k_splits = 1;
    if (k_splits > 1) {
        const int kb = (K + BK - 1) / BK, per = (kb + k_splits - 1) / k_splits;
        if (k_splits > 8 || (k_splits - 1) * per >= kb || (size_t)BM * BN * 4 > (size_t)STAGES * (BM + BN) * BK * 2)
            return CB_ERR_UNSUPPORTED;
    }
    // the output goes through shared memory and TMA where its rows allow it
    const bool f32 = EPI == STORE_F32 || EPI == ACCUM_F32;
    const int esize = f32 ? 4 : 2;
    const int out_cols = EPI == SWIGLU_BF16 ? inter : N;
    int tma_out = ((uintptr_t)C & 15) == 0 && ((size_t)ldc * esize) % 16 == 0 &&
                  (f32 || (EPI == SWIGLU_BF16 ? BN % 128 == 0 : BN % 64 == 0));
    CUtensorMap mc = ma;
    // ROPE_APPEND: only the q heads' columns of C are written
    const uint64_t map_cols = EPI == ROPE_APPEND ? (uint64_t)ra.n_heads * ra.head_dim : (uint64_t)out_cols;
    if (tma_out && !tc::make_out_map_2d(&mc, C, f32, (uint64_t)M, map_cols, (uint64_t)ldc, BM))
        tma_out = 0;
    if ((EPI == ROPE_APPEND || MH > 1 || emit) && !tma_out) return CB_ERR_UNSUPPORTED;
    CUtensorMap ms = ma;
    if (emit && !tc::make_plain_box_map_2d(&ms, na.scaled, (uint64_t)M, (uint64_t)N, (uint64_t)na.ld_scaled, 32, BM))
        return CB_ERR_UNSUPPORTED;
    const int smem = (int)(emit ? smem_emit : smem_plain);
    static int configured = 0;
    if (configured < smem) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, STAGES, EPI, MH, NORM>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = smem;
    }
    const int n_cols = EPI == SWIGLU_BF16 ? 2 * inter : N;
    dim3 grid((n_cols + BN - 1) / BN, (M + BM * MH - 1) / (BM * MH), k_splits);
    cb_launch_cluster(gemm_tcgen05_kernel<BN, STAGES, EPI, MH, NORM>, dim3(grid), dim3(192), smem, stream, k_splits,
                      ma, mw, mc, ms, tma_out, C, M, N, K, ldc, inter, k_splits, status, ra, na);
    return cb_last_error();
}

// The forms that exist: rows ahead of their norm for the products that follow a norm (gate/up
// with SwiGLU, q/k/v with the rotation), the next norm's input from the accumulating product
// with tiles up to 128 columns.
template <int BN, int STAGES, int EPI, int MH = 1>
int launch(const CUtensorMap& ma, const CUtensorMap& mw, void* C, int M, int N, int K, int ldc,
           int inter, int k_splits, int* status, cudaStream_t stream, const RopeArgs& ra = RopeArgs{},
           const NormArgs& na = NormArgs{}) {
    if (na.gain != nullptr && na.sumsq_in != nullptr) return CB_ERR_UNSUPPORTED;
    if (na.sumsq_in != nullptr) {
        if constexpr (EPI == SWIGLU_BF16 || EPI == ROPE_APPEND)
            return launch_norm<BN, STAGES, EPI, MH, NORM_PRE>(ma, mw, C, M, N, K, ldc, inter, k_splits, status, stream, ra, na);
        return CB_ERR_UNSUPPORTED;
    }
    if (na.gain != nullptr) {
        if constexpr (EPI == ACCUM_F32 && BN <= 128 && MH == 1)
            return launch_norm<BN, STAGES, EPI, MH, NORM_EMIT>(ma, mw, C, M, N, K, ldc, inter, k_splits, status, stream, ra, na);
        return CB_ERR_UNSUPPORTED;
    }
    return launch_norm<BN, STAGES, EPI, MH, NORM_NONE>(ma, mw, C, M, N, K, ldc, inter, k_splits, status, stream, ra, na);
}

template <int BN, int STAGES, int MH = 1>
int launch_epi(int epi, const CUtensorMap& ma, const CUtensorMap& mw, void* C, int M, int N,
               int K, int ldc, int inter, int ks, int* status, cudaStream_t stream, const NormArgs& na) {
    const RopeArgs none{};
    switch (epi) {
        case STORE_BF16: return launch<BN, STAGES, STORE_BF16, MH>(ma, mw, C, M, N, K, ldc, inter, ks, status, stream, none, na);
        case STORE_F32: return launch<BN, STAGES, STORE_F32, MH>(ma, mw, C, M, N, K, ldc, inter, ks, status, stream, none, na);
        case ACCUM_F32: return launch<BN, STAGES, ACCUM_F32, MH>(ma, mw, C, M, N, K, ldc, inter, ks, status, stream, none, na);
        case SWIGLU_BF16: return launch<BN, STAGES, SWIGLU_BF16, MH>(ma, mw, C, M, N, K, ldc, inter, ks, status, stream, none, na);
    }
    return CB_ERR_UNSUPPORTED;
}

}  // namespace

// W is [N, K] (for SWIGLU_BF16: [2 * inter, K], N = inter and C is [M, inter]).
// bn: tile width: 64, 96, 128, 160, 192 or 256.  per_sm: 0 = two accumulators (256 rows of
// output per block, bn 256 only, no shares of K); 1 = a deep ring of stages, one
// block per SM; 2 = three stages, so that two blocks share an SM and one's prologue and
// epilogue run beside the other's products (tile widths up to 128).
// status: device int, stays 0 unless a wait ran out.
// k_splits: 1, or the number of blocks (at most 8) that share a tile's K as a cluster.
// norm: null, or what the product knows of the norm after or before it (NormArgs; a host
// pointer, read during the call).
CB_EXPORT int cb_gemm_tcgen05(const void* A, const void* W, void* C, int M, int N, int K, int lda,
                              int ldw, int ldc, int epi, int bn, int per_sm, int k_splits, int* status,
                              void* stream, const void* norm) {
    if (M <= 0 || N <= 0) return 0;
    const NormArgs na = norm ? *static_cast<const NormArgs*>(norm) : NormArgs{};
    if (K <= 0 || (K & 7) || (lda & 7) || (ldw & 7) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15))
        return CB_ERR_UNSUPPORTED;
    const int w_rows = epi == SWIGLU_BF16 ? 2 * N : N;
    const int box_rows = epi == SWIGLU_BF16 ? bn / 2 : bn;
    CUtensorMap ma, mw;
    if (!tc::make_map_2d(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM)) return CB_ERR_UNSUPPORTED;
    if (!tc::make_map_2d(&mw, W, (uint64_t)w_rows, (uint64_t)K, (uint64_t)ldw, box_rows))
        return CB_ERR_UNSUPPORTED;
    cudaStream_t s = (cudaStream_t)stream;
    const int inter = epi == SWIGLU_BF16 ? N : 0;
    if (per_sm == 0) {            // two accumulators: 256 x 256 of output per block
        if (bn == 256) return launch_epi<256, 3, 2>(epi, ma, mw, C, M, N, K, ldc, inter, k_splits, status, s, na);
        return CB_ERR_UNSUPPORTED;
    }
    if (per_sm == 2) {
        switch (bn) {
            case 64: return launch_epi<64, 3>(epi, ma, mw, C, M, N, K, ldc, inter, k_splits, status, s, na);
            case 96: return launch_epi<96, 3>(epi, ma, mw, C, M, N, K, ldc, inter, k_splits, status, s, na);
            case 128: return launch_epi<128, 3>(epi, ma, mw, C, M, N, K, ldc, inter, k_splits, status, s, na);
        }
        return CB_ERR_UNSUPPORTED;
    }
    switch (bn) {
        case 64: return launch_epi<64, 6>(epi, ma, mw, C, M, N, K, ldc, inter, k_splits, status, s, na);
        case 96: return launch_epi<96, 6>(epi, ma, mw, C, M, N, K, ldc, inter, k_splits, status, s, na);
        case 128: return launch_epi<128, 5>(epi, ma, mw, C, M, N, K, ldc, inter, k_splits, status, s, na);
        case 160: return launch_epi<160, 5>(epi, ma, mw, C, M, N, K, ldc, inter, k_splits, status, s, na);
        case 192: return launch_epi<192, 5>(epi, ma, mw, C, M, N, K, ldc, inter, k_splits, status, s, na);
        case 256: return launch_epi<256, 4>(epi, ma, mw, C, M, N, K, ldc, inter, k_splits, status, s, na);
    }
    return CB_ERR_UNSUPPORTED;
}

// The query/key/value projection with the rotation of q and k and the write of k and v
// into the rows' cache pages in the epilogue.  W = [Wq; Wk; Wv] ([(Hq + 2 Hkv) * head_dim, K]);
// rotated q goes to q_out[M, ldq] (bf16).  The whole head is rotated (pairs j, j + head_dim / 2);
// head_dim is a multiple of 64 and divides the tile width bn.
CB_EXPORT int cb_gemm_tcgen05_rope(const void* A, const void* W, void* q_out, int M, int K, int lda,
                                   int ldw, int ldq, int bn, const float* cos_t, const float* sin_t,
                                   const int* positions, const int* row_request,
                                   const int* block_table, int table_stride, void* k_cache,
                                   void* v_cache, int n_heads, int n_kv_heads, int head_dim,
                                   int page_tokens, int write_cache, int k_splits, int tall, int* status,
                                   void* stream, const void* norm) {
    if (M <= 0) return 0;
    const NormArgs na = norm ? *static_cast<const NormArgs*>(norm) : NormArgs{};
    if (K <= 0 || (K & 7) || (lda & 7) || (ldw & 7) || ((uintptr_t)A & 15) || ((uintptr_t)W & 15) ||
        head_dim <= 0 || (head_dim & 63) || bn % head_dim != 0 || (ldq & 7) || ((uintptr_t)q_out & 15) ||
        ((uintptr_t)k_cache & 15) || ((uintptr_t)v_cache & 15) || ((uintptr_t)cos_t & 15) ||
        ((uintptr_t)sin_t & 15))
        return CB_ERR_UNSUPPORTED;
    const int N = (n_heads + 2 * n_kv_heads) * head_dim;
    CUtensorMap ma, mw;
    if (!tc::make_map_2d(&ma, A, (uint64_t)M, (uint64_t)K, (uint64_t)lda, BM)) return CB_ERR_UNSUPPORTED;
    if (!tc::make_map_2d(&mw, W, (uint64_t)N, (uint64_t)K, (uint64_t)ldw, bn)) return CB_ERR_UNSUPPORTED;
    RopeArgs ra;
    ra.cos_t = cos_t; ra.sin_t = sin_t; ra.positions = positions; ra.row_request = row_request;
    ra.block_table = block_table; ra.table_stride = table_stride;
    ra.k_cache = (__nv_bfloat16*)k_cache; ra.v_cache = (__nv_bfloat16*)v_cache;
    ra.n_heads = n_heads; ra.n_kv_heads = n_kv_heads; ra.head_dim = head_dim;
    ra.page_tokens = page_tokens; ra.write_cache = write_cache;
    cudaStream_t s = (cudaStream_t)stream;
    if (tall) {           // two accumulators: 256 rows of output per block
        if (bn == 256) return launch<256, 3, ROPE_APPEND, 2>(ma, mw, q_out, M, N, K, ldq, 0, 1, status, s, ra, na);
        return CB_ERR_UNSUPPORTED;
    }
    switch (bn) {
        case 64: return launch<64, 6, ROPE_APPEND>(ma, mw, q_out, M, N, K, ldq, 0, k_splits, status, s, ra, na);
        case 128: return launch<128, 5, ROPE_APPEND>(ma, mw, q_out, M, N, K, ldq, 0, k_splits, status, s, ra, na);
        case 192: return launch<192, 5, ROPE_APPEND>(ma, mw, q_out, M, N, K, ldq, 0, k_splits, status, s, ra, na);
        case 256: return launch<256, 4, ROPE_APPEND>(ma, mw, q_out, M, N, K, ldq, 0, k_splits, status, s, ra, na);
    }
    return CB_ERR_UNSUPPORTED;
}

// ---------------------------------------------------------------------------
// A wait that runs out, for tests of the failure path: one thread waits, with
// the kernels' own bounded wait and a short limit given by the caller, on an
// mbarrier at which nothing ever arrives; when the limit is reached it records
// ST_PROBE_TIMEOUT in the status word exactly as a real role does, and the
// kernel returns.  Nothing faults, traps or hangs; the context stays usable.
// ---------------------------------------------------------------------------
namespace {
__global__ void wait_probe_kernel(int* status, uint32_t limit) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        tc::mbar_init(&bar, 1);
        tc::fence_barrier_init();
        if (!tc::mbar_wait(&bar, 0, &abort_flag, limit))
            tc::give_up(&abort_flag, status, tc::ST_PROBE_TIMEOUT);
    }
}
}  // namespace

CB_EXPORT int cb_tc_wait_probe(int* status, int limit, void* stream) {
    if (limit <= 0 || limit > (1 << 20)) return CB_ERR_UNSUPPORTED;
    wait_probe_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(status, (uint32_t)limit);
    return (int)cudaGetLastError();
}
