// Paged attention for decoded tokens (a few query rows per request, many keys)
// on the 5th-generation tensor cores, head size 64 or 128, bfloat16.  Such a step only
// has to read the keys and values once; what the mma.sync kernel spends per key
// in instructions keeps it at a third of the memory bandwidth.  Here the KEYS sit
// on the tensor-memory lanes:
//
//   S^T[128 keys, 16 rows] = K_tile Q^T      tcgen05.mma, M = 128 keys, N = 16, K = head size
//   softmax: one thread per key reads its row of S^T from tensor memory and
//            computes p for the block's (at most 16) query rows - a handful of
//            exponentials per thread - and writes P (bf16) to shared memory
//   O[16 rows, hd] += P V_tile               tcgen05.mma, M = 128 (rows 16.. unused), N = 64 per half of hd, K = 128
//
// K and V pages come in by TMA in a ring of three stages: one box per page, or one
// box for a whole tile when its pages follow one another in the pool.  A
// block takes the up to 16 (token, head of the group) rows of one request and
// one KV head against ONE chunk of keys and writes an unnormalised partial
// (vector, maximum, sum); the last block of a row group to arrive (an atomic
// counter; no block waits for another) merges the chunks in ascending order.
// Chunk boundaries are multiples of the chunk from key 0 and the chunk is chosen
// from the launch's shape, so a row's result is a function of its own query and
// keys only.
//
// The reference maximum of a row is raised only when a tile exceeds it by more
// than 2^8 (found with one block-wide OR per tile); only then are the rows'
// maxima reduced over the block and the accumulator in tensor memory rescaled.
//
// The second MMA's A operand is P as [128 rows, 128 keys]; only its first 16 rows
// are real.  Their 2 KB per half of 64 keys lie directly before the K/V ring, and
// the operand's other row groups read on into the ring: whatever they hold ends
// in accumulator rows 16..127, which nobody reads.
//
// Roles: warp 0 loads, warp 1 owns tensor memory and issues the MMAs, warps 2-5
// are the softmax (128 threads = 128 keys).  Every wait on an mbarrier is bounded;
// the softmax warps' block barriers are passed by all of them whatever happened.
//
// Sizes: head size 64 or 128; page size a power of two from 8 to 128; at most 16 packed
// rows per request and KV head; chunk a multiple of 128 keys.  Anything else is
// refused and the mma.sync kernel runs.
// Reference counterparts: `attention_decode_paged_f32` (engine/kernels/kernels.cu:1741)
// and the split idea of `attention_partial_f32` / `attention_combine_f32` (:692-850).
#define CB_PDL_BIT 2      // this file's bit in CRUCIBLE_PDL
#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int KEYS = 128;            // keys per tile = tensor-memory lanes of S^T
constexpr int ROWS = 16;             // query rows per block (N of the first MMA)
constexpr int MAX_STAGES = 3;        // the loader's first copies are written out for three
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RAISE = 8.0f;

struct DecodeParams {
    const __nv_bfloat16* qkv;
    int qkv_stride;
    __nv_bfloat16* out;
    int out_stride;
    const int* req_row_start;
    const int* req_first_pos;
    const int* block_table;
    int table_stride;
    int n_heads, n_kv_heads, n_rep, n_requests, page_shift;
    float scale_log2;
    int window;
    float* partial;          // [rows_total * n_heads][n_chunks][head size + 2]
    int* counters;           // [n_requests * n_kv_heads], zero between launches
    int n_chunks, chunk_keys;
    int n_pages;             // of the pool
    int runs;                // 1: the 4-D maps may be used for tiles whose pages are consecutive
    int* status;
};

// HD: the head size, 64 or 128.  Operands whose contracted or free dimension is the head
// size lie in shared memory as HD / 64 halves of [rows][128 bytes] (one swizzle atom wide).
// STAGES: 3, or 2 for launches whose chunks are at most two tiles long (74 KB instead of 110 KB
// for head size 64: three blocks to an SM instead of two, so that every block of a launch of a few
// hundred finds its place while the product before it still runs).
template <int HD, int STAGES>
struct Storage {
    alignas(1024) uint8_t q[HD / 64][ROWS * 64 * 2];         // [16 rows][128 B] per half, swizzled
    alignas(1024) uint8_t p[2][2][ROWS * 64 * 2];            // P: two buffers of two halves of 64 keys
    alignas(1024) uint8_t k[STAGES][HD / 64][KEYS * 64 * 2]; // directly after P (see above)
    alignas(1024) uint8_t v[STAGES][HD / 64][KEYS * 64 * 2];
    alignas(8) uint64_t kv_full[STAGES];
    uint64_t kv_empty[STAGES];
    uint64_t s_full[2], p_full[2], pv_done[2];
    float red[4][ROWS];
    uint32_t tmem_base;
    int abort_flag;
    int is_last;
};

__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void softmax_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// block-wide OR over the 128 softmax threads
__device__ __forceinline__ bool softmax_any(bool pred) {
    int out;
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.s32 p, %1, 0;\n\t"
        "bar.red.or.pred q, 1, 128, p;\n\t"
        "selp.s32 %0, 1, 0, q;\n\t"
        "}"
        : "=r"(out)
        : "r"((int)pred)
        : "memory");
    return out != 0;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Merges one row's chunks (ascending, with a running maximum) and writes its
// output.  One warp; a lane owns HD / 32 neighbouring features.
template <int HD>
__device__ __forceinline__ void merge_row(const DecodeParams& p, int tok, int head, int pos, int lane) {
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    constexpr int MP = HD + 2;
    constexpr int F = HD / 32;
    const int c_first = lo / p.chunk_keys, c_last = pos / p.chunk_keys;
    const float* base = p.partial + ((size_t)tok * p.n_heads + head) * p.n_chunks * MP;
    float m = -INFINITY, l = 0.f, acc[F];
#pragma unroll
    for (int f = 0; f < F; ++f) acc[f] = 0.f;
    constexpr int ROUND = 8;                             // chunks asked for at once (16: measured slower)
    for (int c0 = c_first; c0 <= c_last; c0 += ROUND) {
        float mc[ROUND], lc[ROUND], o[ROUND][F];
#pragma unroll
        for (int j = 0; j < ROUND; ++j) {
            const bool in = c0 + j <= c_last;
            const float* src = base + (size_t)(in ? c0 + j : c_first) * MP;
            mc[j] = in ? __ldcg(src + HD) : -INFINITY;
            lc[j] = in ? __ldcg(src + HD + 1) : 0.f;
#pragma unroll
            for (int f = 0; f < F; f += 2) {
                const float2 v = in ? __ldcg(reinterpret_cast<const float2*>(src + lane * F + f))
                                    : make_float2(0.f, 0.f);
                o[j][f] = v.x;
                o[j][f + 1] = v.y;
            }
        }
#pragma unroll
        for (int j = 0; j < ROUND; ++j) {                // ascending chunks
            const float m_new = fmaxf(m, mc[j]);
            const float off = m_new == -INFINITY ? 0.f : m_new;
            const float keep = exp2f(m - off), take = exp2f(mc[j] - off);
            l = l * keep + lc[j] * take;
#pragma unroll
            for (int f = 0; f < F; ++f) acc[f] = acc[f] * keep + o[j][f] * take;
            m = m_new;
        }
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    __nv_bfloat16* dst = p.out + (size_t)tok * p.out_stride + (size_t)head * HD + lane * F;
#pragma unroll
    for (int f = 0; f < F; f += 2)
        *reinterpret_cast<__nv_bfloat162*>(dst + f) = __floats2bfloat162_rn(acc[f] * inv, acc[f + 1] * inv);
}

// RMAX: the most packed rows a block of this instantiation takes (4, 8 or 16): the
// softmax's per-row loops are unrolled that far and no further.
template <int HD, int RMAX, int STAGES>
__global__ void __launch_bounds__(192, HD == 64 ? (STAGES == 2 ? 3 : 2) : 1)
attention_decode_tcgen05_kernel(const __grid_constant__ CUtensorMap map_k,
                                const __grid_constant__ CUtensorMap map_v,
                                const __grid_constant__ CUtensorMap run_k,
                                const __grid_constant__ CUtensorMap run_v, const DecodeParams p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    using Store = Storage<HD, STAGES>;
    constexpr int NH = HD / 64;                       // halves of the head size
    constexpr uint32_t TMEM_COLS = HD == 64 ? 128 : 256;
    Store& s = *reinterpret_cast<Store*>(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // grid (chunks, KV heads, requests): a division by a run-time value costs a thread about
    // a hundred cycles, and a late block's way to its first copy is on the step's critical path
    const int chunk = blockIdx.x, kv_head = blockIdx.y, req = blockIdx.z;
    volatile int* abort_flag = &s.abort_flag;

    // ---- which keys: everything below is uniform over the block -------------------------
    const int n_rep = p.n_rep;
    const int row_base = p.req_row_start[req];
    const int n_new = p.req_row_start[req + 1] - row_base;
    const int n_rows = n_new * n_rep;                               // <= 16 (the host checked)
    const int first_pos = p.req_first_pos[req];
    const int* table = p.block_table + (size_t)req * p.table_stride;
    const int max_pos = first_pos + n_new - 1;
    const int key_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
    const int key_end = max_pos + 1;
    const int c0 = chunk * p.chunk_keys;
    // chunks wholly outside the rows' keys take no part
    if (n_rows <= 0 || c0 >= key_end || c0 + p.chunk_keys <= key_lo) return;
    const int n_active = (key_end - 1) / p.chunk_keys - key_lo / p.chunk_keys + 1;
    const int chunk_end = min(key_end, c0 + p.chunk_keys);
    const int tile0 = max(c0, key_lo / KEYS * KEYS);                // first tile's first key
    const int n_tiles = (chunk_end - tile0 + KEYS - 1) / KEYS;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; ++i) {
            tc::mbar_init(&s.kv_full[i], 1);
            tc::mbar_init(&s.kv_empty[i], 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc::mbar_init(&s.s_full[b], 1);
            tc::mbar_init(&s.p_full[b], 4);               // one arrival per softmax warp
            tc::mbar_init(&s.pv_done[b], 1);
        }
        s.abort_flag = 0;
        s.is_last = 0;
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&map_k);
        tc::prefetch_tensormap(&map_v);
        if (p.runs) {
            tc::prefetch_tensormap(&run_k);
            tc::prefetch_tensormap(&run_v);
        }
    }
    if (warp == 1) {
        tc::tmem_alloc(&s.tmem_base, TMEM_COLS);  // S^T: columns 0..15 and 16..31, O: from 64
        tc::tmem_relinquish();
    }

    // ---- the loader's thread: one tile of K and V pages into a stage -----------------------
    const int pages_per_tile = KEYS >> p.page_shift;
    auto lookup = [&](int j, int (&pages)[16]) {
        // the tile's table entries, all in flight at once: the copies are ordered against
        // memory and would take the lookups one by one
        const int key0 = tile0 + j * KEYS;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            int index = (key0 >> p.page_shift) + (i < pages_per_tile ? i : 0);
            index = index < p.table_stride ? index : p.table_stride - 1;
            const int page = table[index];
            pages[i] = page < 0 ? 0 : page;           // an entry given back early: never read
        }
    };
    auto issue = [&](int j, const int (&pages)[16]) -> bool {
        const int st = j % STAGES;
        const uint32_t round = j / STAGES;
        // pages that follow one another in the pool come in with one copy per tile
        bool run = p.runs != 0 && pages[0] + pages_per_tile <= p.n_pages;
#pragma unroll
        for (int i = 1; i < 16; ++i)
            if (i < pages_per_tile && pages[i] != pages[0] + i) run = false;
        if (round > 0 && !tc::mbar_wait(&s.kv_empty[st], (round - 1) & 1, abort_flag)) {
            tc::give_up(abort_flag, p.status, tc::ST_PRODUCER_TIMEOUT);
            return false;
        }
        tc::mbar_expect_tx(&s.kv_full[st], 2 * KEYS * HD * 2);
        if (run) {
#pragma unroll
            for (int h = 0; h < NH; ++h) {
                tc::tma_load_4d(s.k[st][h], &run_k, &s.kv_full[st], h * 64, 0, kv_head, pages[0]);
                tc::tma_load_4d(s.v[st][h], &run_v, &s.kv_full[st], h * 64, 0, kv_head, pages[0]);
            }
            return true;
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (i < pages_per_tile) {
                const int dst = (i << p.page_shift) * 128;
                const int y = (pages[i] * p.n_kv_heads + kv_head) << p.page_shift;
#pragma unroll
                for (int h = 0; h < NH; ++h) {
                    tc::tma_load_2d(s.k[st][h] + dst, &map_k, &s.kv_full[st], h * 64, y);
                    tc::tma_load_2d(s.v[st][h] + dst, &map_v, &s.kv_full[st], h * 64, y);
                }
            }
        }
        return true;
    };
    const int early = n_tiles < STAGES ? n_tiles : STAGES;

    // ---- warp 0's thread starts the first tiles' copies; the others stage the query rows
    // (16-byte pieces into the 128-byte swizzle; rows past the request's are zero) and clear P.
    // The block tables were uploaded before the step began, so the first tiles' lookups need
    // not wait for the kernels ahead in the stream; the copies do (the product before this
    // kernel writes this step's keys; and copies of older keys, or L2 prefetches of them,
    // asked for while that product still runs made a step slower, not faster: 0.300 against
    // 0.289 ms at batch 1, 0.329 against 0.320 ms at batch 8, measured on B200).
    if (warp == 0) {
        if (lane == 0) {
            // the first tiles wait for nothing: all their lookups first, then all their copies
            int y0[16], y1[16], y2[16];
            lookup(0, y0);
            if (early > 1) lookup(1, y1);
            if (early > 2) lookup(2, y2);
            cb_pdl_wait();
            issue(0, y0);
            if (early > 1) issue(1, y1);
            if (early > 2) issue(2, y2);
        } else {
            cb_pdl_wait();
        }
    } else {
        cb_pdl_wait();
        const int tid = threadIdx.x - 32;
        for (int i = tid; i < ROWS * 8 * NH; i += 160) {
            const int r = i / (8 * NH), c = i % (8 * NH);        // row, 16-byte piece of the row
            uint4 val = make_uint4(0, 0, 0, 0);
            if (r < n_rows) {
                const int tok = row_base + r / n_rep, head = kv_head * n_rep + r % n_rep;
                val = *reinterpret_cast<const uint4*>(p.qkv + (size_t)tok * p.qkv_stride +
                                                      (size_t)head * HD + c * 8);
            }
            *reinterpret_cast<uint4*>(s.q[c >> 3] + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = val;
        }
        for (int i = tid; i < (int)sizeof(s.p) / 16; i += 160)
            reinterpret_cast<uint4*>(&s.p[0][0][0])[i] = make_uint4(0, 0, 0, 0);
    }
    tc::fence_proxy_async();
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    // the query rows are staged and the first tiles' copies are on their way: the kernel
    // after this one may start (its first loads then do not get in the way of these)
    cb_pdl_trigger();
    const uint32_t tmem_s = s.tmem_base;          // + 16 for the second buffer
    const uint32_t tmem_o = s.tmem_base + 64;

    if (warp == 0) {
        // ---- loader: the remaining tiles, each once its stage has been read ------------------
        if (lane == 0) {
            int armed = early;
            // a tile's table entries are looked up while the tile before it is awaited
            int y[16];
            if (early < n_tiles) lookup(early, y);
            for (int j = early; j < n_tiles; ++j) {
                int y_now[16];
#pragma unroll
                for (int i = 0; i < 16; ++i) y_now[i] = y[i];
                if (j + 1 < n_tiles) lookup(j + 1, y);
                if (!issue(j, y_now)) break;
                armed = j + 1;
            }
            if (*abort_flag) {
                const int first = armed > STAGES ? armed - STAGES : 0;
                for (int j = first; j < armed; ++j)
                    for (uint32_t t = 0; t < tc::WAIT_LIMIT; ++t)
                        if (tc::mbar_try_wait(&s.kv_full[j % STAGES], (j / STAGES) & 1)) break;
            }
        }
    } else if (warp == 1) {
        // ---- MMA issuer -------------------------------------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc_qk = tc::instr_desc_bf16(KEYS, ROWS);
            constexpr uint32_t idesc_pv = tc::instr_desc_bf16_b_mn(128, 64);
            // Operand descriptors by addition: the low word carries the address in 16-byte
            // units, the high word is the same for every tile (this thread's own instructions
            // are what the tensor cores wait for here: nothing is built per MMA from pointers).
            const uint64_t q_desc0 = tc::smem_desc_sw128(tc::smem_u32(s.q[0]));
            const uint32_t desc_hi = (uint32_t)(q_desc0 >> 32);
            const uint32_t q_lo = (uint32_t)q_desc0;
            const uint32_t k_lo0 = (uint32_t)tc::smem_desc_sw128(tc::smem_u32(s.k[0][0]));
            const uint32_t v_lo0 = (uint32_t)tc::smem_desc_sw128(tc::smem_u32(s.v[0][0]));
            const uint32_t p_lo0 = (uint32_t)tc::smem_desc_sw128(tc::smem_u32(s.p[0][0]));
            constexpr uint32_t Q_HALF = sizeof(s.q[0]) >> 4, KV_HALF = sizeof(s.k[0][0]) >> 4,
                               KV_STAGE = sizeof(s.k[0]) >> 4, P_HALF = sizeof(s.p[0][0]) >> 4,
                               P_BUF = sizeof(s.p[0]) >> 4;
            bool ok = true;
            // S^T_j = K_j Q^T into buffer j & 1: K = 64 in four steps of 16
            // `block`: wait for the tile; else only take it if it has landed (true: issued)
            int qk_st = 0;                        // stage and parity of the next tile of scores
            uint32_t qk_parity = 0;
            auto issue_qk = [&](int j, bool block) -> bool {
                if (block) {
                    if (!tc::mbar_wait(&s.kv_full[qk_st], qk_parity, abort_flag)) return false;
                } else if (!tc::mbar_try_wait(&s.kv_full[qk_st], qk_parity)) {
                    return false;
                }
                tc::tc_fence_after_sync();
                const uint32_t k_lo = k_lo0 + qk_st * KV_STAGE;
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint64_t k_desc = tc::desc_of(k_lo + (k >> 2) * KV_HALF + 2 * (k & 3), desc_hi);
                    const uint64_t q_desc = tc::desc_of(q_lo + (k >> 2) * Q_HALF + 2 * (k & 3), desc_hi);
                    if (k == 0) tc::umma_bf16(tmem_s + (j & 1) * 16, k_desc, q_desc, idesc_qk, 0u);
                    else tc::umma_bf16_add(tmem_s + (j & 1) * 16, k_desc, q_desc, idesc_qk);
                }
                tc::umma_commit(&s.s_full[j & 1]);
                if (++qk_st == STAGES) qk_st = 0, qk_parity ^= 1;
                return true;
            };
            ok = issue_qk(0, true);
            int st = 0;                           // stage of tile j
            for (int j = 0; j < n_tiles && ok; ++j) {
                // the next tile's scores first if its keys have landed (their buffer was last
                // read by the softmax of tile j - 1, whose P this thread has waited for);
                // else after this tile's second product, which must not wait for a copy
                const bool ahead = j + 1 < n_tiles && issue_qk(j + 1, false);
                if (!tc::mbar_wait(&s.p_full[j & 1], (j >> 1) & 1, abort_flag)) {
                    ok = false;
                    break;
                }
                tc::tc_fence_after_sync();
                const uint32_t p_lo = p_lo0 + (j & 1) * P_BUF;
#pragma unroll
                for (int h = 0; h < NH; ++h) {                       // 64 output features at a time
                    const uint32_t v_lo = v_lo0 + st * KV_STAGE + h * KV_HALF;
#pragma unroll
                    for (int k = 0; k < KEYS / 16; ++k) {
                        // 16 keys further in V (keys are its rows of 128 bytes): 128 units
                        const uint64_t p_desc = tc::desc_of(p_lo + (k >> 2) * P_HALF + 2 * (k & 3), desc_hi);
                        const uint64_t v_desc = tc::desc_of(v_lo + 128 * k, desc_hi);
                        if (k == 0) tc::umma_bf16(tmem_o + h * 64, p_desc, v_desc, idesc_pv, j > 0 ? 1u : 0u);
                        else tc::umma_bf16_add(tmem_o + h * 64, p_desc, v_desc, idesc_pv);
                    }
                }
                tc::umma_commit(&s.kv_empty[st]);
                tc::umma_commit(&s.pv_done[j & 1]);
                if (++st == STAGES) st = 0;
                if (j + 1 < n_tiles && !ahead) ok = issue_qk(j + 1, true);
            }
            if (!ok) tc::give_up(abort_flag, p.status, tc::ST_MMA_TIMEOUT);
        }
    } else {
        // ---- softmax: warps 2..5, one thread per key = tensor-memory lane ----------------------
        const int quarter = warp & 3;
        const int t = quarter * 32 + lane;                       // key inside the tile
        const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
        float m_ref[RMAX], l_part[RMAX];
        int pos_of[RMAX], lo_of[RMAX];
#pragma unroll
        for (int r = 0; r < RMAX; ++r) {
            m_ref[r] = -INFINITY;
            l_part[r] = 0.f;
            // rows past the request's never pass the key test
            pos_of[r] = r < n_rows ? first_pos + r / n_rep : -1;
            lo_of[r] = (r < n_rows && p.window > 0) ? max(0, pos_of[r] - p.window + 1) : 0;
        }
        bool ok = true;
        auto wait_all = [&](uint64_t* bar, uint32_t parity) -> bool {
            bool got = tc::mbar_wait(bar, parity, abort_flag);
            if (!got && !*abort_flag) tc::give_up(abort_flag, p.status, tc::ST_EPILOGUE_TIMEOUT);
            return __all_sync(0xffffffffu, got);
        };
        for (int j = 0; j < n_tiles; ++j) {
            const int b = j & 1;
            const int key = tile0 + j * KEYS + t;
            float sc[RMAX];
            bool up = false;
            if (ok) ok = wait_all(&s.s_full[b], (j >> 1) & 1);
            if (ok) {
                tc::tc_fence_after_sync();
                uint32_t raw[16];
                tc::tmem_ld_32x16(tmem_s + b * 16 + lane_bits, raw);
                tc::tmem_ld_wait();
                tc::tc_fence_before_sync();
#pragma unroll
                for (int r = 0; r < RMAX; ++r) {
                    sc[r] = (key <= pos_of[r] && key >= lo_of[r]) ? __uint_as_float(raw[r]) * p.scale_log2
                                                                 : -INFINITY;
                    up |= sc[r] > m_ref[r] + RAISE;
                }
            }
            // every softmax thread passes these block barriers, whatever `ok` says
            if (softmax_any(up)) {
#pragma unroll
                for (int r = 0; r < RMAX; ++r) {
                    const float w = warp_max(ok ? sc[r] : -INFINITY);
                    if (lane == 0) s.red[quarter][r] = w;
                }
                softmax_barrier();
                float corr = 1.0f;                                // of row `lane`, for the rescale
#pragma unroll
                for (int r = 0; r < RMAX; ++r) {
                    const float mx = fmaxf(fmaxf(s.red[0][r], s.red[1][r]), fmaxf(s.red[2][r], s.red[3][r]));
                    const float m_new = fmaxf(m_ref[r], mx);
                    const float c = (m_ref[r] == -INFINITY) ? 0.f : ex2_fast(m_ref[r] - m_new);
                    l_part[r] *= c;
                    m_ref[r] = m_new;
                    if (r == lane) corr = c;
                }
                softmax_barrier();                                // `red` may be written again
                // the accumulator's rows follow their maxima: lanes 0..15 of tensor memory
                // belong to the warp whose quarter is 0
                if (quarter == 0 && j > 0 && ok) {
                    ok = wait_all(&s.pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1);
                    if (ok) {
                        tc::tc_fence_after_sync();
#pragma unroll 1
                        for (int c0c = 0; c0c < HD; c0c += 32) {
                            uint32_t v[32];
                            tc::tmem_ld_32x32(tmem_o + c0c, v);
                            tc::tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
                            tc::tmem_st_32x32(tmem_o + c0c, v);
                        }
                        tc::tmem_st_wait();
                        tc::tc_fence_before_sync();
                    }
                }
            }
            if (ok && j >= 2) ok = wait_all(&s.pv_done[b], ((j - 2) >> 1) & 1);   // P's buffer is free
            if (ok) {
                // P[r][key] = exp2(s - reference) as bf16: rows of 128 bytes per half of 64 keys
                uint8_t* half = s.p[b][t >> 6];
                const int piece = (t & 63) >> 3, within = (t & 7) * 2;
#pragma unroll
                for (int r = 0; r < RMAX; ++r) {
                    const float off = m_ref[r] == -INFINITY ? 0.f : m_ref[r];
                    const float e = ex2_fast(sc[r] - off);
                    l_part[r] += e;
                    *reinterpret_cast<__nv_bfloat16*>(half + r * 128 + ((piece ^ (r & 7)) << 4) + within) =
                        __float2bfloat16_rn(e);
                }
                tc::fence_proxy_async();
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(&s.p_full[b]);
            }
        }
        // ---- the chunk's result -------------------------------------------------------------
        if (ok) ok = wait_all(&s.pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1);
#pragma unroll
        for (int r = 0; r < RMAX; ++r) {
            float w = l_part[r];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
            if (lane == 0) s.red[quarter][r] = w;
        }
        softmax_barrier();
        if (quarter == 0 && ok) {
            // tensor-memory lanes 0..15 are the rows; the whole warp reads, rows' lanes write
            tc::tc_fence_after_sync();
            const int r = lane < n_rows ? lane : 0;
            const bool real = lane < n_rows;
            const float l = (s.red[0][r] + s.red[1][r]) + (s.red[2][r] + s.red[3][r]);
            float m = -INFINITY;
#pragma unroll
            for (int i = 0; i < RMAX; ++i)
                if (i == r) m = m_ref[i];
            const int tok = row_base + r / n_rep, head = kv_head * n_rep + r % n_rep;
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            float* part = p.partial + (((size_t)tok * p.n_heads + head) * p.n_chunks + chunk) * (HD + 2);
            __nv_bfloat16* dst = p.out + (size_t)tok * p.out_stride + (size_t)head * HD;
#pragma unroll 1
            for (int c0c = 0; c0c < HD; c0c += 32) {
                uint32_t v[32];
                tc::tmem_ld_32x32(tmem_o + c0c, v);
                tc::tmem_ld_wait();
                if (!real) continue;
                if (n_active == 1) {
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        __nv_bfloat162 o2 = __floats2bfloat162_rn(__uint_as_float(v[i]) * inv,
                                                                  __uint_as_float(v[i + 1]) * inv);
                        *reinterpret_cast<__nv_bfloat162*>(dst + c0c + i) = o2;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; i += 2)
                        *reinterpret_cast<float2*>(part + c0c + i) =
                            make_float2(__uint_as_float(v[i]), __uint_as_float(v[i + 1]));
                }
            }
            if (real && n_active > 1) {
                part[HD] = m;
                part[HD + 1] = l;
            }
            if (n_active > 1) {
                // This warp wrote the chunk's partial: it arrives for the block.  The warp's
                // stores are ordered before lane 0's arrival by the warp barrier; the arrival
                // releases them and acquires what the blocks that arrived before released.
                __syncwarp();
                if (lane == 0) {
                    int* counter = p.counters + req * p.n_kv_heads + kv_head;
                    int prev;
                    asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;"
                                 : "=r"(prev) : "l"(counter) : "memory");
                    if (prev == n_active - 1) {
                        *counter = 0;                     // ready for the next launch
                        s.is_last = 1;
                    }
                }
            }
        }
    }
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc::tc_fence_after_sync();
        tc::tmem_dealloc(s.tmem_base, TMEM_COLS);
    }
    // ---- the last block to arrive for these rows merges their chunks ------------------------
    // (what the arriving thread acquired holds for the whole block after the barrier above)
    if (n_active == 1 || *abort_flag || !s.is_last) return;
    for (int r = warp; r < n_rows; r += 6) {
        const int tok = row_base + r / n_rep, head = kv_head * n_rep + r % n_rep;
        merge_row<HD>(p, tok, head, first_pos + r / n_rep, lane);
    }
}

template <int HD, int RMAX, int STAGES>
int launch_stages(dim3 grid, cudaStream_t st, const CUtensorMap& mk, const CUtensorMap& mv,
                  const CUtensorMap& rk, const CUtensorMap& rv, const DecodeParams& p) {
    const int smem = (int)sizeof(Storage<HD, STAGES>);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_decode_tcgen05_kernel<HD, RMAX, STAGES>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cb_launch(attention_decode_tcgen05_kernel<HD, RMAX, STAGES>, grid, dim3(192), smem, st, mk, mv, rk, rv, p);
    return cb_last_error();
}

template <int HD, int RMAX>
int launch_as(dim3 grid, cudaStream_t st, const CUtensorMap& mk, const CUtensorMap& mv,
              const CUtensorMap& rk, const CUtensorMap& rv, const DecodeParams& p) {
    // chunks of at most two tiles never use a third stage
    if (HD == 64 && p.chunk_keys <= 2 * KEYS) return launch_stages<HD, RMAX, 2>(grid, st, mk, mv, rk, rv, p);
    return launch_stages<HD, RMAX, MAX_STAGES>(grid, st, mk, mv, rk, rv, p);
}

}  // namespace

// Attention for a step whose requests bring at most 16 (token, head of a group)
// rows each.  k_cache / v_cache: [n_pages][n_kv_heads][page_tokens][head_dim] bf16.
// partial: n_tokens * n_heads * n_chunks * (head_dim + 2) floats; counters: n_requests *
// n_kv_heads ints, zero before the first launch (the kernel leaves them zero).
CB_EXPORT int cb_attention_decode_tcgen05(const void* qkv, int qkv_stride, void* out, int out_stride,
                                          const void* k_cache, const void* v_cache, int n_pages,
                                          const int* req_row_start, const int* req_first_pos,
                                          const int* block_table, int table_stride, int n_requests,
                                          int max_new_tokens, int n_heads, int n_kv_heads,
                                          int head_dim, int page_tokens, float scale, int window,
                                          float* partial, int* counters, int n_chunks,
                                          int chunk_keys, int* status, void* stream) {
    if (n_requests <= 0 || max_new_tokens <= 0) return 0;
    if ((head_dim != 64 && head_dim != 128) || n_heads % n_kv_heads != 0 || page_tokens < 8 || page_tokens > KEYS ||
        (page_tokens & (page_tokens - 1)) || (qkv_stride & 7) || (out_stride & 1) ||
        ((uintptr_t)qkv & 15) || ((uintptr_t)out & 3) || ((uintptr_t)k_cache & 15) ||
        ((uintptr_t)v_cache & 15) || max_new_tokens * (n_heads / n_kv_heads) > ROWS ||
        n_chunks <= 0 || chunk_keys <= 0 || chunk_keys % KEYS != 0 || !partial || !counters)
        return CB_ERR_UNSUPPORTED;
    int shift = 0;
    while ((1 << shift) < page_tokens) ++shift;
    CUtensorMap mk, mv;
    const uint64_t rows = (uint64_t)n_pages * n_kv_heads * page_tokens;
    if (!tc::make_map_2d(&mk, k_cache, rows, head_dim, head_dim, page_tokens)) return CB_ERR_UNSUPPORTED;
    if (!tc::make_map_2d(&mv, v_cache, rows, head_dim, head_dim, page_tokens)) return CB_ERR_UNSUPPORTED;
    // tiles of several pages: a second pair of maps that takes a run of pages at once
    CUtensorMap rk = mk, rv = mv;
    const int pages_per_tile = KEYS / page_tokens;
    const bool runs = pages_per_tile > 1 &&
                      tc::make_map_pages(&rk, k_cache, n_pages, n_kv_heads, page_tokens, head_dim, pages_per_tile) &&
                      tc::make_map_pages(&rv, v_cache, n_pages, n_kv_heads, page_tokens, head_dim, pages_per_tile);
    DecodeParams p;
    p.n_pages = n_pages;
    p.runs = runs ? 1 : 0;
    p.qkv = (const __nv_bfloat16*)qkv;
    p.qkv_stride = qkv_stride;
    p.out = (__nv_bfloat16*)out;
    p.out_stride = out_stride;
    p.req_row_start = req_row_start;
    p.req_first_pos = req_first_pos;
    p.block_table = block_table;
    p.table_stride = table_stride;
    p.n_heads = n_heads;
    p.n_kv_heads = n_kv_heads;
    p.n_rep = n_heads / n_kv_heads;
    p.n_requests = n_requests;
    p.page_shift = shift;
    p.scale_log2 = scale * LOG2E;
    p.window = window;
    p.partial = partial;
    p.counters = counters;
    p.n_chunks = n_chunks;
    p.chunk_keys = chunk_keys;
    p.status = status;
    const int most_rows = max_new_tokens * (n_heads / n_kv_heads);
    if (n_kv_heads > 65535 || n_requests > 65535) return CB_ERR_UNSUPPORTED;
    const dim3 grid(n_chunks, n_kv_heads, n_requests);
    cudaStream_t st = (cudaStream_t)stream;
    if (head_dim == 64) {
        if (most_rows <= 4) return launch_as<64, 4>(grid, st, mk, mv, rk, rv, p);
        if (most_rows <= 8) return launch_as<64, 8>(grid, st, mk, mv, rk, rv, p);
        return launch_as<64, 16>(grid, st, mk, mv, rk, rv, p);
    }
    if (most_rows <= 4) return launch_as<128, 4>(grid, st, mk, mv, rk, rv, p);
    if (most_rows <= 8) return launch_as<128, 8>(grid, st, mk, mv, rk, rv, p);
    return launch_as<128, 16>(grid, st, mk, mv, rk, rv, p);
}
