// Paged causal attention for portions of prompts on the 5th-generation tensor
// cores (head size 64 or 128, bfloat16): S = Q K^T and O += P V are tcgen05.mma with
// the scores and the output accumulator in tensor memory; K and V pages come in
// by TMA; the softmax runs on four warps, one thread per query row, reading S
// from tensor memory and writing P (bf16) to shared memory for the second MMA.
//
// A block takes 128 query rows of one request and one KV head; rows are
// (position, head within the group) pairs, so every query head that shares the
// KV head uses the same K and V tiles.  It walks the keys in tiles of 128.
// Roles: warp 0 loads (one thread: block-table lookups, then one TMA box per tile and
// operand where the tile's pages follow one another in the pool, else one per page),
// warp 1 owns tensor memory and issues the MMAs, warps 2-5 are the softmax.
// S and P are double-buffered: while the softmax works on tile j, the first MMA
// of tile j+1 and the second MMA of tile j-1 run, so a block's time per tile is
// the softmax's alone (about 2,000 cycles: 1,260 for the 128 exponentials per thread,
// their sums and P's way to shared memory, in which the special-function unit's 560 and
// the other pipes' instructions add up instead of overlapping; the rest maxima, barrier
// tests of 100 to 200 cycles each, and the scores' way out of tensor memory).
// Head size 64 with an SM to the block: two such groups of four softmax warps take the
// tiles in turn (tile j: group j % 2), each with its own buffer of scores and of P, its own
// reference maximum, sum and accumulator, merged when the keys are through; two tiles are
// then in work at a time (one group's exponentials beside the other's maxima and waits:
// 1,750 cycles a tile), and a second thread, of a warp of its own, sends the second products,
// since one thread cannot send both products of two tiles in time (1,200 cycles a tile).
//
// Running maximum: a row keeps a reference maximum that is only raised when the
// tile's maximum exceeds it by more than 2^8 (in the base-2 exponent), so P
// stays <= 256 and the accumulator in tensor memory is rescaled rarely; the row
// sum uses the same reference, and the final division makes the result the
// exact softmax-weighted mean whatever the reference was.
//
// Sizes: head size 64 or 128; page size a power of two from 8 to 128; any head
// counts and group sizes; window.  Anything else is refused and the mma.sync
// kernel runs.  Every wait is bounded (tc_common.cuh).
// Reference counterpart: `attention_prefill_exact_*`
// (engine/kernels/kernels.cu:2257-2275).
#define CB_PDL_BIT 1      // this file's bit in CRUCIBLE_PDL
#include "common.cuh"
#include "tc_common.cuh"

namespace {

constexpr int ROWS = 128;            // query rows per block = tensor-memory lanes
constexpr int KEYS = 128;            // keys per tile
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RAISE = 8.0f;        // raise the reference maximum when exceeded by 2^8

struct TcAttnParams {
    const __nv_bfloat16* qkv;
    int qkv_stride;
    __nv_bfloat16* out;
    int out_stride;
    const int* req_row_start;
    const int* req_first_pos;
    const int* block_table;
    int table_stride;
    int n_heads, n_kv_heads, n_rep, n_requests, page_tokens, page_shift;
    float scale_log2;
    int window;
    int n_pages;             // of the pool
    int runs;                // 1: the 4-D maps may be used for tiles whose pages are consecutive
    int* status;
};

// HD: the head size, 64 or 128.  Operands whose contracted or free dimension is the head
// size lie in shared memory as HD / 64 halves of [rows][128 bytes] (one swizzle atom wide).
// Head size 64 has two forms.  The roomy one: four K/V stages, two P buffers, two buffers of
// scores, two softmax groups, an SM to itself (210 KB, 384 columns of tensor memory: with two
// tiles in work a tile's keys are asked for three tiles ahead); it is the quicker block,
// and the right one while all blocks of a launch find a place at once.  The lean one: two
// stages, one P buffer, one buffer of scores (112 KB, 256 columns), so that two blocks share
// an SM and one's waits (for a copy, an MMA, the scores' way out of tensor memory) are filled
// by the other's exponentials; its one buffer of scores is handed back to the MMA thread as
// soon as the softmax has the scores in registers, so the next tile's first MMA still runs
// beside this tile's softmax.  It was the right one for launches with more blocks than places
// while the roomy form had one softmax group (4,096-token prompt of the 120M shape 1.84 against
// 2.01 ms); with two groups the roomy form is quicker there too (1.68 ms) and the launcher
// takes it unless told otherwise.  Head size 128: two stages and one P buffer (what 227 KB hold).
template <int HD, bool LEAN>
struct Storage {
    static constexpr int STAGES = (HD == 64 && !LEAN) ? 4 : 2;
    static constexpr int PB = (HD == 64 && !LEAN) ? 2 : 1;
    static constexpr int S_BUFS = LEAN ? 1 : 2;
    // softmax groups of four warps that take the tiles in turn (tile j: group j % GROUPS), each
    // with its own reference maximum, sum and accumulator, merged at the end
    static constexpr int GROUPS = (HD == 64 && !LEAN) ? 2 : 1;
    // loader, MMA thread, four softmax warps a group; two groups: a warp for a second MMA thread
    static constexpr int THREADS = GROUPS > 1 ? 64 + 128 * GROUPS + 32 : 192;
    alignas(1024) uint8_t q[HD / 64][ROWS * 64 * 2];
    alignas(1024) uint8_t k[STAGES][HD / 64][KEYS * 64 * 2];
    alignas(1024) uint8_t v[STAGES][HD / 64][KEYS * 64 * 2];
    alignas(1024) uint8_t p[PB][2][ROWS * 64 * 2];  // P: buffers of two halves of 64 keys
    alignas(8) uint64_t kv_full[STAGES];
    uint64_t kv_empty[STAGES];
    uint64_t s_full[2], p_full[2], pv_done[2];
    uint64_t s_free;                                // lean form: a tile's scores are in registers
    uint64_t s_taken[2];                            // two groups: buffer b's scores are in registers
    float2 merge[2][ROWS];                          // two groups: a row's (reference, sum) of each
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// 2^x by the special-function unit, flushing denormals: the argument is a score
// minus a maximum, so a result below 2^-126 counts as nothing in the row's sum.
__device__ __forceinline__ float ex2_fast(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// (x0, x1) * a + b in one instruction on the pair
__device__ __forceinline__ void fma_pair(float& x0, float& x1, float a, float b) {
    asm("{\n\t"
        ".reg .b64 x, s, o;\n\t"
        "mov.b64 x, {%0, %1};\n\t"
        "mov.b64 s, {%2, %2};\n\t"
        "mov.b64 o, {%3, %3};\n\t"
        "fma.rn.f32x2 x, x, s, o;\n\t"
        "mov.b64 {%0, %1}, x;\n\t"
        "}"
        : "+f"(x0), "+f"(x1)
        : "f"(a), "f"(b));
}

template <int HD, bool LEAN>
__global__ void __launch_bounds__(Storage<HD, LEAN>::THREADS, LEAN ? 2 : 1)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap map_k,
                         const __grid_constant__ CUtensorMap map_v,
                         const __grid_constant__ CUtensorMap run_k,
                         const __grid_constant__ CUtensorMap run_v, const TcAttnParams p) {
    // 1024-byte alignment (the swizzled tiles need it) is asked of the declaration
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    using Store = Storage<HD, LEAN>;
    constexpr int STAGES = Store::STAGES, PB = Store::PB, NH = HD / 64, S_BUFS = Store::S_BUFS;
    constexpr int GROUPS = Store::GROUPS;
    constexpr int PV_WARP = GROUPS > 1 ? 2 + 4 * GROUPS : -1;    // the second MMA thread's warp
    static_assert(GROUPS == 1 || (PB == 2 && S_BUFS == 2 && HD == 64), "two groups: a buffer of scores, of P and an accumulator each");
    constexpr uint32_t TMEM_COLS = LEAN ? 256 : 512;     // scores: 128 columns a buffer, then O
    Store& s = *reinterpret_cast<Store*>(smem_raw);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // grid (heads, requests, tile ranks), the tile rank slowest: blocks start in order of
    // weight over the whole launch, the longest rows first (and no thread divides by a run-time
    // value to find its place: that costs about a hundred cycles each time)
    const int kv_head = blockIdx.x, req = blockIdx.y, rank = blockIdx.z;
    volatile int* abort_flag = &s.abort_flag;

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
        tc::mbar_init(&s.s_free, 4);
        tc::mbar_init(&s.s_taken[0], 4);
        tc::mbar_init(&s.s_taken[1], 4);
        s.abort_flag = 0;
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&map_k);
        tc::prefetch_tensormap(&map_v);
        if (p.runs) {
            tc::prefetch_tensormap(&run_k);
            tc::prefetch_tensormap(&run_v);
        }
    }
    if (warp == 1) {
        tc::tmem_alloc(&s.tmem_base, TMEM_COLS);
        tc::tmem_relinquish();
    }
    // What follows reads the step's metadata, which was uploaded before the step began: the
    // kernels ahead in the stream write none of it, so it is read, and the first tiles'
    // table entries looked up, before the wait for them.
    const int n_rep = p.n_rep;
    const int row_base = p.req_row_start[req];
    const int n_new = p.req_row_start[req + 1] - row_base;
    const int n_rows = n_new * n_rep;
    const int q_tiles = (n_rows + ROWS - 1) / ROWS;
    const bool active = rank < q_tiles;
    const int qt = active ? q_tiles - 1 - rank : 0;               // heaviest tiles first
    const int first_pos = p.req_first_pos[req];
    const int* table = p.block_table + (size_t)req * p.table_stride;

    // the block's keys: from the first key any of its rows may read to its last position
    const int last_row = min(n_rows - 1, qt * ROWS + ROWS - 1);
    const int max_pos = first_pos + last_row / n_rep;
    const int min_pos = first_pos + (qt * ROWS) / n_rep;
    int key_lo = p.window > 0 ? max(0, min_pos - p.window + 1) : 0;
    key_lo = key_lo / KEYS * KEYS;
    const int key_end = max_pos + 1;
    const int n_tiles = active ? (key_end - key_lo + KEYS - 1) / KEYS : 0;

    // ---- the loader's thread: one tile of K and V pages into a stage --------------------------
    const int pages_per_tile = KEYS >> p.page_shift;
    auto lookup = [&](int j, int (&pages)[16]) {
        // the tile's table entries, all in flight at once: the copies are ordered against
        // memory and would take the lookups one by one
        const int key0 = key_lo + j * KEYS;
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
        // pages that follow one another in the pool come in with one copy per tile and operand
        // (sending a copy costs this thread about 60 cycles whatever the copy's size, and the
        // arithmetic around it more)
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

    // ---- the query rows, by warps 1..5: 16-byte pieces into the 128-byte swizzle; warp 0's
    // thread meanwhile starts the first tiles' copies, which wait for nothing -----------------
    if (warp == 0) {
        if (lane == 0) {
            // the first tiles: all their lookups before the wait, then all their copies (the
            // keys of this step's own tokens are written by the product before this kernel)
            int first[STAGES][16];
#pragma unroll
            for (int j = 0; j < STAGES; ++j)
                if (j < early) lookup(j, first[j]);
            cb_pdl_wait();
#pragma unroll
            for (int j = 0; j < STAGES; ++j)
                if (j < early) issue(j, first[j]);
        } else {
            cb_pdl_wait();
        }
    } else {
        cb_pdl_wait();
        if (active)
        for (int i = threadIdx.x - 32; i < ROWS * 8 * NH; i += blockDim.x - 32) {
            const int r = i / (8 * NH), c = i % (8 * NH);         // row, 16-byte piece of the row
            const int row = qt * ROWS + r;
            uint4 val = make_uint4(0, 0, 0, 0);
            if (row < n_rows) {
                const int tok = row_base + row / n_rep, head = kv_head * n_rep + row % n_rep;
                val = *reinterpret_cast<const uint4*>(p.qkv + (size_t)tok * p.qkv_stride +
                                                      (size_t)head * HD + c * 8);
            }
            *reinterpret_cast<uint4*>(s.q[c >> 3] + r * 128 + (((c & 7) ^ (r & 7)) << 4)) = val;
        }
    }
    tc::fence_proxy_async();                // generic-proxy writes of Q, before the MMAs read them
    tc::tc_fence_before_sync();
    __syncthreads();
    tc::tc_fence_after_sync();
    // only now may the kernel after this one start: every block of this one holds its tensor
    // memory by now, so a successor that asks for tensor memory queues behind it
    cb_pdl_trigger();
    const uint32_t tmem_s = s.tmem_base;          // + 128 for the second buffer
    const uint32_t tmem_o = s.tmem_base + S_BUFS * 128;

    if (warp == 0) {
        // ---- loader: the remaining tiles, each once its stage has been read ------------------
        if (lane == 0 && n_tiles > 0) {
            int armed = early;
            for (int j = early; j < n_tiles; ++j) {
                int pages[16];
                lookup(j, pages);
                if (!issue(j, pages)) break;
                armed = j + 1;
            }
            if (*abort_flag) {
                const int first = armed > STAGES ? armed - STAGES : 0;
                for (int j = first; j < armed; ++j)
                    for (uint32_t t = 0; t < tc::WAIT_LIMIT; ++t)
                        if (tc::mbar_try_wait(&s.kv_full[j % STAGES], (j / STAGES) & 1)) break;
            }
        }
    } else if (warp == 1 || warp == PV_WARP) {
        // ---- MMA issuer: one thread; with two softmax groups two, of different warps: warp 1's
        // sends the first products (scores), the last warp's the second (P V).  Sending twelve
        // MMAs, three commits and the barrier tests between them costs a thread some 1,200
        // cycles a tile, and two groups want a tile every 1,400: one thread would make each
        // product wait for the other.
        if (lane == 0 && n_tiles > 0) {
            constexpr uint32_t idesc_qk = tc::instr_desc_bf16(ROWS, KEYS);
            constexpr uint32_t idesc_pv = tc::instr_desc_bf16_b_mn(ROWS, 64);
            // Operand descriptors by addition: the low word carries the address in 16-byte
            // units, the high word is the same for every tile; stages and parities are carried
            // along.  This thread's own instructions are what a tile's MMAs take (sending one
            // costs 54 cycles, a dependent integer instruction about 5).
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
            // S_j = Q K_j^T into buffer j % S_BUFS: the head size in steps of 16
            int qk_st = 0;                        // stage and parity of the next tile of scores
            uint32_t qk_parity = 0;
            auto send_qk = [&](int j) {
                tc::tc_fence_after_sync();
                const uint32_t k_lo = k_lo0 + qk_st * KV_STAGE;
                const uint32_t d_s = tmem_s + (j % S_BUFS) * 128;
#pragma unroll
                for (int k = 0; k < HD / 16; ++k) {
                    const uint64_t q_desc = tc::desc_of(q_lo + (k >> 2) * Q_HALF + 2 * (k & 3), desc_hi);
                    const uint64_t k_desc = tc::desc_of(k_lo + (k >> 2) * KV_HALF + 2 * (k & 3), desc_hi);
                    if (k == 0) tc::umma_bf16(d_s, q_desc, k_desc, idesc_qk, 0u);
                    else tc::umma_bf16_add(d_s, q_desc, k_desc, idesc_qk);
                }
                tc::umma_commit(&s.s_full[j % S_BUFS]);
                if (++qk_st == STAGES) qk_st = 0, qk_parity ^= 1;
            };
            // `block`: wait for the tile; else only take it if it has landed (true: issued)
            auto issue_qk = [&](int j, bool block) -> bool {
                // one buffer of scores: the softmax of tile j - 1 must have them in registers
                const bool hand_back = S_BUFS == 1 && j > 0;
                if (block) {
                    if (!tc::mbar_wait(&s.kv_full[qk_st], qk_parity, abort_flag)) return false;
                    if (hand_back && !tc::mbar_wait(&s.s_free, (j - 1) & 1, abort_flag)) return false;
                } else if (!tc::mbar_try_wait(&s.kv_full[qk_st], qk_parity) ||
                           (hand_back && !tc::mbar_try_wait(&s.s_free, (j - 1) & 1))) {
                    return false;
                }
                send_qk(j);
                return true;
            };
            // O += P_j V_j: 128 keys in eight steps of 16, 64 output features at a time
            int st = 0;                           // stage of the next tile's values
            auto send_pv = [&](int j) {
                const int pb = j % PB;
                tc::tc_fence_after_sync();
                const uint32_t p_lo = p_lo0 + pb * P_BUF;
#pragma unroll
                for (int h = 0; h < NH; ++h) {
                    const uint32_t v_lo = v_lo0 + st * KV_STAGE + h * KV_HALF;
                    // (two groups: head size 64, so h is 0; a group's accumulator is 64 columns on)
                    const uint32_t d_o = tmem_o + (GROUPS > 1 ? (uint32_t)(j % GROUPS) * 64 : (uint32_t)h * 64);
#pragma unroll
                    for (int k = 0; k < KEYS / 16; ++k) {
                        // 16 keys further down V: 16 rows of 128 bytes = 128 descriptor units
                        const uint64_t p_desc = tc::desc_of(p_lo + (k >> 2) * P_HALF + 2 * (k & 3), desc_hi);
                        const uint64_t v_desc = tc::desc_of(v_lo + 128 * k, desc_hi);
                        if (k == 0) tc::umma_bf16(d_o, p_desc, v_desc, idesc_pv, j >= GROUPS ? 1u : 0u);
                        else tc::umma_bf16_add(d_o, p_desc, v_desc, idesc_pv);
                    }
                }
                tc::umma_commit(&s.kv_empty[st]);
                tc::umma_commit(&s.pv_done[pb]);
                if (++st == STAGES) st = 0;
            };
            if (GROUPS > 1) {
                // Two groups of softmax warps take the tiles in turn, so two tiles are in work
                // at a time.  A tile's first product goes out as soon as its keys have landed
                // and the scores that its buffer held (two tiles earlier) are in registers; its
                // second once its P is written.
                if (warp == 1) {
                    for (int j = 0; j < n_tiles && ok; ++j) {
                        ok = tc::mbar_wait(&s.kv_full[qk_st], qk_parity, abort_flag) &&
                             (j < 2 || tc::mbar_wait(&s.s_taken[j & 1], ((j - 2) >> 1) & 1, abort_flag));
                        if (ok) send_qk(j);
                    }
                } else {
                    for (int j = 0; j < n_tiles && ok; ++j) {
                        ok = tc::mbar_wait(&s.p_full[j & 1], (j >> 1) & 1, abort_flag);
                        if (ok) send_pv(j);
                    }
                }
            } else {
                ok = issue_qk(0, true);
                for (int j = 0; j < n_tiles && ok; ++j) {
                    // the next tile's scores go out first if its keys have landed (their buffer
                    // was last read by the softmax of tile j - 1, whose P this thread has waited
                    // for); else after this tile's second product, which must not wait for a copy
                    bool ahead = j + 1 < n_tiles && issue_qk(j + 1, false);
                    // With one buffer of scores the next tile's first MMA may go as soon as this
                    // tile's softmax has the scores in registers, which happens during this wait.
                    bool got = false;
                    for (uint32_t i = 0; i < tc::WAIT_LIMIT && !got; ++i) {
                        got = tc::mbar_try_wait(&s.p_full[j % PB], (j / PB) & 1);
                        if (S_BUFS == 1 && !got && !ahead && j + 1 < n_tiles) ahead = issue_qk(j + 1, false);
                        if ((i & 1023u) == 1023u && *abort_flag) break;
                    }
                    if (!got) {
                        ok = false;
                        break;
                    }
                    send_pv(j);
                    if (j + 1 < n_tiles && !ahead) ok = issue_qk(j + 1, true);
                }
            }
            if (!ok) tc::give_up(abort_flag, p.status, tc::ST_MMA_TIMEOUT);
        }
    } else if (warp < 2 + 4 * GROUPS) {
        // ---- softmax: warps 2..5 (and 6..9: the second group), one thread per row =
        // tensor-memory lane; a group takes every GROUPS-th tile -------------------------------
        const int quarter = warp & 3;
        const int group = GROUPS > 1 ? (warp - 2) >> 2 : 0;
        const uint32_t tmem_mine = tmem_o + (uint32_t)group * 64;
        const int r = quarter * 32 + lane;
        const int row = qt * ROWS + r;
        const bool real = active && row < n_rows;
        // rows past the request's last are computed like rows that may read every key (their
        // queries are zero) and are not stored: they keep a tile's fast path open
        const int pos = real ? first_pos + row / n_rep : (1 << 30);
        const int lo = real && p.window > 0 ? max(0, pos - p.window + 1) : 0;
        const uint32_t lane_bits = (uint32_t)(quarter * 32) << 16;
        float m_ref = -INFINITY, l = 0.f;
        bool ok = true;
        auto wait_all = [&](uint64_t* bar, uint32_t parity) -> bool {
            bool got = tc::mbar_wait(bar, parity, abort_flag);
            if (!got && !*abort_flag) tc::give_up(abort_flag, p.status, tc::ST_EPILOGUE_TIMEOUT);
            return __all_sync(0xffffffffu, got);
        };
        for (int j = group; j < n_tiles && ok; j += GROUPS) {
            const int key0 = key_lo + j * KEYS;
            const int b = j % S_BUFS;                 // the scores' buffer
            const int pb = j % PB;                    // P's buffer
            ok = wait_all(&s.s_full[b], (j / S_BUFS) & 1);
            if (!ok) break;
            tc::tc_fence_after_sync();
            // the row's 128 scores, once, into registers
            uint32_t sv[4][32];
#pragma unroll
#pragma unroll
            for (int c = 0; c < 4; ++c) tc::tmem_ld_32x32(tmem_s + b * 128 + lane_bits + c * 32, sv[c]);
            tc::tmem_ld_wait();
            tc::tc_fence_before_sync();
            if (S_BUFS == 1 || GROUPS > 1) {          // the buffer may take the next tile's scores
                __syncwarp();
                if (lane == 0) tc::mbar_arrive(GROUPS > 1 ? &s.s_taken[b] : &s.s_free);
            }
            // keys of this tile the row may read: [first, last] relative to key0.  Most tiles
            // lie wholly inside every row's range and skip the test.
            const int last = min(pos - key0, KEYS - 1);
            const int first = max(lo - key0, 0);
            if (!__all_sync(0xffffffffu, last == KEYS - 1 && first == 0)) {
#pragma unroll
                for (int c = 0; c < 4; ++c)
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int kk = c * 32 + i;
                        if (kk > last || kk < first) sv[c][i] = __float_as_uint(-INFINITY);
                    }
            }
            float mc[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                mc[c] = -INFINITY;
#pragma unroll
                for (int i = 0; i < 32; i += 2)
                    mc[c] = max3(mc[c], __uint_as_float(sv[c][i]), __uint_as_float(sv[c][i + 1]));
            }
            float mx = fmaxf(fmaxf(mc[0], mc[1]), fmaxf(mc[2], mc[3]));
            mx *= p.scale_log2;
            // raise the reference maximum only when it is exceeded by far; the accumulator
            // in tensor memory is rescaled then, by the whole warp at once, after the
            // second MMA of the tile before has finished
            float corr = 1.0f;
            if (mx > m_ref + RAISE || (m_ref == -INFINITY && mx > -INFINITY)) {
                corr = m_ref == -INFINITY ? 0.f : exp2f(m_ref - mx);
                m_ref = mx;
            }
            if (j >= GROUPS && __any_sync(0xffffffffu, corr != 1.0f)) {
                ok = wait_all(&s.pv_done[(j - GROUPS) % PB], ((j - GROUPS) / PB) & 1);
                if (!ok) break;
                tc::tc_fence_after_sync();
#pragma unroll 1
                for (int c0 = 0; c0 < HD; c0 += 32) {
                    uint32_t v[32];
                    tc::tmem_ld_32x32(tmem_mine + lane_bits + c0, v);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * corr);
                    tc::tmem_st_32x32(tmem_mine + lane_bits + c0, v);
                }
                tc::tmem_st_wait();
                tc::tc_fence_before_sync();
            }
            l *= corr;
            // P's buffer was last read by the second MMA of tile j - PB.  With two buffers and
            // one group that MMA was sent before this tile's first one, and the commit that
            // announced this tile's scores covers everything its thread had sent by then:
            // nothing to wait for (a barrier test costs a warp 100 to 200 cycles even when it
            // passes).  With two groups this tile's first MMA may have gone out earlier.
            if ((PB == 1 || GROUPS > 1) && j >= PB) {
                ok = wait_all(&s.pv_done[pb], ((j - PB) / PB) & 1);
                if (!ok) break;
            }
            // P = exp2(s * scale - reference), to shared memory in the layout the second MMA
            // reads (rows of 128 bytes per half of 64 keys, 128-byte swizzle)
            const float off = m_ref == -INFINITY ? 0.f : -m_ref;
            float sum[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint8_t* half = s.p[pb][c >> 1] + r * 128;
#pragma unroll
                for (int piece = 0; piece < 4; ++piece) {
                    float e[8];
#pragma unroll
                    for (int i = 0; i < 8; i += 2) {
                        e[i] = __uint_as_float(sv[c][8 * piece + i]);
                        e[i + 1] = __uint_as_float(sv[c][8 * piece + i + 1]);
                        fma_pair(e[i], e[i + 1], p.scale_log2, off);
                        e[i] = ex2_fast(e[i]);
                        e[i + 1] = ex2_fast(e[i + 1]);
                        sum[i >> 1] += e[i] + e[i + 1];
                    }
                    uint4 w;
                    w.x = pack_bf16(e[0], e[1]);
                    w.y = pack_bf16(e[2], e[3]);
                    w.z = pack_bf16(e[4], e[5]);
                    w.w = pack_bf16(e[6], e[7]);
                    const int pc = (c & 1) * 4 + piece;              // 16-byte piece inside the row
                    *reinterpret_cast<uint4*>(half + ((pc ^ (r & 7)) << 4)) = w;
                }
            }
            l += (sum[0] + sum[1]) + (sum[2] + sum[3]);
            tc::fence_proxy_async();             // P is written by the generic proxy, read by the MMA
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&s.p_full[pb]);
        }
        // ---- the output: O / l ------------------------------------------------------------
        // the group's last tile
        const int my_tiles = n_tiles > group ? (n_tiles - group + GROUPS - 1) / GROUPS : 0;
        const int j_last = group + (my_tiles - 1) * GROUPS;
        if (ok && my_tiles > 0) ok = wait_all(&s.pv_done[j_last % PB], (j_last / PB) & 1);
        __nv_bfloat16* dst = nullptr;
        if (real) {
            const int tok = row_base + row / n_rep, head = kv_head * n_rep + row % n_rep;
            dst = p.out + (size_t)tok * p.out_stride + (size_t)head * HD;
        }
        if (GROUPS > 1) {
            // Two groups: each holds the sums over its own tiles against its own reference.
            // A row's two states meet in shared memory; every thread comes to the barrier,
            // whatever happened to its waits.  Then group g writes features [32 g, 32 g + 32).
            s.merge[group][r] = make_float2(my_tiles > 0 ? m_ref : -INFINITY, my_tiles > 0 ? l : 0.f);
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (ok && n_tiles > 0 && !*abort_flag) {
                tc::tc_fence_after_sync();
                const float2 other = s.merge[group ^ 1][r];
                const float m_mine = my_tiles > 0 ? m_ref : -INFINITY;
                const float m_all = fmaxf(m_mine, other.x);
                const float f_mine = m_mine == -INFINITY ? 0.f : exp2f(m_mine - m_all);
                const float f_other = other.x == -INFINITY ? 0.f : exp2f(other.x - m_all);
                const float l_all = (my_tiles > 0 ? l : 0.f) * f_mine + other.y * f_other;
                const float inv = l_all > 0.f ? 1.0f / l_all : 0.f;
                const float w_mine = f_mine * inv, w_other = f_other * inv;
                const int c0 = group * 32;
                uint32_t a[32], b[32];
                // An accumulator that no MMA has written holds whatever was there and is not
                // read.  Whether a group had tiles is the same for every thread of the block,
                // as it must be: the loads are the whole warp's (.sync.aligned).  A row that
                // could read none of a group's keys has weight 0 and finite sums (zeros) there.
                const bool mine_any = my_tiles > 0, other_any = n_tiles > my_tiles;
                if (mine_any) tc::tmem_ld_32x32(tmem_mine + lane_bits + c0, a);
                if (other_any) tc::tmem_ld_32x32(tmem_o + (uint32_t)(group ^ 1) * 64 + lane_bits + c0, b);
                tc::tmem_ld_wait();
                if (real) {
                    float o[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        o[i] = (mine_any ? __uint_as_float(a[i]) * w_mine : 0.f) +
                               (other_any ? __uint_as_float(b[i]) * w_other : 0.f);
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 w;
                        w.x = pack_bf16(o[8 * q4 + 0], o[8 * q4 + 1]);
                        w.y = pack_bf16(o[8 * q4 + 2], o[8 * q4 + 3]);
                        w.z = pack_bf16(o[8 * q4 + 4], o[8 * q4 + 5]);
                        w.w = pack_bf16(o[8 * q4 + 6], o[8 * q4 + 7]);
                        *reinterpret_cast<uint4*>(dst + c0 + 8 * q4) = w;
                    }
                }
            }
        } else if (ok && n_tiles > 0) {
            tc::tc_fence_after_sync();
            const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll 1
            for (int c0 = 0; c0 < HD; c0 += 32) {
                uint32_t v[32];
                tc::tmem_ld_32x32(tmem_o + lane_bits + c0, v);
                tc::tmem_ld_wait();
                if (real) {
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 w;
                        w.x = pack_bf16(__uint_as_float(v[8 * q4 + 0]) * inv, __uint_as_float(v[8 * q4 + 1]) * inv);
                        w.y = pack_bf16(__uint_as_float(v[8 * q4 + 2]) * inv, __uint_as_float(v[8 * q4 + 3]) * inv);
                        w.z = pack_bf16(__uint_as_float(v[8 * q4 + 4]) * inv, __uint_as_float(v[8 * q4 + 5]) * inv);
                        w.w = pack_bf16(__uint_as_float(v[8 * q4 + 6]) * inv, __uint_as_float(v[8 * q4 + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c0 + 8 * q4) = w;
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
}

template <int HD, bool LEAN>
int launch_as(dim3 grid, cudaStream_t st, const CUtensorMap& mk, const CUtensorMap& mv,
              const CUtensorMap& rk, const CUtensorMap& rv, const TcAttnParams& p) {
    const int smem = (int)sizeof(Storage<HD, LEAN>);
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel<HD, LEAN>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    cb_launch(attention_tcgen05_kernel<HD, LEAN>, grid, dim3(Storage<HD, LEAN>::THREADS), smem, st, mk, mv, rk,
              rv, p);
    return cb_last_error();
}

}  // namespace

// Attention for the rows of a step whose requests bring portions of prompts.
// k_cache / v_cache: [n_pages][n_kv_heads][page_tokens][head_dim] bf16; head_dim 64 or 128.
CB_EXPORT int cb_attention_tcgen05(const void* qkv, int qkv_stride, void* out, int out_stride,
                                   const void* k_cache, const void* v_cache, int n_pages,
                                   const int* req_row_start, const int* req_first_pos,
                                   const int* block_table, int table_stride, int n_requests,
                                   int max_new_tokens, int n_heads, int n_kv_heads, int head_dim,
                                   int page_tokens, float scale, int window, int lean, int* status,
                                   void* stream) {
    if (n_requests <= 0 || max_new_tokens <= 0) return 0;
    if ((head_dim != 64 && head_dim != 128) || n_heads % n_kv_heads != 0 || page_tokens < 8 || page_tokens > KEYS ||
        (page_tokens & (page_tokens - 1)) || (qkv_stride & 7) || (out_stride & 7) ||
        ((uintptr_t)qkv & 15) || ((uintptr_t)out & 15) || ((uintptr_t)k_cache & 15) ||
        ((uintptr_t)v_cache & 15))
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
    TcAttnParams p;
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
    p.page_tokens = page_tokens;
    p.page_shift = shift;
    p.scale_log2 = scale * LOG2E;
    p.window = window;
    p.status = status;
    const int n_rep = n_heads / n_kv_heads;
    const int q_tiles = (max_new_tokens * n_rep + ROWS - 1) / ROWS;
    if (n_requests > 65535 || q_tiles > 65535) return CB_ERR_UNSUPPORTED;
    const dim3 grid(n_kv_heads, n_requests, q_tiles);
    // lean: -1 lets the launch decide, 0 and 1 fix the form.  Since the roomy form has two
    // softmax groups it is the quicker one also for launches with more blocks than places
    // (measured on B200: 2,048 tokens at the Llama-3.2-1B layer sizes, 512 blocks, 4.63 against
    // 4.86 ms; 4,096 tokens of the 120M shape, 384 blocks, 1.68 against 1.96 ms), so the launch
    // decides for it; the lean form stays for callers that ask for it.
    if (lean < 0) lean = 0;
    if (head_dim == 64)
        return lean ? launch_as<64, true>(grid, (cudaStream_t)stream, mk, mv, rk, rv, p)
                    : launch_as<64, false>(grid, (cudaStream_t)stream, mk, mv, rk, rv, p);
    return launch_as<128, false>(grid, (cudaStream_t)stream, mk, mv, rk, rv, p);
}
