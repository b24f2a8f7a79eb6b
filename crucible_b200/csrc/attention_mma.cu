// Paged causal attention in bfloat16 on tensor cores (mma.sync m16n8k16, fp32
// accumulation, fp32 softmax), for prompts, portions of prompts and decoded
// tokens alike.  Query rows of one request and one KV head are enumerated as
// (position, head within the group): all query heads that share a KV head sit
// in the same tile, so each key and value is read once per group.
//
// Two launch shapes over the same inner loop:
//   tiles kernel  - a block takes 64 rows (4 warps x 16) and walks all their
//                   keys in tiles of 64 (cp.async, double buffered); flash-style
//                   running maximum; writes the normalised output.  For portions
//                   of prompts.
//   split kernel  - a block takes 16 rows and ONE chunk of 256 * 2^k keys, a
//                   quarter per warp; writes an unnormalised partial (max, sum,
//                   vector) to scratch; the last block of a row group to arrive
//                   (an atomic counter: no block waits for another) merges the
//                   chunks in ascending order.  For decoded tokens, where rows
//                   are few and keys many.
// Chunk boundaries are multiples of the chunk from key 0 whatever the batch
// holds, and the chunk is chosen from the launch's shape, so a row's result is
// a function of its own query and keys only.
//
// Head sizes: multiples of 16 up to 256.  Any head counts and group sizes, any
// page size.  Reference counterparts: `attention_prefill_exact_*`
// (engine/kernels/kernels.cu:2257-2275), `attention_decode_paged_f32` (:1741),
// and the split idea of `attention_partial_f32` / `attention_combine_f32`
// (:692-850).
#define CB_PDL_BIT 7      // this file's bit in CRUCIBLE_PDL
#include "common.cuh"

namespace {

constexpr int TILE_KEYS = 64;
constexpr int SPLIT_KEYS = 256;
constexpr float LOG2E = 1.4426950408889634f;

struct AttnParams {
    const __nv_bfloat16* qkv;
    int qkv_stride;
    __nv_bfloat16* out;
    int out_stride;
    const __nv_bfloat16* k_cache;
    const __nv_bfloat16* v_cache;
    const int* req_row_start;
    const int* req_first_pos;
    const int* block_table;
    int table_stride;
    int n_heads, n_kv_heads, head_dim, page_tokens;
    float scale_log2;      // softmax scale * log2(e)
    int window;            // 0: all earlier keys
    float* partial;        // split kernel: [rows_total * n_heads][n_chunks][head_dim + 2]
    int n_chunks;
    int chunk_keys;        // split kernel: keys per chunk, a multiple of SPLIT_KEYS
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;          // 0: the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem)), "l"(gmem),
                 "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }

template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem)));
}

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(smem_u32(smem)));
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Loads tiles of TILE keys and values of one request and KV head into shared
// memory rows of `pitch` elements, 16 bytes per cp.async, NT threads (a block or
// a warp) taking part.  Which (row, 16-byte piece) a thread copies is fixed for the
// kernel's life and worked out once; per tile only the page lookup remains (a
// shift and a mask when the page size is a power of two).  Keys at or beyond
// `key_end` are zero-filled.
template <int HD_MAX, int NT, int TILE>
struct KvLoader {
    static constexpr int ITEMS = (TILE * (HD_MAX / 8) + NT - 1) / NT;
    int row[ITEMS];          // key row inside the tile, or -1
    int base[ITEMS];         // element offset inside a page: kv_head's block + the piece's column
    int sdst[ITEMS];         // byte offset of the piece inside a shared-memory tile
    size_t page_elems;       // elements of one page (all KV heads)
    int page_shift;          // log2(page_tokens), or -1 if not a power of two

    __device__ __forceinline__ void init(const AttnParams& p, int kv_head, int pitch, int tid) {
        const int chunks_per_row = p.head_dim >> 3;
        const int total = TILE * chunks_per_row;
#pragma unroll
        for (int u = 0; u < ITEMS; ++u) {
            const int i = tid + u * NT;
            const int r = i / chunks_per_row;
            const int col = (i - r * chunks_per_row) * 8;
            row[u] = i < total ? r : -1;
            base[u] = kv_head * p.page_tokens * p.head_dim + col;
            sdst[u] = (r * pitch + col) * 2;
        }
        page_elems = (size_t)p.n_kv_heads * p.page_tokens * p.head_dim;
        page_shift = (p.page_tokens & (p.page_tokens - 1)) == 0 ? 31 - __clz(p.page_tokens) : -1;
    }

    __device__ __forceinline__ void load(const AttnParams& p, const int* table, int key0,
                                         int key_end, __nv_bfloat16* k_smem,
                                         __nv_bfloat16* v_smem) const {
        const uint32_t ks = smem_u32(k_smem), vs = smem_u32(v_smem);
        // in batches of four pieces: first the block-table lookups (loads that may
        // miss), then the copies, so that the lookups' latencies overlap
#pragma unroll
        for (int u0 = 0; u0 < ITEMS; u0 += 4) {
            size_t off[4];
            bool valid[4];
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const int u = u0 + v;
                off[v] = 0;
                valid[v] = false;
                if (u < ITEMS && row[u] >= 0) {
                    const int key = key0 + row[u];
                    valid[v] = key < key_end;
                    if (valid[v]) {
                        int page_index, slot;
                        if (page_shift >= 0) {
                            page_index = key >> page_shift;
                            slot = key & (p.page_tokens - 1);
                        } else {
                            page_index = key / p.page_tokens;
                            slot = key - page_index * p.page_tokens;
                        }
                        // A page that the window has passed was given back and its table
                        // entry is negative: every key in it is masked for every row, so it
                        // is zero-filled like a key past the end instead of being read.
                        const int page = table[page_index];
                        valid[v] = page >= 0;
                        if (valid[v])
                            off[v] = (size_t)page * page_elems +
                                     (size_t)(base[u] + slot * p.head_dim);
                    }
                }
            }
#pragma unroll
            for (int v = 0; v < 4; ++v) {
                const int u = u0 + v;
                if (u < ITEMS && row[u] >= 0) {
                    const int bytes = valid[v] ? 16 : 0;     // 0: zero-filled
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(ks + sdst[u]),
                                 "l"(p.k_cache + off[v]), "r"(bytes) : "memory");
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(vs + sdst[u]),
                                 "l"(p.v_cache + off[v]), "r"(bytes) : "memory");
                }
            }
        }
    }
};

// The query fragments of one warp's 16 rows, for all of head_dim: kept in
// registers for head sizes up to 128, re-read from shared memory beyond that.
template <int HD_MAX>
struct QFrags {
    static constexpr bool IN_REGS = HD_MAX <= 128;
    uint32_t a[IN_REGS ? HD_MAX / 16 : 1][4];
    const __nv_bfloat16* smem;
    int pitch;

    __device__ __forceinline__ void init(const __nv_bfloat16* q_smem, int pitch_, int head_dim) {
        smem = q_smem;
        pitch = pitch_;
        if (IN_REGS) {
#pragma unroll
            for (int kk = 0; kk < HD_MAX / 16; ++kk)
                if (kk * 16 < head_dim) fetch(kk, a[kk]);
        }
    }
    __device__ __forceinline__ void fetch(int kk, uint32_t (&out)[4]) const {
        const int lane = threadIdx.x & 31;
        const int mat = lane >> 3;
        const int row = (mat & 1) * 8 + (lane & 7);
        const int col = kk * 16 + (mat >> 1) * 8;
        ldmatrix_x4(out, smem + row * pitch + col);
    }
    __device__ __forceinline__ void get(int kk, uint32_t (&out)[4]) const {
        if (IN_REGS) {
            out[0] = a[kk][0]; out[1] = a[kk][1]; out[2] = a[kk][2]; out[3] = a[kk][3];
        } else {
            fetch(kk, out);
        }
    }
};

// One warp, 16 query rows, NK keys of a tile in shared memory (NK a multiple of
// 16): scores, running-maximum softmax update and the weighted sum of values.
// Rows g = lane / 4 and g + 8.  `masked`: some key of the tile may lie outside a
// row's range (after its position, before its window, or past the end); when
// the caller knows that none does, the per-element tests are skipped.
template <int HD_MAX, int NK, bool EXACT>
__device__ __forceinline__ void attend_tile(const AttnParams& p, const QFrags<HD_MAX>& q,
                                            const __nv_bfloat16* k_smem,
                                            const __nv_bfloat16* v_smem, int pitch_, bool masked,
                                            int key0,
                                            int pos_a, int pos_b, int lo_a, int lo_b, int key_end,
                                            float (&o)[HD_MAX / 8][4], float& m_a, float& m_b,
                                            float& l_a, float& l_b) {
    const int lane = threadIdx.x & 31;
    const int t = lane & 3;
    // EXACT: the head size is HD_MAX itself, so the loop bounds and the row pitch are
    // constants and the address arithmetic folds away
    const int hd = EXACT ? HD_MAX : p.head_dim;
    const int pitch = EXACT ? HD_MAX + 8 : pitch_;
    const int mat = lane >> 3;
    float s[NK / 8][4];
#pragma unroll
    for (int j = 0; j < NK / 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    // S = Q K^T
    const __nv_bfloat16* k_lane = k_smem + ((mat >> 1) * 8 + (lane & 7)) * pitch + (mat & 1) * 8;
#pragma unroll
    for (int kk = 0; kk < HD_MAX / 16; ++kk) {
        if (kk * 16 < hd) {
            uint32_t a[4];
            q.get(kk, a);
#pragma unroll
            for (int j = 0; j < NK / 8; j += 2) {
                uint32_t b[4];
                ldmatrix_x4(b, k_lane + j * 8 * pitch + kk * 16);
                mma_bf16(s[j], a, b[0], b[1]);
                mma_bf16(s[j + 1], a, b[2], b[3]);
            }
        }
    }
    // mask and row maxima (raw scores; the scale is positive and applied below)
    float mx_a = -INFINITY, mx_b = -INFINITY;
    if (masked) {                    // warp-uniform
        const int hi_a = min(pos_a, key_end - 1), hi_b = min(pos_b, key_end - 1);
#pragma unroll
        for (int j = 0; j < NK / 8; ++j) {
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int key = key0 + j * 8 + 2 * t + e;
                if (key > hi_a || key < lo_a) s[j][e] = -INFINITY;
                if (key > hi_b || key < lo_b) s[j][2 + e] = -INFINITY;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < NK / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            mx_a = fmaxf(mx_a, s[j][e]);
            mx_b = fmaxf(mx_b, s[j][2 + e]);
        }
    }
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1));
    mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1));
    mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
    const float new_a = fmaxf(m_a, mx_a * p.scale_log2), new_b = fmaxf(m_b, mx_b * p.scale_log2);
    // a row that has seen no key yet keeps max = -inf; use 0 as its offset so
    // that exp2(-inf - 0) = 0 instead of exp2(-inf + inf)
    const float off_a = new_a == -INFINITY ? 0.f : new_a;
    const float off_b = new_b == -INFINITY ? 0.f : new_b;
    const bool moved = new_a != m_a || new_b != m_b;
    if (__any_sync(0xffffffffu, moved)) {            // the running maxima rarely move late in a row
        const float corr_a = exp2f(m_a - off_a), corr_b = exp2f(m_b - off_b);
        l_a *= corr_a;
        l_b *= corr_b;
#pragma unroll
        for (int n = 0; n < HD_MAX / 8; ++n) {
            o[n][0] *= corr_a; o[n][1] *= corr_a;
            o[n][2] *= corr_b; o[n][3] *= corr_b;
        }
        m_a = new_a;
        m_b = new_b;
    }
    float sum_a = 0.f, sum_b = 0.f;
#pragma unroll
    for (int j = 0; j < NK / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            s[j][e] = exp2f(fmaf(s[j][e], p.scale_log2, -off_a));
            s[j][2 + e] = exp2f(fmaf(s[j][2 + e], p.scale_log2, -off_b));
            sum_a += s[j][e];
            sum_b += s[j][2 + e];
        }
    }
    l_a += sum_a;                    // per-thread partial sums; reduced over the quad at the end
    l_b += sum_b;
    // O += P V
    const __nv_bfloat16* v_lane = v_smem + ((mat & 1) * 8 + (lane & 7)) * pitch + (mat >> 1) * 8;
#pragma unroll
    for (int kk = 0; kk < NK / 16; ++kk) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
        a[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
        a[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        a[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int n = 0; n < HD_MAX / 8; n += 2) {
            if (n * 8 < hd) {
                uint32_t b[4];
                ldmatrix_x4_trans(b, v_lane + kk * 16 * pitch + n * 8);
                mma_bf16(o[n], a, b[0], b[1]);
                mma_bf16(o[n + 1], a, b[2], b[3]);
            }
        }
    }
}

// Copies the 16 x head_dim query rows of a warp's tile into shared memory
// (zeros for rows past the end); row i of the request's enumeration is
// (position i / n_rep, head kv_head * n_rep + i % n_rep).
__device__ __forceinline__ void load_q_rows(const AttnParams& p, int row_base, int n_rows,
                                            int first_row, int n_rep, int kv_head,
                                            __nv_bfloat16* q_smem, int pitch, int tid, int n_threads,
                                            int tile_rows) {
    const int chunks_per_row = p.head_dim >> 3;
    for (int i = tid; i < tile_rows * chunks_per_row; i += n_threads) {
        const int r = i / chunks_per_row, c = i - r * chunks_per_row;
        const int row = first_row + r;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < n_rows) {
            const int tok = row_base + row / n_rep;
            const int head = kv_head * n_rep + row % n_rep;
            v = *reinterpret_cast<const uint4*>(p.qkv + (size_t)tok * p.qkv_stride +
                                                (size_t)head * p.head_dim + c * 8);
        }
        *reinterpret_cast<uint4*>(q_smem + r * pitch + c * 8) = v;
    }
}

// ---------------------------------------------------------------------------
// tiles kernel
// ---------------------------------------------------------------------------
template <int HD_MAX, bool EXACT>
__global__ void __launch_bounds__(128) attention_tiles_kernel(const AttnParams p) {
    cb_pdl_trigger();
    cb_pdl_wait();
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int pitch = EXACT ? HD_MAX + 8 : p.head_dim + 8;
    __nv_bfloat16* q_smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* kv_smem = q_smem + 64 * pitch;      // [2 stages][K, V][64][pitch]
    const int req = blockIdx.z, kv_head = blockIdx.y;
    const int n_rep = p.n_heads / p.n_kv_heads;
    const int row_base = p.req_row_start[req];
    const int n_new = p.req_row_start[req + 1] - row_base;
    const int n_rows = n_new * n_rep;
    const int q_tiles = (n_rows + 63) >> 6;
    if ((int)blockIdx.x >= q_tiles) return;
    const int qt = q_tiles - 1 - (int)blockIdx.x;      // heaviest tiles first
    const int first_pos = p.req_first_pos[req];
    const int* table = p.block_table + (size_t)req * p.table_stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    load_q_rows(p, row_base, n_rows, qt * 64, n_rep, kv_head, q_smem, pitch, threadIdx.x, 128, 64);

    const int last_row = min(n_rows - 1, qt * 64 + 63);
    const int max_pos = first_pos + last_row / n_rep;
    const int min_pos = first_pos + (qt * 64) / n_rep;
    int key_lo = p.window > 0 ? max(0, min_pos - p.window + 1) : 0;
    key_lo = key_lo / TILE_KEYS * TILE_KEYS;
    const int key_end = max_pos + 1;
    const int n_tiles = (key_end - key_lo + TILE_KEYS - 1) / TILE_KEYS;

    // this warp's two rows
    const int row_a = qt * 64 + warp * 16 + g, row_b = row_a + 8;
    const int pos_a = row_a < n_rows ? first_pos + row_a / n_rep : -1;
    const int pos_b = row_b < n_rows ? first_pos + row_b / n_rep : -1;
    const int lo_a = p.window > 0 ? max(0, pos_a - p.window + 1) : 0;
    const int lo_b = p.window > 0 ? max(0, pos_b - p.window + 1) : 0;
    const int warp_last_row = min(n_rows - 1, qt * 64 + warp * 16 + 15);
    const int warp_max_pos = qt * 64 + warp * 16 < n_rows ? first_pos + warp_last_row / n_rep : -1;
    // interior tiles: all 16 rows of the warp exist, and the tile lies before the
    // lowest position and inside the latest window of the warp's rows
    const bool warp_full = qt * 64 + warp * 16 + 15 < n_rows;
    const int warp_min_pos = warp_full ? first_pos + (qt * 64 + warp * 16) / n_rep : -1;
    const int warp_max_lo = p.window > 0 ? max(0, warp_max_pos - p.window + 1) : 0;
    QFrags<HD_MAX> qf;

    float o[HD_MAX / 8][4];
#pragma unroll
    for (int n = 0; n < HD_MAX / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;

    const int stage_elems = 2 * TILE_KEYS * pitch;
    KvLoader<HD_MAX, 128, TILE_KEYS> loader;
    loader.init(p, kv_head, pitch, threadIdx.x);
    loader.load(p, table, key_lo, key_end, kv_smem, kv_smem + TILE_KEYS * pitch);
    cp_async_commit();
    for (int i = 0; i < n_tiles; ++i) {
        const int st = i & 1;
        if (i + 1 < n_tiles) {
            __nv_bfloat16* nxt = kv_smem + (st ^ 1) * stage_elems;
            loader.load(p, table, key_lo + (i + 1) * TILE_KEYS, key_end, nxt, nxt + TILE_KEYS * pitch);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (i == 0) qf.init(q_smem + warp * 16 * pitch, pitch, p.head_dim);   // the rows are in place now
        const int key0 = key_lo + i * TILE_KEYS;
        if (key0 <= warp_max_pos) {
            const __nv_bfloat16* ks = kv_smem + st * stage_elems;
            // no test per element if every key of the tile is inside every row's range
            const bool interior = key0 + TILE_KEYS - 1 <= warp_min_pos && key0 >= warp_max_lo;
            attend_tile<HD_MAX, TILE_KEYS, EXACT>(p, qf, ks, ks + TILE_KEYS * pitch, pitch, !interior,
                                                  key0, pos_a, pos_b, lo_a, lo_b, key_end, o, m_a,
                                                  m_b, l_a, l_b);
        }
        __syncthreads();
    }
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);
    const float inv_a = l_a > 0.f ? 1.0f / l_a : 0.f, inv_b = l_b > 0.f ? 1.0f / l_b : 0.f;
#pragma unroll
    for (int n = 0; n < HD_MAX / 8; ++n) {
        if (n * 8 < p.head_dim) {
            const int col = n * 8 + 2 * t;
            if (row_a < n_rows) {
                const int tok = row_base + row_a / n_rep, head = kv_head * n_rep + row_a % n_rep;
                *reinterpret_cast<uint32_t*>(p.out + (size_t)tok * p.out_stride +
                                             (size_t)head * p.head_dim + col) =
                    pack_bf16(o[n][0] * inv_a, o[n][1] * inv_a);
            }
            if (row_b < n_rows) {
                const int tok = row_base + row_b / n_rep, head = kv_head * n_rep + row_b % n_rep;
                *reinterpret_cast<uint32_t*>(p.out + (size_t)tok * p.out_stride +
                                             (size_t)head * p.head_dim + col) =
                    pack_bf16(o[n][2] * inv_b, o[n][3] * inv_b);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// split kernel: 16 rows x one chunk of keys (a multiple of 256).  The chunk is
// cut into sub-tiles that are dealt to the four warps in turn; each warp streams
// its sub-tiles through a ring of its own in shared memory (cp.async, several
// in flight, no block-wide barrier in the loop) and attends to them with a
// running maximum.  The warps' results are merged in warp order; if the rows
// have a single chunk the output is written at once, else the chunk's partial
// (max, sum, vector) goes to scratch and the block that arrives last at the rows'
// counter merges the chunks in ascending order.  No block waits for another.
// ---------------------------------------------------------------------------
template <int HD_MAX>
struct SplitShape {
    // keys per sub-tile and ring depth per warp, sized so that two blocks fit an SM
    // for head sizes up to 64 and one beyond
    static constexpr int SUB = HD_MAX <= 128 ? 32 : 16;
    static constexpr int RING = 2;
};


// Merges one row's chunks (ascending, with a running maximum) and writes its
// output.  One warp; lanes own features.  The loads of up to 8 chunks are issued
// together, so the whole merge costs about one memory round trip per 8 chunks.
__device__ __forceinline__ void merge_row(const AttnParams& p, int tok, int head, int pos, int lane) {
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int mp = p.head_dim + 2;
    const int c_first = lo / p.chunk_keys, c_last = pos / p.chunk_keys;
    const float* base = p.partial + ((size_t)tok * p.n_heads + head) * p.n_chunks * mp;
    float m = -INFINITY, l = 0.f;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    for (int c0 = c_first; c0 <= c_last; c0 += 8) {
        float mc[8], lc[8], oc[8][8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const bool in = c0 + j <= c_last;
            const float* src = base + (size_t)(in ? c0 + j : c_first) * mp;
            mc[j] = in ? __ldcg(src + p.head_dim) : -INFINITY;
            lc[j] = in ? __ldcg(src + p.head_dim + 1) : 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int f = lane + 32 * i;
                oc[j][i] = (in && f < p.head_dim) ? __ldcg(src + f) : 0.f;
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {                    // ascending chunks
            const float m_new = fmaxf(m, mc[j]);
            const float off = m_new == -INFINITY ? 0.f : m_new;
            const float keep = exp2f(m - off), take = exp2f(mc[j] - off);
            l = l * keep + lc[j] * take;
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = acc[i] * keep + oc[j][i] * take;
            m = m_new;
        }
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    __nv_bfloat16* dst = p.out + (size_t)tok * p.out_stride + (size_t)head * p.head_dim;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int f = lane + 32 * i;
        if (f < p.head_dim) dst[f] = __float2bfloat16_rn(acc[i] * inv);
    }
}

template <int HD_MAX, bool EXACT>
__global__ void __launch_bounds__(128) attention_split_kernel(const AttnParams p, int* counters,
                                                              int max_q_tiles) {
    cb_pdl_trigger();
    cb_pdl_wait();
    constexpr int SUB = SplitShape<HD_MAX>::SUB;
    constexpr int RING = SplitShape<HD_MAX>::RING;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    __shared__ int is_last;
    const int pitch = EXACT ? HD_MAX + 8 : p.head_dim + 8;
    __nv_bfloat16* q_smem = reinterpret_cast<__nv_bfloat16*>(smem_raw);
    __nv_bfloat16* kv_smem = q_smem + 16 * pitch;      // [warp][RING][K, V][SUB][pitch]
    const int req = blockIdx.z, kv_head = blockIdx.y;
    const int n_rep = p.n_heads / p.n_kv_heads;
    const int row_base = p.req_row_start[req];
    const int n_new = p.req_row_start[req + 1] - row_base;
    const int n_rows = n_new * n_rep;
    const int q_tiles = (n_rows + 15) >> 4;
    const int chunk = blockIdx.x % p.n_chunks;
    const int qt = blockIdx.x / p.n_chunks;
    if (qt >= q_tiles) return;
    const int first_pos = p.req_first_pos[req];
    const int* table = p.block_table + (size_t)req * p.table_stride;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;

    const int last_row = min(n_rows - 1, qt * 16 + 15);
    const int max_pos = first_pos + last_row / n_rep;
    const int min_pos = first_pos + (qt * 16) / n_rep;
    const int key_lo = p.window > 0 ? max(0, min_pos - p.window + 1) : 0;
    const int key_end = max_pos + 1;
    const int c0 = chunk * p.chunk_keys;
    // chunks wholly outside the tile's keys take no part
    if (c0 >= key_end || c0 + p.chunk_keys <= key_lo) return;
    const int n_active = (key_end - 1) / p.chunk_keys - key_lo / p.chunk_keys + 1;
    const int chunk_end = min(key_end, c0 + p.chunk_keys);
    const int n_sub = (chunk_end - c0 + SUB - 1) / SUB;          // sub-tiles of the chunk
    const int mine = warp < n_sub ? (n_sub - warp + 3) / 4 : 0;  // ... of which this warp takes
    const int stage_elems = 2 * SUB * pitch;
    __nv_bfloat16* ring = kv_smem + (size_t)warp * RING * stage_elems;

    // the query rows (all threads), then this warp's first sub-tiles, all in flight at once
    {
        const int chunks_per_row = p.head_dim >> 3;
        for (int i = threadIdx.x; i < 16 * chunks_per_row; i += 128) {
            const int r = i / chunks_per_row, c = i - r * chunks_per_row;
            const int row = qt * 16 + r;
            const bool valid = row < n_rows;
            const int tok = row_base + (valid ? row / n_rep : 0);
            const int head = kv_head * n_rep + (valid ? row % n_rep : 0);
            cp_async_16(q_smem + r * pitch + c * 8,
                        p.qkv + (size_t)tok * p.qkv_stride + (size_t)head * p.head_dim + c * 8, valid);
        }
        cp_async_commit();
    }
    KvLoader<HD_MAX, 32, SUB> loader;
    loader.init(p, kv_head, pitch, lane);
#pragma unroll
    for (int st = 0; st < RING; ++st) {
        if (st < mine) {
            __nv_bfloat16* ks = ring + st * stage_elems;
            loader.load(p, table, c0 + (warp + 4 * st) * SUB, key_end, ks, ks + SUB * pitch);
        }
        cp_async_commit();
    }

    const int row_a = qt * 16 + g, row_b = row_a + 8;
    const int pos_a = row_a < n_rows ? first_pos + row_a / n_rep : -1;
    const int pos_b = row_b < n_rows ? first_pos + row_b / n_rep : -1;
    const int lo_a = p.window > 0 ? max(0, pos_a - p.window + 1) : 0;
    const int lo_b = p.window > 0 ? max(0, pos_b - p.window + 1) : 0;
    float o[HD_MAX / 8][4];
#pragma unroll
    for (int n = 0; n < HD_MAX / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    // interior sub-tiles need no per-element test: all 16 rows exist, the keys lie at
    // or before the lowest position and inside the latest window
    const bool all_rows = qt * 16 + 15 < n_rows;
    const int max_lo = p.window > 0 ? max(0, max_pos - p.window + 1) : 0;
    cp_async_wait<RING>();              // this thread's piece of the query rows has landed
    __syncthreads();                    // ... and everybody else's
    QFrags<HD_MAX> qf;
    qf.init(q_smem, pitch, p.head_dim);
    for (int i = 0; i < mine; ++i) {
        cp_async_wait<RING - 1>();
        __syncwarp();
        const int st = i % RING;
        const __nv_bfloat16* ks = ring + st * stage_elems;
        const int key0 = c0 + (warp + 4 * i) * SUB;
        const bool interior = all_rows && key0 + SUB - 1 <= min_pos && key0 >= max_lo;
        attend_tile<HD_MAX, SUB, EXACT>(p, qf, ks, ks + SUB * pitch, pitch, !interior, key0, pos_a,
                                        pos_b, lo_a, lo_b, key_end, o, m_a, m_b, l_a, l_b);
        __syncwarp();
        if (i + RING < mine) {
            __nv_bfloat16* nxt = ring + st * stage_elems;
            loader.load(p, table, c0 + (warp + 4 * (i + RING)) * SUB, key_end, nxt, nxt + SUB * pitch);
        }
        cp_async_commit();
    }
    cp_async_wait<0>();
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 1);
    l_a += __shfl_xor_sync(0xffffffffu, l_a, 2);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 1);
    l_b += __shfl_xor_sync(0xffffffffu, l_b, 2);

    // merge the four warps through shared memory, reusing the key/value rings: per
    // warp 16 rows x (head_dim + 2) floats.  Warp w holds sub-tiles w, w+4, ...; the
    // merge takes the warps in a fixed order, so the result does not vary
    __syncthreads();
    float* merge = reinterpret_cast<float*>(kv_smem);
    const int mp = p.head_dim + 2;
    {
        float* mine = merge + (size_t)warp * 16 * mp;
#pragma unroll
        for (int n = 0; n < HD_MAX / 8; ++n) {
            if (n * 8 < p.head_dim) {
                const int col = n * 8 + 2 * t;
                mine[g * mp + col] = o[n][0];
                mine[g * mp + col + 1] = o[n][1];
                mine[(g + 8) * mp + col] = o[n][2];
                mine[(g + 8) * mp + col + 1] = o[n][3];
            }
        }
        if (t == 0) {
            mine[g * mp + p.head_dim] = m_a;
            mine[g * mp + p.head_dim + 1] = l_a;
            mine[(g + 8) * mp + p.head_dim] = m_b;
            mine[(g + 8) * mp + p.head_dim + 1] = l_b;
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 16 * mp; i += 128) {
        const int r = i / mp, f = i - r * mp;
        const int row = qt * 16 + r;
        if (row >= n_rows) continue;
        float m = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) m = fmaxf(m, merge[((size_t)w * 16 + r) * mp + p.head_dim]);
        float v;
        if (f == p.head_dim) {
            v = m;
        } else {
            const int src = f == p.head_dim + 1 ? p.head_dim + 1 : f;
            v = 0.f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float mw = merge[((size_t)w * 16 + r) * mp + p.head_dim];
                const float scale = mw == -INFINITY ? 0.f : exp2f(mw - m);
                v += merge[((size_t)w * 16 + r) * mp + src] * scale;
            }
        }
        const int tok = row_base + row / n_rep, head = kv_head * n_rep + row % n_rep;
        if (n_active == 1) {
            // the only chunk of these rows: normalise and write the output at once
            if (f < p.head_dim) {
                float l = 0.f;
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const float mw = merge[((size_t)w * 16 + r) * mp + p.head_dim];
                    l += merge[((size_t)w * 16 + r) * mp + p.head_dim + 1] *
                         (mw == -INFINITY ? 0.f : exp2f(mw - m));
                }
                p.out[(size_t)tok * p.out_stride + (size_t)head * p.head_dim + f] =
                    __float2bfloat16_rn(l > 0.f ? v / l : 0.f);
            }
        } else {
            p.partial[(((size_t)tok * p.n_heads + head) * p.n_chunks + chunk) * mp + f] = v;
        }
    }
    if (n_active == 1) return;
    // the last block to arrive for these rows merges their chunks
    int* counter = counters + ((size_t)req * p.n_kv_heads + kv_head) * max_q_tiles + qt;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int prev = atomicAdd(counter, 1);
        is_last = prev == n_active - 1;
        if (is_last) *counter = 0;                      // ready for the next launch
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int r = warp; r < 16; r += 4) {
        const int row = qt * 16 + r;
        if (row >= n_rows) break;
        const int tok = row_base + row / n_rep, head = kv_head * n_rep + row % n_rep;
        merge_row(p, tok, head, first_pos + row / n_rep, lane);
    }
}

template <int HD_MAX, bool EXACT>
int launch_tiles_as(const AttnParams& p, int n_requests, int max_q_tiles, cudaStream_t s) {
    const int pitch = p.head_dim + 8;
    const int smem = (64 + 4 * TILE_KEYS) * pitch * 2;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attention_tiles_kernel<HD_MAX, EXACT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(max_q_tiles, p.n_kv_heads, n_requests);
    cb_launch(attention_tiles_kernel<HD_MAX, EXACT>, dim3(grid), dim3(128), smem, s, p);
    return cb_last_error();
}

template <int HD_MAX>
int launch_tiles(const AttnParams& p, int n_requests, int max_q_tiles, cudaStream_t s) {
    return p.head_dim == HD_MAX ? launch_tiles_as<HD_MAX, true>(p, n_requests, max_q_tiles, s)
                                : launch_tiles_as<HD_MAX, false>(p, n_requests, max_q_tiles, s);
}

template <int HD_MAX, bool EXACT>
int launch_split_as(const AttnParams& p, int n_requests, int max_q_tiles, int* counters,
                    cudaStream_t s) {
    const int pitch = p.head_dim + 8;
    int smem = (16 + 4 * SplitShape<HD_MAX>::RING * 2 * SplitShape<HD_MAX>::SUB) * pitch * 2;
    const int merge_bytes = 4 * 16 * (p.head_dim + 2) * 4;
    if (16 * pitch * 2 + merge_bytes > smem) smem = 16 * pitch * 2 + merge_bytes;
    static bool configured = false;
    if (!configured && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attention_split_kernel<HD_MAX, EXACT>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(max_q_tiles * p.n_chunks, p.n_kv_heads, n_requests);
    cb_launch(attention_split_kernel<HD_MAX, EXACT>, dim3(grid), dim3(128), smem, s, p, counters,
              max_q_tiles);
    return cb_last_error();
}

template <int HD_MAX>
int launch_split(const AttnParams& p, int n_requests, int max_q_tiles, int* counters, cudaStream_t s) {
    return p.head_dim == HD_MAX
               ? launch_split_as<HD_MAX, true>(p, n_requests, max_q_tiles, counters, s)
               : launch_split_as<HD_MAX, false>(p, n_requests, max_q_tiles, counters, s);
}

}  // namespace

// Floats of scratch the split form needs for `n_tokens` rows and `n_chunks` chunks.
CB_EXPORT long cb_attention_split_scratch_floats(int n_tokens, int n_heads, int head_dim,
                                                 int n_chunks) {
    return (long)n_tokens * n_heads * n_chunks * (head_dim + 2);
}

CB_EXPORT int cb_attention_split_keys() { return SPLIT_KEYS; }

// Counters (ints, zero before the first launch; the kernel leaves them zero) the
// split form needs.
CB_EXPORT long cb_attention_split_counters(int n_requests, int n_kv_heads, int max_new_tokens,
                                           int n_heads) {
    const int max_rows = max_new_tokens * (n_heads / n_kv_heads);
    return (long)n_requests * n_kv_heads * ((max_rows + 15) / 16);
}

// n_chunks == 0: tiles kernel.  n_chunks > 0: split kernel over that many
// chunks of chunk_keys keys (a multiple of 256; together they must cover the
// longest context); `partial` must hold
// cb_attention_split_scratch_floats floats and `counters`
// cb_attention_split_counters zeroed ints.
// max_q_rows: the largest (new tokens x heads per group) of any request.
CB_EXPORT int cb_attention_mma(const void* qkv, int qkv_stride, void* out, int out_stride,
                               const void* k_cache, const void* v_cache, const int* positions,
                               const int* req_row_start, const int* req_first_pos,
                               const int* block_table, int table_stride, int n_tokens,
                               int n_requests, int max_new_tokens, int n_heads, int n_kv_heads,
                               int head_dim, int page_tokens, float scale, int window,
                               float* partial, int* counters, int n_chunks, int chunk_keys,
                               void* stream) {
    if (n_tokens <= 0 || n_requests <= 0) return 0;
    if (head_dim <= 0 || head_dim > 256 || (head_dim & 15) || n_heads % n_kv_heads != 0 ||
        (qkv_stride & 7) || (out_stride & 1) || ((uintptr_t)qkv & 15) || ((uintptr_t)k_cache & 15) ||
        ((uintptr_t)v_cache & 15))
        return CB_ERR_UNSUPPORTED;
    AttnParams p;
    p.qkv = (const __nv_bfloat16*)qkv;
    p.qkv_stride = qkv_stride;
    p.out = (__nv_bfloat16*)out;
    p.out_stride = out_stride;
    p.k_cache = (const __nv_bfloat16*)k_cache;
    p.v_cache = (const __nv_bfloat16*)v_cache;
    p.req_row_start = req_row_start;
    p.req_first_pos = req_first_pos;
    p.block_table = block_table;
    p.table_stride = table_stride;
    p.n_heads = n_heads;
    p.n_kv_heads = n_kv_heads;
    p.head_dim = head_dim;
    p.page_tokens = page_tokens;
    p.scale_log2 = scale * LOG2E;
    p.window = window;
    p.partial = partial;
    p.n_chunks = n_chunks;
    p.chunk_keys = chunk_keys > 0 ? chunk_keys : SPLIT_KEYS;
    cudaStream_t s = (cudaStream_t)stream;
    const int n_rep = n_heads / n_kv_heads;
    const int max_rows = max_new_tokens * n_rep;
    int rc;
    if (n_chunks == 0) {
        const int q_tiles = (max_rows + 63) / 64;
        if (head_dim <= 16) rc = launch_tiles<16>(p, n_requests, q_tiles, s);
        else if (head_dim <= 32) rc = launch_tiles<32>(p, n_requests, q_tiles, s);
        else if (head_dim <= 64) rc = launch_tiles<64>(p, n_requests, q_tiles, s);
        else if (head_dim <= 128) rc = launch_tiles<128>(p, n_requests, q_tiles, s);
        else rc = launch_tiles<256>(p, n_requests, q_tiles, s);
        return rc;
    }
    if (partial == nullptr || counters == nullptr || (chunk_keys % SPLIT_KEYS) != 0)
        return CB_ERR_UNSUPPORTED;
    const int q_tiles = (max_rows + 15) / 16;
    if (head_dim <= 16) rc = launch_split<16>(p, n_requests, q_tiles, counters, s);
    else if (head_dim <= 32) rc = launch_split<32>(p, n_requests, q_tiles, counters, s);
    else if (head_dim <= 64) rc = launch_split<64>(p, n_requests, q_tiles, counters, s);
    else if (head_dim <= 128) rc = launch_split<128>(p, n_requests, q_tiles, counters, s);
    else rc = launch_split<256>(p, n_requests, q_tiles, counters, s);
    return rc;
}
