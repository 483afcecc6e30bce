// Softmax attention over the paged cache in bfloat16 on the tensor cores (mma.sync m16n8k16), with the options of
// masked_attention.cu, whose float32 kernel is its plain twin: key and value heads of different sizes, a tanh cap on the
// scores, a sliding window that may keep the sequence's first tokens visible, a sigmoid gate per output element, and a
// value pool that may be the key pool itself (the values are then the leading part of every key row, and the key tile in
// shared memory serves as the value tile too).
//
// One block of four warps per (tile of 64 rows, group of query heads, slice of value columns).  A row is a (token, head)
// pair: with ``pack`` heads of one key head taken together, a block holds 64 / pack tokens x pack heads, so that in a
// step of single tokens the key tile is read once for up to 16 heads (latent attention has ONE key head for all).  Each
// warp is a flash attention over 16 rows (S = Q K^T in float32, online softmax, P rounded to bfloat16, O += P V in
// float32) over tiles of 64 keys that start at multiples of 64; a row's sums therefore do not depend on the tile it
// falls in, on ``pack`` or on the batch.  Key heads may be wide (a latent row of several hundred elements), so the query
// fragments are read from shared memory at every step instead of living in registers; wide value heads are
// cut into slices (of 256 for prompts, of 128 in steps of single tokens), each a block of its own that computes the scores again.
//
// K and V tiles come from the pages by cp.async into two buffers, a tile ahead of the arithmetic; the page of every key
// row of a tile is looked up two tiles ahead.  Key tiles that no row of the block can see (between the kept first tokens
// and the window) are passed over.  A key tile has 64 keys, or 32 where wide key rows would otherwise leave room for one
// block an SM only.
//
// A block of at most 16 rows (a step of single tokens) is work for one warp, whose instructions one after another are what
// the block's time is made of.  Where the launch has no more blocks than the GPU has SMs, the kernel gets four buffers and
// the four warps take four tiles of keys side by side, each with a running maximum and sum of its own; their partial rows
// are merged through shared memory in the order of the warps.
#include "common.cuh"

#define MM_BM 64
#define MM_SUB 32                // keys of a tile whose scores a warp holds at a time
#define MM_THREADS 128
#define MM_PAD 8                 // bf16 elements of padding per shared-memory row (16 bytes: conflict-free ldmatrix)

struct MaskedMmaArgs {
    const __nv_bfloat16* q;      // [T, q_stride]; head h at column h * q_head
    const __nv_bfloat16* k_pool; // [pages, nkv, page, ldk]
    const __nv_bfloat16* v_pool; // [pages, nkv, page, ldv]; may be k_pool
    const __nv_bfloat16* gate;   // [T, gate_stride], element (h, j) at column h * dv + j; or null
    __nv_bfloat16* out;          // [T, nh * dv]
    const int* positions;
    const int* seq_slot;
    const int* q_start;
    const int* block_table;
    const int* tiles;            // (sequence, first token of the tile within the sequence's tokens of the step), 64 tokens a tile
    int* status;
    const float* sinks;          // [nh] or null: exp(sinks[h]) joins the softmax's denominator, with no key and no value
    int nh, nkv, d, dv, q_stride, q_head, ldk, ldv, gate_stride, page_size, max_pages, num_pages, window, keep_first;
    int pack;                    // heads of one key head a block takes (a power of two up to 16 that divides nh / nkv)
    int slice;                   // value columns a block takes (a multiple of 16)
    int share;                   // 1: four K/V buffers are there, and blocks of at most 16 rows spread their key tiles over the warps
    float scale, softcap;
    float out_scale;             // the stored result is multiplied by this (the mixer's weight in a sum of mixers)
};

__device__ __forceinline__ void mm_ldmatrix_x4(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mm_ldmatrix_x4_trans(unsigned& r0, unsigned& r1, unsigned& r2, unsigned& r3, const void* p) {
    unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(s));
}
__device__ __forceinline__ void mm_mma(float* c, const unsigned* a, unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// tanh in one MUFU instruction (absolute error about 5e-4): the capped score is rounded far more coarsely by its bfloat16 operands
__device__ __forceinline__ float mm_tanh_fast(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ unsigned mm_pack(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// DVT: 8-column tiles of a value slice the registers hold (slice <= 8 DVT); ALIAS: the values are the key rows' leading part
template <int DVT, bool ALIAS, int MM_BN>
__global__ void __launch_bounds__(MM_THREADS, (DVT <= 16 ? 3 : 2)) masked_attention_mma_kernel(MaskedMmaArgs a) {
    ce_pdl_begin();
    extern __shared__ __align__(16) unsigned char mm_smem[];
    const int d = a.d, ldq = d + MM_PAD, ldks = d + MM_PAD;
    const int pack = a.pack, tpb = MM_BM / pack;             // tokens a block takes
    const int tile = (gridDim.x - 1 - blockIdx.x) / pack, sub_tile = (gridDim.x - 1 - blockIdx.x) % pack;
    const int b = a.tiles[2 * tile], q0 = a.tiles[2 * tile + 1] + sub_tile * tpb;
    const int seq_tokens = a.q_start[b + 1] - a.q_start[b];
    const int n_tok = min(tpb, min(seq_tokens, a.tiles[2 * tile + 1] + MM_BM) - q0);
    if (n_tok <= 0) return;                                   // (the same for every thread of the block)
    const int n_rows = n_tok * pack;
    const int head0 = blockIdx.y * pack, kvh = head0 / (a.nh / a.nkv);
    const int col0 = blockIdx.z * a.slice, ncol = min(a.slice, a.dv - col0), ldvs = a.slice + MM_PAD;
    const int t0 = a.q_start[b] + q0;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    __nv_bfloat16* Qs = (__nv_bfloat16*)mm_smem;             // [64][ldq]
    __nv_bfloat16* stage0 = Qs + MM_BM * ldq;                // two buffers of K [64][ldks] (and V [64][ldvs])
    const int stage_elems = MM_BN * ldks + (ALIAS ? 0 : MM_BN * ldvs);
    __shared__ int s_pos[MM_BM];
    __shared__ int s_page[4][MM_BN];                         // page of every key row of the tile a buffer will hold

    const int* table = a.block_table + (size_t)a.seq_slot[b] * a.max_pages;
    if (tid < MM_BM) s_pos[tid] = tid < n_rows ? a.positions[t0 + tid / pack] : -1;
    const int c8 = d >> 3;
    for (int e = tid; e < MM_BM * c8; e += MM_THREADS) {
        int r = e / c8, c = (e % c8) * 8;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < n_rows) v = *reinterpret_cast<const uint4*>(a.q + (size_t)(t0 + r / pack) * a.q_stride + (size_t)(head0 + r % pack) * a.q_head + c);
        *reinterpret_cast<uint4*>(Qs + r * ldq + c) = v;
    }
    __syncthreads();
    const int pos_first = s_pos[0], pos_last = s_pos[n_rows - 1];
    const int keep = a.window > 0 ? a.keep_first : 0;
    const int lo_blk = a.window > 0 ? max(0, pos_first - a.window + 1) : 0;
    // few rows: the warps all take rows 0..15 and share the key tiles; else warp w takes rows 16 w ..
    const bool share_keys = a.share != 0 && n_rows <= 16 && pos_last - lo_blk / MM_BN * MM_BN >= MM_BN;
    // this thread's two rows
    const int row0 = share_keys ? 0 : warp * 16;
    const int ra = row0 + (lane >> 2), rb = ra + 8;
    const int pos_a = s_pos[ra], pos_b = s_pos[rb];
    const int lo_a = a.window > 0 ? max(0, pos_a - a.window + 1) : 0, lo_b = a.window > 0 ? max(0, pos_b - a.window + 1) : 0;

    float o[DVT][4];
#pragma unroll
    for (int i = 0; i < DVT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
    float m_a = -INFINITY, m_b = -INFINITY, l_a = 0.f, l_b = 0.f;
    // scores are kept in the base-2 domain: 2^(s - m) is one subtraction and one MUFU
    const float log2e = 1.4426950408889634f;
    const float scale2 = a.scale * log2e;
    const float cap2 = a.softcap * log2e, pre_cap = a.softcap > 0.f ? a.scale / a.softcap : 0.f;

    auto page_of = [&](int k0, int r) -> int {
        int key = k0 + r;
        if (key > pos_last || k0 < 0) return -1;
        int page = table[key / a.page_size];
        if (page < 0 || page >= a.num_pages) { atomicExch(a.status, 4); return -1; }
        return page;
    };
    auto stage = [&](int k0, int which) {
        __nv_bfloat16* Kd = stage0 + which * stage_elems;
        const int* pages = s_page[which];
        constexpr int TPR = MM_THREADS / MM_BN;           // threads a key row: each takes every TPR-th 16-byte piece
        const int r = tid / TPR, c_first = (tid % TPR) * 8;
        const int page = pages[r];
        {
            __nv_bfloat16* dst = Kd + r * ldks;
            if (page >= 0) {
                const __nv_bfloat16* src = a.k_pool + (((size_t)page * a.nkv + kvh) * a.page_size + (k0 + r) % a.page_size) * a.ldk;
                for (int c = c_first; c < d; c += TPR * 8) {
                    unsigned sa = (unsigned)__cvta_generic_to_shared(dst + c);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(src + c));
                }
            } else {
                for (int c = c_first; c < d; c += TPR * 8) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        if (!ALIAS) {
            __nv_bfloat16* dst = Kd + MM_BN * ldks + r * ldvs;
            if (page >= 0) {
                const __nv_bfloat16* src = a.v_pool + (((size_t)page * a.nkv + kvh) * a.page_size + (k0 + r) % a.page_size) * a.ldv + col0;
                for (int c = c_first; c < ncol; c += TPR * 8) {
                    unsigned sa = (unsigned)__cvta_generic_to_shared(dst + c);
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(src + c));
                }
            } else {
                for (int c = c_first; c < ncol; c += TPR * 8) *reinterpret_cast<uint4*>(dst + c) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    // a tile of keys that every row of this warp sees whole needs no mask
    const bool rows_full = row0 + 15 < n_rows;
    const int warp_pos_first = s_pos[row0];
    int warp_lo_last = 0;
    if (rows_full) warp_lo_last = a.window > 0 ? max(0, s_pos[row0 + 15] - a.window + 1) : 0;

    auto tile_math = [&](int k0, int cur) {
        const __nv_bfloat16* Ks = stage0 + cur * stage_elems;
        const __nv_bfloat16* Vs = ALIAS ? Ks + col0 : Ks + MM_BN * ldks;
        const int ldv_s = ALIAS ? ldks : ldvs;
        if (row0 >= n_rows) return;              // a warp none of whose rows is a token only helps with the copies
#pragma unroll 1
        for (int sub = 0; sub < MM_BN; sub += MM_SUB) {
            const int ks0 = k0 + sub;
            if (ks0 > pos_last) break;
            float s[MM_SUB / 8][4];
#pragma unroll
            for (int i = 0; i < MM_SUB / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll 2
            for (int ks = 0; ks < d; ks += 16) {
                unsigned qf[4];
                mm_ldmatrix_x4(qf[0], qf[1], qf[2], qf[3], Qs + (row0 + (lane & 15)) * ldq + ks + (lane >> 4) * 8);
#pragma unroll
                for (int nt = 0; nt < MM_SUB / 8; nt += 2) {
                    unsigned b0, b1, b2, b3;
                    mm_ldmatrix_x4(b0, b1, b2, b3, Ks + (sub + nt * 8 + (lane >> 4) * 8 + (lane & 7)) * ldks + ks + ((lane >> 3) & 1) * 8);
                    mm_mma(s[nt], qf, b0, b1);
                    mm_mma(s[nt + 1], qf, b2, b3);
                }
            }
            // scale (and cap), mask, running maximum
            float mx_a = -INFINITY, mx_b = -INFINITY;
            const bool whole = rows_full && ks0 + MM_SUB - 1 <= warp_pos_first && ks0 >= warp_lo_last;
#pragma unroll
            for (int nt = 0; nt < MM_SUB / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const bool upper = e < 2;
                    bool see = true;
                    if (!whole) {
                        int key = ks0 + nt * 8 + (lane & 3) * 2 + (e & 1);
                        see = upper ? (key <= pos_a && (key >= lo_a || key < keep)) : (key <= pos_b && (key >= lo_b || key < keep));
                    }
                    float v = a.softcap > 0.f ? cap2 * mm_tanh_fast(s[nt][e] * pre_cap) : s[nt][e] * scale2;
                    v = see ? v : -INFINITY;
                    s[nt][e] = v;
                    if (upper) mx_a = fmaxf(mx_a, v); else mx_b = fmaxf(mx_b, v);
                }
            }
            mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 1)); mx_a = fmaxf(mx_a, __shfl_xor_sync(0xffffffffu, mx_a, 2));
            mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 1)); mx_b = fmaxf(mx_b, __shfl_xor_sync(0xffffffffu, mx_b, 2));
            float n_a = fmaxf(m_a, mx_a), n_b = fmaxf(m_b, mx_b);
            float use_a = n_a == -INFINITY ? 0.f : n_a, use_b = n_b == -INFINITY ? 0.f : n_b;
            float f_a = m_a == -INFINITY ? 0.f : ce_exp2_fast(m_a - use_a);
            float f_b = m_b == -INFINITY ? 0.f : ce_exp2_fast(m_b - use_b);
            const bool moved = n_a != m_a || n_b != m_b;
            m_a = n_a; m_b = n_b;
            float sum_a = 0.f, sum_b = 0.f;
            unsigned pf[MM_SUB / 16][4];
#pragma unroll
            for (int nt = 0; nt < MM_SUB / 8; ++nt) {
                float p0 = ce_exp2_fast(s[nt][0] - use_a), p1 = ce_exp2_fast(s[nt][1] - use_a);
                float p2 = ce_exp2_fast(s[nt][2] - use_b), p3 = ce_exp2_fast(s[nt][3] - use_b);
                sum_a += p0 + p1;
                sum_b += p2 + p3;
                pf[nt >> 1][(nt & 1) * 2] = mm_pack(p0, p1);
                pf[nt >> 1][(nt & 1) * 2 + 1] = mm_pack(p2, p3);
            }
            sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 1); sum_a += __shfl_xor_sync(0xffffffffu, sum_a, 2);
            sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 1); sum_b += __shfl_xor_sync(0xffffffffu, sum_b, 2);
            l_a = l_a * f_a + sum_a;
            l_b = l_b * f_b + sum_b;
            if (__any_sync(0xffffffffu, moved)) {            // a maximum rose somewhere in the warp: what is summed so far shrinks
#pragma unroll
                for (int i = 0; i < DVT; ++i) { o[i][0] *= f_a; o[i][1] *= f_a; o[i][2] *= f_b; o[i][3] *= f_b; }
            }
            // O += P V
#pragma unroll
            for (int kk = 0; kk < MM_SUB / 16; ++kk) {
#pragma unroll
                for (int nt = 0; nt < DVT; nt += 2) {
                    if (nt * 8 < ncol) {
                        unsigned b0, b1, b2, b3;
                        mm_ldmatrix_x4_trans(b0, b1, b2, b3, Vs + (sub + kk * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * ldv_s + nt * 8 + (lane >> 4) * 8);
                        mm_mma(o[nt], pf[kk], b0, b1);
                        mm_mma(o[nt + 1], pf[kk], b2, b3);
                    }
                }
            }
        }
    };
    // the tiles of keys this block walks: those that hold kept first tokens below the window's first tile, then from the
    // window's first tile to the last row's position
    const int k_first = lo_blk / MM_BN * MM_BN;
    const int n_keep = min((keep + MM_BN - 1) / MM_BN, k_first / MM_BN);
    const int n_key_tiles = n_keep + (pos_last - k_first) / MM_BN + 1;
    auto k0_of = [&](int i) -> int { return i < n_key_tiles ? (i < n_keep ? i * MM_BN : k_first + (i - n_keep) * MM_BN) : -MM_BN; };
    if (share_keys) {
        // four tiles of keys at a time, one for each warp; the partial rows are merged afterwards
        for (int g0 = 0; g0 < n_key_tiles; g0 += 4) {
            if (tid < MM_BN)
                for (int w = 0; w < 4; ++w) s_page[w][tid] = page_of(k0_of(g0 + w), tid);
            __syncthreads();
            for (int w = 0; w < 4; ++w)
                if (g0 + w < n_key_tiles) stage(k0_of(g0 + w), w);
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();
            if (g0 + warp < n_key_tiles) tile_math(k0_of(g0 + warp), warp);
            __syncthreads();
        }
        // partial rows of warps 1..3: the sums so far [3][16][slice] and (maximum, sum) [3][16][2]; warp 0 adds them up in order
        float* part = (float*)stage0;
        float* ml = part + 3 * 16 * a.slice;
        const int r_lo = lane >> 2, r_hi = r_lo + 8, cq2 = (lane & 3) * 2;
        if (warp != 0) {
            float* mine = part + (warp - 1) * 16 * a.slice;
#pragma unroll
            for (int nt = 0; nt < DVT; ++nt) {
                if (nt * 8 < ncol) {
                    *reinterpret_cast<float2*>(mine + r_lo * a.slice + nt * 8 + cq2) = make_float2(o[nt][0], o[nt][1]);
                    *reinterpret_cast<float2*>(mine + r_hi * a.slice + nt * 8 + cq2) = make_float2(o[nt][2], o[nt][3]);
                }
            }
            if ((lane & 3) == 0) {
                float* m2 = ml + (warp - 1) * 16 * 2;
                m2[r_lo * 2] = m_a; m2[r_lo * 2 + 1] = l_a;
                m2[r_hi * 2] = m_b; m2[r_hi * 2 + 1] = l_b;
            }
        }
        __syncthreads();
        if (warp != 0) return;
        float big_a = m_a, big_b = m_b;
#pragma unroll
        for (int w = 0; w < 3; ++w) {
            big_a = fmaxf(big_a, ml[(w * 16 + r_lo) * 2]);
            big_b = fmaxf(big_b, ml[(w * 16 + r_hi) * 2]);
        }
        float f_a = m_a == -INFINITY ? 0.f : ce_exp2_fast(m_a - big_a), f_b = m_b == -INFINITY ? 0.f : ce_exp2_fast(m_b - big_b);
        l_a *= f_a; l_b *= f_b;
#pragma unroll
        for (int i = 0; i < DVT; ++i) { o[i][0] *= f_a; o[i][1] *= f_a; o[i][2] *= f_b; o[i][3] *= f_b; }
#pragma unroll
        for (int w = 0; w < 3; ++w) {
            const float* theirs = part + w * 16 * a.slice;
            float ma = ml[(w * 16 + r_lo) * 2], mb = ml[(w * 16 + r_hi) * 2];
            float g_a = ma == -INFINITY ? 0.f : ce_exp2_fast(ma - big_a), g_b = mb == -INFINITY ? 0.f : ce_exp2_fast(mb - big_b);
            l_a = fmaf(ml[(w * 16 + r_lo) * 2 + 1], g_a, l_a);
            l_b = fmaf(ml[(w * 16 + r_hi) * 2 + 1], g_b, l_b);
#pragma unroll
            for (int nt = 0; nt < DVT; ++nt) {
                if (nt * 8 < ncol) {
                    float2 xa = *reinterpret_cast<const float2*>(theirs + r_lo * a.slice + nt * 8 + cq2);
                    float2 xb = *reinterpret_cast<const float2*>(theirs + r_hi * a.slice + nt * 8 + cq2);
                    o[nt][0] = fmaf(xa.x, g_a, o[nt][0]); o[nt][1] = fmaf(xa.y, g_a, o[nt][1]);
                    o[nt][2] = fmaf(xb.x, g_b, o[nt][2]); o[nt][3] = fmaf(xb.y, g_b, o[nt][3]);
                }
            }
        }
        m_a = big_a; m_b = big_b;            // what the merged sums are relative to (the sink below joins them)
    } else {
    if (tid < MM_BN) {
        s_page[0][tid] = page_of(k0_of(0), tid);
        s_page[1][tid] = page_of(k0_of(1), tid);
    }
    __syncthreads();
    stage(k0_of(0), 0);
    for (int it = 0; it < n_key_tiles; ++it) {
        const int cur = it & 1;
        const bool more = it + 1 < n_key_tiles;
        int page_ahead = -1;                    // for the tile after the next: asked for now, stored after the arithmetic
        if (tid < MM_BN && it + 2 < n_key_tiles) page_ahead = page_of(k0_of(it + 2), tid);
        if (more) {
            stage(k0_of(it + 1), cur ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        tile_math(k0_of(it), cur);
        if (tid < MM_BN) s_page[cur][tid] = page_ahead;      // buffer ``cur`` will hold the tile after the next
        __syncthreads();
    }
    }
    const int cq = (lane & 3) * 2;
    const size_t tok_a = (size_t)(t0 + ra / pack), tok_b = (size_t)(t0 + rb / pack);
    const int head_a = head0 + ra % pack, head_b = head0 + rb % pack;
    float sh_a = 1.0f, sh_b = 1.0f;
    if (a.sinks) {                       // the sink, in the base-2 domain like the running maxima; it is neither scaled nor capped
        float sk_a = (ra < n_rows ? a.sinks[head_a] : 0.f) * log2e, sk_b = (rb < n_rows ? a.sinks[head_b] : 0.f) * log2e;
        float big_a = fmaxf(m_a, sk_a), big_b = fmaxf(m_b, sk_b);
        sh_a = m_a == -INFINITY ? 0.f : exp2f(m_a - big_a);
        sh_b = m_b == -INFINITY ? 0.f : exp2f(m_b - big_b);
        l_a = l_a * sh_a + exp2f(sk_a - big_a);
        l_b = l_b * sh_b + exp2f(sk_b - big_b);
    }
    float i_a = (l_a > 0.f ? sh_a / l_a : 0.f) * a.out_scale, i_b = (l_b > 0.f ? sh_b / l_b : 0.f) * a.out_scale;
#pragma unroll
    for (int nt = 0; nt < DVT; ++nt) {
        if (nt * 8 < ncol) {
            int col = col0 + nt * 8 + cq;
            if (ra < n_rows) {
                float x = o[nt][0] * i_a, y = o[nt][1] * i_a;
                if (a.gate) {
                    const __nv_bfloat16* g = a.gate + tok_a * a.gate_stride + (size_t)head_a * a.dv + col;
                    x *= 1.0f / (1.0f + expf(-__bfloat162float(g[0])));
                    y *= 1.0f / (1.0f + expf(-__bfloat162float(g[1])));
                }
                *reinterpret_cast<unsigned*>(a.out + (tok_a * a.nh + head_a) * a.dv + col) = mm_pack(x, y);
            }
            if (rb < n_rows) {
                float x = o[nt][2] * i_b, y = o[nt][3] * i_b;
                if (a.gate) {
                    const __nv_bfloat16* g = a.gate + tok_b * a.gate_stride + (size_t)head_b * a.dv + col;
                    x *= 1.0f / (1.0f + expf(-__bfloat162float(g[0])));
                    y *= 1.0f / (1.0f + expf(-__bfloat162float(g[1])));
                }
                *reinterpret_cast<unsigned*>(a.out + (tok_b * a.nh + head_b) * a.dv + col) = mm_pack(x, y);
            }
        }
    }
}

// Value columns a block takes: 128 at most in a step of single tokens (more blocks for the few rows), 256 at most for prompts
// (a slice computes the scores again, so fewer slices are less arithmetic: latent attention over rows of 288 with values of
// 256 took 480 us in two slices and 395 us in one, on 2,048 tokens; the single tokens of a decode step 61 against 80 us).
static int mm_slice(int dv, int buffers) {
    int cap = buffers == 4 ? 128 : 256;
    return dv <= cap ? dv : cap;
}

static size_t mm_smem_for(int d, int slice, bool alias, int buffers, int bn) {
    size_t stage = (size_t)bn * (d + MM_PAD) + (alias ? 0 : (size_t)bn * (slice + MM_PAD));
    size_t bytes = (size_t)buffers * stage * sizeof(__nv_bfloat16);
    size_t merge = (size_t)(3 * 16 * slice + 3 * 16 * 2) * sizeof(float);           // the partial rows of a shared walk
    if (buffers == 4 && bytes < merge) bytes = merge;
    return (size_t)MM_BM * (d + MM_PAD) * sizeof(__nv_bfloat16) + bytes;
}

// Keys a tile.  Two buffers (prompts): 64, or 32 where tiles of 64 would leave room for fewer than the three blocks an SM that
// the registers allow (the kernel hides its latencies by the number of blocks an SM holds; measured on 2,048 tokens with heads
// of 128: 323 -> 272 us).  Four buffers (a step of single tokens, one block an SM): 64 wherever four of them fit, since fewer,
// larger tiles are fewer rounds of the warps (62 against 72 us).
static int mm_key_tile(int d, int slice, bool alias, int buffers) {
    if (buffers == 4) return mm_smem_for(d, slice, alias, 4, 64) <= 200 * 1024 ? 64 : 32;
    return mm_smem_for(d, slice, alias, 2, 64) > 72 * 1024 ? 32 : 64;
}

static size_t mm_smem_bytes(int d, int slice, bool alias, int buffers) {
    return mm_smem_for(d, slice, alias, buffers, mm_key_tile(d, slice, alias, buffers));
}

// alias != 0: the value pool is the key pool (values = the key rows' leading dv elements)
extern "C" int ce_masked_attention_mma_supported(int d, int dv, int q_stride, int q_head, int ldk, int ldv, int alias) {
    if (d < 16 || d % 16 || dv < 16 || dv % 16 || q_stride % 8 || q_head % 8 || ldk % 8 || ldv % 8) return 0;
    if (alias && dv > d) return 0;
    return mm_smem_bytes(d, mm_slice(dv, 4), alias != 0, 2) <= 200 * 1024;
}

template <int DVT, bool ALIAS, int BN>
static void mm_launch(const MaskedMmaArgs& a, dim3 grid, size_t smem, cudaStream_t stream) {
    if (smem > 40 * 1024)            // the kernel's static arrays count toward the 48 KB a launch gets without asking
        cudaFuncSetAttribute(masked_attention_mma_kernel<DVT, ALIAS, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ce_note("masked_attention_mma_kernel");
    ce_launch(masked_attention_mma_kernel<DVT, ALIAS, BN>, grid, MM_THREADS, smem, stream, a);
}

template <int DVT, bool ALIAS>
static void mm_launch_bn(const MaskedMmaArgs& a, int bn, dim3 grid, size_t smem, cudaStream_t stream) {
    if (bn == 32) mm_launch<DVT, ALIAS, 32>(a, grid, smem, stream);
    else mm_launch<DVT, ALIAS, 64>(a, grid, smem, stream);
}

extern "C" int ce_masked_attention_mma(const void* q, const void* k_pool, const void* v_pool, const void* gate, void* out,
                                       const int* positions, const int* seq_slot, const int* q_start, const int* block_table,
                                       const int* tiles, int* status, int n_tiles, int n_tokens, int nh, int nkv, int d, int dv,
                                       int q_stride, int q_head, int ldk, int ldv, int gate_stride, int page_size, int max_pages,
                                       int num_pages, int window, int keep_first, float scale, float softcap, const float* sinks,
                                       float out_scale, cudaStream_t stream) {
    if (n_tiles == 0) return CE_OK;
    if (!q || !k_pool || !v_pool || !out || !positions || !seq_slot || !q_start || !block_table || !tiles || !status)
        return ce_fail(CE_ERR_ARG, "ce_masked_attention_mma: null pointer");
    bool alias = v_pool == k_pool;
    if (!ce_masked_attention_mma_supported(d, dv, q_stride, q_head, ldk, ldv, alias))
        return ce_fail(CE_ERR_SIZE, "ce_masked_attention_mma: head sizes %d / %d or strides not supported", d, dv);
    if (nkv <= 0 || nh % nkv != 0)
        return ce_fail(CE_ERR_SIZE, "ce_masked_attention_mma: %d heads are not a multiple of %d kv heads", nh, nkv);
    if ((((uintptr_t)q | (uintptr_t)k_pool | (uintptr_t)v_pool) & 15) || (((uintptr_t)out) & 3) || (gate && (((uintptr_t)gate) & 3)) ||
        (gate && gate_stride % 2))
        return ce_fail(CE_ERR_SIZE, "ce_masked_attention_mma: operands must be 16-byte aligned");
    // Heads of one key head taken together: with few tokens a tile (a step of single tokens) a block's rows are heads, and
    // the key tile is read once for all of them.  The choice depends on the step's shape only; no row's sums depend on it.
    int group = nh / nkv, pack = 1;
    if ((long long)n_tokens * 4 <= (long long)n_tiles * MM_BM)          // at most 16 tokens a tile on average
        while (pack < 16 && group % (pack * 2) == 0) pack *= 2;
    // Few blocks (a step of single tokens): four buffers, so that the warps can take four tiles of keys side by side.  Blocks
    // of a packed tile that hold no token leave at once, so what counts is the tiles, not the grid.
    int buffers = 2, slice = mm_slice(dv, 4);
    if ((long long)n_tiles * (nh / pack) * ((dv + slice - 1) / slice) <= (long long)ce_sm_count() &&
        mm_smem_bytes(d, slice, alias, 4) <= 200 * 1024) buffers = 4;
    if (buffers == 2) {
        slice = mm_slice(dv, 2);
        if (mm_smem_bytes(d, slice, alias, 2) > 200 * 1024) slice = mm_slice(dv, 4);
    }
    MaskedMmaArgs a{(const __nv_bfloat16*)q, (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, (const __nv_bfloat16*)gate,
                    (__nv_bfloat16*)out, positions, seq_slot, q_start, block_table, tiles, status, sinks, nh, nkv, d, dv, q_stride, q_head,
                    ldk, ldv, gate_stride, page_size, max_pages, num_pages, window, keep_first, pack, slice, buffers == 4, scale, softcap,
                    out_scale};
    dim3 grid(n_tiles * pack, nh / pack, (dv + slice - 1) / slice);
    size_t smem = mm_smem_bytes(d, slice, alias, buffers);
    int bn = mm_key_tile(d, slice, alias, buffers);
    if (alias) {
        if (slice <= 64) mm_launch_bn<8, true>(a, bn, grid, smem, stream);
        else if (slice <= 128) mm_launch_bn<16, true>(a, bn, grid, smem, stream);
        else mm_launch_bn<32, true>(a, bn, grid, smem, stream);
    } else {
        if (slice <= 64) mm_launch_bn<8, false>(a, bn, grid, smem, stream);
        else if (slice <= 128) mm_launch_bn<16, false>(a, bn, grid, smem, stream);
        else mm_launch_bn<32, false>(a, bn, grid, smem, stream);
    }
    return ce_check_launch("ce_masked_attention_mma");
}
