// Mixture of experts: routing, the layout of a step's (token, expert) pairs by expert, the experts' two products as
// grouped products over that layout, and the weighted sum back into token order.
//
//   route    z [T, ld] float32 router logits -> s = softmax(z[:E]); experts in `groups` equal groups of neighbours, a
//            group's score the largest s in it, only the best `keep` groups' experts eligible; the `top` eligible experts
//            with the largest s are chosen (ties: the lower index); weights s / (sum of the chosen s + 1e-20) * scale.
//            Column E of z, where there is one, is the logit of a shared expert's gate: sgate[t] = sigmoid(z[t, E]).
//   align    the T*top pairs sorted by expert into rows of a padded layout: every expert's rows start at a multiple of
//            the tile height BM, so a tile of BM rows belongs to ONE expert.  row_token[p] is the token of row p (-1: a
//            padding row), pair_row[i] the row of pair i, tile_expert[j] the expert of tile j, n_tiles[0] their count.
//            Nothing of it reaches the host: the products launch a grid for the most tiles a step of that size can have,
//            and blocks past n_tiles leave at once, so a captured graph replays with any routing.
//   products out[p] = act(in[row p's token, or p] W[e]^T), e = tile_expert[p / BM]; act = relu^2 or none.  Every output
//            element is a sum over k in a fixed order that depends on neither the row's place in its tile nor on the
//            other rows, so a token's result does not depend on the batch.  float32 FMA for any size and both dtypes;
//            bfloat16 on the tensor cores (wmma m16n16k16, float32 sums) for sizes in multiples of 16.
//   combine  y[t] (+)= sum_k weight[t, k] out[pair_row[t*top + k]] + sgate[t] shared[t], in the order of k, float32.
#include "common.cuh"
#include <mma.h>

#define MOE_MAX_EXPERTS 4096

// ---------------------------------------------------------------------------------------------
// routing: one warp a token
// ---------------------------------------------------------------------------------------------
struct MoeRouteArgs {
    const float* z;
    int* ids;           // [T, top]
    float* weights;     // [T, top]
    float* sgate;       // [T] or null
    int T, ld, E, top, groups, keep;
    float scale;
};

__device__ __forceinline__ void moe_warp_argmax(float& v, int& i) {
    for (int o = 16; o > 0; o >>= 1) {
        float ov = __shfl_xor_sync(0xffffffffu, v, o);
        int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

__global__ void __launch_bounds__(128) moe_route_kernel(MoeRouteArgs a) {
    ce_pdl_begin();
    extern __shared__ float moe_route_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + warp;
    if (t >= a.T) return;
    float* s = moe_route_smem + (size_t)warp * 2 * a.E;      // scores; a chosen or barred expert's score becomes -1
    float* gs = s + a.E;                                     // the groups' scores
    const float* zr = a.z + (size_t)t * a.ld;
    float mx = -INFINITY;
    for (int e = lane; e < a.E; e += 32) mx = fmaxf(mx, zr[e]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int e = lane; e < a.E; e += 32) { float v = expf(zr[e] - mx); s[e] = v; sum += v; }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.0f / sum;
    for (int e = lane; e < a.E; e += 32) s[e] *= inv;
    __syncwarp();
    if (a.groups > 1 && a.keep < a.groups) {
        const int size = a.E / a.groups;
        for (int g = lane; g < a.groups; g += 32) {
            float best = -1.f;
            for (int j = 0; j < size; ++j) best = fmaxf(best, s[g * size + j]);
            gs[g] = best;
        }
        __syncwarp();
        for (int k = 0; k < a.keep; ++k) {                   // the best groups' scores become 2 (a score is at most 1)
            float v = -1.f; int i = 0x7fffffff;
            for (int g = lane; g < a.groups; g += 32) if (gs[g] <= 1.f && gs[g] > v) { v = gs[g]; i = g; }
            moe_warp_argmax(v, i);
            if (lane == 0) gs[i] = 2.f;
            __syncwarp();
        }
        for (int e = lane; e < a.E; e += 32) if (gs[e / size] <= 1.f) s[e] = -1.f;
        __syncwarp();
    }
    float total = 0.f, mine = 0.f;                           // lane k keeps the k-th pick (32 picks at a time)
    int mine_id = 0;
    for (int k0 = 0; k0 < a.top; k0 += 32) {
        const int n = min(32, a.top - k0);
        for (int k = 0; k < n; ++k) {
            float v = -1.f; int i = 0x7fffffff;
            for (int e = lane; e < a.E; e += 32) if (s[e] > v) { v = s[e]; i = e; }
            moe_warp_argmax(v, i);
            if (lane == k) { mine = v; mine_id = i; }
            if (lane == 0) s[i] = -1.f;
            total += v;
            __syncwarp();
        }
        if (lane < n) {
            a.ids[(size_t)t * a.top + k0 + lane] = mine_id;
            a.weights[(size_t)t * a.top + k0 + lane] = mine;        // divided below, once the sum is known
        }
    }
    __syncwarp();
    const float norm = a.scale / (total + 1e-20f);
    for (int k = lane; k < a.top; k += 32) a.weights[(size_t)t * a.top + k] *= norm;
    if (a.sgate && lane == 0) a.sgate[t] = 1.0f / (1.0f + expf(-zr[a.E]));
}

extern "C" int ce_moe_route(const float* z, int* ids, float* weights, float* sgate, int T, int ld, int E, int top, int groups,
                            int keep, float scale, cudaStream_t stream) {
    if (T == 0) return CE_OK;
    if (!z || !ids || !weights) return ce_fail(CE_ERR_ARG, "ce_moe_route: null pointer");
    if (E <= 0 || E > MOE_MAX_EXPERTS || top <= 0 || top > E || groups <= 0 || E % groups || keep <= 0 || keep > groups ||
        (long long)keep * (E / groups) < top || ld < E + (sgate ? 1 : 0))
        return ce_fail(CE_ERR_SIZE, "ce_moe_route: %d experts, top %d, %d groups of which %d are kept", E, top, groups, keep);
    MoeRouteArgs a{z, ids, weights, sgate, T, ld, E, top, groups, keep, scale};
    size_t smem = (size_t)4 * 2 * E * sizeof(float);
    if (smem > 40 * 1024) cudaFuncSetAttribute(moe_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    ce_note("moe_route_kernel");
    ce_launch(moe_route_kernel, (T + 3) / 4, 128, smem, stream, a);
    return ce_check_launch("ce_moe_route");
}

// ---------------------------------------------------------------------------------------------
// the pairs laid out by expert: one block
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) moe_align_kernel(const int* __restrict__ ids, int n, int top, int E, int BM, int max_rows,
                                                         int* __restrict__ row_token, int* __restrict__ pair_row,
                                                         int* __restrict__ tile_expert, int* __restrict__ n_tiles) {
    ce_pdl_begin();
    extern __shared__ int moe_align_smem[];
    int* count = moe_align_smem;          // [E], then the next free row of every expert
    int* first = count + E;               // [E + 1]: an expert's first row
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        int e = ids[i];
        if (e >= 0 && e < E) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x < 32) {               // a warp's running sum over the experts, 32 at a time
        int base = 0;
        for (int e0 = 0; e0 < E; e0 += 32) {
            int e = e0 + threadIdx.x;
            int c = e < E ? (count[e] + BM - 1) / BM * BM : 0, incl = c;
            for (int o = 1; o < 32; o <<= 1) {
                int v = __shfl_up_sync(0xffffffffu, incl, o);
                if ((int)threadIdx.x >= o) incl += v;
            }
            if (e < E) first[e] = base + incl - c;
            base += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (threadIdx.x == 0) { first[E] = base; n_tiles[0] = base / BM; }
    }
    __syncthreads();
    const int rows = first[E];
    for (int p = threadIdx.x; p < rows && p < max_rows; p += blockDim.x) row_token[p] = -1;
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        for (int p = first[e]; p < first[e + 1]; p += BM) tile_expert[p / BM] = e;
        count[e] = first[e];
    }
    __syncthreads();
    // an expert's rows in the order of the pairs: a thread's pairs are consecutive, and the threads take their turns by
    // counting how many earlier pairs name the same expert (ranks through shared-memory counters, chunk by chunk)
    for (int i0 = 0; i0 < n; i0 += blockDim.x) {
        int i = i0 + threadIdx.x;
        int e = i < n ? ids[i] : -1;
        // rank among the chunk's pairs of the same expert: warp by warp, in order
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
            if ((int)(threadIdx.x >> 5) == w && e >= 0 && e < E) {
                unsigned same = __match_any_sync(__activemask(), e);
                int rank = __popc(same & ((1u << (threadIdx.x & 31)) - 1));
                int base = count[e];
                __syncwarp(__activemask());
                int p = base + rank;
                pair_row[i] = p;
                row_token[p] = i / top;
                if (rank == __popc(same) - 1) count[e] = base + rank + 1;
            }
            __syncthreads();
        }
    }
}

extern "C" int ce_moe_max_tiles(int n_pairs, int E, int BM) {
    int busy = n_pairs < E ? n_pairs : E;                   // experts that can have a part-filled tile
    return n_pairs / BM + busy;
}

extern "C" int ce_moe_align(const int* ids, int n_pairs, int top, int E, int BM, int max_rows, int* row_token, int* pair_row,
                            int* tile_expert, int* n_tiles, cudaStream_t stream) {
    if (n_pairs == 0) return CE_OK;
    if (!ids || !row_token || !pair_row || !tile_expert || !n_tiles) return ce_fail(CE_ERR_ARG, "ce_moe_align: null pointer");
    if (E <= 0 || E > MOE_MAX_EXPERTS || BM <= 0 || top <= 0 || max_rows < ce_moe_max_tiles(n_pairs, E, BM) * BM)
        return ce_fail(CE_ERR_SIZE, "ce_moe_align: %d experts, tiles of %d, room for %d rows", E, BM, max_rows);
    size_t smem = (size_t)(2 * E + 1) * sizeof(int);
    ce_note("moe_align_kernel");
    int threads = n_pairs >= 1024 ? 1024 : (n_pairs + 31) / 32 * 32;
    ce_launch(moe_align_kernel, 1, threads, smem, stream, ids, n_pairs, top, E, BM, max_rows, row_token, pair_row, tile_expert, n_tiles);
    return ce_check_launch("ce_moe_align");
}

// ---------------------------------------------------------------------------------------------
// grouped products
// ---------------------------------------------------------------------------------------------
enum { MOE_ACT_NONE = 0, MOE_ACT_RELU2 = 1 };

__device__ __forceinline__ float moe_act(int act, float v) {
    if (act == MOE_ACT_RELU2) { v = fmaxf(v, 0.f); return v * v; }
    return v;
}

struct MoeMatmulArgs {
    const void* in;              // [*, ldi]: row p's input is row row_token[p] (gather) or row p
    const void* W;               // [E, N, K]
    void* out;                   // [rows, ldo]
    const int* row_token;        // or null: rows are taken as they lie
    const int* tile_expert;
    const int* n_tiles;          // or null: every tile of the grid
    int ldi, ldo, N, K, BM, act, n_rows;     // n_rows: rows of `in` when they are taken as they lie (later rows are padding)
};

#define MP_BN 64
#define MP_BK 16

// float32 FMA: a block of 256 threads takes BM (16 or 64) rows x 64 outputs; a thread (BM / 16) x 4 of them
template <typename T, int BM>
__global__ void __launch_bounds__(256) moe_matmul_plain_kernel(MoeMatmulArgs a) {
    ce_pdl_begin();
    const int tile = blockIdx.y;
    if (a.n_tiles && tile >= a.n_tiles[0]) return;
    constexpr int RPT = BM / 16;
    __shared__ float As[MP_BK][BM + 1];
    __shared__ float Ws[MP_BK][MP_BN + 1];
    __shared__ int src[BM];
    const int tid = threadIdx.x, n0 = blockIdx.x * MP_BN, p0 = tile * BM;
    const T* W = (const T*)a.W + (size_t)(a.tile_expert ? a.tile_expert[tile] : 0) * a.N * a.K;
    if (tid < BM) src[tid] = a.row_token ? a.row_token[p0 + tid] : (p0 + tid < a.n_rows ? p0 + tid : -1);
    __syncthreads();
    const int tm = (tid / 16) * RPT, tn = (tid % 16) * 4;
    float acc[RPT][4];
#pragma unroll
    for (int i = 0; i < RPT; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < a.K; k0 += MP_BK) {
        for (int e = tid; e < BM * MP_BK; e += 256) {
            int r = e / MP_BK, c = e % MP_BK, row = src[r];
            As[c][r] = (row >= 0 && k0 + c < a.K) ? CeType<T>::load((const T*)a.in + (size_t)row * a.ldi + k0 + c) : 0.f;
        }
        for (int e = tid; e < MP_BN * MP_BK; e += 256) {
            int r = e / MP_BK, c = e % MP_BK;
            Ws[c][r] = (n0 + r < a.N && k0 + c < a.K) ? CeType<T>::load(W + (size_t)(n0 + r) * a.K + k0 + c) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < MP_BK; ++kk) {
            float wv[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) wv[j] = Ws[kk][tn + j];
#pragma unroll
            for (int i = 0; i < RPT; ++i) {
                float av = As[kk][tm + i];
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av, wv[j], acc[i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < RPT; ++i) {
        if (src[tm + i] < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j)
            if (n0 + tn + j < a.N) CeType<T>::store((T*)a.out + (size_t)(p0 + tm + i) * a.ldo + n0 + tn + j, moe_act(a.act, acc[i][j]));
    }
}

// bfloat16 on the tensor cores: four warps; with tiles of 64 rows a warp takes 16 rows x 64 outputs, with tiles of 16 rows
// the warps take the four 16-column parts of the 64 outputs for the same rows.  The rows go through shared memory 64
// elements of K at a time; the weights' fragments come straight from memory (W[e] is [N, K] row-major: K x N column-major).
#define MW_BN 64
#define MW_BK 64

template <int BM>
__global__ void __launch_bounds__(128) moe_matmul_wmma_kernel(MoeMatmulArgs a) {
    using namespace nvcuda;
    ce_pdl_begin();
    const int tile = blockIdx.y;
    if (a.n_tiles && tile >= a.n_tiles[0]) return;
    constexpr bool FEW = BM == 16;
    __shared__ __align__(32) __nv_bfloat16 As[BM][MW_BK + 16];
    __shared__ __align__(32) float Cs[BM][MW_BN + 8];
    __shared__ int src[BM];
    const int tid = threadIdx.x, warp = tid >> 5, n0 = blockIdx.x * MW_BN, p0 = tile * BM;
    const __nv_bfloat16* W = (const __nv_bfloat16*)a.W + (size_t)(a.tile_expert ? a.tile_expert[tile] : 0) * a.N * a.K;
    const __nv_bfloat16* in = (const __nv_bfloat16*)a.in;
    if (tid < BM) src[tid] = a.row_token ? a.row_token[p0 + tid] : (p0 + tid < a.n_rows ? p0 + tid : -1);
    __syncthreads();
    const int n_frag = min(MW_BN, a.N - n0) / 16;
    constexpr int NF = FEW ? 1 : MW_BN / 16;
    const int wrow = FEW ? 0 : warp * 16, f0 = FEW ? warp : 0;
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[NF];
#pragma unroll
    for (int j = 0; j < NF; ++j) wmma::fill_fragment(acc[j], 0.f);
    for (int k0 = 0; k0 < a.K; k0 += MW_BK) {
        const int kw = min(MW_BK, a.K - k0);
        for (int e = tid; e < BM * (MW_BK / 8); e += 128) {
            int r = e / (MW_BK / 8), c = (e % (MW_BK / 8)) * 8, row = src[r];
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (row >= 0 && c < kw) v = *reinterpret_cast<const uint4*>(in + (size_t)row * a.ldi + k0 + c);
            *reinterpret_cast<uint4*>(&As[r][c]) = v;
        }
        __syncthreads();
        for (int kk = 0; kk < kw; kk += 16) {
            wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa;
            wmma::load_matrix_sync(fa, &As[wrow][kk], MW_BK + 16);
#pragma unroll
            for (int j = 0; j < NF; ++j) {
                if (f0 + j < n_frag) {
                    wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb;
                    wmma::load_matrix_sync(fb, W + (size_t)(n0 + (f0 + j) * 16) * a.K + k0 + kk, a.K);
                    wmma::mma_sync(acc[j], fa, fb, acc[j]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < NF; ++j)
        if (f0 + j < n_frag) wmma::store_matrix_sync(&Cs[wrow][(f0 + j) * 16], acc[j], MW_BN + 8, wmma::mem_row_major);
    __syncthreads();
    for (int e = tid; e < BM * (MW_BN / 2); e += 128) {
        int r = e / (MW_BN / 2), c = (e % (MW_BN / 2)) * 2;
        if (src[r] < 0 || n0 + c >= a.N) continue;
        __nv_bfloat162 v = __floats2bfloat162_rn(moe_act(a.act, Cs[r][c]), moe_act(a.act, Cs[r][c + 1]));
        *reinterpret_cast<__nv_bfloat162*>((__nv_bfloat16*)a.out + (size_t)(p0 + r) * a.ldo + n0 + c) = v;
    }
}

// in [*, ldi], W [E, N, K], out [max_tiles * BM, ldo]; BM is 16 or 64 and is the tile height the layout was made with.
// Without the layout's tables (all three null) it is one expert's product over n_rows rows as they lie.
extern "C" int ce_moe_matmul(const void* in, const void* W, void* out, const int* row_token, const int* tile_expert,
                             const int* n_tiles, int dtype, int max_tiles, int BM, int N, int K, int ldi, int ldo, int act,
                             int n_rows, cudaStream_t stream) {
    if (max_tiles == 0 || N == 0) return CE_OK;
    if (!in || !W || !out || K <= 0) return ce_fail(CE_ERR_ARG, "ce_moe_matmul: null pointer or K=%d", K);
    if ((BM != 16 && BM != 64) || max_tiles > 65535) return ce_fail(CE_ERR_SIZE, "ce_moe_matmul: tiles of %d rows, %d tiles", BM, max_tiles);
    MoeMatmulArgs a{in, W, out, row_token, tile_expert, n_tiles, ldi, ldo, N, K, BM, act, n_rows};
    if (dtype == CE_BF16 && N % 16 == 0 && K % 16 == 0 && ldi % 8 == 0 && ldo % 2 == 0 &&
        ((((uintptr_t)in) & 15) == 0) && ((((uintptr_t)W) & 31) == 0) && ((((uintptr_t)out) & 3) == 0)) {
        dim3 grid((N + MW_BN - 1) / MW_BN, max_tiles);
        ce_note("moe_matmul_wmma_kernel");
        if (BM == 16) ce_launch(moe_matmul_wmma_kernel<16>, grid, 128, 0, stream, a);
        else ce_launch(moe_matmul_wmma_kernel<64>, grid, 128, 0, stream, a);
        return ce_check_launch("ce_moe_matmul");
    }
    dim3 grid((N + MP_BN - 1) / MP_BN, max_tiles);
    ce_note("moe_matmul_plain_kernel");
    if (dtype == CE_F32 && BM == 16) ce_launch(moe_matmul_plain_kernel<float, 16>, grid, 256, 0, stream, a);
    else if (dtype == CE_F32) ce_launch(moe_matmul_plain_kernel<float, 64>, grid, 256, 0, stream, a);
    else if (dtype == CE_BF16 && BM == 16) ce_launch(moe_matmul_plain_kernel<__nv_bfloat16, 16>, grid, 256, 0, stream, a);
    else if (dtype == CE_BF16) ce_launch(moe_matmul_plain_kernel<__nv_bfloat16, 64>, grid, 256, 0, stream, a);
    else return ce_fail(CE_ERR_ARG, "ce_moe_matmul: unknown dtype %d", dtype);
    return ce_check_launch("ce_moe_matmul");
}

// ---------------------------------------------------------------------------------------------
// the tokens' rows copied into the layout's order (what a product that loads its rows by TMA reads): row p of the
// live tiles receives row row_token[p] of the input, zeros where p is padding.  Rows are copied 16 bytes a thread.
// ---------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) moe_gather_kernel(const uint4* __restrict__ in, long long ldi16, const int* __restrict__ row_token,
                                                         const int* __restrict__ n_tiles, int BM, uint4* __restrict__ out, int row16,
                                                         int max_rows) {
    ce_pdl_begin();
    const int rows = min(n_tiles[0] * BM, max_rows);
    const int per = blockDim.x / row16 > 0 ? blockDim.x / row16 : 1;          // rows a block copies at a time
    for (int p0 = blockIdx.x * per; p0 < rows; p0 += gridDim.x * per) {
        if (row16 <= (int)blockDim.x) {
            int p = p0 + threadIdx.x / row16, j = threadIdx.x % row16;
            if (threadIdx.x < per * row16 && p < rows) {
                int t = row_token[p];
                out[(size_t)p * row16 + j] = t >= 0 ? in[(size_t)t * ldi16 + j] : make_uint4(0, 0, 0, 0);
            }
        } else {
            int t = row_token[p0];
            for (int j = threadIdx.x; j < row16; j += blockDim.x)
                out[(size_t)p0 * row16 + j] = t >= 0 ? in[(size_t)t * ldi16 + j] : make_uint4(0, 0, 0, 0);
        }
    }
}

// in [T, ldi] -> out [max_rows, K] (contiguous), elements of `elsize` bytes; K * elsize and ldi * elsize multiples of 16
extern "C" int ce_moe_gather(const void* in, int ldi, int K, int elsize, const int* row_token, const int* n_tiles, int BM, void* out,
                             int max_rows, cudaStream_t stream) {
    if (max_rows == 0 || K == 0) return CE_OK;
    if (!in || !row_token || !n_tiles || !out) return ce_fail(CE_ERR_ARG, "ce_moe_gather: null pointer");
    if (((long long)K * elsize) % 16 || ((long long)ldi * elsize) % 16 || (((uintptr_t)in | (uintptr_t)out) & 15) || BM <= 0)
        return ce_fail(CE_ERR_SIZE, "ce_moe_gather: rows of %d elements of %d bytes are not whole 16-byte pieces", K, elsize);
    int row16 = (int)((long long)K * elsize / 16);
    int per = 256 / row16 > 0 ? 256 / row16 : 1;
    int blocks = (max_rows + per - 1) / per;
    int cap = ce_sm_count() * 8;
    if (blocks > cap) blocks = cap;
    ce_note("moe_gather_kernel");
    ce_launch(moe_gather_kernel, blocks, 256, 0, stream, (const uint4*)in, (long long)ldi * elsize / 16, row_token, n_tiles, BM, (uint4*)out,
              row16, max_rows);
    return ce_check_launch("ce_moe_gather");
}

// ---------------------------------------------------------------------------------------------
// back to token order
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ rows, int ld, const int* __restrict__ pair_row, const float* __restrict__ weights,
                                   const T* __restrict__ shared, const float* __restrict__ sgate, float* __restrict__ y, int top,
                                   int W, int accumulate) {
    ce_pdl_begin();
    const int t = blockIdx.x;
    for (int j = threadIdx.x; j < W; j += blockDim.x) {
        float v = 0.f;
        for (int k = 0; k < top; ++k)
            v = fmaf(weights[(size_t)t * top + k], CeType<T>::load(rows + (size_t)pair_row[(size_t)t * top + k] * ld + j), v);
        if (shared) v = fmaf(sgate ? sgate[t] : 1.0f, CeType<T>::load(shared + (size_t)t * W + j), v);
        float* o = y + (size_t)t * W + j;
        *o = accumulate ? *o + v : v;
    }
}

extern "C" int ce_moe_combine(const void* rows, int dtype, int ld, const int* pair_row, const float* weights, const void* shared,
                              const float* sgate, float* y, int T, int top, int W, int accumulate, cudaStream_t stream) {
    if (T == 0 || W == 0) return CE_OK;
    if (!rows || !pair_row || !weights || !y) return ce_fail(CE_ERR_ARG, "ce_moe_combine: null pointer");
    int threads = W >= 1024 ? 256 : 128;
    ce_note("moe_combine_kernel");
    if (dtype == CE_F32) ce_launch(moe_combine_kernel<float>, T, threads, 0, stream, (const float*)rows, ld, pair_row, weights, (const float*)shared, sgate, y, top, W, accumulate);
    else if (dtype == CE_BF16) ce_launch(moe_combine_kernel<__nv_bfloat16>, T, threads, 0, stream, (const __nv_bfloat16*)rows, ld, pair_row, weights, (const __nv_bfloat16*)shared, sgate, y, top, W, accumulate);
    else return ce_fail(CE_ERR_ARG, "ce_moe_combine: unknown dtype %d", dtype);
    return ce_check_launch("ce_moe_combine");
}
