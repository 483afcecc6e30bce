// Softmax attention over the paged cache with the options that several designs combine differently, each a
// parameter: key and value heads of different sizes, a tanh cap on the scores, a sliding window that may keep a
// sequence's first tokens visible, a sigmoid gate per output element, and a value pool that is a view of the key
// pool (latent attention keeps ONE row per token, of which the values are the leading part).  Float32 arithmetic,
// any number of new tokens per sequence; it is the float32 path and the plain twin of the tensor-core kernel.
//
// Also here: the blend of a layer's values with the values another layer computed for the same tokens, the
// preparation of latent attention's operands (query latent norm, key latent norm, rotation of the shared key
// part, the cache write), the rotation of the queries' rotated parts, and a product per head
// (out[t, h] = W[h] in[t, h]) with an optional sigmoid gate.
#include "common.cuh"

__device__ __forceinline__ float ma_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// ---------------------------------------------------------------------------------------------
// v <- (1 - lam) v + lam v_first on the value columns of a product's output rows, in place
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void value_mix_kernel(T* __restrict__ rows, int stride, int off, int n, const T* __restrict__ first, int first_stride,
                                 int first_off, float lam, size_t total) {
    ce_pdl_begin();
    size_t step = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += step) {
        size_t t = e / n;
        int j = (int)(e % n);
        T* p = rows + t * stride + off + j;
        float v = CeType<T>::load(p), f = CeType<T>::load(first + t * first_stride + first_off + j);
        CeType<T>::store(p, (1.0f - lam) * v + lam * f);
    }
}

extern "C" int ce_value_mix(void* rows, int dtype, int stride, int off, int n, const void* first, int first_stride, int first_off,
                            float lam, int T, cudaStream_t stream) {
    if (T == 0 || n == 0) return CE_OK;
    if (!rows || !first) return ce_fail(CE_ERR_ARG, "ce_value_mix: null pointer");
    size_t total = (size_t)T * n, want = (total + 255) / 256;
    int blocks = (int)(want < (size_t)148 * 8 ? want : (size_t)148 * 8);
    ce_note("value_mix_kernel");
    if (dtype == CE_F32) ce_launch(value_mix_kernel<float>, blocks, 256, 0, stream, (float*)rows, stride, off, n, (const float*)first, first_stride, first_off, lam, total);
    else if (dtype == CE_BF16) ce_launch(value_mix_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (__nv_bfloat16*)rows, stride, off, n, (const __nv_bfloat16*)first, first_stride, first_off, lam, total);
    else return ce_fail(CE_ERR_ARG, "ce_value_mix: unknown dtype %d", dtype);
    return ce_check_launch("ce_value_mix");
}

// ---------------------------------------------------------------------------------------------
// Operands of attention with a norm per head: proj [T, ld] float32 holds, per token, nh query heads of d from off_q, nkv key
// heads of d from off_k and nkv value heads of dv from off_v.  Each query and key head is divided by its root mean square and
// multiplied by a weight of size d (wq, wk; null: no norm), then rotated over its first rd elements (element i with
// i + rd/2) by the token's position; query head h is also multiplied by head_scale[h] (a temperature per head folded into
// the query; null: none).  Queries go to q_out [T, nh * d], keys and values to the token's place in the pools.  The values
// may be the keys as projected (off_v = off_k, dv = d): they are read before the norm and the rotation.
// A warp per head in turn.
// ---------------------------------------------------------------------------------------------
struct NormRopeArgs {
    const float* proj;
    void* q_out;
    void* k_pool;                // [num_pages, nkv, page_size, d]
    void* v_pool;                // [num_pages, nkv, page_size, dv]
    const float* wq;
    const float* wk;
    const float* head_scale;
    const float* cos_table;      // [max_pos, rd/2] or null
    const float* sin_table;
    const int* positions;
    const int* seq_of_token;
    const int* seq_slot;
    const int* block_table;
    int* status;
    int ld, off_q, off_k, off_v, nh, nkv, d, dv, rd, page_size, max_pages, num_pages, max_pos, write_kv;
    float eps;
};

template <typename T>
__global__ void norm_rope_kvwrite_kernel(NormRopeArgs a) {
    ce_pdl_begin();
    int t = blockIdx.x, lane = threadIdx.x & 31, nwarp = (blockDim.x >> 5) * gridDim.y;
    int warp = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int d = a.d, half = a.rd / 2;
    int p = a.positions[t];
    const float* row = a.proj + (size_t)t * a.ld;
    bool rotate = a.cos_table != nullptr && half > 0;
    if (rotate && (p < 0 || p >= a.max_pos)) {
        if (threadIdx.x == 0) atomicExch(a.status, 3);
        rotate = false;
    }
    int page = -1, off = 0;
    if (a.write_kv) {
        int slot = a.seq_slot[a.seq_of_token[t]];
        page = a.block_table[(size_t)slot * a.max_pages + p / a.page_size];
        off = p % a.page_size;
        if (page < 0 || page >= a.num_pages) {
            if (threadIdx.x == 0) atomicExch(a.status, 2);
            page = -1;
        }
    }
    const float* cs = rotate ? a.cos_table + (size_t)p * half : nullptr;
    const float* sn = rotate ? a.sin_table + (size_t)p * half : nullptr;
    for (int hh = warp; hh < a.nh + a.nkv; hh += nwarp) {
        bool is_q = hh < a.nh;
        const float* src = row + (is_q ? a.off_q + hh * d : a.off_k + (hh - a.nh) * d);
        const float* w = is_q ? a.wq : a.wk;
        T* dst;
        if (is_q) dst = (T*)a.q_out + ((size_t)t * a.nh + hh) * d;
        else {
            if (page < 0) continue;
            dst = (T*)a.k_pool + (((size_t)page * a.nkv + (hh - a.nh)) * a.page_size + off) * d;
        }
        float inv = 1.0f;
        if (w) {
            float ss = 0.f;
            for (int j = lane; j < d; j += 32) ss = fmaf(src[j], src[j], ss);
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            inv = 1.0f / sqrtf(ss / (float)d + a.eps);
        }
        float hs = is_q && a.head_scale ? a.head_scale[hh] : 1.0f;
        for (int j = lane; j < d; j += 32) {
            float x = w ? src[j] * inv * w[j] : src[j];
            if (rotate && j < a.rd) {
                int partner = j < half ? j + half : j - half;
                float y = w ? src[partner] * inv * w[partner] : src[partner];
                x = j < half ? x * cs[j] - y * sn[j] : x * cs[j - half] + y * sn[j - half];
            }
            CeType<T>::store(dst + j, x * hs);
        }
    }
    if (page >= 0) {
        for (int e = blockIdx.y * blockDim.x + threadIdx.x; e < a.nkv * a.dv; e += blockDim.x * gridDim.y) {
            int h = e / a.dv, j = e % a.dv;
            CeType<T>::store((T*)a.v_pool + (((size_t)page * a.nkv + h) * a.page_size + off) * a.dv + j, row[a.off_v + e]);
        }
    }
}

extern "C" int ce_norm_rope_kvwrite(const float* proj, void* q_out, void* k_pool, void* v_pool, int dtype, const float* wq,
                                    const float* wk, const float* head_scale, const float* cos_table, const float* sin_table,
                                    const int* positions, const int* seq_of_token, const int* seq_slot, const int* block_table,
                                    int* status, int T, int ld, int off_q, int off_k, int off_v, int nh, int nkv, int d, int dv, int rd,
                                    int page_size, int max_pages, int num_pages, int max_pos, int write_kv, float eps,
                                    cudaStream_t stream) {
    if (T == 0) return CE_OK;
    if (!proj || !q_out || !positions || !seq_of_token || !seq_slot || !status) return ce_fail(CE_ERR_ARG, "ce_norm_rope_kvwrite: null pointer");
    if (write_kv && (!k_pool || !v_pool || !block_table)) return ce_fail(CE_ERR_ARG, "ce_norm_rope_kvwrite: no cache to write to");
    if (rd < 0 || rd > d || rd % 2) return ce_fail(CE_ERR_SIZE, "ce_norm_rope_kvwrite: %d rotated elements of %d", rd, d);
    if (rd > 0 && (!cos_table || !sin_table)) return ce_fail(CE_ERR_ARG, "ce_norm_rope_kvwrite: no rotation tables");
    if (nh <= 0 || nkv <= 0 || d <= 0 || dv <= 0) return ce_fail(CE_ERR_SIZE, "ce_norm_rope_kvwrite: sizes");
    NormRopeArgs a{proj, q_out, k_pool, v_pool, wq, wk, head_scale, rd > 0 ? cos_table : nullptr, sin_table, positions, seq_of_token,
                   seq_slot, block_table, status, ld, off_q, off_k, off_v, nh, nkv, d, dv, rd, page_size, max_pages, num_pages, max_pos,
                   write_kv, eps};
    // a token's heads are dealt to the warps of gridDim.y blocks in turn: one block a token in a long step, a block per
    // handful of heads in a step of few tokens
    int heads = nh + nkv;
    int threads = heads >= 8 ? 256 : 32 * heads;
    int per_block = threads / 32, want = (heads + per_block - 1) / per_block, room = 4 * 148 / T;
    int split = want < room ? want : room;
    dim3 grid(T, split < 1 ? 1 : split);
    ce_note("norm_rope_kvwrite_kernel");
    if (dtype == CE_F32) ce_launch(norm_rope_kvwrite_kernel<float>, grid, threads, 0, stream, a);
    else if (dtype == CE_BF16) ce_launch(norm_rope_kvwrite_kernel<__nv_bfloat16>, grid, threads, 0, stream, a);
    else return ce_fail(CE_ERR_ARG, "ce_norm_rope_kvwrite: unknown dtype %d", dtype);
    return ce_check_launch("ce_norm_rope_kvwrite");
}

// ---------------------------------------------------------------------------------------------
// Latent attention's operands.  proj [T, ld] float32 holds, per token, the query latent (qr columns from off_q)
// and the key/value row (r latent columns, then dr columns of the rotated key part, from off_kv).
//   cq[t]  = rms_norm(query latent) * wq                                    -> [T, qr], activation dtype
//   page row of the token = [ rms_norm(latent) * wkv | rotate(key part) ]   -> K pool [pages, 1, page, r + dr]
// The rotation turns element i of the part's first rd with element i + rd/2 by the angle of the token's position.
// ---------------------------------------------------------------------------------------------
struct LatentPrepArgs {
    const float* proj;
    const float* wq;             // [qr]
    const float* wkv;            // [r]
    void* cq;                    // [T, qr]
    void* k_pool;
    const float* cos_table;      // [max_pos, rd/2]
    const float* sin_table;
    const int* positions;
    const int* seq_of_token;
    const int* seq_slot;
    const int* block_table;
    int* status;
    int ld, off_q, qr, off_kv, r, dr, rd, page_size, max_pages, num_pages, max_pos, write_kv;
    float eps;
};

template <typename T>
__global__ void latent_prepare_kernel(LatentPrepArgs a) {
    ce_pdl_begin();
    __shared__ float scratch[32];
    int t = blockIdx.x, p = a.positions[t];
    const float* row = a.proj + (size_t)t * a.ld;
    // the query latent
    float ss = 0.f;
    for (int j = threadIdx.x; j < a.qr; j += blockDim.x) ss = fmaf(row[a.off_q + j], row[a.off_q + j], ss);
    float inv = a.qr > 0 ? 1.0f / sqrtf(ce_block_sum(ss, scratch) / (float)a.qr + a.eps) : 0.f;    // qr 0: the queries are no latent
    for (int j = threadIdx.x; j < a.qr; j += blockDim.x)
        CeType<T>::store((T*)a.cq + (size_t)t * a.qr + j, row[a.off_q + j] * inv * a.wq[j]);
    if (!a.write_kv) return;
    int slot = a.seq_slot[a.seq_of_token[t]];
    int page = a.block_table[(size_t)slot * a.max_pages + p / a.page_size];
    if (page < 0 || page >= a.num_pages) {
        if (threadIdx.x == 0) atomicExch(a.status, 2);
        return;
    }
    T* dst = (T*)a.k_pool + ((size_t)page * a.page_size + p % a.page_size) * (a.r + a.dr);
    const float* kv = row + a.off_kv;
    ss = 0.f;
    for (int j = threadIdx.x; j < a.r; j += blockDim.x) ss = fmaf(kv[j], kv[j], ss);
    inv = 1.0f / sqrtf(ce_block_sum(ss, scratch) / (float)a.r + a.eps);
    for (int j = threadIdx.x; j < a.r; j += blockDim.x) CeType<T>::store(dst + j, kv[j] * inv * a.wkv[j]);
    int half = a.rd / 2;
    bool rotate = half > 0;
    if (rotate && (p < 0 || p >= a.max_pos)) {
        if (threadIdx.x == 0) atomicExch(a.status, 3);
        rotate = false;
    }
    const float* part = kv + a.r;
    for (int i = threadIdx.x; i < a.dr; i += blockDim.x) {
        float v;
        if (rotate && i < half) v = part[i] * a.cos_table[(size_t)p * half + i] - part[i + half] * a.sin_table[(size_t)p * half + i];
        else if (rotate && i < a.rd) v = part[i] * a.cos_table[(size_t)p * half + i - half] + part[i - half] * a.sin_table[(size_t)p * half + i - half];
        else v = part[i];
        CeType<T>::store(dst + a.r + i, v);
    }
}

extern "C" int ce_latent_prepare(const float* proj, const float* wq, const float* wkv, void* cq, void* k_pool, int dtype,
                                 const float* cos_table, const float* sin_table, const int* positions, const int* seq_of_token,
                                 const int* seq_slot, const int* block_table, int* status, int T, int ld, int off_q, int qr,
                                 int off_kv, int r, int dr, int rd, int page_size, int max_pages, int num_pages, int max_pos,
                                 int write_kv, float eps, cudaStream_t stream) {
    if (T == 0) return CE_OK;
    if (!proj || !positions || !seq_of_token || !seq_slot || !status || (qr > 0 && (!wq || !cq)))
        return ce_fail(CE_ERR_ARG, "ce_latent_prepare: null pointer");
    if (write_kv && (!k_pool || !block_table || !wkv)) return ce_fail(CE_ERR_ARG, "ce_latent_prepare: no cache to write to");
    if (rd < 0 || rd > dr || rd % 2 || (rd > 0 && (!cos_table || !sin_table)))
        return ce_fail(CE_ERR_SIZE, "ce_latent_prepare: %d rotated elements of %d", rd, dr);
    LatentPrepArgs a{proj, wq, wkv, cq, k_pool, cos_table, sin_table, positions, seq_of_token, seq_slot, block_table, status,
                     ld, off_q, qr, off_kv, r, dr, rd, page_size, max_pages, num_pages, max_pos, write_kv, eps};
    int threads = (qr > r ? qr : r) >= 1024 ? 256 : 128;
    ce_note("latent_prepare_kernel");
    if (dtype == CE_F32) ce_launch(latent_prepare_kernel<float>, T, threads, 0, stream, a);
    else if (dtype == CE_BF16) ce_launch(latent_prepare_kernel<__nv_bfloat16>, T, threads, 0, stream, a);
    else return ce_fail(CE_ERR_ARG, "ce_latent_prepare: unknown dtype %d", dtype);
    return ce_check_launch("ce_latent_prepare");
}

// ---------------------------------------------------------------------------------------------
// dst[t, h, dst_off + i] = rotate(src[t, h, src_off + i]) for i < dr: the rotated part of every query head moves
// into the row the attention reads, turned by the angle of the token's position.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_part_kernel(const T* __restrict__ src, int src_stride, int src_head, int src_off, T* __restrict__ dst,
                                 int dst_stride, int dst_head, int dst_off, const float* __restrict__ cos_table,
                                 const float* __restrict__ sin_table, const int* __restrict__ positions, int* __restrict__ status,
                                 int H, int dr, int rd, int max_pos) {
    ce_pdl_begin();
    int t = blockIdx.x, p = positions[t], half = rd / 2;
    bool rotate = half > 0;
    if (rotate && (p < 0 || p >= max_pos)) {
        if (threadIdx.x == 0) atomicExch(status, 3);
        rotate = false;
    }
    for (int e = threadIdx.x; e < H * dr; e += blockDim.x) {
        int h = e / dr, i = e % dr;
        const T* s = src + (size_t)t * src_stride + (size_t)h * src_head + src_off;
        float v;
        if (rotate && i < half)
            v = CeType<T>::load(s + i) * cos_table[(size_t)p * half + i] - CeType<T>::load(s + i + half) * sin_table[(size_t)p * half + i];
        else if (rotate && i < rd)
            v = CeType<T>::load(s + i) * cos_table[(size_t)p * half + i - half] + CeType<T>::load(s + i - half) * sin_table[(size_t)p * half + i - half];
        else v = CeType<T>::load(s + i);
        CeType<T>::store(dst + (size_t)t * dst_stride + (size_t)h * dst_head + dst_off + i, v);
    }
}

extern "C" int ce_rope_part(const void* src, int src_stride, int src_head, int src_off, void* dst, int dst_stride, int dst_head,
                            int dst_off, int dtype, const float* cos_table, const float* sin_table, const int* positions,
                            int* status, int T, int H, int dr, int rd, int max_pos, cudaStream_t stream) {
    if (T == 0 || H == 0 || dr == 0) return CE_OK;
    if (!src || !dst || !positions || !status) return ce_fail(CE_ERR_ARG, "ce_rope_part: null pointer");
    if (rd < 0 || rd > dr || rd % 2 || (rd > 0 && (!cos_table || !sin_table)))
        return ce_fail(CE_ERR_SIZE, "ce_rope_part: %d rotated elements of %d", rd, dr);
    int threads = H * dr >= 1024 ? 256 : 128;
    ce_note("rope_part_kernel");
    if (dtype == CE_F32) ce_launch(rope_part_kernel<float>, T, threads, 0, stream, (const float*)src, src_stride, src_head, src_off, (float*)dst, dst_stride, dst_head, dst_off, cos_table, sin_table, positions, status, H, dr, rd, max_pos);
    else if (dtype == CE_BF16) ce_launch(rope_part_kernel<__nv_bfloat16>, T, threads, 0, stream, (const __nv_bfloat16*)src, src_stride, src_head, src_off, (__nv_bfloat16*)dst, dst_stride, dst_head, dst_off, cos_table, sin_table, positions, status, H, dr, rd, max_pos);
    else return ce_fail(CE_ERR_ARG, "ce_rope_part: unknown dtype %d", dtype);
    return ce_check_launch("ce_rope_part");
}

// ---------------------------------------------------------------------------------------------
// A product per head: out[t, h*out_head + j] = sum_i in[t, h*in_head + i] * W[h, j, i]  (j < N, i < K), float32
// sums in the order of i; optionally times sigmoid(gate[t, h*N + j]) (gate logits float32), or, with one gate a head
// (gate_head), times sigmoid(gate[t, h]).  Tiles of 16 tokens x 64 outputs of one head.
// ---------------------------------------------------------------------------------------------
#define HM_TM 16
#define HM_TN 64
#define HM_TK 32

template <typename T>
__global__ void __launch_bounds__(256) head_matmul_kernel(const T* __restrict__ in, int in_stride, int in_head, const T* __restrict__ W,
                                                          T* __restrict__ out, int out_stride, int out_head, const float* __restrict__ gate,
                                                          int gate_stride, int gate_head, int M, int N, int K) {
    ce_pdl_begin();
    __shared__ float As[HM_TM][HM_TK + 1];
    __shared__ float Ws[HM_TN][HM_TK + 1];
    int h = blockIdx.z, m0 = blockIdx.y * HM_TM, n0 = blockIdx.x * HM_TN, tid = threadIdx.x;
    int tm = tid / 16, tn = tid % 16;           // this thread: token tm, outputs tn, tn + 16, tn + 32, tn + 48
    const T* Wh = W + (size_t)h * N * K;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < K; k0 += HM_TK) {
        for (int e = tid; e < HM_TM * HM_TK; e += 256) {
            int r = e / HM_TK, c = e % HM_TK;
            As[r][c] = (m0 + r < M && k0 + c < K) ? CeType<T>::load(in + (size_t)(m0 + r) * in_stride + (size_t)h * in_head + k0 + c) : 0.f;
        }
        for (int e = tid; e < HM_TN * HM_TK; e += 256) {
            int r = e / HM_TK, c = e % HM_TK;
            Ws[r][c] = (n0 + r < N && k0 + c < K) ? CeType<T>::load(Wh + (size_t)(n0 + r) * K + k0 + c) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HM_TK; ++kk) {
            float av = As[tm][kk];
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = fmaf(av, Ws[tn + 16 * j][kk], acc[j]);
        }
        __syncthreads();
    }
    int m = m0 + tm;
    if (m >= M) return;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        int n = n0 + tn + 16 * j;
        if (n >= N) continue;
        float v = acc[j];
        if (gate) v *= ma_sigmoid(gate[(size_t)m * gate_stride + (gate_head ? (size_t)h : (size_t)h * N + n)]);
        CeType<T>::store(out + (size_t)m * out_stride + (size_t)h * out_head + n, v);
    }
}

// The same product in bfloat16 on the tensor cores (wmma m16n16k16, float32 sums): a block of four warps takes 64 tokens x 64
// outputs of one head; the tokens' rows go through shared memory 64 elements of K at a time (rows past the last token are
// zeros), the weights' fragments come straight from memory (W[h] is [N, K] row-major, that is K x N column-major with
// leading dimension K).  Wants N and K in multiples of 16 and rows that start on 32-byte boundaries.  With at most 16 tokens
// (FEW) the four warps take the four 16-column parts of the block's outputs for the same 16 rows instead of 16 rows each: a
// warp then walks K with one weight fragment a step instead of four, and its chain of loads is a quarter as long.
#include <mma.h>
#define HW_TM 64
#define HW_TN 64
#define HW_TK 64

template <bool FEW>
__global__ void __launch_bounds__(128) head_matmul_wmma_kernel(const __nv_bfloat16* __restrict__ in, int in_stride, int in_head,
                                                               const __nv_bfloat16* __restrict__ W, __nv_bfloat16* __restrict__ out,
                                                               int out_stride, int out_head, const float* __restrict__ gate,
                                                               int gate_stride, int gate_head, int M, int N, int K) {
    using namespace nvcuda;
    ce_pdl_begin();
    __shared__ __align__(32) __nv_bfloat16 As[HW_TM][HW_TK + 16];
    __shared__ __align__(32) float Cs[HW_TM][HW_TN + 8];
    int h = blockIdx.z, m0 = blockIdx.y * HW_TM, n0 = blockIdx.x * HW_TN, tid = threadIdx.x, warp = tid >> 5;
    const __nv_bfloat16* Wh = W + (size_t)h * N * K;
    int n_frag = min(HW_TN, N - n0) / 16;
    constexpr int NF = FEW ? 1 : HW_TN / 16;              // fragments a warp holds
    const int wrow = FEW ? 0 : warp * 16, f0 = FEW ? warp : 0;
    wmma::fragment<wmma::accumulator, 16, 16, 16, float> acc[NF];
#pragma unroll
    for (int j = 0; j < NF; ++j) wmma::fill_fragment(acc[j], 0.f);
    for (int k0 = 0; k0 < K; k0 += HW_TK) {
        int kw = min(HW_TK, K - k0);                      // a multiple of 16
        for (int e = tid; e < (FEW ? 16 : HW_TM) * (HW_TK / 8); e += 128) {
            int r = e / (HW_TK / 8), c = (e % (HW_TK / 8)) * 8;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (m0 + r < M && c < kw) v = *reinterpret_cast<const uint4*>(in + (size_t)(m0 + r) * in_stride + (size_t)h * in_head + k0 + c);
            *reinterpret_cast<uint4*>(&As[r][c]) = v;
        }
        __syncthreads();
        for (int kk = 0; kk < kw; kk += 16) {
            wmma::fragment<wmma::matrix_a, 16, 16, 16, __nv_bfloat16, wmma::row_major> fa;
            wmma::load_matrix_sync(fa, &As[wrow][kk], HW_TK + 16);
#pragma unroll
            for (int j = 0; j < NF; ++j) {
                if (f0 + j < n_frag) {
                    wmma::fragment<wmma::matrix_b, 16, 16, 16, __nv_bfloat16, wmma::col_major> fb;
                    wmma::load_matrix_sync(fb, Wh + (size_t)(n0 + (f0 + j) * 16) * K + k0 + kk, K);
                    wmma::mma_sync(acc[j], fa, fb, acc[j]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int j = 0; j < NF; ++j)
        if (f0 + j < n_frag) wmma::store_matrix_sync(&Cs[wrow][(f0 + j) * 16], acc[j], HW_TN + 8, wmma::mem_row_major);
    __syncthreads();
    for (int e = tid; e < (FEW ? 16 : HW_TM) * (HW_TN / 2); e += 128) {
        int r = e / (HW_TN / 2), c = (e % (HW_TN / 2)) * 2;
        int m = m0 + r, n = n0 + c;
        if (m >= M || n >= N) continue;
        float x = Cs[r][c], y = Cs[r][c + 1];
        if (gate) {
            if (gate_head) {
                float gv = ma_sigmoid(gate[(size_t)m * gate_stride + h]);
                x *= gv;
                y *= gv;
            } else {
                const float* g = gate + (size_t)m * gate_stride + (size_t)h * N + n;
                x *= ma_sigmoid(g[0]);
                y *= ma_sigmoid(g[1]);
            }
        }
        __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
        *reinterpret_cast<__nv_bfloat162*>(out + (size_t)m * out_stride + (size_t)h * out_head + n) = v;
    }
}

extern "C" int ce_head_matmul(const void* in, int in_stride, int in_head, const void* W, void* out, int out_stride, int out_head,
                              const float* gate, int gate_stride, int gate_head, int dtype, int M, int H, int N, int K, cudaStream_t stream) {
    if (M == 0 || H == 0 || N == 0) return CE_OK;
    if (!in || !W || !out || K <= 0) return ce_fail(CE_ERR_ARG, "ce_head_matmul: null pointer or K=%d", K);
    if (H > 65535 || (M + HM_TM - 1) / HM_TM > 65535) return ce_fail(CE_ERR_SIZE, "ce_head_matmul: %d heads, %d tokens", H, M);
    if (dtype == CE_BF16 && N % 16 == 0 && K % 16 == 0 && in_stride % 16 == 0 && in_head % 16 == 0 && out_stride % 2 == 0 &&
        out_head % 2 == 0 && (((uintptr_t)in | (uintptr_t)W) & 31) == 0 && (((uintptr_t)out) & 3) == 0) {
        dim3 grid((N + HW_TN - 1) / HW_TN, (M + HW_TM - 1) / HW_TM, H);
        ce_note("head_matmul_wmma_kernel");
        if (M <= 16)
            ce_launch(head_matmul_wmma_kernel<true>, grid, 128, 0, stream, (const __nv_bfloat16*)in, in_stride, in_head, (const __nv_bfloat16*)W,
                      (__nv_bfloat16*)out, out_stride, out_head, gate, gate_stride, gate_head, M, N, K);
        else
            ce_launch(head_matmul_wmma_kernel<false>, grid, 128, 0, stream, (const __nv_bfloat16*)in, in_stride, in_head, (const __nv_bfloat16*)W,
                      (__nv_bfloat16*)out, out_stride, out_head, gate, gate_stride, gate_head, M, N, K);
        return ce_check_launch("ce_head_matmul");
    }
    dim3 grid((N + HM_TN - 1) / HM_TN, (M + HM_TM - 1) / HM_TM, H);
    ce_note("head_matmul_kernel");
    if (dtype == CE_F32) ce_launch(head_matmul_kernel<float>, grid, 256, 0, stream, (const float*)in, in_stride, in_head, (const float*)W, (float*)out, out_stride, out_head, gate, gate_stride, gate_head, M, N, K);
    else if (dtype == CE_BF16) ce_launch(head_matmul_kernel<__nv_bfloat16>, grid, 256, 0, stream, (const __nv_bfloat16*)in, in_stride, in_head, (const __nv_bfloat16*)W, (__nv_bfloat16*)out, out_stride, out_head, gate, gate_stride, gate_head, M, N, K);
    else return ce_fail(CE_ERR_ARG, "ce_head_matmul: unknown dtype %d", dtype);
    return ce_check_launch("ce_head_matmul");
}

// ---------------------------------------------------------------------------------------------
// The attention.  One block per (token, query head).  The query at position p sees the keys j <= p with
// p - j < window or j < keep_first (window 0: all of them).  Keys are taken in runs of 128 positions that start at
// multiples of 128 (runs without a visible key are passed over), with an online softmax across the runs, so the
// order of every sum depends on p only: not on how the tokens were cut into steps, not on the batch, not on pages.
// ---------------------------------------------------------------------------------------------
#define MA_THREADS 128
#define MA_MAX_ACC 8             // dv <= MA_THREADS * MA_MAX_ACC

struct MaskedAttnArgs {
    const void* q;               // [T, q_stride]; head h at column h * q_head
    const void* k_pool;          // [num_pages, nkv, page_size, ldk]
    const void* v_pool;          // [num_pages, nkv, page_size, ldv]
    const void* gate;            // [T, gate_stride], element (h, j) at column h * dv + j; null: no gate
    void* out;                   // [T, nh * dv]
    const int* positions;
    const int* seq_of_token;
    const int* seq_slot;
    const int* block_table;
    int* status;
    const float* sinks;          // [nh] or null: exp(sinks[h]) joins the softmax's denominator, with no key and no value
    int T, nh, nkv, d, dv, q_stride, q_head, ldk, ldv, gate_stride, page_size, max_pages, num_pages, window, keep_first;
    float scale, softcap;
    float out_scale;             // the stored result is multiplied by this (the mixer's weight in a sum of mixers)
};

template <typename T>
__global__ void masked_attention_kernel(MaskedAttnArgs a) {
    ce_pdl_begin();
    extern __shared__ __align__(16) unsigned char ma_smem[];
    long long* vrow = (long long*)ma_smem;            // MA_THREADS
    float* probs = (float*)(vrow + MA_THREADS);       // MA_THREADS
    float* scratch = probs + MA_THREADS;              // 32
    float* qs = scratch + 32;                         // d

    int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x, d = a.d, dv = a.dv;
    int kvh = h / (a.nh / a.nkv);
    int p = a.positions[t];
    int slot = a.seq_slot[a.seq_of_token[t]];
    const int* table = a.block_table + (size_t)slot * a.max_pages;
    const T* qrow = (const T*)a.q + (size_t)t * a.q_stride + (size_t)h * a.q_head;
    for (int j = tid; j < d; j += MA_THREADS) qs[j] = CeType<T>::load(qrow + j);
    __syncthreads();

    int lo = a.window > 0 ? max(0, p - a.window + 1) : 0;
    int keep = a.window > 0 ? a.keep_first : 0;
    float inv_cap = a.softcap > 0.f ? 1.0f / a.softcap : 0.f;
    float m_run = -INFINITY, l_run = 0.f;
    float acc[MA_MAX_ACC];
#pragma unroll
    for (int i = 0; i < MA_MAX_ACC; ++i) acc[i] = 0.f;

    for (int k0 = 0; k0 <= p; k0 += MA_THREADS) {
        if (k0 + MA_THREADS <= lo && k0 >= keep) continue;         // no key of this run is visible
        int key = k0 + tid;
        bool valid = key <= p && (key >= lo || key < keep);
        float s = -INFINITY;
        long long row = -1;
        if (valid) {
            int page = table[key / a.page_size];
            if (page < 0 || page >= a.num_pages) {
                atomicExch(a.status, 4);
                valid = false;
            } else {
                row = ((long long)page * a.nkv + kvh) * a.page_size + key % a.page_size;
                const T* kr = (const T*)a.k_pool + row * a.ldk;
                float dot = 0.f;
                for (int j = 0; j < d; ++j) dot = fmaf(qs[j], CeType<T>::load(kr + j), dot);
                s = dot * a.scale;
                if (a.softcap > 0.f) s = a.softcap * tanhf(s * inv_cap);
            }
        }
        float m_chunk = ce_block_max(s, scratch);
        float m_new = fmaxf(m_run, m_chunk);
        float pr = valid ? expf(s - m_new) : 0.f;
        __syncthreads();                 // everyone has read scratch before it is reused
        probs[tid] = pr;
        vrow[tid] = row;
        float l_chunk = ce_block_sum(pr, scratch);   // syncs: probs/vrow visible afterwards
        float alpha = m_run == -INFINITY ? 0.f : expf(m_run - m_new);
        l_run = l_run * alpha + l_chunk;
        m_run = m_new;
        int n = min(MA_THREADS, p - k0 + 1);
#pragma unroll
        for (int i = 0; i < MA_MAX_ACC; ++i) {
            int j = tid + i * MA_THREADS;
            if (j < dv) {
                float o = acc[i] * alpha;
                for (int kk = 0; kk < n; ++kk) {
                    long long r = vrow[kk];
                    if (r >= 0) o = fmaf(probs[kk], CeType<T>::load((const T*)a.v_pool + r * a.ldv + j), o);
                }
                acc[i] = o;
            }
        }
        __syncthreads();
    }
    T* orow = (T*)a.out + ((size_t)t * a.nh + h) * dv;
    float shrink = 1.0f;
    if (a.sinks) {                       // the sink: one more term of the denominator, taken as it is (no scale, no cap)
        float sk = a.sinks[h], m_all = fmaxf(m_run, sk);
        shrink = m_run == -INFINITY ? 0.f : expf(m_run - m_all);
        l_run = l_run * shrink + expf(sk - m_all);
    }
    float inv = l_run > 0.f ? shrink / l_run : 0.f;
#pragma unroll
    for (int i = 0; i < MA_MAX_ACC; ++i) {
        int j = tid + i * MA_THREADS;
        if (j < dv) {
            float o = acc[i] * inv * a.out_scale;
            if (a.gate) o *= ma_sigmoid(CeType<T>::load((const T*)a.gate + (size_t)t * a.gate_stride + (size_t)h * dv + j));
            CeType<T>::store(orow + j, o);
        }
    }
}

extern "C" int ce_masked_attention(const void* q, const void* k_pool, const void* v_pool, const void* gate, void* out, int dtype,
                                   const int* positions, const int* seq_of_token, const int* seq_slot, const int* block_table,
                                   int* status, int T, int nh, int nkv, int d, int dv, int q_stride, int q_head, int ldk, int ldv,
                                   int gate_stride, int page_size, int max_pages, int num_pages, int window, int keep_first,
                                   float scale, float softcap, const float* sinks, float out_scale, cudaStream_t stream) {
    if (T == 0) return CE_OK;
    if (!q || !k_pool || !v_pool || !out || !positions || !seq_of_token || !seq_slot || !block_table || !status)
        return ce_fail(CE_ERR_ARG, "ce_masked_attention: null pointer");
    if (d <= 0 || dv <= 0 || dv > MA_THREADS * MA_MAX_ACC || d > 8192)
        return ce_fail(CE_ERR_SIZE, "ce_masked_attention: head sizes %d / %d", d, dv);
    if (nkv <= 0 || nh % nkv != 0) return ce_fail(CE_ERR_SIZE, "ce_masked_attention: %d heads are not a multiple of %d kv heads", nh, nkv);
    if (ldk < d || ldv < dv || nh > 65535) return ce_fail(CE_ERR_SIZE, "ce_masked_attention: a pool's rows are shorter than a head");
    MaskedAttnArgs a{q, k_pool, v_pool, gate, out, positions, seq_of_token, seq_slot, block_table, status, sinks, T, nh, nkv, d, dv,
                     q_stride, q_head, ldk, ldv, gate_stride, page_size, max_pages, num_pages, window, keep_first, scale, softcap,
                     out_scale};
    size_t smem = (d + MA_THREADS + 32) * sizeof(float) + MA_THREADS * sizeof(long long);
    dim3 grid(T, nh);
    ce_note("masked_attention_kernel");
    if (dtype == CE_F32) ce_launch(masked_attention_kernel<float>, grid, MA_THREADS, smem, stream, a);
    else if (dtype == CE_BF16) ce_launch(masked_attention_kernel<__nv_bfloat16>, grid, MA_THREADS, smem, stream, a);
    else return ce_fail(CE_ERR_ARG, "ce_masked_attention: unknown dtype %d", dtype);
    return ce_check_launch("ce_masked_attention");
}
