// Layer norm with weight and bias, an RMS norm that adds into the residual stream, the tanh cap of a row of
// numbers, a copy of a run of float32 columns into the activation dtype, and the gate of a per-token side input.
//
// All arithmetic is float32; a result is rounded once, at the store.  Sums over a row are taken by one block in
// an order that depends on the row's width only.
#include "common.cuh"

// ---------------------------------------------------------------------------------------------
// y = (x - mean) / sqrt(var + eps) * w + b, var the mean of the squared deviations (two passes over the row,
// which is kept in registers when it fits).  rows: optional gather of the rows to normalise.
// ---------------------------------------------------------------------------------------------
#define LN_MAX_PER_THREAD 16

template <typename T>
__global__ void layernorm_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                 T* __restrict__ out, const int* __restrict__ rows, int H, float eps) {
    ce_pdl_begin();
    __shared__ float scratch[32];
    int r = blockIdx.x;
    const float* xr = x + (size_t)(rows ? rows[r] : r) * H;
    float v[LN_MAX_PER_THREAD];
    float s = 0.f;
    int n = 0;
    for (int j = threadIdx.x; j < H; j += blockDim.x, ++n) {
        float e = xr[j];
        if (n < LN_MAX_PER_THREAD) v[n] = e;
        s += e;
    }
    float mean = ce_block_sum(s, scratch) / (float)H;
    float q = 0.f;
    n = 0;
    for (int j = threadIdx.x; j < H; j += blockDim.x, ++n) {
        float e = (n < LN_MAX_PER_THREAD ? v[n] : xr[j]) - mean;
        q = fmaf(e, e, q);
    }
    float inv = 1.0f / sqrtf(ce_block_sum(q, scratch) / (float)H + eps);
    n = 0;
    for (int j = threadIdx.x; j < H; j += blockDim.x, ++n) {
        float e = (n < LN_MAX_PER_THREAD ? v[n] : xr[j]) - mean;
        CeType<T>::store(out + (size_t)r * H + j, e * inv * w[j] + b[j]);
    }
}

// The same with float4 loads for widths in multiples of 4 up to 4 * 1024 * LNV_MAX: a thread keeps its float4s in registers.
#define LNV_MAX 4
template <typename T>
__global__ void layernorm_vec_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ b,
                                     T* __restrict__ out, const int* __restrict__ rows, int H, float eps) {
    ce_pdl_begin();
    __shared__ float scratch[32];
    int r = blockIdx.x, H4 = H >> 2;
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)(rows ? rows[r] : r) * H);
    float4 v[LNV_MAX];
    float s = 0.f;
#pragma unroll
    for (int n = 0; n < LNV_MAX; ++n) {
        int j = threadIdx.x + n * blockDim.x;
        v[n] = j < H4 ? xr[j] : make_float4(0.f, 0.f, 0.f, 0.f);
        s += (v[n].x + v[n].y) + (v[n].z + v[n].w);
    }
    float mean = ce_block_sum(s, scratch) / (float)H;
    float q = 0.f;
#pragma unroll
    for (int n = 0; n < LNV_MAX; ++n) {
        int j = threadIdx.x + n * blockDim.x;
        if (j < H4) {
            v[n].x -= mean; v[n].y -= mean; v[n].z -= mean; v[n].w -= mean;
            q += (v[n].x * v[n].x + v[n].y * v[n].y) + (v[n].z * v[n].z + v[n].w * v[n].w);
        }
    }
    float inv = 1.0f / sqrtf(ce_block_sum(q, scratch) / (float)H + eps);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    const float4* b4 = reinterpret_cast<const float4*>(b);
#pragma unroll
    for (int n = 0; n < LNV_MAX; ++n) {
        int j = threadIdx.x + n * blockDim.x;
        if (j < H4) {
            float4 ww = w4[j], bb = b4[j];
            T* o = out + (size_t)r * H + 4 * j;
            CeType<T>::store(o, v[n].x * inv * ww.x + bb.x); CeType<T>::store(o + 1, v[n].y * inv * ww.y + bb.y);
            CeType<T>::store(o + 2, v[n].z * inv * ww.z + bb.z); CeType<T>::store(o + 3, v[n].w * inv * ww.w + bb.w);
        }
    }
}

extern "C" int ce_layernorm(const float* x, const float* w, const float* b, void* out, int out_dtype, const int* rows,
                            int R, int H, float eps, cudaStream_t stream) {
    if (R == 0) return CE_OK;
    if (!x || !w || !b || !out) return ce_fail(CE_ERR_ARG, "ce_layernorm: null pointer");
    if (H <= 0) return ce_fail(CE_ERR_SIZE, "ce_layernorm: width %d", H);
    if (out_dtype != CE_F32 && out_dtype != CE_BF16) return ce_fail(CE_ERR_ARG, "ce_layernorm: unknown dtype %d", out_dtype);
    if (H % 4 == 0 && H >= 256 && ((((uintptr_t)x | (uintptr_t)w | (uintptr_t)b) & 15) == 0)) {
        int H4 = H / 4, vt = H4 >= 2048 ? 1024 : H4 >= 512 ? 512 : H4 >= 256 ? 256 : 128;
        if (H4 <= vt * LNV_MAX) {
            ce_note("layernorm_vec_kernel");
            if (out_dtype == CE_F32) ce_launch(layernorm_vec_kernel<float>, R, vt, 0, stream, x, w, b, (float*)out, rows, H, eps);
            else ce_launch(layernorm_vec_kernel<__nv_bfloat16>, R, vt, 0, stream, x, w, b, (__nv_bfloat16*)out, rows, H, eps);
            return ce_check_launch("ce_layernorm");
        }
    }
    int threads = H >= 4096 ? 512 : H >= 1024 ? 256 : 128;
    ce_note("layernorm_kernel");
    if (out_dtype == CE_F32) ce_launch(layernorm_kernel<float>, R, threads, 0, stream, x, w, b, (float*)out, rows, H, eps);
    else if (out_dtype == CE_BF16) ce_launch(layernorm_kernel<__nv_bfloat16>, R, threads, 0, stream, x, w, b, (__nv_bfloat16*)out, rows, H, eps);
    else return ce_fail(CE_ERR_ARG, "ce_layernorm: unknown dtype %d", out_dtype);
    return ce_check_launch("ce_layernorm");
}

// ---------------------------------------------------------------------------------------------
// x[t] += y[t] / sqrt(mean(y[t]^2) + eps) * w      (y float32, x the float32 residual stream)
// ---------------------------------------------------------------------------------------------
__global__ void rmsnorm_add_kernel(const float* __restrict__ y, const float* __restrict__ w, float* __restrict__ x,
                                   __nv_bfloat16* __restrict__ xb, int H, float eps) {
    ce_pdl_begin();
    __shared__ float scratch[32];
    int t = blockIdx.x;
    const float* yr = y + (size_t)t * H;
    float q = 0.f;
    for (int j = threadIdx.x; j < H; j += blockDim.x) q = fmaf(yr[j], yr[j], q);
    float inv = 1.0f / sqrtf(ce_block_sum(q, scratch) / (float)H + eps);
    for (int j = threadIdx.x; j < H; j += blockDim.x) {
        float v = x[(size_t)t * H + j] + yr[j] * inv * w[j];
        x[(size_t)t * H + j] = v;
        if (xb) xb[(size_t)t * H + j] = __float2bfloat16_rn(v);
    }
}

// The same with float4 loads, y kept in registers between the two passes (widths in multiples of 4 up to 4 * threads * LNV_MAX)
__global__ void rmsnorm_add_vec_kernel(const float* __restrict__ y, const float* __restrict__ w, float* __restrict__ x,
                                       __nv_bfloat16* __restrict__ xb, int H, float eps) {
    ce_pdl_begin();
    __shared__ float scratch[32];
    int t = blockIdx.x, H4 = H >> 2;
    const float4* yr = reinterpret_cast<const float4*>(y + (size_t)t * H);
    float4 v[LNV_MAX];
    float q = 0.f;
#pragma unroll
    for (int n = 0; n < LNV_MAX; ++n) {
        int j = threadIdx.x + n * blockDim.x;
        v[n] = j < H4 ? yr[j] : make_float4(0.f, 0.f, 0.f, 0.f);
        q += (v[n].x * v[n].x + v[n].y * v[n].y) + (v[n].z * v[n].z + v[n].w * v[n].w);
    }
    float inv = 1.0f / sqrtf(ce_block_sum(q, scratch) / (float)H + eps);
    float4* xr = reinterpret_cast<float4*>(x + (size_t)t * H);
    const float4* w4 = reinterpret_cast<const float4*>(w);
#pragma unroll
    for (int n = 0; n < LNV_MAX; ++n) {
        int j = threadIdx.x + n * blockDim.x;
        if (j < H4) {
            float4 xv = xr[j], ww = w4[j];
            xv.x += v[n].x * inv * ww.x; xv.y += v[n].y * inv * ww.y; xv.z += v[n].z * inv * ww.z; xv.w += v[n].w * inv * ww.w;
            xr[j] = xv;
            if (xb) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(xv.x, xv.y), hi = __floats2bfloat162_rn(xv.z, xv.w);
                uint2 packed = make_uint2(*reinterpret_cast<unsigned*>(&lo), *reinterpret_cast<unsigned*>(&hi));
                reinterpret_cast<uint2*>(xb + (size_t)t * H)[j] = packed;
            }
        }
    }
}

// xb (or null): receives the new x rounded to bfloat16, what a sublayer that reads the residual itself takes as its input
extern "C" int ce_rmsnorm_add(const float* y, const float* w, float* x, void* xb, int T, int H, float eps, cudaStream_t stream) {
    if (T == 0) return CE_OK;
    if (!y || !w || !x) return ce_fail(CE_ERR_ARG, "ce_rmsnorm_add: null pointer");
    if (H % 4 == 0 && H >= 256 && ((((uintptr_t)x | (uintptr_t)w | (uintptr_t)y) & 15) == 0) && (((uintptr_t)xb) & 7) == 0) {
        int H4 = H / 4, vt = H4 >= 2048 ? 1024 : H4 >= 512 ? 512 : H4 >= 256 ? 256 : 128;
        if (H4 <= vt * LNV_MAX) {
            ce_note("rmsnorm_add_vec_kernel");
            ce_launch(rmsnorm_add_vec_kernel, T, vt, 0, stream, y, w, x, (__nv_bfloat16*)xb, H, eps);
            return ce_check_launch("ce_rmsnorm_add");
        }
    }
    ce_note("rmsnorm_add_kernel");
    ce_launch(rmsnorm_add_kernel, T, H >= 4096 ? 512 : H >= 1024 ? 256 : 128, 0, stream, y, w, x, (__nv_bfloat16*)xb, H, eps);
    return ce_check_launch("ce_rmsnorm_add");
}

// ---------------------------------------------------------------------------------------------
// x <- cap * tanh(x / cap), in place (the cap of the logits)
// ---------------------------------------------------------------------------------------------
__global__ void tanh_cap_kernel(float* __restrict__ x, size_t n, float cap, float inv_cap) {
    ce_pdl_begin();
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < n; e += stride) x[e] = cap * tanhf(x[e] * inv_cap);
}

extern "C" int ce_tanh_cap(float* x, long long n, float cap, cudaStream_t stream) {
    if (n == 0) return CE_OK;
    if (!x || !(cap > 0.f)) return ce_fail(CE_ERR_ARG, "ce_tanh_cap: null pointer or a cap that is not positive");
    long long blocks = (n + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    ce_note("tanh_cap_kernel");
    ce_launch(tanh_cap_kernel, (int)blocks, 256, 0, stream, x, (size_t)n, cap, 1.0f / cap);
    return ce_check_launch("ce_tanh_cap");
}

// ---------------------------------------------------------------------------------------------
// out[t, l] = src[t, off + l] for l < L, rounded to the activation dtype: the input of a narrow second product
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void copy_cols_kernel(const float* __restrict__ src, T* __restrict__ out, int ld, int off, int L, size_t total) {
    ce_pdl_begin();
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        size_t t = e / L;
        int l = (int)(e % L);
        CeType<T>::store(out + e, src[t * ld + off + l]);
    }
}

extern "C" int ce_copy_cols(const float* src, void* out, int out_dtype, int T, int ld, int off, int L, cudaStream_t stream) {
    if (T == 0 || L == 0) return CE_OK;
    if (!src || !out) return ce_fail(CE_ERR_ARG, "ce_copy_cols: null pointer");
    size_t total = (size_t)T * L;
    size_t want = (total + 255) / 256;
    int blocks = (int)(want < (size_t)148 * 8 ? want : (size_t)148 * 8);
    ce_note("copy_cols_kernel");
    if (out_dtype == CE_F32) ce_launch(copy_cols_kernel<float>, blocks, 256, 0, stream, src, (float*)out, ld, off, L, total);
    else if (out_dtype == CE_BF16) ce_launch(copy_cols_kernel<__nv_bfloat16>, blocks, 256, 0, stream, src, (__nv_bfloat16*)out, ld, off, L, total);
    else return ce_fail(CE_ERR_ARG, "ce_copy_cols: unknown dtype %d", out_dtype);
    return ce_check_launch("ce_copy_cols");
}

// ---------------------------------------------------------------------------------------------
// Side input of a layer: g[t, j] = gelu_tanh(z[t, j]) * table[token[t], off + j]
// gelu_tanh(z) = 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3)))
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void side_gate_kernel(const float* __restrict__ z, const T* __restrict__ table, const int* __restrict__ tokens,
                                 T* __restrict__ out, int D, int ld, int off, int V, int* __restrict__ status, size_t total) {
    ce_pdl_begin();
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += stride) {
        size_t t = e / D;
        int j = (int)(e % D);
        int tok = tokens[t];
        float g = 0.f;
        if (tok < 0 || tok >= V) atomicExch(status, 1);
        else {
            float v = z[e];
            float inner = 0.79788456080286536f * (v + 0.044715f * v * v * v);
            g = 0.5f * v * (1.0f + tanhf(inner)) * CeType<T>::load(table + (size_t)tok * ld + off + j);
        }
        CeType<T>::store(out + e, g);
    }
}

extern "C" int ce_side_gate(const float* z, const void* table, int dtype, const int* tokens, void* out, int T, int D, int ld,
                            int off, int V, int* status, cudaStream_t stream) {
    if (T == 0 || D == 0) return CE_OK;
    if (!z || !table || !tokens || !out || !status) return ce_fail(CE_ERR_ARG, "ce_side_gate: null pointer");
    if (off < 0 || off + D > ld) return ce_fail(CE_ERR_SIZE, "ce_side_gate: columns %d..%d of a table %d wide", off, off + D, ld);
    size_t total = (size_t)T * D;
    size_t want = (total + 255) / 256;
    int blocks = (int)(want < (size_t)148 * 8 ? want : (size_t)148 * 8);
    ce_note("side_gate_kernel");
    if (dtype == CE_F32) ce_launch(side_gate_kernel<float>, blocks, 256, 0, stream, z, (const float*)table, tokens, (float*)out, D, ld, off, V, status, total);
    else if (dtype == CE_BF16) ce_launch(side_gate_kernel<__nv_bfloat16>, blocks, 256, 0, stream, z, (const __nv_bfloat16*)table, tokens, (__nv_bfloat16*)out, D, ld, off, V, status, total);
    else return ce_fail(CE_ERR_ARG, "ce_side_gate: unknown dtype %d", dtype);
    return ce_check_launch("ce_side_gate");
}
