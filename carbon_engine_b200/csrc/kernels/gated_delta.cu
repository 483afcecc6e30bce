// Recurrent mixers whose per-head state S [d, dv] (key channel x value channel, float32) is carried from token to token.
// The gated delta rule (rule 0):
//
//     S <- diag(g_t) S;    u_t = beta_t (v_t - S^T k_t);    S <- S + k_t u_t^T;    o_t = S^T q_t
//
// (the read-out sees the token's own write), and the plain decaying sum of outer products, "retention" (rule 1): the same
// with u_t = v_t.  The options are arguments, so that the family's mixers share the four kernels:
//   decay     0: one per head and key channel from logits [T, H d];  1: one per head from logits [T, H];
//             2: a constant per head (``a_log`` then holds the constants themselves, nothing is learned per token)
//   operands  0: short convolution, SiLU, unit q and k (below);  1: no convolution: q and k are rotated over their first
//             ``rd`` elements by the token's position (element i with i + rd/2), k times d^-1/2, v as projected
//   gate      0: sigmoid, 1: SiLU of the gate logits;  the weight after the root mean square may be absent;  the stored
//             result is multiplied by ``out_scale`` (the mixer's weight in a sum of mixers)
// With the convolution:  q, k and v come out of a short causal convolution over time per channel
// followed by SiLU; q and k are then brought to unit length per head (q also times d^-1/2); the decay is
// g_t = exp(-exp(A_h) softplus(z_t + bias)) with z_t the token's decay logits (a product of their own);
// beta_t = sigmoid of a projection, one per head.  Query/key head of value head h: h / (H / G).  Afterwards every
// head's o_t is divided by its root mean square, multiplied by a weight of size dv and by sigmoid(gate logits).
//
// Four kernels, all float32:
//   prepare     every token on its own: convolution (the inputs before a portion's first token come from the
//               request's kept rows), SiLU, unit q and k, decay, beta                       (parallel over tokens)
//   keep        the last taps-1 convolution inputs of every sequence go to its kept rows   (parallel over channels)
//   walk        one block per (head, sequence, slice of value channels) walks the sequence's tokens of this step
//               in order, from the state its slot holds, and stores the state back           (the recurrence)
//   finish      every (token, head): root mean square, weight, gate, one rounding at the store   (parallel)
//
// The columns of S (value channels) are independent of one another, so a slice of GD_COLS columns is a block of
// its own and a column lives in the registers of 16 neighbouring lanes (32 for more than 128 key channels, so that a
// thread holds at most 8 rows); the two sums over rows a token needs
// are a per-thread run plus a butterfly over those lanes: the order of every sum depends on d only, never on
// how the tokens were cut into steps or on the batch.  The decay is applied as S^T (k * g) for the dot product and
// as g * S + k u for the new state, which is the same arithmetic as decaying first, term by term.
#include "common.cuh"

#define GD_COLS 8                // value channels a block walks
#define GD_TILE 16               // tokens a buffer holds (at most the lanes of a column: lane g stores token g's output)

__device__ __forceinline__ float gd_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float gd_softplus(float z) { return z > 20.f ? z : log1pf(expf(z)); }

struct GatedDeltaArgs {
    const float* proj;           // [T, ld]: the convolution's inputs q | k | v from off_conv (C = 2 G d + H dv columns), beta logits at off_b
    const float* dec;            // decay logits before the bias, rows of ld_dec: [T, H*d] (decay 0) or [T, H] (decay 1); unused with decay 2
    const float* gz;             // [T, H*dv] gate logits, rows of ld_gz
    const float* taps;           // [C, K] convolution weights, the last column the current token's (operands 0)
    const float* a_log;          // [H]; with decay 2 the heads' constant decays themselves
    const float* dt_bias;        // [H*d] (decay 0) or [H] (decay 1)
    const float* norm_w;         // [dv] or null
    float* prep;                 // [T, P]: q (G d) | k (G d) | v (H dv) | decay (H d) | beta (H); P padded to a multiple of 4
    float* raw;                  // [T, H*dv] o_t before the norm
    float* state;                // [slots, H, d, dv]
    float* kept;                 // [slots, K-1, C] the convolution inputs of the last K-1 tokens, oldest first
    void* out;                   // [T, H*dv]
    const int* seq_of_token;
    const int* seq_slot;
    const int* q_start;
    int ld, off_conv, off_b, H, G, d, dv, K, P;
    float eps;
    int ld_dec, ld_gz;
    int decay_mode, operands, rule, gate_act;
    float out_scale;
    const float* cos_table;      // [max_pos, rd/2] (operands 1; null or rd 0: no rotation)
    const float* sin_table;
    const int* positions;        // [T]
    int* status;
    int rd, max_pos;
};

// A token's heads of q, of k (unit vectors) and of v are dealt to the warps of gridDim.y blocks in turn (one block a token
// in a long step; in a step of few tokens a block per handful of heads, so that the step is not eight blocks' work); the
// decays and beta are dealt the same way.
__global__ void gated_delta_prepare_kernel(GatedDeltaArgs a) {
    ce_pdl_begin();
    int t = blockIdx.x, lane = threadIdx.x & 31, nwarp = (blockDim.x >> 5) * gridDim.y;
    int warp = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int d = a.d, dv = a.dv, G = a.G, H = a.H, K = a.K;
    int C = 2 * G * d + H * dv;
    int b = a.seq_of_token[t];
    int rel = t - a.q_start[b];                     // tokens of the same sequence before this one in the step
    const float* kept = a.kept + (size_t)a.seq_slot[b] * (K - 1) * C;
    float* pw = a.prep + (size_t)t * a.P;
    float q_scale = rsqrtf((float)d);
    int nthr = blockDim.x * gridDim.y, thr = blockIdx.y * blockDim.x + threadIdx.x;
    if (a.operands == 1) {
        // no convolution: q and k rotated by the position, k scaled, v as it is
        const float* row = a.proj + (size_t)t * a.ld + a.off_conv;
        int half = a.rd / 2;
        bool rotate = a.cos_table != nullptr && half > 0;
        int pos = rotate ? a.positions[t] : 0;
        if (rotate && (pos < 0 || pos >= a.max_pos)) {
            if (thr == 0) atomicExch(a.status, 3);
            rotate = false;
        }
        const float* cs = rotate ? a.cos_table + (size_t)pos * half : nullptr;
        const float* sn = rotate ? a.sin_table + (size_t)pos * half : nullptr;
        int nqk = 2 * G * d;
        for (int e = thr; e < nqk; e += nthr) {
            int i = e % d, base = e - i;
            float x = row[e];
            if (rotate && i < half) x = x * cs[i] - row[base + i + half] * sn[i];
            else if (rotate && i < a.rd) x = x * cs[i - half] + row[base + i - half] * sn[i - half];
            pw[e] = e >= G * d ? x * q_scale : x;
        }
        for (int e = thr; e < H * dv; e += nthr) pw[nqk + e] = row[nqk + e];
        float* decay1 = pw + C;
        for (int e = thr; e < H * d; e += nthr) decay1[e] = a.a_log[e / d];
        for (int h = thr; h < H; h += nthr) decay1[H * d + h] = 1.0f;
        return;
    }
    // convolution + SiLU of channel c at this token
    auto conv = [&](int c) -> float {
        float y = 0.f;
        for (int j = 0; j < K; ++j) {
            int back = K - 1 - j;                   // how many tokens before this one
            float x = back <= rel ? a.proj[(size_t)(t - back) * a.ld + a.off_conv + c]
                                  : kept[(size_t)(K - 1 + rel - back) * C + c];
            y = fmaf(a.taps[(size_t)c * K + j], x, y);
        }
        return y / (1.0f + expf(-y));
    };
    int heads = 2 * G + H;
    for (int hh = warp; hh < heads; hh += nwarp) {
        bool is_v = hh >= 2 * G;
        int size = is_v ? dv : d;
        int c0 = is_v ? 2 * G * d + (hh - 2 * G) * dv : hh * d;
        if (is_v) {
            for (int c = lane; c < size; c += 32) pw[c0 + c] = conv(c0 + c);
            continue;
        }
        float ss = 0.f;
        for (int c = lane; c < size; c += 32) {
            float y = conv(c0 + c);
            pw[c0 + c] = y;
            ss = fmaf(y, y, ss);
        }
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        float inv = 1.0f / sqrtf(ss + 1e-6f) * (hh < G ? q_scale : 1.0f);
        __syncwarp();
        for (int c = lane; c < size; c += 32) pw[c0 + c] *= inv;
    }
    float* decay = pw + C;
    if (a.decay_mode == 0) {
        for (int e = thr; e < H * d; e += nthr)
            decay[e] = expf(-expf(a.a_log[e / d]) * gd_softplus(a.dec[(size_t)t * a.ld_dec + e] + a.dt_bias[e]));
    } else if (a.decay_mode == 1) {          // one decay per head, written to all its key channels
        for (int e = thr; e < H * d; e += nthr) {
            int h = e / d;
            decay[e] = expf(-expf(a.a_log[h]) * gd_softplus(a.dec[(size_t)t * a.ld_dec + h] + a.dt_bias[h]));
        }
    } else {
        for (int e = thr; e < H * d; e += nthr) decay[e] = a.a_log[e / d];
    }
    for (int h = thr; h < H; h += nthr) decay[H * d + h] = gd_sigmoid(a.proj[(size_t)t * a.ld + a.off_b + h]);
}

// One thread per (sequence, channel): the kept rows move up by the portion's length and take the portion's last inputs.
__global__ void gated_delta_keep_kernel(GatedDeltaArgs a, int B) {
    ce_pdl_begin();
    int C = 2 * a.G * a.d + a.H * a.dv, K = a.K;
    size_t total = (size_t)B * C;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
        int b = (int)(e / C), c = (int)(e % C);
        int t0 = a.q_start[b], n = a.q_start[b + 1] - t0;
        float* kept = a.kept + (size_t)a.seq_slot[b] * (K - 1) * C + c;
        for (int j = 0; j < K - 1; ++j) {           // ascending: row j + n is read before it is overwritten
            int rel = n - (K - 1) + j;
            kept[(size_t)j * C] = rel >= 0 ? a.proj[(size_t)(t0 + rel) * a.ld + a.off_conv + c] : kept[(size_t)(j + n) * C];
        }
    }
}

__device__ __forceinline__ void gd_cp4(float* dst, const float* src) {
    unsigned s = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(src));
}
__device__ __forceinline__ void gd_cp16(float* dst, const float* src) {
    unsigned s = (unsigned)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(src));
}

// Copies of one tile of tokens into a buffer: three vectors of d per token (decay, key, query; rows padded to DP floats),
// BC values (the block's value channels) and beta.
template <int DP, bool VEC, int BC>
__device__ __forceinline__ void gd_stage(const GatedDeltaArgs& a, float* buf, int t0, int n_tok, int h, int col0, int ncols) {
    int d = a.d, G = a.G, H = a.H, tid = threadIdx.x, nthr = blockDim.x;
    int g = h / (H / G);
    int C = 2 * G * d + H * a.dv;
    int offs[3] = {C + h * d, G * d + g * d, g * d};          // decay, key, query within a prep row
    float* vbuf = buf + 3 * GD_TILE * DP;
    if (VEC) {
        constexpr int DP4 = DP / 4;
        for (int e = tid; e < 3 * GD_TILE * DP4; e += nthr) {
            int which = e / (GD_TILE * DP4), tok = (e / DP4) % GD_TILE, c = (e % DP4) * 4;
            if (tok < n_tok && c < d) gd_cp16(buf + (which * GD_TILE + tok) * DP + c, a.prep + (size_t)(t0 + tok) * a.P + offs[which] + c);
        }
    } else {
        for (int e = tid; e < 3 * GD_TILE * DP; e += nthr) {
            int which = e / (GD_TILE * DP), tok = (e / DP) % GD_TILE, c = e % DP;
            if (tok < n_tok && c < d) gd_cp4(buf + (which * GD_TILE + tok) * DP + c, a.prep + (size_t)(t0 + tok) * a.P + offs[which] + c);
        }
    }
    for (int e = tid; e < GD_TILE * (BC + 1); e += nthr) {
        int tok = e / (BC + 1), c = e % (BC + 1);
        if (tok >= n_tok) continue;
        const float* row = a.prep + (size_t)(t0 + tok) * a.P;
        if (c < ncols) gd_cp4(vbuf + tok * (BC + 1) + c, row + 2 * G * d + h * a.dv + col0 + c);
        else if (c == BC) gd_cp4(vbuf + tok * (BC + 1) + c, row + C + H * d + h);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
}

// A thread's rows: for m < RPT / 4 the four rows (m * GD_R + g) * 4 .. + 3, so that the lanes of a column read
// consecutive float4 of a staged vector at a time (no bank conflicts; the other column of the warp reads the same
// addresses).  What a token's step costs is the chain of instructions that depend on the state: the staged vectors of the
// NEXT token are read, and k * decay formed, while the current token's sums travel over the lanes; the decayed state
// decay * S is formed beside the dot product (k * decay)^T S of the old state instead of before it; the read-out q^T S is
// off the chain altogether.  A thread holds its rows of NC columns (value channels): the columns are independent chains that
// share the staged vectors, so the instructions that fetch them and form k * decay are issued once for NC columns, and the
// chains' latencies overlap; every column's arithmetic is the same whatever NC is.
// (Registers: with one column a thread four blocks of 128 threads share an SM, as many as the grid of a long prompt brings; with
// two columns the grid is half as large and a thread may hold twice the registers, which spares it the spills.)
template <int RPT, bool VEC, int GD_R, bool DELTA, int NC>
__global__ void __launch_bounds__(GD_R * GD_COLS, (NC == 1 ? 512 : 256) / (GD_R * GD_COLS)) gated_delta_walk_kernel(GatedDeltaArgs a, int n_buf) {
    ce_pdl_begin();
    extern __shared__ __align__(16) float gd_smem[];
    constexpr int R4 = RPT / 4, BC = GD_COLS * NC;
    int d = a.d, dv = a.dv;
    int h = blockIdx.x, b = blockIdx.y, col0 = blockIdx.z * BC, tid = threadIdx.x;
    int t_begin = a.q_start[b], t_end = a.q_start[b + 1];
    if (t_end <= t_begin) return;
    int ncols = min(BC, dv - col0);
    constexpr bool delta = DELTA;              // false: the plain sum of outer products, whose write needs no dot product
    int jj = (tid / GD_R) * NC, g = tid % GD_R;          // this thread's columns: col0 + jj .. + NC - 1
    bool owner[NC];
    float* sp = a.state + ((size_t)a.seq_slot[b] * a.H + h) * d * dv;
    float S[NC][RPT];
#pragma unroll
    for (int n = 0; n < NC; ++n) {
        owner[n] = jj + n < ncols;
#pragma unroll
        for (int m = 0; m < RPT; ++m) {
            int row = ((m >> 2) * GD_R + g) * 4 + (m & 3);
            S[n][m] = (owner[n] && row < d) ? sp[(size_t)row * dv + col0 + jj + n] : 0.f;
        }
    }
    // a row of the staged vectors is padded to GD_R * RPT floats, so that every thread reads whole float4
    constexpr int dp = GD_R * RPT;
    int buf_floats = 3 * GD_TILE * dp + GD_TILE * (BC + 1);
    buf_floats = (buf_floats + 3) / 4 * 4;
    // the padding of every staged row stays zero (rows of tokens a tile does not have are read ahead but never used)
    if (dp > d)
        for (int e = tid; e < n_buf * 3 * GD_TILE * (dp - d); e += blockDim.x) {
            int row = e / (dp - d), c = d + e % (dp - d);
            gd_smem[(row / (3 * GD_TILE)) * buf_floats + (row % (3 * GD_TILE)) * dp + c] = 0.f;
        }
    __syncthreads();
    int n_tiles = (t_end - t_begin + GD_TILE - 1) / GD_TILE;
    gd_stage<dp, VEC, BC>(a, gd_smem, t_begin, min(GD_TILE, t_end - t_begin), h, col0, ncols);
    for (int tile = 0; tile < n_tiles; ++tile) {
        int t0 = t_begin + tile * GD_TILE, n_tok = min(GD_TILE, t_end - t0);
        float* buf = gd_smem + (tile & (n_buf - 1)) * buf_floats;
        if (tile + 1 < n_tiles && n_buf == 2) {
            gd_stage<dp, VEC, BC>(a, gd_smem + ((tile + 1) & 1) * buf_floats, t0 + GD_TILE, min(GD_TILE, t_end - t0 - GD_TILE), h, col0, ncols);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            if (tile > 0 && n_buf == 1) gd_stage<dp, VEC, BC>(a, buf, t0, n_tok, h, col0, ncols);     // one buffer: a tile is staged when its turn comes
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const float* vbuf = buf + 3 * GD_TILE * dp;
        // The sum over rows of S^T q is not needed by the next token: every thread keeps its part for each token of
        // the tile, and the butterflies of all tokens run together after the walk (their latencies overlap).
        float part[NC][GD_TILE];
        float4 w[R4], kw[R4], k[R4], q[R4];
        float vj[NC], beta;
        auto lo2 = [](const float4& v) { return make_float2(v.x, v.y); };
        auto hi2 = [](const float4& v) { return make_float2(v.z, v.w); };
        auto fetch = [&](int tok) {                 // a token's vectors; nothing here depends on the state
#pragma unroll
            for (int m = 0; m < R4; ++m) {
                w[m] = *reinterpret_cast<const float4*>(buf + (0 * GD_TILE + tok) * dp + (m * GD_R + g) * 4);
                k[m] = *reinterpret_cast<const float4*>(buf + (1 * GD_TILE + tok) * dp + (m * GD_R + g) * 4);
                q[m] = *reinterpret_cast<const float4*>(buf + (2 * GD_TILE + tok) * dp + (m * GD_R + g) * 4);
                float2 a0 = __fmul2_rn(lo2(k[m]), lo2(w[m])), a1 = __fmul2_rn(hi2(k[m]), hi2(w[m]));
                kw[m] = make_float4(a0.x, a0.y, a1.x, a1.y);
            }
#pragma unroll
            for (int n = 0; n < NC; ++n) vj[n] = owner[n] ? vbuf[tok * (BC + 1) + jj + n] : 0.f;
            beta = vbuf[tok * (BC + 1) + BC];
        };
        fetch(0);
        // The arithmetic on the state runs on pairs of rows (fma.f32x2: two IEEE operations an instruction, the same results):
        // a token's step is a chain of instructions a warp issues nearly one after another, so their number is its time.
#pragma unroll
        for (int tok = 0; tok < GD_TILE; ++tok) {
#pragma unroll
            for (int n = 0; n < NC; ++n) part[n][tok] = 0.f;
            if (tok < n_tok) {
                // (k * decay)^T S over this thread's rows in four runs (a fixed order), and the decayed state beside it
                float2 dS[NC][RPT / 2];
                float dot[NC];
                float4 kc[R4], qc[R4];
#pragma unroll
                for (int m = 0; m < R4; ++m) { kc[m] = k[m]; qc[m] = q[m]; }
#pragma unroll
                for (int n = 0; n < NC; ++n) {
                    float2 p01 = make_float2(0.f, 0.f), p23 = make_float2(0.f, 0.f);
#pragma unroll
                    for (int m = 0; m < R4; ++m) {
                        float2 s01 = make_float2(S[n][4 * m], S[n][4 * m + 1]), s23 = make_float2(S[n][4 * m + 2], S[n][4 * m + 3]);
                        if (delta) {
                            p01 = __ffma2_rn(lo2(kw[m]), s01, p01);
                            p23 = __ffma2_rn(hi2(kw[m]), s23, p23);
                        }
                        dS[n][2 * m] = __fmul2_rn(lo2(w[m]), s01);
                        dS[n][2 * m + 1] = __fmul2_rn(hi2(w[m]), s23);
                    }
                    dot[n] = (p01.x + p01.y) + (p23.x + p23.y);
                }
                float v_now[NC];
#pragma unroll
                for (int n = 0; n < NC; ++n) v_now[n] = vj[n];
                const float beta_now = beta;
                if (tok + 1 < GD_TILE) fetch(tok + 1);          // (rows past the tile's tokens hold older tokens: unused)
                // over the column's lanes in rounds of four: every lane adds the same pairs, so all hold the same sum
                if (delta) {
                    float e1[NC], e2[NC], e3[NC];
#pragma unroll
                    for (int n = 0; n < NC; ++n) {
                        e1[n] = __shfl_xor_sync(0xffffffffu, dot[n], 1); e2[n] = __shfl_xor_sync(0xffffffffu, dot[n], 2);
                        e3[n] = __shfl_xor_sync(0xffffffffu, dot[n], 3);
                    }
#pragma unroll
                    for (int n = 0; n < NC; ++n) dot[n] = (dot[n] + e1[n]) + (e2[n] + e3[n]);
#pragma unroll
                    for (int n = 0; n < NC; ++n) {
                        e1[n] = __shfl_xor_sync(0xffffffffu, dot[n], 4); e2[n] = __shfl_xor_sync(0xffffffffu, dot[n], 8);
                        e3[n] = __shfl_xor_sync(0xffffffffu, dot[n], 12);
                    }
#pragma unroll
                    for (int n = 0; n < NC; ++n) dot[n] = (dot[n] + e1[n]) + (e2[n] + e3[n]);
                    if (GD_R == 32) {
#pragma unroll
                        for (int n = 0; n < NC; ++n) dot[n] += __shfl_xor_sync(0xffffffffu, dot[n], 16);
                    }
                }
#pragma unroll
                for (int n = 0; n < NC; ++n) {
                    float u = delta ? beta_now * (v_now[n] - dot[n]) : v_now[n];         // the plain sum of outer products writes v itself
                    const float2 uu = make_float2(u, u);
                    float2 q01 = make_float2(0.f, 0.f), q23 = make_float2(0.f, 0.f);
#pragma unroll
                    for (int m = 0; m < R4; ++m) {
                        float2 s01 = __ffma2_rn(lo2(kc[m]), uu, dS[n][2 * m]), s23 = __ffma2_rn(hi2(kc[m]), uu, dS[n][2 * m + 1]);
                        S[n][4 * m] = s01.x; S[n][4 * m + 1] = s01.y; S[n][4 * m + 2] = s23.x; S[n][4 * m + 3] = s23.y;
                        q01 = __ffma2_rn(s01, lo2(qc[m]), q01);
                        q23 = __ffma2_rn(s23, hi2(qc[m]), q23);
                    }
                    part[n][tok] = (q01.x + q01.y) + (q23.x + q23.y);
                }
            }
        }
#pragma unroll
        for (int n = 0; n < NC; ++n) {
#pragma unroll
            for (int o = 1; o < GD_R; o <<= 1)
#pragma unroll
                for (int tok = 0; tok < GD_TILE; ++tok) part[n][tok] += __shfl_xor_sync(0xffffffffu, part[n][tok], o);
            // lane g of a column stores token g of the tile (GD_TILE <= GD_R)
            float mine = part[n][0];
#pragma unroll
            for (int tok = 1; tok < GD_TILE; ++tok) mine = g == tok ? part[n][tok] : mine;
            if (owner[n] && g < n_tok) a.raw[(size_t)(t0 + g) * a.H * dv + h * dv + col0 + jj + n] = mine;
        }
        __syncthreads();             // the buffer is free for the tile after the next
    }
#pragma unroll
    for (int n = 0; n < NC; ++n)
#pragma unroll
        for (int m = 0; m < RPT; ++m) {
            int row = ((m >> 2) * GD_R + g) * 4 + (m & 3);
            if (owner[n] && row < d) sp[(size_t)row * dv + col0 + jj + n] = S[n][m];
        }
}

// A step of single tokens (every sequence brings exactly one): the walk's arithmetic for one token, laid out for bandwidth.
// The state moves once, so what counts is how it is read and written: a block takes (head, sequence, 32 value channels), a warp
// 32 neighbouring channels of the rows of one "lane" of the walk, so every load and store of the state is 128 contiguous bytes.
// Thread (g, c) does exactly what lane g of column c does in the walk, term by term and in the same order; the two sums over
// the lanes, which the walk takes with butterflies, are taken from shared memory in the butterflies' order (a balanced tree over
// the lanes for the read-out; quads, then quads of quads, for the dot product).  A token therefore gets the same bits whether
// it arrives alone or inside a portion.
#define GD_STEP_COLS 32
template <int RPT, int GD_R, bool DELTA>
__global__ void __launch_bounds__(GD_R * GD_STEP_COLS) gated_delta_step_kernel(GatedDeltaArgs a) {
    ce_pdl_begin();
    constexpr int R4 = RPT / 4, dp = GD_R * RPT;
    __shared__ __align__(16) float vec[3 * dp];                    // decay, key, query of the token, padded with zeros
    __shared__ float dots[GD_R * GD_STEP_COLS], parts[GD_R * GD_STEP_COLS];
    int d = a.d, dv = a.dv, H = a.H, G = a.G;
    int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x;
    int c = tid % GD_STEP_COLS, g = tid / GD_STEP_COLS, j = blockIdx.z * GD_STEP_COLS + c;
    int t = a.q_start[b];
    if (a.q_start[b + 1] <= t) return;
    bool owner = j < dv;
    int C = 2 * G * d + H * dv, kh = h / (H / G);
    const float* row = a.prep + (size_t)t * a.P;
    int offs[3] = {C + h * d, G * d + kh * d, kh * d};          // decay, key, query within a prep row
    for (int e = tid; e < 3 * dp; e += blockDim.x) {
        int which = e / dp, i = e % dp;
        vec[e] = i < d ? row[offs[which] + i] : 0.f;
    }
    float* sp = a.state + ((size_t)a.seq_slot[b] * H + h) * d * dv;
    float S[RPT];
#pragma unroll
    for (int m = 0; m < RPT; ++m) {
        int r = ((m >> 2) * GD_R + g) * 4 + (m & 3);
        S[m] = (owner && r < d) ? sp[(size_t)r * dv + j] : 0.f;
    }
    float vj = owner ? row[2 * G * d + h * dv + j] : 0.f, beta = row[C + H * d + h];
    __syncthreads();
    float w[RPT], k[RPT], q[RPT], dS[RPT];
    float p0 = 0.f, p1 = 0.f, p2 = 0.f, p3 = 0.f;
#pragma unroll
    for (int m4 = 0; m4 < R4; ++m4) {
        const float4 w4 = *reinterpret_cast<const float4*>(vec + 0 * dp + (m4 * GD_R + g) * 4);
        const float4 k4 = *reinterpret_cast<const float4*>(vec + 1 * dp + (m4 * GD_R + g) * 4);
        const float4 q4 = *reinterpret_cast<const float4*>(vec + 2 * dp + (m4 * GD_R + g) * 4);
        w[4 * m4] = w4.x; w[4 * m4 + 1] = w4.y; w[4 * m4 + 2] = w4.z; w[4 * m4 + 3] = w4.w;
        k[4 * m4] = k4.x; k[4 * m4 + 1] = k4.y; k[4 * m4 + 2] = k4.z; k[4 * m4 + 3] = k4.w;
        q[4 * m4] = q4.x; q[4 * m4 + 1] = q4.y; q[4 * m4 + 2] = q4.z; q[4 * m4 + 3] = q4.w;
        if (DELTA) {
            p0 = fmaf(__fmul_rn(k[4 * m4], w[4 * m4]), S[4 * m4], p0);
            p1 = fmaf(__fmul_rn(k[4 * m4 + 1], w[4 * m4 + 1]), S[4 * m4 + 1], p1);
            p2 = fmaf(__fmul_rn(k[4 * m4 + 2], w[4 * m4 + 2]), S[4 * m4 + 2], p2);
            p3 = fmaf(__fmul_rn(k[4 * m4 + 3], w[4 * m4 + 3]), S[4 * m4 + 3], p3);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) dS[4 * m4 + i] = __fmul_rn(w[4 * m4 + i], S[4 * m4 + i]);
    }
    float u = vj;
    if (DELTA) {
        dots[g * GD_STEP_COLS + c] = __fadd_rn(__fadd_rn(p0, p1), __fadd_rn(p2, p3));
        __syncthreads();
        // the lanes' sums in the order of the walk's butterfly: quads of lanes, then quads of quads (then the two halves of 32)
        float quad[GD_R / 4];
#pragma unroll
        for (int n = 0; n < GD_R / 4; ++n)
            quad[n] = __fadd_rn(__fadd_rn(dots[(4 * n) * GD_STEP_COLS + c], dots[(4 * n + 1) * GD_STEP_COLS + c]),
                                __fadd_rn(dots[(4 * n + 2) * GD_STEP_COLS + c], dots[(4 * n + 3) * GD_STEP_COLS + c]));
        float dot = __fadd_rn(__fadd_rn(quad[0], quad[1]), __fadd_rn(quad[2], quad[3]));
        if (GD_R == 32) dot = __fadd_rn(dot, __fadd_rn(__fadd_rn(quad[GD_R / 4 - 4], quad[GD_R / 4 - 3]), __fadd_rn(quad[GD_R / 4 - 2], quad[GD_R / 4 - 1])));
        u = __fmul_rn(beta, __fsub_rn(vj, dot));
    }
    float q0 = 0.f, q1 = 0.f, q2 = 0.f, q3 = 0.f;
#pragma unroll
    for (int m4 = 0; m4 < R4; ++m4) {
#pragma unroll
        for (int i = 0; i < 4; ++i) S[4 * m4 + i] = fmaf(k[4 * m4 + i], u, dS[4 * m4 + i]);
        q0 = fmaf(S[4 * m4], q[4 * m4], q0);
        q1 = fmaf(S[4 * m4 + 1], q[4 * m4 + 1], q1);
        q2 = fmaf(S[4 * m4 + 2], q[4 * m4 + 2], q2);
        q3 = fmaf(S[4 * m4 + 3], q[4 * m4 + 3], q3);
    }
#pragma unroll
    for (int m = 0; m < RPT; ++m) {
        int r = ((m >> 2) * GD_R + g) * 4 + (m & 3);
        if (owner && r < d) sp[(size_t)r * dv + j] = S[m];
    }
    parts[g * GD_STEP_COLS + c] = __fadd_rn(__fadd_rn(q0, q1), __fadd_rn(q2, q3));
    __syncthreads();
    if (g == 0 && owner) {
        // a balanced tree over the lanes: neighbours, then pairs of pairs, and so on (the walk's butterfly with offsets 1, 2, 4, ...)
        float tree[GD_R];
#pragma unroll
        for (int n = 0; n < GD_R; ++n) tree[n] = parts[n * GD_STEP_COLS + c];
#pragma unroll
        for (int o = 1; o < GD_R; o <<= 1)
#pragma unroll
            for (int n = 0; n < GD_R; n += 2 * o) tree[n] = __fadd_rn(tree[n], tree[n + o]);
        a.raw[(size_t)t * H * dv + h * dv + j] = tree[0];
    }
}

// A token's heads are dealt to the warps of gridDim.y blocks in turn: root mean square over the head's values, weight, gate.
template <typename T>
__global__ void gated_delta_finish_kernel(GatedDeltaArgs a) {
    ce_pdl_begin();
    int t = blockIdx.x, lane = threadIdx.x & 31, nwarp = (blockDim.x >> 5) * gridDim.y;
    int warp = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);
    int dv = a.dv, n = a.H * dv;
    const float* o = a.raw + (size_t)t * n;
    const float* gz = a.gz + (size_t)t * a.ld_gz;
    for (int h = warp; h < a.H; h += nwarp) {
        float ss = 0.f;
        for (int c = lane; c < dv; c += 32) ss = fmaf(o[h * dv + c], o[h * dv + c], ss);
        for (int k = 16; k > 0; k >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, k);
        float inv = 1.0f / sqrtf(ss / (float)dv + a.eps);
        for (int c = lane; c < dv; c += 32) {
            int col = h * dv + c;
            float z = gz[col], g = gd_sigmoid(z);
            if (a.gate_act == 1) g *= z;
            float y = o[col] * inv;
            if (a.norm_w) y *= a.norm_w[c];
            CeType<T>::store((T*)a.out + (size_t)t * n + col, y * g * a.out_scale);
        }
    }
}

// n_buf 1: every sequence has one tile: one staging buffer, twice the blocks an SM.  nc: value channels a thread holds.
template <int RPT, int R, int NC>
static void gd_launch_walk_nc(const GatedDeltaArgs& a, int B, bool vec, int n_buf, cudaStream_t stream) {
    constexpr int BC = GD_COLS * NC;
    size_t floats = 3 * GD_TILE * R * RPT + GD_TILE * (BC + 1);
    size_t smem = (size_t)n_buf * ((floats + 3) / 4 * 4) * sizeof(float);
    dim3 grid(a.H, B, (a.dv + BC - 1) / BC);
    ce_note("gated_delta_walk_kernel");
    auto go = [&](auto kernel) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        ce_launch(kernel, grid, R * GD_COLS, smem, stream, a, n_buf);
    };
    if (a.rule == 0) {
        if (vec) go(gated_delta_walk_kernel<RPT, true, R, true, NC>);
        else go(gated_delta_walk_kernel<RPT, false, R, true, NC>);
    } else {
        if (vec) go(gated_delta_walk_kernel<RPT, true, R, false, NC>);
        else go(gated_delta_walk_kernel<RPT, false, R, false, NC>);
    }
}

// Two value channels a thread where that still leaves three blocks for every two SMs (CE_DELTA_WALK_COLS=1 or 2 forces one or
// two, for measurement).  A column's sums are the same either way, so the choice may follow the number of sequences.  Measured
// on one 2,048-token prompt with heads of 128 x 128, four launches: 32 heads (256 blocks of two columns a thread) 3.49 -> 2.85 ms;
// 16 heads (128 blocks) 2.45 -> 2.50 ms, where a block's chain of dependent instructions, not the issue rate, sets the time.
template <int RPT, int R>
static void gd_launch_walk(const GatedDeltaArgs& a, int B, bool vec, int n_buf, cudaStream_t stream) {
    static int cols = getenv("CE_DELTA_WALK_COLS") ? atoi(getenv("CE_DELTA_WALK_COLS")) : 0;
    bool fits = a.dv % (2 * GD_COLS) == 0;
    long long blocks2 = (long long)a.H * B * (a.dv / (2 * GD_COLS));
    bool two = cols == 0 ? fits && 2 * blocks2 >= 3LL * ce_sm_count() : cols >= 2 && fits;
    if (two) gd_launch_walk_nc<RPT, R, 2>(a, B, vec, n_buf, stream);
    else gd_launch_walk_nc<RPT, R, 1>(a, B, vec, n_buf, stream);
}

// Floats of a ``prep`` row for these sizes.
extern "C" int ce_gated_delta_prep_width(int H, int G, int d, int dv) {
    return (2 * G * d + H * dv + H * d + H + 3) / 4 * 4;
}

// stage: 1 prepare, 2 keep, 3 walk, 4 finish (each one launch, so that each is counted and timed by itself)
extern "C" int ce_gated_delta(const float* proj, const float* dec, const float* gz, const float* taps, const float* a_log,
                              const float* dt_bias, const float* norm_w, float* prep, float* raw, float* state, float* kept,
                              void* out, int out_dtype, const int* seq_of_token, const int* seq_slot, const int* q_start,
                              int T, int B, int ld, int off_conv, int off_b, int H, int G, int d, int dv, int K, float eps,
                              int ld_dec, int ld_gz, int decay_mode, int operands, int rule, int gate_act, float out_scale,
                              const float* cos_table, const float* sin_table, const int* positions, int* status, int rd, int max_pos,
                              int stage, cudaStream_t stream) {
    if (B == 0 || T == 0) return CE_OK;
    if (stage < 1 || stage > 4) return ce_fail(CE_ERR_ARG, "ce_gated_delta: stage %d", stage);
    if (decay_mode < 0 || decay_mode > 2 || operands < 0 || operands > 1 || rule < 0 || rule > 1 || gate_act < 0 || gate_act > 1)
        return ce_fail(CE_ERR_ARG, "ce_gated_delta: decay %d, operands %d, rule %d, gate %d", decay_mode, operands, rule, gate_act);
    if (!proj || !gz || !a_log || !prep || !raw || !state || !out || !seq_of_token || !seq_slot || !q_start ||
        (decay_mode != 2 && (!dec || !dt_bias)) || (operands == 0 && (!taps || (K > 1 && !kept))))
        return ce_fail(CE_ERR_ARG, "ce_gated_delta: null pointer");
    if (operands == 1) {
        if (K != 1 || decay_mode != 2) return ce_fail(CE_ERR_ARG, "ce_gated_delta: rotated operands come without a convolution and with constant decays");
        if (rd < 0 || rd > d || rd % 2) return ce_fail(CE_ERR_SIZE, "ce_gated_delta: %d rotated elements of %d", rd, d);
        if (rd > 0 && (!cos_table || !sin_table || !positions || !status)) return ce_fail(CE_ERR_ARG, "ce_gated_delta: no rotation tables");
    }
    if (d <= 0 || d > 256 || dv <= 0) return ce_fail(CE_ERR_SIZE, "ce_gated_delta: head sizes %d / %d (keys up to 256)", d, dv);
    if (H <= 0 || G <= 0 || H % G || B > 65535 || K < 1 || K > 64)
        return ce_fail(CE_ERR_SIZE, "ce_gated_delta: %d heads, %d key heads, %d sequences, %d taps", H, G, B, K);
    if (out_dtype != CE_F32 && out_dtype != CE_BF16) return ce_fail(CE_ERR_ARG, "ce_gated_delta: unknown dtype %d", out_dtype);
    int P = ce_gated_delta_prep_width(H, G, d, dv);
    GatedDeltaArgs a{proj, dec, gz, taps, a_log, dt_bias, norm_w, prep, raw, state, kept, out, seq_of_token, seq_slot, q_start,
                     ld, off_conv, off_b, H, G, d, dv, K, P, eps, ld_dec, ld_gz, decay_mode, operands, rule, gate_act, out_scale,
                     rd > 0 ? cos_table : nullptr, sin_table, positions, status, rd, max_pos};
    int heads = 2 * G + H;
    int threads = heads >= 8 ? 256 : 32 * heads;
    if (stage == 1) {
        ce_note("gated_delta_prepare_kernel");
        int per_block = threads / 32, want = (heads + per_block - 1) / per_block, room = 4 * 148 / T;
        int split = want < room ? want : room;
        ce_launch(gated_delta_prepare_kernel, dim3(T, split < 1 ? 1 : split), threads, 0, stream, a);
    } else if (stage == 2) {
        if (K == 1) return CE_OK;
        size_t total = (size_t)B * (2 * G * d + H * dv), want = (total + 255) / 256;
        ce_note("gated_delta_keep_kernel");
        ce_launch(gated_delta_keep_kernel, (int)(want < 148 * 8 ? want : 148 * 8), 256, 0, stream, a, B);
    } else if (stage == 4) {
        ce_note("gated_delta_finish_kernel");
        int th = H >= 8 ? 256 : 32 * H;
        int want = (H + th / 32 - 1) / (th / 32), room = 4 * 148 / T, split = want < room ? want : room;
        dim3 grid(T, split < 1 ? 1 : split);
        if (out_dtype == CE_F32) ce_launch(gated_delta_finish_kernel<float>, grid, th, 0, stream, a);
        else ce_launch(gated_delta_finish_kernel<__nv_bfloat16>, grid, th, 0, stream, a);
    } else {
        // 16-byte copies where every source address is a multiple of 16
        int C = 2 * G * d + H * dv;
        bool vec = d % 4 == 0 && C % 4 == 0 && ((uintptr_t)prep & 15) == 0;
        // lanes a column and rows a thread by the key size alone (never by the batch: a request's sums do not depend on its neighbours)
        // Measured at 2,048 tokens with heads of 128 x 128: 16 lanes a column took 0.63 ms (16 heads) and 0.90 ms (32 heads) a
        // launch, 32 lanes 0.61 and 1.21: twice the warps for the same columns, and with 32 heads the SMs' issue slots run out.
        int n_buf = T == B ? 1 : 2;             // as many tokens as sequences: every sequence brings exactly one
        static int no_step = getenv("CE_DELTA_NO_STEP") ? 1 : 0;       // (for measurement: single tokens on the walk)
        if (T == B && !no_step) {
            dim3 grid(H, B, (dv + GD_STEP_COLS - 1) / GD_STEP_COLS);
            ce_note("gated_delta_step_kernel");
#define GD_STEP_CASE(RPT, R)                                                                                      \
            if (a.rule == 0) ce_launch(gated_delta_step_kernel<RPT, R, true>, grid, R * GD_STEP_COLS, 0, stream, a);  \
            else ce_launch(gated_delta_step_kernel<RPT, R, false>, grid, R * GD_STEP_COLS, 0, stream, a);
            if (d <= 64) { GD_STEP_CASE(4, 16) } else if (d <= 128) { GD_STEP_CASE(8, 16) } else { GD_STEP_CASE(8, 32) }
#undef GD_STEP_CASE
            return ce_check_launch("ce_gated_delta");
        }
        if (d <= 64) gd_launch_walk<4, 16>(a, B, vec, n_buf, stream);
        else if (d <= 128) gd_launch_walk<8, 16>(a, B, vec, n_buf, stream);
        else gd_launch_walk<8, 32>(a, B, vec, n_buf, stream);
    }
    return ce_check_launch("ce_gated_delta");
}
