// Kernels of mixers that carry a fixed-size state from token to token, and the small steps around them:
//   k_sinusoid_add     sinusoidal position vector added to the embedding output
//   k_mix_cat          [residual + pending branch | embedding output] as one row, the input of a pass's mixing product
//   k_short_conv       causal convolution over time per channel, its last taps - 1 inputs kept per sequence
//   k_delta_rule       gated delta rule: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q
//   k_head_norm_gate   RMS norm of every head over its own elements, shared gains, gate
//   k_min_gru          S <- (1 - z) S + z c, element by element, gates from the current token alone
//   k_branch_norm_mean the mean of several branches, each RMS-normed over the model width with gains of its own
//   k_moe_gate_mul     gated expert: act(w g) * (w u) over sorted pairs (the pick's weight scales the expert's input)
//   k_row_gate         rows times the logistic function of one number per row
// Storage is float or bf16, all arithmetic 32-bit (angles 64-bit); every sum has an order that depends on sizes and
// positions only, so a row's result does not depend on the batch or on how a prompt was cut into steps. Rows whose
// position is -1 are padding of a recorded step: they read and write no state.
#include "common.cuh"
#include <math.h>

template <typename TIN>
__device__ __forceinline__ float rc_rd(const TIN* src, int n_planes, size_t plane_stride, size_t i) {
    float v = kb_to_f<TIN>(src[i]);
    for (int s = 1; s < n_planes; s++) v += kb_to_f<TIN>(src[(size_t)s * plane_stride + i]);
    return v;
}
__device__ __forceinline__ float rc_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float rc_silu(float z) { return z / (1.0f + expf(-z)); }
__device__ __forceinline__ float rc_softplus(float z) { return log1pf(expf(-fabsf(z))) + fmaxf(z, 0.0f); }
#define RC_GATE_NONE 0
#define RC_GATE_SIGMOID 1
#define RC_GATE_SILU 2
__device__ __forceinline__ float rc_gate(float z, int kind) {
    return kind == RC_GATE_SIGMOID ? rc_sigmoid(z) : kind == RC_GATE_SILU ? rc_silu(z) : z;
}

// ------------------------------------------------------------------------------------------------ sinusoidal positions
// x[t][2i] += sin(p f_i), x[t][2i + 1] += cos(p f_i); the angle and the functions in 64-bit (freq: E / 2 doubles)
__global__ void __launch_bounds__(256) k_sinusoid_add(float* KB_STEP_DATA x, const int* __restrict__ pos,
                                                      const double* __restrict__ freq, int E) {
    kb_pdl_launch();
    const int t = blockIdx.x;
    const int p = pos[t];
    kb_pdl_wait();
    if (p < 0) return;
    float* xr = x + (size_t)t * E;
    for (int c = threadIdx.x; c < E; c += 256) {
        const double a = (double)p * freq[c >> 1];
        xr[c] += (float)((c & 1) ? cos(a) : sin(a));
    }
}

extern "C" int kb_sinusoid_add(float* x, const int* pos, const double* freq, int T, int E, cudaStream_t st) {
    if (T <= 0) return 0;
    kb_launch(k_sinusoid_add, T, 256, 0, st, x, pos, freq, E);
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ input of a pass
// out[t] = [x[t] + ls * (sum of the planes)[t] | x0[t]]; ls: a scale per column or null
template <typename TO>
__global__ void __launch_bounds__(256) k_mix_cat(const float* KB_STEP_DATA x, const float* KB_STEP_DATA delta,
        int n_delta, size_t delta_stride, const float* __restrict__ ls, const float* KB_STEP_DATA x0,
        TO* __restrict__ out, int E) {
    kb_pdl_launch();
    kb_pdl_wait();
    const size_t t = blockIdx.x;
    for (int c = threadIdx.x; c < E; c += 256) {
        float v = x[t * E + c];
        if (n_delta > 0) {
            float d = delta[t * E + c];
            for (int s = 1; s < n_delta; s++) d += delta[(size_t)s * delta_stride + t * E + c];
            v += ls ? __fmul_rn(ls[c], d) : d;
        }
        out[t * 2 * E + c] = kb_from_f<TO>(v);
        out[t * 2 * E + E + c] = kb_from_f<TO>(x0[t * E + c]);
    }
}

extern "C" int kb_mix_cat(const float* x, const float* delta, int n_delta, long long delta_stride, const float* ls,
                          const float* x0, void* out, int odtype, int T, int E, cudaStream_t st) {
    if (T <= 0) return 0;
    if (odtype == KB_F32)
        kb_launch(k_mix_cat<float>, T, 256, 0, st, x, delta, n_delta, (size_t)delta_stride, ls, x0, (float*)out, E);
    else
        kb_launch(k_mix_cat<bf16>, T, 256, 0, st, x, delta, n_delta, (size_t)delta_stride, ls, x0, (bf16*)out, E);
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ short convolution
// y[t][c] = act(sum_j w[c][j] * u[t - (taps - 1) + j][c]), u = input columns col0.. (+ bias), over the positions of
// the row's own sequence; positions before this step's rows come from the sequence's tails (state: [taps - 1][C],
// oldest first, zero when the sequence starts), and the step's last taps - 1 inputs become the new tails. The thread
// of a sequence's first row of the step works its first taps - 1 rows (the only ones that read tails) and then writes
// the new tails, so no other thread touches them.
#define SC_MAX_TAPS 8
template <typename TIN, typename TO>
__global__ void __launch_bounds__(128) k_short_conv(const TIN* KB_STEP_DATA in, int n_planes, size_t plane_stride,
        int ld_in, int col0, int C, const float* __restrict__ bias, const float* __restrict__ w, int taps, int act,
        float* state, size_t state_stride, const int* __restrict__ pos, const int* __restrict__ seq,
        const int* __restrict__ slot, const int* __restrict__ q_start, TO* __restrict__ out, int ldo) {
    kb_pdl_launch();
    const int t = blockIdx.x;
    const int c = blockIdx.y * 128 + threadIdx.x;
    const int p = pos[t];
    if (p < 0 || c >= C) {
        kb_pdl_wait();
        return;
    }
    const int b = seq[t];
    const int r0 = q_start[b], n = q_start[b + 1] - r0;
    const int i = t - r0;
    float wr[SC_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < SC_MAX_TAPS; j++) wr[j] = j < taps ? w[(size_t)c * taps + j] : 0.0f;
    const float bs = bias ? bias[c] : 0.0f;
    kb_pdl_wait();
#define SC_U(row) (rc_rd<TIN>(in + (size_t)(row) * ld_in, n_planes, plane_stride, (size_t)col0 + c) + bs)
    if (i >= taps - 1) {
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < SC_MAX_TAPS; j++)
            if (j < taps) acc = fmaf(wr[j], SC_U(t - (taps - 1) + j), acc);
        out[(size_t)t * ldo + c] = kb_from_f<TO>(act ? rc_silu(acc) : acc);
        return;
    }
    if (i != 0) return;
    float* tails = state + (size_t)slot[b] * state_stride;
    float tl[SC_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < SC_MAX_TAPS; j++) tl[j] = j < taps - 1 ? tails[(size_t)j * C + c] : 0.0f;
    const int head = n < taps - 1 ? n : taps - 1;
    for (int i2 = 0; i2 < head; i2++) {
        float acc = 0.0f;
#pragma unroll
        for (int j = 0; j < SC_MAX_TAPS; j++) {
            if (j >= taps) continue;
            const int idx = i2 - (taps - 1) + j;
            float u;
            if (idx < 0) {
                u = 0.0f;
#pragma unroll
                for (int q = 0; q < SC_MAX_TAPS; q++)
                    if (q == taps - 1 + idx) u = tl[q];
            } else {
                u = SC_U(r0 + idx);
            }
            acc = fmaf(wr[j], u, acc);
        }
        out[(size_t)(r0 + i2) * ldo + c] = kb_from_f<TO>(act ? rc_silu(acc) : acc);
    }
    for (int j = 0; j < taps - 1; j++) {
        const int idx = n - (taps - 1) + j;
        float u;
        if (idx < 0) {
            u = 0.0f;
#pragma unroll
            for (int q = 0; q < SC_MAX_TAPS; q++)
                if (q == taps - 1 + idx) u = tl[q];
        } else {
            u = SC_U(r0 + idx);
        }
        tails[(size_t)j * C + c] = u;
    }
#undef SC_U
}

extern "C" int kb_short_conv(const void* in, int idtype, int n_planes, long long plane_stride, int ld_in, int col0,
                             int C, const float* bias, const float* w, int taps, int act, float* state,
                             long long state_stride, const int* pos, const int* seq, const int* slot,
                             const int* q_start, void* out, int odtype, int ldo, int T, cudaStream_t st) {
    if (T <= 0 || C <= 0) return 0;
    if (taps < 1 || taps > SC_MAX_TAPS) return (int)cudaErrorInvalidValue;
    dim3 grid(T, (C + 127) / 128);
#define KB_SC(TIN, TO)                                                                                              \
    kb_launch(k_short_conv<TIN, TO>, grid, 128, 0, st, (const TIN*)in, n_planes, (size_t)plane_stride, ld_in, col0, \
              C, bias, w, taps, act, state, (size_t)state_stride, pos, seq, slot, q_start, (TO*)out, ldo)
    if (idtype == KB_F32 && odtype == KB_F32) KB_SC(float, float);
    else if (idtype == KB_BF16 && odtype == KB_F32) KB_SC(bf16, float);
    else if (idtype == KB_F32 && odtype == KB_BF16) KB_SC(float, bf16);
    else if (idtype == KB_BF16 && odtype == KB_BF16) KB_SC(bf16, bf16);
    else return (int)cudaErrorInvalidValue;
#undef KB_SC
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ gated delta rule
// qkv: 32-bit rows [q (G d) | k (G d) | v (H dv)] (after convolution and activation). Per head h (query/key head
// h / (H / G)): q and k are made unit vectors, x / sqrt(sum x^2 + unit_eps), q times d^(-1/2);
// beta = sigmoid(b), g = exp(-exp(A_log_h) softplus(a + dt_bias_h)) from the projections' columns ob + h, oa + h;
// then, with the state S [d][dv] kept as [dv][d]:
//   S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q = (g S_old)^T q + u (k . q).
// A block works one (sequence, head) and RC_COLS columns of the state, a warp one column with its d elements over
// the lanes; tokens are staged RC_CHUNK at a time.
#define RC_COLS 8
#define RC_CHUNK 16
#define RC_MAX_DPL 8
template <typename TIN>
__global__ void __launch_bounds__(32 * RC_COLS) k_delta_rule(const float* KB_STEP_DATA qkv, int ldq,
        const TIN* KB_STEP_DATA proj, int n_planes, size_t plane_stride, int ldp, int ob, int oa,
        const float* __restrict__ a_log, const float* __restrict__ dt_bias, int H, int G, int d, int dv, float unit_eps,
        const int* __restrict__ q_start, const int* __restrict__ slot, float* state, size_t state_stride,
        float* __restrict__ out, int ldo) {
    extern __shared__ float sm[];
    float* qs = sm;                                   // [RC_CHUNK][d]
    float* ks = qs + RC_CHUNK * d;                    // [RC_CHUNK][d]
    float* vs = ks + RC_CHUNK * d;                    // [RC_CHUNK][RC_COLS]
    float* gs = vs + RC_CHUNK * RC_COLS;              // [RC_CHUNK]: decay
    float* bs = gs + RC_CHUNK;                        // [RC_CHUNK]: beta
    float* kq = bs + RC_CHUNK;                        // [RC_CHUNK]: k . q
    kb_pdl_launch();
    const int b = blockIdx.x / H, h = blockIdx.x % H;
    const int hg = h / (H / G);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e0 = blockIdx.y * RC_COLS, e = e0 + warp;
    const int r0 = q_start[b], r1 = q_start[b + 1];
    const float rate = expf(a_log[h]), dtb = dt_bias[h];
    const float qmul = 1.0f / sqrtf((float)d);
    float* srow = state + (size_t)slot[b] * state_stride + ((size_t)h * dv + (e < dv ? e : 0)) * d;
    kb_pdl_wait();
    float S[RC_MAX_DPL];
#pragma unroll
    for (int i = 0; i < RC_MAX_DPL; i++) {
        const int j = lane + 32 * i;
        S[i] = (e < dv && j < d) ? srow[j] : 0.0f;
    }
    const size_t oq = (size_t)hg * d, ok = (size_t)G * d + (size_t)hg * d, ov = (size_t)2 * G * d + (size_t)h * dv;
    for (int c0 = r0; c0 < r1; c0 += RC_CHUNK) {
        const int n = min(RC_CHUNK, r1 - c0);
        for (int idx = threadIdx.x; idx < n * d; idx += 32 * RC_COLS) {
            const int t = idx / d, j = idx % d;
            const float* src = qkv + (size_t)(c0 + t) * ldq;
            qs[t * d + j] = src[oq + j];
            ks[t * d + j] = src[ok + j];
        }
        for (int idx = threadIdx.x; idx < n * RC_COLS; idx += 32 * RC_COLS) {
            const int t = idx / RC_COLS, w = idx % RC_COLS;
            vs[idx] = (e0 + w < dv) ? qkv[(size_t)(c0 + t) * ldq + ov + e0 + w] : 0.0f;
        }
        if (threadIdx.x < n) {
            const TIN* src = proj + (size_t)(c0 + threadIdx.x) * ldp;
            bs[threadIdx.x] = rc_sigmoid(rc_rd<TIN>(src, n_planes, plane_stride, (size_t)ob + h));
            gs[threadIdx.x] = expf(-rate * rc_softplus(rc_rd<TIN>(src, n_planes, plane_stride, (size_t)oa + h) + dtb));
        }
        __syncthreads();
        // unit vectors: warp w takes the chunk's tokens w, w + RC_COLS, ...
        for (int t = warp; t < n; t += RC_COLS) {
            float sq = 0.0f, sk = 0.0f;
            for (int j = lane; j < d; j += 32) {
                sq = fmaf(qs[t * d + j], qs[t * d + j], sq);
                sk = fmaf(ks[t * d + j], ks[t * d + j], sk);
            }
            sq = kb_warp_sum(sq);
            sk = kb_warp_sum(sk);
            const float fq = qmul / sqrtf(sq + unit_eps), fk = 1.0f / sqrtf(sk + unit_eps);
            float dot = 0.0f;
            for (int j = lane; j < d; j += 32) {
                const float qv = qs[t * d + j] * fq, kv = ks[t * d + j] * fk;
                qs[t * d + j] = qv;
                ks[t * d + j] = kv;
                dot = fmaf(qv, kv, dot);
            }
            dot = kb_warp_sum(dot);
            if (lane == 0) kq[t] = dot;
        }
        __syncthreads();
        for (int t = 0; t < n; t++) {
            const float g = gs[t];
            float a = 0.0f, c = 0.0f;
#pragma unroll
            for (int i = 0; i < RC_MAX_DPL; i++) {
                const int j = lane + 32 * i;
                if (j < d) {
                    S[i] = __fmul_rn(g, S[i]);
                    a = fmaf(S[i], ks[t * d + j], a);
                    c = fmaf(S[i], qs[t * d + j], c);
                }
            }
            a = kb_warp_sum(a);
            c = kb_warp_sum(c);
            const float u = __fmul_rn(bs[t], vs[t * RC_COLS + warp] - a);
#pragma unroll
            for (int i = 0; i < RC_MAX_DPL; i++) {
                const int j = lane + 32 * i;
                if (j < d) S[i] = fmaf(ks[t * d + j], u, S[i]);
            }
            if (lane == 0 && e < dv) out[(size_t)(c0 + t) * ldo + (size_t)h * dv + e] = fmaf(u, kq[t], c);
        }
        __syncthreads();
    }
    if (e < dv && r1 > r0) {
#pragma unroll
        for (int i = 0; i < RC_MAX_DPL; i++) {
            const int j = lane + 32 * i;
            if (j < d) srow[j] = S[i];
        }
    }
}

extern "C" int kb_delta_rule(const float* qkv, int ldq, const void* proj, int pdtype, int n_planes,
                             long long plane_stride, int ldp, int ob, int oa, const float* a_log, const float* dt_bias,
                             int B, int H, int G, int d, int dv, float unit_eps, const int* q_start, const int* slot,
                             float* state, long long state_stride, float* out, int ldo, cudaStream_t st) {
    if (B <= 0) return 0;
    if (d > 32 * RC_MAX_DPL || G <= 0 || H % G) return (int)cudaErrorInvalidValue;
    dim3 grid(B * H, (dv + RC_COLS - 1) / RC_COLS);
    const size_t sm = (size_t)(2 * RC_CHUNK * d + RC_CHUNK * RC_COLS + 3 * RC_CHUNK) * sizeof(float);
    if (pdtype == KB_F32)
        kb_launch(k_delta_rule<float>, grid, 32 * RC_COLS, sm, st, qkv, ldq, (const float*)proj, n_planes,
                  (size_t)plane_stride, ldp, ob, oa, a_log, dt_bias, H, G, d, dv, unit_eps, q_start, slot, state,
                  (size_t)state_stride, out, ldo);
    else
        kb_launch(k_delta_rule<bf16>, grid, 32 * RC_COLS, sm, st, qkv, ldq, (const bf16*)proj, n_planes,
                  (size_t)plane_stride, ldp, ob, oa, a_log, dt_bias, H, G, d, dv, unit_eps, q_start, slot, state,
                  (size_t)state_stride, out, ldo);
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ per-head norm + gate
// out[t][h n + e] = x[t][h n + e] / sqrt(mean_e x^2 + eps) * w[e] * gate(g[t][og + h n + e]); a warp per (row, head)
template <typename TG, typename TO>
__global__ void __launch_bounds__(128) k_head_norm_gate(const float* KB_STEP_DATA x, int ldx, int T, int H, int n,
        const float* __restrict__ w, float eps, const TG* KB_STEP_DATA g, int n_planes, size_t plane_stride, int ldg,
        int og, int gate_kind, TO* __restrict__ out, int ldo) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (item >= (long long)T * H) return;
    const size_t t = (size_t)(item / H);
    const int h = (int)(item % H);
    const float* xr = x + t * ldx + (size_t)h * n;
    float ss = 0.0f;
    for (int e = lane; e < n; e += 32) ss = fmaf(xr[e], xr[e], ss);
    ss = kb_warp_sum(ss);
    const float f = 1.0f / sqrtf(ss / (float)n + eps);
    for (int e = lane; e < n; e += 32) {
        float y = __fmul_rn(__fmul_rn(f, xr[e]), w[e]);
        if (g != nullptr)
            y *= rc_gate(rc_rd<TG>(g + t * ldg, n_planes, plane_stride, (size_t)og + (size_t)h * n + e), gate_kind);
        out[t * ldo + (size_t)h * n + e] = kb_from_f<TO>(y);
    }
}

extern "C" int kb_head_norm_gate(const float* x, int ldx, int T, int H, int n, const float* w, float eps,
                                 const void* g, int gdtype, int n_planes, long long plane_stride, int ldg, int og,
                                 int gate_kind, void* out, int odtype, int ldo, cudaStream_t st) {
    if (T <= 0 || H <= 0) return 0;
    const int grid = (int)(((long long)T * H + 3) / 4);
#define KB_HN(TG, TO)                                                                                              \
    kb_launch(k_head_norm_gate<TG, TO>, grid, 128, 0, st, x, ldx, T, H, n, w, eps, (const TG*)g, n_planes,        \
              (size_t)plane_stride, ldg, og, gate_kind, (TO*)out, ldo)
    if (gdtype == KB_F32 && odtype == KB_F32) KB_HN(float, float);
    else if (gdtype == KB_F32 && odtype == KB_BF16) KB_HN(float, bf16);
    else if (gdtype == KB_BF16 && odtype == KB_BF16) KB_HN(bf16, bf16);
    else return (int)cudaErrorInvalidValue;
#undef KB_HN
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ minGRU
// in: rows or planes with columns [oz: z | ox: x | og: g], W each; z = sigmoid(. + bz), u = . + bx, the candidate is
// u + 1/2 where u >= 0 and sigmoid(u) where u < 0; S <- (1 - z) S + z * candidate; out = S * silu(g). A thread per
// (sequence, element); four rows' inputs are fetched ahead of the dependent chain.
// Long prompts run in chunks of MG_CHUNK rows side by side (nc > 0, a thread per (sequence, chunk, element)), in two
// launches. The recurrence is linear in S, so a chunk is S_out = A S_in + L with A the product of its (1 - z) and L its
// state from zero: MODE 1 leaves (A, L) of every chunk but a sequence's last in `part` [B][nc][2][W]; MODE 2 folds the
// chunks before its own, in order, into the state its chunk starts from and then runs the chunk token by token, as
// MODE 0 (one chunk: the whole sequence) does.
#define MG_CHUNK 64
template <typename TIN, typename TO, int MODE>
__global__ void __launch_bounds__(128) k_min_gru(const TIN* KB_STEP_DATA in, int n_planes, size_t plane_stride,
        int ld_in, int oz, int ox, int og, int W, const float* __restrict__ bz, const float* __restrict__ bx,
        const int* __restrict__ q_start, const int* __restrict__ slot, float* state, size_t state_stride,
        TO* __restrict__ out, int ldo, float* part, int nc) {
    kb_pdl_launch();
    const int b = MODE == 0 ? blockIdx.y : blockIdx.z, ch = MODE == 0 ? 0 : blockIdx.y;
    const int c = blockIdx.x * 128 + threadIdx.x;
    const int s0 = q_start[b], s1 = q_start[b + 1];
    const int r0 = MODE == 0 ? s0 : s0 + ch * MG_CHUNK, r1 = MODE == 0 ? s1 : min(s1, r0 + MG_CHUNK);
    if (c >= W || r1 <= r0 || (MODE == 1 && r1 == s1)) {
        kb_pdl_wait();
        return;
    }
    const float vz = bz ? bz[c] : 0.0f, vx = bx ? bx[c] : 0.0f;
    float* sp = state + (size_t)slot[b] * state_stride + c;
    kb_pdl_wait();
    float S = 0.0f, A = 1.0f;
    if (MODE != 1) {
        S = *sp;
        const float* pp = part + (size_t)b * nc * 2 * W + c;
        for (int j = 0; j < ch; j++) S = fmaf(pp[(size_t)j * 2 * W], S, pp[(size_t)j * 2 * W + W]);
    }
    for (int r = r0; r < r1; r += 4) {
        float z[4], u[4], g[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int rr = r + k < r1 ? r + k : r1 - 1;
            const TIN* src = in + (size_t)rr * ld_in;
            z[k] = rc_rd<TIN>(src, n_planes, plane_stride, (size_t)oz + c);
            u[k] = rc_rd<TIN>(src, n_planes, plane_stride, (size_t)ox + c);
            if (MODE != 1) g[k] = rc_rd<TIN>(src, n_planes, plane_stride, (size_t)og + c);
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {
            if (r + k >= r1) break;
            const float zz = rc_sigmoid(z[k] + vz), uu = u[k] + vx;
            const float cand = uu >= 0.0f ? uu + 0.5f : rc_sigmoid(uu);
            S = fmaf(1.0f - zz, S, __fmul_rn(zz, cand));
            if (MODE == 1) A *= 1.0f - zz;
            else out[(size_t)(r + k) * ldo + c] = kb_from_f<TO>(S * rc_silu(g[k]));
        }
    }
    if (MODE == 1) {
        float* pp = part + ((size_t)b * nc + ch) * 2 * W + c;
        pp[0] = A;
        pp[W] = S;
    } else if (r1 == s1) {
        *sp = S;
    }
}

// nc > 0: every sequence's rows in nc chunks of MG_CHUNK (nc * MG_CHUNK >= the most rows of a sequence), `part` float
// scratch [B][nc][2][W]; nc == 0: a thread walks its sequence's rows alone
extern "C" int kb_min_gru(const void* in, int idtype, int n_planes, long long plane_stride, int ld_in, int oz, int ox,
                          int og, int W, const float* bz, const float* bx, int B, const int* q_start, const int* slot,
                          float* state, long long state_stride, void* out, int odtype, int ldo, float* part, int nc,
                          cudaStream_t st) {
    if (B <= 0 || W <= 0) return 0;
    if (nc > 65535 || B > 65535 || (nc > 0 && part == nullptr)) return (int)cudaErrorInvalidValue;
    dim3 grid((W + 127) / 128, B), gridc((W + 127) / 128, nc > 0 ? nc : 1, B);
#define KB_MG1(TIN, TO, MODE, GRID)                                                                                \
    kb_launch(k_min_gru<TIN, TO, MODE>, GRID, 128, 0, st, (const TIN*)in, n_planes, (size_t)plane_stride, ld_in,  \
              oz, ox, og, W, bz, bx, q_start, slot, state, (size_t)state_stride, (TO*)out, ldo, part, nc)
#define KB_MG(TIN, TO)                                                                                             \
    do {                                                                                                           \
        if (nc > 0) {                                                                                              \
            KB_MG1(TIN, TO, 1, gridc);                                                                             \
            KB_MG1(TIN, TO, 2, gridc);                                                                             \
        } else {                                                                                                   \
            KB_MG1(TIN, TO, 0, grid);                                                                              \
        }                                                                                                          \
    } while (0)
    if (idtype == KB_F32 && odtype == KB_F32) KB_MG(float, float);
    else if (idtype == KB_F32 && odtype == KB_BF16) KB_MG(float, bf16);
    else if (idtype == KB_BF16 && odtype == KB_BF16) KB_MG(bf16, bf16);
    else return (int)cudaErrorInvalidValue;
#undef KB_MG
#undef KB_MG1
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ mean of normed branches
// out[t][c] = (1 / n) sum_i v_i[t][c] / sqrt(mean_c v_i^2 + eps) * gain_i[c], v_i = (sum of branch i's planes) + bias_i
#define BN_MAX 4
struct KbBranches {
    const float* planes[BN_MAX];
    int n_planes[BN_MAX];
    long long plane_stride[BN_MAX];
    const float* bias[BN_MAX];
    const float* gain[BN_MAX];
};

__device__ __forceinline__ float bn_value(const KbBranches& br, int i, size_t at, int c) {
    float v = br.planes[i][at];
    for (int s = 1; s < br.n_planes[i]; s++) v += br.planes[i][(size_t)s * br.plane_stride[i] + at];
    return br.bias[i] ? v + br.bias[i][c] : v;
}

__global__ void __launch_bounds__(256) k_branch_norm_mean(KbBranches br, int n, float eps, float* __restrict__ out,
                                                          int E) {
    __shared__ float red[BN_MAX][8];
    kb_pdl_launch();
    kb_pdl_wait();
    const size_t t = blockIdx.x;
    float ss[BN_MAX];
    for (int i = 0; i < n; i++) {
        float a = 0.0f;
        for (int c = threadIdx.x; c < E; c += 256) {
            const float v = bn_value(br, i, t * E + c, c);
            a = fmaf(v, v, a);
        }
        a = kb_warp_sum(a);
        if ((threadIdx.x & 31) == 0) red[i][threadIdx.x >> 5] = a;
    }
    __syncthreads();
    for (int i = 0; i < n; i++) {
        float tot = 0.0f;
        for (int k = 0; k < 8; k++) tot += red[i][k];
        ss[i] = 1.0f / sqrtf(tot / (float)E + eps);
    }
    const float inv = 1.0f / (float)n;
    for (int c = threadIdx.x; c < E; c += 256) {
        float acc = 0.0f;
        for (int i = 0; i < n; i++)
            acc += __fmul_rn(__fmul_rn(ss[i], bn_value(br, i, t * E + c, c)), br.gain[i][c]);
        out[t * E + c] = acc * inv;
    }
}

extern "C" int kb_branch_norm_mean(int n, const float* const* planes, const int* n_planes,
                                   const long long* plane_stride, const float* const* bias, const float* const* gain,
                                   float eps, float* out, int T, int E, cudaStream_t st) {
    if (T <= 0) return 0;
    if (n < 1 || n > BN_MAX) return (int)cudaErrorInvalidValue;
    KbBranches br = {};
    for (int i = 0; i < n; i++) {
        br.planes[i] = planes[i];
        br.n_planes[i] = n_planes[i];
        br.plane_stride[i] = plane_stride[i];
        br.bias[i] = bias[i];
        br.gain[i] = gain[i];
    }
    kb_launch(k_branch_norm_mean, T, 256, 0, st, br, n, eps, out, E);
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ gated experts
// gu: sorted rows [n_pairs][2 F] = [gate | up] of every (row, pick) pair; w = the pick's weight (pair perm[r]);
// h[r][c] = act(w g) * (w u): the expert's input is the row times w, and the two products are linear in it
template <typename T>
__global__ void __launch_bounds__(256) k_moe_gate_mul(const T* KB_STEP_DATA gu, int ldgu, const float* KB_STEP_DATA wts,
        const int* KB_STEP_DATA perm, const int* KB_STEP_DATA n_rows_of, int F, int act, T* __restrict__ h, int ldh) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int c = blockIdx.y * 256 + threadIdx.x;
    if (c >= F) return;
    const size_t r = blockIdx.x;
    const float w = wts ? wts[perm[r]] : 1.0f;
    const float g = __fmul_rn(w, kb_to_f<T>(gu[r * ldgu + c])), u = __fmul_rn(w, kb_to_f<T>(gu[r * ldgu + F + c]));
    h[r * ldh + c] = kb_from_f<T>(kb_act(g, act) * u);
}

extern "C" int kb_moe_gate_mul(const void* gu, int dtype, int ldgu, const float* wts, const int* perm, int n_pairs,
                               int F, int act, void* h, int ldh, cudaStream_t st) {
    if (n_pairs <= 0 || F <= 0) return 0;
    dim3 grid(n_pairs, (F + 255) / 256);
    if (dtype == KB_F32)
        kb_launch(k_moe_gate_mul<float>, grid, 256, 0, st, (const float*)gu, ldgu, wts, perm, (const int*)nullptr, F,
                  act, (float*)h, ldh);
    else
        kb_launch(k_moe_gate_mul<bf16>, grid, 256, 0, st, (const bf16*)gu, ldgu, wts, perm, (const int*)nullptr, F, act,
                  (bf16*)h, ldh);
    KB_LAUNCH_RET();
}

// h[t][c] *= sigmoid(z[t * ldz]): one number per row gates the whole row
template <typename T>
__global__ void __launch_bounds__(256) k_row_gate(T* KB_STEP_DATA h, int ldh, const float* KB_STEP_DATA z, int ldz,
                                                  int N) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int c = blockIdx.y * 256 + threadIdx.x;
    if (c >= N) return;
    const size_t t = blockIdx.x;
    h[t * ldh + c] = kb_from_f<T>(kb_to_f<T>(h[t * ldh + c]) * rc_sigmoid(z[t * ldz]));
}

extern "C" int kb_row_gate(void* h, int dtype, int ldh, const float* z, int ldz, int T, int N, cudaStream_t st) {
    if (T <= 0 || N <= 0) return 0;
    dim3 grid(T, (N + 255) / 256);
    if (dtype == KB_F32) kb_launch(k_row_gate<float>, grid, 256, 0, st, (float*)h, ldh, z, ldz, N);
    else kb_launch(k_row_gate<bf16>, grid, 256, 0, st, (bf16*)h, ldh, z, ldz, N);
    KB_LAUNCH_RET();
}
