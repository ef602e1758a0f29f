// The gated delta rule over long prompts, a sequence's runs of DC_C tokens at a time (32-bit throughout).
//
// Token by token, per head with state S [d][dv]:  S <- g_t S;  u_t = beta_t (v_t - S^T k_t);  S <- S + k_t u_t^T;
// o_t = S^T q_t. Within a run that starts from S0, with G_t = g_0 ... g_t:
//     g_t S_(t-1) = G_t S0 + sum_(s<t) (G_t / G_s) k_s u_s^T
//     u_t = beta_t (v_t - G_t S0^T k_t) - sum_(s<t) A[t][s] u_s,      A[t][s] = beta_t (G_t / G_s) (k_t . k_s)
// so U = (I + A)^-1 R with R_t = beta_t (v_t - G_t S0^T k_t): the inverse of a unit lower-triangular DC_C x DC_C matrix
// that depends on keys, beta and decays only, not on the state. Then
//     o_t = G_t S0^T q_t + sum_(s<=t) P[t][s] u_s,                     P[t][s] = (G_t / G_s) (q_t . k_s)
//     S_end = G_last S0 + sum_s (G_last / G_s) k_s u_s^T.
// k_delta_prep works every (sequence, run, head) side by side: unit vectors, beta, the decays' running products (as sums
// of logarithms), A, its inverse by forward substitution (a thread per column) and P. k_delta_chunk then walks a
// sequence's runs in order, a block per (sequence, head, 16 or 32 columns of the state): five small products a run,
// every thread a few outputs, nothing passed between lanes. Rows past a sequence's end in its last run count as
// tokens with beta = 0, g = 1 and zero vectors: they change nothing and are not written.
#include "common.cuh"
#include <math.h>

#define DC_C 64
#define DC_THREADS 256

__device__ __forceinline__ float dc_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float dc_softplus(float z) { return log1pf(expf(-fabsf(z))) + fmaxf(z, 0.0f); }
template <typename TIN>
__device__ __forceinline__ float dc_rd(const TIN* src, int n_planes, size_t plane_stride, size_t i) {
    float v = kb_to_f<TIN>(src[i]);
    for (int s = 1; s < n_planes; s++) v += kb_to_f<TIN>(src[(size_t)s * plane_stride + i]);
    return v;
}

// scratch of one (sequence, run, head): T^-1 [C][C] | P [C][C] | beta [C] | G [C] | G_last / G [C]
#define DC_HEAD_FLOATS (2 * DC_C * DC_C + 3 * DC_C)

// grid (runs, H, B). qk: per (sequence, run, key head) the unit vectors k [C][dp] | q [C][dp], dp = d rounded up to 4
template <typename TIN>
__global__ void __launch_bounds__(DC_THREADS) k_delta_prep(const float* KB_STEP_DATA qkv, int ldq,
        const TIN* KB_STEP_DATA proj, int n_planes, size_t plane_stride, int ldp, int ob, int oa,
        const float* __restrict__ a_log, const float* __restrict__ dt_bias, int H, int G, int d, int dp, float unit_eps,
        const int* __restrict__ q_start, float* __restrict__ head_scratch, float* __restrict__ qk_scratch, int nc) {
    extern __shared__ __align__(16) float sm[];
    const int ld = dp + 4;                             // rows 16 bytes apart in the banks
    float* ks = sm;                                    // [C][ld]
    float* qs = ks + DC_C * ld;                        // [C][ld]
    float* As = qs + DC_C * ld;                        // [C][C + 1]
    float* Xs = As + DC_C * (DC_C + 1);                // [C][C + 1]
    float* bs = Xs + DC_C * (DC_C + 1);                // [C] beta
    float* lg = bs + DC_C;                             // [C] sum of log g up to and with t
    kb_pdl_launch();
    const int ci = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
    const int hg = h / (H / G);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int r0 = q_start[b] + ci * DC_C, r1 = min(q_start[b + 1], r0 + DC_C);
    const int n = r1 - r0;
    if (n <= 0) {
        kb_pdl_wait();
        return;
    }
    const float rate = expf(a_log[h]), dtb = dt_bias[h];
    const float qmul = 1.0f / sqrtf((float)d);
    kb_pdl_wait();
    const size_t oq = (size_t)hg * d, ok = (size_t)G * d + (size_t)hg * d;
    for (int idx = threadIdx.x; idx < DC_C * dp; idx += DC_THREADS) {
        const int t = idx / dp, j = idx % dp;
        const bool in = t < n && j < d;
        const float* src = qkv + (size_t)(r0 + t) * ldq;
        qs[t * ld + j] = in ? src[oq + j] : 0.0f;
        ks[t * ld + j] = in ? src[ok + j] : 0.0f;
    }
    if (threadIdx.x < DC_C) {
        const int t = threadIdx.x;
        float bv = 0.0f, l = 0.0f;
        if (t < n) {
            const TIN* src = proj + (size_t)(r0 + t) * ldp;
            bv = dc_sigmoid(dc_rd<TIN>(src, n_planes, plane_stride, (size_t)ob + h));
            l = -rate * dc_softplus(dc_rd<TIN>(src, n_planes, plane_stride, (size_t)oa + h) + dtb);
        }
        bs[t] = bv;
        lg[t] = l;
    }
    __syncthreads();
    // unit vectors (warp w: tokens w, w + 8, ...); the running sum of log g by one thread
    for (int t = warp; t < n; t += DC_THREADS / 32) {
        float sq = 0.0f, sk = 0.0f;
        for (int j = lane; j < d; j += 32) {
            sq = fmaf(qs[t * ld + j], qs[t * ld + j], sq);
            sk = fmaf(ks[t * ld + j], ks[t * ld + j], sk);
        }
        sq = kb_warp_sum(sq);
        sk = kb_warp_sum(sk);
        const float fq = qmul / sqrtf(sq + unit_eps), fk = 1.0f / sqrtf(sk + unit_eps);
        for (int j = lane; j < d; j += 32) {
            qs[t * ld + j] *= fq;
            ks[t * ld + j] *= fk;
        }
    }
    if (threadIdx.x == 0) {
        float acc = 0.0f;
        for (int t = 0; t < DC_C; t++) {
            acc += lg[t];
            lg[t] = acc;
        }
    }
    __syncthreads();
    float* hs = head_scratch + (((size_t)b * nc + ci) * H + h) * DC_HEAD_FLOATS;
    // k . k and q . k: thread (ty, tx) takes rows ty + 16 a against rows tx + 16 b
    {
        const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
        float kk[4][4], qk[4][4];
#pragma unroll
        for (int a = 0; a < 4; a++)
#pragma unroll
            for (int c = 0; c < 4; c++) kk[a][c] = qk[a][c] = 0.0f;
        for (int j = 0; j < dp; j += 4) {
            float4 kt[4], qt[4], kc[4];
#pragma unroll
            for (int a = 0; a < 4; a++) {
                kt[a] = *(const float4*)&ks[(ty + 16 * a) * ld + j];
                qt[a] = *(const float4*)&qs[(ty + 16 * a) * ld + j];
                kc[a] = *(const float4*)&ks[(tx + 16 * a) * ld + j];
            }
#pragma unroll
            for (int a = 0; a < 4; a++)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    kk[a][c] = fmaf(kt[a].x, kc[c].x, kk[a][c]);
                    kk[a][c] = fmaf(kt[a].y, kc[c].y, kk[a][c]);
                    kk[a][c] = fmaf(kt[a].z, kc[c].z, kk[a][c]);
                    kk[a][c] = fmaf(kt[a].w, kc[c].w, kk[a][c]);
                    qk[a][c] = fmaf(qt[a].x, kc[c].x, qk[a][c]);
                    qk[a][c] = fmaf(qt[a].y, kc[c].y, qk[a][c]);
                    qk[a][c] = fmaf(qt[a].z, kc[c].z, qk[a][c]);
                    qk[a][c] = fmaf(qt[a].w, kc[c].w, qk[a][c]);
                }
        }
        float* P = hs + DC_C * DC_C;
#pragma unroll
        for (int a = 0; a < 4; a++)
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const int t = ty + 16 * a, s = tx + 16 * c;
                const float ratio = s <= t ? expf(lg[t] - lg[s]) : 0.0f;
                As[t * (DC_C + 1) + s] = s < t ? bs[t] * ratio * kk[a][c] : 0.0f;
                P[t * DC_C + s] = ratio * qk[a][c];
            }
    }
    __syncthreads();
    // X = (I + A)^-1 by forward substitution, thread c its column c: X[t][c] = [t == c] - sum_(s<t) A[t][s] X[s][c]
    if (threadIdx.x < DC_C) {
        const int c = threadIdx.x;
        for (int t = 0; t < DC_C; t++) {
            float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
            const float* ar = As + t * (DC_C + 1);
            int s = 0;
            for (; s + 4 <= t; s += 4) {
                a0 = fmaf(ar[s], Xs[s * (DC_C + 1) + c], a0);
                a1 = fmaf(ar[s + 1], Xs[(s + 1) * (DC_C + 1) + c], a1);
                a2 = fmaf(ar[s + 2], Xs[(s + 2) * (DC_C + 1) + c], a2);
                a3 = fmaf(ar[s + 3], Xs[(s + 3) * (DC_C + 1) + c], a3);
            }
            for (; s < t; s++) a0 = fmaf(ar[s], Xs[s * (DC_C + 1) + c], a0);
            Xs[t * (DC_C + 1) + c] = (t == c ? 1.0f : 0.0f) - ((a0 + a1) + (a2 + a3));
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < DC_C * DC_C; idx += DC_THREADS)
        hs[idx] = Xs[(idx / DC_C) * (DC_C + 1) + idx % DC_C];
    if (threadIdx.x < DC_C) {
        const int t = threadIdx.x;
        float* vec = hs + 2 * DC_C * DC_C;
        vec[t] = bs[t];
        vec[DC_C + t] = expf(lg[t]);
        vec[2 * DC_C + t] = expf(lg[DC_C - 1] - lg[t]);
    }
    if (h % (H / G) == 0) {
        float* dst = qk_scratch + ((size_t)b * nc + ci) * G * 2 * DC_C * dp + (size_t)hg * 2 * DC_C * dp;
        for (int idx = threadIdx.x; idx < DC_C * dp; idx += DC_THREADS) {
            const int t = idx / dp, j = idx % dp;
            dst[idx] = ks[t * ld + j];
            dst[DC_C * dp + idx] = qs[t * ld + j];
        }
    }
}

// grid (B * H, ceil(dv / COLS)), DC_TB threads: thread (ty, tx) works column tx and the tokens (or state rows)
// ty + NTY a. state per head [dv][d]. The staging loads of a run are all in flight before the first store.
#define DC_TB 512
template <int COLS>
__global__ void __launch_bounds__(DC_TB) k_delta_chunk(const float* KB_STEP_DATA qkv, int ldq, int H, int G, int d,
        int dp, int dv, const int* __restrict__ q_start, const int* __restrict__ slot, float* state, size_t state_stride,
        const float* KB_STEP_DATA head_scratch, const float* KB_STEP_DATA qk_scratch, int nc, float* __restrict__ out,
        int ldo) {
    constexpr int NTY = DC_TB / COLS, NA = DC_C / NTY;         // 32 x 2 at 16 columns, 16 x 4 at 32
    extern __shared__ __align__(16) float sm[];
    const int ld = dp + 4;
    float* ks = sm;                                    // [C][ld]
    float* qs = ks + DC_C * ld;                        // [C][ld]
    float* Ts = qs + DC_C * ld;                        // [C][C]
    float* Ps = Ts + DC_C * DC_C;                      // [C][C]
    float* vec = Ps + DC_C * DC_C;                     // beta | G | G_last / G
    float* Ss = vec + 3 * DC_C;                        // [dp][COLS]
    float* Rs = Ss + dp * COLS;                        // [C][COLS]: v, then R
    float* Us = Rs + DC_C * COLS;                      // [C][COLS]
    float* Zs = Us + DC_C * COLS;                      // [C][COLS]: G_t S0^T q_t
    kb_pdl_launch();
    const int b = blockIdx.x / H, h = blockIdx.x % H, hg = h / (H / G);
    const int e0 = blockIdx.y * COLS;
    const int ty = threadIdx.x / COLS, tx = threadIdx.x % COLS;
    const int s0 = q_start[b], s1 = q_start[b + 1];
    float* sbase = state + (size_t)slot[b] * state_stride + (size_t)h * dv * d;
    kb_pdl_wait();
    if (s1 <= s0) return;
    for (int idx = threadIdx.x; idx < dp * COLS; idx += DC_TB) {
        const int c = idx / dp, j = idx % dp;          // (a column's d elements lie together in the state)
        Ss[j * COLS + c] = (e0 + c < dv && j < d) ? sbase[(size_t)(e0 + c) * d + j] : 0.0f;
    }
    const size_t ov = (size_t)2 * G * d + (size_t)h * dv;
    const int n_runs = (s1 - s0 + DC_C - 1) / DC_C;
    const int n_kq = DC_C * dp;                        // floats of a run's keys (and of its queries)
    for (int ci = 0; ci < n_runs; ci++) {
        const int r0 = s0 + ci * DC_C, n = min(DC_C, s1 - r0);
        const float* hs = head_scratch + (((size_t)b * nc + ci) * H + h) * DC_HEAD_FLOATS;
        const float* kq = qk_scratch + ((size_t)b * nc + ci) * G * 2 * DC_C * dp + (size_t)hg * 2 * DC_C * dp;
        __syncthreads();                               // the run before is done with the tiles
        {
            // keys and queries: up to 2 x 64 x 256 floats = 16 float4 a thread; T^-1, P and the vectors (which lie in
            // this order in the scratch and in shared memory): 8384 floats = 5 float4 a thread
            float4 kv4[8], qv4[8], hv4[5];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int idx = (threadIdx.x + i * DC_TB) * 4;
                if (idx < n_kq) {
                    kv4[i] = *(const float4*)&kq[idx];
                    qv4[i] = *(const float4*)&kq[n_kq + idx];
                }
            }
#pragma unroll
            for (int i = 0; i < 5; i++) {
                const int idx = (threadIdx.x + i * DC_TB) * 4;
                if (idx < DC_HEAD_FLOATS) hv4[i] = *(const float4*)&hs[idx];
            }
            float vv[NA];
#pragma unroll
            for (int a = 0; a < NA; a++) {
                const int t = ty + NTY * a;
                vv[a] = (t < n && e0 + tx < dv) ? qkv[(size_t)(r0 + t) * ldq + ov + e0 + tx] : 0.0f;
            }
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const int idx = (threadIdx.x + i * DC_TB) * 4;
                if (idx < n_kq) {
                    const int t = idx / dp, j = idx % dp;
                    *(float4*)&ks[t * ld + j] = kv4[i];
                    *(float4*)&qs[t * ld + j] = qv4[i];
                }
            }
#pragma unroll
            for (int i = 0; i < 5; i++) {
                const int idx = (threadIdx.x + i * DC_TB) * 4;
                if (idx < DC_HEAD_FLOATS) *(float4*)&Ts[idx] = hv4[i];
            }
#pragma unroll
            for (int a = 0; a < NA; a++) Rs[(ty + NTY * a) * COLS + tx] = vv[a];
        }
        __syncthreads();
        // W = K S0, Z = Q S0
        {
            float w[NA], z[NA];
#pragma unroll
            for (int a = 0; a < NA; a++) w[a] = z[a] = 0.0f;
#pragma unroll 2
            for (int j = 0; j < dp; j += 4) {
                const float c0 = Ss[j * COLS + tx], c1 = Ss[(j + 1) * COLS + tx];
                const float c2 = Ss[(j + 2) * COLS + tx], c3 = Ss[(j + 3) * COLS + tx];
#pragma unroll
                for (int a = 0; a < NA; a++) {
                    const float4 kv = *(const float4*)&ks[(ty + NTY * a) * ld + j];
                    const float4 qv = *(const float4*)&qs[(ty + NTY * a) * ld + j];
                    w[a] = fmaf(kv.x, c0, w[a]);
                    w[a] = fmaf(kv.y, c1, w[a]);
                    w[a] = fmaf(kv.z, c2, w[a]);
                    w[a] = fmaf(kv.w, c3, w[a]);
                    z[a] = fmaf(qv.x, c0, z[a]);
                    z[a] = fmaf(qv.y, c1, z[a]);
                    z[a] = fmaf(qv.z, c2, z[a]);
                    z[a] = fmaf(qv.w, c3, z[a]);
                }
            }
#pragma unroll
            for (int a = 0; a < NA; a++) {
                const int t = ty + NTY * a;
                const float gt = vec[DC_C + t];
                Rs[t * COLS + tx] = vec[t] * (Rs[t * COLS + tx] - gt * w[a]);
                Zs[t * COLS + tx] = gt * z[a];
            }
        }
        __syncthreads();
        // U = T^-1 R (T^-1 and P are lower triangular: row t ends at column t), four columns of a row a load
        const int s_end = min(DC_C, (ty + NTY * (NA - 1) + 4) & ~3);
        {
            float u[NA];
#pragma unroll
            for (int a = 0; a < NA; a++) u[a] = 0.0f;
#pragma unroll 2
            for (int s = 0; s < s_end; s += 4) {
                const float r0v = Rs[s * COLS + tx], r1v = Rs[(s + 1) * COLS + tx];
                const float r2v = Rs[(s + 2) * COLS + tx], r3v = Rs[(s + 3) * COLS + tx];
#pragma unroll
                for (int a = 0; a < NA; a++) {
                    const float4 tv = *(const float4*)&Ts[(ty + NTY * a) * DC_C + s];
                    u[a] = fmaf(tv.x, r0v, u[a]);
                    u[a] = fmaf(tv.y, r1v, u[a]);
                    u[a] = fmaf(tv.z, r2v, u[a]);
                    u[a] = fmaf(tv.w, r3v, u[a]);
                }
            }
#pragma unroll
            for (int a = 0; a < NA; a++) Us[(ty + NTY * a) * COLS + tx] = u[a];
        }
        __syncthreads();
        // o = Z + P U; R is done with: its place takes u_s (G_last / G_s) for the state's update
        {
            float o[NA];
#pragma unroll
            for (int a = 0; a < NA; a++) {
                const int t = ty + NTY * a;
                o[a] = Zs[t * COLS + tx];
                Rs[t * COLS + tx] = Us[t * COLS + tx] * vec[2 * DC_C + t];
            }
#pragma unroll 2
            for (int s = 0; s < s_end; s += 4) {
                const float u0 = Us[s * COLS + tx], u1 = Us[(s + 1) * COLS + tx];
                const float u2 = Us[(s + 2) * COLS + tx], u3 = Us[(s + 3) * COLS + tx];
#pragma unroll
                for (int a = 0; a < NA; a++) {
                    const float4 pv = *(const float4*)&Ps[(ty + NTY * a) * DC_C + s];
                    o[a] = fmaf(pv.x, u0, o[a]);
                    o[a] = fmaf(pv.y, u1, o[a]);
                    o[a] = fmaf(pv.z, u2, o[a]);
                    o[a] = fmaf(pv.w, u3, o[a]);
                }
            }
#pragma unroll
            for (int a = 0; a < NA; a++) {
                const int t = ty + NTY * a;
                if (t < n && e0 + tx < dv) out[(size_t)(r0 + t) * ldo + (size_t)h * dv + e0 + tx] = o[a];
            }
        }
        __syncthreads();
        // S <- G_last S + sum_s k_s (u_s G_last / G_s)^T: thread (ty, tx) takes four neighbouring rows of column tx
        {
            const float gl = vec[DC_C + DC_C - 1];
            for (int j = 4 * ty; j < dp; j += 4 * NTY) {
                float a0 = 0.0f, a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
#pragma unroll 4
                for (int s = 0; s < DC_C; s++) {
                    const float uv = Rs[s * COLS + tx];
                    const float4 kv = *(const float4*)&ks[s * ld + j];
                    a0 = fmaf(kv.x, uv, a0);
                    a1 = fmaf(kv.y, uv, a1);
                    a2 = fmaf(kv.z, uv, a2);
                    a3 = fmaf(kv.w, uv, a3);
                }
                Ss[j * COLS + tx] = fmaf(gl, Ss[j * COLS + tx], a0);
                Ss[(j + 1) * COLS + tx] = fmaf(gl, Ss[(j + 1) * COLS + tx], a1);
                Ss[(j + 2) * COLS + tx] = fmaf(gl, Ss[(j + 2) * COLS + tx], a2);
                Ss[(j + 3) * COLS + tx] = fmaf(gl, Ss[(j + 3) * COLS + tx], a3);
            }
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < dp * COLS; idx += DC_TB) {
        const int c = idx / dp, j = idx % dp;
        if (e0 + c < dv && j < d) sbase[(size_t)(e0 + c) * d + j] = Ss[j * COLS + c];
    }
}

static int dc_sm_count() {
    static int n = 0;
    if (n == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

// head_scratch: B * nc * H * DC_HEAD_FLOATS floats; qk_scratch: B * nc * G * 2 * DC_C * dp floats, dp = d rounded up to a
// multiple of 4; nc runs of DC_C rows cover the longest sequence's rows of this step
extern "C" int kb_delta_chunked(const float* qkv, int ldq, const void* proj, int pdtype, int n_planes,
                                long long plane_stride, int ldp, int ob, int oa, const float* a_log,
                                const float* dt_bias, int B, int H, int G, int d, int dv, float unit_eps,
                                const int* q_start, const int* slot, float* state, long long state_stride,
                                float* head_scratch, float* qk_scratch, int nc, float* out, int ldo, cudaStream_t st) {
    if (B <= 0 || nc <= 0) return 0;
    if (d > 256 || G <= 0 || H % G || nc > 65535 || B > 65535 || H > 65535) return (int)cudaErrorInvalidValue;
    const int dp = (d + 3) / 4 * 4, ld = dp + 4;
    const size_t sm_a = (size_t)(2 * DC_C * ld + 2 * DC_C * (DC_C + 1) + 2 * DC_C) * sizeof(float);
    // 16 columns of the state a block; 32 when that would be more blocks than SMs (a block fills an SM)
    const int cols = (long long)B * H * ((dv + 15) / 16) > dc_sm_count() ? 32 : 16;
    const size_t sm_b = (size_t)(2 * DC_C * ld + 2 * DC_C * DC_C + 3 * DC_C + dp * cols + 3 * DC_C * cols) * sizeof(float);
    static char tag_a32, tag_a16, tag_b16, tag_b32;
    if (kb_first_use(pdtype == KB_F32 ? &tag_a32 : &tag_a16)) {
        cudaError_t e = pdtype == KB_F32
            ? cudaFuncSetAttribute(k_delta_prep<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024)
            : cudaFuncSetAttribute(k_delta_prep<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    if (kb_first_use(cols == 16 ? &tag_b16 : &tag_b32)) {
        cudaError_t e = cols == 16
            ? cudaFuncSetAttribute(k_delta_chunk<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024)
            : cudaFuncSetAttribute(k_delta_chunk<32>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        if (e != cudaSuccess) return (int)e;
    }
    dim3 grid_a(nc, H, B);
    if (pdtype == KB_F32)
        kb_launch(k_delta_prep<float>, grid_a, DC_THREADS, sm_a, st, qkv, ldq, (const float*)proj, n_planes,
                  (size_t)plane_stride, ldp, ob, oa, a_log, dt_bias, H, G, d, dp, unit_eps, q_start, head_scratch,
                  qk_scratch, nc);
    else
        kb_launch(k_delta_prep<bf16>, grid_a, DC_THREADS, sm_a, st, qkv, ldq, (const bf16*)proj, n_planes,
                  (size_t)plane_stride, ldp, ob, oa, a_log, dt_bias, H, G, d, dp, unit_eps, q_start, head_scratch,
                  qk_scratch, nc);
    dim3 grid_b(B * H, (dv + cols - 1) / cols);
    if (cols == 16)
        kb_launch(k_delta_chunk<16>, grid_b, DC_TB, sm_b, st, qkv, ldq, H, G, d, dp, dv, q_start, slot, state,
                  (size_t)state_stride, (const float*)head_scratch, (const float*)qk_scratch, nc, out, ldo);
    else
        kb_launch(k_delta_chunk<32>, grid_b, DC_TB, sm_b, st, qkv, ldq, H, G, d, dp, dv, q_start, slot, state,
                  (size_t)state_stride, (const float*)head_scratch, (const float*)qk_scratch, nc, out, ldo);
    KB_LAUNCH_RET();
}
