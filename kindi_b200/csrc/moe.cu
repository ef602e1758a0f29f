// Mixture of experts: the pick of each row's experts, the plan that sorts (row, pick) pairs by expert, and the two
// grouped products of the general (fixed-order, 32-bit accumulate) path.
//
// k_moe_topk: z = logits + bias (32-bit); the `top` largest of a row's E values are taken one after the other (of
// equal values the one with the lower index first); their weights are the softmax over the chosen values only.
// Pair p = row * top + k names the k-th pick of a row.
//
// k_moe_plan (one block): counts the pairs of every expert, lays the experts' pairs one after another
// (offs[e]..offs[e + 1]), lists the pairs in that order (perm) and cuts every expert's stretch into tiles of `tile`
// rows (tile_e, tile_r0; n_tiles[0] tiles in all). Products then run over tiles; a tile belongs to one expert.
// Which place a pair gets inside its expert's stretch depends on the order in which threads arrive, but a pair's
// result does not depend on its place.
//
// k_moe_gemm: C[r][n] = sum_k A[r][k] * W[e][n][k] for every sorted row r of every tile, k in order with 32-bit fused
// multiply-adds. Up form: A's row is the row of the pair's token (gathered through perm), the activation is applied
// and C is the sorted intermediate. Down form: A is the sorted intermediate, the result is multiplied by the pair's
// weight and written to plane k of the pair's token, so that the planes' sum in order is the weighted sum of the
// chosen experts (the next norm adds the planes).
#include "common.cuh"
#include <math.h>

#define MOE_MAX_TOP 32
#define MOE_SCORE_SOFTMAX 0
#define MOE_SCORE_SIGMOID 1

__global__ void __launch_bounds__(128) k_moe_topk(const float* KB_STEP_DATA logits, int ldz,
        const float* __restrict__ bias, int T, int E, int top, int* __restrict__ idx, float* __restrict__ wts,
        int score) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= T) return;
    const float* z = logits + (size_t)t * ldz;
    int chosen[MOE_MAX_TOP];
    float val[MOE_MAX_TOP];
    for (int k = 0; k < top; k++) {
        int best = -1;
        float bv = 0.0f;
        for (int e = 0; e < E; e++) {
            bool taken = false;
            for (int j = 0; j < k; j++) taken |= chosen[j] == e;
            if (taken) continue;
            const float v = z[e] + (bias ? bias[e] : 0.0f);
            if (best < 0 || v > bv) {
                best = e;
                bv = v;
            }
        }
        chosen[k] = best;
        val[k] = bv;
    }
    if (score == MOE_SCORE_SIGMOID) {
        // every chosen expert keeps its own sigmoid(z); nothing is normalised over the chosen ones
        for (int k = 0; k < top; k++) {
            idx[(size_t)t * top + k] = chosen[k];
            wts[(size_t)t * top + k] = 1.0f / (1.0f + expf(-val[k]));
        }
        return;
    }
    float mx = val[0];
    for (int k = 1; k < top; k++) mx = fmaxf(mx, val[k]);
    float sum = 0.0f;
    for (int k = 0; k < top; k++) {
        val[k] = expf(val[k] - mx);
        sum += val[k];
    }
    for (int k = 0; k < top; k++) {
        idx[(size_t)t * top + k] = chosen[k];
        wts[(size_t)t * top + k] = val[k] / sum;
    }
}

// The same pick with a warp per row, for up to 32 * MOE_PER experts: lane l holds the values of experts l, l + 32, ...
// in registers; each of the `top` rounds takes the largest value not yet taken (of equal values the lower index), found
// by a lane-local scan and five shuffle steps. The chosen values and their softmax are the same bits as k_moe_topk's.
#define MOE_PER 8
__global__ void __launch_bounds__(128) k_moe_topk_warp(const float* KB_STEP_DATA logits, int ldz,
        const float* __restrict__ bias, int T, int E, int top, int* __restrict__ idx, float* __restrict__ wts,
        int score) {
    kb_pdl_launch();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
    float b[MOE_PER];
#pragma unroll
    for (int j = 0; j < MOE_PER; j++) b[j] = (bias && lane + 32 * j < E) ? bias[lane + 32 * j] : 0.0f;
    kb_pdl_wait();
    if (t >= T) return;
    const float* z = logits + (size_t)t * ldz;
    float v[MOE_PER];
    bool free_[MOE_PER];
#pragma unroll
    for (int j = 0; j < MOE_PER; j++) {
        const int e = lane + 32 * j;
        free_[j] = e < E;
        v[j] = free_[j] ? z[e] + b[j] : 0.0f;
    }
    float my_val = 0.0f, mx = 0.0f, sum = 0.0f;          // lane k keeps the k-th chosen value
    int my_idx = 0;
    for (int k = 0; k < top; k++) {
        // the lane's best free entry; "none" = index E (loses against every real entry)
        int be = E;
        float bv = 0.0f;
#pragma unroll
        for (int j = 0; j < MOE_PER; j++) {
            const int e = lane + 32 * j;
            if (free_[j] && (be == E || v[j] > bv)) {
                be = e;
                bv = v[j];
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            // the other wins when it is a real entry and (this is none, or it is larger, or equal with a lower index)
            if (oe < E && (be == E || ov > bv || (ov == bv && oe < be) || (bv != bv && oe < be))) {
                bv = ov;
                be = oe;
            }
        }
#pragma unroll
        for (int j = 0; j < MOE_PER; j++)
            if (lane + 32 * j == be) free_[j] = false;
        if (lane == k) {
            my_val = bv;
            my_idx = be;
        }
        mx = k == 0 ? bv : fmaxf(mx, bv);
    }
    // softmax over the chosen values, summed in the order they were chosen
    const float ex = lane < top ? expf(my_val - mx) : 0.0f;
    for (int k = 0; k < top; k++) sum += __shfl_sync(0xffffffffu, ex, k);
    if (lane < top) {
        idx[(size_t)t * top + lane] = my_idx < E ? my_idx : 0;
        wts[(size_t)t * top + lane] = score == MOE_SCORE_SIGMOID ? 1.0f / (1.0f + expf(-my_val)) : ex / sum;
    }
}

extern "C" int kb_moe_topk(const float* logits, int ldz, const float* bias, int T, int E, int top, int* idx,
                           float* wts, cudaStream_t st, int score) {
    // score: MOE_SCORE_SOFTMAX (weights = softmax over the chosen values) or MOE_SCORE_SIGMOID (weights = sigmoid of
    // each chosen value, not normalised; the order of the values is the order of their sigmoids)
    if (T <= 0) return 0;
    if (top < 1 || top > MOE_MAX_TOP || top > E) return (int)cudaErrorInvalidValue;
    if (E <= 32 * MOE_PER)
        kb_launch(k_moe_topk_warp, (T + 3) / 4, 128, 0, st, logits, ldz, bias, T, E, top, idx, wts, score);
    else
        kb_launch(k_moe_topk, (T + 127) / 128, 128, 0, st, logits, ldz, bias, T, E, top, idx, wts, score);
    KB_LAUNCH_RET();
}

// The pick of a router whose scores are the softmax over ALL its outputs: s = softmax(z) over n outputs, choice scores
// c = s + correction; the outputs form `groups` equal groups of neighbours, a group's score is its largest c, and only
// outputs of the `keep` best groups can be chosen (groups == 1: all); the `top` largest c among those are taken one
// after the other (of equal values the lower index first); the weights are the chosen outputs' s over their sum
// (+ 1e-20). One warp per row, lane l holding outputs l, l + 32, ... (up to 32 * MOE_PER outputs, up to 32 groups).
// Outputs from n_experts on are "identity experts" of the caller: the pick treats them like any other.
__global__ void __launch_bounds__(128) k_moe_route_warp(const float* KB_STEP_DATA logits, int ldz,
        const float* __restrict__ correction, int T, int n, int top, int groups, int keep, int* __restrict__ idx,
        float* __restrict__ wts) {
    kb_pdl_launch();
    const int lane = threadIdx.x & 31;
    const int t = blockIdx.x * 4 + (threadIdx.x >> 5);
    float b[MOE_PER];
#pragma unroll
    for (int j = 0; j < MOE_PER; j++) b[j] = (correction && lane + 32 * j < n) ? correction[lane + 32 * j] : 0.0f;
    kb_pdl_wait();
    if (t >= T) return;
    const float* z = logits + (size_t)t * ldz;
    float s[MOE_PER], v[MOE_PER];
    bool free_[MOE_PER];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < MOE_PER; j++) {
        const int e = lane + 32 * j;
        free_[j] = e < n;
        s[j] = free_[j] ? z[e] : -INFINITY;
        mx = fmaxf(mx, s[j]);
    }
    mx = kb_warp_max(mx);
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < MOE_PER; j++) {
        s[j] = free_[j] ? expf(s[j] - mx) : 0.0f;
        sum += s[j];
    }
    sum = kb_warp_sum(sum);
#pragma unroll
    for (int j = 0; j < MOE_PER; j++) {
        s[j] = s[j] / sum;
        v[j] = s[j] + b[j];
    }
    if (groups > 1) {
        // lane g keeps group g's score; then `keep` rounds take the best group not yet taken
        const int size = n / groups;
        float gs = 0.0f;
        for (int g = 0; g < groups; g++) {
            float m = -INFINITY;
#pragma unroll
            for (int j = 0; j < MOE_PER; j++)
                if (free_[j] && (lane + 32 * j) / size == g) m = fmaxf(m, v[j]);
            m = kb_warp_max(m);
            if (lane == g) gs = m;
        }
        bool gfree = lane < groups;
        unsigned kept = 0u;
        for (int k = 0; k < keep; k++) {
            float bv = gs;
            int bg = gfree ? lane : 32;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const int og = __shfl_xor_sync(0xffffffffu, bg, o);
                if (og < 32 && (bg == 32 || ov > bv || (ov == bv && og < bg) || (bv != bv && og < bg))) {
                    bv = ov;
                    bg = og;
                }
            }
            if (bg < 32) kept |= 1u << bg;
            if (lane == bg) gfree = false;
        }
#pragma unroll
        for (int j = 0; j < MOE_PER; j++)
            if (free_[j] && !((kept >> ((lane + 32 * j) / size)) & 1u)) free_[j] = false;
    }
    float my_s = 0.0f;
    int my_idx = 0;
    for (int k = 0; k < top; k++) {
        int be = n;
        float bv = 0.0f, bs = 0.0f;
#pragma unroll
        for (int j = 0; j < MOE_PER; j++) {
            const int e = lane + 32 * j;
            if (free_[j] && (be == n || v[j] > bv)) {
                be = e;
                bv = v[j];
                bs = s[j];
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const float os = __shfl_xor_sync(0xffffffffu, bs, o);
            const int oe = __shfl_xor_sync(0xffffffffu, be, o);
            if (oe < n && (be == n || ov > bv || (ov == bv && oe < be) || (bv != bv && oe < be))) {
                bv = ov;
                bs = os;
                be = oe;
            }
        }
#pragma unroll
        for (int j = 0; j < MOE_PER; j++)
            if (lane + 32 * j == be) free_[j] = false;
        if (lane == k) {
            my_s = bs;
            my_idx = be;
        }
    }
    float tot = 0.0f;                               // summed in the order they were chosen
    for (int k = 0; k < top; k++) tot += __shfl_sync(0xffffffffu, my_s, k);
    if (lane < top) {
        // (fewer free outputs than `top`: the kept groups are too small; the pick names no expert and weighs nothing)
        idx[(size_t)t * top + lane] = my_idx < n ? my_idx : -1;
        wts[(size_t)t * top + lane] = my_idx < n ? my_s / (tot + 1e-20f) : 0.0f;
    }
}

extern "C" int kb_moe_route(const float* logits, int ldz, const float* correction, int T, int n, int top, int groups,
                            int keep, int* idx, float* wts, cudaStream_t st) {
    if (T <= 0) return 0;
    if (top < 1 || top > 32 || top > n || n > 32 * MOE_PER || groups < 1 || groups > 32 || n % groups || keep < 1 ||
        keep > groups)
        return (int)cudaErrorInvalidValue;
    kb_launch(k_moe_route_warp, (T + 3) / 4, 128, 0, st, logits, ldz, correction, T, n, top, groups, keep, idx, wts);
    KB_LAUNCH_RET();
}

// Picks that name an "identity expert" (an index from n_experts on) have no product: plane k of the pair's token is
// the pick's weight times the expert's input row itself. Picks below n_experts are left to the grouped products;
// a pick that names nothing (-1) gets zeros.
template <typename TY>
__global__ void __launch_bounds__(256) k_moe_identity(const TY* KB_STEP_DATA y, int ldy, const int* KB_STEP_DATA idx,
        const float* KB_STEP_DATA wts, float* planes, size_t plane_stride, int n_pairs, int top, int n_experts,
        int width) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int pair = blockIdx.x;
    const int e = idx[pair];
    if (e >= 0 && e < n_experts) return;
    const float w = e < 0 ? 0.0f : wts[pair];
    const size_t t = pair / top;
    float* dst = planes + (size_t)(pair % top) * plane_stride + t * width;
    for (int c = threadIdx.x; c < width; c += 256) dst[c] = e < 0 ? 0.0f : __fmul_rn(w, kb_to_f<TY>(y[t * ldy + c]));
}

extern "C" int kb_moe_identity(const void* y, int ydtype, int ldy, const int* idx, const float* wts, float* planes,
                               long long plane_stride, int n_pairs, int top, int n_experts, int width,
                               cudaStream_t st) {
    if (n_pairs <= 0) return 0;
    if (ydtype == KB_F32)
        kb_launch(k_moe_identity<float>, n_pairs, 256, 0, st, (const float*)y, ldy, idx, wts, planes,
                  (size_t)plane_stride, n_pairs, top, n_experts, width);
    else if (ydtype == KB_BF16)
        kb_launch(k_moe_identity<bf16>, n_pairs, 256, 0, st, (const bf16*)y, ldy, idx, wts, planes,
                  (size_t)plane_stride, n_pairs, top, n_experts, width);
    else return (int)cudaErrorInvalidValue;
    KB_LAUNCH_RET();
}

#define MOE_PLAN_THREADS 1024
// shared: counts[E], cursor[E]
__global__ void __launch_bounds__(MOE_PLAN_THREADS) k_moe_plan(const int* KB_STEP_DATA idx, int n_pairs, int E,
        int tile, int* __restrict__ offs, int* __restrict__ perm, int* __restrict__ tile_e,
        int* __restrict__ tile_r0, int* __restrict__ n_tiles) {
    extern __shared__ int sh[];
    __shared__ int s_total;
    int* counts = sh;
    int* cursor = sh + E;
    kb_pdl_launch();
    for (int e = threadIdx.x; e < E; e += MOE_PLAN_THREADS) counts[e] = 0;
    __syncthreads();
    kb_pdl_wait();
    for (int p = threadIdx.x; p < n_pairs; p += MOE_PLAN_THREADS) {
        const int e = idx[p];
        if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, nt = 0;
        for (int e = 0; e < E; e++) {
            offs[e] = at;
            cursor[e] = at;
            for (int r = 0; r < counts[e]; r += tile) {
                tile_e[nt] = e;
                tile_r0[nt] = at + r;
                nt++;
            }
            at += counts[e];
        }
        offs[E] = at;
        n_tiles[0] = nt;
        s_total = at;
    }
    __syncthreads();
    for (int p = threadIdx.x; p < n_pairs; p += MOE_PLAN_THREADS) {
        const int e = idx[p];
        if (e >= 0 && e < E) perm[atomicAdd(&cursor[e], 1)] = p;
    }
    // pairs that name no expert of these products (an index outside 0..E-1) have no place in the order: the rest of
    // the list names pair 0, so that a kernel that walks all n_pairs entries reads a row that exists
    for (int p = s_total + threadIdx.x; p < n_pairs; p += MOE_PLAN_THREADS) perm[p] = 0;
}

extern "C" int kb_moe_plan(const int* idx, int n_pairs, int E, int tile, int* offs, int* perm, int* tile_e,
                           int* tile_r0, int* n_tiles, cudaStream_t st) {
    if (n_pairs <= 0) return 0;
    if (E < 1 || E > 4096 || tile < 1) return (int)cudaErrorInvalidValue;
    kb_launch(k_moe_plan, 1, MOE_PLAN_THREADS, (size_t)2 * E * sizeof(int), st, idx, n_pairs, E, tile, offs, perm,
              tile_e, tile_r0, n_tiles);
    KB_LAUNCH_RET();
}

#define MG_BM 64
#define MG_BN 64
#define MG_BK 32
// UP: A rows are gathered (token of the pair), C = act(A W^T) at the sorted row. !UP: A rows are the sorted rows,
// C = weight of the pair * (A W^T) at plane (pair % top), row (pair / top).
template <typename TA, typename TW, typename TC, bool UP>
__global__ void __launch_bounds__(256) k_moe_gemm(const TA* KB_STEP_DATA A, int lda, const TW* __restrict__ W,
        TC* __restrict__ C, int ldc, size_t plane_stride, int N, int K, const int* KB_STEP_DATA n_tiles,
        const int* KB_STEP_DATA tile_e, const int* KB_STEP_DATA tile_r0, const int* KB_STEP_DATA offs,
        const int* KB_STEP_DATA perm, const float* KB_STEP_DATA wts, int top, int act) {
    __shared__ float As[MG_BK][MG_BM + 1];
    __shared__ float Ws[MG_BK][MG_BN + 1];
    __shared__ int arow[MG_BM];                      // UP: the token's row of A; else the pair
    kb_pdl_launch();
    kb_pdl_wait();
    if ((int)blockIdx.y >= n_tiles[0]) return;
    const int e = tile_e[blockIdx.y], r0 = tile_r0[blockIdx.y];
    const int r_end = min(offs[e + 1], r0 + MG_BM);
    const int n0 = blockIdx.x * MG_BN;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    if (tid < MG_BM) {
        const int r = r0 + tid;
        int v = -1;
        if (r < r_end) v = UP ? perm[r] / top : perm[r];
        arow[tid] = v;
    }
    __syncthreads();
    const TW* We = W + (size_t)e * N * K;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.0f;
    constexpr int PER = MG_BM * MG_BK / 256;
    float ra[PER], rw[PER];
    auto fetch = [&](int k0) {
#pragma unroll
        for (int j = 0; j < PER; j++) {
            const int el = tid + 256 * j, r = el / MG_BK, c = el % MG_BK;
            const int n = n0 + r, k = k0 + c;
            const bool live = r0 + r < r_end && k < K;
            const size_t row = UP ? (size_t)(live ? arow[r] : 0) : (size_t)(r0 + r);
            ra[j] = live ? kb_to_f<TA>(A[row * lda + k]) : 0.0f;
            rw[j] = (n < N && k < K) ? kb_to_f<TW>(We[(size_t)n * K + k]) : 0.0f;
        }
    };
    fetch(0);
    for (int k0 = 0; k0 < K; k0 += MG_BK) {
#pragma unroll
        for (int j = 0; j < PER; j++) {
            const int el = tid + 256 * j, r = el / MG_BK, c = el % MG_BK;
            As[c][r] = ra[j];
            Ws[c][r] = rw[j];
        }
        __syncthreads();
        if (k0 + MG_BK < K) fetch(k0 + MG_BK);
#pragma unroll
        for (int k = 0; k < MG_BK; k++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) a[i] = As[k][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) b[j] = Ws[k][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int rl = ty * 4 + i;
        if (r0 + rl >= r_end) continue;
        TC* crow;
        float f = 1.0f;
        if (UP) {
            crow = C + (size_t)(r0 + rl) * ldc;
        } else {
            const int pair = arow[rl];
            crow = C + (size_t)(pair % top) * plane_stride + (size_t)(pair / top) * ldc;
            f = wts[pair];
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int n = n0 + tx * 4 + j;
            if (n < N) crow[n] = kb_from_f<TC>(UP ? kb_act(acc[i][j], act) : __fmul_rn(f, acc[i][j]));
        }
    }
}

// the tile size the plan has to be made with for these products
extern "C" int kb_moe_gemm_tile() { return MG_BM; }

extern "C" int kb_moe_gemm(const void* A, int adtype, int lda, const void* W, int wdtype, void* C, int cdtype,
                           int ldc, long long plane_stride, int N, int K, int max_tiles, const int* n_tiles,
                           const int* tile_e, const int* tile_r0, const int* offs, const int* perm,
                           const float* wts, int top, int act, int up, cudaStream_t st) {
    if (max_tiles <= 0 || N <= 0) return 0;
    dim3 grid((N + MG_BN - 1) / MG_BN, max_tiles);
#define KB_MG(TA, TW, TC, UP)                                                                                       \
    kb_launch(k_moe_gemm<TA, TW, TC, UP>, grid, 256, 0, st, (const TA*)A, lda, (const TW*)W, (TC*)C, ldc,           \
              (size_t)plane_stride, N, K, n_tiles, tile_e, tile_r0, offs, perm, wts, top, act)
    if (up) {
        if (adtype == KB_F32 && wdtype == KB_F32 && cdtype == KB_F32) KB_MG(float, float, float, true);
        else if (adtype == KB_BF16 && wdtype == KB_BF16 && cdtype == KB_BF16) KB_MG(bf16, bf16, bf16, true);
        else if (adtype == KB_BF16 && wdtype == KB_F32 && cdtype == KB_BF16) KB_MG(bf16, float, bf16, true);
        else if (adtype == KB_F32 && wdtype == KB_BF16 && cdtype == KB_F32) KB_MG(float, bf16, float, true);
        else return (int)cudaErrorInvalidValue;
    } else {
        if (cdtype != KB_F32) return (int)cudaErrorInvalidValue;
        if (adtype == KB_F32 && wdtype == KB_F32) KB_MG(float, float, float, false);
        else if (adtype == KB_BF16 && wdtype == KB_BF16) KB_MG(bf16, bf16, float, false);
        else if (adtype == KB_BF16 && wdtype == KB_F32) KB_MG(bf16, float, float, false);
        else if (adtype == KB_F32 && wdtype == KB_BF16) KB_MG(float, bf16, float, false);
        else return (int)cudaErrorInvalidValue;
    }
#undef KB_MG
    KB_LAUNCH_RET();
}
