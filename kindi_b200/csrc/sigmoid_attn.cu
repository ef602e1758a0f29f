// Causal attention without a softmax: the weight of a visible key is sigmoid(q . k * scale + bias[h][i - j]), weights
// are not normalised over keys, and the output is the weighted sum of the values. bias is a table per head over the
// distance i - j (the last entry stands for every larger distance; a learned distance bias by buckets and a constant
// per head are folded into it by the host), or null.
//   k_sigattn_prep     queries times a temperature that grows with the position; keys into the cache; values, each head
//                      divided by its root mean square, into the cache
//   k_sigmoid_attn     the general kernel (float or bf16 storage, 32-bit arithmetic): a warp per (row, head), keys in
//                      runs of 32 absolute positions, so every sum's order depends on positions only
//   k_sigattn_mma      prompts on the tensor cores (bf16): a tile of 64 query rows of one head against pages of 64
//                      keys, S = Q K^T and O += P V by mma.sync m16n8k16, P = sigmoid(S scale + bias) in registers
//   k_sigattn_decode   single tokens: the keys of a (sequence, key/value head) split over CTAs, partial sums added in
//                      split order by k_sigattn_sum
#include "common.cuh"
#include <math.h>

__device__ __forceinline__ float sa_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }

// ------------------------------------------------------------------------------------------------ prepare and store
// c: 32-bit rows [q (H d) | k (G d) | v (G dv)]. q_out[t][h][0..hd) = q * (1 + coef ln((p + 1) / every + 1)) (integer
// division), zero beyond d; the cache gets k (zero beyond d) and v / sqrt(mean v^2 + eps) per head (zero beyond dv).
template <typename T>
__global__ void __launch_bounds__(256) k_sigattn_prep(const float* KB_STEP_DATA c, int ldc, int H, int G, int d, int dv,
        int hd, float coef, int every, int v_norm, float eps, const int* __restrict__ pos, const int* __restrict__ seq,
        const int* __restrict__ slot, T* __restrict__ q_out, int ldq, KbCacheView cv, int* status) {
    kb_pdl_launch();
    const int t = blockIdx.x;
    const int p = pos[t];
    T* qr = q_out + (size_t)t * ldq;
    kb_pdl_wait();
    if (p < 0) {
        for (int i = threadIdx.x; i < H * hd; i += 256) qr[i] = kb_from_f<T>(0.0f);
        return;
    }
    const float* cr = c + (size_t)t * ldc;
    const float temp = coef != 0.0f ? 1.0f + coef * logf((float)((p + 1) / every + 1)) : 1.0f;
    for (int i = threadIdx.x; i < H * hd; i += 256) {
        const int h = i / hd, e = i % hd;
        qr[i] = kb_from_f<T>(e < d ? __fmul_rn(cr[(size_t)h * d + e], temp) : 0.0f);
    }
    const int page = cv.table[(size_t)slot[seq[t]] * cv.table_stride + p / KB_PAGE];
    if (page < 0 || page >= cv.n_pages) {
        if (threadIdx.x == 0) atomicOr(status, KB_ST_BAD_PAGE);
        return;
    }
    const float* kr = cr + (size_t)H * d;
    for (int i = threadIdx.x; i < G * hd; i += 256) {
        const int g = i / hd, e = i % hd;
        ((T*)cv.pool)[kb_kv_offset(cv, page, 0, g, p % KB_PAGE) + e] = kb_from_f<T>(e < d ? kr[(size_t)g * d + e] : 0.0f);
    }
    const float* vr = kr + (size_t)G * d;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int g = warp; g < G; g += 8) {
        float f = 1.0f;
        if (v_norm) {
            float ss = 0.0f;
            for (int e = lane; e < dv; e += 32) ss = fmaf(vr[(size_t)g * dv + e], vr[(size_t)g * dv + e], ss);
            ss = kb_warp_sum(ss);
            f = 1.0f / sqrtf(ss / (float)dv + eps);
        }
        T* dst = (T*)cv.pool + kb_kv_offset(cv, page, 1, g, p % KB_PAGE);
        for (int e = lane; e < hd; e += 32) dst[e] = kb_from_f<T>(e < dv ? __fmul_rn(vr[(size_t)g * dv + e], f) : 0.0f);
    }
}

extern "C" int kb_sigattn_prep(const float* c, int ldc, int T, int H, int G, int d, int dv, int hd, float coef,
                               int every, int v_norm, float eps, const int* pos, const int* seq, const int* slot,
                               void* q_out, int dtype, int ldq, void* pool, const int* table, int table_stride,
                               int n_pages, int* status, cudaStream_t st) {
    if (T <= 0) return 0;
    if (every < 1 || d > hd || dv > hd) return (int)cudaErrorInvalidValue;
    KbCacheView cv{pool, table, table_stride, n_pages, G, hd};
    if (dtype == KB_F32)
        kb_launch(k_sigattn_prep<float>, T, 256, 0, st, c, ldc, H, G, d, dv, hd, coef, every, v_norm, eps, pos, seq,
                  slot, (float*)q_out, ldq, cv, status);
    else
        kb_launch(k_sigattn_prep<bf16>, T, 256, 0, st, c, ldc, H, G, d, dv, hd, coef, every, v_norm, eps, pos, seq, slot,
                  (bf16*)q_out, ldq, cv, status);
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ the general kernel
#define SA_MAX_HD 512
template <typename T>
__global__ void __launch_bounds__(128) k_sigmoid_attn(const T* KB_STEP_DATA q, int ldq, T* __restrict__ out, int ldo,
        const int* __restrict__ pos, const int* __restrict__ seq, const int* __restrict__ slot, int Tn, int nh,
        int group, int hd, float scale, const float* __restrict__ bias, int n_bias, KbCacheView cv, int* status) {
    __shared__ float qs[4][SA_MAX_HD];
    kb_pdl_launch();
    kb_pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * 4 + warp;
    if (item >= (long long)Tn * nh) return;
    const int t = (int)(item / nh), h = (int)(item % nh);
    const int hk = h / group;
    const int p_q = pos[t];
    if (p_q < 0) return;
    const int s = slot[seq[t]];
    const T* qr = q + (size_t)t * ldq + (size_t)h * hd;
    for (int e = lane; e < hd; e += 32) qs[warp][e] = __fmul_rn(kb_to_f<T>(qr[e]), scale);
    __syncwarp();
    const int* trow = cv.table + (size_t)s * cv.table_stride;
    const float* brow = bias ? bias + (size_t)h * n_bias : nullptr;
    float o[SA_MAX_HD / 32];
#pragma unroll
    for (int i = 0; i < SA_MAX_HD / 32; i++) o[i] = 0.0f;
    for (int c0 = 0; c0 <= p_q; c0 += 32) {
        const int p = c0 + lane;
        bool ok = p <= p_q;
        float pr = 0.0f;
        const T* vrow = nullptr;
        if (ok) {
            const int page = trow[p / KB_PAGE];
            if (page < 0 || page >= cv.n_pages) {
                atomicOr(status, KB_ST_BAD_PAGE);
                ok = false;
            } else {
                const T* kr = (const T*)cv.pool + kb_kv_offset(cv, page, 0, hk, p % KB_PAGE);
                vrow = (const T*)cv.pool + kb_kv_offset(cv, page, 1, hk, p % KB_PAGE);
                float a = 0.0f;
                for (int e = 0; e < hd; e++) a = fmaf(qs[warp][e], kb_to_f<T>(kr[e]), a);
                if (brow) a += brow[min(p_q - p, n_bias - 1)];
                pr = sa_sigmoid(a);
            }
        }
        const unsigned mask = __ballot_sync(0xffffffffu, ok);
        for (int j = 0; j < 32; j++) {
            if (!((mask >> j) & 1u)) continue;
            const float pj = __shfl_sync(0xffffffffu, pr, j);
            const T* vj = (const T*)__shfl_sync(0xffffffffu, (unsigned long long)vrow, j);
#pragma unroll
            for (int i = 0; i < SA_MAX_HD / 32; i++) {
                const int e = i * 32 + lane;
                if (e < hd) o[i] = fmaf(pj, kb_to_f<T>(vj[e]), o[i]);
            }
        }
    }
    T* orow = out + (size_t)t * ldo + (size_t)h * hd;
#pragma unroll
    for (int i = 0; i < SA_MAX_HD / 32; i++) {
        const int e = i * 32 + lane;
        if (e < hd) orow[e] = kb_from_f<T>(o[i]);
    }
}

extern "C" int kb_sigmoid_attn(const void* q, int dtype, int ldq, void* out, int ldo, const int* pos, const int* seq,
                               const int* slot, int T, int nh, int nkv, int hd, float scale, const float* bias,
                               int n_bias, void* pool, const int* table, int table_stride, int n_pages, int* status,
                               cudaStream_t st) {
    if (T <= 0) return 0;
    if (hd > SA_MAX_HD || nkv <= 0 || nh % nkv || (bias && n_bias < 1)) return (int)cudaErrorInvalidValue;
    KbCacheView cv{pool, table, table_stride, n_pages, nkv, hd};
    const int grid = (int)(((long long)T * nh + 3) / 4);
    if (dtype == KB_F32)
        kb_launch(k_sigmoid_attn<float>, grid, 128, 0, st, (const float*)q, ldq, (float*)out, ldo, pos, seq, slot, T, nh,
                  nh / nkv, hd, scale, bias, n_bias, cv, status);
    else
        kb_launch(k_sigmoid_attn<bf16>, grid, 128, 0, st, (const bf16*)q, ldq, (bf16*)out, ldo, pos, seq, slot, T, nh,
                  nh / nkv, hd, scale, bias, n_bias, cv, status);
    KB_LAUNCH_RET();
}
