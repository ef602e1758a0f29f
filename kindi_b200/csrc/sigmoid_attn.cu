// Causal attention without a softmax: the weight of a visible key is sigmoid(q . k * scale + bias[h][i - j]), weights
// are not normalised over keys, and the output is the weighted sum of the values. bias is a table per head over the
// distance i - j (the last entry stands for every larger distance; a learned distance bias by buckets and a constant
// per head are folded into it by the host), or null.
//   k_sigattn_prep     queries times a temperature that grows with the position; keys into the cache; values, each head
//                      divided by its root mean square, into the cache
//   k_sigmoid_attn     the general kernel (float or bf16 storage, 32-bit arithmetic): a warp per (row, head), keys in
//                      runs of 32 absolute positions, so every sum's order depends on positions only
//   k_sigattn_decode   single tokens (float or bf16 storage, 32-bit arithmetic): the pages of a (sequence, key/value
//                      head) split over CTAs, partial sums added in split order by k_sigattn_sum
// Prompt-sized steps in bf16 with head sizes 64 and 128 run on the tcgen05 attention kernel (attn_tc.cu), whose softmax
// warps then only turn scores into weights.
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

// ------------------------------------------------------------------------------------------------ single tokens
// One CTA: one sequence (row b of q and out), up to SD_G query heads of one key/value head, one split of the sequence's
// pages. A warp takes runs of 32 positions: each lane scores one key against the CTA's queries (the key's row read 16
// bytes a time), the weights pass through shared memory, and the lanes then share the elements of the run's value rows,
// two neighbours a lane. A CTA adds its warps' sums in warp order; k_sigattn_sum adds the splits' in split order.
#define SD_G 4
template <typename T> __device__ __forceinline__ void sd_load16(const T* p, float* f);
template <> __device__ __forceinline__ void sd_load16<bf16>(const bf16* p, float* f) {
    const uint4 v = *(const uint4*)p;
    const __nv_bfloat162* h = (const __nv_bfloat162*)&v;
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float2 x = __bfloat1622float2(h[k]);
        f[2 * k] = x.x;
        f[2 * k + 1] = x.y;
    }
}
template <> __device__ __forceinline__ void sd_load16<float>(const float* p, float* f) {
    const float4 v = *(const float4*)p;
    f[0] = v.x, f[1] = v.y, f[2] = v.z, f[3] = v.w;
}
template <typename T> __device__ __forceinline__ float2 sd_load2(const T* p);
template <> __device__ __forceinline__ float2 sd_load2<bf16>(const bf16* p) {
    return __bfloat1622float2(*(const __nv_bfloat162*)p);
}
template <> __device__ __forceinline__ float2 sd_load2<float>(const float* p) { return *(const float2*)p; }

// EM2 = ceil(hd / 64): pairs of elements a lane holds of every head's sum
template <typename T, int EM2>
__global__ void __launch_bounds__(128) k_sigattn_decode(const T* KB_STEP_DATA q, int ldq, T* __restrict__ out, int ldo,
        float* __restrict__ part, const int* __restrict__ slot, const int* __restrict__ kv_len, int nh, int group,
        int hd, float scale, const float* __restrict__ bias, int n_bias, KbCacheView cv, int* status) {
    constexpr int NV = 16 / (int)sizeof(T);
    __shared__ __align__(16) float qs[SD_G][EM2 * 64];
    __shared__ __align__(16) float os[SD_G][EM2 * 64];
    __shared__ float ws[4][SD_G][32];
    kb_pdl_launch();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_split = gridDim.x, sp = blockIdx.x, b = blockIdx.z;
    const int n_grp = (group + SD_G - 1) / SD_G;
    const int hk = blockIdx.y / n_grp, g0 = (blockIdx.y % n_grp) * SD_G;
    const int ng = min(SD_G, group - g0), h0 = hk * group + g0;
    kb_pdl_wait();
    const int kvl = max(kv_len[b], 0), p_q = kvl - 1;
    const int n_pg = (kvl + KB_PAGE - 1) / KB_PAGE, pps = (n_pg + n_split - 1) / n_split;
    const int k0 = min(kvl, sp * pps * KB_PAGE), k1 = min(kvl, (sp + 1) * pps * KB_PAGE);
    const T* qr = q + (size_t)b * ldq + (size_t)h0 * hd;
    for (int i = threadIdx.x; i < SD_G * EM2 * 64; i += 128) {
        const int g = i / (EM2 * 64), e = i % (EM2 * 64);
        qs[g][e] = (g < ng && e < hd) ? __fmul_rn(kb_to_f<T>(qr[(size_t)g * hd + e]), scale) : 0.0f;
    }
    __syncthreads();
    float o[SD_G][EM2][2];
#pragma unroll
    for (int g = 0; g < SD_G; g++)
#pragma unroll
        for (int i = 0; i < EM2; i++) o[g][i][0] = o[g][i][1] = 0.0f;
    const int* trow = cv.table + (size_t)slot[b] * cv.table_stride;
    for (int r0 = k0 + warp * 32; r0 < k1; r0 += 128) {
        const int page = trow[r0 / KB_PAGE];              // a run lies in one page
        if (page < 0 || page >= cv.n_pages) {
            if (lane == 0) atomicOr(status, KB_ST_BAD_PAGE);
            continue;
        }
        const int p = r0 + lane;
        const bool ok = p < k1;
        float a[SD_G];
#pragma unroll
        for (int g = 0; g < SD_G; g++) a[g] = 0.0f;
        if (ok) {
            const T* kr = (const T*)cv.pool + kb_kv_offset(cv, page, 0, hk, p % KB_PAGE);
#pragma unroll 4
            for (int e = 0; e < hd; e += NV) {
                float kf[NV];
                sd_load16<T>(kr + e, kf);
#pragma unroll
                for (int g = 0; g < SD_G; g++) {
#pragma unroll
                    for (int x = 0; x < NV; x += 4) {
                        const float4 qv = *(const float4*)&qs[g][e + x];
                        a[g] = fmaf(qv.x, kf[x], a[g]);
                        a[g] = fmaf(qv.y, kf[x + 1], a[g]);
                        a[g] = fmaf(qv.z, kf[x + 2], a[g]);
                        a[g] = fmaf(qv.w, kf[x + 3], a[g]);
                    }
                }
            }
        }
#pragma unroll
        for (int g = 0; g < SD_G; g++) {
            float z = a[g];
            if (bias != nullptr && ok && g < ng) z += bias[(size_t)(h0 + g) * n_bias + min(p_q - p, n_bias - 1)];
            ws[warp][g][lane] = ok ? sa_sigmoid(z) : 0.0f;
        }
        __syncwarp();
        const int nv = min(32, k1 - r0);
        const T* vb = (const T*)cv.pool + kb_kv_offset(cv, page, 1, hk, r0 % KB_PAGE);
#pragma unroll 4
        for (int j = 0; j < nv; j++) {
            float w[SD_G];
#pragma unroll
            for (int g = 0; g < SD_G; g++) w[g] = ws[warp][g][j];
#pragma unroll
            for (int i = 0; i < EM2; i++) {
                const int e = (i * 32 + lane) * 2;
                if (e < hd) {
                    const float2 v = sd_load2<T>(vb + (size_t)j * hd + e);
#pragma unroll
                    for (int g = 0; g < SD_G; g++) {
                        o[g][i][0] = fmaf(w[g], v.x, o[g][i][0]);
                        o[g][i][1] = fmaf(w[g], v.y, o[g][i][1]);
                    }
                }
            }
        }
        __syncwarp();
    }
    for (int w = 0; w < 4; w++) {
        if (warp == w) {
#pragma unroll
            for (int g = 0; g < SD_G; g++)
#pragma unroll
                for (int i = 0; i < EM2; i++) {
                    const int e = (i * 32 + lane) * 2;
                    os[g][e] = w == 0 ? o[g][i][0] : os[g][e] + o[g][i][0];
                    os[g][e + 1] = w == 0 ? o[g][i][1] : os[g][e + 1] + o[g][i][1];
                }
        }
        __syncthreads();
    }
    for (int i = threadIdx.x; i < ng * hd; i += 128) {
        const int g = i / hd, e = i % hd;
        if (part == nullptr) out[(size_t)b * ldo + (size_t)(h0 + g) * hd + e] = kb_from_f<T>(os[g][e]);
        else part[(((size_t)b * nh + h0 + g) * n_split + sp) * hd + e] = os[g][e];
    }
}

// out[b][h][e] = the sum over the splits, in order, of part[b][h][split][e]
template <typename T>
__global__ void __launch_bounds__(128) k_sigattn_sum(const float* KB_STEP_DATA part, int n_split, int nh, int hd,
        T* __restrict__ out, int ldo) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int h = blockIdx.x, b = blockIdx.y;
    const float* p = part + ((size_t)b * nh + h) * n_split * hd;
    for (int e = threadIdx.x; e < hd; e += 128) {
        float s = 0.0f;
        for (int i = 0; i < n_split; i++) s += p[(size_t)i * hd + e];
        out[(size_t)b * ldo + (size_t)h * hd + e] = kb_from_f<T>(s);
    }
}

// one row per sequence (row b of q and out belongs to sequence b, whose newest position is kv_len[b] - 1); n_split
// splits of every sequence's pages, part = float scratch [B][nh][n_split][hd] when n_split > 1. Head sizes that are a
// multiple of 16 bytes, pool 16-byte aligned.
extern "C" int kb_sigattn_decode(const void* q, int dtype, int ldq, void* out, int ldo, float* part, const int* slot,
                                 const int* kv_len, int B, int nh, int nkv, int hd, float scale, const float* bias,
                                 int n_bias, void* pool, const int* table, int table_stride, int n_pages, int n_split,
                                 int* status, cudaStream_t st) {
    if (B <= 0) return 0;
    const int nv = dtype == KB_F32 ? 4 : 8;
    if (hd > SA_MAX_HD || hd % nv || nkv <= 0 || nh % nkv || (bias && n_bias < 1) || n_split < 1 || n_split > 65535 ||
        (n_split > 1 && part == nullptr) || ((uintptr_t)pool & 15) || B > 65535)
        return (int)cudaErrorInvalidValue;
    const int group = nh / nkv, n_grp = (group + SD_G - 1) / SD_G;
    if ((long long)nkv * n_grp > 65535) return (int)cudaErrorInvalidValue;
    KbCacheView cv{pool, table, table_stride, n_pages, nkv, hd};
    dim3 grid(n_split, nkv * n_grp, B);
    float* pt = n_split > 1 ? part : nullptr;
#define KB_SD(T, EM2)                                                                                              \
    kb_launch(k_sigattn_decode<T, EM2>, grid, 128, 0, st, (const T*)q, ldq, (T*)out, ldo, pt, slot, kv_len, nh,   \
              group, hd, scale, bias, n_bias, cv, status)
#define KB_SD_HD(T)                                                                                                \
    do {                                                                                                           \
        if (hd <= 64) KB_SD(T, 1);                                                                                 \
        else if (hd <= 128) KB_SD(T, 2);                                                                           \
        else if (hd <= 256) KB_SD(T, 4);                                                                           \
        else KB_SD(T, 8);                                                                                          \
    } while (0)
    if (dtype == KB_F32) KB_SD_HD(float);
    else KB_SD_HD(bf16);
#undef KB_SD_HD
#undef KB_SD
    if (n_split > 1) {
        if (dtype == KB_F32)
            kb_launch(k_sigattn_sum<float>, dim3(nh, B), 128, 0, st, (const float*)part, n_split, nh, hd, (float*)out, ldo);
        else
            kb_launch(k_sigattn_sum<bf16>, dim3(nh, B), 128, 0, st, (const float*)part, n_split, nh, hd, (bf16*)out, ldo);
    }
    KB_LAUNCH_RET();
}
