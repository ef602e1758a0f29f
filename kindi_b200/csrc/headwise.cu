// Per-head steps around softmax attention, a norm on a sub-layer's OUTPUT, and a clamped gated activation.
//
// k_headnorm_rope_store: the row is [q heads | k heads | v heads], every head hd wide (heads narrower than hd were
// widened with zeros by the weights), as rows in the run dtype or as 32-bit planes summed in order. Every query head
// and every key head is, in the order the part asks for,
//   - divided by ITS OWN root mean square, sqrt(sum(v^2) / dim + eps) with dim the head's true size, and multiplied by
//     gains [hd] that all heads share (no gains: a unit norm),
//   - rotated: the pairs (i, i + rot/2) turn by pos * inv_freq[i] (rot = 0: no rotation),
// the norm before the rotation (mode 1) or after it (mode 2; mode 0: no norm). Query heads are then multiplied by a
// temperature that grows with the position, 1 + coef * ln(floor((pos + 1) / every) + 1) (coef = 0: none). Queries go
// to qout, keys and values to the row's place in its cache page. A warp owns a head from its load to its store and a
// block is a row's next eight heads, so a decode step of few rows still fills the SMs and nothing but the angles
// meets a block barrier. All of it is 32-bit (EXACT: angles,
// cosines and sines in 64-bit from a 64-bit frequency table, for the true 32-bit path); each value is rounded to the
// run dtype once, when it is written.
//
// k_diff_combine: differential attention's last step. The attention kernels ran 2 H query heads in the order
// (key/value group, map, head of the group); head h = g * r + i of the model is
//   o = a[g][0][i] - lambda * a[g][1][i],  out = o / sqrt(mean(o^2) + eps) * mult    over the head's vd true values.
//
// k_head_gate_mul: out[t][h][c] = a[t][h][c] * sigmoid(z[t][h]), one gate per head; z rows or 32-bit planes.
//
// k_postnorm_add: x += ls * (w * (v / sqrt(mean(v^2) + eps))) with v the sum of a branch's planes in order: the norm
// sits on the sub-layer's output, the residual takes the normed and scaled branch; y = x in the run dtype is what the
// next sub-layer reads (it reads the stream itself, not a normed copy).
//
// k_cast_rows: y = x in the run dtype.
//
// k_glu_clamp: out = g' * sigmoid(alpha * g') * (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit), with
// [g | u] in column groups as the gated products lay them out.
#include "common.cuh"
#include <math.h>

#define HW_THREADS 256

#define HW_HEADS (HW_THREADS / 32)      // heads of a block: one per warp
template <typename TIN, typename T, bool EXACT>
__global__ void __launch_bounds__(HW_THREADS) k_headnorm_rope_store(const TIN* KB_STEP_DATA in, int n_planes,
        size_t plane_stride, int ld_in, T* qout, int ldq, const float* __restrict__ gq, const float* __restrict__ gk,
        float eps, int dim_true, int norm_mode, const float* __restrict__ inv_freq,
        const double* __restrict__ inv_freq64, int rot, float t_coef, int t_every, const int* __restrict__ pos,
        const int* __restrict__ seq, const int* __restrict__ slot, int nh, int nkv, int nkv_store, int hd,
        KbCacheView cv, int* status) {
    extern __shared__ float sm[];
    kb_pdl_launch();
    const int t = blockIdx.x;
    const int p = pos[t];
    if (p < 0) return;                               // a padding row of a recorded step
    const int half = rot / 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* hr = sm + (size_t)warp * hd;              // this warp's head
    float2* cs = (float2*)(sm + (((size_t)HW_HEADS * hd + 1) & ~(size_t)1));    // [half]: cosine and sine of the row's angles
    int page = -1;
    if (nkv_store > 0) {
        const int s = slot[seq[t]];
        page = cv.table[(size_t)s * cv.table_stride + p / KB_PAGE];
        if (page < 0 || page >= cv.n_pages) page = -1;
    }
    for (int i = threadIdx.x; i < half; i += HW_THREADS) {
        if (EXACT) {
            double s_, c_;
            sincos((double)p * inv_freq64[i], &s_, &c_);
            cs[i] = make_float2((float)c_, (float)s_);
        } else {
            const float ang = __fmul_rn((float)p, inv_freq[i]);
            cs[i] = make_float2(cosf(ang), sinf(ang));
        }
    }
    float temp = 1.0f;
    if (t_coef != 0.0f) temp = 1.0f + t_coef * logf((float)((p + 1) / t_every + 1));
    __syncthreads();                                 // (the angles)
    kb_pdl_wait();
    if (nkv_store > 0 && page < 0 && threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, KB_ST_BAD_PAGE);
    const int h = blockIdx.y * HW_HEADS + warp;      // among [q heads | k heads | v heads]
    if (h >= nh + 2 * nkv) return;
    const TIN* src = in + (size_t)t * ld_in + (size_t)h * hd;
    for (int i = lane; i < hd; i += 32) {
        float v = kb_to_f<TIN>(src[i]);
        for (int s = 1; s < n_planes; s++) v += kb_to_f<TIN>(src[(size_t)s * plane_stride + i]);
        hr[i] = v;
    }
    __syncwarp();
    if (h < nh + nkv) {
        const float* gain = h < nh ? gq : gk;
        for (int step = 0; step < 2; step++) {
            const bool do_norm = (step == 0 && norm_mode == 1) || (step == 1 && norm_mode == 2);
            const bool do_rot = (step == 0 && norm_mode == 2) || (step == 1 && norm_mode != 2);
            if (do_norm) {
                float ss = 0.0f;
                for (int i = lane; i < hd; i += 32) ss = fmaf(hr[i], hr[i], ss);
                ss = kb_warp_sum(ss);
                const float f = 1.0f / sqrtf(ss / (float)dim_true + eps);
                for (int i = lane; i < hd; i += 32) {
                    const float v = __fmul_rn(hr[i], f);
                    hr[i] = gain ? __fmul_rn(v, gain[i]) : v;
                }
                __syncwarp();
            }
            if (do_rot && half > 0) {
                for (int i = lane; i < half; i += 32) {
                    const float a = hr[i], b = hr[i + half];
                    const float2 c = cs[i];
                    hr[i] = __fsub_rn(__fmul_rn(a, c.x), __fmul_rn(b, c.y));
                    hr[i + half] = __fadd_rn(__fmul_rn(b, c.x), __fmul_rn(a, c.y));
                }
                __syncwarp();
            }
        }
    }
    if (h < nh) {
        T* dst = qout + (size_t)t * ldq + (size_t)h * hd;
        for (int i = lane; i < hd; i += 32) dst[i] = kb_from_f<T>(t_coef != 0.0f ? __fmul_rn(hr[i], temp) : hr[i]);
    } else if (page >= 0) {
        const int kv = h >= nh + nkv ? 1 : 0, hk = h - nh - kv * nkv;
        T* dst = (T*)cv.pool + kb_kv_offset(cv, page, kv, hk, p % KB_PAGE);
        for (int i = lane; i < hd; i += 32) dst[i] = kb_from_f<T>(hr[i]);
    }
}

// The same for heads of 32 * NE elements that are rotated as a whole or not at all (rot == hd or 0), with 16-byte
// aligned rows: a lane holds NE neighbouring elements of the head in registers (one load), its partner in the
// rotation is lane ^ 16, the head's sum of squares is one warp reduction, and nothing goes through shared memory.
// A warp walks the heads h, h + 8 gridDim.y, ... of its row with the row's cosines and sines in registers.
template <int N> struct HwVec;
template <> struct HwVec<2> { typedef uint32_t b; typedef float2 f; };
template <> struct HwVec<4> { typedef uint2 b; typedef float4 f; };
template <int NE> __device__ __forceinline__ void hw_load(const float* p, float* o) {
    const typename HwVec<NE>::f v = *(const typename HwVec<NE>::f*)p;
#pragma unroll
    for (int e = 0; e < NE; e++) o[e] = ((const float*)&v)[e];
}
template <int NE> __device__ __forceinline__ void hw_load(const bf16* p, float* o) {
    const typename HwVec<NE>::b v = *(const typename HwVec<NE>::b*)p;
#pragma unroll
    for (int e = 0; e < NE; e++) o[e] = __bfloat162float(((const bf16*)&v)[e]);
}
template <int NE> __device__ __forceinline__ void hw_store(float* p, const float* o) {
    typename HwVec<NE>::f v;
#pragma unroll
    for (int e = 0; e < NE; e++) ((float*)&v)[e] = o[e];
    *(typename HwVec<NE>::f*)p = v;
}
template <int NE> __device__ __forceinline__ void hw_store(bf16* p, const float* o) {
    typename HwVec<NE>::b v;
#pragma unroll
    for (int e = 0; e < NE; e++) ((bf16*)&v)[e] = __float2bfloat16_rn(o[e]);
    *(typename HwVec<NE>::b*)p = v;
}

template <typename TIN, typename T, int NE, bool EXACT>
__global__ void __launch_bounds__(HW_THREADS) k_headnorm_rope_store_reg(const TIN* KB_STEP_DATA in, int n_planes,
        size_t plane_stride, int ld_in, T* qout, int ldq, const float* __restrict__ gq, const float* __restrict__ gk,
        float eps, int dim_true, int norm_mode, const float* __restrict__ inv_freq,
        const double* __restrict__ inv_freq64, int rot, float t_coef, int t_every, const int* __restrict__ pos,
        const int* __restrict__ seq, const int* __restrict__ slot, int nh, int nkv, int nkv_store, KbCacheView cv,
        int* status) {
    constexpr int hd = 32 * NE;
    kb_pdl_launch();
    const int t = blockIdx.x;
    const int p = pos[t];
    if (p < 0) return;                               // a padding row of a recorded step
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e0 = lane * NE;                        // this lane's elements of a head
    int page = -1;
    if (nkv_store > 0) {
        const int s = slot[seq[t]];
        page = cv.table[(size_t)s * cv.table_stride + p / KB_PAGE];
        if (page < 0 || page >= cv.n_pages) page = -1;
    }
    float c[NE], sn[NE], wq[NE], wk[NE];
#pragma unroll
    for (int e = 0; e < NE; e++) {
        c[e] = 1.0f;
        sn[e] = 0.0f;
        if (rot > 0) {
            const int i = (lane & 15) * NE + e;      // the pair's index: elements i and i + hd / 2
            if (EXACT) {
                double s_, c_;
                sincos((double)p * inv_freq64[i], &s_, &c_);
                c[e] = (float)c_;
                sn[e] = (float)s_;
            } else {
                const float ang = __fmul_rn((float)p, inv_freq[i]);
                c[e] = cosf(ang);
                sn[e] = sinf(ang);
            }
            if (lane < 16) sn[e] = -sn[e];           // element i: a c - b s; element i + hd / 2: b c + a s
        }
        wq[e] = gq ? gq[e0 + e] : 1.0f;
        wk[e] = gk ? gk[e0 + e] : 1.0f;
    }
    float temp = 1.0f;
    if (t_coef != 0.0f) temp = 1.0f + t_coef * logf((float)((p + 1) / t_every + 1));
    kb_pdl_wait();
    if (nkv_store > 0 && page < 0 && threadIdx.x == 0 && blockIdx.y == 0) atomicOr(status, KB_ST_BAD_PAGE);
    for (int h = blockIdx.y * HW_HEADS + warp; h < nh + 2 * nkv; h += gridDim.y * HW_HEADS) {
        const TIN* src = in + (size_t)t * ld_in + (size_t)h * hd + e0;
        float v[NE];
        hw_load<NE>(src, v);
        for (int s = 1; s < n_planes; s++) {
            float u[NE];
            hw_load<NE>(src + (size_t)s * plane_stride, u);
#pragma unroll
            for (int e = 0; e < NE; e++) v[e] += u[e];
        }
        if (h < nh + nkv) {
#pragma unroll
            for (int step = 0; step < 2; step++) {
                const bool do_norm = (step == 0 && norm_mode == 1) || (step == 1 && norm_mode == 2);
                const bool do_rot = (step == 0 && norm_mode == 2) || (step == 1 && norm_mode != 2);
                if (do_norm) {
                    float ss = 0.0f;
#pragma unroll
                    for (int e = 0; e < NE; e++) ss = fmaf(v[e], v[e], ss);
                    ss = kb_warp_sum(ss);
                    const float f = 1.0f / sqrtf(ss / (float)dim_true + eps);
#pragma unroll
                    for (int e = 0; e < NE; e++) v[e] = __fmul_rn(__fmul_rn(v[e], f), h < nh ? wq[e] : wk[e]);
                }
                if (do_rot && rot > 0) {
#pragma unroll
                    for (int e = 0; e < NE; e++) {
                        const float o = __shfl_xor_sync(0xffffffffu, v[e], 16);
                        v[e] = __fadd_rn(__fmul_rn(v[e], c[e]), __fmul_rn(o, sn[e]));
                    }
                }
            }
        }
        if (h < nh) {
            if (t_coef != 0.0f) {
#pragma unroll
                for (int e = 0; e < NE; e++) v[e] = __fmul_rn(v[e], temp);
            }
            hw_store<NE>(qout + (size_t)t * ldq + (size_t)h * hd + e0, v);
        } else if (page >= 0) {
            const int kv = h >= nh + nkv ? 1 : 0, hk = h - nh - kv * nkv;
            hw_store<NE>((T*)cv.pool + kb_kv_offset(cv, page, kv, hk, p % KB_PAGE) + e0, v);
        }
    }
}

extern "C" int kb_headnorm_rope_store(const void* in, int in_dtype, int n_planes, long long plane_stride, int ld_in,
                                      void* qout, int dtype, int ldq, const float* gq, const float* gk, float eps,
                                      int dim_true, int norm_mode, const float* inv_freq, const double* inv_freq64,
                                      int rot, float t_coef, int t_every, const int* pos, const int* seq,
                                      const int* slot, int T, int nh, int nkv, int nkv_store, int hd, void* pool,
                                      const int* table, int table_stride, int n_pages, int* status, cudaStream_t st) {
    if (T <= 0) return 0;
    if (rot < 0 || rot % 2 || rot > hd || norm_mode < 0 || norm_mode > 2 || dim_true < 1 || dim_true > hd ||
        (t_coef != 0.0f && t_every < 1) || (nkv_store != 0 && nkv_store != nkv))
        return (int)cudaErrorInvalidValue;
    KbCacheView cv{pool, table, table_stride, n_pages, nkv, hd};
    const int n_heads = nh + 2 * nkv;
    const size_t smem = ((size_t)(HW_HEADS * hd + 1) & ~(size_t)1) * sizeof(float) + (size_t)(rot / 2) * sizeof(float2);
    if (smem > 200 * 1024 || n_heads > 65535 * HW_HEADS) return (int)cudaErrorInvalidValue;
    const dim3 grid(T, (n_heads + HW_HEADS - 1) / HW_HEADS);
    cudaError_t e = cudaSuccess;
    // heads of 64 or 128 rotated as a whole or not at all, aligned rows: the form that keeps a head in registers; a
    // prompt-sized step gives a block all heads of its row, a small step spreads a row's heads over blocks
    const int in_el = in_dtype == KB_F32 ? 4 : 2, out_el = dtype == KB_F32 ? 4 : 2;
    const int ne = hd / 32;
    if ((hd == 64 || hd == 128) && (rot == 0 || rot == hd) && ld_in % ne == 0 && ldq % ne == 0 && plane_stride % ne == 0 &&
        ((uintptr_t)in % (ne * in_el)) == 0 && ((uintptr_t)qout % (ne * out_el)) == 0 &&
        ((uintptr_t)pool % (ne * out_el)) == 0) {
        const int want = (n_heads + HW_HEADS - 1) / HW_HEADS;
        const int gy = T >= 1024 ? 1 : T >= 256 ? (want < 2 ? want : 2) : want;
        const dim3 gridr(T, gy);
#define KB_HWR(TIN, T_, NE, EX)                                                                                    \
        e = kb_launch(k_headnorm_rope_store_reg<TIN, T_, NE, EX>, gridr, HW_THREADS, 0, st, (const TIN*)in, n_planes, \
                      (size_t)plane_stride, ld_in, (T_*)qout, ldq, gq, gk, eps, dim_true, norm_mode, inv_freq,     \
                      inv_freq64, rot, t_coef, t_every, pos, seq, slot, nh, nkv, nkv_store, cv, status)
#define KB_HWR2(TIN, T_, EX) do { if (ne == 4) KB_HWR(TIN, T_, 4, EX); else KB_HWR(TIN, T_, 2, EX); } while (0)
        if (in_dtype == KB_F32 && dtype == KB_F32) {
            if (rot > 0 && inv_freq64 == nullptr) return (int)cudaErrorInvalidValue;
            KB_HWR2(float, float, true);
        } else if (rot > 0 && inv_freq == nullptr) return (int)cudaErrorInvalidValue;
        else if (in_dtype == KB_F32 && dtype == KB_BF16) KB_HWR2(float, bf16, false);
        else if (in_dtype == KB_BF16 && dtype == KB_BF16) KB_HWR2(bf16, bf16, false);
        else return (int)cudaErrorInvalidValue;
#undef KB_HWR2
#undef KB_HWR
        return (int)e;
    }
#define KB_HW(TIN, T_, EX)                                                                                         \
    do {                                                                                                           \
        if (smem > 48 * 1024)                                                                                      \
            cudaFuncSetAttribute(k_headnorm_rope_store<TIN, T_, EX>, cudaFuncAttributeMaxDynamicSharedMemorySize,  \
                                 (int)smem);                                                                       \
        e = kb_launch(k_headnorm_rope_store<TIN, T_, EX>, grid, HW_THREADS, smem, st, (const TIN*)in, n_planes,    \
                      (size_t)plane_stride, ld_in, (T_*)qout, ldq, gq, gk, eps, dim_true, norm_mode, inv_freq,     \
                      inv_freq64, rot, t_coef, t_every, pos, seq, slot, nh, nkv, nkv_store, hd, cv, status);       \
    } while (0)
    if (in_dtype == KB_F32 && dtype == KB_F32) {
        if (rot > 0 && inv_freq64 == nullptr) return (int)cudaErrorInvalidValue;
        KB_HW(float, float, true);
    } else if (rot > 0 && inv_freq == nullptr) return (int)cudaErrorInvalidValue;
    else if (in_dtype == KB_F32 && dtype == KB_BF16) KB_HW(float, bf16, false);
    else if (in_dtype == KB_BF16 && dtype == KB_BF16) KB_HW(bf16, bf16, false);
    else return (int)cudaErrorInvalidValue;
#undef KB_HW
    return (int)e;
}

// ------------------------------------------------------------------------------------------------ differential combine
// a: [T][G * 2 * r heads of hd] in the order (group, map, head of the group); out: [T][G * r heads of hd] (columns
// from vd on are written as zero). A warp per (row, head).
template <typename T>
__global__ void __launch_bounds__(HW_THREADS) k_diff_combine(const T* KB_STEP_DATA a, int lda, T* out, int ldo,
        int n_rows, int H, int r, int hd, int vd, float lambda, float eps, float mult) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (HW_THREADS / 32) + (threadIdx.x >> 5);
    if (item >= (long long)n_rows * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    const int g = h / r, i = h % r;
    const T* a1 = a + (size_t)t * lda + (size_t)((g * 2 + 0) * r + i) * hd;
    const T* a2 = a + (size_t)t * lda + (size_t)((g * 2 + 1) * r + i) * hd;
    T* o = out + (size_t)t * ldo + (size_t)h * hd;
    float ss = 0.0f;
    for (int c = lane; c < vd; c += 32) {
        const float v = __fsub_rn(kb_to_f<T>(a1[c]), __fmul_rn(lambda, kb_to_f<T>(a2[c])));
        ss = fmaf(v, v, ss);
    }
    ss = kb_warp_sum(ss);
    const float f = 1.0f / sqrtf(ss / (float)vd + eps);
    for (int c = lane; c < hd; c += 32) {
        float v = 0.0f;
        if (c < vd) {
            v = __fsub_rn(kb_to_f<T>(a1[c]), __fmul_rn(lambda, kb_to_f<T>(a2[c])));
            v = __fmul_rn(__fmul_rn(v, f), mult);
        }
        o[c] = kb_from_f<T>(v);
    }
}

// the same with VEC neighbouring elements a lane (bf16, hd = 32 VEC): one load of each map, one store
template <int VEC>
__global__ void __launch_bounds__(HW_THREADS) k_diff_combine_vec(const bf16* KB_STEP_DATA a, int lda, bf16* out,
        int ldo, int n_rows, int H, int r, int vd, float lambda, float eps, float mult) {
    constexpr int hd = 32 * VEC;
    kb_pdl_launch();
    kb_pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (HW_THREADS / 32) + (threadIdx.x >> 5);
    if (item >= (long long)n_rows * H) return;
    const int t = (int)(item / H), h = (int)(item % H);
    const int g = h / r, i = h % r;
    const bf16* a1 = a + (size_t)t * lda + (size_t)((g * 2 + 0) * r + i) * hd + lane * VEC;
    const bf16* a2 = a + (size_t)t * lda + (size_t)((g * 2 + 1) * r + i) * hd + lane * VEC;
    bf16 x1[VEC], x2[VEC], y[VEC];
    if (VEC == 4) {
        *(uint2*)x1 = *(const uint2*)a1;
        *(uint2*)x2 = *(const uint2*)a2;
    } else {
        *(uint32_t*)x1 = *(const uint32_t*)a1;
        *(uint32_t*)x2 = *(const uint32_t*)a2;
    }
    float v[VEC], ss = 0.0f;
#pragma unroll
    for (int c = 0; c < VEC; c++) {
        v[c] = lane * VEC + c < vd ? __fsub_rn(__bfloat162float(x1[c]), __fmul_rn(lambda, __bfloat162float(x2[c]))) : 0.0f;
        ss = fmaf(v[c], v[c], ss);
    }
    ss = kb_warp_sum(ss);
    const float f = 1.0f / sqrtf(ss / (float)vd + eps);
#pragma unroll
    for (int c = 0; c < VEC; c++) y[c] = __float2bfloat16_rn(__fmul_rn(__fmul_rn(v[c], f), mult));
    bf16* o = out + (size_t)t * ldo + (size_t)h * hd + lane * VEC;
    if (VEC == 4) *(uint2*)o = *(const uint2*)y;
    else *(uint32_t*)o = *(const uint32_t*)y;
}

extern "C" int kb_diff_combine(const void* a, int dtype, int lda, void* out, int ldo, int T, int H, int r, int hd,
                               int vd, float lambda, float eps, float mult, cudaStream_t st) {
    if (T <= 0 || H <= 0) return 0;
    if (r < 1 || H % r || vd < 1 || vd > hd) return (int)cudaErrorInvalidValue;
    const long long items = (long long)T * H;
    const int grid = (int)((items + HW_THREADS / 32 - 1) / (HW_THREADS / 32));
    const bool al = lda % 4 == 0 && ldo % 4 == 0 && ((uintptr_t)a % 8) == 0 && ((uintptr_t)out % 8) == 0;
    if (dtype == KB_BF16 && al && hd == 128)
        kb_launch(k_diff_combine_vec<4>, grid, HW_THREADS, 0, st, (const bf16*)a, lda, (bf16*)out, ldo, T, H, r, vd,
                  lambda, eps, mult);
    else if (dtype == KB_BF16 && al && hd == 64)
        kb_launch(k_diff_combine_vec<2>, grid, HW_THREADS, 0, st, (const bf16*)a, lda, (bf16*)out, ldo, T, H, r, vd,
                  lambda, eps, mult);
    else if (dtype == KB_F32)
        kb_launch(k_diff_combine<float>, grid, HW_THREADS, 0, st, (const float*)a, lda, (float*)out, ldo, T, H, r, hd,
                  vd, lambda, eps, mult);
    else if (dtype == KB_BF16)
        kb_launch(k_diff_combine<bf16>, grid, HW_THREADS, 0, st, (const bf16*)a, lda, (bf16*)out, ldo, T, H, r, hd, vd,
                  lambda, eps, mult);
    else return (int)cudaErrorInvalidValue;
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ a gate per head
template <typename TA, typename TG>
__global__ void __launch_bounds__(HW_THREADS) k_head_gate_mul(const TA* KB_STEP_DATA a, int lda,
        const TG* KB_STEP_DATA g, int n_planes, size_t plane_stride, int ldg, TA* out, int ldo, int N, int hd) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int c = blockIdx.y * HW_THREADS + threadIdx.x;
    if (c >= N) return;
    const size_t t = blockIdx.x;
    const TG* gp = g + t * ldg + c / hd;
    float z = kb_to_f<TG>(gp[0]);
    for (int s = 1; s < n_planes; s++) z += kb_to_f<TG>(gp[(size_t)s * plane_stride]);
    out[t * ldo + c] = kb_from_f<TA>(kb_to_f<TA>(a[t * lda + c]) * (1.0f / (1.0f + expf(-z))));
}

// bf16 rows, eight neighbouring elements a thread (hd a multiple of 8: they share a head and its gate)
template <typename TG>
__global__ void __launch_bounds__(HW_THREADS) k_head_gate_mul8(const bf16* KB_STEP_DATA a, int lda,
        const TG* KB_STEP_DATA g, int n_planes, size_t plane_stride, int ldg, bf16* out, int ldo, int N, int hd) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int c = (blockIdx.y * HW_THREADS + threadIdx.x) * 8;
    if (c >= N) return;
    const size_t t = blockIdx.x;
    const TG* gp = g + t * ldg + c / hd;
    float z = kb_to_f<TG>(gp[0]);
    for (int s = 1; s < n_planes; s++) z += kb_to_f<TG>(gp[(size_t)s * plane_stride]);
    const float w = __fdividef(1.0f, 1.0f + __expf(-z));
    uint4 v = *(const uint4*)(a + t * lda + c);
    __nv_bfloat162* v2 = (__nv_bfloat162*)&v;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const float2 f = __bfloat1622float2(v2[j]);
        v2[j] = __floats2bfloat162_rn(f.x * w, f.y * w);
    }
    *(uint4*)(out + t * ldo + c) = v;
}

extern "C" int kb_head_gate_mul(const void* a, int adtype, int lda, const void* g, int gdtype, int n_planes,
                                long long plane_stride, int ldg, void* out, int ldo, int T, int N, int hd,
                                cudaStream_t st) {
    if (T <= 0 || N <= 0) return 0;
    if (hd < 1) return (int)cudaErrorInvalidValue;
    if (adtype == KB_BF16 && hd % 8 == 0 && lda % 8 == 0 && ldo % 8 == 0 && ((uintptr_t)a % 16) == 0 &&
        ((uintptr_t)out % 16) == 0) {
        dim3 grid8(T, (N / 8 + HW_THREADS - 1) / HW_THREADS);
        if (gdtype == KB_BF16)
            kb_launch(k_head_gate_mul8<bf16>, grid8, HW_THREADS, 0, st, (const bf16*)a, lda, (const bf16*)g, n_planes,
                      (size_t)plane_stride, ldg, (bf16*)out, ldo, N, hd);
        else if (gdtype == KB_F32)
            kb_launch(k_head_gate_mul8<float>, grid8, HW_THREADS, 0, st, (const bf16*)a, lda, (const float*)g,
                      n_planes, (size_t)plane_stride, ldg, (bf16*)out, ldo, N, hd);
        else return (int)cudaErrorInvalidValue;
        KB_LAUNCH_RET();
    }
    dim3 grid(T, (N + HW_THREADS - 1) / HW_THREADS);
#define KB_HG(TA, TG)                                                                                              \
    kb_launch(k_head_gate_mul<TA, TG>, grid, HW_THREADS, 0, st, (const TA*)a, lda, (const TG*)g, n_planes,         \
              (size_t)plane_stride, ldg, (TA*)out, ldo, N, hd)
    if (adtype == KB_F32 && gdtype == KB_F32) KB_HG(float, float);
    else if (adtype == KB_BF16 && gdtype == KB_BF16) KB_HG(bf16, bf16);
    else if (adtype == KB_BF16 && gdtype == KB_F32) KB_HG(bf16, float);
    else return (int)cudaErrorInvalidValue;
#undef KB_HG
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ norm on the output
#define PN_THREADS 256
__device__ __forceinline__ float pn_block_sum(float v, float* red) {
    v = kb_warp_sum(v);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = red[0];
#pragma unroll
    for (int k = 1; k < PN_THREADS / 32; k++) tot += red[k];
    return tot;
}

// one block per row; the summed branch is kept in shared memory between the sum of squares and the update. VEC: the
// width is a multiple of 4 and rows are 16-byte aligned
template <typename TY, typename TW, bool VEC>
__global__ void __launch_bounds__(PN_THREADS) k_postnorm_add(float* KB_STEP_DATA x, const float* KB_STEP_DATA delta,
        int n_delta, size_t delta_stride, const float* __restrict__ bias, const TW* __restrict__ w,
        const TW* __restrict__ ls, float eps, TY* y, int E) {
    extern __shared__ float sv[];
    __shared__ float red[PN_THREADS / 32];
    kb_pdl_launch();
    kb_pdl_wait();
    const size_t t = blockIdx.x;
    float* xr = x + t * E;
    const float* dr = delta + t * E;
    float ss = 0.0f;
    if (VEC) {
        for (int i = threadIdx.x * 4; i < E; i += PN_THREADS * 4) {
            float4 v = *(const float4*)(dr + i);
            for (int s = 1; s < n_delta; s++) {
                const float4 d = *(const float4*)(dr + (size_t)s * delta_stride + i);
                v.x += d.x; v.y += d.y; v.z += d.z; v.w += d.w;
            }
            if (bias) { v.x += bias[i]; v.y += bias[i + 1]; v.z += bias[i + 2]; v.w += bias[i + 3]; }
            *(float4*)(sv + i) = v;
            ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
        }
    } else {
        for (int i = threadIdx.x; i < E; i += PN_THREADS) {
            float v = dr[i];
            for (int s = 1; s < n_delta; s++) v += dr[(size_t)s * delta_stride + i];
            if (bias) v += bias[i];
            sv[i] = v;
            ss = fmaf(v, v, ss);
        }
    }
    const float tot = pn_block_sum(ss, red);
    const float f = 1.0f / sqrtf(tot / (float)E + eps);
    if (VEC) {
        for (int i = threadIdx.x * 4; i < E; i += PN_THREADS * 4) {
            const float4 v = *(const float4*)(sv + i);
            float4 xv = *(const float4*)(xr + i);
            float b[4] = {v.x, v.y, v.z, v.w};
            float* xs = (float*)&xv;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                float u = __fmul_rn(__fmul_rn(b[c], f), kb_to_f<TW>(w[i + c]));
                if (ls) u = __fmul_rn(u, kb_to_f<TW>(ls[i + c]));
                xs[c] = __fadd_rn(xs[c], u);
            }
            *(float4*)(xr + i) = xv;
            if (y) {
#pragma unroll
                for (int c = 0; c < 4; c++) y[t * E + i + c] = kb_from_f<TY>(xs[c]);
            }
        }
    } else {
        for (int i = threadIdx.x; i < E; i += PN_THREADS) {
            float u = __fmul_rn(__fmul_rn(sv[i], f), kb_to_f<TW>(w[i]));
            if (ls) u = __fmul_rn(u, kb_to_f<TW>(ls[i]));
            const float xv = __fadd_rn(xr[i], u);
            xr[i] = xv;
            if (y) y[t * E + i] = kb_from_f<TY>(xv);
        }
    }
}

extern "C" int kb_postnorm_add(float* x, const float* delta, int n_delta, long long delta_stride, const float* bias,
                               const void* w, const void* ls, int wdtype, float eps, void* y, int ydtype, int T, int E,
                               cudaStream_t st) {
    if (T <= 0 || E <= 0) return 0;
    if (n_delta < 1) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)E * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    const bool vec = E % 4 == 0 && delta_stride % 4 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)delta % 16) == 0;
    cudaError_t e = cudaSuccess;
#define KB_PN(TY, TW, V)                                                                                           \
    do {                                                                                                           \
        if (smem > 48 * 1024)                                                                                      \
            cudaFuncSetAttribute(k_postnorm_add<TY, TW, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        e = kb_launch(k_postnorm_add<TY, TW, V>, T, PN_THREADS, smem, st, x, delta, n_delta, (size_t)delta_stride, \
                      bias, (const TW*)w, (const TW*)ls, eps, (TY*)y, E);                                          \
    } while (0)
#define KB_PN2(TY, TW) do { if (vec) KB_PN(TY, TW, true); else KB_PN(TY, TW, false); } while (0)
    const bool yf = y == nullptr || ydtype == KB_F32;
    if (yf && wdtype == KB_F32) KB_PN2(float, float);
    else if (yf && wdtype == KB_BF16) KB_PN2(float, bf16);
    else if (ydtype == KB_BF16 && wdtype == KB_BF16) KB_PN2(bf16, bf16);
    else if (ydtype == KB_BF16 && wdtype == KB_F32) KB_PN2(bf16, float);
    else return (int)cudaErrorInvalidValue;
#undef KB_PN2
#undef KB_PN
    return (int)e;
}

template <typename TY>
__global__ void __launch_bounds__(256) k_cast_rows(const float* KB_STEP_DATA x, TY* y, long long n) {
    kb_pdl_launch();
    kb_pdl_wait();
    const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
    if (i < n) y[i] = kb_from_f<TY>(x[i]);
}

extern "C" int kb_cast_rows(const float* x, void* y, int ydtype, long long n, cudaStream_t st) {
    if (n <= 0) return 0;
    const int grid = (int)((n + 255) / 256);
    if (ydtype == KB_BF16) kb_launch(k_cast_rows<bf16>, grid, 256, 0, st, x, (bf16*)y, n);
    else if (ydtype == KB_F32) kb_launch(k_cast_rows<float>, grid, 256, 0, st, x, (float*)y, n);
    else return (int)cudaErrorInvalidValue;
    KB_LAUNCH_RET();
}

// ------------------------------------------------------------------------------------------------ clamped gated unit
// gu: [n_planes][R][2F] (planes summed in order), 32-bit or the output's type; columns come in groups: `group` gate
// columns, then the `group` up columns of the same outputs (group == F: all gates, then all ups)
template <typename TIN, typename T>
__global__ void __launch_bounds__(256) k_glu_clamp(const TIN* KB_STEP_DATA gu, int n_planes, size_t plane_stride,
        int ldg, T* out, int ldo, int F, int group, float limit, float alpha) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c >= F) return;
    const size_t t = blockIdx.y;
    const TIN* g0 = gu + t * ldg + (size_t)(c / group) * 2 * group + c % group;
    float g = kb_to_f<TIN>(g0[0]), u = kb_to_f<TIN>(g0[group]);
    for (int s = 1; s < n_planes; s++) {
        g += kb_to_f<TIN>(g0[(size_t)s * plane_stride]);
        u += kb_to_f<TIN>(g0[(size_t)s * plane_stride + group]);
    }
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    out[t * ldo + c] = kb_from_f<T>(g / (1.0f + expf(-alpha * g)) * (u + 1.0f));
}

// bf16 rows in, bf16 out, eight columns a thread with 16-byte accesses; exp and the division by the fast intrinsics
// (their error is far below one bf16 rounding)
__global__ void __launch_bounds__(256) k_glu_clamp8(const bf16* KB_STEP_DATA gu, int ldg, bf16* out, int ldo, int F,
                                                    int group, float limit, float alpha) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int c = (blockIdx.x * 256 + threadIdx.x) * 8;
    if (c >= F) return;
    const size_t t = blockIdx.y;
    const bf16* g0 = gu + t * ldg + (size_t)(c / group) * 2 * group + c % group;
    const uint4 gv = *(const uint4*)g0, uv = *(const uint4*)(g0 + group);
    const __nv_bfloat162* g2 = (const __nv_bfloat162*)&gv;
    const __nv_bfloat162* u2 = (const __nv_bfloat162*)&uv;
    uint4 ov;
    __nv_bfloat162* o2 = (__nv_bfloat162*)&ov;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        float2 g = __bfloat1622float2(g2[j]), u = __bfloat1622float2(u2[j]);
        g.x = fminf(g.x, limit);
        g.y = fminf(g.y, limit);
        u.x = fminf(fmaxf(u.x, -limit), limit) + 1.0f;
        u.y = fminf(fmaxf(u.y, -limit), limit) + 1.0f;
        o2[j] = __floats2bfloat162_rn(__fdividef(g.x, 1.0f + __expf(-alpha * g.x)) * u.x,
                                      __fdividef(g.y, 1.0f + __expf(-alpha * g.y)) * u.y);
    }
    *(uint4*)(out + t * ldo + c) = ov;
}

extern "C" int kb_glu_clamp(const void* gu, int in_dtype, int n_planes, long long plane_stride, int ldg, void* out,
                            int dtype, int ldo, int R, int F, int group, float limit, float alpha, cudaStream_t st) {
    if (R <= 0 || F <= 0) return 0;
    if (group <= 0 || F % group || R > 65535 * 64) return (int)cudaErrorInvalidValue;
    for (int r0 = 0; r0 < R; r0 += 65535) {
        const int n = R - r0 < 65535 ? R - r0 : 65535;
        dim3 grid((F + 255) / 256, n);
        const size_t in_el = in_dtype == KB_F32 ? 4 : 2, out_el = dtype == KB_F32 ? 4 : 2;
        const void* gi = (const char*)gu + (size_t)r0 * ldg * in_el;
        void* oi = (char*)out + (size_t)r0 * ldo * out_el;
        if (in_dtype == KB_BF16 && dtype == KB_BF16 && n_planes == 1 && F % 8 == 0 && group % 8 == 0 && ldg % 8 == 0 &&
            ldo % 8 == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)out % 16) == 0) {
            dim3 g8((F / 8 + 255) / 256, n);
            kb_launch(k_glu_clamp8, g8, 256, 0, st, (const bf16*)gi, ldg, (bf16*)oi, ldo, F, group, limit, alpha);
        } else if (in_dtype == KB_F32 && dtype == KB_F32)
            kb_launch(k_glu_clamp<float, float>, grid, 256, 0, st, (const float*)gi, n_planes, (size_t)plane_stride,
                      ldg, (float*)oi, ldo, F, group, limit, alpha);
        else if (in_dtype == KB_F32 && dtype == KB_BF16)
            kb_launch(k_glu_clamp<float, bf16>, grid, 256, 0, st, (const float*)gi, n_planes, (size_t)plane_stride,
                      ldg, (bf16*)oi, ldo, F, group, limit, alpha);
        else if (in_dtype == KB_BF16 && dtype == KB_BF16)
            kb_launch(k_glu_clamp<bf16, bf16>, grid, 256, 0, st, (const bf16*)gi, n_planes, (size_t)plane_stride, ldg,
                      (bf16*)oi, ldo, F, group, limit, alpha);
        else return (int)cudaErrorInvalidValue;
    }
    KB_LAUNCH_RET();
}
