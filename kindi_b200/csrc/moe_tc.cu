// The experts' grouped products on the 5th-generation tensor cores (bfloat16 in, 32-bit accumulate).
//
// The rows are the (row, pick) pairs sorted by expert (k_moe_plan with tiles of 128 rows). A work unit is one tile of up
// to 128 sorted rows of ONE expert times BN columns of that expert's weight matrix, over all of K: D = A_tile W_e^T.
// A [n_pairs][K] holds the sorted activation rows (for the up product they are gathered first, k_moe_gather; for the
// down product they are the up product's output), W [E * N][K] the experts' matrices one after another; both are
// read by TMA (boxes of 64 K-elements, 128-byte swizzle, zero fill past the tensors' ends, no multicast). A tile
// that ends inside the 128 rows or the BN columns reads on into the next expert's rows: those lanes and columns
// are computed and never stored. CTAs are persistent and take units c, c + gridDim.x, ...; the unit count comes from
// the plan on the device. Roles as in k_gemm_tc: a producer warp keeps a ring of stages full, one thread issues
// tcgen05.mma into one of two accumulators in tensor memory, four epilogue warps drain the other with tcgen05.ld.
//   up form:   H[r][n] = act(D) as bf16 at the sorted row r; for gated experts whose rows alternate in groups of 16
//              gate and 16 up rows, H[r][n / 2] = the finished unit (act(gate) * up, or the clamped unit);
//   down form: planes[pair % top][pair / top][n] = weight[pair] * D as float, pair = perm[r]: each row goes to
//              its token's row of the plane of its pick, so the planes' sum in order is the experts' weighted sum.
#include "sm100.cuh"

#define MT_BM 128
#define MT_BK 64
#define MT_THREADS 192          // warp 0: TMA, warp 1: MMA + TMEM owner, warps 2-5: epilogue

template <int BN, int STAGES>
struct MoeSmem {
    static constexpr int A_BYTES = MT_BM * MT_BK * 2;
    static constexpr int B_BYTES = BN * MT_BK * 2;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int BAR_OFF = STAGES * STAGE_BYTES;
    static constexpr int N_BARS = 2 * STAGES + 4;
    static constexpr int TOTAL = BAR_OFF + N_BARS * 8 + 16 + 1024;
    static_assert(TOTAL <= 227 * 1024, "shared memory of a CTA");
};

template <int BN, int STAGES, bool UP>
__global__ void __launch_bounds__(MT_THREADS) k_moe_gemm_tc(const __grid_constant__ CUtensorMap mapA,
        const __grid_constant__ CUtensorMap mapW, void* __restrict__ C, int ldc, size_t plane_stride, int N, int K,
        const int* KB_STEP_DATA n_tiles, const int* KB_STEP_DATA tile_e, const int* KB_STEP_DATA tile_r0,
        const int* KB_STEP_DATA offs, const int* KB_STEP_DATA perm, const float* KB_STEP_DATA wts, int top, int act,
        int* status, KbGate glu) {
    using S = MoeSmem<BN, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    const uint32_t sbase = smem_u32(smem);
    const uint32_t bar_full = sbase + S::BAR_OFF, bar_empty = bar_full + STAGES * 8;
    const uint32_t bar_acc_full = bar_empty + STAGES * 8, bar_acc_empty = bar_acc_full + 16;
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(smem + S::BAR_OFF + S::N_BARS * 8);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tilesQ = (N + BN - 1) / BN;
    const int total_kb = (K + MT_BK - 1) / MT_BK;
    constexpr uint32_t TMEM_COLS = BN <= 64 ? 128 : BN <= 128 ? 256 : 512;
    constexpr uint32_t ACC_COLS = TMEM_COLS / 2;

    kb_pdl_launch();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(bar_full + s * 8, 1);
            mbar_init(bar_empty + s * 8, 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(bar_acc_full + a * 8, 1);
            mbar_init(bar_acc_empty + a * 8, 4);
        }
        mbar_fence_init();
        tma_prefetch_desc(&mapA);
        tma_prefetch_desc(&mapW);
    }
    if (warp == 1) {
        tmem_alloc(smem_u32((const void*)tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    kb_pdl_wait();                                       // the plan and the rows come from earlier kernels of the step
    const int n_units = n_tiles[0] * tilesQ;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t n = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
                const int t = u / tilesQ, tq = u % tilesQ;
                const int e = tile_e[t], r0 = tile_r0[t];
                for (int kb = 0; kb < total_kb; kb++, n++) {
                    const int s = n % STAGES;
                    const uint32_t ph = (n / STAGES) & 1u;
                    if (!(ok = mbar_wait(bar_empty + s * 8, ph ^ 1u, status))) break;
                    mbar_expect_tx(bar_full + s * 8, S::STAGE_BYTES);
                    const uint32_t dst = sbase + s * S::STAGE_BYTES;
                    tma_load_2d(dst, &mapA, kb * MT_BK, r0, bar_full + s * 8);
                    tma_load_2d(dst + S::A_BYTES, &mapW, kb * MT_BK, e * N + tq * BN, bar_full + s * 8);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(MT_BM, BN);
            uint32_t n = 0, it = 0;
            bool ok = true;
            for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, it++) {
                const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
                if (!(ok = mbar_wait(bar_acc_empty + acc * 8, acc_ph ^ 1u, status))) break;
                tc_fence_after();
                const uint32_t d = tmem + acc * ACC_COLS;
                for (int kb = 0; kb < total_kb; kb++, n++) {
                    const int s = n % STAGES;
                    const uint32_t ph = (n / STAGES) & 1u;
                    if (!(ok = mbar_wait(bar_full + s * 8, ph, status))) break;
                    tc_fence_after();
                    const uint32_t a = sbase + s * S::STAGE_BYTES, b = a + S::A_BYTES;
#pragma unroll
                    for (int k = 0; k < MT_BK / 16; k++)
                        umma_bf16(d, umma_desc_sw128(a + k * 32), umma_desc_sw128(b + k * 32), idesc,
                                  (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(bar_empty + s * 8);
                }
                umma_commit(bar_acc_full + acc * 8);
            }
        }
    } else {
        // epilogue warps 2..5 own TMEM lanes 32 * (warp % 4) .. + 31; a thread holds one sorted row
        const int quarter = warp & 3;
        uint32_t it = 0;
        bool ok = true;
        for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, it++) {
            const int t = u / tilesQ, tq = u % tilesQ;
            const int e = tile_e[t], r0 = tile_r0[t];
            const int r = r0 + quarter * 32 + lane;
            const bool live = r < offs[e + 1];
            const int q0 = tq * BN;
            const uint32_t acc = it & 1u, acc_ph = (it >> 1) & 1u;
            if (!(ok = mbar_wait(bar_acc_full + acc * 8, acc_ph, status))) break;
            tc_fence_after();
            const uint32_t tbase = tmem + acc * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
            float f = 1.0f;
            uint8_t* crow = nullptr;
            if (live) {
                if (UP) {
                    crow = (uint8_t*)C + (size_t)r * ldc * 2;
                } else {
                    const int pair = perm[r];
                    f = wts[pair];
                    crow = (uint8_t*)C + ((size_t)(pair % top) * plane_stride + (size_t)(pair / top) * ldc) * 4;
                }
            }
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (q0 + c0 >= N) break;                         // past the expert's columns (uniform over the warp)
                uint32_t v[32];
                tmem_ld_32x32(tbase + c0, v);
                tmem_ld_wait();
                if (!live) continue;
                const int g0 = q0 + c0;
                if (UP && glu.act != 0) {
                    // gated experts whose unit is finished here: the expert's rows come in groups of 16 gate rows and
                    // the 16 up rows of the same outputs (N a multiple of 32), so this piece holds 16 whole outputs
                    bf16* dst = (bf16*)crow + (g0 >> 1);
                    if ((((uintptr_t)dst) & 15) == 0) {
                        uint32_t h[8];
#pragma unroll
                        for (int c = 0; c < 8; c++) {
                            __nv_bfloat162 p = __floats2bfloat162_rn(
                                kb_glu_fast(__uint_as_float(v[2 * c]), __uint_as_float(v[16 + 2 * c]), glu),
                                kb_glu_fast(__uint_as_float(v[2 * c + 1]), __uint_as_float(v[16 + 2 * c + 1]), glu));
                            h[c] = *(uint32_t*)&p;
                        }
                        *(uint4*)(dst) = make_uint4(h[0], h[1], h[2], h[3]);
                        *(uint4*)(dst + 8) = make_uint4(h[4], h[5], h[6], h[7]);
                    } else {
#pragma unroll
                        for (int c = 0; c < 16; c++)
                            dst[c] = __float2bfloat16_rn(kb_glu_fast(__uint_as_float(v[c]), __uint_as_float(v[16 + c]), glu));
                    }
                } else if (UP) {
                    bf16* dst = (bf16*)crow + g0;
                    if (g0 + 32 <= N && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            uint32_t h[4];
#pragma unroll
                            for (int c = 0; c < 4; c++) {
                                __nv_bfloat162 p = __floats2bfloat162_rn(kb_act(__uint_as_float(v[8 * j + 2 * c]), act),
                                                                         kb_act(__uint_as_float(v[8 * j + 2 * c + 1]), act));
                                h[c] = *(uint32_t*)&p;
                            }
                            *(uint4*)(dst + 8 * j) = make_uint4(h[0], h[1], h[2], h[3]);
                        }
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; c++)
                            if (g0 + c < N) dst[c] = __float2bfloat16_rn(kb_act(__uint_as_float(v[c]), act));
                    }
                } else {
                    float* dst = (float*)crow + g0;
                    if (g0 + 32 <= N && (((uintptr_t)dst) & 15) == 0) {
#pragma unroll
                        for (int j = 0; j < 8; j++)
                            *(float4*)(dst + 4 * j) = make_float4(__fmul_rn(f, __uint_as_float(v[4 * j])),
                                                                  __fmul_rn(f, __uint_as_float(v[4 * j + 1])),
                                                                  __fmul_rn(f, __uint_as_float(v[4 * j + 2])),
                                                                  __fmul_rn(f, __uint_as_float(v[4 * j + 3])));
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; c++)
                            if (g0 + c < N) dst[c] = __fmul_rn(f, __uint_as_float(v[c]));
                    }
                }
            }
            // this warp has read its lanes of the accumulator: hand them back to the MMA thread
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + acc * 8);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

static int moe_sm_count() {
    static int n = 0;
    if (!n) {
        int dev = 0;
        cudaGetDevice(&dev);
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    }
    return n;
}

template <int BN, int STAGES, bool UP>
static int launch_moe_tc(const CUtensorMap& ma, const CUtensorMap& mw, void* C, int ldc, long long plane_stride, int N,
                         int K, int max_tiles, const int* n_tiles, const int* tile_e, const int* tile_r0,
                         const int* offs, const int* perm, const float* wts, int top, int act, int* status,
                         cudaStream_t st, KbGate glu) {
    using S = MoeSmem<BN, STAGES>;
    auto kern = k_moe_gemm_tc<BN, STAGES, UP>;
    static char once_tag;
    if (kb_first_use(&once_tag)) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL);
        if (e != cudaSuccess) return (int)e;
    }
    const long long units = (long long)max_tiles * ((N + BN - 1) / BN);
    const int grid = units < moe_sm_count() ? (int)units : moe_sm_count();
    kb_launch(kern, grid, MT_THREADS, S::TOTAL, st, ma, mw, C, ldc, (size_t)plane_stride, N, K, n_tiles, tile_e,
              tile_r0, offs, perm, wts, top, act, status, glu);
    return (int)cudaGetLastError();
}

// the tile size the plan has to be made with for these products
extern "C" int kb_moe_gemm_tc_tile() { return MT_BM; }

// A: sorted rows [n_rows][K] bf16 (row stride lda); W: [E * N][K] bf16, contiguous. up != 0: C = H [n_rows][ldc] bf16;
// else C = planes (float) with row stride ldc and plane_stride elements between planes. bn: 64, 128 or 256.
// glu != 0 (up form, N a multiple of 32): every expert's rows are 16 gate rows, then the 16 up rows of the same outputs,
// group after group; `act` names the gated unit (KB_ACT_SILU, KB_ACT_GELU_TANH, or KB_ACT_GLU_CLAMP with its limit and
// alpha) and C = H [n_rows][N / 2] holds the finished unit.
extern "C" int kb_moe_gemm_tc(const void* A, int n_rows, int lda, const void* W, int E, int N, int K, void* C, int ldc,
                              long long plane_stride, int max_tiles, const int* n_tiles, const int* tile_e,
                              const int* tile_r0, const int* offs, const int* perm, const float* wts, int top, int act,
                              int up, int bn, int* status, cudaStream_t st, int glu = 0, float act_lim = 0.0f,
                              float act_alpha = 0.0f) {
    if (n_rows <= 0 || max_tiles <= 0 || N <= 0 || K <= 0) return 0;
    if ((K % 8) || (lda % 8)) return (int)cudaErrorInvalidValue;
    if (glu && (!up || (N % 32))) return (int)cudaErrorInvalidValue;
    KbGate gate = kb_gate_of(act, act_lim, act_alpha);
    if (!glu) gate.act = 0;
    CUtensorMap ma, mw;
    int rc;
    if ((rc = kb_make_map_bf16(&ma, A, (uint64_t)n_rows, K, lda, MT_BM))) return rc;
    if ((rc = kb_make_map_bf16(&mw, W, (uint64_t)E * N, K, K, bn))) return rc;
#define MT_GO(BN, ST)                                                                                             \
    return up ? launch_moe_tc<BN, ST, true>(ma, mw, C, ldc, plane_stride, N, K, max_tiles, n_tiles, tile_e, tile_r0, \
                                            offs, perm, wts, top, act, status, st, gate)                          \
              : launch_moe_tc<BN, ST, false>(ma, mw, C, ldc, plane_stride, N, K, max_tiles, n_tiles, tile_e,      \
                                             tile_r0, offs, perm, wts, top, act, status, st, gate)
    switch (bn) {
        case 64: MT_GO(64, 6);
        case 128: MT_GO(128, 6);
        case 256: MT_GO(256, 4);
        default: return (int)cudaErrorInvalidValue;
    }
#undef MT_GO
}

// Ys[r] = Y[perm[r] / top]: the activation rows in the plan's order (bf16 rows of K elements, K a multiple of 8)
__global__ void __launch_bounds__(256) k_moe_gather(const bf16* KB_STEP_DATA Y, int ldy, bf16* __restrict__ Ys, int K,
        const int* KB_STEP_DATA perm, int n_pairs, int top) {
    kb_pdl_launch();
    kb_pdl_wait();
    const int per_row = K / 8;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < (long long)n_pairs * per_row;
         i += (long long)gridDim.x * blockDim.x) {
        const int r = (int)(i / per_row), c = (int)(i % per_row);
        const int t = perm[r] / top;
        *(uint4*)(Ys + (size_t)r * K + c * 8) = *(const uint4*)(Y + (size_t)t * ldy + c * 8);
    }
}

extern "C" int kb_moe_gather(const void* Y, int ldy, void* Ys, int K, const int* perm, int n_pairs, int top,
                             cudaStream_t st) {
    if (n_pairs <= 0) return 0;
    if ((K % 8) || (ldy % 8) || ((uintptr_t)Y & 15) || ((uintptr_t)Ys & 15)) return (int)cudaErrorInvalidValue;
    const long long want = ((long long)n_pairs * (K / 8) + 255) / 256;
    const int blocks = (int)(want < 2368 ? want : 2368);
    kb_launch(k_moe_gather, blocks, 256, 0, st, (const bf16*)Y, ldy, (bf16*)Ys, K, perm, n_pairs, top);
    KB_LAUNCH_RET();
}
