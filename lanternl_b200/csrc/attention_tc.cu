// Causal flash attention for training and prefill on the sm_100a tensor cores (bf16, head_dim 64 or 128):
// QK^T and PV are tcgen05.mma tiles with the accumulators in tensor memory, operands staged by TMA
// (128-byte swizzle), softmax on the CUDA cores in between with one thread per query row.
//
// What it replaces: the reference computes attention as per-sequence batched score GEMMs, a
// [B*H*T, T] softmax and a second batched GEMM (ai/gpu/gpu_transformer.lua:333-352, backward :431-470),
// materialising the T x T probabilities; here they never leave the SM.
//
// Every tensor-core operand is K-major (contraction dimension contiguous), the one layout the GEMM
// kernel of this library already uses.  Operands whose natural layout has the other orientation are
// transposed once per layer into head-major copies [B*H*hd, T] by a small kernel (V for the forward;
// Q, K and dO for the backward) instead of being addressed through MN-major descriptors.
//
// Forward, one CTA per (128 query rows, head, sequence), key tiles of 128, double-buffered:
//   warp 0    TMA producer: Q once, then K_j (from qkv) and V^T_j (from the head-major copy) per tile
//   warp 1    MMA issuer:   S = Q K_j^T  -> TMEM[0,128);  O_j = P V_j -> TMEM[128,128+hd)
//   warps 2-5 softmax:      thread r owns query row r: reads S from TMEM, online max / sum, writes P (bf16)
//                           into shared memory in the swizzled K-major layout, then folds O_j into its
//                           fp32 output row held in registers (rescaled when the maximum moves).
// All waits are bounded; one that runs out raises the library's error flag and the CTA winds down.
#include <cuda.h>

#include "ops.h"
#include "tc_common.cuh"

namespace {

using namespace tc;

constexpr int QT = 128, KT = 128;        // query rows and keys per tile
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

// [R, 3D] -> head-major transposes: dst[((b*H + h)*HD + d) * T + t] = src[(b*T + t) * pitch + col0 + h*HD + d]
__global__ void __launch_bounds__(256)
head_transpose_kernel(const bf16* __restrict__ src, bf16* __restrict__ dst, int T, int H, int HD, long long pitch, int col0)
{
    __shared__ bf16 tile[64][66];
    const int b = blockIdx.z / H, h = blockIdx.z % H;
    const int t0 = blockIdx.x * 64, d0 = blockIdx.y * 64;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int j = ty; j < 64; j += 8) {
        const int t = t0 + j;
        __nv_bfloat162 v = __floats2bfloat162_rn(0.0f, 0.0f);
        if (t < T) v = *reinterpret_cast<const __nv_bfloat162*>(src + ((size_t)b * T + t) * pitch + col0 + h * HD + d0 + 2 * tx);
        tile[j][2 * tx] = __low2bfloat16(v); tile[j][2 * tx + 1] = __high2bfloat16(v);
    }
    __syncthreads();
    for (int j = ty; j < 64; j += 8) {
        const int d = d0 + j, t = t0 + 2 * tx;
        if (t < T) {
            bf16* o = dst + ((size_t)(b * H + h) * HD + d) * T + t;
            if (t + 1 < T) *reinterpret_cast<__nv_bfloat162*>(o) = __halves2bfloat162(tile[2 * tx][j], tile[2 * tx + 1][j]);
            else o[0] = tile[2 * tx][j];
        }
    }
}

template <int HD>
struct FwdSmem {
    static constexpr int QB = QT * 128;                 // bytes of one 64-column k-block of a 128-row tile
    alignas(1024) uint8_t q[HD / 64][QT * 128];
    alignas(1024) uint8_t k[2][HD / 64][KT * 128];
    alignas(1024) uint8_t vt[2][KT / 64][HD * 128];
    alignas(1024) uint8_t p[KT / 64][QT * 128];
    alignas(8) uint64_t q_full, kv_full[2], kv_free[2], s_ready, p_ready, o_ready;
    uint32_t tmem_base;
};

template <int HD>
__global__ void __launch_bounds__(192, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_vt,
                   bf16* __restrict__ out, float* __restrict__ lse, int T, int H, float scale, int causal,
                   int* __restrict__ err)
{
    extern __shared__ uint8_t smem_raw[];
    FwdSmem<HD>& sm = *reinterpret_cast<FwdSmem<HD>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int KB = HD / 64;                         // k-blocks of the QK^T contraction
    constexpr uint32_t TMEM_COLS = 256;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q0 = blockIdx.x * QT, h = blockIdx.y, b = blockIdx.z;
    const int D = H * HD;
    const int ntiles = causal ? min((q0 + QT - 1) / KT + 1, (T + KT - 1) / KT) : (T + KT - 1) / KT;

    if (threadIdx.x == 0) {
        mbar_init(&sm.q_full, 1);
        for (int s = 0; s < 2; ++s) { mbar_init(&sm.kv_full[s], 1); mbar_init(&sm.kv_free[s], 1); }
        mbar_init(&sm.s_ready, 1); mbar_init(&sm.p_ready, 128); mbar_init(&sm.o_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sm.tmem_base;
    bool ok = true;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----
        const int row_q = b * T + q0;
        mbar_expect_tx(&sm.q_full, QT * HD * 2);
        for (int kb = 0; kb < KB; ++kb) tma_load_2d(sm.q[kb], &map_qkv, h * HD + kb * 64, row_q, &sm.q_full);
        for (int j = 0; j < ntiles && ok; ++j) {
            const int s = j & 1;
            if (j >= 2) ok = mbar_wait(&sm.kv_free[s], ((j >> 1) - 1) & 1);
            if (!ok) break;
            mbar_expect_tx(&sm.kv_full[s], 2 * KT * HD * 2);
            for (int kb = 0; kb < KB; ++kb) tma_load_2d(sm.k[s][kb], &map_qkv, D + h * HD + kb * 64, b * T + j * KT, &sm.kv_full[s]);
            for (int kb = 0; kb < KT / 64; ++kb) tma_load_2d(sm.vt[s][kb], &map_vt, j * KT + kb * 64, (b * H + h) * HD, &sm.kv_full[s]);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        constexpr uint32_t idesc_s = umma_idesc_bf16(QT, KT), idesc_o = umma_idesc_bf16(QT, HD);
        ok = mbar_wait(&sm.q_full, 0);
        for (int j = 0; j < ntiles && ok; ++j) {
            const int s = j & 1;
            ok = mbar_wait(&sm.kv_full[s], (j >> 1) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                const uint64_t da = umma_desc_sw128(smem_u32(sm.q[kb])), db = umma_desc_sw128(smem_u32(sm.k[s][kb]));
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_s, (kb | k) ? 1u : 0u);
            }
            umma_commit(&sm.s_ready);
            ok = mbar_wait(&sm.p_ready, j & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int kb = 0; kb < KT / 64; ++kb) {
                const uint64_t da = umma_desc_sw128(smem_u32(sm.p[kb])), db = umma_desc_sw128(smem_u32(sm.vt[s][kb]));
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(tmem + 128, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_o, (kb | k) ? 1u : 0u);
            }
            umma_commit(&sm.o_ready);
            umma_commit(&sm.kv_free[s]);
        }
    } else if (warp >= 2) {
        // ---- softmax: one thread per query row ----
        const int quad = warp & 3, r = quad * 32 + lane;
        const int qi = q0 + r;
        const uint32_t trow = tmem + ((uint32_t)(quad * 32) << 16);
        const float sl2 = scale * LOG2E;
        float m = -INFINITY, l = 0.0f;
        float acc[HD];
#pragma unroll
        for (int d = 0; d < HD; ++d) acc[d] = 0.0f;
        for (int j = 0; j < ntiles; ++j) {
            if (!mbar_wait(&sm.s_ready, j & 1)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int kbase = j * KT;
            const int klim = min(T, causal ? qi + 1 : T) - kbase;          // keys [0, klim) of this tile are visible
            float mx = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < KT; c += 32) {
                uint32_t v[32];
                tmem_ld32(trow + (uint32_t)c, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 32; ++i) if (c + i < klim) mx = fmaxf(mx, __uint_as_float(v[i]));
            }
            const float mn = fmaxf(m, mx * sl2);
            const float base = mn == -INFINITY ? 0.0f : mn;
            const float corr = exp2f(m - base);                           // m = -inf -> 0
            float sum = 0.0f;
#pragma unroll 1
            for (int c = 0; c < KT; c += 32) {
                uint32_t v[32];
                tmem_ld32(trow + (uint32_t)c, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const float p0 = c + i < klim ? exp2f(fmaf(__uint_as_float(v[i]), sl2, -base)) : 0.0f;
                    const float p1 = c + i + 1 < klim ? exp2f(fmaf(__uint_as_float(v[i + 1]), sl2, -base)) : 0.0f;
                    const __nv_bfloat162 t = __floats2bfloat162_rn(p0, p1);
                    // the sum uses the rounded probabilities, the values the second GEMM multiplies with
                    sum += __low2float(t) + __high2float(t);
                    pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&t);
                }
                // columns c .. c+31 of row r: four 16-byte chunks of k-block c / 64, swizzled by the row
                uint8_t* prow = sm.p[c >> 6] + r * 128;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int chunk = ((c & 63) >> 3) + q4;
                    *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
                }
            }
            l = fmaf(l, corr, sum);
            m = mn;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // P visible to the tensor core's reads
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.p_ready)) : "memory");
            if (!mbar_wait(&sm.o_ready, j & 1)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int c = 0; c < HD; c += 32) {
                uint32_t v[32];
                tmem_ld32(trow + 128u + (uint32_t)c, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[c + i] = fmaf(acc[c + i], corr, __uint_as_float(v[i]));
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        if (ok && qi < T) {
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            bf16* orow = out + ((size_t)b * T + qi) * D + h * HD;
#pragma unroll
            for (int d = 0; d < HD; d += 8) {
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = acc[d + i] * inv;
                st16<bf16>(orow + d, o);
            }
            if (lse) lse[((size_t)b * H + h) * T + qi] = (m == -INFINITY ? -INFINITY : m * LN2) + logf(fmaxf(l, 1e-30f));
        }
    }
    if (!ok && err) atomicExch(err, 1);
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}

template <int HD>
int launch_fwd_tc(const bf16* qkv, bf16* vt, bf16* out, float* lse, int B, int T, int H, float scale, int causal, cudaStream_t s)
{
    const int D = H * HD;
    dim3 tg((T + 63) / 64, HD / 64, B * H);
    head_transpose_kernel<<<tg, 256, 0, s>>>(qkv, vt, T, H, HD, 3LL * D, 2 * D);
    LTL_TRY(ltl_check_launch("attn head transpose"));
    CUtensorMap mq, mv;
    LTL_TRY(ltl_tensor_map_bf16(qkv, B * T, 3 * D, 3LL * D, 128, &mq));
    LTL_TRY(ltl_tensor_map_bf16(vt, B * H * HD, T, T, HD, &mv));
    const size_t smem = sizeof(FwdSmem<HD>) + 1024;
    static bool attr = false;
    if (!attr) {
        LTL_CUDA("attn_fwd_tc attr", cudaFuncSetAttribute(attn_fwd_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr = true;
    }
    dim3 grid((T + QT - 1) / QT, H, B);
    attn_fwd_tc_kernel<HD><<<grid, 192, smem, s>>>(mq, mv, out, lse, T, H, scale, causal, ltl_tc_err_flag());
    return ltl_check_launch("attn_fwd_tc");
}


// ---------------------------------------------------------------------------------------------------
// Backward, part 1: dQ.  One CTA per (128 query rows, head, sequence) walking the key tiles as the forward does.
//   S = Q K_j^T and dP = dO V_j^T (tensor memory)  ->  thread r: P = exp(S*scale - lse_r), dS = P (dP - delta_r) scale
//   -> dS (bf16) in shared memory, K-major  ->  dQ += dS K_j  with K_j^T read from the head-major copy of K.
// ---------------------------------------------------------------------------------------------------
template <int HD>
struct DqSmem {
    alignas(1024) uint8_t q[HD / 64][QT * 128];
    alignas(1024) uint8_t dout[HD / 64][QT * 128];
    alignas(1024) uint8_t k[HD / 64][KT * 128];
    alignas(1024) uint8_t v[HD / 64][KT * 128];
    alignas(1024) uint8_t kt[KT / 64][HD * 128];
    alignas(1024) uint8_t ds[KT / 64][QT * 128];
    alignas(8) uint64_t q_full, kv_full, kv_free, s_ready, ds_ready, acc_ready;
    uint32_t tmem_base;
};

template <int HD>
__global__ void __launch_bounds__(192, 1)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap map_qkv, const __grid_constant__ CUtensorMap map_do,
                      const __grid_constant__ CUtensorMap map_kt, const float* __restrict__ lse,
                      const float* __restrict__ delta, bf16* __restrict__ dqkv, int T, int H, float scale, int causal,
                      int* __restrict__ err)
{
    extern __shared__ uint8_t smem_raw[];
    DqSmem<HD>& sm = *reinterpret_cast<DqSmem<HD>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int KB = HD / 64;
    constexpr uint32_t TMEM_COLS = 512, COL_DP = 128, COL_DQ = 256;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q0 = blockIdx.x * QT, h = blockIdx.y, b = blockIdx.z;
    const int D = H * HD;
    const int ntiles = causal ? min((q0 + QT - 1) / KT + 1, (T + KT - 1) / KT) : (T + KT - 1) / KT;

    if (threadIdx.x == 0) {
        mbar_init(&sm.q_full, 1); mbar_init(&sm.kv_full, 1); mbar_init(&sm.kv_free, 1);
        mbar_init(&sm.s_ready, 1); mbar_init(&sm.ds_ready, 128); mbar_init(&sm.acc_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sm.tmem_base;
    bool ok = true;

    if (warp == 0 && lane == 0) {
        mbar_expect_tx(&sm.q_full, 2 * QT * HD * 2);
        for (int kb = 0; kb < KB; ++kb) {
            tma_load_2d(sm.q[kb], &map_qkv, h * HD + kb * 64, b * T + q0, &sm.q_full);
            tma_load_2d(sm.dout[kb], &map_do, h * HD + kb * 64, b * T + q0, &sm.q_full);
        }
        for (int j = 0; j < ntiles && ok; ++j) {
            if (j >= 1) ok = mbar_wait(&sm.kv_free, (j - 1) & 1);
            if (!ok) break;
            mbar_expect_tx(&sm.kv_full, 3 * KT * HD * 2);
            for (int kb = 0; kb < KB; ++kb) {
                tma_load_2d(sm.k[kb], &map_qkv, D + h * HD + kb * 64, b * T + j * KT, &sm.kv_full);
                tma_load_2d(sm.v[kb], &map_qkv, 2 * D + h * HD + kb * 64, b * T + j * KT, &sm.kv_full);
            }
            for (int kb = 0; kb < KT / 64; ++kb) tma_load_2d(sm.kt[kb], &map_kt, j * KT + kb * 64, (b * H + h) * HD, &sm.kv_full);
        }
    } else if (warp == 1 && lane == 0) {
        constexpr uint32_t idesc_s = umma_idesc_bf16(QT, KT), idesc_o = umma_idesc_bf16(QT, HD);
        ok = mbar_wait(&sm.q_full, 0);
        for (int j = 0; j < ntiles && ok; ++j) {
            ok = mbar_wait(&sm.kv_full, j & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                const uint64_t da = umma_desc_sw128(smem_u32(sm.q[kb])), db = umma_desc_sw128(smem_u32(sm.k[kb]));
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_s, (kb | k) ? 1u : 0u);
            }
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                const uint64_t da = umma_desc_sw128(smem_u32(sm.dout[kb])), db = umma_desc_sw128(smem_u32(sm.v[kb]));
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(tmem + COL_DP, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_s, (kb | k) ? 1u : 0u);
            }
            umma_commit(&sm.s_ready);
            ok = mbar_wait(&sm.ds_ready, j & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int kb = 0; kb < KT / 64; ++kb) {
                const uint64_t da = umma_desc_sw128(smem_u32(sm.ds[kb])), db = umma_desc_sw128(smem_u32(sm.kt[kb]));
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(tmem + COL_DQ, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_o, (j | kb | k) ? 1u : 0u);
            }
            umma_commit(&sm.kv_free);
        }
        if (ok) umma_commit(&sm.acc_ready);
    } else if (warp >= 2) {
        const int quad = warp & 3, r = quad * 32 + lane;
        const int qi = q0 + r;
        const uint32_t trow = tmem + ((uint32_t)(quad * 32) << 16);
        const float sl2 = scale * LOG2E;
        const size_t li = ((size_t)b * H + h) * T + (qi < T ? qi : 0);
        const float lse2 = lse[li] * LOG2E, dl = delta[li];
        for (int j = 0; j < ntiles; ++j) {
            if (!mbar_wait(&sm.s_ready, j & 1)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int klim = qi < T ? min(T, causal ? qi + 1 : T) - j * KT : 0;
#pragma unroll 1
            for (int c = 0; c < KT; c += 32) {
                uint32_t sv[32], dv[32];
                tmem_ld32(trow + (uint32_t)c, sv);
                tmem_ld32(trow + COL_DP + (uint32_t)c, dv);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                uint32_t pk[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float d0 = 0.0f, d1 = 0.0f;
                    if (c + i < klim) d0 = exp2f(fmaf(__uint_as_float(sv[i]), sl2, -lse2)) * (__uint_as_float(dv[i]) - dl) * scale;
                    if (c + i + 1 < klim) d1 = exp2f(fmaf(__uint_as_float(sv[i + 1]), sl2, -lse2)) * (__uint_as_float(dv[i + 1]) - dl) * scale;
                    const __nv_bfloat162 t = __floats2bfloat162_rn(d0, d1);
                    pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&t);
                }
                uint8_t* prow = sm.ds[c >> 6] + r * 128;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int chunk = ((c & 63) >> 3) + q4;
                    *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.ds_ready)) : "memory");
        }
        if (ok) ok = mbar_wait(&sm.acc_ready, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            bf16* orow = dqkv + ((size_t)b * T + qi) * 3 * D + h * HD;
#pragma unroll 1
            for (int c = 0; c < HD; c += 32) {
                uint32_t v[32];
                tmem_ld32(trow + COL_DQ + (uint32_t)c, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (qi < T) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        float o[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) o[e] = __uint_as_float(v[i + e]);
                        st16<bf16>(orow + c + i, o);
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    if (!ok && err) atomicExch(err, 1);
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}


// ---------------------------------------------------------------------------------------------------
// Backward, part 2: dK and dV.  One CTA per (128 keys, head, sequence) walking the query tiles (64 queries each)
// that can see those keys.  Everything is computed transposed, so that thread r owns key row r:
//   S^T = K Q_i^T and dP^T = V dO_i^T (tensor memory)
//   -> P^T = exp(S^T scale - lse_q), dS^T = P^T (dP^T - delta_q) scale, both bf16 into shared memory (K-major)
//   -> dV += P^T dO_i and dK += dS^T Q_i, with dO_i^T and Q_i^T read from the head-major copies, accumulated in
//      tensor memory over the whole walk.
// ---------------------------------------------------------------------------------------------------
constexpr int QS = 64;                   // queries per step of the dK / dV walk

template <int HD>
struct DkvSmem {
    alignas(1024) uint8_t k[HD / 64][KT * 128];
    alignas(1024) uint8_t v[HD / 64][KT * 128];
    alignas(1024) uint8_t q[HD / 64][QS * 128];         // Q_i   [64 queries x hd]   (B of S^T)
    alignas(1024) uint8_t dout[HD / 64][QS * 128];      // dO_i  [64 queries x hd]   (B of dP^T)
    alignas(1024) uint8_t qt[HD * 128];                 // Q_i^T [hd x 64 queries]   (B of dK)
    alignas(1024) uint8_t dot[HD * 128];                // dO_i^T[hd x 64 queries]   (B of dV)
    alignas(1024) uint8_t pt[KT * 128];                 // P^T   [128 keys x 64 queries]
    alignas(1024) uint8_t dst[KT * 128];                // dS^T  [128 keys x 64 queries]
    alignas(8) uint64_t kv_full, q_full, q_free, s_ready, p_ready, acc_ready;
    uint32_t tmem_base;
};

template <int HD>
__global__ void __launch_bounds__(192, 1)
attn_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap map_qkv,    // boxes of 128 rows (K, V tiles)
                       const __grid_constant__ CUtensorMap map_qkv64,  // boxes of 64 rows (Q_i)
                       const __grid_constant__ CUtensorMap map_do64,   // dO [R, D], boxes of 64 rows
                       const __grid_constant__ CUtensorMap map_qt,     // head-major Q^T, boxes hd x 64
                       const __grid_constant__ CUtensorMap map_dot,    // head-major dO^T, boxes hd x 64
                       const float* __restrict__ lse, const float* __restrict__ delta, bf16* __restrict__ dqkv,
                       int T, int H, float scale, int causal, int* __restrict__ err)
{
    extern __shared__ uint8_t smem_raw[];
    DkvSmem<HD>& sm = *reinterpret_cast<DkvSmem<HD>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int KB = HD / 64;
    constexpr uint32_t TMEM_COLS = 512, COL_DP = 64, COL_DV = 128, COL_DK = 256;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k0 = blockIdx.x * KT, h = blockIdx.y, b = blockIdx.z;
    const int D = H * HD;
    const int nq = (T + QS - 1) / QS;
    const int i0 = causal ? k0 / QS : 0;                // first query tile that sees key k0
    const int nsteps = nq - i0;

    if (threadIdx.x == 0) {
        mbar_init(&sm.kv_full, 1); mbar_init(&sm.q_full, 1); mbar_init(&sm.q_free, 1);
        mbar_init(&sm.s_ready, 1); mbar_init(&sm.p_ready, 128); mbar_init(&sm.acc_ready, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sm.tmem_base;
    bool ok = true;

    if (warp == 0 && lane == 0) {
        mbar_expect_tx(&sm.kv_full, 2 * KT * HD * 2);
        for (int kb = 0; kb < KB; ++kb) {
            tma_load_2d(sm.k[kb], &map_qkv, D + h * HD + kb * 64, b * T + k0, &sm.kv_full);
            tma_load_2d(sm.v[kb], &map_qkv, 2 * D + h * HD + kb * 64, b * T + k0, &sm.kv_full);
        }
        for (int st = 0; st < nsteps && ok; ++st) {
            const int qrow = (i0 + st) * QS;
            if (st >= 1) ok = mbar_wait(&sm.q_free, (st - 1) & 1);
            if (!ok) break;
            mbar_expect_tx(&sm.q_full, 4 * QS * HD * 2);
            for (int kb = 0; kb < KB; ++kb) {
                tma_load_2d(sm.q[kb], &map_qkv64, h * HD + kb * 64, b * T + qrow, &sm.q_full);
                tma_load_2d(sm.dout[kb], &map_do64, h * HD + kb * 64, b * T + qrow, &sm.q_full);
            }
            tma_load_2d(sm.qt, &map_qt, qrow, (b * H + h) * HD, &sm.q_full);
            tma_load_2d(sm.dot, &map_dot, qrow, (b * H + h) * HD, &sm.q_full);
        }
    } else if (warp == 1 && lane == 0) {
        constexpr uint32_t idesc_s = umma_idesc_bf16(KT, QS), idesc_o = umma_idesc_bf16(KT, HD);
        ok = mbar_wait(&sm.kv_full, 0);
        for (int st = 0; st < nsteps && ok; ++st) {
            ok = mbar_wait(&sm.q_full, st & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                const uint64_t da = umma_desc_sw128(smem_u32(sm.k[kb])), db = umma_desc_sw128(smem_u32(sm.q[kb]));
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_s, (kb | k) ? 1u : 0u);
            }
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                const uint64_t da = umma_desc_sw128(smem_u32(sm.v[kb])), db = umma_desc_sw128(smem_u32(sm.dout[kb]));
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(tmem + COL_DP, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_s, (kb | k) ? 1u : 0u);
            }
            umma_commit(&sm.s_ready);
            ok = mbar_wait(&sm.p_ready, st & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            {
                const uint64_t da = umma_desc_sw128(smem_u32(sm.pt)), db = umma_desc_sw128(smem_u32(sm.dot));
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(tmem + COL_DV, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_o, (st | k) ? 1u : 0u);
            }
            {
                const uint64_t da = umma_desc_sw128(smem_u32(sm.dst)), db = umma_desc_sw128(smem_u32(sm.qt));
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(tmem + COL_DK, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_o, (st | k) ? 1u : 0u);
            }
            umma_commit(&sm.q_free);
        }
        if (ok) umma_commit(&sm.acc_ready);
    } else if (warp >= 2) {
        const int quad = warp & 3, r = quad * 32 + lane;     // key row of the tile
        const int kj = k0 + r;
        const uint32_t trow = tmem + ((uint32_t)(quad * 32) << 16);
        const float sl2 = scale * LOG2E;
        // lse and delta of the queries are read straight from global memory: every thread of the CTA reads the same
        // 64 values per step (broadcast, L1 resident), and no CTA-wide barrier is needed inside the walk.
        const float* lse_h = lse + ((size_t)b * H + h) * T;
        const float* delta_h = delta + ((size_t)b * H + h) * T;
        for (int st = 0; st < nsteps; ++st) {
            const int qrow = (i0 + st) * QS;
            if (!mbar_wait(&sm.s_ready, st & 1)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // query q (column) sees key kj iff kj <= q (causal), q < T, kj < T
            const int qmin = causal ? kj : 0;
#pragma unroll 1
            for (int c = 0; c < QS; c += 32) {
                uint32_t sv[32], dv[32];
                tmem_ld32(trow + (uint32_t)c, sv);
                tmem_ld32(trow + COL_DP + (uint32_t)c, dv);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                uint32_t pp[16], pd[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float p0 = 0.0f, p1 = 0.0f, d0 = 0.0f, d1 = 0.0f;
                    const int qa = qrow + c + i;
                    if (kj < T && qa < T && qa >= qmin) {
                        p0 = exp2f(fmaf(__uint_as_float(sv[i]), sl2, -__ldg(lse_h + qa) * LOG2E));
                        d0 = p0 * (__uint_as_float(dv[i]) - __ldg(delta_h + qa)) * scale;
                    }
                    if (kj < T && qa + 1 < T && qa + 1 >= qmin) {
                        p1 = exp2f(fmaf(__uint_as_float(sv[i + 1]), sl2, -__ldg(lse_h + qa + 1) * LOG2E));
                        d1 = p1 * (__uint_as_float(dv[i + 1]) - __ldg(delta_h + qa + 1)) * scale;
                    }
                    const __nv_bfloat162 tp = __floats2bfloat162_rn(p0, p1), td = __floats2bfloat162_rn(d0, d1);
                    pp[i >> 1] = *reinterpret_cast<const uint32_t*>(&tp);
                    pd[i >> 1] = *reinterpret_cast<const uint32_t*>(&td);
                }
                uint8_t* prow = sm.pt + r * 128;
                uint8_t* drow = sm.dst + r * 128;
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const int chunk = (c >> 3) + q4;
                    *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = make_uint4(pp[4 * q4], pp[4 * q4 + 1], pp[4 * q4 + 2], pp[4 * q4 + 3]);
                    *reinterpret_cast<uint4*>(drow + ((chunk ^ (r & 7)) << 4)) = make_uint4(pd[4 * q4], pd[4 * q4 + 1], pd[4 * q4 + 2], pd[4 * q4 + 3]);
                }
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.p_ready)) : "memory");
        }
        if (ok) ok = mbar_wait(&sm.acc_ready, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            bf16* krow = dqkv + ((size_t)b * T + kj) * 3 * D + D + h * HD;
            bf16* vrow = krow + D;
#pragma unroll 1
            for (int c = 0; c < HD; c += 32) {
                uint32_t vk[32], vv[32];
                tmem_ld32(trow + COL_DK + (uint32_t)c, vk);
                tmem_ld32(trow + COL_DV + (uint32_t)c, vv);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (kj < T) {
#pragma unroll
                    for (int i = 0; i < 32; i += 8) {
                        float a[8], bb[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) { a[e] = __uint_as_float(vk[i + e]); bb[e] = __uint_as_float(vv[i + e]); }
                        st16<bf16>(krow + c + i, a);
                        st16<bf16>(vrow + c + i, bb);
                    }
                }
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    if (!ok && err) atomicExch(err, 1);
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLS) : "memory");
    }
}


template <int HD>
int launch_bwd_tc(const bf16* qkv, const bf16* dout, const float* lse, const float* delta, bf16* scratch, bf16* dqkv,
                  int B, int T, int H, float scale, int causal, cudaStream_t s)
{
    const int D = H * HD;
    const size_t hm = (size_t)B * H * HD * T;            // elements of one head-major copy
    bf16 *qt = scratch, *kt = scratch + hm, *dot = scratch + 2 * hm;
    dim3 tg((T + 63) / 64, HD / 64, B * H);
    head_transpose_kernel<<<tg, 256, 0, s>>>(qkv, qt, T, H, HD, 3LL * D, 0);
    head_transpose_kernel<<<tg, 256, 0, s>>>(qkv, kt, T, H, HD, 3LL * D, D);
    head_transpose_kernel<<<tg, 256, 0, s>>>(dout, dot, T, H, HD, (long long)D, 0);
    LTL_TRY(ltl_check_launch("attn head transpose"));
    CUtensorMap mq128, mq64, mdo128, mdo64, mqt, mkt, mdot;
    LTL_TRY(ltl_tensor_map_bf16(qkv, B * T, 3 * D, 3LL * D, 128, &mq128));
    LTL_TRY(ltl_tensor_map_bf16(qkv, B * T, 3 * D, 3LL * D, 64, &mq64));
    LTL_TRY(ltl_tensor_map_bf16(dout, B * T, D, D, 128, &mdo128));
    LTL_TRY(ltl_tensor_map_bf16(dout, B * T, D, D, 64, &mdo64));
    LTL_TRY(ltl_tensor_map_bf16(qt, B * H * HD, T, T, HD, &mqt));
    LTL_TRY(ltl_tensor_map_bf16(kt, B * H * HD, T, T, HD, &mkt));
    LTL_TRY(ltl_tensor_map_bf16(dot, B * H * HD, T, T, HD, &mdot));
    static bool attr = false;
    const size_t smem_q = sizeof(DqSmem<HD>) + 1024, smem_kv = sizeof(DkvSmem<HD>) + 1024;
    if (!attr) {
        LTL_CUDA("attn_bwd_tc attr", cudaFuncSetAttribute(attn_bwd_dq_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q));
        LTL_CUDA("attn_bwd_tc attr", cudaFuncSetAttribute(attn_bwd_dkv_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv));
        attr = true;
    }
    dim3 gq((T + QT - 1) / QT, H, B), gk((T + KT - 1) / KT, H, B);
    attn_bwd_dq_tc_kernel<HD><<<gq, 192, smem_q, s>>>(mq128, mdo128, mkt, lse, delta, dqkv, T, H, scale, causal, ltl_tc_err_flag());
    LTL_TRY(ltl_check_launch("attn_bwd_dq_tc"));
    attn_bwd_dkv_tc_kernel<HD><<<gk, 192, smem_kv, s>>>(mq128, mq64, mdo64, mqt, mdot, lse, delta, dqkv, T, H, scale, causal,
                                                        ltl_tc_err_flag());
    return ltl_check_launch("attn_bwd_dkv_tc");
}

}  // namespace

bool ltl_attn_tc_supported(int T, int H, int hd, int dtype)
{
    return dtype == LTL_BF16 && (hd == 64 || hd == 128) && T % 8 == 0 && T >= 64;
}

// vt: scratch of B*H*hd*T bf16 elements (the head-major copy of V).
int ltl_attn_fwd_tc(const void* qkv, void* vt, void* out, float* lse, int B, int T, int H, int hd, float scale, int causal,
                    cudaStream_t s)
{
    if (!qkv || !vt || !out) return ltl_fail(LTL_ERR_NULL, "attn_fwd_tc: null pointer");
    if (!ltl_attn_tc_supported(T, H, hd, LTL_BF16)) return ltl_fail(LTL_ERR_UNSUPPORTED, "attn_fwd_tc: head_dim %d, T %d", hd, T);
    if (B <= 0 || H <= 0 || B > 65535 || (long long)B * H > 65535) return ltl_fail(LTL_ERR_SHAPE, "attn_fwd_tc: grid too large");
    if (hd == 64) return launch_fwd_tc<64>((const bf16*)qkv, (bf16*)vt, (bf16*)out, lse, B, T, H, scale, causal, s);
    return launch_fwd_tc<128>((const bf16*)qkv, (bf16*)vt, (bf16*)out, lse, B, T, H, scale, causal, s);
}

// scratch: 3 * B*H*hd*T bf16 elements (head-major copies of Q, K and dO).  delta [B*H*T] is written here too.
int ltl_attn_bwd_tc(const void* qkv, const void* out, const void* dout, const float* lse, float* delta, void* scratch,
                    void* dqkv, int B, int T, int H, int hd, float scale, int causal, cudaStream_t s)
{
    if (!qkv || !out || !dout || !lse || !delta || !scratch || !dqkv) return ltl_fail(LTL_ERR_NULL, "attn_bwd_tc: null pointer");
    if (!ltl_attn_tc_supported(T, H, hd, LTL_BF16)) return ltl_fail(LTL_ERR_UNSUPPORTED, "attn_bwd_tc: head_dim %d, T %d", hd, T);
    if (B <= 0 || H <= 0 || B > 65535 || (long long)B * H > 65535) return ltl_fail(LTL_ERR_SHAPE, "attn_bwd_tc: grid too large");
    LTL_TRY(ltl_attn_delta(out, dout, delta, B, T, H, hd, LTL_BF16, s));
    if (hd == 64) return launch_bwd_tc<64>((const bf16*)qkv, (const bf16*)dout, lse, delta, (bf16*)scratch, (bf16*)dqkv, B, T, H, scale, causal, s);
    return launch_bwd_tc<128>((const bf16*)qkv, (const bf16*)dout, lse, delta, (bf16*)scratch, (bf16*)dqkv, B, T, H, scale, causal, s);
}
