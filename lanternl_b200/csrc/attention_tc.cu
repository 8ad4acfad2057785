// Causal flash attention for training and prefill on the sm_100a tensor cores (bf16, head_dim 64 or 128):
// QK^T and PV are tcgen05.mma tiles with the accumulators in tensor memory, operands staged by TMA
// (128-byte swizzle), softmax on the CUDA cores in between with one thread per query row.
//
// What it replaces: the reference computes attention as per-sequence batched score GEMMs, a
// [B*H*T, T] softmax and a second batched GEMM (ai/gpu/gpu_transformer.lua:333-352, backward :431-470),
// materialising the T x T probabilities; here they never leave the SM.
//
// Every operand is read from the packed qkv / dO matrices as it lies.  Tiles whose contraction dimension is the
// contiguous one (Q, K for the scores; V, dO for dP) are K-major operands; the same tiles serve as MN-major B
// operands where the contraction runs over their rows (V in P V; K in dS K; Q in dS^T Q; dO in P^T dO) - one
// shared-memory copy, two descriptors.  P, dS, P^T and dS^T are written by the softmax threads in the swizzled
// K-major layout.
//
// Forward, one CTA per (128 query rows, head, sequence), key tiles of 128, double-buffered:
//   warp 0    TMA producer: Q once, then K_j and V_j per tile
//   warp 1    MMA issuer:   S_j = Q K_j^T and O_j = P_j V_j into double-buffered tensor memory (S_{j+1} is issued
//                           before P_j V_j, so it runs while the softmax threads work on S_j)
//   warps 2-9 softmax:      two threads per query row, each owning 64 score columns and hd/2 output columns: S from
//                           TMEM, online max / sum, P (bf16) into shared memory in the swizzled K-major layout,
//                           O_j folded into the fp32 output row held in registers (rescaled when the maximum moves).
// All waits are bounded; one that runs out raises the library's error flag and the CTA winds down.
#include <cuda.h>

#include <type_traits>

#include "ops.h"
#include "tc_common.cuh"

namespace {

using namespace tc;

constexpr int QT = 128, KT = 128;        // query rows and keys per tile
constexpr float LOG2E = 1.4426950408889634f, LN2 = 0.6931471805599453f;

// 2^x on the special-function unit, one instruction (inputs here are <= 0 up to rounding; tiny results flush to 0).
__device__ __forceinline__ float ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int HD>
struct FwdSmem {
    alignas(1024) uint8_t q[HD / 64][QT * 128];
    alignas(1024) uint8_t k[2][HD / 64][KT * 128];
    alignas(1024) uint8_t v[2][HD / 64][KT * 128];
    alignas(1024) uint8_t p[KT / 64][QT * 128];
    float mx[2][2][QT];                                 // [tile parity][column half][row]: partial row maxima
    float lsum[2][QT];                                  // final exchange of the partial denominators
    int fail;
    alignas(8) uint64_t q_full, k_full[2], k_free[2], v_full[2], v_free[2], s_ready[2], p_ready, o_ready[2];
    uint32_t tmem_base;
};

// Software pipeline: S and O_j are double-buffered in tensor memory (S0, S1, O0, O1 = 512 columns at hd 128), so the
// tensor core computes S_{j+1} while the softmax threads work on S_j, and P_j V_j while they fold O_{j-1} into their
// output rows (the fold of a tile is deferred by one tile; the rescale factor of each tile is kept until then).
// Two threads per query row (eight softmax warps): thread (r, half) owns the 64 score columns and the hd/2 output
// columns of its half; the two exchange their partial row maximum through shared memory once per tile and their
// partial denominators once at the end.
constexpr int FWD_THREADS = 320;

template <int HD>
__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_tc_kernel(const __grid_constant__ CUtensorMap map_qkv, bf16* __restrict__ out, float* __restrict__ lse, int T, int H, float scale, int causal,
                   int* __restrict__ err)
{
    extern __shared__ uint8_t smem_raw[];
    FwdSmem<HD>& sm = *reinterpret_cast<FwdSmem<HD>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int KB = HD / 64;                         // k-blocks of the QK^T contraction
    constexpr int HH = HD / 2;                          // output columns per thread
    constexpr uint32_t TMEM_COLS = 512, COL_O = 256;    // S_b at 128 b, O_b at 256 + 128 b
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q0 = blockIdx.x * QT, h = blockIdx.y, b = blockIdx.z;
    const int D = H * HD;
    const int ntiles = causal ? min((q0 + QT - 1) / KT + 1, (T + KT - 1) / KT) : (T + KT - 1) / KT;

    if (threadIdx.x == 0) {
        mbar_init(&sm.q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&sm.k_full[s], 1); mbar_init(&sm.k_free[s], 1); mbar_init(&sm.v_full[s], 1); mbar_init(&sm.v_free[s], 1);
            mbar_init(&sm.s_ready[s], 1); mbar_init(&sm.o_ready[s], 1);
        }
        mbar_init(&sm.p_ready, 256);
        sm.fail = 0;
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
        // ---- TMA producer, K side: a K stage is free as soon as the scores that read it are done, one tile before
        //      the matching V stage, so K_{j+2} is requested early enough to hide its latency ----
        const int row_q = b * T + q0;
        mbar_expect_tx(&sm.q_full, QT * HD * 2);
        for (int kb = 0; kb < KB; ++kb) tma_load_2d(sm.q[kb], &map_qkv, h * HD + kb * 64, row_q, &sm.q_full);
        for (int j = 0; j < ntiles && ok; ++j) {
            const int s = j & 1;
            if (j >= 2) ok = mbar_wait(&sm.k_free[s], ((j >> 1) - 1) & 1);
            if (!ok) break;
            mbar_expect_tx(&sm.k_full[s], KT * HD * 2);
            for (int kb = 0; kb < KB; ++kb) tma_load_2d(sm.k[s][kb], &map_qkv, D + h * HD + kb * 64, b * T + j * KT, &sm.k_full[s]);
        }
    } else if (warp == 0 && lane == 16) {
        // ---- TMA producer, V side ----
        for (int j = 0; j < ntiles && ok; ++j) {
            const int s = j & 1;
            if (j >= 2) ok = mbar_wait(&sm.v_free[s], ((j >> 1) - 1) & 1);
            if (!ok) break;
            mbar_expect_tx(&sm.v_full[s], KT * HD * 2);
            for (int kb = 0; kb < KB; ++kb) tma_load_2d(sm.v[s][kb], &map_qkv, 2 * D + h * HD + kb * 64, b * T + j * KT, &sm.v_full[s]);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        constexpr uint32_t idesc_s = umma_idesc_bf16(QT, KT), idesc_o = umma_idesc_bf16_bmn(QT, HD);
        auto issue_s = [&](int j) {
            const int s = j & 1;
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                const uint64_t da = umma_desc_sw128(smem_u32(sm.q[kb])), db = umma_desc_sw128(smem_u32(sm.k[s][kb]));
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_bf16(tmem + (uint32_t)(s * 128), da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_s, (kb | k) ? 1u : 0u);
            }
            umma_commit(&sm.s_ready[s]);
            umma_commit(&sm.k_free[s]);
        };
        ok = mbar_wait(&sm.q_full, 0) && mbar_wait(&sm.k_full[0], 0);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_s(0);
        }
        for (int j = 0; j < ntiles && ok; ++j) {
            const int s = j & 1;
            if (j + 1 < ntiles) {
                // S buffer (j+1)&1 was last read for tile j-1: its softmax finished before p_ready(j-1), waited below
                ok = mbar_wait(&sm.k_full[s ^ 1], ((j + 1) >> 1) & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                issue_s(j + 1);
            }
            ok = mbar_wait(&sm.p_ready, j & 1) && mbar_wait(&sm.v_full[s], (j >> 1) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // O_j = P V_j: P is K-major (two blocks of 64 keys); V_j is read as it lies, [128 keys x hd] = an MN-major B
            // operand: hd column blocks KT * 128 bytes apart, 16 key rows (2048 bytes) further per UMMA.
#pragma unroll
            for (int ks = 0; ks < KT / 16; ++ks) {
                const uint64_t da = umma_desc_sw128(smem_u32(sm.p[ks >> 2])) + (uint64_t)((ks & 3) * 2);
                const uint64_t db = umma_desc_sw128_mn(smem_u32(sm.v[s][0]) + ks * 2048, KT * 128, 1024);
                umma_bf16(tmem + COL_O + (uint32_t)(s * 128), da, db, idesc_o, ks ? 1u : 0u);
            }
            umma_commit(&sm.o_ready[s]);
            umma_commit(&sm.v_free[s]);
        }
    } else if (warp >= 2) {
        // ---- softmax: two threads per query row ----
        const int quad = warp & 3, r = quad * 32 + lane, half = (warp - 2) >> 2;
        const int qi = q0 + r;
        const uint32_t trow = tmem + ((uint32_t)(quad * 32) << 16);
        const float sl2 = scale * LOG2E;
        volatile int* failp = &sm.fail;
        float m = -INFINITY, l = 0.0f, corr_prev = 0.0f;
        float acc[HH];
#pragma unroll
        for (int d = 0; d < HH; ++d) acc[d] = 0.0f;
        // acc = acc * corr + (this thread's half of) O_t, the product in O buffer t & 1
        auto fold = [&](int t, float corr) {
            const uint32_t ocol = trow + COL_O + (uint32_t)((t & 1) * 128 + half * HH);
            uint32_t v[HH];
#pragma unroll
            for (int c = 0; c < HH; c += 32) tmem_ld32(ocol + (uint32_t)c, *reinterpret_cast<uint32_t(*)[32]>(&v[c]));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int i = 0; i < HH; ++i) acc[i] = fmaf(acc[i], corr, __uint_as_float(v[i]));
        };
        // A wait that runs out must not strand the other threads at the per-tile barrier: the thread raises sm.fail,
        // keeps walking to the barrier, and everybody leaves together right after it.
        for (int j = 0; j < ntiles; ++j) {
            const uint32_t scol = trow + (uint32_t)((j & 1) * 128 + half * 64);
            if (!mbar_wait(&sm.s_ready[j & 1], (j >> 1) & 1)) *failp = 1;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int klim = min(T, causal ? qi + 1 : T) - j * KT - half * 64;   // visible columns among this thread's 64
            uint32_t v[64];
            tmem_ld32(scol, *reinterpret_cast<uint32_t(*)[32]>(&v[0]));
            tmem_ld32(scol + 32u, *reinterpret_cast<uint32_t(*)[32]>(&v[32]));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            // Only the tile on the diagonal (and a ragged last tile) needs the per-column mask.
            const bool full = klim >= 64;
            float mx = -INFINITY;
            if (full) {
                float m0 = __uint_as_float(v[0]), m1 = __uint_as_float(v[1]), m2 = __uint_as_float(v[2]), m3 = __uint_as_float(v[3]);
#pragma unroll
                for (int i = 4; i < 64; i += 4) {
                    m0 = fmaxf(m0, __uint_as_float(v[i])); m1 = fmaxf(m1, __uint_as_float(v[i + 1]));
                    m2 = fmaxf(m2, __uint_as_float(v[i + 2])); m3 = fmaxf(m3, __uint_as_float(v[i + 3]));
                }
                mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
            } else {
#pragma unroll
                for (int i = 0; i < 64; ++i) if (i < klim) mx = fmaxf(mx, __uint_as_float(v[i]));
            }
            sm.mx[j & 1][half][r] = mx;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (*failp) { ok = false; break; }
            mx = fmaxf(mx, sm.mx[j & 1][half ^ 1][r]);
            const float mn = fmaxf(m, mx * sl2);
            const float base = mn == -INFINITY ? 0.0f : mn;
            const float corr = ex2(m - base);                             // m = -inf -> 0
            // P of the previous tile must have been consumed before it is overwritten (and O_{j-1} is then complete)
            if (j > 0 && !mbar_wait(&sm.o_ready[(j - 1) & 1], ((j - 1) >> 1) & 1)) *failp = 1;
            float sum0 = 0.0f, sum1 = 0.0f;
            uint8_t* prow = sm.p[half] + r * 128;                        // k-block `half` holds this thread's 64 columns
            auto probs = [&](auto full_c) {
                constexpr bool FULL = decltype(full_c)::value;
#pragma unroll
                for (int c = 0; c < 64; c += 8) {
                    uint32_t pk[4];
#pragma unroll
                    for (int i = 0; i < 8; i += 2) {
                        float p0 = ex2(fmaf(__uint_as_float(v[c + i]), sl2, -base));
                        float p1 = ex2(fmaf(__uint_as_float(v[c + i + 1]), sl2, -base));
                        if (!FULL) { p0 = c + i < klim ? p0 : 0.0f; p1 = c + i + 1 < klim ? p1 : 0.0f; }
                        sum0 += p0; sum1 += p1;
                        const __nv_bfloat162 t = __floats2bfloat162_rn(p0, p1);
                        pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&t);
                    }
                    *reinterpret_cast<uint4*>(prow + (((c >> 3) ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
            };
            if (full) probs(std::true_type{}); else probs(std::false_type{});
            const float sum = sum0 + sum1;
            l = fmaf(l, corr, sum);
            m = mn;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // P visible to the tensor core's reads
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.p_ready)) : "memory");
            if (j > 0) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                fold(j - 1, corr_prev);
            }
            corr_prev = corr;
        }
        if (ok && ntiles > 0) {
            if (!mbar_wait(&sm.o_ready[(ntiles - 1) & 1], ((ntiles - 1) >> 1) & 1)) *failp = 1;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            fold(ntiles - 1, corr_prev);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        if (ok) {                                        // uniform: `ok` only falls right after a barrier, for everybody
            sm.lsum[half][r] = l;
            asm volatile("bar.sync 1, 256;" ::: "memory");
            if (*failp) ok = false;
            l += sm.lsum[half ^ 1][r];
        }
        if (ok && qi < T) {
            const float inv = l > 0.0f ? 1.0f / l : 0.0f;
            bf16* orow = out + ((size_t)b * T + qi) * D + h * HD + half * HH;
#pragma unroll
            for (int d = 0; d < HH; d += 8) {
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = acc[d + i] * inv;
                st16<bf16>(orow + d, o);
            }
            if (lse && half == 0) lse[((size_t)b * H + h) * T + qi] = (m == -INFINITY ? -INFINITY : m * LN2) + logf(fmaxf(l, 1e-30f));
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
int launch_fwd_tc(const bf16* qkv, bf16* out, float* lse, int B, int T, int H, float scale, int causal, cudaStream_t s)
{
    const int D = H * HD;
    CUtensorMap mq;
    LTL_TRY(ltl_tensor_map_bf16(qkv, B * T, 3 * D, 3LL * D, 128, &mq));
    const size_t smem = sizeof(FwdSmem<HD>) + 1024;
    static bool attr = false;
    if (!attr) {
        LTL_CUDA("attn_fwd_tc attr", cudaFuncSetAttribute(attn_fwd_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr = true;
    }
    dim3 grid((T + QT - 1) / QT, H, B);
    attn_fwd_tc_kernel<HD><<<grid, FWD_THREADS, smem, s>>>(mq, out, lse, T, H, scale, causal, ltl_tc_err_flag());
    return ltl_check_launch("attn_fwd_tc");
}

// ---------------------------------------------------------------------------------------------------
// Backward, part 1: dQ.  One CTA per (128 query rows, head, sequence) walking key tiles of 64.
//   S = Q K_j^T and dP = dO V_j^T (tensor memory, double-buffered: the pair for tile j+1 is computed while the
//   threads work on tile j)  ->  P = exp(S scale - lse_r), dS = P (dP - delta_r) scale  ->  dS (bf16) in shared
//   memory, K-major  ->  dQ += dS K_j with K_j^T read from the head-major copy of K.
// Two threads per query row (eight warps), 32 key columns each; nothing is exchanged between them.
// ---------------------------------------------------------------------------------------------------
constexpr int KS = 64;                   // keys per tile of the dQ walk
constexpr int BWD_THREADS = 320;

constexpr int DQ_ST = 4;                 // K / V ring depth of the dQ walk (S / dP stay double-buffered in tensor memory)

template <int HD>
struct DqSmem {
    alignas(1024) uint8_t q[HD / 64][QT * 128];
    alignas(1024) uint8_t dout[HD / 64][QT * 128];
    alignas(1024) uint8_t k[DQ_ST][HD / 64][KS * 128];
    alignas(1024) uint8_t v[DQ_ST][HD / 64][KS * 128];
    alignas(1024) uint8_t ds[QT * 128];
    alignas(8) uint64_t q_full, kv_full[DQ_ST], kv_free[DQ_ST], sd_ready[2], ds_ready, acc_ready;
    uint32_t tmem_base;
};

template <int HD>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dq_tc_kernel(const __grid_constant__ CUtensorMap map_qkv,     // boxes of 128 rows (Q)
                      const __grid_constant__ CUtensorMap map_qkv64,   // boxes of 64 rows (K_j, V_j)
                      const __grid_constant__ CUtensorMap map_do,      // dO, boxes of 128 rows
                      const float* __restrict__ lse, const float* __restrict__ delta, bf16* __restrict__ dqkv,
                      int T, int H, float scale, int causal, int* __restrict__ err)
{
    extern __shared__ uint8_t smem_raw[];
    DqSmem<HD>& sm = *reinterpret_cast<DqSmem<HD>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int KB = HD / 64;
    constexpr uint32_t TMEM_COLS = 512, COL_DP = 128, COL_DQ = 256;      // S_b at 64 b, dP_b at 128 + 64 b
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q0 = blockIdx.x * QT, h = blockIdx.y, b = blockIdx.z;
    const int D = H * HD;
    const int ntiles = causal ? min((q0 + QT - 1) / KS + 1, (T + KS - 1) / KS) : (T + KS - 1) / KS;

    if (threadIdx.x == 0) {
        mbar_init(&sm.q_full, 1);
        for (int s = 0; s < DQ_ST; ++s) { mbar_init(&sm.kv_full[s], 1); mbar_init(&sm.kv_free[s], 1); }
        for (int s = 0; s < 2; ++s) mbar_init(&sm.sd_ready[s], 1);
        mbar_init(&sm.ds_ready, 256); mbar_init(&sm.acc_ready, 1);
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
            const int s = j % DQ_ST;
            if (j >= DQ_ST) ok = mbar_wait(&sm.kv_free[s], ((j / DQ_ST) - 1) & 1);
            if (!ok) break;
            mbar_expect_tx(&sm.kv_full[s], 2 * KS * HD * 2);
            for (int kb = 0; kb < KB; ++kb) {
                tma_load_2d(sm.k[s][kb], &map_qkv64, D + h * HD + kb * 64, b * T + j * KS, &sm.kv_full[s]);
                tma_load_2d(sm.v[s][kb], &map_qkv64, 2 * D + h * HD + kb * 64, b * T + j * KS, &sm.kv_full[s]);
            }
        }
    } else if (warp == 1 && lane == 0) {
        constexpr uint32_t idesc_s = umma_idesc_bf16(QT, KS), idesc_o = umma_idesc_bf16_bmn(QT, HD);
        auto issue_sd = [&](int j) {
            const int s = j % DQ_ST, tb = j & 1;        // shared-memory stage, tensor-memory buffer
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                const uint64_t da = umma_desc_sw128(smem_u32(sm.q[kb])), db = umma_desc_sw128(smem_u32(sm.k[s][kb]));
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_bf16(tmem + (uint32_t)(tb * KS), da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_s, (kb | k) ? 1u : 0u);
            }
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                const uint64_t da = umma_desc_sw128(smem_u32(sm.dout[kb])), db = umma_desc_sw128(smem_u32(sm.v[s][kb]));
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_bf16(tmem + COL_DP + (uint32_t)(tb * KS), da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_s, (kb | k) ? 1u : 0u);
            }
            umma_commit(&sm.sd_ready[tb]);
        };
        ok = mbar_wait(&sm.q_full, 0) && mbar_wait(&sm.kv_full[0], 0);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_sd(0);
        }
        for (int j = 0; j < ntiles && ok; ++j) {
            const int s = j % DQ_ST;
            if (j + 1 < ntiles) {
                ok = mbar_wait(&sm.kv_full[(j + 1) % DQ_ST], ((j + 1) / DQ_ST) & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                issue_sd(j + 1);
            }
            ok = mbar_wait(&sm.ds_ready, j & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // dQ += dS K_j: K_j as it lies, [64 keys x hd] = an MN-major B operand (hd column blocks KS * 128 bytes apart)
            const uint64_t da = umma_desc_sw128(smem_u32(sm.ds));
#pragma unroll
            for (int k = 0; k < 4; ++k)
                umma_bf16(tmem + COL_DQ, da + (uint64_t)(k * 2), umma_desc_sw128_mn(smem_u32(sm.k[s][0]) + k * 2048, KS * 128, 1024),
                          idesc_o, (j | k) ? 1u : 0u);
            umma_commit(&sm.kv_free[s]);                 // also: dS of tile j has been consumed
        }
        if (ok) umma_commit(&sm.acc_ready);
    } else if (warp >= 2) {
        const int quad = warp & 3, r = quad * 32 + lane, half = (warp - 2) >> 2;
        const int qi = q0 + r;
        const uint32_t trow = tmem + ((uint32_t)(quad * 32) << 16);
        const float sl2 = scale * LOG2E;
        const size_t li = ((size_t)b * H + h) * T + (qi < T ? qi : 0);
        const float lse2 = lse[li] * LOG2E, dls = delta[li] * scale;
        for (int j = 0; j < ntiles; ++j) {
            const uint32_t col = (uint32_t)((j & 1) * KS + half * 32);
            if (!mbar_wait(&sm.sd_ready[j & 1], (j >> 1) & 1)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int klim = qi < T ? min(T, causal ? qi + 1 : T) - j * KS - half * 32 : 0;
            uint32_t sv[32], dv[32];
            tmem_ld32(trow + col, sv);
            tmem_ld32(trow + COL_DP + col, dv);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            uint32_t pk[16];
            auto body = [&](auto full_c) {
                constexpr bool FULL = decltype(full_c)::value;
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float d0 = ex2(fmaf(__uint_as_float(sv[i]), sl2, -lse2)) * fmaf(__uint_as_float(dv[i]), scale, -dls);
                    float d1 = ex2(fmaf(__uint_as_float(sv[i + 1]), sl2, -lse2)) * fmaf(__uint_as_float(dv[i + 1]), scale, -dls);
                    if (!FULL) { d0 = i < klim ? d0 : 0.0f; d1 = i + 1 < klim ? d1 : 0.0f; }
                    const __nv_bfloat162 t = __floats2bfloat162_rn(d0, d1);
                    pk[i >> 1] = *reinterpret_cast<const uint32_t*>(&t);
                }
            };
            if (klim >= 32) body(std::true_type{}); else body(std::false_type{});
            // dS of the previous tile must have been consumed by its dQ product before it is overwritten
            if (j > 0 && !mbar_wait(&sm.kv_free[(j - 1) % DQ_ST], ((j - 1) / DQ_ST) & 1)) { ok = false; break; }
            uint8_t* prow = sm.ds + r * 128;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                const int chunk = half * 4 + q4;
                *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = make_uint4(pk[4 * q4], pk[4 * q4 + 1], pk[4 * q4 + 2], pk[4 * q4 + 3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.ds_ready)) : "memory");
        }
        if (ok) ok = mbar_wait(&sm.acc_ready, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            constexpr int HH = HD / 2;
            bf16* orow = dqkv + ((size_t)b * T + qi) * 3 * D + h * HD + half * HH;
#pragma unroll 1
            for (int c = 0; c < HH; c += 32) {
                uint32_t v[32];
                tmem_ld32(trow + COL_DQ + (uint32_t)(half * HH + c), v);
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
// that can see those keys.  Everything is computed transposed, so that a thread owns a key row:
//   S^T = K Q_i^T and dP^T = V dO_i^T (tensor memory, double-buffered: step i+1 is computed while the threads work
//   on step i)  ->  P^T = exp(S^T scale - lse_q), dS^T = P^T (dP^T - delta_q) scale, both bf16 into shared memory
//   (K-major)  ->  dV += P^T dO_i and dK += dS^T Q_i, with dO_i^T and Q_i^T read from the head-major copies,
//   accumulated in tensor memory over the whole walk.
// Two threads per key row (eight warps), 32 query columns each.  lse and delta of a step's 64 queries are staged in
// shared memory by the producer warp.
// ---------------------------------------------------------------------------------------------------
constexpr int QS = 64;                   // queries per step of the dK / dV walk

constexpr int KV_ST = 3;                 // Q / dO ring depth of the dK / dV walk

template <int HD>
struct DkvSmem {
    alignas(1024) uint8_t k[HD / 64][KT * 128];
    alignas(1024) uint8_t v[HD / 64][KT * 128];
    alignas(1024) uint8_t q[KV_ST][HD / 64][QS * 128];      // Q_i  [64 queries x hd]: K-major B of S^T, MN-major B of dK
    alignas(1024) uint8_t dout[KV_ST][HD / 64][QS * 128];   // dO_i [64 queries x hd]: K-major B of dP^T, MN-major B of dV
    alignas(1024) uint8_t pt[KT * 128];                 // P^T   [128 keys x 64 queries]
    alignas(1024) uint8_t dst[KT * 128];                // dS^T  [128 keys x 64 queries]
    float lse2[KV_ST][QS], dls[KV_ST][QS];                      // per step: lse * log2(e), delta * scale
    alignas(8) uint64_t kv_full, q_full[KV_ST], q_free[KV_ST], aux_full[KV_ST], sd_ready[2], p_ready, acc_ready;
    uint32_t tmem_base;
};

template <int HD>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_dkv_tc_kernel(const __grid_constant__ CUtensorMap map_qkv,    // boxes of 128 rows (K, V tiles)
                       const __grid_constant__ CUtensorMap map_qkv64,  // boxes of 64 rows (Q_i)
                       const __grid_constant__ CUtensorMap map_do64,   // dO [R, D], boxes of 64 rows
                       const float* __restrict__ lse, const float* __restrict__ delta, bf16* __restrict__ dqkv,
                       int T, int H, float scale, int causal, int* __restrict__ err)
{
    extern __shared__ uint8_t smem_raw[];
    DkvSmem<HD>& sm = *reinterpret_cast<DkvSmem<HD>*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int KB = HD / 64;
    constexpr uint32_t TMEM_COLS = 512, COL_DP = 128, COL_DV = 256, COL_DK = 384;   // S^T_b at 64 b, dP^T_b at 128 + 64 b
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int k0 = blockIdx.x * KT, h = blockIdx.y, b = blockIdx.z;
    const int D = H * HD;
    const int nq = (T + QS - 1) / QS;
    const int i0 = causal ? k0 / QS : 0;                // first query tile that sees key k0
    const int nsteps = nq - i0;

    if (threadIdx.x == 0) {
        mbar_init(&sm.kv_full, 1); mbar_init(&sm.p_ready, 256); mbar_init(&sm.acc_ready, 1);
        for (int s = 0; s < KV_ST; ++s) { mbar_init(&sm.q_full[s], 1); mbar_init(&sm.q_free[s], 1); mbar_init(&sm.aux_full[s], 1); }
        for (int s = 0; s < 2; ++s) mbar_init(&sm.sd_ready[s], 1);
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

    if (warp == 0) {
        // ---- producer warp: lane 0 issues the TMA loads, all lanes stage lse / delta of the step's queries ----
        if (lane == 0) {
            mbar_expect_tx(&sm.kv_full, 2 * KT * HD * 2);
            for (int kb = 0; kb < KB; ++kb) {
                tma_load_2d(sm.k[kb], &map_qkv, D + h * HD + kb * 64, b * T + k0, &sm.kv_full);
                tma_load_2d(sm.v[kb], &map_qkv, 2 * D + h * HD + kb * 64, b * T + k0, &sm.kv_full);
            }
        }
        const float* lse_h = lse + ((size_t)b * H + h) * T;
        const float* delta_h = delta + ((size_t)b * H + h) * T;
        for (int st = 0; st < nsteps; ++st) {
            const int s = st % KV_ST, qrow = (i0 + st) * QS;
            // stage s (operands and lse / delta) was last used by step st - KV_ST: free once its dV / dK products are done
            if (st >= KV_ST && lane == 0) ok = mbar_wait(&sm.q_free[s], ((st / KV_ST) - 1) & 1);
            ok = __shfl_sync(0xFFFFFFFFu, (int)ok, 0) != 0;
            if (!ok) break;
            if (lane == 0) {
                mbar_expect_tx(&sm.q_full[s], 2 * QS * HD * 2);
                for (int kb = 0; kb < KB; ++kb) {
                    tma_load_2d(sm.q[s][kb], &map_qkv64, h * HD + kb * 64, b * T + qrow, &sm.q_full[s]);
                    tma_load_2d(sm.dout[s][kb], &map_do64, h * HD + kb * 64, b * T + qrow, &sm.q_full[s]);
                }
            }
#pragma unroll
            for (int e = lane; e < QS; e += 32) {
                const int qq = qrow + e;
                sm.lse2[s][e] = qq < T ? lse_h[qq] * LOG2E : 0.0f;
                sm.dls[s][e] = qq < T ? delta_h[qq] * scale : 0.0f;
            }
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.aux_full[s])) : "memory");
        }
    } else if (warp == 1 && lane == 0) {
        constexpr uint32_t idesc_s = umma_idesc_bf16(KT, QS), idesc_o = umma_idesc_bf16_bmn(KT, HD);
        auto issue_sd = [&](int st) {
            const int s = st % KV_ST, tb = st & 1;      // shared-memory stage, tensor-memory buffer
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                const uint64_t da = umma_desc_sw128(smem_u32(sm.k[kb])), db = umma_desc_sw128(smem_u32(sm.q[s][kb]));
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_bf16(tmem + (uint32_t)(tb * QS), da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_s, (kb | k) ? 1u : 0u);
            }
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                const uint64_t da = umma_desc_sw128(smem_u32(sm.v[kb])), db = umma_desc_sw128(smem_u32(sm.dout[s][kb]));
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_bf16(tmem + COL_DP + (uint32_t)(tb * QS), da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc_s, (kb | k) ? 1u : 0u);
            }
            umma_commit(&sm.sd_ready[tb]);
        };
        ok = mbar_wait(&sm.kv_full, 0) && mbar_wait(&sm.q_full[0], 0);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_sd(0);
        }
        for (int st = 0; st < nsteps && ok; ++st) {
            const int s = st % KV_ST;
            if (st + 1 < nsteps) {
                ok = mbar_wait(&sm.q_full[(st + 1) % KV_ST], ((st + 1) / KV_ST) & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                issue_sd(st + 1);
            }
            ok = mbar_wait(&sm.p_ready, st & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            {   // dV += P^T dO_i and dK += dS^T Q_i: dO_i and Q_i as they lie, [64 queries x hd] = MN-major B operands
                const uint64_t dp = umma_desc_sw128(smem_u32(sm.pt)), dd = umma_desc_sw128(smem_u32(sm.dst));
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_bf16(tmem + COL_DV, dp + (uint64_t)(k * 2), umma_desc_sw128_mn(smem_u32(sm.dout[s][0]) + k * 2048, QS * 128, 1024),
                              idesc_o, (st | k) ? 1u : 0u);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_bf16(tmem + COL_DK, dd + (uint64_t)(k * 2), umma_desc_sw128_mn(smem_u32(sm.q[s][0]) + k * 2048, QS * 128, 1024),
                              idesc_o, (st | k) ? 1u : 0u);
            }
            umma_commit(&sm.q_free[s]);                  // the step's operands, and P^T / dS^T, have been consumed
        }
        if (ok) umma_commit(&sm.acc_ready);
    } else if (warp >= 2) {
        const int quad = warp & 3, r = quad * 32 + lane, half = (warp - 2) >> 2;     // key row, column half
        const int kj = k0 + r;
        const uint32_t trow = tmem + ((uint32_t)(quad * 32) << 16);
        const float sl2 = scale * LOG2E;
        for (int st = 0; st < nsteps; ++st) {
            const int s = st % KV_ST, tb = st & 1, qbase = (i0 + st) * QS + half * 32;   // first query of this thread's columns
            const uint32_t col = (uint32_t)(tb * QS + half * 32);
            if (!mbar_wait(&sm.sd_ready[tb], (st >> 1) & 1) || !mbar_wait(&sm.aux_full[s], (st / KV_ST) & 1)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t sv[32], dv[32];
            tmem_ld32(trow + col, sv);
            tmem_ld32(trow + COL_DP + col, dv);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            // column i (query qbase + i) sees key kj iff kj <= query (causal), query < T, kj < T
            const int lo = (causal ? kj : 0) - qbase, hi = (kj < T ? T : 0) - qbase;   // visible: lo <= i < hi
            const float* l2p = sm.lse2[s] + half * 32;
            const float* dlp = sm.dls[s] + half * 32;
            uint32_t pp[16], pd[16];
            auto body = [&](auto full_c) {
                constexpr bool FULL = decltype(full_c)::value;
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    float p0 = ex2(fmaf(__uint_as_float(sv[i]), sl2, -l2p[i]));
                    float p1 = ex2(fmaf(__uint_as_float(sv[i + 1]), sl2, -l2p[i + 1]));
                    if (!FULL) { p0 = (i >= lo && i < hi) ? p0 : 0.0f; p1 = (i + 1 >= lo && i + 1 < hi) ? p1 : 0.0f; }
                    const float d0 = p0 * fmaf(__uint_as_float(dv[i]), scale, -dlp[i]);
                    const float d1 = p1 * fmaf(__uint_as_float(dv[i + 1]), scale, -dlp[i + 1]);
                    const __nv_bfloat162 tp = __floats2bfloat162_rn(p0, p1), td = __floats2bfloat162_rn(d0, d1);
                    pp[i >> 1] = *reinterpret_cast<const uint32_t*>(&tp);
                    pd[i >> 1] = *reinterpret_cast<const uint32_t*>(&td);
                }
            };
            if (lo <= 0 && hi >= 32) body(std::true_type{}); else body(std::false_type{});
            // P^T / dS^T of the previous step must have been consumed before they are overwritten
            if (st > 0 && !mbar_wait(&sm.q_free[(st - 1) % KV_ST], ((st - 1) / KV_ST) & 1)) { ok = false; break; }
            uint8_t* prow = sm.pt + r * 128;
            uint8_t* drow = sm.dst + r * 128;
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
                const int chunk = half * 4 + q4;
                *reinterpret_cast<uint4*>(prow + ((chunk ^ (r & 7)) << 4)) = make_uint4(pp[4 * q4], pp[4 * q4 + 1], pp[4 * q4 + 2], pp[4 * q4 + 3]);
                *reinterpret_cast<uint4*>(drow + ((chunk ^ (r & 7)) << 4)) = make_uint4(pd[4 * q4], pd[4 * q4 + 1], pd[4 * q4 + 2], pd[4 * q4 + 3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.p_ready)) : "memory");
        }
        if (ok) ok = mbar_wait(&sm.acc_ready, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            constexpr int HH = HD / 2;
            bf16* krow = dqkv + ((size_t)b * T + kj) * 3 * D + D + h * HD + half * HH;
            bf16* vrow = krow + D;
#pragma unroll 1
            for (int c = 0; c < HH; c += 32) {
                uint32_t vk[32], vv[32];
                tmem_ld32(trow + COL_DK + (uint32_t)(half * HH + c), vk);
                tmem_ld32(trow + COL_DV + (uint32_t)(half * HH + c), vv);
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
int launch_bwd_tc(const bf16* qkv, const bf16* dout, const float* lse, const float* delta, bf16* dqkv,
                  int B, int T, int H, float scale, int causal, cudaStream_t s)
{
    const int D = H * HD;
    CUtensorMap mq128, mq64, mdo128, mdo64;
    LTL_TRY(ltl_tensor_map_bf16(qkv, B * T, 3 * D, 3LL * D, 128, &mq128));
    LTL_TRY(ltl_tensor_map_bf16(qkv, B * T, 3 * D, 3LL * D, 64, &mq64));
    LTL_TRY(ltl_tensor_map_bf16(dout, B * T, D, D, 128, &mdo128));
    LTL_TRY(ltl_tensor_map_bf16(dout, B * T, D, D, 64, &mdo64));
    static bool attr = false;
    const size_t smem_q = sizeof(DqSmem<HD>) + 1024, smem_kv = sizeof(DkvSmem<HD>) + 1024;
    if (!attr) {
        LTL_CUDA("attn_bwd_tc attr", cudaFuncSetAttribute(attn_bwd_dq_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_q));
        LTL_CUDA("attn_bwd_tc attr", cudaFuncSetAttribute(attn_bwd_dkv_tc_kernel<HD>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_kv));
        attr = true;
    }
    dim3 gq((T + QT - 1) / QT, H, B), gk((T + KT - 1) / KT, H, B);
    attn_bwd_dq_tc_kernel<HD><<<gq, BWD_THREADS, smem_q, s>>>(mq128, mq64, mdo128, lse, delta, dqkv, T, H, scale, causal, ltl_tc_err_flag());
    LTL_TRY(ltl_check_launch("attn_bwd_dq_tc"));
    attn_bwd_dkv_tc_kernel<HD><<<gk, BWD_THREADS, smem_kv, s>>>(mq128, mq64, mdo64, lse, delta, dqkv, T, H, scale, causal, ltl_tc_err_flag());
    return ltl_check_launch("attn_bwd_dkv_tc");
}

}  // namespace

bool ltl_attn_tc_supported(int T, int H, int hd, int dtype)
{
    return dtype == LTL_BF16 && (hd == 64 || hd == 128) && T % 8 == 0 && T >= 64;
}

int ltl_attn_fwd_tc(const void* qkv, void* out, float* lse, int B, int T, int H, int hd, float scale, int causal, cudaStream_t s)
{
    if (!qkv || !out) return ltl_fail(LTL_ERR_NULL, "attn_fwd_tc: null pointer");
    if (!ltl_attn_tc_supported(T, H, hd, LTL_BF16)) return ltl_fail(LTL_ERR_UNSUPPORTED, "attn_fwd_tc: head_dim %d, T %d", hd, T);
    if (B <= 0 || H <= 0 || B > 65535 || H > 65535) return ltl_fail(LTL_ERR_SHAPE, "attn_fwd_tc: grid too large");
    if (hd == 64) return launch_fwd_tc<64>((const bf16*)qkv, (bf16*)out, lse, B, T, H, scale, causal, s);
    return launch_fwd_tc<128>((const bf16*)qkv, (bf16*)out, lse, B, T, H, scale, causal, s);
}

// delta [B*H*T] (fp32 scratch) is written here.
int ltl_attn_bwd_tc(const void* qkv, const void* out, const void* dout, const float* lse, float* delta, void* dqkv,
                    int B, int T, int H, int hd, float scale, int causal, cudaStream_t s)
{
    if (!qkv || !out || !dout || !lse || !delta || !dqkv) return ltl_fail(LTL_ERR_NULL, "attn_bwd_tc: null pointer");
    if (!ltl_attn_tc_supported(T, H, hd, LTL_BF16)) return ltl_fail(LTL_ERR_UNSUPPORTED, "attn_bwd_tc: head_dim %d, T %d", hd, T);
    if (B <= 0 || H <= 0 || B > 65535 || H > 65535) return ltl_fail(LTL_ERR_SHAPE, "attn_bwd_tc: grid too large");
    LTL_TRY(ltl_attn_delta(out, dout, delta, B, T, H, hd, LTL_BF16, s));
    if (hd == 64) return launch_bwd_tc<64>((const bf16*)qkv, (const bf16*)dout, lse, delta, (bf16*)dqkv, B, T, H, scale, causal, s);
    return launch_bwd_tc<128>((const bf16*)qkv, (const bf16*)dout, lse, delta, (bf16*)dqkv, B, T, H, scale, causal, s);
}
