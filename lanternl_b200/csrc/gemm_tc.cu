// Tensor-core GEMM for sm_100a: C[M,N] = A[M,K] * B[N,K]^T (+ R), bf16 operands, fp32
// accumulation in tensor memory.
//
//   - operands are staged by TMA (cp.async.bulk.tensor.2d, 128-byte swizzle, zero fill outside
//     the matrix) into a shared-memory ring (6 to 10 stages) guarded by full/empty mbarriers;
//   - one elected thread issues tcgen05.mma (UMMA 128 x BN x 16, kind::f16, cta_group::1); the
//     accumulator (128 lanes x BN fp32 columns) lives in TMEM allocated by the same warp;
//   - four epilogue warps read their lane quadrant with tcgen05.ld, add the residual, convert
//     and store rows of 32 consecutive columns.
// Warp roles: warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2..5 = epilogue.
// Every mbarrier wait is bounded; a wait that runs out raises a flag the host turns into an
// error, and the kernel still releases its tensor memory and returns.
//
// Both operands are K-major: A is the activation matrix [M, K], B is a weight stored [N, K]
// (the layout of the bf16 weight mirror, and of tok_emb when it is the tied lm_head).
// No cluster launch and no TMA multicast: the kernel is the same on 1 and on N GPUs.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>
#include <map>
#include <tuple>

#include "ops.h"
#include "tc_common.cuh"

namespace {

constexpr int BM = 128, BK = 64, UMMA_K = 16;
// Ring depth per tile width: about 190 KB of operands in flight per CTA.  The GEMMs of a decode
// step are short (K = 512 ... 1408, 8 ... 22 k-blocks); with a deep ring most of a CTA's operand
// bytes are requested at once and the kernel is bound by one memory round trip, not by one per
// four k-blocks.
template <int BN> struct Ring { static constexpr int STAGES = BN == 32 ? 10 : (BN == 64 ? 8 : (BN == 128 ? 6 : 4)); };
enum { EPI_NONE = 0, EPI_SWIGLU = 1, EPI_ATOMIC = 2, EPI_RESID = 3 };
using namespace tc;

// Shared memory of one CTA, carved from the dynamic allocation (1024-byte aligned for the 128-byte
// swizzle): `stages` A tiles, `stages` B tiles, then the barriers.  The ring depth is a launch
// parameter: a grid of a few latency-bound CTAs (a decode step) takes the deep ring and an SM each;
// a grid of many tiles (prefill, training) takes a ring shallow enough for two CTAs per SM, so that
// one CTA's epilogue overlaps the other's loads and MMAs.
constexpr int MAX_STAGES = 10;
struct Bars {
    uint64_t full[MAX_STAGES];
    uint64_t empty[MAX_STAGES];
    uint64_t acc_ready;
    uint32_t tmem_base;
    int ticket;                    // EPI_RESID: arrival order of this CTA at its output tile
};
template <int BN> constexpr size_t stage_bytes() { return (size_t)(BM + BN) * BK * 2; }
template <int BN> size_t smem_bytes(int stages) { return stages * stage_bytes<BN>() + sizeof(Bars) + 1024; }

// EPI_SWIGLU: the B rows are interleaved (gate_j, up_j, gate_j+1, ...); the epilogue rounds both to
// the output type (what a stored gate|up tensor would hold), applies silu(gate) * up and writes
// N / 2 columns.  R is ignored.
// EPI_ATOMIC: C (fp32) += the product, with red.global.add; every split-K slice adds into the same C.
// This is the weight-gradient form (dW += X^T dY with a long reduction over the tokens).
// EPI_RESID (BN = 32, fp32 slices, N a multiple of 32): split-K whose last-arriving CTA per output tile finishes the
// tile - see LtlGemmFuse.  No CTA waits for another: every CTA publishes its slice (fence, then a ticket from an
// atomic counter) and only the one that draws the last ticket reads the others' slices.
// MAJ = 1: both operands MN-major - A is X [K, M] and B is Y [K, N] in memory (the contraction runs down the
// rows), i.e. C = X^T Y, the weight-gradient product of two token-major activations without a transpose.
// FZ selects the instantiations that take the fusion arguments; the others keep an empty parameter, so the kernels of
// the plain paths are exactly what they were without the fused forms (their presence alone cost 1 - 2 % of a decode pass).
struct NoFuse {};
template <bool FZ> struct FuseArg { typedef NoFuse type; };
template <> struct FuseArg<true> { typedef LtlGemmFuse type; };

template <int BN, typename TC, int EPI, int MAJ = 0, bool FZ = false>
__global__ void __launch_bounds__(192, 2)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
               TC* C, const TC* R, int M, int N, int K, int STAGES, int b_early, const typename FuseArg<FZ>::type fz, int* __restrict__ err)
{
    // b_early: B holds weights that no kernel of the surrounding programmatic-launch chain writes (the decode
    // step), so the first ring of B tiles is requested before griddepcontrol.wait and lands under the tail of
    // the predecessor; only the A tiles wait for it.
    // gridDim.z > 1: split-K.  Slice z covers a contiguous range of k-blocks and writes its partial
    // sums to C + z * M * N (the consumer adds the slices in a fixed order).
    extern __shared__ uint8_t smem_raw[];
    uint8_t* const tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* const tiles_b = tiles + (size_t)STAGES * (BM * BK * 2);
    Bars& sm = *reinterpret_cast<Bars*>(tiles_b + (size_t)STAGES * (BN * BK * 2));
    auto a_tile = [&](int st) { return tiles + (size_t)st * (BM * BK * 2); };
    auto b_tile = [&](int st) { return tiles_b + (size_t)st * (BN * BK * 2); };
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    constexpr uint32_t STAGE_BYTES = BM * BK * 2 + BN * BK * 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int kb_all = (K + BK - 1) / BK;
    const int kb_per = (kb_all + gridDim.z - 1) / gridDim.z;
    const int kb0 = blockIdx.z * kb_per;
    const int kblocks = max(0, min(kb_all, kb0 + kb_per) - kb0);
    TC* const Cbase = C;
    if (EPI != EPI_ATOMIC) C += (size_t)blockIdx.z * M * N;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        mbar_init(&sm.acc_ready, 1);
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
    int npre = 0;                                         // stages whose B tile is already on its way
    if (MAJ == 0 && b_early && warp == 0 && lane == 0) {
        npre = min(STAGES, kblocks);
        for (int s = 0; s < npre; ++s) {
            mbar_expect_tx(&sm.full[s], STAGE_BYTES);
            tma_load_2d(b_tile(s), &map_b, (kb0 + s) * BK, n0, &sm.full[s]);
        }
    }
    pdl_trigger();          // the next kernel may set itself up
    pdl_wait();             // barriers and TMEM are ready; now the predecessor's output may be read

    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----
        int s = 0;
        uint32_t round = 0;                               // kb / STAGES, kept without a division
        for (int kb = 0; kb < kblocks && ok; ++kb, ++s) {
            if (s == STAGES) { s = 0; ++round; }
            if (MAJ == 0 && kb < npre) {                  // first ring: expect_tx and the B tile were issued above
                tma_load_2d(a_tile(s), &map_a, (kb0 + kb) * BK, m0, &sm.full[s]);
                continue;
            }
            if (round > 0) ok = mbar_wait(&sm.empty[s], (round - 1) & 1);
            if (!ok) break;
            mbar_expect_tx(&sm.full[s], STAGE_BYTES);
            if (MAJ == 0) {
                tma_load_2d(a_tile(s), &map_a, (kb0 + kb) * BK, m0, &sm.full[s]);
                tma_load_2d(b_tile(s), &map_b, (kb0 + kb) * BK, n0, &sm.full[s]);
            } else {
                // column blocks of 64 features: BK token rows of 128 bytes each
#pragma unroll
                for (int cb = 0; cb < BM / 64; ++cb) tma_load_2d(a_tile(s) + cb * (BK * 128), &map_a, m0 + cb * 64, (kb0 + kb) * BK, &sm.full[s]);
#pragma unroll
                for (int cb = 0; cb < BN / 64; ++cb) tma_load_2d(b_tile(s) + cb * (BK * 128), &map_b, n0 + cb * 64, (kb0 + kb) * BK, &sm.full[s]);
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        constexpr uint32_t idesc = MAJ ? umma_idesc_bf16_mn(BM, BN) : umma_idesc_bf16(BM, BN);
        int s = 0;
        uint32_t round = 0;
        for (int kb = 0; kb < kblocks && ok; ++kb, ++s) {
            if (s == STAGES) { s = 0; ++round; }
            ok = mbar_wait(&sm.full[s], round & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            if (MAJ == 0) {
                const uint64_t da = umma_desc_sw128(smem_u32(a_tile(s)));
                const uint64_t db = umma_desc_sw128(smem_u32(b_tile(s)));
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k)        // 32 bytes further along K per UMMA
                    umma_bf16(tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) ? 1u : 0u);
            } else {
                // 16 token rows (2048 bytes) further per UMMA; column blocks BK * 128 bytes apart, 8-row groups 1024
                constexpr uint32_t lbo = BK * 128, sbo = 1024;
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    const uint64_t da = umma_desc_sw128_mn(smem_u32(a_tile(s)) + k * 2048, lbo, sbo);
                    const uint64_t db = umma_desc_sw128_mn(smem_u32(b_tile(s)) + k * 2048, lbo, sbo);
                    umma_bf16(tmem, da, db, idesc, (kb | k) ? 1u : 0u);
                }
            }
            umma_commit(&sm.empty[s]);                    // frees the stage when these MMAs retire
        }
        umma_commit(&sm.acc_ready);
    } else if (warp >= 2) {
        // ---- epilogue: TMEM -> registers -> global ----
        ok = mbar_wait(&sm.acc_ready, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int quad = warp & 3;                        // TMEM lane quadrant this warp may read
        const int row = m0 + quad * 32 + lane;
        float rscale = 1.0f;                              // deferred RMSNorm factor of this row
        constexpr bool scaled = FZ && (EPI == EPI_NONE || EPI == EPI_SWIGLU);
        if constexpr (scaled) {
            if (row < M) {
                float ss = 0.0f;
                for (int t = 0; t < fz.ssq_tiles; ++t) ss += fz.ssq_in[(size_t)row * fz.ssq_tiles + t];
                rscale = 1.0f / sqrtf(ss * fz.inv_dim + fz.eps);
            }
        }
        if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (kblocks == 0) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0u;
                }
                if (scaled) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) * rscale);
                }
                if (EPI == EPI_SWIGLU) {
                    if (row < M) {
                        const int No = N >> 1;
                        const int ncols = min(32, N - (n0 + c0)) >> 1;
                        const size_t base = (size_t)row * No + ((n0 + c0) >> 1);
                        float o[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            float g = __uint_as_float(v[2 * j]), u = __uint_as_float(v[2 * j + 1]);
                            if (sizeof(TC) == 2) { g = __bfloat162float(__float2bfloat16_rn(g)); u = __bfloat162float(__float2bfloat16_rn(u)); }
                            o[j] = silu_f(g) * u;
                        }
                        if (ncols == 16 && (No % 8) == 0 && sizeof(TC) == 2) {
                            float lo[8], hi[8];
#pragma unroll
                            for (int j = 0; j < 8; ++j) { lo[j] = o[j]; hi[j] = o[8 + j]; }
                            st16<bf16>(reinterpret_cast<bf16*>(C) + base, lo);
                            st16<bf16>(reinterpret_cast<bf16*>(C) + base + 8, hi);
                        } else {
                            for (int j = 0; j < ncols; ++j) Cvt<TC>::st(C, base + j, o[j]);
                        }
                    }
                } else if (EPI == EPI_ATOMIC) {
                    if (row < M && kblocks > 0) {
                        float* dst = reinterpret_cast<float*>(C) + (size_t)row * N + n0 + c0;
                        const int ncols = min(32, N - (n0 + c0));
                        if (ncols == 32 && (N & 3) == 0) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + j),
                                             "f"(__uint_as_float(v[j])), "f"(__uint_as_float(v[j + 1])),
                                             "f"(__uint_as_float(v[j + 2])), "f"(__uint_as_float(v[j + 3])) : "memory");
                        } else {
                            for (int j = 0; j < ncols; ++j) atomicAdd(dst + j, __uint_as_float(v[j]));
                        }
                    }
                } else if (row < M) {
                    const size_t base = (size_t)row * N + n0 + c0;
                    const int ncols = min(32, N - (n0 + c0));
                    if (ncols == 32 && (N % Vec16<TC>::N) == 0) {
                        constexpr int NV = Vec16<TC>::N;
#pragma unroll
                        for (int j = 0; j < 32; j += NV) {
                            float o[NV];
#pragma unroll
                            for (int i = 0; i < NV; ++i) o[i] = __uint_as_float(v[j + i]);
                            if (R) {
                                float rr[NV];
                                ld16<TC>(R + base + j, rr);
#pragma unroll
                                for (int i = 0; i < NV; ++i) o[i] += rr[i];
                            }
                            st16<TC>(C + base + j, o);
                        }
                    } else {
                        for (int j = 0; j < ncols; ++j) {
                            float o = __uint_as_float(v[j]);
                            if (R) o += Cvt<TC>::ld(R, base + j);
                            Cvt<TC>::st(C, base + j, o);
                        }
                    }
                }
            }
        }
        if constexpr (EPI == EPI_RESID && FZ) {
            // Every epilogue thread gets here whatever its wait returned, so the named barrier always completes.
            __threadfence();                                              // this CTA's slice is visible ...
            asm volatile("bar.sync 1, 128;" ::: "memory");
            const int tile = blockIdx.y * gridDim.x + blockIdx.x;
            if (threadIdx.x == 64) sm.ticket = atomicAdd(fz.counters + tile, 1);   // ... before its ticket is drawn
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (sm.ticket == (int)gridDim.z - 1) {
                __threadfence();
                // 8 threads per row (4 columns each), 16 rows per pass; two passes and all their slices in flight at once
                const int te = threadIdx.x - 64, c4 = te & 7, col = n0 + c4 * 4;
                const int ks = (int)gridDim.z;
                const float* part = reinterpret_cast<const float*>(Cbase);
                const float4 g = *reinterpret_cast<const float4*>(fz.gain + col);
#pragma unroll 1
                for (int i0 = 0; i0 < 8; i0 += 2) {
                    float4 q[2][8], xv[2];
                    int rr[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        rr[u] = m0 + (te >> 3) + 16 * (i0 + u);
                        if (rr[u] < M) {
                            xv[u] = *reinterpret_cast<const float4*>(fz.x + (size_t)rr[u] * N + col);
#pragma unroll
                            for (int p = 0; p < 8; ++p)
                                if (p < ks) q[u][p] = __ldcg(reinterpret_cast<const float4*>(part + (size_t)p * M * N + (size_t)rr[u] * N + col));
                        }
                    }
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        float ss = 0.0f;
                        if (rr[u] < M) {
                            float4 a4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                            for (int p = 0; p < 8; ++p)                  // slice order: the sum does not depend on arrival order
                                if (p < ks) { a4.x += q[u][p].x; a4.y += q[u][p].y; a4.z += q[u][p].z; a4.w += q[u][p].w; }
                            for (int p = 8; p < ks; ++p) {               // more than eight slices: the rest one by one
                                const float4 e = __ldcg(reinterpret_cast<const float4*>(part + (size_t)p * M * N + (size_t)rr[u] * N + col));
                                a4.x += e.x; a4.y += e.y; a4.z += e.z; a4.w += e.w;
                            }
                            float4 v4 = xv[u];
                            v4.x += a4.x; v4.y += a4.y; v4.z += a4.z; v4.w += a4.w;
                            *reinterpret_cast<float4*>(fz.x + (size_t)rr[u] * N + col) = v4;
                            ss = fmaf(v4.x, v4.x, fmaf(v4.y, v4.y, fmaf(v4.z, v4.z, v4.w * v4.w)));
                            uint2 pk;
                            pk.x = pack_bf16x2(v4.x * g.x, v4.y * g.y);
                            pk.y = pack_bf16x2(v4.z * g.z, v4.w * g.w);
                            *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(fz.h) + (size_t)rr[u] * N + col) = pk;
                        }
                        ss += __shfl_xor_sync(0xFFFFFFFFu, ss, 1);
                        ss += __shfl_xor_sync(0xFFFFFFFFu, ss, 2);
                        ss += __shfl_xor_sync(0xFFFFFFFFu, ss, 4);
                        if (rr[u] < M && c4 == 0) fz.ssq_out[(size_t)rr[u] * gridDim.x + blockIdx.x] = ss;
                    }
                }
                if (threadIdx.x == 64) fz.counters[tile] = 0;             // ready for the next launch
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

// ------------------------------------------------------------------------------------------------------------
// Persistent form for many-tile problems (training, prefill): one CTA per SM walks 128 x 256 output tiles.
//   - the TMA ring (4 stages of 48 KB) never drains between tiles;
//   - two accumulators of 256 columns in tensor memory: the MMA warp fills one while the four epilogue warps
//     read the other, so the epilogue of tile i runs under the main loop of tile i + 1;
//   - consecutive CTAs take consecutive M tiles of the same N tile, so the wide B (weight) tile is shared in L2.
// MAJ = 0: C = A B^T (+ R), K-major operands, TC = bf16 or fp32.  MAJ = 1: C (fp32) += X^T Y, MN-major operands,
// work items = (K slice, tile), atomic accumulation.
// ------------------------------------------------------------------------------------------------------------
constexpr int PBN = 256, PSTAGES = 4;
struct PBars {
    uint64_t full[PSTAGES], empty[PSTAGES], acc_full[2], acc_empty[2];
    uint32_t tmem_base;
};
constexpr size_t PSMEM = (size_t)PSTAGES * (BM + PBN) * BK * 2 + sizeof(PBars) + 1024;

template <typename TC, int MAJ>
__global__ void __launch_bounds__(192, 1)
gemm_tc_persist_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                       TC* C, const TC* R, int M, int N, int K, int ksplit, int* __restrict__ err)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* const tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* const tiles_b = tiles + (size_t)PSTAGES * (BM * BK * 2);
    PBars& sm = *reinterpret_cast<PBars*>(tiles_b + (size_t)PSTAGES * (PBN * BK * 2));
    auto a_tile = [&](int st) { return tiles + (size_t)st * (BM * BK * 2); };
    auto b_tile = [&](int st) { return tiles_b + (size_t)st * (PBN * BK * 2); };
    constexpr uint32_t STAGE_BYTES = (BM + PBN) * BK * 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + PBN - 1) / PBN, ntiles = tiles_m * tiles_n;
    const int kb_all = (K + BK - 1) / BK;
    const int kb_per = (kb_all + ksplit - 1) / ksplit;
    const int nitems = ntiles * ksplit;                  // item = slice * ntiles + tile; tile = nt * tiles_m + mt

    if (threadIdx.x == 0) {
        for (int s = 0; s < PSTAGES; ++s) { mbar_init(&sm.full[s], 1); mbar_init(&sm.empty[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&sm.acc_full[s], 1); mbar_init(&sm.acc_empty[s], 128); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sm.tmem_base;
    bool ok = true;

    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----
        int s = 0;
        uint32_t round = 0;
        for (int it = blockIdx.x; it < nitems && ok; it += gridDim.x) {
            const int tile = it % ntiles, slice = it / ntiles;
            const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * PBN;
            const int kb0 = slice * kb_per, kb1 = min(kb_all, kb0 + kb_per);
            for (int kb = kb0; kb < kb1; ++kb) {
                if (round > 0) ok = mbar_wait(&sm.empty[s], (round - 1) & 1);
                if (!ok) break;
                mbar_expect_tx(&sm.full[s], STAGE_BYTES);
                if (MAJ == 0) {
                    tma_load_2d(a_tile(s), &map_a, kb * BK, m0, &sm.full[s]);
                    tma_load_2d(b_tile(s), &map_b, kb * BK, n0, &sm.full[s]);
                } else {
#pragma unroll
                    for (int cb = 0; cb < BM / 64; ++cb) tma_load_2d(a_tile(s) + cb * (BK * 128), &map_a, m0 + cb * 64, kb * BK, &sm.full[s]);
#pragma unroll
                    for (int cb = 0; cb < PBN / 64; ++cb) tma_load_2d(b_tile(s) + cb * (BK * 128), &map_b, n0 + cb * 64, kb * BK, &sm.full[s]);
                }
                if (++s == PSTAGES) { s = 0; ++round; }
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        constexpr uint32_t idesc = MAJ ? umma_idesc_bf16_mn(BM, PBN) : umma_idesc_bf16(BM, PBN);
        int s = 0;
        uint32_t round = 0, i = 0;
        for (int it = blockIdx.x; it < nitems && ok; it += gridDim.x, ++i) {
            const int slice = it / ntiles;
            const int kb0 = slice * kb_per, kb1 = min(kb_all, kb0 + kb_per);
            const uint32_t buf = i & 1, acc = tmem + buf * PBN;
            if (i >= 2) ok = mbar_wait(&sm.acc_empty[buf], ((i >> 1) - 1) & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int kb = kb0; kb < kb1; ++kb) {
                ok = mbar_wait(&sm.full[s], round & 1);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                if (MAJ == 0) {
                    const uint64_t da = umma_desc_sw128(smem_u32(a_tile(s))), db = umma_desc_sw128(smem_u32(b_tile(s)));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16(acc, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb > kb0 || k) ? 1u : 0u);
                } else {
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k)
                        umma_bf16(acc, umma_desc_sw128_mn(smem_u32(a_tile(s)) + k * 2048, BK * 128, 1024),
                                  umma_desc_sw128_mn(smem_u32(b_tile(s)) + k * 2048, BK * 128, 1024), idesc, (kb > kb0 || k) ? 1u : 0u);
                }
                umma_commit(&sm.empty[s]);
                if (++s == PSTAGES) { s = 0; ++round; }
            }
            if (ok) umma_commit(&sm.acc_full[buf]);
        }
    } else if (warp >= 2) {
        // ---- epilogue ----
        const int quad = warp & 3;
        uint32_t i = 0;
        for (int it = blockIdx.x; it < nitems; it += gridDim.x, ++i) {
            const int tile = it % ntiles, slice = it / ntiles;
            const int m0 = (tile % tiles_m) * BM, n0 = (tile / tiles_m) * PBN;
            const bool empty_slice = slice * kb_per >= kb_all;
            const uint32_t buf = i & 1;
            if (!mbar_wait(&sm.acc_full[buf], (i >> 1) & 1)) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = m0 + quad * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < PBN; c0 += 32) {
                if (n0 + c0 >= N) break;
                uint32_t v[32];
                tmem_ld32(tmem + buf * PBN + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row >= M || empty_slice) continue;
                const size_t base = (size_t)row * N + n0 + c0;
                const int ncols = min(32, N - (n0 + c0));
                if (MAJ == 1) {
                    float* dst = reinterpret_cast<float*>(C) + base;
                    if (ncols == 32 && (N & 3) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + j),
                                         "f"(__uint_as_float(v[j])), "f"(__uint_as_float(v[j + 1])),
                                         "f"(__uint_as_float(v[j + 2])), "f"(__uint_as_float(v[j + 3])) : "memory");
                    } else {
                        for (int j = 0; j < ncols; ++j) atomicAdd(dst + j, __uint_as_float(v[j]));
                    }
                } else if (ncols == 32 && (N % Vec16<TC>::N) == 0) {
                    constexpr int NV = Vec16<TC>::N;
#pragma unroll
                    for (int j = 0; j < 32; j += NV) {
                        float o[NV];
#pragma unroll
                        for (int e = 0; e < NV; ++e) o[e] = __uint_as_float(v[j + e]);
                        if (R) {
                            float rr[NV];
                            ld16<TC>(R + base + j, rr);
#pragma unroll
                            for (int e = 0; e < NV; ++e) o[e] += rr[e];
                        }
                        st16<TC>(C + base + j, o);
                    }
                } else {
                    for (int j = 0; j < ncols; ++j) {
                        float o = __uint_as_float(v[j]);
                        if (R) o += Cvt<TC>::ld(R, base + j);
                        Cvt<TC>::st(C, base + j, o);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&sm.acc_empty[buf])) : "memory");
        }
    }
    if (!ok && err) atomicExch(err, 1);
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

typedef CUresult (*encode_fn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                              const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
encode_fn g_encode = nullptr;

int get_encode()
{
    if (g_encode) return LTL_OK;
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    const cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || !fn || q != cudaDriverEntryPointSuccess) {
        cudaGetLastError();
        return ltl_fail(LTL_ERR_UNSUPPORTED, "gemm_tc: cuTensorMapEncodeTiled is not available from this driver");
    }
    g_encode = (encode_fn)fn;
    return LTL_OK;
}

// 2-D bf16 matrix [rows, cols] whose rows are `pitch` elements apart, with a box of box_rows x 64 columns,
// 128-byte swizzle, zero fill outside.
std::map<std::tuple<const void*, int, int, long long, int>, CUtensorMap> g_maps;

int tensor_map(const void* base, int rows, int cols, long long pitch, int box_rows, CUtensorMap* out)
{
    const auto key = std::make_tuple(base, rows, cols, pitch, box_rows);
    const auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return LTL_OK; }
    LTL_TRY(get_encode());
    const cuuint64_t dims[2] = { (cuuint64_t)cols, (cuuint64_t)rows };
    const cuuint64_t strides[1] = { (cuuint64_t)pitch * 2 };
    const cuuint32_t box[2] = { (cuuint32_t)BK, (cuuint32_t)box_rows };
    const cuuint32_t estr[2] = { 1, 1 };
    const CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ltl_fail(LTL_ERR_CUDA, "gemm_tc: cuTensorMapEncodeTiled failed (%d) for %dx%d", (int)r, rows, cols);
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps[key] = *out;
    return LTL_OK;
}

int* g_err_flag = nullptr;

// LUATL_GEMM_PERSIST: 0 = never, 1 = K-major only, 2 (default) = K-major and the weight-gradient (MN-major) form
int persist_mode()
{
    static const int mode = [] { const char* e = getenv("LUATL_GEMM_PERSIST"); return e ? atoi(e) : 2; }();
    return mode;
}
bool persist_enabled() { return persist_mode() >= 1; }
// LUATL_GEMM_B_EARLY=0: weights of a decode-step GEMM wait for the predecessor like the activations (A/B comparison).
bool b_early_enabled()
{
    static const bool on = [] { const char* e = getenv("LUATL_GEMM_B_EARLY"); return !(e && e[0] == '0'); }();
    return on;
}

template <typename TC, int MAJ>
int launch_persist(const CUtensorMap& ma, const CUtensorMap& mb, void* C, const void* R, int M, int N, int K, int ksplit, cudaStream_t s)
{
    static bool attr_set = false;
    if (!attr_set) {
        LTL_CUDA("gemm_tc attr", cudaFuncSetAttribute(gemm_tc_persist_kernel<TC, MAJ>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PSMEM));
        attr_set = true;
    }
    if (ksplit < 1) ksplit = 1;
    const long long items = (long long)((M + BM - 1) / BM) * ((N + PBN - 1) / PBN) * ksplit;
    const int grid = (int)std::min<long long>(items, ltl_sm_count());
    gemm_tc_persist_kernel<TC, MAJ><<<grid, 192, PSMEM, s>>>(ma, mb, (TC*)C, (const TC*)R, M, N, K, ksplit, g_err_flag);
    return ltl_check_launch("gemm_tc_persist");
}

// Host-side switch for the launches that follow: shallow rings whose shared memory is allocated at its real size (see launch).
bool g_lean = false;

template <int BN, typename TC, int EPI>
int launch(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int ksplit, cudaStream_t s,
           const LtlGemmFuse& fz = LtlGemmFuse{})
{
    CUtensorMap ma, mb;
    LTL_TRY(tensor_map(A, M, K, K, BM, &ma));
    LTL_TRY(tensor_map(B, N, K, K, BN, &mb));
    if constexpr (BN == 256 && EPI == EPI_NONE) {
        // long reductions run a little faster as two co-resident CTAs (measured: K = 5632 .. 11264, fp32 output)
        if (persist_enabled() && ksplit <= 1 && K <= 4096 && !fz.ssq_in) return launch_persist<TC, 0>(ma, mb, C, R, M, N, K, 1, s);
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, ksplit < 1 ? 1 : ksplit);
    const int kb_all = (K + BK - 1) / BK;
    const int kb_per = (kb_all + (int)grid.z - 1) / (int)grid.z;
    int stages = Ring<BN>::STAGES;
    // Many tiles per SM: two CTAs per SM (about 100 KB of ring each).  Otherwise the allocation stays that of
    // the full ring whatever the depth used, which keeps one CTA per SM (each then has an SM's load path alone).
    // The narrowest tile with more CTAs than SMs shares the SMs two by two as well (a second wave would cost a whole launch).
    const long long nctas = (long long)grid.x * grid.y * grid.z;
    const bool many = nctas >= 2LL * ltl_sm_count() || (BN == 32 && nctas > ltl_sm_count());
    if (many) stages = BN == 256 ? 2 : (BN == 128 ? 3 : (BN == 64 ? 4 : 5));
    if (g_lean) {
        // a ring of at most ~80 KB, allocated as such: the CTA then fits beside the kernels of another stream
        const int cap = BN == 32 ? 4 : (BN == 64 ? 3 : (BN == 128 ? 2 : 1));
        if (stages > cap) stages = cap;
    }
    if (stages > kb_per) stages = kb_per;
    if (stages < 1) stages = 1;
    const size_t smem = smem_bytes<BN>((many || g_lean) ? stages : Ring<BN>::STAGES);
    static bool attr_set = false;
    if (!attr_set) {
        LTL_CUDA("gemm_tc attr", cudaFuncSetAttribute(gemm_tc_kernel<BN, TC, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                      (int)smem_bytes<BN>(Ring<BN>::STAGES)));
        attr_set = true;
    }
    const int early = b_early_enabled() && ltl_pdl_enabled() ? 1 : 0;
    if (EPI == EPI_RESID || fz.ssq_in) {
        if constexpr (EPI == EPI_ATOMIC) {
            return ltl_fail(LTL_ERR_ARG, "gemm_tc: the accumulating epilogue takes no fusion");
        } else {
            static bool fz_attr_set = false;
            if (!fz_attr_set) {
                LTL_CUDA("gemm_tc attr", cudaFuncSetAttribute(gemm_tc_kernel<BN, TC, EPI, 0, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                              (int)smem_bytes<BN>(Ring<BN>::STAGES)));
                fz_attr_set = true;
            }
            LTL_CUDA("gemm_tc launch", ltl_launch(gemm_tc_kernel<BN, TC, EPI, 0, true>, grid, dim3(192), smem, s, ltl_pdl_enabled(),
                                                  ma, mb, (TC*)C, (const TC*)R, M, N, K, stages, early, fz, g_err_flag));
            return ltl_check_launch("gemm_tc");
        }
    }
    if constexpr (EPI == EPI_RESID) {
        return ltl_fail(LTL_ERR_ARG, "gemm_tc: the residual form needs its fusion arguments");
    } else {
        LTL_CUDA("gemm_tc launch", ltl_launch(gemm_tc_kernel<BN, TC, EPI>, grid, dim3(192), smem, s, ltl_pdl_enabled(),
                                              ma, mb, (TC*)C, (const TC*)R, M, N, K, stages, early, NoFuse{}, g_err_flag));
        return ltl_check_launch("gemm_tc");
    }
}

template <int BN>
int launch_mn(const void* X, const void* Y, float* C, int M, int N, int K, int ksplit, cudaStream_t s)
{
    static_assert(BN % 64 == 0, "MN-major tiles are loaded in column blocks of 64");
    CUtensorMap ma, mb;
    LTL_TRY(tensor_map(X, K, M, M, 64, &ma));
    LTL_TRY(tensor_map(Y, K, N, N, 64, &mb));
    if constexpr (BN == 256) {
        if (persist_mode() >= 2) return launch_persist<float, 1>(ma, mb, C, nullptr, M, N, K, ksplit, s);
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, ksplit < 1 ? 1 : ksplit);
    const int kb_all = (K + BK - 1) / BK;
    const int kb_per = (kb_all + (int)grid.z - 1) / (int)grid.z;
    int stages = BN == 256 ? 2 : (BN == 128 ? 3 : 4);
    if (stages > kb_per) stages = kb_per;
    const size_t smem = smem_bytes<BN>(stages);
    static bool attr_set = false;
    if (!attr_set) {
        LTL_CUDA("gemm_tc attr", cudaFuncSetAttribute(gemm_tc_kernel<BN, float, EPI_ATOMIC, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                      (int)smem_bytes<BN>(BN == 256 ? 2 : 4)));
        attr_set = true;
    }
    gemm_tc_kernel<BN, float, EPI_ATOMIC, 1><<<grid, 192, smem, s>>>(ma, mb, C, nullptr, M, N, K, stages, 0, NoFuse{}, g_err_flag);
    return ltl_check_launch("gemm_tc_mn");
}

}  // namespace

// C[M, N] (fp32) += X^T Y with X [K, M] and Y [K, N] bf16 row-major (both MN-major operands): the weight gradient
// dW += X^T dY straight from the token-major activations.  M and N must be multiples of 8 (16-byte row pitch).
int ltl_gemm_tc_xty(const void* X, const void* Y, float* C, int M, int N, int K, int ksplit, cudaStream_t s)
{
    if (!X || !Y || !C) return ltl_fail(LTL_ERR_NULL, "gemm_tc_xty: null operand");
    if (M <= 0 || N <= 0 || K <= 0 || M % 8 || N % 8 || (reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(Y) & 15))
        return ltl_fail(LTL_ERR_UNSUPPORTED, "gemm_tc_xty: M and N must be multiples of 8 and the operands 16-byte aligned (M=%d N=%d K=%d)", M, N, K);
    if (!ltl_tc_err_flag()) return ltl_fail(LTL_ERR_OOM, "gemm_tc_xty: error flag");
    if (N >= 256 && (long long)((M + BM - 1) / BM) * ((N + 255) / 256) * (ksplit < 1 ? 1 : ksplit) >= 4LL * ltl_sm_count())
        return launch_mn<256>(X, Y, C, M, N, K, ksplit, s);
    if (N >= 128) return launch_mn<128>(X, Y, C, M, N, K, ksplit, s);
    return launch_mn<64>(X, Y, C, M, N, K, ksplit, s);
}

int ltl_tensor_map_bf16(const void* base, int rows, int cols, long long pitch, int box_rows, void* out_map)
{
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (pitch * 2) % 16)
        return ltl_fail(LTL_ERR_ARG, "tensor map: base and row pitch must be 16-byte aligned");
    return tensor_map(base, rows, cols, pitch, box_rows, reinterpret_cast<CUtensorMap*>(out_map));
}
int* ltl_tc_err_flag()
{
    if (!g_err_flag) {
        if (cudaMalloc(&g_err_flag, sizeof(int)) != cudaSuccess) { g_err_flag = nullptr; return nullptr; }
        cudaMemset(g_err_flag, 0, sizeof(int));
    }
    return g_err_flag;
}

bool ltl_gemm_tc_supported(const void* A, const void* B, int M, int N, int K)
{
    return M > 0 && N > 0 && K > 0 && K % 8 == 0 && (reinterpret_cast<uintptr_t>(A) & 15) == 0 &&
           (reinterpret_cast<uintptr_t>(B) & 15) == 0;
}

static int pick_bn(int M, int N)
{
    // Widest single wave: the tile width with the most CTAs that still fit the SMs at one CTA each.
    const int mt = (M + BM - 1) / BM, sms = ltl_sm_count();
    int best = 128, best_ctas = -1;
    const int cand[3] = { 128, 64, 32 };
    for (int c : cand) {
        const int ctas = mt * ((N + c - 1) / c);
        if (ctas <= sms && ctas > best_ctas) { best = c; best_ctas = ctas; }
    }
    // Many tiles: the 128 x 256 tile (a third fewer L2 bytes per FLOP than 128 x 128; two CTAs per SM with a two-stage
    // ring each) for grids of at least four such tiles per SM.  LUATL_GEMM_BN=128 keeps the narrower tile.
    static const int wide = [] { const char* e = getenv("LUATL_GEMM_BN"); return e ? atoi(e) : 256; }();
    if (best_ctas < 0 && wide == 256 && N >= 256 && (long long)mt * ((N + 255) / 256) >= 4LL * sms) best = 256;
    return best;
}

void ltl_gemm_tc_set_lean(int on) { g_lean = on != 0; }

// Split-K plan for a skinny GEMM: tile width and slice count that fill the SMs in one wave.
void ltl_gemm_tc_plan_split(int M, int N, int K, int* bn, int* ksplit)
{
    const int mt = (M + BM - 1) / BM, sms = ltl_sm_count(), kb = (K + BK - 1) / BK;
    *bn = 32;
    const int tiles = mt * ((N + 31) / 32);
    int s = tiles > 0 ? sms / tiles : 1;
    if (s > 8) s = 8;
    if (s > kb) s = kb;
    if (s < 1) s = 1;
    *ksplit = s;
}

// Slice count for an accumulating GEMM (epi = 2) with tiles of width bn: enough slices of at least 4
// k-blocks to give every SM about two CTAs.
int ltl_gemm_tc_plan_accum(int M, int N, int K, int bn)
{
    const int tiles = ((M + BM - 1) / BM) * ((N + bn - 1) / bn), kb = (K + BK - 1) / BK;
    int s = (2 * ltl_sm_count() + tiles - 1) / tiles;
    if (s > kb / 4) s = kb / 4;
    if (s > 64) s = 64;
    return s < 1 ? 1 : s;
}

// C[M,N] (c_dtype f32 or bf16, row-major) = A[M,K] B[N,K]^T + R.  bn = 0 picks the tile width.
// epi = 2: C (fp32) += A B^T through atomic adds, over ksplit slices of K.
// epi = 1: SwiGLU epilogue (see the kernel), C is [M, N/2] bf16.
// ksplit > 1: split-K, C receives ksplit fp32 partial matrices [ksplit][M][N] (bn should then be the
// width the caller sized the grid for; see ltl_gemm_tc_plan_split).
int ltl_gemm_tc(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int c_dtype, int bn,
                int epi, int ksplit, cudaStream_t s, const LtlGemmFuse* fuse)
{
    const LtlGemmFuse fz = fuse ? *fuse : LtlGemmFuse{};
    if (epi == EPI_RESID) {
        if (c_dtype != LTL_F32 || R || (N % 32) || (bn != 0 && bn != 32) || !fz.x || !fz.gain || !fz.h || !fz.ssq_out || !fz.counters)
            return ltl_fail(LTL_ERR_ARG, "gemm_tc: the residual form needs fp32 slices, N %% 32 == 0, tiles of 32 columns and all of x, gain, h, ssq_out, counters");
        if (!A || !B || !C) return ltl_fail(LTL_ERR_NULL, "gemm_tc: null operand");
        if (!ltl_gemm_tc_supported(A, B, M, N, K))
            return ltl_fail(LTL_ERR_UNSUPPORTED, "gemm_tc: needs K %% 8 == 0 and 16-byte aligned operands (M=%d N=%d K=%d)", M, N, K);
        if (!ltl_tc_err_flag()) return ltl_fail(LTL_ERR_OOM, "gemm_tc: error flag");
        return launch<32, float, EPI_RESID>(A, B, C, nullptr, M, N, K, ksplit < 1 ? 1 : ksplit, s, fz);
    }
    if (fz.ssq_in && (epi == EPI_ATOMIC || ksplit > 1 || R))
        return ltl_fail(LTL_ERR_ARG, "gemm_tc: the row-scale epilogue takes no residual, split-K or accumulation");
    if (epi == EPI_ATOMIC && (c_dtype != LTL_F32 || R))
        return ltl_fail(LTL_ERR_ARG, "gemm_tc: the accumulating epilogue adds into an fp32 C and takes no residual");
    if (epi != EPI_ATOMIC && ksplit > 1 && (c_dtype != LTL_F32 || R || epi))
        return ltl_fail(LTL_ERR_ARG, "gemm_tc: split-K writes fp32 partial sums and takes no residual or epilogue");
    if (!A || !B || !C) return ltl_fail(LTL_ERR_NULL, "gemm_tc: null operand");
    if (!ltl_gemm_tc_supported(A, B, M, N, K))
        return ltl_fail(LTL_ERR_UNSUPPORTED, "gemm_tc: needs K %% 8 == 0 and 16-byte aligned operands (M=%d N=%d K=%d)", M, N, K);
    if (epi == EPI_SWIGLU && (c_dtype != LTL_BF16 || (N & 1)))
        return ltl_fail(LTL_ERR_ARG, "gemm_tc: the SwiGLU epilogue writes bf16 and needs an even N");
    if (!g_err_flag) {
        LTL_CUDA("gemm_tc flag", cudaMalloc(&g_err_flag, sizeof(int)));
        LTL_CUDA("gemm_tc flag", cudaMemset(g_err_flag, 0, sizeof(int)));
    }
    if (bn == 0) {
        bn = pick_bn(M, N);
        // SwiGLU epilogue over two row tiles (decode step of 129 .. 256 sequences): 32-column tiles, two CTAs per SM, beat
        // 64-column tiles at one per SM - measured in a captured chain at 256 rows x 2816 x 512: 5.6 us against 6.6 us.
        const int mt = (M + BM - 1) / BM, c32 = mt * ((N + 31) / 32), sms = ltl_sm_count();
        if (epi == EPI_SWIGLU && bn == 64 && c32 > sms && c32 <= 2 * sms) bn = 32;
    }
#define TC_CASE(BNV)                                                                                     \
    if (bn == BNV) {                                                                                     \
        if (epi == EPI_SWIGLU) return launch<BNV, bf16, EPI_SWIGLU>(A, B, C, nullptr, M, N, K, 1, s, fz);   \
        if (epi == EPI_ATOMIC) return launch<BNV, float, EPI_ATOMIC>(A, B, C, nullptr, M, N, K, ksplit, s);    \
        if (c_dtype == LTL_F32) return launch<BNV, float, EPI_NONE>(A, B, C, R, M, N, K, ksplit, s, fz);         \
        if (c_dtype == LTL_BF16) return launch<BNV, bf16, EPI_NONE>(A, B, C, R, M, N, K, 1, s, fz);         \
        return ltl_fail(LTL_ERR_DTYPE, "gemm_tc: output dtype %d", c_dtype);                             \
    }
    TC_CASE(32) TC_CASE(64) TC_CASE(128) TC_CASE(256)
#undef TC_CASE
    return ltl_fail(LTL_ERR_ARG, "gemm_tc: tile width %d not in {32, 64, 128, 256}", bn);
}

// 1 when a bounded wait inside the kernel ran out since the last call (and clears the flag).
int ltl_gemm_tc_check(cudaStream_t s)
{
    if (!g_err_flag) return LTL_OK;
    int v = 0;
    LTL_CUDA("gemm_tc flag read", cudaMemcpyAsync(&v, g_err_flag, sizeof(int), cudaMemcpyDeviceToHost, s));
    LTL_CUDA("gemm_tc flag sync", cudaStreamSynchronize(s));
    if (v) {
        cudaMemsetAsync(g_err_flag, 0, sizeof(int), s);
        return ltl_fail(LTL_ERR_CUDA, "gemm_tc: a pipeline wait ran out inside the kernel (TMA or MMA never arrived)");
    }
    return LTL_OK;
}
