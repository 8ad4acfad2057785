// Few-row GEMM for the decode step of a small shard: C[M <= 64, N] = A[M,K] B[N,K]^T, bf16 in, fp32
// accumulate.  With a few dozen sequences a decode GEMM moves a few hundred KB of weights and is bound by
// the latency of one dependent launch, not by bytes or flops: a 128-row tcgen05 tile would spend
// its time on barrier, TMA and TMEM round trips for a tile that is at most a quarter full.  This kernel
// keeps the whole chain to one memory round trip:
//   * every thread reads its slice of the WEIGHTS straight into mma.sync B fragments with 128-bit
//     loads, issued before griddepcontrol.wait - weights do not change inside a decode step, so the
//     loads overlap the tail of the predecessor kernel;
//   * the activations (M x k-slice, shared by the four warps) are staged once with cp.async;
//   * m16n8k16 bf16 mma.sync, one n8 tile per warp, MT m16 tiles per warp; results are stored from
//     the accumulator fragments.
// The k index inside a 32-wide chunk is permuted identically for A and B (thread t of a quad owns
// k = 8t ... 8t+7), which turns the fragment loads into one 16-byte access per row and chunk and
// leaves the sum unchanged.
// Split-K writes fp32 partial matrices [ksplit][M][N] that the residual + RMSNorm kernel adds in a
// fixed order, exactly like the tcgen05 path (reference op: luaTL_matmul, cuda/luaTL_core.cu:1506).
// The decode step uses it up to 32 sequences (measured faster than tcgen05 tiles there, slower at 64,
// where four row tiles per warp and a 64 KB activation stage per CTA weigh more than the tile set-up).
#include "common.cuh"
#include "ops.h"

namespace {

enum { ROWS_EPI_NONE = 0, ROWS_EPI_SWIGLU = 1, ROWS_EPI_RESID = 3 };
constexpr int ROWS_NC = 32;          // columns of C per CTA (one n8 tile per warp)
constexpr int ROWS_BATCH = 16;       // 32-wide k chunks whose weights are in registers at once
constexpr int ROWS_MAX_SMEM = 200 * 1024;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc)
{
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Bytes between rows of the staged activations: the slice plus padding that makes the pitch an odd
// multiple of 64 bytes, so that the eight threads of a 128-bit shared load phase hit 32 distinct banks.
__host__ __device__ inline int rows_pitch(int cps) { return cps * 64 + ((cps & 1) ? 0 : 64); }

// grid (ceil(N / 32), ksplit), 128 threads.  cps = 32-wide k chunks per slice.
// fz.ssq_in: rows are scaled by the deferred RMSNorm factor.  ROWS_EPI_RESID (N a multiple of 32): the CTA that
// draws the last ticket of its 32-column group adds the slices in slice order and the residual (see LtlGemmFuse);
// no CTA waits for another.
// FZ selects the instantiations that take the fusion arguments; the plain ones keep an empty parameter and none of the code.
struct NoFuse {};
template <bool FZ> struct FuseArg { typedef NoFuse type; };
template <> struct FuseArg<true> { typedef LtlGemmFuse type; };

template <int MT, typename TC, int EPI, bool FZ>
__global__ void __launch_bounds__(128)
gemm_rows_kernel(const bf16* __restrict__ A, const bf16* __restrict__ B, TC* __restrict__ C, int M, int N, int K, int cps,
                 const typename FuseArg<FZ>::type fz)
{
    extern __shared__ __align__(16) unsigned char rows_smem[];
    __shared__ float rsc[FZ ? MT * 16 : 1];
    __shared__ int ticket;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int n0 = blockIdx.x * ROWS_NC + warp * 8;
    const int c_begin = blockIdx.y * cps;
    const int nch = max(0, min(cps, K / 32 - c_begin));
    const int kbase = c_begin * 32;
    const int pitch = rows_pitch(cps);
    const int nrow = min(n0 + g, N - 1);                      // clamp: columns past N are computed and dropped
    const uint4* bp = reinterpret_cast<const uint4*>(B + (size_t)nrow * K + kbase) + t;

    uint4 bv[ROWS_BATCH];
#pragma unroll
    for (int j = 0; j < ROWS_BATCH; ++j)
        if (j < nch) bv[j] = __ldg(bp + j * 4);
    pdl_trigger();
    pdl_wait();
    constexpr bool scaled = FZ && EPI != ROWS_EPI_RESID;
    if constexpr (scaled) {
        if (threadIdx.x < MT * 16) {
            float sc = 1.0f;
            if ((int)threadIdx.x < M) {
                float ss = 0.0f;
                for (int q = 0; q < fz.ssq_tiles; ++q) ss += fz.ssq_in[(size_t)threadIdx.x * fz.ssq_tiles + q];
                sc = 1.0f / sqrtf(ss * fz.inv_dim + fz.eps);
            }
            rsc[threadIdx.x] = sc;                            // visible after the barrier below
        }
    }
    {
        const int per_row = nch * 4;                          // 16-byte pieces per activation row
        for (int i = threadIdx.x; i < MT * 16 * per_row; i += 128) {
            const int r = i / per_row, p = i - r * per_row;
            unsigned char* dst = rows_smem + r * pitch + p * 16;
            if (r < M) cp_async16(dst, A + (size_t)r * K + kbase + p * 8);
            else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
        }
        cp_async_wait_all();
        __syncthreads();
    }

    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) { acc[mt][0] = 0.0f; acc[mt][1] = 0.0f; acc[mt][2] = 0.0f; acc[mt][3] = 0.0f; }

    for (int c0 = 0; c0 < nch; c0 += ROWS_BATCH) {
        if (c0 > 0) {
#pragma unroll
            for (int j = 0; j < ROWS_BATCH; ++j)
                if (c0 + j < nch) bv[j] = __ldg(bp + (c0 + j) * 4);
        }
#pragma unroll
        for (int j = 0; j < ROWS_BATCH; ++j) {
            if (c0 + j < nch) {
                const unsigned char* ap = rows_smem + g * pitch + (c0 + j) * 64 + t * 16;
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const uint4 lo = *reinterpret_cast<const uint4*>(ap + (mt * 16) * pitch);
                    const uint4 hi = *reinterpret_cast<const uint4*>(ap + (mt * 16 + 8) * pitch);
                    mma_bf16_16816(acc[mt], lo.x, hi.x, lo.y, hi.y, bv[j].x, bv[j].y);
                    mma_bf16_16816(acc[mt], lo.z, hi.z, lo.w, hi.w, bv[j].z, bv[j].w);
                }
            }
        }
    }

    // Accumulator fragment: c0, c1 = (row g, columns 2t, 2t + 1), c2, c3 = (row g + 8, same columns).
    const int n = n0 + 2 * t;
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = mt * 16 + g + 8 * h;
            float v0 = acc[mt][2 * h], v1 = acc[mt][2 * h + 1];
            if (row >= M || n >= N) continue;
            if (scaled) { v0 *= rsc[row]; v1 *= rsc[row]; }
            if (EPI == ROWS_EPI_SWIGLU) {
                // interleaved (gate, up) columns; both rounded to bf16 first, as a stored gate|up tensor would be
                const float gt = __bfloat162float(__float2bfloat16_rn(v0)), up = __bfloat162float(__float2bfloat16_rn(v1));
                Cvt<TC>::st(C, (size_t)row * (N >> 1) + (n >> 1), silu_f(gt) * up);
            } else {
                TC* dst = C + (size_t)blockIdx.y * M * N + (size_t)row * N + n;
                if (n + 1 < N && (N & 1) == 0) {
                    if (sizeof(TC) == 4) *reinterpret_cast<float2*>(dst) = make_float2(v0, v1);
                    else *reinterpret_cast<uint32_t*>(dst) = pack_bf16x2(v0, v1);
                } else {
                    Cvt<TC>::st(dst, 0, v0);
                    if (n + 1 < N) Cvt<TC>::st(dst, 1, v1);
                }
            }
        }
    }
    if constexpr (EPI == ROWS_EPI_RESID && FZ) {
        __threadfence();                                      // this CTA's slice is visible before its ticket is drawn
        __syncthreads();
        if (threadIdx.x == 0) ticket = atomicAdd(fz.counters + blockIdx.x, 1);
        __syncthreads();
        if (ticket != (int)gridDim.y - 1) return;
        __threadfence();
        const int c4 = threadIdx.x & 7, col = blockIdx.x * ROWS_NC + c4 * 4;
        for (int base = 0; base < M * 8; base += 128) {       // 8 threads per row, 4 columns each; uniform trip count
            const int r = (base + (int)threadIdx.x) >> 3;
            float ss = 0.0f;
            if (r < M) {
                const float* pr = reinterpret_cast<const float*>(C) + (size_t)r * N + col;
                float* xr = fz.x + (size_t)r * N + col;
                float4 xv = *reinterpret_cast<const float4*>(xr);
                const float4 g = *reinterpret_cast<const float4*>(fz.gain + col);
                float4 a = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                for (int p0 = 0; p0 < (int)gridDim.y; p0 += 8) {          // eight slices in flight at a time
                    float4 q[8];
#pragma unroll
                    for (int p = 0; p < 8; ++p)
                        if (p0 + p < (int)gridDim.y) q[p] = __ldcg(reinterpret_cast<const float4*>(pr + (size_t)(p0 + p) * M * N));
#pragma unroll
                    for (int p = 0; p < 8; ++p)                            // slice order: the sum does not depend on arrival order
                        if (p0 + p < (int)gridDim.y) { a.x += q[p].x; a.y += q[p].y; a.z += q[p].z; a.w += q[p].w; }
                }
                xv.x += a.x; xv.y += a.y; xv.z += a.z; xv.w += a.w;
                *reinterpret_cast<float4*>(xr) = xv;
                ss = fmaf(xv.x, xv.x, fmaf(xv.y, xv.y, fmaf(xv.z, xv.z, xv.w * xv.w)));
                uint2 pk;
                pk.x = pack_bf16x2(xv.x * g.x, xv.y * g.y);
                pk.y = pack_bf16x2(xv.z * g.z, xv.w * g.w);
                *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(fz.h) + (size_t)r * N + col) = pk;
            }
            ss += __shfl_xor_sync(0xFFFFFFFFu, ss, 1);
            ss += __shfl_xor_sync(0xFFFFFFFFu, ss, 2);
            ss += __shfl_xor_sync(0xFFFFFFFFu, ss, 4);
            if (r < M && c4 == 0) fz.ssq_out[(size_t)r * gridDim.x + blockIdx.x] = ss;
        }
        if (threadIdx.x == 0) fz.counters[blockIdx.x] = 0;    // ready for the next launch
    }
}

template <int MT, typename TC, int EPI, bool FZ, typename FA>
int launch_rows_fz(const void* A, const void* B, void* C, int M, int N, int K, int ksplit, cudaStream_t s, const FA& fa)
{
    const int kc = K / 32, cps = (kc + ksplit - 1) / ksplit;
    const size_t smem = (size_t)MT * 16 * rows_pitch(cps);
    static bool attr_set = false;
    if (!attr_set) {
        LTL_CUDA("gemm_rows smem attribute", cudaFuncSetAttribute(gemm_rows_kernel<MT, TC, EPI, FZ>, cudaFuncAttributeMaxDynamicSharedMemorySize, ROWS_MAX_SMEM));
        attr_set = true;
    }
    LTL_CUDA("gemm_rows launch", ltl_launch(gemm_rows_kernel<MT, TC, EPI, FZ>, dim3((N + ROWS_NC - 1) / ROWS_NC, ksplit), dim3(128), smem, s,
                                            ltl_pdl_enabled(), (const bf16*)A, (const bf16*)B, (TC*)C, M, N, K, cps, fa));
    return ltl_check_launch("gemm_rows");
}

template <int MT, typename TC, int EPI>
int launch_rows(const void* A, const void* B, void* C, int M, int N, int K, int ksplit, cudaStream_t s, const LtlGemmFuse& fz)
{
    if (EPI == ROWS_EPI_RESID || fz.ssq_in) return launch_rows_fz<MT, TC, EPI, true>(A, B, C, M, N, K, ksplit, s, fz);
    if constexpr (EPI == ROWS_EPI_RESID) return ltl_fail(LTL_ERR_ARG, "gemm_rows: the residual form needs its fusion arguments");
    else return launch_rows_fz<MT, TC, EPI, false>(A, B, C, M, N, K, ksplit, s, NoFuse{});
}

template <typename TC, int EPI>
int launch_rows_mt(const void* A, const void* B, void* C, int M, int N, int K, int ksplit, cudaStream_t s, const LtlGemmFuse& fz)
{
    switch ((M + 15) / 16) {
    case 1: return launch_rows<1, TC, EPI>(A, B, C, M, N, K, ksplit, s, fz);
    case 2: return launch_rows<2, TC, EPI>(A, B, C, M, N, K, ksplit, s, fz);
    case 3: return launch_rows<3, TC, EPI>(A, B, C, M, N, K, ksplit, s, fz);
    default: return launch_rows<4, TC, EPI>(A, B, C, M, N, K, ksplit, s, fz);
    }
}

}  // namespace

// 1 ... 64 rows, K a multiple of 32, 16-byte aligned operands, and an activation slice that fits shared memory.
bool ltl_gemm_rows_supported(const void* A, const void* B, int M, int N, int K, int ksplit)
{
    if (M < 1 || M > 64 || N < 1 || K < 32 || (K % 32) || ksplit < 1) return false;
    if (((uintptr_t)A | (uintptr_t)B) & 15) return false;
    const int kc = K / 32, cps = (kc + ksplit - 1) / ksplit;
    return (size_t)((M + 15) / 16) * 16 * rows_pitch(cps) <= (size_t)ROWS_MAX_SMEM;
}

// Slice count for a GEMM whose output goes to fp32 partial matrices: enough slices to give every SM a CTA,
// at most max_parts and at most one per 32-wide k chunk.
int ltl_gemm_rows_plan_split(int N, int K, int max_parts)
{
    const int groups = (N + ROWS_NC - 1) / ROWS_NC, kc = K / 32;
    int s = groups > 0 ? (ltl_sm_count() + groups - 1) / groups : 1;
    if (s > max_parts) s = max_parts;
    if (s > kc) s = kc;
    if (s < 1) s = 1;
    const int cps = (kc + s - 1) / s;
    return (kc + cps - 1) / cps;                               // no empty trailing slices
}

// C (c_dtype f32 or bf16) = A[M,K] B[N,K]^T.  epi = 1: SwiGLU over interleaved (gate, up) rows of B, C is
// [M, N/2] bf16.  ksplit > 1: C receives ksplit fp32 partial matrices [ksplit][M][N].
int ltl_gemm_rows(const void* A, const void* B, void* C, int M, int N, int K, int c_dtype, int epi, int ksplit, cudaStream_t s,
                  const LtlGemmFuse* fuse)
{
    const LtlGemmFuse fz = fuse ? *fuse : LtlGemmFuse{};
    if (!A || !B || !C) return ltl_fail(LTL_ERR_NULL, "gemm_rows: null operand");
    if (!ltl_gemm_rows_supported(A, B, M, N, K, ksplit))
        return ltl_fail(LTL_ERR_UNSUPPORTED, "gemm_rows: needs 1 <= M <= 64, K %% 32 == 0, 16-byte aligned operands (M=%d N=%d K=%d ksplit=%d)", M, N, K, ksplit);
    if (epi == ROWS_EPI_RESID) {
        if (c_dtype != LTL_F32 || (N % 32) || !fz.x || !fz.gain || !fz.h || !fz.ssq_out || !fz.counters)
            return ltl_fail(LTL_ERR_ARG, "gemm_rows: the residual form needs fp32 slices, N %% 32 == 0 and all of x, gain, h, ssq_out, counters");
        return launch_rows_mt<float, ROWS_EPI_RESID>(A, B, C, M, N, K, ksplit, s, fz);
    }
    if (ksplit > 1 && (c_dtype != LTL_F32 || epi || fz.ssq_in))
        return ltl_fail(LTL_ERR_ARG, "gemm_rows: split-K writes fp32 partial sums and takes no epilogue");
    if (epi == ROWS_EPI_SWIGLU) {
        if (c_dtype != LTL_BF16 || (N & 1)) return ltl_fail(LTL_ERR_ARG, "gemm_rows: the SwiGLU epilogue writes bf16 and needs an even N");
        return launch_rows_mt<bf16, ROWS_EPI_SWIGLU>(A, B, C, M, N, K, 1, s, fz);
    }
    if (epi != ROWS_EPI_NONE) return ltl_fail(LTL_ERR_ARG, "gemm_rows: epilogue %d", epi);
    if (c_dtype == LTL_F32) return launch_rows_mt<float, ROWS_EPI_NONE>(A, B, C, M, N, K, ksplit, s, fz);
    if (c_dtype == LTL_BF16) return launch_rows_mt<bf16, ROWS_EPI_NONE>(A, B, C, M, N, K, 1, s, fz);
    return ltl_fail(LTL_ERR_DTYPE, "gemm_rows: output dtype %d", c_dtype);
}
