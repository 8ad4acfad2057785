// CUDA-core GEMM with explicit element strides and a batch dimension:
//   C[b][m][n] = post(alpha * sum_k A[b][m][k] * B[b][k][n] + bias[n]) + beta * C[b][m][n] + R[b][m][n]
// with A(m,k) at A + b*a_bs + m*a_rs + k*a_cs and likewise for B and C (R shares C's strides).
// This is the contract of the reference's luaTL_gemm_ex (cuda/luaTL_train.cu:112-123): one
// kernel serves row-major, logically transposed (dX = dY W^T, dW = X^T dY, tied head
// B = emb^T) and per-head batched operands without materialising a transpose.
//
// It is the exact-fp32 path (fp32 multiply-add, the accuracy the 1e-4 parity bound needs)
// and the shape-agnostic path for operands the tensor-core kernel cannot take.  64x64x16
// tiles, 256 threads, 4x4 outputs per thread; the tile loader walks whichever operand
// dimension has unit stride so global loads stay coalesced for every layout above.
#include "ops.h"

namespace {

constexpr int BM = 64, BN = 64, BK = 16, PAD = 4;

__device__ __forceinline__ float act_apply(int op, float v)
{
    switch (op) {
        case 1: return fmaxf(v, 0.0f);
        case 2: { const float t = 0.7978845608028654f * (v + 0.044715f * v * v * v);
                  return 0.5f * v * (1.0f + tanhf(t)); }
        case 3: return v / (1.0f + expf(-v));
        case 4: return tanhf(v);
        case 5: return 1.0f / (1.0f + expf(-v));
        default: return v;
    }
}

// PRE: the instantiation that carries the prologue on A; the plain one has none of its code (the tile loader is the hot loop).
template <typename TI, typename TC, bool PRE>
__global__ void __launch_bounds__(256)
gemm_simt_kernel(const TI* __restrict__ A, const TI* __restrict__ B, TC* C,
                 const TI* __restrict__ bias, const TC* R, int M, int N, int K,
                 long long a_rs, long long a_cs, long long b_rs, long long b_cs,
                 long long c_rs, long long c_cs, long long a_bs, long long b_bs, long long c_bs,
                 float alpha, float beta, int post_op, int ksplit,
                 int pre_op, const TI* __restrict__ gamma, const float* __restrict__ rowscale, float eps)
{
    __shared__ __align__(16) float As[BK][BM + PAD];
    __shared__ __align__(16) float Bs[BK][BN + PAD];
    __shared__ float rowsc[PRE ? BM : 1];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    // ksplit > 1 (batch == 1 only): blockIdx.z selects a slice of K and the partial product is
    // added to C with atomics (the caller guarantees beta == 1, fp32 C, no bias / activation / R).
    int k_begin = 0, k_end = K;
    if (ksplit > 1) {
        const int per = ((K + ksplit - 1) / ksplit + BK - 1) / BK * BK;
        k_begin = blockIdx.z * per;
        k_end = min(K, k_begin + per);
    } else {
        A += (long long)blockIdx.z * a_bs;
        B += (long long)blockIdx.z * b_bs;
        C += (long long)blockIdx.z * c_bs;
        if (R) R += (long long)blockIdx.z * c_bs;
    }
    const int tx = tid & 15, ty = tid >> 4;
    if (PRE && pre_op == 1) {
        // RMSNorm prologue: the factor of each of the tile's 64 rows - taken from rowscale, or computed here over the
        // whole of K (four threads per row; every CTA of a row block repeats it, which keeps the op free of scratch).
        const int r = tid >> 2, q = tid & 3, gm = m0 + r;
        float part = 0.0f;
        if (!rowscale && gm < M)
            for (int k = q; k < K; k += 4) {
                const float a = Cvt<TI>::ld(A, (size_t)(gm * a_rs + k * a_cs));
                part = fmaf(a, a, part);
            }
        part += __shfl_xor_sync(0xFFFFFFFFu, part, 1);
        part += __shfl_xor_sync(0xFFFFFFFFu, part, 2);
        if (q == 0) rowsc[r] = gm < M ? (rowscale ? rowscale[gm] : rsqrtf(part / (float)K + eps)) : 0.0f;
        __syncthreads();
    }
    const bool a_kfast = (a_cs == 1);      // k contiguous in memory
    const bool b_nfast = (b_cs == 1);      // n contiguous in memory

    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0f;

    for (int k0 = k_begin; k0 < k_end; k0 += BK) {
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            int mm, kk;
            if (a_kfast) { kk = tid & 15; mm = (tid >> 4) + 16 * p; }
            else         { mm = tid & 63; kk = (tid >> 6) + 4 * p; }
            const int gm = m0 + mm, gk = k0 + kk;
            float av = (gm < M && gk < k_end) ? Cvt<TI>::ld(A, (size_t)(gm * a_rs + gk * a_cs)) : 0.0f;
            if (PRE) {
                if (pre_op == 1) av = av * rowsc[mm] * ((gamma && gk < k_end) ? Cvt<TI>::ld(gamma, gk) : 1.0f);
                else if (pre_op == 2) av = act_apply(2, av);
                else if (pre_op == 3) av = act_apply(3, av);
                else if (pre_op == 4) av = fmaxf(av, 0.0f);
            }
            As[kk][mm] = av;
            int nn, kb;
            if (b_nfast) { nn = tid & 63; kb = (tid >> 6) + 4 * p; }
            else         { kb = tid & 15; nn = (tid >> 4) + 16 * p; }
            const int gn = n0 + nn, gkb = k0 + kb;
            Bs[kb][nn] = (gn < N && gkb < k_end) ? Cvt<TI>::ld(B, (size_t)(gkb * b_rs + gn * b_cs)) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            const float4 a = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
            const float av[4] = { a.x, a.y, a.z, a.w }, bv[4] = { b.x, b.y, b.z, b.w };
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            const size_t ci = (size_t)(gm * c_rs + gn * c_cs);
            if (ksplit > 1) {
                if (sizeof(TC) == 4) atomicAdd(reinterpret_cast<float*>(C) + ci, alpha * acc[i][j]);
                continue;
            }
            float v = alpha * acc[i][j];
            if (bias) v += Cvt<TI>::ld(bias, gn);
            v = act_apply(post_op, v);
            if (beta != 0.0f) v += beta * Cvt<TC>::ld(C, ci);
            if (R) v += Cvt<TC>::ld(R, ci);
            Cvt<TC>::st(C, ci, v);
        }
    }
}

template <typename TI, typename TC>
int launch(const GemmDesc& g, cudaStream_t s)
{
    // Weight-gradient shape (dW += X^T dY): a small output with a very long reduction would run on a
    // handful of CTAs; spread K over the SMs and accumulate with fp32 atomics instead.
    int ksplit = 1;
    const int tiles = ((g.N + BN - 1) / BN) * ((g.M + BM - 1) / BM);
    if (g.batch == 1 && g.beta == 1.0f && !g.bias && !g.R && g.post_op == 0 && g.pre_op == 0 && sizeof(TC) == 4 &&
        tiles * 2 <= ltl_sm_count() && g.K >= 8 * BK) {
        ksplit = (2 * ltl_sm_count() + tiles - 1) / tiles;
        if (ksplit > g.K / (2 * BK)) ksplit = g.K / (2 * BK);
        if (ksplit > 64) ksplit = 64;
        if (ksplit < 1) ksplit = 1;
    }
    dim3 grid((g.N + BN - 1) / BN, (g.M + BM - 1) / BM, ksplit > 1 ? ksplit : g.batch);
    if (g.pre_op)
        gemm_simt_kernel<TI, TC, true><<<grid, 256, 0, s>>>(
            (const TI*)g.A, (const TI*)g.B, (TC*)g.C, (const TI*)g.bias, (const TC*)g.R, g.M, g.N, g.K,
            g.a_rs, g.a_cs, g.b_rs, g.b_cs, g.c_rs, g.c_cs, g.a_bs, g.b_bs, g.c_bs, g.alpha, g.beta,
            g.post_op, ksplit, g.pre_op, (const TI*)g.gamma, g.rowscale, g.eps);
    else
        gemm_simt_kernel<TI, TC, false><<<grid, 256, 0, s>>>(
            (const TI*)g.A, (const TI*)g.B, (TC*)g.C, (const TI*)g.bias, (const TC*)g.R, g.M, g.N, g.K,
            g.a_rs, g.a_cs, g.b_rs, g.b_cs, g.c_rs, g.c_cs, g.a_bs, g.b_bs, g.c_bs, g.alpha, g.beta,
            g.post_op, ksplit, 0, nullptr, nullptr, 0.0f);
    return ltl_check_launch("gemm");
}

}  // namespace

int ltl_gemm_simt(const GemmDesc& g, cudaStream_t s)
{
    if (!g.A || !g.B || !g.C) return ltl_fail(LTL_ERR_NULL, "gemm: null operand");
    if (g.M < 0 || g.N < 0 || g.K < 0 || g.batch < 0)
        return ltl_fail(LTL_ERR_SHAPE, "gemm: bad shape M=%d N=%d K=%d batch=%d", g.M, g.N, g.K, g.batch);
    if (g.M == 0 || g.N == 0 || g.batch == 0) return LTL_OK;
    if (g.batch > 65535 || (g.M + BM - 1) / BM > 65535)
        return ltl_fail(LTL_ERR_SHAPE, "gemm: grid too large (M=%d batch=%d)", g.M, g.batch);
    if (g.a_dtype != g.b_dtype) return ltl_fail(LTL_ERR_DTYPE, "gemm: A and B dtypes differ");
    if (g.post_op < 0 || g.post_op > 5) return ltl_fail(LTL_ERR_ARG, "gemm: unknown post_op %d", g.post_op);
    if (g.pre_op < 0 || g.pre_op > 4) return ltl_fail(LTL_ERR_ARG, "gemm: unknown pre_op %d", g.pre_op);
    const int ti = g.a_dtype, tc = g.c_dtype;
    if (ti == LTL_F32 && tc == LTL_F32) return launch<float, float>(g, s);
    if (ti == LTL_BF16 && tc == LTL_BF16) return launch<bf16, bf16>(g, s);
    if (ti == LTL_BF16 && tc == LTL_F32) return launch<bf16, float>(g, s);
    if (ti == LTL_F16 && tc == LTL_F16) return launch<__half, __half>(g, s);
    if (ti == LTL_F16 && tc == LTL_F32) return launch<__half, float>(g, s);
    return ltl_fail(LTL_ERR_DTYPE, "gemm: unsupported dtype combination in=%d out=%d", ti, tc);
}
