// Tensor-core GEMM for fp32 models: C[M,N] (+)= A[M,K] * B[N,K]^T (+ R), fp32 operands read by the tensor cores as TF32
// (10-bit mantissa), fp32 accumulation in tensor memory.
//
// It takes the place of the reference's dominant kernel for fp32 models - the register-tiled CUDA-core GEMM
// (cuda/luaTL_train.cu:242, chosen at :425) - wherever the 2e-3 tolerance of tensor-core arithmetic is accepted
// (luaTL_lm_set_tf32); the exact CUDA-core kernel (gemm_simt.cu) stays the default of fp32 models and the 1e-4 path.
//
//   - both operands K-major (the contraction index contiguous): A is an activation matrix [M, K], B a matrix stored
//     [N, K] - a transposed weight mirror in the forward, the fp32 master itself in dX = dY W^T, transposed activations
//     in dW = X^T dY;
//   - TMA (cp.async.bulk.tensor.2d, fp32 boxes of 32 columns = 128 bytes, 128-byte swizzle, zero fill outside the
//     matrix) into a ring of shared-memory stages guarded by full / empty mbarriers;
//   - one elected thread issues tcgen05.mma kind::tf32 (UMMA 128 x BN x 8), accumulator in TMEM;
//   - four epilogue warps read their lane quadrant with tcgen05.ld and store (+ residual), or add with red.global.add
//     (accumulating form: split-K slices of a long reduction, and beta = 1).
// Warp roles as in the bf16 kernel: warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer, warps 2..5 = epilogue.
// Every wait is bounded and raises the shared error flag; no cluster launch, no TMA multicast.
#include <cuda.h>

#include <algorithm>
#include <map>
#include <tuple>

#include "ops.h"
#include "tc_common.cuh"

namespace {

using namespace tc;
constexpr int BM = 128, BK = 32, UMMA_K = 8;          // 32 fp32 = 128 bytes per swizzled row; 8 elements = 32 bytes per UMMA
constexpr int MAX_STAGES = 6;

struct Bars {
    uint64_t full[MAX_STAGES], empty[MAX_STAGES], acc_ready;
    uint32_t tmem_base;
};
template <int BN> constexpr size_t stage_bytes() { return (size_t)(BM + BN) * BK * 4; }
template <int BN> constexpr int ring_depth() { return BN == 128 ? 5 : 6; }
template <int BN> size_t smem_bytes(int stages) { return stages * stage_bytes<BN>() + sizeof(Bars) + 1024; }

// ACC = 0: C = product (+ R).  ACC = 1: C += product with atomic adds (gridDim.z slices of K add into the same C).
template <int BN, int ACC>
__global__ void __launch_bounds__(192, 1)
gemm_tf32_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 float* C, const float* R, int M, int N, int K, int STAGES, int* __restrict__ err)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* const tiles = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* const tiles_b = tiles + (size_t)STAGES * (BM * BK * 4);
    Bars& sm = *reinterpret_cast<Bars*>(tiles_b + (size_t)STAGES * (BN * BK * 4));
    auto a_tile = [&](int st) { return tiles + (size_t)st * (BM * BK * 4); };
    auto b_tile = [&](int st) { return tiles_b + (size_t)st * (BN * BK * 4); };
    constexpr uint32_t TMEM_COLS = BN < 32 ? 32 : BN;
    constexpr uint32_t STAGE_BYTES = (BM + BN) * BK * 4;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int kb_all = (K + BK - 1) / BK;
    const int kb_per = (kb_all + gridDim.z - 1) / gridDim.z;
    const int kb0 = blockIdx.z * kb_per;
    const int kblocks = max(0, min(kb_all, kb0 + kb_per) - kb0);

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

    if (warp == 0 && lane == 0) {
        // ---- TMA producer ----
        int s = 0;
        uint32_t round = 0;
        for (int kb = 0; kb < kblocks && ok; ++kb, ++s) {
            if (s == STAGES) { s = 0; ++round; }
            if (round > 0) ok = mbar_wait(&sm.empty[s], (round - 1) & 1);
            if (!ok) break;
            mbar_expect_tx(&sm.full[s], STAGE_BYTES);
            tma_load_2d(a_tile(s), &map_a, (kb0 + kb) * BK, m0, &sm.full[s]);
            tma_load_2d(b_tile(s), &map_b, (kb0 + kb) * BK, n0, &sm.full[s]);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ----
        constexpr uint32_t idesc = umma_idesc_tf32(BM, BN);
        int s = 0;
        uint32_t round = 0;
        for (int kb = 0; kb < kblocks && ok; ++kb, ++s) {
            if (s == STAGES) { s = 0; ++round; }
            ok = mbar_wait(&sm.full[s], round & 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da = umma_desc_sw128(smem_u32(a_tile(s)));
            const uint64_t db = umma_desc_sw128(smem_u32(b_tile(s)));
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)            // 32 bytes further along K per UMMA
                umma_tf32(tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) ? 1u : 0u);
            umma_commit(&sm.empty[s]);                        // frees the stage when these MMAs retire
        }
        umma_commit(&sm.acc_ready);
    } else if (warp >= 2) {
        // ---- epilogue: TMEM -> registers -> global ----
        ok = mbar_wait(&sm.acc_ready, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int quad = warp & 3;                            // TMEM lane quadrant this warp may read
        const int row = m0 + quad * 32 + lane;
        if (ok) {
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (n0 + c0 >= N) break;
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)(quad * 32) << 16) + (uint32_t)c0, v);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row >= M || (ACC && kblocks == 0)) continue;
                if (kblocks == 0) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0u;
                }
                const size_t base = (size_t)row * N + n0 + c0;
                const int ncols = min(32, N - (n0 + c0));
                float* dst = C + base;
                if (ACC) {
                    if (ncols == 32 && (N & 3) == 0) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst + j),
                                         "f"(__uint_as_float(v[j])), "f"(__uint_as_float(v[j + 1])),
                                         "f"(__uint_as_float(v[j + 2])), "f"(__uint_as_float(v[j + 3])) : "memory");
                    } else {
                        for (int j = 0; j < ncols; ++j) atomicAdd(dst + j, __uint_as_float(v[j]));
                    }
                } else if (ncols == 32 && (N & 3) == 0) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        float4 o = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]), __uint_as_float(v[j + 3]));
                        if (R) {
                            const float4 r = *reinterpret_cast<const float4*>(R + base + j);
                            o.x += r.x; o.y += r.y; o.z += r.z; o.w += r.w;
                        }
                        *reinterpret_cast<float4*>(dst + j) = o;
                    }
                } else {
                    for (int j = 0; j < ncols; ++j) dst[j] = __uint_as_float(v[j]) + (R ? R[base + j] : 0.0f);
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
        return ltl_fail(LTL_ERR_UNSUPPORTED, "gemm_tf32: cuTensorMapEncodeTiled is not available from this driver");
    }
    g_encode = (encode_fn)fn;
    return LTL_OK;
}

// fp32 matrix [rows, cols] with rows `pitch` elements apart; boxes of box_rows x 32 columns, 128-byte swizzle, zero fill.
std::map<std::tuple<const void*, int, int, long long, int>, CUtensorMap> g_maps;

int tensor_map(const void* base, int rows, int cols, long long pitch, int box_rows, CUtensorMap* out)
{
    const auto key = std::make_tuple(base, rows, cols, pitch, box_rows);
    const auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return LTL_OK; }
    LTL_TRY(get_encode());
    const cuuint64_t dims[2] = { (cuuint64_t)cols, (cuuint64_t)rows };
    const cuuint64_t strides[1] = { (cuuint64_t)pitch * 4 };
    const cuuint32_t box[2] = { (cuuint32_t)BK, (cuuint32_t)box_rows };
    const cuuint32_t estr[2] = { 1, 1 };
    const CUresult r = g_encode(out, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(base), dims, strides, box, estr,
                                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return ltl_fail(LTL_ERR_CUDA, "gemm_tf32: cuTensorMapEncodeTiled failed (%d) for %dx%d", (int)r, rows, cols);
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps[key] = *out;
    return LTL_OK;
}

template <int BN, int ACC>
int launch(const float* A, const float* B, float* C, const float* R, int M, int N, int K, int ksplit, cudaStream_t s)
{
    CUtensorMap ma, mb;
    LTL_TRY(tensor_map(A, M, K, K, BM, &ma));
    LTL_TRY(tensor_map(B, N, K, K, BN, &mb));
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, ksplit < 1 ? 1 : ksplit);
    const int kb_all = (K + BK - 1) / BK;
    const int kb_per = (kb_all + (int)grid.z - 1) / (int)grid.z;
    int stages = ring_depth<BN>();
    if (stages > kb_per) stages = kb_per;
    if (stages < 1) stages = 1;
    static bool attr_set = false;
    if (!attr_set) {
        LTL_CUDA("gemm_tf32 attr", cudaFuncSetAttribute(gemm_tf32_kernel<BN, ACC>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                        (int)smem_bytes<BN>(ring_depth<BN>())));
        attr_set = true;
    }
    gemm_tf32_kernel<BN, ACC><<<grid, 192, smem_bytes<BN>(stages), s>>>(ma, mb, C, R, M, N, K, stages, ltl_tc_err_flag());
    return ltl_check_launch("gemm_tf32");
}

}  // namespace

bool ltl_gemm_tf32_supported(const void* A, const void* B, const void* C, int M, int N, int K)
{
    return M > 0 && N > 0 && K > 0 && K % 4 == 0 &&
           ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(C)) & 15) == 0;
}

// C[M,N] = A[M,K] B[N,K]^T + R (accumulate = 0; R optional, may be C), or C += A B^T (accumulate = 1, R ignored): fp32 in
// memory, TF32 products, fp32 accumulation.  ksplit > 1 (accumulate only): slices of K add into C with atomics;
// ksplit = 0 picks a slice count that fills the SMs.
int ltl_gemm_tf32(const float* A, const float* B, float* C, const float* R, int M, int N, int K, int accumulate, int ksplit,
                  cudaStream_t s)
{
    if (!A || !B || !C) return ltl_fail(LTL_ERR_NULL, "gemm_tf32: null operand");
    if (!ltl_gemm_tf32_supported(A, B, C, M, N, K))
        return ltl_fail(LTL_ERR_UNSUPPORTED, "gemm_tf32: needs K %% 4 == 0 and 16-byte aligned operands (M=%d N=%d K=%d)", M, N, K);
    if (!ltl_tc_err_flag()) return ltl_fail(LTL_ERR_OOM, "gemm_tf32: error flag");
    const int mt = (M + BM - 1) / BM, sms = ltl_sm_count();
    // the widest tile that still gives every SM a CTA; the narrow one otherwise
    const int bn = (N >= 128 && (long long)mt * ((N + 127) / 128) >= sms) ? 128 : 64;
    if (!accumulate) {
        if (bn == 128) return launch<128, 0>(A, B, C, R, M, N, K, 1, s);
        return launch<64, 0>(A, B, C, R, M, N, K, 1, s);
    }
    if (ksplit <= 0) {
        const int tiles = mt * ((N + bn - 1) / bn), kb = (K + BK - 1) / BK;
        ksplit = (2 * sms + tiles - 1) / tiles;
        if (ksplit > kb / 4) ksplit = kb / 4;
        if (ksplit > 64) ksplit = 64;
        if (ksplit < 1) ksplit = 1;
    }
    if (bn == 128) return launch<128, 1>(A, B, C, nullptr, M, N, K, ksplit, s);
    return launch<64, 1>(A, B, C, nullptr, M, N, K, ksplit, s);
}
