// The part of the reference's FFI surface that the token loop itself never calls, kept so that the reference's
// LuaJIT bindings (ai/gpu/luaTL.lua:66-167, ai/gpu/luaTL_train.lua:27-89) resolve every symbol they declare:
// streams and page-locked host memory, extra pools and bump arenas, the legacy raw-pointer calls, the GEMM planner,
// the small row / column ops, the legacy float-only wrappers and the v1 Pipeline command buffer.
//
// Each entry point keeps the reference's argument meaning and status codes (definitions cited per function); the
// kernels behind them are plain, correct, coalesced kernels - nothing here is on the token loop's critical path.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/luatl_b200.h"
#include "ops.h"

namespace {

#define COMPAT_DISPATCH_T(dt, ...)                                                   \
    do {                                                                             \
        if ((dt) == LTL_F32) { typedef float T; __VA_ARGS__; }                       \
        else if ((dt) == LTL_BF16) { typedef bf16 T; __VA_ARGS__; }                  \
        else if ((dt) == LTL_F16) { typedef __half T; __VA_ARGS__; }                 \
        else return ltl_fail(LTL_ERR_DTYPE, "unknown dtype %d", (int)(dt));          \
    } while (0)

unsigned grid_for(uint64_t items, int block)
{
    uint64_t g = (items + block - 1) / block;
    const uint64_t cap = (uint64_t)ltl_sm_count() * 16;
    if (g > cap) g = cap;
    return (unsigned)(g < 1 ? 1 : g);
}

// One thread per column, rows walked in order: consecutive threads read consecutive addresses.
template <typename T>
__global__ void reduce_cols_kernel(const T* __restrict__ x, float* __restrict__ out, int rows, int cols,
                                   long long rs, float alpha, float beta)
{
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float acc = 0.0f;
    for (int r = 0; r < rows; ++r) acc += Cvt<T>::ld(x, (size_t)(r * rs + c));
    out[c] = alpha * acc + (beta != 0.0f ? beta * out[c] : 0.0f);
}

template <typename T>
__global__ void bcast_add_kernel(const T* __restrict__ x, const T* __restrict__ v, T* __restrict__ out,
                                 uint64_t n, int cols, float alpha)
{
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
        const float b = v ? Cvt<T>::ld(v, (size_t)(i % (uint64_t)cols)) : 0.0f;
        Cvt<T>::st(out, (size_t)i, Cvt<T>::ld(x, (size_t)i) + alpha * b);
    }
}

// 32 x 32 tile through shared memory (row of 33 floats: no bank conflicts); reads and writes both coalesced.
template <typename T>
__global__ void transpose_kernel(const T* __restrict__ in, T* __restrict__ out, int rows, int cols)
{
    __shared__ float tile[32][33];
    const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int r = r0 + j, c = c0 + threadIdx.x;
        tile[j][threadIdx.x] = (r < rows && c < cols) ? Cvt<T>::ld(in, (size_t)r * cols + c) : 0.0f;
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int oc = c0 + j, orow = r0 + threadIdx.x;          // out[oc][orow]
        if (oc < cols && orow < rows) Cvt<T>::st(out, (size_t)oc * rows + orow, tile[threadIdx.x][j]);
    }
}

template <typename T>
__global__ void gather_rows_kernel(const T* __restrict__ src, const int32_t* __restrict__ idx, T* __restrict__ dst,
                                   int n, int cols, int src_rows)
{
    const uint64_t total = (uint64_t)n * cols;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (uint64_t)gridDim.x * blockDim.x) {
        const int r = (int)(i / (uint64_t)cols), c = (int)(i - (uint64_t)r * cols);
        const int sr = idx[r];
        Cvt<T>::st(dst, (size_t)i, (sr >= 0 && sr < src_rows) ? Cvt<T>::ld(src, (size_t)sr * cols + c) : 0.0f);
    }
}

// One warp per row, shuffle reduction.
template <typename T>
__global__ void row_rms_kernel(const T* __restrict__ x, float* __restrict__ out, int rows, int cols,
                               long long rs, long long cs, float eps)
{
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows) return;
    float acc = 0.0f;
    for (int c = lane; c < cols; c += 32) {
        const float v = Cvt<T>::ld(x, (size_t)(row * rs + c * cs));
        acc = fmaf(v, v, acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) out[row] = rsqrtf(acc / (float)cols + eps);
}

}  // namespace

int ltl_reduce_cols(const void* x, float* out, int rows, int cols, long long row_stride, float alpha, float beta,
                    int dtype, cudaStream_t s)
{
    if (!x || !out) return ltl_fail(LTL_ERR_NULL, "reduce_cols: null pointer");
    if (rows < 0 || cols <= 0) return ltl_fail(LTL_ERR_SHAPE, "reduce_cols: bad shape %dx%d", rows, cols);
    COMPAT_DISPATCH_T(dtype, reduce_cols_kernel<T><<<(cols + 127) / 128, 128, 0, s>>>((const T*)x, out, rows, cols,
                                                                                      row_stride, alpha, beta));
    return ltl_check_launch("reduce_cols");
}

int ltl_transpose(const void* in, void* out, int rows, int cols, int dtype, cudaStream_t s)
{
    if (!in || !out) return ltl_fail(LTL_ERR_NULL, "transpose: null pointer");
    if (rows <= 0 || cols <= 0) return ltl_fail(LTL_ERR_SHAPE, "transpose: bad shape %dx%d", rows, cols);
    const dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
    if (grid.y > 65535) return ltl_fail(LTL_ERR_SHAPE, "transpose: %d rows exceed the grid", rows);
    COMPAT_DISPATCH_T(dtype, transpose_kernel<T><<<grid, block, 0, s>>>((const T*)in, (T*)out, rows, cols));
    return ltl_check_launch("transpose");
}

int ltl_bcast_add(const void* x, const void* v, void* out, int rows, int cols, float alpha, int dtype, cudaStream_t s)
{
    if (!x || !out) return ltl_fail(LTL_ERR_NULL, "bcast_add: null pointer");
    if (rows <= 0 || cols <= 0) return ltl_fail(LTL_ERR_SHAPE, "bcast_add: bad shape %dx%d", rows, cols);
    const uint64_t n = (uint64_t)rows * cols;
    COMPAT_DISPATCH_T(dtype, bcast_add_kernel<T><<<grid_for(n, 256), 256, 0, s>>>((const T*)x, (const T*)v, (T*)out, n, cols, alpha));
    return ltl_check_launch("bcast_add");
}

int ltl_gather_rows(const void* src, const int32_t* idx, void* dst, int n, int cols, int src_rows, int dtype, cudaStream_t s)
{
    if (!src || !idx || !dst) return ltl_fail(LTL_ERR_NULL, "gather_rows: null pointer");
    if (n < 0 || cols <= 0) return ltl_fail(LTL_ERR_SHAPE, "gather_rows: bad shape %dx%d", n, cols);
    if (n == 0) return LTL_OK;
    COMPAT_DISPATCH_T(dtype, gather_rows_kernel<T><<<grid_for((uint64_t)n * cols, 256), 256, 0, s>>>(
        (const T*)src, idx, (T*)dst, n, cols, src_rows));
    return ltl_check_launch("gather_rows");
}

int ltl_row_rms(const void* x, float* out, int rows, int cols, long long rs, long long cs, float eps, int dtype, cudaStream_t s)
{
    if (!x || !out) return ltl_fail(LTL_ERR_NULL, "row_rms: null pointer");
    if (rows <= 0 || cols <= 0) return ltl_fail(LTL_ERR_SHAPE, "row_rms: bad shape %dx%d", rows, cols);
    COMPAT_DISPATCH_T(dtype, row_rms_kernel<T><<<(rows + 7) / 8, 256, 0, s>>>((const T*)x, out, rows, cols, rs, cs, eps));
    return ltl_check_launch("row_rms");
}

#define ONE_SHOT(ctx, call)                         \
    do {                                            \
        LTL_TRY(ltl_require_init(ctx));             \
        LTL_TRY(call);                              \
        return ltl_sync_stream(ctx);                \
    } while (0)

extern "C" {

// ---------------- streams and page-locked host memory (cuda/luaTL_core.cu:1776-1813) -----------------------------
void* luaTL_stream_create(int nonblocking)
{
    if (ltl_require_init("stream_create") != LTL_OK) return nullptr;
    cudaStream_t s = nullptr;
    const cudaError_t e = nonblocking ? cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) : cudaStreamCreate(&s);
    if (e != cudaSuccess) { ltl_cuda_fail("cudaStreamCreate", e); return nullptr; }
    return (void*)s;
}
void luaTL_stream_destroy(void* s)
{
    if (!s) return;
    cudaStreamDestroy((cudaStream_t)s);
    cudaGetLastError();
}
int luaTL_stream_sync(void* s)
{
    LTL_TRY(ltl_require_init("stream_sync"));
    LTL_CUDA("cudaStreamSynchronize", cudaStreamSynchronize((cudaStream_t)s));
    return LTL_OK;
}
void* luaTL_host_alloc_pinned(uint64_t bytes)
{
    if (ltl_require_init("host_alloc_pinned") != LTL_OK) return nullptr;
    void* p = nullptr;
    const cudaError_t e = cudaHostAlloc(&p, (size_t)bytes, cudaHostAllocPortable);
    if (e != cudaSuccess) { ltl_cuda_fail("cudaHostAlloc", e); return nullptr; }
    return p;
}
void luaTL_host_free_pinned(void* p)
{
    if (!p) return;
    cudaFreeHost(p);
    cudaGetLastError();
}

// ---------------- bump arena over a pool block (cuda/luaTL_core.cu:1880-1927) ------------------------------------
// Layout read and written by the host language (ai/gpu/luaTL.lua:42-46, :345-356).
luaTL_arena_t* luaTL_arena_create(luaTL_pool_t* P, uint64_t bytes)
{
    if (ltl_require_init("arena_create") != LTL_OK) return nullptr;
    luaTL_arena_t* A = (luaTL_arena_t*)calloc(1, sizeof(luaTL_arena_t));
    if (!A) { ltl_fail(LTL_ERR_OOM, "arena_create: host allocation failed"); return nullptr; }
    if (!P) P = luaTL_default_pool();
    A->base = (char*)luaTL_tensor_alloc(P, bytes);
    if (!A->base) { free(A); return nullptr; }
    A->capacity = bytes; A->offset = 0; A->peak = 0; A->alignment = 256; A->pool = (void*)P;
    return A;
}
void luaTL_arena_destroy(luaTL_arena_t* A)
{
    if (!A) return;
    if (A->base) luaTL_tensor_free((luaTL_pool_t*)A->pool, A->base);
    free(A);
}
void* luaTL_arena_alloc(luaTL_arena_t* A, uint64_t bytes)
{
    if (!A || !A->base) { ltl_fail(LTL_ERR_NULL, "arena_alloc: null arena"); return nullptr; }
    const uint64_t al = A->alignment > 0 ? A->alignment : 256ull;
    const uint64_t off = (A->offset + al - 1ull) / al * al;
    if (off + bytes > A->capacity) {
        ltl_fail(LTL_ERR_CAPACITY, "arena_alloc: out of arena space (%llu + %llu > %llu)", (unsigned long long)off,
                 (unsigned long long)bytes, (unsigned long long)A->capacity);
        return nullptr;
    }
    A->offset = off + bytes;
    if (A->offset > A->peak) A->peak = A->offset;
    return (void*)(A->base + off);
}
void luaTL_arena_reset(luaTL_arena_t* A) { if (A) A->offset = 0; }

// ---------------- legacy raw-pointer calls (cuda/luaTL_core.cu:2147-2159) ----------------------------------------
float* luaTL_gpu_malloc(uint64_t nelem)
{
    if (nelem == 0) { ltl_fail(LTL_ERR_ARG, "gpu_malloc: zero size"); return nullptr; }
    return (float*)luaTL_tensor_alloc(nullptr, nelem * 4ull);
}
void luaTL_gpu_free(float* p) { luaTL_tensor_free(nullptr, (void*)p); }
int luaTL_to_gpu(const float* host, float* dev, uint64_t nelem)
{
    if (!host || !dev || nelem == 0) return ltl_fail(LTL_ERR_NULL, "to_gpu: null pointer or zero length");
    LTL_TRY(ltl_require_init("to_gpu"));
    LTL_CUDA("to_gpu", cudaMemcpyAsync(dev, host, (size_t)nelem * 4, cudaMemcpyHostToDevice, ltl_default_stream()));
    return ltl_sync_stream("to_gpu");
}
int luaTL_to_cpu(const float* dev, float* host, uint64_t nelem)
{
    if (!host || !dev || nelem == 0) return ltl_fail(LTL_ERR_NULL, "to_cpu: null pointer or zero length");
    LTL_TRY(ltl_require_init("to_cpu"));
    LTL_CUDA("to_cpu", cudaMemcpyAsync(host, dev, (size_t)nelem * 4, cudaMemcpyDeviceToHost, ltl_default_stream()));
    LTL_CUDA("to_cpu", cudaStreamSynchronize(ltl_default_stream()));     // the host reads the buffer on return
    return LTL_OK;
}

// ---------------- GEMM planner (cuda/luaTL_core.cu:1436-1509, :2163-2266) ---------------------------------------
// The reference picks among four CUDA-core / wmma tile shapes and can benchmark them.  This backend has one plan per
// route, fixed by shape: the planner reports it in the reference's struct (tile, block, grid, shared memory,
// kernel_id, use_tensor_core), the override is accepted and ignored, and the benchmark call times that one plan.
static int g_tile_override = -1;

static void fixed_plan(int M, int N, int K, int dtype, int allow_tc, luaTL_plan_t* p)
{
    (void)K;
    memset(p, 0, sizeof(*p));
    // luaTL_gemm / luaTL_gemm_ex take row-major [K, N] B operands with arbitrary strides: the CUDA-core kernel
    // (64 x 64 x 16 tiles, 256 threads).  The tcgen05 kernels are reached through luaTL_gemm_bf16_tc* and the model.
    p->tm = 64; p->tn = 64; p->tk = 16; p->block_x = 256; p->block_y = 1;
    p->grid_x = (N + 63) / 64; p->grid_y = (M + 63) / 64;
    p->shmem_bytes = 2 * 16 * 68 * 4 + 64 * 4;
    p->kernel_id = 0; p->unroll = 16;
    p->use_tensor_core = 0; (void)dtype; (void)allow_tc;
    p->from_cache = 0; p->measured_ms = -1.0;
}
int luaTL_plan_gemm(int M, int N, int K, int dtype, int allow_tc, luaTL_plan_t* out)
{
    if (!out) return ltl_fail(LTL_ERR_NULL, "plan_gemm: null output");
    if (M <= 0 || N <= 0 || K <= 0) return ltl_fail(LTL_ERR_SHAPE, "plan_gemm: bad shape %dx%dx%d", M, N, K);
    fixed_plan(M, N, K, dtype, allow_tc, out);
    return LTL_OK;
}
void luaTL_set_tile_override(int kernel_id) { g_tile_override = kernel_id; }
void luaTL_tune_reset(void) { g_tile_override = -1; }
int luaTL_autotune_benchmark(int M, int N, int K, int dtype, int iters, luaTL_plan_t* out)
{
    LTL_TRY(ltl_require_init("autotune_benchmark"));
    if (M <= 0 || N <= 0 || K <= 0) return ltl_fail(LTL_ERR_SHAPE, "autotune_benchmark: bad shape %dx%dx%d", M, N, K);
    if (dtype < 0 || dtype > 2) return ltl_fail(LTL_ERR_DTYPE, "autotune_benchmark: unknown dtype %d", dtype);
    if (iters <= 0) iters = 8;
    const size_t e = ltl_dtype_size(dtype);
    void* dA = luaTL_tensor_alloc(nullptr, (uint64_t)M * K * e);
    void* dB = luaTL_tensor_alloc(nullptr, (uint64_t)K * N * e);
    void* dC = luaTL_tensor_alloc(nullptr, (uint64_t)M * N * e);
    int rc = (dA && dB && dC) ? LTL_OK : LTL_ERR_OOM;
    float ms = -1.0f;
    cudaStream_t s = ltl_default_stream();
    if (rc == LTL_OK) {
        cudaMemsetAsync(dA, 0, (size_t)M * K * e, s); cudaMemsetAsync(dB, 0, (size_t)K * N * e, s);
        GemmDesc g;
        memset(&g, 0, sizeof(g));
        g.A = dA; g.B = dB; g.C = dC; g.M = M; g.N = N; g.K = K; g.batch = 1;
        g.a_rs = K; g.a_cs = 1; g.b_rs = N; g.b_cs = 1; g.c_rs = N; g.c_cs = 1; g.alpha = 1.0f;
        g.a_dtype = g.b_dtype = g.c_dtype = dtype;
        cudaEvent_t e0 = nullptr, e1 = nullptr;
        cudaEventCreate(&e0); cudaEventCreate(&e1);
        rc = ltl_gemm_simt(g, s);                                   // warm-up
        cudaEventRecord(e0, s);
        for (int i = 0; i < iters && rc == LTL_OK; ++i) rc = ltl_gemm_simt(g, s);
        cudaEventRecord(e1, s);
        if (cudaStreamSynchronize(s) != cudaSuccess && rc == LTL_OK) rc = ltl_cuda_fail("autotune_benchmark", cudaGetLastError());
        if (rc == LTL_OK && cudaEventElapsedTime(&ms, e0, e1) == cudaSuccess) ms /= (float)iters;
        cudaEventDestroy(e0); cudaEventDestroy(e1);
    }
    luaTL_tensor_free(nullptr, dA); luaTL_tensor_free(nullptr, dB); luaTL_tensor_free(nullptr, dC);
    if (rc != LTL_OK) return rc;
    if (out) { fixed_plan(M, N, K, dtype, 0, out); out->from_cache = 1; out->measured_ms = ms; }
    return LTL_OK;
}

// ---------------- small ops (cuda/luaTL_core.cu:2373-2410, cuda/luaTL_train.cu:1203-1270) ------------------------
int luaTL_bcast_add(const void* x, const void* v, void* out, int rows, int cols, float alpha, int dtype)
{
    ONE_SHOT("bcast_add", ltl_bcast_add(x, v, out, rows, cols, alpha, dtype, ltl_default_stream()));
}
int luaTL_transpose(const void* in, void* out, int rows, int cols, int dtype)
{
    ONE_SHOT("transpose", ltl_transpose(in, out, rows, cols, dtype, ltl_default_stream()));
}
int luaTL_rms_rowscale(const void* x, float* scale, int rows, int cols, float eps, int dtype)
{
    ONE_SHOT("rms_rowscale", ltl_row_rms(x, scale, rows, cols, cols, 1, eps, dtype, ltl_default_stream()));
}
int luaTL_reduce_cols(const void* x, float* out, int rows, int cols, long long row_stride, float alpha, float beta, int dtype)
{
    ONE_SHOT("reduce_cols", ltl_reduce_cols(x, out, rows, cols, row_stride > 0 ? row_stride : cols, alpha, beta, dtype,
                                            ltl_default_stream()));
}
int luaTL_gather_rows(const void* src, const void* idx, void* dst, int n, int cols, int src_rows, int dtype)
{
    ONE_SHOT("gather_rows", ltl_gather_rows(src, (const int32_t*)idx, dst, n, cols, src_rows, dtype, ltl_default_stream()));
}
int luaTL_row_rms(const void* x, float* out, int rows, int cols, long long rs, long long cs, float eps, int dtype)
{
    ONE_SHOT("row_rms", ltl_row_rms(x, out, rows, cols, rs > 0 ? rs : cols, cs > 0 ? cs : 1, eps, dtype, ltl_default_stream()));
}

// ---------------- legacy float-only wrappers (cuda/luaTL_core.cu:2289-2371) -------------------------------------
int matmul_cuda(const float* A, const float* B, float* C, int M, int N, int K)
{
    return luaTL_gemm(A, B, C, nullptr, nullptr, nullptr, M, N, K, LTL_F32, 1.0f, 0.0f, 1e-5f, 0, 0);
}
int fused_rmsnorm_matmul_cuda(const float* x, const float* gamma, const float* W, float* out, const float* bias,
                              int M, int N, int K, float eps)
{
    return luaTL_gemm(x, W, out, bias, gamma, nullptr, M, N, K, LTL_F32, 1.0f, 0.0f, eps, 1, 0);
}
int fused_gelu_matmul_cuda(const float* x, const float* W, float* out, const float* bias, int M, int N, int K)
{
    return luaTL_gemm(x, W, out, bias, nullptr, nullptr, M, N, K, LTL_F32, 1.0f, 0.0f, 1e-5f, 2, 0);
}
int fused_silu_matmul_cuda(const float* x, const float* W, float* out, const float* bias, int M, int N, int K)
{
    return luaTL_gemm(x, W, out, bias, nullptr, nullptr, M, N, K, LTL_F32, 1.0f, 0.0f, 1e-5f, 3, 0);
}
int fused_matmul_gelu_cuda(const float* A, const float* B, float* C, const float* bias, int M, int N, int K)
{
    return luaTL_gemm(A, B, C, bias, nullptr, nullptr, M, N, K, LTL_F32, 1.0f, 0.0f, 1e-5f, 0, 2);
}
int add_cuda(const float* A, const float* B, float* C, uint64_t n)
{
    return luaTL_elementwise(A, B, C, n, LTL_F32, 1, 1.0f, 1.0f);
}
int add_inplace_cuda(float* A, const float* B, uint64_t n, float alpha)
{
    return luaTL_elementwise(A, B, A, n, LTL_F32, 6, alpha, 0.0f);
}
int rmsnorm_cuda(const float* x, const float* w, float* out, int rows, int cols, float eps)
{
    return luaTL_rmsnorm(x, w, out, rows, cols, eps, LTL_F32);
}
int rmsnorm_inplace_cuda(float* x, const float* w, int rows, int cols, float eps)
{
    return luaTL_rmsnorm(x, w, x, rows, cols, eps, LTL_F32);
}
int softmax_cuda(const float* x, float* out, int rows, int cols)
{
    return luaTL_softmax(x, nullptr, out, rows, cols, 1.0f, 0, 0, LTL_F32);
}
int fused_add_bias_softmax_cuda(const float* x, const float* bias, float* out, int rows, int cols, float scale, int causal)
{
    return luaTL_softmax(x, bias, out, rows, cols, scale, causal, 0, LTL_F32);
}

// ---------------- v1 Pipeline (cuda/luaTL_core.cu:2431-2686) ----------------------------------------------------
// The narrow command buffer that predates the Program: same run / wait / timing behaviour, commands translated one
// by one to the launchers the Program interpreter uses.  Opcodes: cuda/luaTL_core.cu:92-105.
enum { V1_NOP = 0, V1_GEMM = 1, V1_EW = 2, V1_RMSNORM = 3, V1_SOFTMAX = 4, V1_CAST = 5, V1_TRANSPOSE = 6,
       V1_BCAST_ADD = 7, V1_ADAMW = 8, V1_ZERO = 9, V1_COPY = 10, V1_SYNC = 11 };

luaTL_pipeline_t* luaTL_pipeline_create(int capacity, int timing)
{
    if (ltl_require_init("pipeline_create") != LTL_OK) return nullptr;
    if (capacity <= 0) capacity = 512;
    luaTL_pipeline_t* P = (luaTL_pipeline_t*)calloc(1, sizeof(luaTL_pipeline_t));
    luaTL_cmd_t* cmds = (luaTL_cmd_t*)calloc((size_t)capacity, sizeof(luaTL_cmd_t));
    cudaStream_t s = nullptr;
    if (!P || !cmds || cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) {
        free(P); free(cmds);
        cudaGetLastError();
        ltl_fail(LTL_ERR_OOM, "pipeline_create: could not allocate %d commands and a stream", capacity);
        return nullptr;
    }
    P->cmds = cmds; P->capacity = capacity; P->stream = s; P->owns_stream = 1;
    P->timing = timing ? 1 : 0; P->flags = 1; P->last_ms = -1.0;
    if (P->timing) {
        cudaEvent_t a = nullptr, b = nullptr;
        cudaEventCreate(&a); cudaEventCreate(&b);
        P->ev_start = a; P->ev_stop = b;
    }
    return P;
}
void luaTL_pipeline_destroy(luaTL_pipeline_t* P)
{
    if (!P) return;
    if (P->stream) cudaStreamSynchronize((cudaStream_t)P->stream);
    if (P->ev_start) cudaEventDestroy((cudaEvent_t)P->ev_start);
    if (P->ev_stop) cudaEventDestroy((cudaEvent_t)P->ev_stop);
    if (P->stream && P->owns_stream) cudaStreamDestroy((cudaStream_t)P->stream);
    free(P->cmds);
    free(P);
    cudaGetLastError();
}
void luaTL_pipeline_reset(luaTL_pipeline_t* P) { if (P) { P->count = 0; P->status = LTL_OK; } }
int luaTL_pipeline_push(luaTL_pipeline_t* P, const luaTL_cmd_t* cmd)
{
    if (!P || !cmd) return ltl_fail(LTL_ERR_NULL, "pipeline_push: null pointer");
    if (P->count >= P->capacity) return ltl_fail(LTL_ERR_CAPACITY, "pipeline_push: queue full (%d)", P->capacity);
    P->cmds[P->count++] = *cmd;
    return LTL_OK;
}

static int exec_cmd(const luaTL_cmd_t* c, cudaStream_t s)
{
    switch (c->op) {
    case V1_NOP: return LTL_OK;
    case V1_GEMM: {                // contiguous row-major; i3 = pre_op, p3 bias, p4 gamma, p5 rowscale, f0 alpha, f1 beta, f2 eps
        const int M = c->i0, N = c->i1, K = c->i2;
        if (M <= 0 || N <= 0 || K <= 0) return ltl_fail(LTL_ERR_SHAPE, "gemm: bad shape %dx%dx%d", M, N, K);
        GemmDesc g = { c->p0, c->p1, c->p2, c->p3, nullptr, M, N, K, 1, K, 1, N, 1, N, 1, 0, 0, 0, c->f0, c->f1, c->act,
                       c->dtype, c->dtype, c->dtype, c->i3, c->p4, (const float*)c->p5, c->f2 };
        return ltl_gemm_simt(g, s);
    }
    case V1_EW:
        if (c->n == 0) return LTL_OK;
        return ltl_elementwise(c->p0, c->p1, c->p2, c->n, c->dtype, c->i0, c->f0, c->f1, s);
    case V1_RMSNORM:
        return ltl_rmsnorm(c->p0, c->p1, c->p2, c->i0, c->i1, c->f0, c->dtype, s);
    case V1_SOFTMAX:
        return ltl_softmax(c->p0, c->p1, c->p2, c->i0, c->i1, c->f0, c->i2, 0, c->i3, c->dtype, s);
    case V1_CAST:
        return ltl_cast(c->p0, c->i0, c->p2, c->i1, c->n, s);
    case V1_TRANSPOSE:
        return ltl_transpose(c->p0, c->p2, c->i0, c->i1, c->dtype, s);
    case V1_BCAST_ADD:
        return ltl_bcast_add(c->p0, c->p1, c->p2, c->i0, c->i1, c->f0, c->dtype, s);
    case V1_ADAMW:
        if (c->n == 0) return LTL_OK;
        return ltl_adamw((float*)c->p0, c->p1, (float*)c->p2, (float*)c->p3, c->p4, c->n, c->dtype, c->f0, c->f1, c->f2,
                         c->f3, c->f4, c->i0, c->f5, s);
    case V1_ZERO:
        if (!c->p2 || c->n == 0) return LTL_OK;
        LTL_CUDA("cudaMemsetAsync", cudaMemsetAsync(c->p2, 0, (size_t)c->n, s));
        return LTL_OK;
    case V1_COPY:
        if (!c->p0 || !c->p2 || c->n == 0) return LTL_OK;
        LTL_CUDA("cudaMemcpyAsync", cudaMemcpyAsync(c->p2, c->p0, (size_t)c->n, cudaMemcpyDeviceToDevice, s));
        return LTL_OK;
    case V1_SYNC:
        LTL_CUDA("cudaStreamSynchronize", cudaStreamSynchronize(s));
        return LTL_OK;
    default:
        return ltl_fail(LTL_ERR_ARG, "pipeline: unknown opcode %d", c->op);
    }
}

static void pipeline_timing(luaTL_pipeline_t* P)
{
    if (!P->timing || !P->ev_start || !P->ev_stop) return;
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, (cudaEvent_t)P->ev_start, (cudaEvent_t)P->ev_stop) == cudaSuccess) P->last_ms = (double)ms;
    else cudaGetLastError();
}

int luaTL_pipeline_run(luaTL_pipeline_t* P)
{
    if (!P) return ltl_fail(LTL_ERR_NULL, "pipeline_run: null pipeline");
    if (P->count <= 0) { P->status = LTL_OK; return LTL_OK; }
    if (P->count > P->capacity) {
        P->status = ltl_fail(LTL_ERR_CAPACITY, "pipeline_run: count %d exceeds capacity %d", P->count, P->capacity);
        return P->status;
    }
    cudaStream_t s = (cudaStream_t)P->stream;
    if (P->timing && P->ev_start) cudaEventRecord((cudaEvent_t)P->ev_start, s);
    for (int i = 0; i < P->count; ++i) {
        const int rc = exec_cmd(&P->cmds[i], s);
        if (rc != LTL_OK) {
            char inner[768];
            snprintf(inner, sizeof(inner), "%s", luaTL_get_last_error());
            ltl_fail(rc, "pipeline_run: command %d (op %d) failed: %s", i, P->cmds[i].op, inner);
            P->status = rc;
            cudaStreamSynchronize(s);
            cudaGetLastError();
            return rc;
        }
    }
    if (P->timing && P->ev_stop) cudaEventRecord((cudaEvent_t)P->ev_stop, s);
    if (P->flags & 1) {
        const cudaError_t e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) { P->status = ltl_cuda_fail("pipeline_run: stream sync", e); return P->status; }
        pipeline_timing(P);
    }
    P->total_runs++;
    P->total_ops += (uint64_t)P->count;
    P->status = LTL_OK;
    return LTL_OK;
}
int luaTL_pipeline_wait(luaTL_pipeline_t* P)
{
    if (!P || !P->stream) return ltl_fail(LTL_ERR_NULL, "pipeline_wait: null pipeline");
    LTL_CUDA("cudaStreamSynchronize", cudaStreamSynchronize((cudaStream_t)P->stream));
    pipeline_timing(P);
    return LTL_OK;
}

}  // extern "C"
