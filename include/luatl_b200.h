/*
 * luaTL.so for B200 (sm_100a): C ABI of the lanternl language-model token loop.
 *
 * Two groups of entry points:
 *
 *  1. The reference's own FFI surface for this path, with identical names, argument
 *     meaning, struct layouts, status codes and error-string behaviour, so that the
 *     reference's LuaJIT bindings (ai/gpu/luaTL.lua:4-168, ai/gpu/luaTL_train.lua:8-90)
 *     load this library unchanged.  Each declaration cites the reference definition it
 *     replaces (file:line inside the reference project).
 *
 *  2. New entry points (luaTL_lm_*, luaTL_sgd, luaTL_comm_*): the fused, device-resident
 *     model (training step, KV-cache prefill/decode, batched greedy generation, data-parallel
 *     gradient all-reduce).  The reference builds the same computation from Lua as a list of
 *     ops (ai/gpu/gpu_transformer.lua:309-517); these calls run it natively.
 *
 * Conventions (reference: cuda/luaTL_core.cu:108-156):
 *   - int-returning functions return 0 on success or a negative status; the message is in
 *     luaTL_get_last_error() until luaTL_clear_error().  Constructors return NULL on failure.
 *   - luaTL_init returns the device COUNT (0 = failure).
 *   - One-shot math entry points run on the library's stream and synchronise before they
 *     return; Program / lm entry points synchronise at the end of run unless told otherwise.
 *   - A GPU failure is always reported; nothing falls back to the CPU.
 *   - Single host thread per process (unsynchronised globals), as in the reference.
 */
#ifndef LUATL_B200_H
#define LUATL_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* status codes: cuda/luaTL_core.cu:108-118 */
#define LUATL_OK              0
#define LUATL_ERR_NULL       -1
#define LUATL_ERR_SHAPE      -2
#define LUATL_ERR_DTYPE      -3
#define LUATL_ERR_CUDA       -4
#define LUATL_ERR_OOM        -5
#define LUATL_ERR_ARG        -6
#define LUATL_ERR_CAPACITY   -7
#define LUATL_ERR_UNSUPPORT  -8

/* dtype tags: ai/gpu/luaTL.lua:193 */
#define LUATL_F32  0
#define LUATL_F16  1
#define LUATL_BF16 2

/* cuda/luaTL_core.cu:163-196 */
typedef struct {
    int32_t  device, major, minor, mp_count, warp_size, max_threads_per_block,
             max_threads_per_mp, max_blocks_per_mp, regs_per_block, regs_per_mp, clock_khz,
             memory_clock_khz, memory_bus_width, l2_cache_size, concurrent_kernels,
             async_engines, unified_addressing, cooperative_launch, has_tensor_cores, has_fp16,
             has_bf16, ecc_enabled, integrated, cores_per_mp;
    uint64_t shared_mem_per_block, shared_mem_per_mp, total_global_mem, free_global_mem;
    double   peak_mem_bandwidth_gbs, peak_fp32_gflops, peak_fp16_gflops;
    char     name[256];
} luaTL_devinfo_t;

/* cuda/luaTL_core.cu:214-227 */
typedef struct {
    uint64_t bytes_reserved, bytes_in_use, peak_in_use, block_count, free_block_count, n_alloc,
             n_free, n_cuda_malloc, n_cuda_free, n_cache_hit, n_cache_miss, n_trim;
} luaTL_pool_stats_t;

typedef struct luaTL_pool_s luaTL_pool_t;

/* cuda/luaTL_core.cu:199-212: what the GEMM planner reports */
typedef struct {
    int32_t tm, tn, tk, block_x, block_y, grid_x, grid_y;
    int32_t shmem_bytes, kernel_id, unroll, use_tensor_core, from_cache;
    double  measured_ms;
} luaTL_plan_t;

/* cuda/luaTL_core.cu:251-257: bump arena over one pool block; the host bumps offset / peak itself
 * (ai/gpu/luaTL.lua:345-356) */
typedef struct {
    char*    base;
    uint64_t capacity, offset, peak, alignment;
    void*    pool;
} luaTL_arena_t;

/* cuda/luaTL_core.cu:259-277: command and queue of the v1 Pipeline (ai/gpu/luaTL.lua:48-63, :797-819) */
typedef struct {
    int32_t  op, dtype, act, flags;
    int32_t  i0, i1, i2, i3;
    float    f0, f1, f2, f3, f4, f5;
    uint64_t n;
    void    *p0, *p1, *p2, *p3, *p4, *p5;
} luaTL_cmd_t;
typedef struct {
    luaTL_cmd_t* cmds;
    int32_t      count, capacity, flags, status;
    void        *stream, *ev_start, *ev_stop;
    double       last_ms;
    uint64_t     total_runs, total_ops;
    int32_t      owns_stream, timing;
} luaTL_pipeline_t;

/* cuda/luaTL_core.cu:238-249 (56 bytes; Lua reads and writes the fields directly) */
typedef struct {
    void*    data;
    uint64_t nelem;
    uint64_t nbytes;
    int32_t  rows, cols, dtype, owns;
    void*    pool;
    int32_t  device, flags;
} luaTL_tensor_t;

/* cuda/luaTL_train.cu:94-101 (224 bytes; Lua fills every field, ai/gpu/luaTL_train.lua:344-363) */
typedef struct {
    int32_t  op, dtype, act, pre;
    int32_t  i0, i1, i2, i3, i4, i5, i6, i7;
    float    f0, f1, f2, f3, f4, f5, f6, f7;
    int64_t  s0, s1, s2, s3, s4, s5, s6, s7, s8;
    uint64_t n;
    void    *p0, *p1, *p2, *p3, *p4, *p5, *p6, *p7;
} luaTL_op_t;

/* cuda/luaTL_train.cu:103-110 */
typedef struct {
    luaTL_op_t* ops;
    int32_t     count, capacity, flags, status;
    void       *stream, *ev_start, *ev_stop, *graph, *graph_exec;
    double      last_ms;
    uint64_t    total_runs, total_ops;
    int32_t     owns_stream, timing, captured, capturing;
} luaTL_prog_t;

/* Program opcodes: cuda/luaTL_train.cu:57-86.  LUATL_P_SGD is new (the reference's GPU path
 * has AdamW only; SGD follows ai/optim/optim2.lua:93-99). */
enum {
    LUATL_P_NOP = 0, LUATL_P_GEMM = 1, LUATL_P_EW = 2, LUATL_P_RMSNORM = 3, LUATL_P_RMSNORM_BWD = 4,
    LUATL_P_SOFTMAX = 5, LUATL_P_SOFTMAX_BWD = 6, LUATL_P_SWIGLU = 7, LUATL_P_SWIGLU_BWD = 8,
    LUATL_P_ROPE = 9, LUATL_P_EMBED = 10, LUATL_P_EMBED_BWD = 11, LUATL_P_CE = 12,
    LUATL_P_REDUCE_COLS = 13, LUATL_P_L2 = 14, LUATL_P_CLIP = 15, LUATL_P_ADAMW = 16,
    LUATL_P_ZERO = 17, LUATL_P_COPY = 18, LUATL_P_CAST = 19, LUATL_P_TRANSPOSE = 20,
    LUATL_P_BCAST_ADD = 21, LUATL_P_SYNC = 22, LUATL_P_ARGMAX = 23, LUATL_P_SUM = 24,
    LUATL_P_GATHER = 25, LUATL_P_ROWRMS = 26, LUATL_P_SGD = 27
};

/* ---------------- runtime (cuda/luaTL_core.cu:1674-1770, cuda/luaTL_train.cu:36-53,1305) --- */
const char* luaTL_version(void);                         /* core.cu:1674 */
const char* luaTL_train_version(void);                   /* train.cu:1073 */
void        luaTL_set_verbose(int on);                   /* core.cu:1676 */
int         luaTL_init(int device);                      /* core.cu:1678 */
void        luaTL_shutdown(void);                        /* core.cu:1717 */
void        luaTL_shutdown_safe(void);                   /* train.cu:39 */
void        luaTL_finalize(void);                        /* train.cu:1305 */
uint64_t    luaTL_epoch(void);                           /* train.cu:37 */
const char* luaTL_device_name(void);                     /* core.cu:1738 */
const char* luaTL_get_last_error(void);                  /* core.cu:1739 */
int         luaTL_has_error(void);                       /* core.cu:1740 */
void        luaTL_clear_error(void);                     /* core.cu:1742 */
int         luaTL_sync(void);                            /* core.cu:1749 */
int         luaTL_get_devinfo(int device, luaTL_devinfo_t* out);     /* core.cu:1755 */
int         luaTL_mem_info(uint64_t* freeb, uint64_t* totalb);       /* core.cu:1765 */

/* ---------------- streams and page-locked host memory (cuda/luaTL_core.cu:1776-1813) ------ */
void* luaTL_stream_create(int nonblocking);              /* core.cu:1776 */
void  luaTL_stream_destroy(void* s);                     /* core.cu:1786 */
int   luaTL_stream_sync(void* s);                        /* core.cu:1793 */
void* luaTL_host_alloc_pinned(uint64_t bytes);           /* core.cu:1801 */
void  luaTL_host_free_pinned(void* p);                   /* core.cu:1809 */

/* ---------------- pool and tensors (cuda/luaTL_core.cu:585-886,1818-2159) ---------------- */
luaTL_pool_t* luaTL_pool_create(int device);             /* core.cu:1818; device < 0: the bound device */
void          luaTL_pool_destroy(luaTL_pool_t* P);       /* core.cu:1826; the default pool is left alone */
luaTL_arena_t* luaTL_arena_create(luaTL_pool_t* P, uint64_t bytes);   /* core.cu:1880 */
void           luaTL_arena_destroy(luaTL_arena_t* A);                 /* core.cu:1901 */
void*          luaTL_arena_alloc(luaTL_arena_t* A, uint64_t bytes);   /* core.cu:1908: 256-byte aligned bump */
void           luaTL_arena_reset(luaTL_arena_t* A);                   /* core.cu:1924 */
/* legacy raw-pointer calls, cuda/luaTL_core.cu:2147-2153 */
float* luaTL_gpu_malloc(uint64_t nelem);
void   luaTL_gpu_free(float* p);
int    luaTL_to_gpu(const float* host, float* dev, uint64_t nelem);
int    luaTL_to_cpu(const float* dev, float* host, uint64_t nelem);
luaTL_pool_t* luaTL_default_pool(void);
void*         luaTL_tensor_alloc(luaTL_pool_t* P, uint64_t bytes);
void          luaTL_tensor_free(luaTL_pool_t* P, void* ptr);
void          luaTL_pool_trim(luaTL_pool_t* P);
int           luaTL_pool_get_stats(luaTL_pool_t* P, luaTL_pool_stats_t* out);
int           luaTL_pool_owns(luaTL_pool_t* P, void* ptr);
int  luaTL_tensor_init(luaTL_tensor_t* t, int rows, int cols, int dtype, luaTL_pool_t* P);
int  luaTL_tensor_wrap(luaTL_tensor_t* t, void* data, int rows, int cols, int dtype);
void luaTL_tensor_release(luaTL_tensor_t* t);
void luaTL_tensor_release_safe(luaTL_tensor_t* t);       /* train.cu:47 */
int  luaTL_tensor_view(luaTL_tensor_t* dst, const luaTL_tensor_t* src, int row_off, int rows, int cols);
int  luaTL_tensor_zero(luaTL_tensor_t* t);
int  luaTL_tensor_upload(luaTL_tensor_t* t, const float* host, uint64_t nelem);
int  luaTL_tensor_download(const luaTL_tensor_t* t, float* host, uint64_t nelem);
int  luaTL_tensor_copy(const luaTL_tensor_t* src, luaTL_tensor_t* dst);
int  luaTL_tensor_cast(const luaTL_tensor_t* src, luaTL_tensor_t* dst);
int  luaTL_gpu_copy(const float* src, float* dst, uint64_t nelem);
int  luaTL_gpu_zero(float* p, uint64_t nelem);
int  luaTL_upload_i32(void* dev, const int32_t* host, uint64_t n);       /* train.cu:1274 */
int  luaTL_download_i32(const void* dev, int32_t* host, uint64_t n);     /* train.cu:1282 */
int  luaTL_download_f32(const void* dev, float* host, uint64_t n);       /* train.cu:1290 */

/* ---------------- one-shot math on the path (synchronous) ------------------------------- */
/* cuda/luaTL_train.cu:1075: C = post(alpha * pre(A) B + bias) + beta * C with explicit strides.
 * pre_op (cuda/luaTL_core.cu:84-90): 0 none; 1 RMSNorm prologue - A(m,k) * rowscale[m] * gamma[k], rowscale computed
 * from A with eps when NULL (cuda/luaTL_train.cu:159-204); 2 gelu, 3 silu, 4 relu on A. */
int luaTL_gemm_ex(const void* A, const void* B, void* C, const void* bias, const void* gamma,
                  const float* rowscale, int M, int N, int K, int dtype,
                  long long a_rs, long long a_cs, long long b_rs, long long b_cs,
                  long long c_rs, long long c_cs, long long a_bs, long long b_bs, long long c_bs,
                  int batch, float alpha, float beta, float eps, int pre_op, int post_op);
/* cuda/luaTL_core.cu:2272 (contiguous row-major form of the above) */
int luaTL_gemm(const void* A, const void* B, void* C, const void* bias, const void* gamma,
               const float* rowscale, int M, int N, int K, int dtype, float alpha, float beta,
               float eps, int pre_op, int post_op);
int luaTL_rmsnorm(const void* x, const void* w, void* out, int rows, int cols, float eps, int dtype);     /* core.cu:2329 */
int luaTL_rmsnorm_bwd(const void* x, const void* gamma, const void* dy, void* dx, float* dgamma,
                      int rows, int cols, float eps, int dtype);                                          /* train.cu:1096 */
/* No counterpart in the reference.  Same result as luaTL_rmsnorm_bwd, but allocates nothing: the
 * per-warp dgamma partials go to a fixed 4.6 MB array inside the library's device image instead of
 * a cudaMalloc'ed workspace.  For callers that cannot allocate when they need a gradient (all device
 * memory already handed to their own arena, loops that cannot take cudaMalloc's device
 * synchronisation).  Limits: with dgamma, rows of at most 1024 columns on a
 * 148-SM GPU (LUATL_ERR_CAPACITY beyond); every call shares the array, so calls that overlap on the
 * GPU race; the first call on a device looks the array's address up and should come before any
 * stream capture. */
int luaTL_rmsnorm_bwd_noalloc(const void* x, const void* gamma, const void* dy, void* dx, float* dgamma,
                              int rows, int cols, float eps, int dtype);
int luaTL_softmax(const void* x, const void* bias, void* out, int rows, int cols, float scale,
                  int causal, int mask_offset, int dtype);                                                /* core.cu:2351 */
int luaTL_softmax_ex(const void* x, const void* bias, void* out, int rows, int cols, float scale,
                     int causal, int group, int mask_offset, int dtype);                                  /* train.cu:1108 */
int luaTL_softmax_bwd(const void* y, const void* dy, void* dx, int rows, int cols, float scale,
                      int causal, int group, int mask_offset, int dtype);                                 /* train.cu:1120 */
int luaTL_swiglu_fwd(const void* a, const void* b, void* out, int rows, int cols, int lda, int ldb,
                     int ldo, int dtype);                                                                 /* train.cu:1131 */
int luaTL_swiglu_bwd(const void* a, const void* b, const void* dout, void* da, void* db, int rows,
                     int cols, int lda, int ldb, int ldo, int dtype);                                     /* train.cu:1142 */
int luaTL_rope(void* x, const void* pos_ids, int rows, int heads, int head_dim, int row_stride,
               int pos_offset, float theta, int interleaved, int inverse, int dtype);                     /* train.cu:1154 */
int luaTL_embed_fwd(const void* ids, const void* table, void* out, int rows, int dim, int vocab, int dtype);   /* train.cu:1169 */
int luaTL_embed_bwd(const void* ids, const void* dout, float* dtable, int rows, int dim, int vocab,
                    float scale, int dtype);                                                              /* train.cu:1179 */
int luaTL_cross_entropy(const void* logits, const void* targets, float* losses, void* dlogits,
                        int rows, int vocab, int ignore_index, float grad_scale, int dtype);              /* train.cu:1189 */
int luaTL_l2_accum(const void* x, uint64_t n, float* out, int dtype);                                     /* train.cu:1215 */
int luaTL_clip_by_nsq(void* x, uint64_t n, const float* nsq, float max_norm, int dtype);                  /* train.cu:1223 */
int luaTL_sum_f32(const float* x, uint64_t n, float* out, float scale);                                   /* train.cu:1233 */
int luaTL_argmax_rows(const void* x, void* out_i32, int rows, int cols, int dtype);                       /* train.cu:1241 */
int luaTL_elementwise(const void* A, const void* B, void* C, uint64_t n, int dtype, int op,
                      float alpha, float beta);                                                           /* core.cu:2308 */
int luaTL_adamw(float* w, const void* g, float* m, float* v, void* w_lp, uint64_t n, int grad_dtype,
                float lr, float beta1, float beta2, float eps, float wd, int step, float clip);           /* core.cu:2412 */
/* cuda/luaTL_core.cu:2373-2410, cuda/luaTL_train.cu:1203-1270: small ops the model itself does not queue */
int luaTL_bcast_add(const void* x, const void* v, void* out, int rows, int cols, float alpha, int dtype);   /* out = x + alpha * v[c] */
int luaTL_transpose(const void* in, void* out, int rows, int cols, int dtype);
int luaTL_rms_rowscale(const void* x, float* scale, int rows, int cols, float eps, int dtype);             /* 1/sqrt(mean x^2 + eps) */
int luaTL_reduce_cols(const void* x, float* out, int rows, int cols, long long row_stride, float alpha,
                      float beta, int dtype);                                                             /* train.cu:1203 */
int luaTL_gather_rows(const void* src, const void* idx, void* dst, int n, int cols, int src_rows, int dtype);  /* train.cu:1251 */
int luaTL_row_rms(const void* x, float* out, int rows, int cols, long long rs, long long cs, float eps, int dtype); /* train.cu:1261 */
/* GEMM planner, cuda/luaTL_core.cu:2163-2266.  One fixed plan per shape here: plan_gemm reports it, the override is
 * accepted and has no effect, autotune_benchmark times that plan. */
int  luaTL_plan_gemm(int M, int N, int K, int dtype, int allow_tc, luaTL_plan_t* out);
void luaTL_set_tile_override(int kernel_id);
void luaTL_tune_reset(void);
int  luaTL_autotune_benchmark(int M, int N, int K, int dtype, int iters, luaTL_plan_t* out);
/* legacy float-only wrappers, cuda/luaTL_core.cu:2289-2371 */
int matmul_cuda(const float* A, const float* B, float* C, int M, int N, int K);
int fused_rmsnorm_matmul_cuda(const float* x, const float* gamma, const float* W, float* out, const float* bias,
                              int M, int N, int K, float eps);
int fused_gelu_matmul_cuda(const float* x, const float* W, float* out, const float* bias, int M, int N, int K);
int fused_silu_matmul_cuda(const float* x, const float* W, float* out, const float* bias, int M, int N, int K);
int fused_matmul_gelu_cuda(const float* A, const float* B, float* C, const float* bias, int M, int N, int K);
int add_cuda(const float* A, const float* B, float* C, uint64_t n);
int add_inplace_cuda(float* A, const float* B, uint64_t n, float alpha);
int rmsnorm_cuda(const float* x, const float* w, float* out, int rows, int cols, float eps);
int rmsnorm_inplace_cuda(float* x, const float* w, int rows, int cols, float eps);
int softmax_cuda(const float* x, float* out, int rows, int cols);
int fused_add_bias_softmax_cuda(const float* x, const float* bias, float* out, int rows, int cols, float scale, int causal);
/* New: w -= lr * (f * g + wd * w) with f = min(1, max_norm / (sqrt(*nsq) + 1e-6)) when nsq != NULL
 * and max_norm > 0 (rule: ai/optim/optim2.lua:93-99; clip factor: cuda/luaTL_train.cu:950-952). */
int luaTL_sgd(float* w, const float* g, uint64_t n, float lr, float wd, const float* nsq, float max_norm);

/* New: tensor-core GEMM (tcgen05 + TMA).  C[M,N] = A[M,K] * B[N,K]^T + R with bf16 A and B (both
 * K contiguous), fp32 accumulation, C and R of c_dtype (LUATL_F32 or LUATL_BF16), R optional.
 * K must be a multiple of 8 and the operands 16-byte aligned.  tile_n bits 0-15: tile width, 0 = choose,
 * else 32/64/128.  tile_n bit 16: SwiGLU epilogue - the rows of B alternate gate_j / up_j, both are rounded to
 * bf16 and C [M, N/2] (bf16) = silu(gate) * up.  tile_n bit 17: accumulating epilogue - C (fp32) += A B^T with
 * atomic adds (R must be NULL).  tile_n bits 20-27: split-K slice count (0/1 = none); without bit 17 C then
 * receives the slices' partial products [slices][M][N].
 * The reference has no tensor-core path for bf16 (its only one is fp16 wmma, cuda/luaTL_core.cu:1296). */
int luaTL_gemm_bf16_tc(const void* A, const void* B, void* C, const void* R, int M, int N, int K,
                       int c_dtype, int tile_n);
/* New: the same product on fp32 operands read by the tensor cores as TF32: C[M,N] = A[M,K] B[N,K]^T + R (accumulate = 0;
 * R optional) or C += A B^T (accumulate = 1; ksplit slices of K added with atomics, 0 = choose).  K a multiple of 4,
 * operands 16-byte aligned.  Replaces the CUDA-core kernels behind luaTL_gemm_ex (cuda/luaTL_train.cu:127,242) where a
 * 2e-3 tolerance is accepted. */
int luaTL_gemm_tf32_tc(const float* A, const float* B, float* C, const float* R, int M, int N, int K, int accumulate, int ksplit);
/* New: fused causal attention over a packed qkv [B*T, 3*H*head_dim] (q | k | v in every row): out [B*T, H*head_dim],
 * lse [B*H*T] (natural log of the softmax denominator, may be NULL).  The reference composes attention from
 * batched score GEMMs, a [B*H*T, T] softmax and a second GEMM (ai/gpu/gpu_transformer.lua:333-352); it has no fused
 * counterpart.  impl: 0 = choose, 1 = CUDA-core kernel (f32 / bf16, head_dim 16..128), 2 = tcgen05 kernel (bf16,
 * head_dim 64 or 128, T a multiple of 8). */
int luaTL_attention_fwd(const void* qkv, void* out, float* lse, int B, int T, int H, int hd, float scale, int causal,
                        int dtype, int impl);
/* New: backward of luaTL_attention_fwd.  dqkv [B*T, 3*H*head_dim] (dq | dk | dv per row, before the inverse RoPE)
 * from out and dout [B*T, H*head_dim] and the lse the forward wrote.  Same impl values. */
int luaTL_attention_bwd(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv, int B, int T,
                        int H, int hd, float scale, int causal, int dtype, int impl);
/* New: C[M,N] (fp32) += X^T Y with X [K, M] and Y [K, N] bf16 row-major: the weight-gradient product of two
 * token-major matrices (both tensor-core operands MN-major, nothing is transposed in memory).  M, N multiples
 * of 8.  ksplit: slices of K added with atomics (0/1 = one). */
int luaTL_gemm_bf16_tc_xty(const void* X, const void* Y, float* C, int M, int N, int K, int ksplit);
/* New: few-row GEMM of the decode step (mma.sync, weights read straight into fragments): C = A[M,K] B[N,K]^T for
 * 1 <= M <= 64 and K a multiple of 32, bf16 operands, fp32 accumulate.  c_dtype 0 (f32) or 2 (bf16); epilogue 1 =
 * SwiGLU over interleaved (gate, up) rows of B, C [M, N/2] bf16; ksplit > 1: C receives ksplit fp32 partial
 * matrices [ksplit][M][N].  The product of the reference's matmul op (cuda/luaTL_core.cu:1506) on a transposed weight. */
int luaTL_gemm_bf16_rows(const void* A, const void* B, void* C, int M, int N, int K, int c_dtype, int epilogue, int ksplit);
/* New: the two fused forms of the decode-step GEMMs (impl 0 = tcgen05 tiles, 1 = the few-row kernel).  The reference
 * runs matmul, add and rmsnorm as three ops (ai/gpu/gpu_transformer.lua:354-372); these have no counterpart there.
 *  resid: split-K product A[M,K] B[N,K]^T into `slices` [ksplit][M][N]; the CTA that finishes an output tile last adds
 *    the slices in slice order and the residual, x[M,N] += product, and writes h = bf16(x * gain) and, per row, the
 *    sum of x^2 over each 32-column tile to ssq [M][N/32].  N a multiple of 32.
 *  rowscale: C = diag(s) A B^T with s_r = 1 / sqrt(sum_t ssq[r][t] / K + eps): the RMSNorm factor of the activation
 *    that produced A (A holds x * gain), applied in the epilogue; epilogue / c_dtype as in luaTL_gemm_bf16_rows. */
int luaTL_gemm_bf16_resid(const void* A, const void* B, float* slices, float* x, const float* gain, void* h, float* ssq,
                          int M, int N, int K, int ksplit, int impl);
int luaTL_gemm_bf16_rowscale(const void* A, const void* B, void* C, const float* ssq, int ssq_tiles, float eps, int M, int N,
                             int K, int c_dtype, int epilogue, int impl);
/* New: device-side timing of immediate ops.  luaTL_set_deferred(1) makes the immediate entry points return
 * without waiting for the stream (errors of queued kernels then surface at the next luaTL_sync / luaTL_timer_stop);
 * luaTL_timer_start / luaTL_timer_stop bracket a stretch of the library stream with CUDA events and return the
 * elapsed milliseconds.  The reference times from the host (ai/gpu/luaTL.lua); it has no counterpart. */
void luaTL_set_deferred(int on);
int  luaTL_timer_start(void);
int  luaTL_timer_stop(float* ms);
/* New: RMSNorm backward fused with the residual add of the backward pass: res += d(rmsnorm)/dx (fp32, in place),
 * res_bf16 (optional) = bf16 copy of the updated res, dgamma (optional) += the gain gradient.  fp32 x / dy, cols a
 * multiple of 4, at most 4096.  Equals luaTL_rmsnorm_bwd followed by an add and a cast. */
int luaTL_rmsnorm_bwd_residual(const float* x, const float* gamma, const float* dy, float* res, void* res_bf16, float* dgamma,
                               int rows, int cols, float eps);
/* New: sampling beyond greedy on the device, the rule of pick_token (ai/optim/lmtrain.lua:1364-1436): temperature
 * <= 0 is the argmax; top_k in 1..vocab-1 keeps the k largest logits (descending, ties by lower index); top_p in (0, 1)
 * cuts the nucleus inside that set, or inside the whole row sorted descending when no top_k is given; top_k = 0 without
 * top_p walks the whole row in index order.  The uniform draw is a 24-bit counter-based hash of (seed, row, counter),
 * so results are reproducible.
 * luaTL_sample_rows: one index per row of fp32 logits [rows, vocab], counters[r] = position of row r (NULL: 0).
 * luaTL_lm_set_sampling: the same rule inside luaTL_lm_generate*, counter = the sequence's position; stop_id >= 0:
 * a sequence that emitted it keeps emitting it (stop_id = -1: none).  The reference samples on the host from
 * downloaded logits with math.random. */
int luaTL_sample_rows(const float* logits, int rows, int vocab, float temperature, int top_k, float top_p, uint64_t seed,
                      const int32_t* counters, int32_t* out);
/* New: the same GEMM launched `iters` times back to back on the library stream and timed with CUDA events
 * (ms per launch), for roofline measurements without host gaps.  No residual operand. */
int luaTL_gemm_bf16_tc_time(const void* A, const void* B, void* C, int M, int N, int K, int c_dtype, int tile_n,
                            int iters, float* ms_per_launch);

/* ---------------- Program: command buffer + CUDA graph (cuda/luaTL_train.cu:1506-1712) ---- */
luaTL_prog_t* luaTL_prog_create(int capacity, int timing);
void          luaTL_prog_destroy(luaTL_prog_t* P);
void          luaTL_prog_reset(luaTL_prog_t* P);
int           luaTL_prog_push(luaTL_prog_t* P, const luaTL_op_t* op);
int           luaTL_prog_run(luaTL_prog_t* P);
int           luaTL_prog_capture(luaTL_prog_t* P);
int           luaTL_prog_replay(luaTL_prog_t* P);
int           luaTL_prog_wait(luaTL_prog_t* P);
void          luaTL_prog_graph_free(luaTL_prog_t* P);

/* ---------------- v1 Pipeline (cuda/luaTL_core.cu:2431-2686) ---------------------------------- */
luaTL_pipeline_t* luaTL_pipeline_create(int capacity, int timing);
void              luaTL_pipeline_destroy(luaTL_pipeline_t* P);
void              luaTL_pipeline_reset(luaTL_pipeline_t* P);
int               luaTL_pipeline_push(luaTL_pipeline_t* P, const luaTL_cmd_t* cmd);
int               luaTL_pipeline_run(luaTL_pipeline_t* P);
int               luaTL_pipeline_wait(luaTL_pipeline_t* P);

/* ---------------- fused device-resident model (new) ------------------------------------- */
typedef struct {
    int32_t vocab, dim, layers, heads, ffn;
    int32_t max_seq;           /* T: training window and KV-cache length                      */
    int32_t batch;             /* B: sequences per training / eval step                        */
    int32_t decode_batch;      /* sequences held by the KV cache (0 = no cache)                */
    int32_t tie;               /* 1: lm_head shares tok_emb                                    */
    int32_t dtype;             /* LUATL_F32: fp32 weights and math; LUATL_BF16: bf16 weights   */
                               /* and GEMM inputs, fp32 accumulation and residual stream       */
    int32_t use_rope, rope_interleaved, causal;
    int32_t kv_splits;         /* split-KV factor of decode attention, 0 = choose              */
    float   eps, rope_base;
} luaTL_lm_config_t;

typedef struct {
    float   loss;              /* mean CE over the valid targets of all ranks                  */
    float   grad_norm;         /* global L2 norm of the gradient (0 if not computed)           */
    int32_t correct, valid, finite;
    float   step_ms;           /* device time of the step                                      */
} luaTL_lm_result_t;

typedef struct luaTL_lm_s luaTL_lm_t;

luaTL_lm_t* luaTL_lm_create(const luaTL_lm_config_t* cfg);
void        luaTL_lm_destroy(luaTL_lm_t* m);
/* Parameters live in one flat fp32 buffer in the reference's GPU order
 * tok_emb, {ln1, wqkv, wo, ln2, w13, w2} x L, lnf [, head]  (ai/gpu/gpu_transformer.lua:224-239). */
int64_t luaTL_lm_nparams(const luaTL_lm_t* m);
int     luaTL_lm_ntensors(const luaTL_lm_t* m);
int     luaTL_lm_tensor_info(const luaTL_lm_t* m, int i, char* name32, int32_t* rows, int32_t* cols,
                             int64_t* offset, int32_t* decay);
int luaTL_lm_write_params(luaTL_lm_t* m, int64_t offset, int64_t count, const float* host);
int luaTL_lm_read_params(luaTL_lm_t* m, int64_t offset, int64_t count, float* host);
int luaTL_lm_read_grads(luaTL_lm_t* m, int64_t offset, int64_t count, float* host);
float* luaTL_lm_params_device(luaTL_lm_t* m);
float* luaTL_lm_grads_device(luaTL_lm_t* m);

/* One optimizer step on host id/target blocks [batch, max_seq] (pad: id 0, target -1).
 * optimizer: 0 = SGD, 1 = AdamW.  valid_global <= 0: count the valid targets of this block.
 * dtype f32: exact fp32 arithmetic (CUDA-core GEMMs).  dtype bf16: mixed precision - fp32 master
 * weights, gradients and residual stream, bf16 activations, every contraction on the tensor cores with
 * fp32 accumulation; needs dim, ffn and vocab to be multiples of 8.  The first training
 * call of a bf16 model switches it to the training weight layout (captured decode graphs are dropped). */
typedef struct {
    int32_t optimizer, step;
    float   lr, weight_decay, clip_norm, beta1, beta2, adam_eps;
    int32_t valid_global;      /* denominator of loss and gradient across all ranks            */
    int32_t no_update;         /* 1: forward + backward only (gradients stay readable)         */
    int32_t accumulate;        /* 1: add to the gradients and loss already in the buffer (micro-batches of one
                                *    optimizer step: first call 0, later calls 1, no_update = 1 on all but the last) */
    int32_t skip_allreduce;    /* 1: leave the gradients rank-local (set on all but the last micro-batch)  */
} luaTL_lm_train_args_t;
int luaTL_lm_train_step(luaTL_lm_t* m, const int32_t* ids, const int32_t* targets,
                        const luaTL_lm_train_args_t* a, luaTL_lm_result_t* out);
/* Same with ids/targets already on the device. */
int luaTL_lm_train_step_dev(luaTL_lm_t* m, const int32_t* d_ids, const int32_t* d_targets,
                            const luaTL_lm_train_args_t* a, luaTL_lm_result_t* out);
/* The captured training step (ai/gpu/gpu_transformer.lua:714-733 capture / maybe_capture, :643 replay rule): with
 * on = 1, the forward + loss + backward of luaTL_lm_train_step* is captured as one CUDA graph on the third step and
 * replayed on every later step whose valid-target count, accumulate flag and id / target buffers are those of the
 * capture (otherwise it is captured again); the optimizer launches stay outside, their scalars change per step.
 * Steps whose gradient exchange overlaps the backward (bf16 model, more than one rank) are not captured.
 * luaTL_lm_graph_ready: 1 while a captured step exists. */
int luaTL_lm_set_graph(luaTL_lm_t* m, int on);
int luaTL_lm_graph_ready(const luaTL_lm_t* m);
/* fp32 models: on = 1 runs every weight product of the forward, the backward and the decode step on the tensor cores
 * (tcgen05 kind::tf32: fp32 operands read with a 10-bit mantissa, fp32 accumulation), results within 2e-3 of the exact
 * path; on = 0 (the default) keeps the exact CUDA-core products (1e-4).  The reference's dominant kernel for these
 * products is its register-tiled CUDA-core GEMM (cuda/luaTL_train.cu:242, chosen at :425). */
int luaTL_lm_set_tf32(luaTL_lm_t* m, int on);
/* Forward only: loss / accuracy, optionally the logits [rows_out, vocab] to the host
 * (last_only = 1: only row n_tokens - 1 of sequence 0, what generate reads). */
int luaTL_lm_eval_step(luaTL_lm_t* m, const int32_t* ids, const int32_t* targets, luaTL_lm_result_t* out);
int luaTL_lm_forward(luaTL_lm_t* m, const int32_t* ids, int nseq, int ntok, float* logits_host, int last_only);

/* KV-cache generation.  Sequences are independent; slot b uses cache slot b. */
int luaTL_lm_state_reset(luaTL_lm_t* m);             /* every slot back to length 0 */
int luaTL_lm_slot_reset(luaTL_lm_t* m, int slot);    /* one slot: what Transformer:new_state() gives */
/* Mirrors Transformer:step (ai/nn/transformer.lua:297): feed one token to sequence slot
 * `slot`, append its K/V, return the logits row [vocab] on the host. */
int luaTL_lm_step(luaTL_lm_t* m, int slot, int32_t id, float* logits_host);
int luaTL_lm_state_len(luaTL_lm_t* m, int slot);
/* Batched greedy generation: prompts [nseq, n_prompt] on the host, out [nseq, n_new]. */
int luaTL_lm_generate(luaTL_lm_t* m, const int32_t* prompts, int nseq, int n_prompt, int n_new,
                      int32_t* out, luaTL_lm_result_t* timing);
/* Same with prompts and out on the device (nothing crosses PCIe). */
int luaTL_lm_generate_dev(luaTL_lm_t* m, const int32_t* d_prompts, int nseq, int n_prompt, int n_new,
                          int32_t* d_out, luaTL_lm_result_t* timing);
/* Measurement aid: average device time (CUDA events on the library stream, 3 warm-up rounds) of one
 * decode-attention launch with every sequence at `cache_len` cached positions; one round = one
 * launch per layer, each over its own layer of the cache (inputs larger than L2).  Leaves the
 * generation state reset. */
int luaTL_lm_time_decode_attn(luaTL_lm_t* m, int nseq, int cache_len, int iters, float* ms_per_launch);
/* Measurement aid: microseconds per launch of each kind of launch of the decode step (bf16 tensor-core path), measured
 * as 60 copies back to back in a captured chain, `reps` replays after 3 warm-up replays, every sequence at `cache_len`:
 *   us[0] embed + RMSNorm, [1] QKV, [2] Wo (split-K), [3] reduce + RMSNorm, [4] W13 + SwiGLU, [5] W2 (split-K),
 *   [6] reduce + RMSNorm with the prefetch rider, [7] lm_head, [8] pick, [9] one layer's chain Wo .. next QKV (six
 *   launches, total).  n >= 10.  Attention is timed by luaTL_lm_time_decode_attn.  Leaves the generation state reset.
 * New entry point: no counterpart in the reference. */
int luaTL_lm_time_decode_launches(luaTL_lm_t* m, int nseq, int cache_len, int reps, float* us, int n);
/* Sampling rule of luaTL_lm_generate* (see luaTL_sample_rows); temperature <= 0 restores the greedy pick. */
int luaTL_lm_set_sampling(luaTL_lm_t* m, float temperature, int top_k, float top_p, uint64_t seed, int stop_id);
/* Device time (ms) and kernel launches of the last prefill and decode phases. */
int luaTL_lm_last_timing(luaTL_lm_t* m, float* prefill_ms, float* decode_ms, int64_t* launches);

/* ---------------- data-parallel gradient exchange (new; NCCL over NVLink) ---------------- */
int luaTL_comm_unique_id(char* id128);                   /* rank 0 creates, caller broadcasts */
int luaTL_comm_init(const char* id128, int world, int rank);
int luaTL_comm_world(void);
int luaTL_comm_allreduce_f32(float* dev, uint64_t n);
void luaTL_comm_destroy(void);
/* Failure handling of the exchange.  No entry point blocks on a collective without a limit: the host polls the stream
 * and the communicator's asynchronous error state; on an error, or when `ms` milliseconds pass (default 120000, or
 * LUATL_COMM_TIMEOUT_MS), the communicator is aborted and the call returns LUATL_ERR_CUDA ("... did not finish within
 * ... ms (a rank did not arrive?)").  After that luaTL_comm_world() is 1 until luaTL_comm_init is called again. */
void luaTL_comm_set_timeout(int ms);
/* The same wait loop run against fakes, usable without a GPU: the fake collective finishes when the file `arrive_path`
 * exists (NULL: never), the fake communicator reports `async_error` from the `error_after`-th poll on (0: never).
 * *aborted receives 1 when the loop tore the communicator down.  Neither has a counterpart in the reference, which has
 * no collective. */
int luaTL_comm_selftest_wait(const char* arrive_path, int timeout_ms, int async_error, int error_after, int* aborted);

#ifdef __cplusplus
}
#endif
#endif
