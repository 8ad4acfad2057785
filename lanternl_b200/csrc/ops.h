// Internal launchers shared by the C ABI, the Program interpreter and the LM runtime.
// Every function enqueues on `s` and returns a status; none of them synchronises.
#pragma once
#include "common.cuh"

// ---- bandwidth-bound row / element kernels (ops.cu) ----
int ltl_rmsnorm(const void* x, const void* w, void* out, int rows, int cols, float eps,
                int dtype, cudaStream_t s);
// `scratch` holds rmsnorm_bwd_scratch_floats(cols) floats (per-CTA dgamma partials).
size_t ltl_rmsnorm_bwd_scratch_floats(int cols);
int ltl_rmsnorm_bwd_residual(const float* x, const float* gamma, const float* dy, float* res, bf16* res_bf16, float* dgamma,
                             int rows, int cols, float eps, float* scratch, cudaStream_t s);
int ltl_rmsnorm_bwd(const void* x, const void* gamma, const void* dy, void* dx, float* dgamma,
                    int rows, int cols, float eps, int dtype, float* scratch, cudaStream_t s);
int ltl_softmax(const void* x, const void* bias, void* out, int rows, int cols, float scale,
                int causal, int group, int mask_offset, int dtype, cudaStream_t s);
int ltl_softmax_bwd(const void* y, const void* dy, void* dx, int rows, int cols, float scale,
                    int causal, int group, int mask_offset, int dtype, cudaStream_t s);
int ltl_swiglu_fwd(const void* a, const void* b, void* out, int rows, int cols, int lda, int ldb,
                   int ldo, int dtype, cudaStream_t s);
int ltl_swiglu_bwd(const void* a, const void* b, const void* dout, void* da, void* db, int rows,
                   int cols, int lda, int ldb, int ldo, int dtype, cudaStream_t s);
// cs_table: optional [npos, head_dim/2] float2 (cos, sin) table; NULL = compute angles inline.
int ltl_rope(void* x, const int32_t* pos_ids, int rows, int heads, int head_dim, int row_stride,
             int pos_offset, float theta, int interleaved, int inverse, int dtype,
             const float2* cs_table, int table_rows, cudaStream_t s);
int ltl_rope_table(float2* table, int npos, int head_dim, float theta, cudaStream_t s);
int ltl_embed_fwd(const int32_t* ids, const void* table, void* out, int rows, int dim, int vocab,
                  int dtype, cudaStream_t s);
int ltl_embed_bwd(const int32_t* ids, const void* dout, float* dtable, int rows, int dim,
                  int vocab, float scale, int dtype, cudaStream_t s);
// pred (optional): row argmax of the logits (ties -> lowest index), written before dlogits.
bool ltl_cross_entropy_bf16_grad_supported(const void* logits, int vocab);
int ltl_cross_entropy_bf16_grad(const float* logits, const int32_t* targets, float* losses, bf16* dlogits_bf16, int32_t* pred,
                                int rows, int vocab, int ignore_index, float grad_scale, cudaStream_t s);
int ltl_cross_entropy(const void* logits, const int32_t* targets, float* losses, void* dlogits,
                      int32_t* pred, int rows, int vocab, int ignore_index, float grad_scale,
                      int dtype, cudaStream_t s);
int ltl_argmax_rows(const void* x, int32_t* out, int rows, int cols, int dtype, cudaStream_t s);
int ltl_l2_accum(const void* x, uint64_t n, float* out, int dtype, cudaStream_t s);
int ltl_clip_by_nsq(void* x, uint64_t n, const float* nsq, float max_norm, int dtype,
                    cudaStream_t s);
int ltl_sum_f32(const float* x, uint64_t n, float* out, float scale, cudaStream_t s);
int ltl_elementwise(const void* a, const void* b, void* c, uint64_t n, int dtype, int op,
                    float alpha, float beta, cudaStream_t s);
int ltl_cast(const void* src, int src_dtype, void* dst, int dst_dtype, uint64_t n, cudaStream_t s);
int ltl_adamw(float* w, const void* g, float* m, float* v, void* w_lp, uint64_t n, int grad_dtype,
              float lr, float beta1, float beta2, float eps, float wd, int step, float clip,
              cudaStream_t s);
// w -= lr * (f * g + wd * w), f = clip factor from *nsq (NULL or max_norm <= 0: f = 1).
// w_lp (optional) receives the bf16 copy of the updated weights.
int ltl_sgd(float* w, const float* g, bf16* w_lp, uint64_t n, float lr, float wd,
            const float* nsq, float max_norm, cudaStream_t s);
// One launch over a whole flat parameter buffer.  d_nodecay: device array of npairs sorted [begin, end) element ranges
// that take no weight decay; loss (optional, device): a non-finite value makes the launch a no-op.
int ltl_opt_ranges_ok(const long long* host_pairs, int npairs, const void* w, const void* g);
int ltl_sgd_flat(float* w, const float* g, uint64_t n, const long long* d_nodecay, int npairs, const float* loss,
                 const float* nsq, float lr, float wd, float max_norm, cudaStream_t s);
int ltl_adamw_flat(float* w, const float* g, float* m, float* v, uint64_t n, const long long* d_nodecay, int npairs,
                   const float* loss, float lr, float beta1, float beta2, float eps, float wd, int step, cudaStream_t s);
// out[c, r] = (bf16) in[r, c]
// interleave_half = F > 0: output row j < F goes to row 2j, row F + j to row 2j + 1 (gate/up pairs).
int ltl_transpose_any_to_bf16(const void* in, int in_dtype, bf16* out, int rows, int cols, cudaStream_t s);
int ltl_transpose_to_bf16(const float* in, bf16* out, int rows, int cols, int interleave_half, cudaStream_t s);

// ---- small ops of the reference's ABI that the token loop itself does not queue (compat.cu) ----
// out[c] = alpha * sum_r x[r * row_stride + c] + beta * out[c]
int ltl_reduce_cols(const void* x, float* out, int rows, int cols, long long row_stride, float alpha, float beta,
                    int dtype, cudaStream_t s);
// out [cols, rows] = in [rows, cols]^T
int ltl_transpose(const void* in, void* out, int rows, int cols, int dtype, cudaStream_t s);
// out[r, c] = x[r, c] + alpha * v[c]  (v may be NULL)
int ltl_bcast_add(const void* x, const void* v, void* out, int rows, int cols, float alpha, int dtype, cudaStream_t s);
// dst[r, :] = src[idx[r], :], rows outside [0, src_rows) give zeros
int ltl_gather_rows(const void* src, const int32_t* idx, void* dst, int n, int cols, int src_rows, int dtype, cudaStream_t s);
// out[r] = 1 / sqrt(mean_c x(r, c)^2 + eps) with x(r, c) at r * rs + c * cs
int ltl_row_rms(const void* x, float* out, int rows, int cols, long long rs, long long cs, float eps, int dtype, cudaStream_t s);

// ---- CUDA-core GEMM with explicit strides (gemm_simt.cu) ----
struct GemmDesc {
    const void* A; const void* B; void* C;
    const void* bias;      // [N], optional
    const void* R;         // residual with C's strides, optional: C = post(alpha*AB + bias) + beta*C + R
    int M, N, K, batch;
    long long a_rs, a_cs, b_rs, b_cs, c_rs, c_cs, a_bs, b_bs, c_bs;
    float alpha, beta;
    int post_op;           // 0 none, 1 relu, 2 gelu, 3 silu, 4 tanh, 5 sigmoid
    int a_dtype, b_dtype, c_dtype;
    // Prologue on A (the reference's pre_op, cuda/luaTL_train.cu:159-204): 0 none; 1 RMSNorm - A(m,k) is multiplied by
    // rowscale[m] (given, or 1/sqrt(mean_k A(m,k)^2 + eps) computed by the kernel) and by gamma[k] (optional);
    // 2 gelu, 3 silu, 4 relu applied to every element of A.
    int pre_op;
    const void* gamma;     // [K], A's dtype
    const float* rowscale; // [M] fp32
    float eps;
};
int ltl_gemm_simt(const GemmDesc& g, cudaStream_t s);

// ---- attention (attention.cu) ----
// Causal self-attention over packed [rows, 3D] q|k|v (after RoPE), sequences of T rows.
// out [rows, D]; lse [B*H*T] (log-sum-exp of the scaled scores, kept for the backward).
int ltl_attn_fwd(const void* qkv, void* out, float* lse, int B, int T, int H, int hd, float scale,
                 int causal, int dtype, cudaStream_t s);
// dqkv [rows, 3D]; delta [B*H*T] scratch.
int ltl_attn_bwd(const void* qkv, const void* out, const void* dout, const float* lse,
                 float* delta, void* dqkv, int B, int T, int H, int hd, float scale, int causal,
                 int dtype, cudaStream_t s);

// ---- token-loop kernels (lm_kernels.cu) ----
// res[r, :] = (float) table[ids[r], :]; table dtype f32 or bf16; ids outside [0, vocab) -> 0.
int ltl_lm_embed(const int32_t* ids, const void* table, int table_dtype, float* res, int rows,
                 int dim, int vocab, cudaStream_t s);
// out[r, :] = rmsnorm(x[r, :]) * gain, x and gain fp32, out f32 or bf16.
int ltl_lm_rmsnorm(const float* x, const float* gain, void* out, int out_dtype, int rows, int cols,
                   float eps, cudaStream_t s);
// x[r, :] += sum_s partial[s][r, :] (s = 0 .. nparts-1 in order; slices rows*cols apart), then
// out[r, :] = rmsnorm(x[r, :]) * gain.  The consumer side of the split-K GEMMs.
// Optional rider of ltl_lm_residual_rmsnorm in the decode step: CTA b asks the memory system to bring the first rows of
// sequence b's K and V cache of the NEXT attention kernel into L2 (cp.async.bulk.prefetch.L2, a hint: no data reaches
// the SM), so that HBM works during the latency-bound products between two attention kernels.  k / v: that layer's
// cache [nseq][heads][ctx][row_bytes]; the number of rows is min(pos[b] + pos_add, max_rows, ctx).
struct LtlKvPrefetch { const void* k; const void* v; const int32_t* pos; int heads, ctx, row_bytes, nseq, pos_add, max_rows; };
int ltl_lm_residual_rmsnorm(float* x, const float* partial, int nparts, const float* gain, void* out,
                            int out_dtype, int rows, int cols, float eps, cudaStream_t s, const LtlKvPrefetch* pf = nullptr);
// x[r, :] = table[ids[r], :] and out[r, :] = rmsnorm(x[r, :]) * gain in one launch.
int ltl_lm_embed_rmsnorm(const int32_t* ids, const void* table, int table_dtype, float* x, const float* gain,
                         void* out, int out_dtype, int rows, int cols, int vocab, float eps, cudaStream_t s);
// Prefill: copy rotated k and v of rows [B, T] of qkv [B*T, 3D] into the caches at 0..T-1.
int ltl_kv_store(const void* qkv, void* kcache, void* vcache, int B, int T, int H, int hd, int ctx,
                 int dtype, cudaStream_t s);
// Decode attention of one new token per sequence, fused with its RoPE and KV-cache append:
// q and k of row b of qkv [B, 3D] are rotated for position pos[b], k and v are written to that
// position of the caches, and the query attends cache positions 0..pos[b].
// splits > 1 spreads the keys of one (sequence, head) over several CTAs; scratch then holds
// decode_attn_scratch_floats(B, H, hd, splits) floats.  err is set to 1 if a position is outside
// [0, ctx).
size_t ltl_decode_attn_scratch_floats(int B, int H, int hd, int splits);
void ltl_decode_attn_shape(int ctas_per_sm, int stages);   // 0, 0 = one CTA per item, default ring depth
int ltl_decode_attn(const void* qkv, void* kcache, void* vcache, void* out,
                    const int32_t* pos, int B, int H, int hd, int ctx, float scale, int dtype,
                    int splits, float* scratch, const float2* cs_table, int interleaved, int use_rope,
                    int* err, cudaStream_t s, const float* qkv_parts = nullptr, int nparts = 0);
// nparts > 0: q | k | v are read as the sum of nparts fp32 slices [nparts][B][3 D] (a split-K projection), rounded to the
// storage type, instead of from qkv (which may then be null).  Only where ltl_decode_attn_takes_parts says so.
bool ltl_decode_attn_takes_parts(int hd, int dtype);
// Greedy pick and bookkeeping of one decode step, per sequence b:
//   next[b] = argmax(logits[b, :]) (ties -> lowest index);
//   out_ids[b * out_stride + count[b]] = next[b] when count[b] < out_stride; count[b] += 1; pos[b] += 1.
//   hist (optional): hist[b * hist_stride + hist_base + count[b]] = next[b] as well.
int ltl_pick_advance(const float* logits, int B, int V, int32_t* next, int32_t* out_ids,
                     int out_stride, int32_t* count, int32_t* pos, int32_t* hist, int hist_stride,
                     int hist_base, cudaStream_t s);
int ltl_sample_advance(const float* logits, int B, int V, int32_t* next, int32_t* out_ids, int out_stride, int32_t* count,
                       int32_t* pos, int32_t* hist, int hist_stride, int hist_base, float temperature, int top_k, float top_p,
                       uint64_t seed, int stop_id, int32_t* done, int slot0, cudaStream_t s);
int ltl_sample_rows(const float* logits, int rows, int V, float temperature, int top_k, float top_p, uint64_t seed,
                    const int32_t* counters, int32_t* out, cudaStream_t s);
int ltl_fill_i32(int32_t* p, int n, int32_t value, cudaStream_t s);
// correct[0] += #{r : tgt[r] >= 0 and pred[r] == tgt[r]}  (as float)
int ltl_count_correct(const int32_t* pred, const int32_t* tgt, int n, float* correct, cudaStream_t s);
// Gather row (b * T + last) of x [B*T, cols] into out [B, cols].
int ltl_gather_last_rows(const float* x, float* out, int B, int T, int cols, int last, cudaStream_t s);

// Fusions of the decode step around a GEMM (both GEMM kernels take it by value; all-null = none).
//  * residual form (epi = 3, split-K): the CTA that arrives last at an output tile adds the slices (in slice order)
//    and the residual x, writes x back, h = bf16(x * gain) and the tile's share of sum(x^2) per row to ssq_out
//    [M][tiles]; the RMSNorm factor itself is left to the consumer;
//  * row-scale form (ssq_in != null): the epilogue multiplies row r by 1 / sqrt(sum_t ssq_in[r][t] * inv_dim + eps).
struct LtlGemmFuse {
    float* x;
    const float* gain;
    void* h;
    float* ssq_out;
    int* counters;
    const float* ssq_in;
    int ssq_tiles;
    float inv_dim, eps;
};

// ---- tcgen05 / TMA GEMM (gemm_tc.cu): C[M,N] = A[M,K] B[N,K]^T + R, bf16 in, fp32 accumulate ----
bool ltl_gemm_tc_supported(const void* A, const void* B, int M, int N, int K);
// epi = 1: B rows interleave gate/up, C [M, N/2] bf16 = silu(gate) * up (R ignored).
// ksplit > 1: C receives ksplit fp32 partial matrices [ksplit][M][N] (no residual, no epilogue).
int ltl_gemm_tc(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int c_dtype,
                int bn, int epi, int ksplit, cudaStream_t s, const LtlGemmFuse* fuse = nullptr);
void ltl_gemm_tc_set_lean(int on);   // shallow shared-memory rings (a CTA that shares its SM with another stream's kernels)
void ltl_gemm_tc_plan_split(int M, int N, int K, int* bn, int* ksplit);
int ltl_gemm_tc_check(cudaStream_t s);
int ltl_gemm_tc_plan_accum(int M, int N, int K, int bn);
int ltl_gemm_tc_xty(const void* X, const void* Y, float* C, int M, int N, int K, int ksplit, cudaStream_t s);
// Few-row GEMM (gemm_rows.cu, mma.sync): 1 <= M <= 64, K a multiple of 32; same epi / ksplit meaning as above.
bool ltl_gemm_rows_supported(const void* A, const void* B, int M, int N, int K, int ksplit);
int ltl_gemm_rows_plan_split(int N, int K, int max_parts);
int ltl_gemm_rows(const void* A, const void* B, void* C, int M, int N, int K, int c_dtype, int epi, int ksplit, cudaStream_t s,
                  const LtlGemmFuse* fuse = nullptr);
// ---- the products of a decode step between two attention kernels as one cooperative launch (decode_chain.cu) ----
// A phase: out = epilogue(load(A) [M, K] . B[N, K]^T).  a_kind 0: A is bf16 [M, K]; 1: A = RMSNorm(x fp32 [M, K]) * gain rounded
// to bf16; 2: the same over rows gathered from a bf16 table by desc.tok (also written to desc.x).  epi 0: out (fp32 [M, N])
// += product; 1: SwiGLU over interleaved (gate, up) rows of B, out bf16 [M, N / 2]; 2: out bf16 [M, N]; 3: out fp32 [M, N].
// Phases run in order, a grid barrier between them; `bar` = two zero-initialised words, `err` is raised (3) by a wait that ran out.
struct LtlChainPhase { int a_kind, epi, N, K; const void* a; const float* gain; const void* b; void* out; };
struct LtlChainDesc {
    int M, nphases;
    float eps;
    const int32_t* tok; int vocab; float* x;
    unsigned* bar; int* err;
    int allow_pdl;
    LtlChainPhase ph[4];
};
bool ltl_decode_chain_supported(int D, int F, int V);
int ltl_decode_chain(const LtlChainDesc& d, cudaStream_t s);

// ---- tcgen05 / TMA GEMM on fp32 operands read as TF32 (gemm_tf32.cu): C[M,N] (+)= A[M,K] B[N,K]^T (+ R) ----
bool ltl_gemm_tf32_supported(const void* A, const void* B, const void* C, int M, int N, int K);
int ltl_gemm_tf32(const float* A, const float* B, float* C, const float* R, int M, int N, int K, int accumulate, int ksplit,
                  cudaStream_t s);

// CUtensorMap (128 bytes, written to out_map) of a bf16 matrix [rows, cols] with rows `pitch` elements apart:
// boxes of box_rows x 64 columns, 128-byte swizzle.  Cached per (base, shape).
int ltl_tensor_map_bf16(const void* base, int rows, int cols, long long pitch, int box_rows, void* out_map);
// Tensor-core flash attention (attention_tc.cu): bf16, head_dim 64 / 128, T a multiple of 8.
bool ltl_attn_tc_supported(int T, int H, int hd, int dtype);
int ltl_attn_fwd_tc(const void* qkv, void* out, float* lse, int B, int T, int H, int hd, float scale, int causal, cudaStream_t s);
int ltl_attn_bwd_tc(const void* qkv, const void* out, const void* dout, const float* lse, float* delta, void* dqkv,
                    int B, int T, int H, int hd, float scale, int causal, cudaStream_t s);
int ltl_attn_delta(const void* out, const void* dout, float* delta, int B, int T, int H, int hd, int dtype, cudaStream_t s);
int* ltl_tc_err_flag();        // device flag raised by a bounded wait that ran out (read by ltl_gemm_tc_check)
