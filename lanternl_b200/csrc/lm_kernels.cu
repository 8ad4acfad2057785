// Kernels that exist only inside the token loop: embedding gather into the fp32 residual
// stream, RMSNorm from the fp32 stream into the GEMM input type, decode attention over the
// device-resident KV cache (fused with RoPE and the cache append), greedy pick + position advance.
//
// KV cache layout: K and V are separate arrays [B, H, ctx, hd]; all positions of one
// (sequence, head) are contiguous, so decode attention streams each head's keys and values
// front to back with 16-byte loads.  The reference has no device KV cache (its GPU model
// re-runs a full forward per token, ai/gpu/gpu_transformer.lua:677); the semantics follow the
// CPU model's step() (ai/nn/transformer.lua:297-434).
#include <stdlib.h>

#include "ops.h"

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ------------------------------------------------------------------------------------------
template <typename TW>
__global__ void lm_embed_kernel(const int32_t* __restrict__ ids, const TW* __restrict__ table,
                                float* __restrict__ res, int rows, int dim, int vocab)
{
    const uint64_t n = (uint64_t)rows * dim;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (uint64_t)gridDim.x * blockDim.x) {
        const int r = (int)(idx / dim), c = (int)(idx - (uint64_t)r * dim);
        const int t = ids[r];
        res[idx] = (t >= 0 && t < vocab) ? Cvt<TW>::ld(table, (size_t)t * dim + c) : 0.0f;
    }
}

int ltl_lm_embed(const int32_t* ids, const void* table, int table_dtype, float* res, int rows,
                 int dim, int vocab, cudaStream_t s)
{
    if (!ids || !table || !res) return ltl_fail(LTL_ERR_NULL, "lm_embed: null pointer");
    if (rows <= 0) return LTL_OK;
    const uint64_t n = (uint64_t)rows * dim;
    unsigned grid = (unsigned)((n + 255) / 256);
    const unsigned cap = (unsigned)ltl_sm_count() * 16;
    if (grid > cap) grid = cap;
    if (table_dtype == LTL_F32) lm_embed_kernel<float><<<grid, 256, 0, s>>>(ids, (const float*)table, res, rows, dim, vocab);
    else if (table_dtype == LTL_BF16) lm_embed_kernel<bf16><<<grid, 256, 0, s>>>(ids, (const bf16*)table, res, rows, dim, vocab);
    else return ltl_fail(LTL_ERR_DTYPE, "lm_embed: table dtype %d", table_dtype);
    return ltl_check_launch("lm_embed");
}

// ------------------------------------------------------------------------------------------
// RMSNorm from the fp32 residual stream, one warp per row, the row read once.
template <typename TO>
__global__ void __launch_bounds__(128)
lm_rmsnorm_kernel(const float* __restrict__ x, const float* __restrict__ gain, TO* __restrict__ out,
                  int rows, int cols, float eps)
{
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const float* xr = x + (size_t)row * cols;
    float ss = 0.0f;
    for (int c = lane * 4; c < cols; c += 128) {
        const float4 v = *reinterpret_cast<const float4*>(xr + c);
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
    ss = warp_sum(ss);
    const float sc = 1.0f / sqrtf(ss / (float)cols + eps);
    TO* orow = out + (size_t)row * cols;
    for (int c = lane * 4; c < cols; c += 128) {
        const float4 v = *reinterpret_cast<const float4*>(xr + c);   // second read hits L1
        const float4 g = *reinterpret_cast<const float4*>(gain + c);
        Cvt<TO>::st(orow, c, v.x * sc * g.x);
        Cvt<TO>::st(orow, c + 1, v.y * sc * g.y);
        Cvt<TO>::st(orow, c + 2, v.z * sc * g.z);
        Cvt<TO>::st(orow, c + 3, v.w * sc * g.w);
    }
}

int ltl_lm_rmsnorm(const float* x, const float* gain, void* out, int out_dtype, int rows, int cols,
                   float eps, cudaStream_t s)
{
    if (!x || !gain || !out) return ltl_fail(LTL_ERR_NULL, "lm_rmsnorm: null pointer");
    if (cols % 4 || !aligned16(x) || !aligned16(gain))
        return ltl_fail(LTL_ERR_SHAPE, "lm_rmsnorm: width %d must be a multiple of 4 and 16-byte aligned", cols);
    if (rows <= 0) return LTL_OK;
    const int grid = (rows + 3) / 4;
    if (out_dtype == LTL_F32) lm_rmsnorm_kernel<float><<<grid, 128, 0, s>>>(x, gain, (float*)out, rows, cols, eps);
    else if (out_dtype == LTL_BF16) lm_rmsnorm_kernel<bf16><<<grid, 128, 0, s>>>(x, gain, (bf16*)out, rows, cols, eps);
    else return ltl_fail(LTL_ERR_DTYPE, "lm_rmsnorm: out dtype %d", out_dtype);
    return ltl_check_launch("lm_rmsnorm");
}


// Consumer of the split-K GEMMs: x += partial[0] + partial[1] + ... (fixed order, so the result
// does not depend on scheduling), then RMSNorm of the updated row.  One warp per row.
template <typename TO>
__global__ void __launch_bounds__(128)
lm_residual_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ partial, int nparts,
                           const float* __restrict__ gain, TO* __restrict__ out, int rows, int cols, float eps)
{
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    float* xr = x + (size_t)row * cols;
    const size_t slice = (size_t)rows * cols;
    float ss = 0.0f;
    for (int c = lane * 4; c < cols; c += 128) {
        float4 v = *reinterpret_cast<const float4*>(xr + c);
        float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int p = 0; p < nparts; ++p) {
            const float4 q = *reinterpret_cast<const float4*>(partial + p * slice + (size_t)row * cols + c);
            acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
        }
        v.x += acc.x; v.y += acc.y; v.z += acc.z; v.w += acc.w;
        *reinterpret_cast<float4*>(xr + c) = v;
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
    ss = warp_sum(ss);
    const float sc = 1.0f / sqrtf(ss / (float)cols + eps);
    TO* orow = out + (size_t)row * cols;
    for (int c = lane * 4; c < cols; c += 128) {
        const float4 v = *reinterpret_cast<const float4*>(xr + c);   // written by this lane above
        const float4 g = *reinterpret_cast<const float4*>(gain + c);
        Cvt<TO>::st(orow, c, v.x * sc * g.x);
        Cvt<TO>::st(orow, c + 1, v.y * sc * g.y);
        Cvt<TO>::st(orow, c + 2, v.z * sc * g.z);
        Cvt<TO>::st(orow, c + 3, v.w * sc * g.w);
    }
}

// The same with one CTA per row and one 16-byte chunk per thread (rows of up to 4096 columns): every load
// of a thread is independent and issued at once, the updated row stays in registers, and the sum of
// squares crosses the warps through shared memory.  Same summation order per element as above.
template <typename TO>
__global__ void __launch_bounds__(1024)
lm_residual_rmsnorm_row_kernel(float* __restrict__ x, const float* __restrict__ partial, int nparts,
                               const float* __restrict__ gain, TO* __restrict__ out, int rows, int cols, float eps,
                               const LtlKvPrefetch pf)
{
    __shared__ float red[32];
    pdl_trigger();
    if (pf.k && (int)blockIdx.x < pf.nseq && (int)threadIdx.x < 2 * pf.heads) {
        // L2 prefetch hint for the next attention kernel (ahead of the dependency wait: nothing in flight writes these rows;
        // a stale position only changes how much is asked for, and the range is clamped to this sequence's slab)
        const int h = threadIdx.x >> 1, isv = threadIdx.x & 1;
        int n = pf.pos[blockIdx.x] + pf.pos_add;
        n = min(min(n, pf.max_rows), pf.ctx);
        if (n > 0) {
            const char* base = reinterpret_cast<const char*>(isv ? pf.v : pf.k) +
                               ((size_t)blockIdx.x * pf.heads + h) * pf.ctx * pf.row_bytes;
            const uint32_t bytes = (uint32_t)n * (uint32_t)pf.row_bytes;
            asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base), "r"(bytes) : "memory");
        }
    }
    pdl_wait();
    const int row = blockIdx.x, c = threadIdx.x * 4;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
    const bool live = c < cols;
    const size_t slice = (size_t)rows * cols, off = (size_t)row * cols + c;
    float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f), g = v, acc = v;
    if (live) {
        v = *reinterpret_cast<const float4*>(x + off);
        g = *reinterpret_cast<const float4*>(gain + c);
#pragma unroll 4
        for (int p = 0; p < nparts; ++p) {
            const float4 q = *reinterpret_cast<const float4*>(partial + p * slice + off);
            acc.x += q.x; acc.y += q.y; acc.z += q.z; acc.w += q.w;
        }
        v.x += acc.x; v.y += acc.y; v.z += acc.z; v.w += acc.w;
        *reinterpret_cast<float4*>(x + off) = v;
    }
    float ss = warp_sum(fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w))));
    if (lane == 0) red[warp] = ss;
    __syncthreads();
    ss = 0.0f;
    for (int w = 0; w < nwarps; ++w) ss += red[w];             // same order in every thread
    const float sc = 1.0f / sqrtf(ss / (float)cols + eps);
    if (live) {
        const float o[4] = { v.x * sc * g.x, v.y * sc * g.y, v.z * sc * g.z, v.w * sc * g.w };
        if (sizeof(TO) == 2) {
            uint2 pk;
            pk.x = pack_bf16x2(o[0], o[1]);
            pk.y = pack_bf16x2(o[2], o[3]);
            *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(out) + off) = pk;
        } else {
            *reinterpret_cast<float4*>(reinterpret_cast<float*>(out) + off) = make_float4(o[0], o[1], o[2], o[3]);
        }
    }
}

int ltl_lm_residual_rmsnorm(float* x, const float* partial, int nparts, const float* gain, void* out,
                            int out_dtype, int rows, int cols, float eps, cudaStream_t s, const LtlKvPrefetch* pfp)
{
    LtlKvPrefetch pf = {};
    if (pfp && pfp->k && pfp->v && pfp->pos && pfp->row_bytes % 16 == 0 && pfp->max_rows > 0 && 2 * pfp->heads <= 32 &&
        aligned16(pfp->k) && aligned16(pfp->v))
        pf = *pfp;
    if (!x || !partial || !gain || !out) return ltl_fail(LTL_ERR_NULL, "lm_residual_rmsnorm: null pointer");
    if (cols % 4 || !aligned16(x) || !aligned16(gain) || !aligned16(partial))
        return ltl_fail(LTL_ERR_SHAPE, "lm_residual_rmsnorm: width %d must be a multiple of 4 and 16-byte aligned", cols);
    if (rows <= 0) return LTL_OK;
    if (cols <= 4096 && out_dtype == LTL_BF16 && aligned16(out) && cols % 8 == 0) {
        const int threads = ((cols / 4) + 31) / 32 * 32;
        LTL_CUDA("lm_residual_rmsnorm launch", ltl_launch(lm_residual_rmsnorm_row_kernel<bf16>, dim3(rows), dim3(threads), 0, s,
                                                          ltl_pdl_enabled(), x, partial, nparts, gain, (bf16*)out, rows, cols, eps, pf));
        return ltl_check_launch("lm_residual_rmsnorm");
    }
    const int grid = (rows + 3) / 4;
    if (out_dtype == LTL_F32) lm_residual_rmsnorm_kernel<float><<<grid, 128, 0, s>>>(x, partial, nparts, gain, (float*)out, rows, cols, eps);
    else if (out_dtype == LTL_BF16) LTL_CUDA("lm_residual_rmsnorm launch", ltl_launch(lm_residual_rmsnorm_kernel<bf16>, dim3(grid), dim3(128), 0, s, ltl_pdl_enabled(), x, partial, nparts, gain, (bf16*)out, rows, cols, eps));
    else return ltl_fail(LTL_ERR_DTYPE, "lm_residual_rmsnorm: out dtype %d", out_dtype);
    return ltl_check_launch("lm_residual_rmsnorm");
}

// Embedding gather into the residual stream fused with the first RMSNorm (one warp per row).
template <typename TW, typename TO>
__global__ void __launch_bounds__(128)
lm_embed_rmsnorm_kernel(const int32_t* __restrict__ ids, const TW* __restrict__ table, float* __restrict__ x,
                        const float* __restrict__ gain, TO* __restrict__ out, int rows, int cols, int vocab, float eps)
{
    pdl_trigger();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int t = ids[row];
    const bool okid = t >= 0 && t < vocab;
    float* xr = x + (size_t)row * cols;
    float ss = 0.0f;
    for (int c = lane * 4; c < cols; c += 128) {
        float4 v = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (okid) {
            const TW* src = table + (size_t)t * cols + c;
            v = make_float4(Cvt<TW>::ld(src, 0), Cvt<TW>::ld(src, 1), Cvt<TW>::ld(src, 2), Cvt<TW>::ld(src, 3));
        }
        *reinterpret_cast<float4*>(xr + c) = v;
        ss = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, ss))));
    }
    ss = warp_sum(ss);
    const float sc = 1.0f / sqrtf(ss / (float)cols + eps);
    TO* orow = out + (size_t)row * cols;
    for (int c = lane * 4; c < cols; c += 128) {
        const float4 v = *reinterpret_cast<const float4*>(xr + c);
        const float4 g = *reinterpret_cast<const float4*>(gain + c);
        Cvt<TO>::st(orow, c, v.x * sc * g.x);
        Cvt<TO>::st(orow, c + 1, v.y * sc * g.y);
        Cvt<TO>::st(orow, c + 2, v.z * sc * g.z);
        Cvt<TO>::st(orow, c + 3, v.w * sc * g.w);
    }
}

int ltl_lm_embed_rmsnorm(const int32_t* ids, const void* table, int table_dtype, float* x, const float* gain,
                         void* out, int out_dtype, int rows, int cols, int vocab, float eps, cudaStream_t s)
{
    if (!ids || !table || !x || !gain || !out) return ltl_fail(LTL_ERR_NULL, "lm_embed_rmsnorm: null pointer");
    if (cols % 4 || !aligned16(x) || !aligned16(gain))
        return ltl_fail(LTL_ERR_SHAPE, "lm_embed_rmsnorm: width %d must be a multiple of 4 and 16-byte aligned", cols);
    if (rows <= 0) return LTL_OK;
    const int grid = (rows + 3) / 4;
    if (table_dtype == LTL_F32 && out_dtype == LTL_F32)
        lm_embed_rmsnorm_kernel<float, float><<<grid, 128, 0, s>>>(ids, (const float*)table, x, gain, (float*)out, rows, cols, vocab, eps);
    else if (table_dtype == LTL_BF16 && out_dtype == LTL_BF16)
        LTL_CUDA("lm_embed_rmsnorm launch", ltl_launch(lm_embed_rmsnorm_kernel<bf16, bf16>, dim3(grid), dim3(128), 0, s, ltl_pdl_enabled(), ids, (const bf16*)table, x, gain, (bf16*)out, rows, cols, vocab, eps));
    else return ltl_fail(LTL_ERR_DTYPE, "lm_embed_rmsnorm: table dtype %d / out dtype %d", table_dtype, out_dtype);
    return ltl_check_launch("lm_embed_rmsnorm");
}

// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ qkv, T* __restrict__ kc, T* __restrict__ vc,
                                int B, int T_, int H, int hd, int ctx)
{
    const int D = H * hd;
    const uint64_t n = (uint64_t)B * T_ * D;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (uint64_t)gridDim.x * blockDim.x) {
        const int d = (int)(idx % hd);
        const int h = (int)((idx / hd) % H);
        const int t = (int)((idx / D) % T_);
        const int b = (int)(idx / ((uint64_t)D * T_));
        const size_t src = ((size_t)b * T_ + t) * 3 * D + (size_t)h * hd + d;
        const size_t dst = (((size_t)b * H + h) * ctx + t) * hd + d;
        kc[dst] = qkv[src + D];
        vc[dst] = qkv[src + 2 * D];
    }
}

// The same in 16-byte packets (head_dim a multiple of the packet, aligned operands): one thread moves one packet of k and
// one of v; consecutive threads walk a token's row, so reads are contiguous and writes run in head_dim-sized pieces.
template <typename T>
__global__ void kv_store_vec_kernel(const T* __restrict__ qkv, T* __restrict__ kc, T* __restrict__ vc,
                                    int B, int T_, int H, int hd, int ctx)
{
    constexpr int N = 16 / (int)sizeof(T);
    const int D = H * hd, pr = hd / N, prow = D / N;          // packets per head row and per token row
    const uint64_t n = (uint64_t)B * T_ * prow;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (uint64_t)gridDim.x * blockDim.x) {
        const int p = (int)(idx % prow);
        const uint64_t bt = idx / prow;
        const int t = (int)(bt % T_), b = (int)(bt / T_);
        const int h = p / pr, d = (p - h * pr) * N;
        const size_t src = (size_t)bt * 3 * D + (size_t)h * hd + d;
        const size_t dst = (((size_t)b * H + h) * ctx + t) * hd + d;
        *reinterpret_cast<uint4*>(kc + dst) = __ldg(reinterpret_cast<const uint4*>(qkv + src + D));
        *reinterpret_cast<uint4*>(vc + dst) = __ldg(reinterpret_cast<const uint4*>(qkv + src + 2 * D));
    }
}

int ltl_kv_store(const void* qkv, void* kcache, void* vcache, int B, int T, int H, int hd, int ctx,
                 int dtype, cudaStream_t s)
{
    if (!qkv || !kcache || !vcache) return ltl_fail(LTL_ERR_NULL, "kv_store: null pointer");
    if (T > ctx) return ltl_fail(LTL_ERR_SHAPE, "kv_store: %d positions exceed the cache (%d)", T, ctx);
    const uint64_t n = (uint64_t)B * T * H * hd;
    if (n == 0) return LTL_OK;
    const unsigned cap = (unsigned)ltl_sm_count() * 16;
    const int pk = dtype == LTL_F32 ? 4 : 8;                  // elements per 16-byte packet
    if ((dtype == LTL_F32 || dtype == LTL_BF16) && hd % pk == 0 && aligned16(qkv) && aligned16(kcache) && aligned16(vcache)) {
        unsigned grid = (unsigned)((n / pk + 255) / 256);
        if (grid > cap) grid = cap;
        if (dtype == LTL_F32) kv_store_vec_kernel<float><<<grid, 256, 0, s>>>((const float*)qkv, (float*)kcache, (float*)vcache, B, T, H, hd, ctx);
        else kv_store_vec_kernel<bf16><<<grid, 256, 0, s>>>((const bf16*)qkv, (bf16*)kcache, (bf16*)vcache, B, T, H, hd, ctx);
        return ltl_check_launch("kv_store");
    }
    unsigned grid = (unsigned)((n + 255) / 256);
    if (grid > cap) grid = cap;
    if (dtype == LTL_F32) kv_store_kernel<float><<<grid, 256, 0, s>>>((const float*)qkv, (float*)kcache, (float*)vcache, B, T, H, hd, ctx);
    else if (dtype == LTL_BF16) kv_store_kernel<bf16><<<grid, 256, 0, s>>>((const bf16*)qkv, (bf16*)kcache, (bf16*)vcache, B, T, H, hd, ctx);
    else return ltl_fail(LTL_ERR_DTYPE, "kv_store: dtype %d", dtype);
    return ltl_check_launch("kv_store");
}

// ------------------------------------------------------------------------------------------
// Decode attention, fused with RoPE of the new token and the KV-cache append.
// One CTA (128 threads) per (head, sequence, split).  A key of hd elements is covered by
// GL = hd * sizeof(T) / 16 lanes, each holding one 16-byte packet; the 128 / GL lane groups of
// the CTA walk the cached keys 0 .. pos-1 round-robin, four keys in flight per group, each group
// keeping its own online-softmax state; the groups are merged through shared memory.  The new
// token's q and k are rotated in registers (rounded to the storage type, as a stored tensor would
// be), its k and v are written to position pos of the cache by one group and enter the softmax
// from registers.  Bytes per (sequence, head): 2 * pos * hd * sizeof(T) read once - HBM-bound.
// ------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float round_to(float x);
template <> __device__ __forceinline__ float round_to<float>(float x) { return x; }
template <> __device__ __forceinline__ float round_to<bf16>(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

template <typename T, int HD>
__global__ void __launch_bounds__(128)
decode_attn_kernel(const T* __restrict__ qkv, T* __restrict__ kc, T* __restrict__ vc,
                   T* __restrict__ out, const int32_t* __restrict__ pos, int H, int ctx, float scale,
                   int splits, float* __restrict__ scratch, const float2* __restrict__ cs,
                   int interleaved, int use_rope, int* __restrict__ err)
{
    constexpr int N = Vec16<T>::N;
    constexpr int GL = HD / N;           // lanes per key
    constexpr int NG = 128 / GL;         // key groups per CTA
    constexpr int U = 4;                 // keys in flight per group
    static_assert(GL >= 2 && GL <= 32 && (GL & (GL - 1)) == 0, "head_dim / packet must be a power of two in 2..32");
    __shared__ float sm_m[NG], sm_l[NG];
    __shared__ float sm_acc[NG][HD + 1];
    const int h = blockIdx.x, b = blockIdx.y, z = blockIdx.z;
    const int D = H * HD;
    const int g = threadIdx.x / GL, r = threadIdx.x % GL;
    int ps = pos[b];
    const bool in_range = ps >= 0 && ps < ctx;
    if (!in_range) { if (err && threadIdx.x == 0) *err = 1; ps = ps < 0 ? 0 : ctx; }

    // the new token: q, k, v of this head from the projection row
    const T* row = qkv + (size_t)b * 3 * D + (size_t)h * HD + r * N;
    float q[N], kn[N], vn[N];
    ld16<T>(row, q);
    ld16<T>(row + D, kn);
    ld16<T>(row + 2 * D, vn);
    if (use_rope) {
        const float2* tab = cs + (size_t)(in_range ? ps : 0) * (HD / 2);
        if (interleaved) {
#pragma unroll
            for (int i = 0; i < N; i += 2) {
                const float2 t = tab[(r * N + i) >> 1];
                const float q0 = q[i], q1 = q[i + 1], k0 = kn[i], k1 = kn[i + 1];
                q[i] = q0 * t.x - q1 * t.y; q[i + 1] = q1 * t.x + q0 * t.y;
                kn[i] = k0 * t.x - k1 * t.y; kn[i + 1] = k1 * t.x + k0 * t.y;
            }
        } else {
            // pairs (p, p + hd/2): the partner element lives GL/2 lanes away
            const bool low = r < GL / 2;
            const int pbase = (r % (GL / 2)) * N;
#pragma unroll
            for (int i = 0; i < N; ++i) {
                const float qo = __shfl_xor_sync(0xFFFFFFFFu, q[i], GL / 2);
                const float ko = __shfl_xor_sync(0xFFFFFFFFu, kn[i], GL / 2);
                const float2 t = tab[pbase + i];
                q[i] = low ? q[i] * t.x - qo * t.y : q[i] * t.x + qo * t.y;
                kn[i] = low ? kn[i] * t.x - ko * t.y : kn[i] * t.x + ko * t.y;
            }
        }
#pragma unroll
        for (int i = 0; i < N; ++i) { q[i] = round_to<T>(q[i]); kn[i] = round_to<T>(kn[i]); }
    }
    const size_t cbase = ((size_t)b * H + h) * ctx * HD + r * N;
    if (z == 0 && g == 0 && in_range) {
        st16<T>(kc + cbase + (size_t)ps * HD, kn);
        st16<T>(vc + cbase + (size_t)ps * HD, vn);
    }
#pragma unroll
    for (int i = 0; i < N; ++i) q[i] *= scale;

    const int chunk = (ps + splits - 1) / splits;            // cached keys 0 .. ps-1 over the splits
    const int kbeg = z * chunk, kend = min(ps, kbeg + chunk);
    const T* kb = kc + cbase;
    const T* vb = vc + cbase;

    float m = -INFINITY, l = 0.0f, acc[N];
#pragma unroll
    for (int i = 0; i < N; ++i) acc[i] = 0.0f;

    // Uniform trip count across the CTA: the shuffles below need every lane of a warp.
    for (int kb0 = kbeg; kb0 < kend; kb0 += NG * U) {
        const int k0 = kb0 + g;
        float kv[U][N], vv[U][N];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = k0 + u * NG;
            if (k < kend) ld16<T>(kb + (size_t)k * HD, kv[u]);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = k0 + u * NG;
            if (k < kend) ld16<T>(vb + (size_t)k * HD, vv[u]);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = k0 + u * NG;
            float sdot = 0.0f;
            if (k < kend) {
#pragma unroll
                for (int i = 0; i < N; ++i) sdot = fmaf(q[i], kv[u][i], sdot);
            }
#pragma unroll
            for (int o = GL / 2; o > 0; o >>= 1) sdot += __shfl_xor_sync(0xFFFFFFFFu, sdot, o);
            if (k < kend) {
                const float mn = fmaxf(m, sdot);
                const float corr = expf(m - mn);          // m = -inf -> 0
                const float p = expf(sdot - mn);
                l = l * corr + p;
#pragma unroll
                for (int i = 0; i < N; ++i) acc[i] = fmaf(p, vv[u][i], acc[i] * corr);
                m = mn;
            }
        }
    }
    {   // the new token itself, from registers (every group computes the dot, one group uses it)
        float sdot = 0.0f;
#pragma unroll
        for (int i = 0; i < N; ++i) sdot = fmaf(q[i], kn[i], sdot);
#pragma unroll
        for (int o = GL / 2; o > 0; o >>= 1) sdot += __shfl_xor_sync(0xFFFFFFFFu, sdot, o);
        if (z == 0 && g == 0) {
            const float mn = fmaxf(m, sdot);
            const float corr = expf(m - mn);
            const float p = expf(sdot - mn);
            l = l * corr + p;
#pragma unroll
            for (int i = 0; i < N; ++i) acc[i] = fmaf(p, vn[i], acc[i] * corr);
            m = mn;
        }
    }
    if (r == 0) { sm_m[g] = m; sm_l[g] = l; }
#pragma unroll
    for (int i = 0; i < N; ++i) sm_acc[g][r * N + i] = acc[i];
    __syncthreads();
    if (threadIdx.x < HD) {
        const int d = threadIdx.x;
        float M = -INFINITY;
#pragma unroll 4
        for (int i = 0; i < NG; ++i) M = fmaxf(M, sm_m[i]);
        float L = 0.0f, o = 0.0f;
        if (M > -INFINITY) {
            for (int i = 0; i < NG; ++i) {
                const float w = expf(sm_m[i] - M);       // empty group: exp(-inf) = 0
                L = fmaf(sm_l[i], w, L);
                o = fmaf(sm_acc[i][d], w, o);
            }
        }
        if (splits == 1) {
            Cvt<T>::st(out, (size_t)b * D + (size_t)h * HD + d, L > 0.0f ? o / L : 0.0f);
        } else {
            float* sp = scratch + (((size_t)b * H + h) * splits + z) * (HD + 2);
            sp[2 + d] = o;
            if (d == 0) { sp[0] = M; sp[1] = L; }
        }
    }
}

// ------------------------------------------------------------------------------------------
// Decode attention, bulk-copy staged (rows of 128 bytes: bf16 head_dim 64, fp32 head_dim 32).
// The K and V rows of one (sequence, head) are contiguous in the cache, so one thread streams
// them into a 4-stage shared-memory ring with cp.async.bulk (64 keys = 8 KB of K and 8 KB of V
// per stage, completion on an mbarrier) while the four warps consume: two threads per key form
// the score from 16-byte chunks read in a rotated order (bank-conflict free), each warp keeps an
// online-softmax state for its 16 keys of the tile and accumulates P V with one 4-byte word of
// every V row per lane.  192 KB of loads can be in flight per SM without holding registers.
// The new token (RoPE, cache append, its own score) is handled as in the register kernel.
// ------------------------------------------------------------------------------------------
namespace bulk {
constexpr int KT = 64, ROWB = 128;
constexpr uint32_t SPIN = 1u << 22;
__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ bool wait(uint64_t* bar, uint32_t parity)
{
    const uint32_t a = s32(bar);
    for (uint32_t i = 0; i < SPIN; ++i) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(a), "r"(parity) : "memory");
        if (done) return true;
    }
    return false;
}
// The cache is read once per step and is far larger than L2: its lines are marked evict-first so that
// they do not push the weights and activations (re-read every step) out of L2.
__device__ __forceinline__ uint64_t evict_first_policy()
{
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void copy(void* dst, const void* src, uint32_t bytes, uint64_t* bar, uint64_t policy)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(s32(dst)), "l"(src), "r"(bytes), "r"(s32(bar)), "l"(policy) : "memory");
}
// Maximum over the warp with one redux instruction: floats are mapped to integers of the same order.
__device__ __forceinline__ float warp_max_redux(float x)
{
    int i = __float_as_int(x);
    i = i >= 0 ? i : i ^ 0x7FFFFFFF;
    i = __reduce_max_sync(0xFFFFFFFFu, i);
    return __int_as_float(i >= 0 ? i : i ^ 0x7FFFFFFF);
}
// The four 16-byte chunks of q a thread multiplies with (key j, half): the chunks of its half of the
// row, in the rotated order that keeps the 16-byte reads of the K rows free of bank conflicts.
template <int N>
__device__ __forceinline__ void load_q_chunks(const float* qs, int j, int half, float (&qr)[4][N])
{
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const int cc = (2 * c + half + 2 * j) & 7;
#pragma unroll
        for (int e = 0; e < N; e += 4) {
            const float4 t = *reinterpret_cast<const float4*>(qs + cc * N + e);
            qr[c][e] = t.x; qr[c][e + 1] = t.y; qr[c][e + 2] = t.z; qr[c][e + 3] = t.w;
        }
    }
}
// One 64-key tile for one warp: scores of the warp's 16 keys (two threads per key), online-softmax
// update of the warp's running maximum m, the thread's share of the denominator (lsum: summed over
// the warp at the end of the item; every key is counted by two threads) and P V with one 4-byte word
// of every V row per lane.
template <typename T, int N, int EPW>
__device__ __forceinline__ void consume_tile(const uint8_t* ks, const uint8_t* vs, int nk, const float (&qr)[4][N],
                                             int j, int half, int warp, int lane, float& m, float& lsum, float (&acc)[EPW])
{
    const T* krow = reinterpret_cast<const T*>(ks + j * ROWB);
    float part[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        const int cc = (2 * c + half + 2 * j) & 7;
        float kv[N];
        ld16<T>(krow + cc * N, kv);
        part[c] = 0.0f;
#pragma unroll
        for (int e = 0; e < N; ++e) part[c] = fmaf(qr[c][e], kv[e], part[c]);
    }
    float sdot = (part[0] + part[1]) + (part[2] + part[3]);
    sdot += __shfl_xor_sync(0xFFFFFFFFu, sdot, 1);
    const bool valid = j < nk;
    const float sv = valid ? sdot : -INFINITY;
    const float mn = fmaxf(m, warp_max_redux(sv));
    const float corr = (mn == -INFINITY) ? 1.0f : __expf(m - mn);
    const float pr = valid ? __expf(sv - mn) : 0.0f;
    lsum = fmaf(lsum, corr, pr);
    m = mn;
#pragma unroll
    for (int e = 0; e < EPW; ++e) acc[e] *= corr;
    const uint32_t* vrows = reinterpret_cast<const uint32_t*>(vs) + (size_t)(warp * 16) * (ROWB / 4) + lane;
    const int nmine = nk - warp * 16;                    // rows past the tile's end hold stale bytes: read as zero
    // All 16 row words and probabilities are fetched before the multiply-adds (no early exit in the
    // loop), so the shared-memory and shuffle latencies overlap; two partial sums halve the add chain.
    uint32_t w[16];
    float pj[16];
#pragma unroll
    for (int jj = 0; jj < 16; ++jj) w[jj] = jj < nmine ? vrows[jj * (ROWB / 4)] : 0u;
#pragma unroll
    for (int jj = 0; jj < 16; ++jj) pj[jj] = __shfl_sync(0xFFFFFFFFu, pr, 2 * jj);
    float odd[EPW];
#pragma unroll
    for (int e = 0; e < EPW; ++e) odd[e] = 0.0f;
#pragma unroll
    for (int jj = 0; jj < 16; jj += 2) {
        if (sizeof(T) == 2) {
            acc[0] = fmaf(pj[jj], __uint_as_float(w[jj] << 16), acc[0]);
            acc[EPW - 1] = fmaf(pj[jj], __uint_as_float(w[jj] & 0xFFFF0000u), acc[EPW - 1]);
            odd[0] = fmaf(pj[jj + 1], __uint_as_float(w[jj + 1] << 16), odd[0]);
            odd[EPW - 1] = fmaf(pj[jj + 1], __uint_as_float(w[jj + 1] & 0xFFFF0000u), odd[EPW - 1]);
        } else {
            acc[0] = fmaf(pj[jj], __uint_as_float(w[jj]), acc[0]);
            odd[0] = fmaf(pj[jj + 1], __uint_as_float(w[jj + 1]), odd[0]);
        }
    }
#pragma unroll
    for (int e = 0; e < EPW; ++e) acc[e] += odd[e];
}
template <int STG, int G>
struct Smem {
    alignas(128) uint8_t k[G * STG][KT * ROWB];
    alignas(128) uint8_t v[G * STG][KT * ROWB];
    alignas(16) float q[64], kn[64], vn[64];
    float wm[4 * G], wl[4 * G], wacc[4 * G][64];
    alignas(8) uint64_t full[G * STG];
};
}  // namespace bulk

// MINB: resident CTAs per SM the register allocation is held to.  5: 96 registers, the kernel that runs alone, one item
// per CTA (0.86 of HBM; with 80 registers it measures 0.83, with the 116 an unbounded allocation takes 0.78).
// 6: 80 registers and the item walk - the form that leaves registers and shared memory for another stream's GEMM CTAs.
// G: groups of four warps per CTA.  G = 2 (small batches, where an SM holds one or two items and a CTA's chain of tiles is
// what the launch waits for): the groups take alternate tiles of the item from rings of their own and meet in the final
// combine, which halves that chain without a second launch.
template <typename T, int HD, int STG, int MINB, int G>
__global__ void __launch_bounds__(128 * G, G == 1 ? MINB : 2)
decode_attn_bulk_kernel(const T* __restrict__ qkv, T* __restrict__ kc, T* __restrict__ vc,
                        T* __restrict__ out, const int32_t* __restrict__ pos, int B, int H, int ctx, float scale,
                        int splits, float* __restrict__ scratch, const float2* __restrict__ cs,
                        int interleaved, int use_rope, int* __restrict__ err,
                        const float* __restrict__ qparts, int nparts)
{
    using namespace bulk;
    static_assert(HD * sizeof(T) == ROWB && HD <= 64, "rows of 128 bytes");
    constexpr int N = Vec16<T>::N;           // elements per 16-byte chunk
    constexpr int GL = HD / N;               // 8 chunks per row
    constexpr int EPW = 4 / sizeof(T);       // elements per 4-byte word (dims per lane in P V)
    extern __shared__ uint8_t smem_raw[];
    Smem<STG, G>& sm = *reinterpret_cast<Smem<STG, G>*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const int D = H * HD, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int grp = G > 1 ? warp >> 2 : 0, lw = warp & 3, ltid = tid & 127;     // group, warp and thread inside the group
    pdl_trigger();
    pdl_wait();
    const uint64_t pol = evict_first_policy();
    if (tid == 0) {
        for (int s = 0; s < G * STG; ++s)
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(&sm.full[s])));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    // Work items are (head, sequence, cache slice) triples.  A grid that covers them all gives each CTA one; a smaller
    // grid (a fixed number of CTAs per SM, which leaves room on every SM for the kernels of another stream) walks them
    // with a stride.  The ring's stage index and barrier parity run on across items (tbase = tiles consumed so far).
    // MINB == 5 is the one-item form (grid = H x B x splits), compiled without the loop.
    constexpr bool WALK = MINB > 5;
    static_assert(!(WALK && G > 1), "the item walk runs with one group");
    const int nitems = H * B * splits;
    uint32_t tbase = 0;
    int item = WALK ? (int)blockIdx.x : 0;
    do {
        const int h = WALK ? item % H : (int)blockIdx.x;
        const int b = WALK ? (item / H) % B : (int)blockIdx.y;
        const int z = WALK ? item / (H * B) : (int)blockIdx.z;
        int ps = pos[b];
        const bool in_range = ps >= 0 && ps < ctx;
        if (!in_range) { if (err && tid == 0) *err = 1; ps = ps < 0 ? 0 : ctx; }
        const int chunk = (ps + splits - 1) / splits;
        const int kbeg = z * chunk, kend = min(ps, kbeg + chunk);
        const int ntiles = kend > kbeg ? (kend - kbeg + KT - 1) / KT : 0;
        const size_t cbase = ((size_t)b * H + h) * ctx * HD;
        const uint8_t* kg = reinterpret_cast<const uint8_t*>(kc + cbase);
        const uint8_t* vg = reinterpret_cast<const uint8_t*>(vc + cbase);

        if (tid == 0) {
            // first STG tiles of every group (this thread initialised the barriers; the groups' own producers take over below)
            for (int g = 0; g < G; ++g)
                for (int lt = 0; lt < STG && lt * G + g < ntiles; ++lt) {
                    const int k0 = kbeg + (lt * G + g) * KT, s = g * STG + (WALK ? (int)((tbase + lt) % STG) : lt);
                    const uint32_t bytes = (uint32_t)min(KT, kend - k0) * ROWB;
                    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(&sm.full[s])), "r"(2 * bytes) : "memory");
                    copy(sm.k[s], kg + (size_t)k0 * ROWB, bytes, &sm.full[s], pol);
                    copy(sm.v[s], vg + (size_t)k0 * ROWB, bytes, &sm.full[s], pol);
                }
        }
        // new token: the first GL lanes of warp 1 rotate q and k, append k / v, publish q, k, v as fp32
        if (warp == 1 && lane < GL) {
            const int r = lane;
            float q[N], kn[N], vn[N];
            if (nparts > 0) {
                // q | k | v arrive as split-K partial sums [nparts][B][3 D] of the projection: added in slice order and rounded
                // to the storage type, which is what the stored row would hold
                const size_t off = (size_t)b * 3 * D + (size_t)h * HD + r * N, slice = (size_t)B * 3 * D;
#pragma unroll
                for (int i = 0; i < N; ++i) { q[i] = 0.0f; kn[i] = 0.0f; vn[i] = 0.0f; }
                for (int p = 0; p < nparts; ++p) {
                    const float* pp = qparts + p * slice + off;
#pragma unroll
                    for (int i = 0; i < N; i += 4) {
                        const float4 a = __ldcg(reinterpret_cast<const float4*>(pp + i));
                        const float4 c = __ldcg(reinterpret_cast<const float4*>(pp + D + i));
                        const float4 d = __ldcg(reinterpret_cast<const float4*>(pp + 2 * D + i));
                        q[i] += a.x; q[i + 1] += a.y; q[i + 2] += a.z; q[i + 3] += a.w;
                        kn[i] += c.x; kn[i + 1] += c.y; kn[i + 2] += c.z; kn[i + 3] += c.w;
                        vn[i] += d.x; vn[i + 1] += d.y; vn[i + 2] += d.z; vn[i + 3] += d.w;
                    }
                }
#pragma unroll
                for (int i = 0; i < N; ++i) { q[i] = round_to<T>(q[i]); kn[i] = round_to<T>(kn[i]); vn[i] = round_to<T>(vn[i]); }
            } else {
                const T* row = qkv + (size_t)b * 3 * D + (size_t)h * HD + r * N;
                ld16<T>(row, q); ld16<T>(row + D, kn); ld16<T>(row + 2 * D, vn);
            }
            if (use_rope) {
                const float2* tab = cs + (size_t)(in_range ? ps : 0) * (HD / 2);
                constexpr unsigned GM = (1u << GL) - 1u;
                if (interleaved) {
#pragma unroll
                    for (int i = 0; i < N; i += 2) {
                        const float2 t = tab[(r * N + i) >> 1];
                        const float q0 = q[i], q1 = q[i + 1], k0 = kn[i], k1 = kn[i + 1];
                        q[i] = q0 * t.x - q1 * t.y; q[i + 1] = q1 * t.x + q0 * t.y;
                        kn[i] = k0 * t.x - k1 * t.y; kn[i + 1] = k1 * t.x + k0 * t.y;
                    }
                } else {
                    const bool low = r < GL / 2;
                    const int pbase = (r % (GL / 2)) * N;
#pragma unroll
                    for (int i = 0; i < N; ++i) {
                        const float qo = __shfl_xor_sync(GM, q[i], GL / 2);
                        const float ko = __shfl_xor_sync(GM, kn[i], GL / 2);
                        const float2 t = tab[pbase + i];
                        q[i] = low ? q[i] * t.x - qo * t.y : q[i] * t.x + qo * t.y;
                        kn[i] = low ? kn[i] * t.x - ko * t.y : kn[i] * t.x + ko * t.y;
                    }
                }
#pragma unroll
                for (int i = 0; i < N; ++i) { q[i] = round_to<T>(q[i]); kn[i] = round_to<T>(kn[i]); }
            }
            if (z == 0 && in_range) {
                st16<T>(kc + cbase + (size_t)ps * HD + r * N, kn);
                st16<T>(vc + cbase + (size_t)ps * HD + r * N, vn);
            }
#pragma unroll
            for (int i = 0; i < N; ++i) { sm.q[r * N + i] = q[i] * scale; sm.kn[r * N + i] = kn[i]; sm.vn[r * N + i] = vn[i]; }
        }
        __syncthreads();

        const int j = ltid >> 1, half = ltid & 1;        // two threads per key of the tile
        float m = -INFINITY, lsum = 0.0f, acc[EPW];
#pragma unroll
        for (int i = 0; i < EPW; ++i) acc[i] = 0.0f;
        float qr[4][N];
        load_q_chunks<N>(sm.q, j, half, qr);
        bool ok = true;
        const int mine = ntiles > grp ? (ntiles - grp + G - 1) / G : 0;      // tiles grp, grp + G, ... of the item
        for (int lt = 0; lt < mine; ++lt) {
            const int s = grp * STG + (WALK ? (int)((tbase + lt) % STG) : lt % STG);
            ok = wait(&sm.full[s], (WALK ? (tbase + lt) / STG : (uint32_t)(lt / STG)) & 1) && ok;
            const int nk = min(KT, kend - (kbeg + (lt * G + grp) * KT));
            consume_tile<T, N, EPW>(sm.k[s], sm.v[s], nk, qr, j, half, lw, lane, m, lsum, acc);
            if (G == 1) __syncthreads();                          // everyone is done with stage s
            else if (grp == 0) asm volatile("bar.sync 1, 128;" ::: "memory");      // the group's own barrier (immediate ids: 3 in use)
            else asm volatile("bar.sync 2, 128;" ::: "memory");
            if (ltid == 0 && lt + STG < mine) {
                const int k0 = kbeg + ((lt + STG) * G + grp) * KT;
                const uint32_t bytes = (uint32_t)min(KT, kend - k0) * ROWB;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(&sm.full[s])), "r"(2 * bytes) : "memory");
                copy(sm.k[s], kg + (size_t)k0 * ROWB, bytes, &sm.full[s], pol);
                copy(sm.v[s], vg + (size_t)k0 * ROWB, bytes, &sm.full[s], pol);
            }
        }
        if (WALK) tbase += (uint32_t)ntiles;
        if (!ok && err && tid == 0) *err = 2;
        float l = 0.5f * warp_sum(lsum);                             // every key sits in two lanes
        if (warp == 0 && z == 0) {     // the new token's own score, from the fp32 copies
            float sdot = 0.0f;
#pragma unroll
            for (int i = 0; i < EPW; ++i) sdot = fmaf(sm.q[lane * EPW + i], sm.kn[lane * EPW + i], sdot);
            sdot = warp_sum(sdot);
            const float mn = fmaxf(m, sdot);
            const float corr = (m == -INFINITY) ? 0.0f : expf(m - mn);
            const float p = expf(sdot - mn);
            l = l * corr + p;
#pragma unroll
            for (int i = 0; i < EPW; ++i) acc[i] = fmaf(p, sm.vn[lane * EPW + i], acc[i] * corr);
            m = mn;
        }
        if (lane == 0) { sm.wm[warp] = m; sm.wl[warp] = l; }
#pragma unroll
        for (int i = 0; i < EPW; ++i) sm.wacc[warp][lane * EPW + i] = acc[i];
        __syncthreads();
        if (tid < HD) {
            const int d = tid;
            float M = fmaxf(fmaxf(sm.wm[0], sm.wm[1]), fmaxf(sm.wm[2], sm.wm[3]));
#pragma unroll
            for (int w = 4; w < 4 * G; ++w) M = fmaxf(M, sm.wm[w]);
            float L = 0.0f, o = 0.0f;
            if (M > -INFINITY) {
#pragma unroll
                for (int w = 0; w < 4 * G; ++w) {
                    const float e = expf(sm.wm[w] - M);
                    L = fmaf(sm.wl[w], e, L);
                    o = fmaf(sm.wacc[w][d], e, o);
                }
            }
            if (splits == 1) {
                Cvt<T>::st(out, (size_t)b * D + (size_t)h * HD + d, L > 0.0f ? o / L : 0.0f);
            } else {
                float* sp = scratch + (((size_t)b * H + h) * splits + z) * (HD + 2);
                sp[2 + d] = o;
                if (d == 0) { sp[0] = M; sp[1] = L; }
            }
        }
        if (!WALK) break;
        __syncthreads();                                          // the next item rewrites q, kn, vn and the per-warp states
        item += (int)gridDim.x;
    } while (item < nitems);
}

template <typename T, int HD>
__global__ void decode_attn_combine_kernel(const float* __restrict__ scratch, T* __restrict__ out,
                                           int H, int splits)
{
    const int h = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
    if (d >= HD) return;
    const float* sp = scratch + ((size_t)b * H + h) * splits * (HD + 2);
    float M = -INFINITY;
    for (int z = 0; z < splits; ++z) M = fmaxf(M, sp[z * (HD + 2)]);
    float L = 0.0f, o = 0.0f;
    if (M > -INFINITY) {
        for (int z = 0; z < splits; ++z) {
            const float w = expf(sp[z * (HD + 2)] - M);
            L = fmaf(sp[z * (HD + 2) + 1], w, L);
            o = fmaf(sp[z * (HD + 2) + 2 + d], w, o);
        }
    }
    Cvt<T>::st(out, (size_t)b * H * HD + (size_t)h * HD + d, L > 0.0f ? o / L : 0.0f);
}

// Launch shape of the bulk kernel for the calls that follow (host-side, like the programmatic-launch switch):
// ctas_per_sm > 0 caps the grid at that many CTAs per SM, which then walk the (head, sequence) items - the form used when
// a second stream runs beside this kernel and needs shared memory and registers on every SM; stages > 0 overrides the ring depth.
static int g_attn_ctas_per_sm = 0, g_attn_stages = 0;
void ltl_decode_attn_shape(int ctas_per_sm, int stages) { g_attn_ctas_per_sm = ctas_per_sm; g_attn_stages = stages; }

// 1 when ltl_decode_attn can take q | k | v as split-K partial sums for this head size and type (the bulk-copy kernel:
// cache rows of 128 bytes, and the register kernel not forced).
bool ltl_decode_attn_takes_parts(int hd, int dtype)
{
    const char* e = getenv("LUATL_ATTN_REGS");
    if (e && e[0] == '1') return false;
    return (dtype == LTL_BF16 && hd == 64) || (dtype == LTL_F32 && hd == 32);
}

size_t ltl_decode_attn_scratch_floats(int B, int H, int hd, int splits)
{
    return splits > 1 ? (size_t)B * H * splits * (hd + 2) : 0;
}

template <typename T, int HD>
static int launch_decode_attn(const void* qkv, void* kc, void* vc, void* out,
                              const int32_t* pos, int B, int H, int ctx, float scale, int splits,
                              float* scratch, const float2* cs, int interleaved, int use_rope, int* err,
                              cudaStream_t s, const float* qparts, int nparts)
{
    dim3 grid(H, B, splits);
    if constexpr (HD * sizeof(T) == 128 && HD <= 64) {
        static const int env_ctas = [] { const char* e = getenv("LUATL_ATTN_CTAS"); return e ? atoi(e) : 0; }();   // A/B aid
        const int per_sm = g_attn_ctas_per_sm > 0 ? g_attn_ctas_per_sm : env_ctas;
        const int nitems = H * B * splits, cap = per_sm > 0 ? per_sm * ltl_sm_count() : nitems;
        const dim3 bgrid(nitems < cap ? nitems : cap);
        // 128-byte rows: the bulk-copy staged kernel (LUATL_ATTN_REGS=1 selects the register kernel)
        static const bool use_regs = [] { const char* e = getenv("LUATL_ATTN_REGS"); return e && e[0] == '1'; }();
        static const int stages = [] { const char* e = getenv("LUATL_ATTN_STAGES"); return e ? atoi(e) : 2; }();
        if (!use_regs) {
#define BULK_LAUNCH_M(STG, MINB, G)                                                                                \
            {                                                                                                      \
                const size_t smem = sizeof(bulk::Smem<STG, G>) + 128;                                              \
                static bool attr = false;                                                                          \
                if (!attr) {                                                                                       \
                    LTL_CUDA("decode_attn attr", cudaFuncSetAttribute(decode_attn_bulk_kernel<T, HD, STG, MINB, G>, \
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));                             \
                    attr = true;                                                                                   \
                }                                                                                                  \
                LTL_CUDA("decode_attn launch", ltl_launch(decode_attn_bulk_kernel<T, HD, STG, MINB, G>, MINB > 5 ? bgrid : grid, dim3(128 * G), smem, s, \
                    ltl_pdl_enabled() && splits == 1, (const T*)qkv, (T*)kc, (T*)vc, (T*)out, pos, B, H, ctx, scale, \
                    splits, scratch, cs, interleaved, use_rope, err, qparts, nparts));                             \
            }
#define BULK_LAUNCH(STG) { if (per_sm > 0) BULK_LAUNCH_M(STG, 6, 1) else if (groups == 2) BULK_LAUNCH_M(STG, 5, 2) else BULK_LAUNCH_M(STG, 5, 1) }
            // Two groups of warps per item when the cache is not sliced and an SM holds fewer than two items: measured per pass
            // of 511 steps at 32 sequences x 8 heads 130.7 -> 123.2 ms; slower from 64 sequences up (145.7 -> 148.7 ms, 128:
            // 182.9 -> 192.6) and on sliced caches (8 sequences: 101.6 -> 109.6).  LUATL_ATTN_GROUPS=1|2 overrides.
            const char* eg = getenv("LUATL_ATTN_GROUPS");        // read per launch: a test switches it between models
            const int env_groups = eg ? atoi(eg) : 0;
            const int groups = env_groups > 0 ? env_groups : (splits == 1 && nitems < 2 * ltl_sm_count() ? 2 : 1);
            const int stg = g_attn_stages > 0 ? g_attn_stages : stages;
            if (stg <= 1) BULK_LAUNCH(1) else if (stg == 2) BULK_LAUNCH(2) else if (stg == 3) BULK_LAUNCH(3) else BULK_LAUNCH(4)
#undef BULK_LAUNCH
#undef BULK_LAUNCH_M
            if (splits > 1) {
                dim3 g2(H, B);
                decode_attn_combine_kernel<T, HD><<<g2, HD < 32 ? 32 : HD, 0, s>>>(scratch, (T*)out, H, splits);
            }
            return ltl_check_launch("decode_attn");
        }
    }
    if (nparts > 0) return ltl_fail(LTL_ERR_UNSUPPORTED, "decode_attn: only the bulk-copy kernel takes q | k | v as partial sums");
    decode_attn_kernel<T, HD><<<grid, 128, 0, s>>>((const T*)qkv, (T*)kc, (T*)vc, (T*)out, pos, H, ctx, scale,
                                                   splits, scratch, cs, interleaved, use_rope, err);
    if (splits > 1) {
        dim3 g2(H, B);
        decode_attn_combine_kernel<T, HD><<<g2, HD < 32 ? 32 : HD, 0, s>>>(scratch, (T*)out, H, splits);
    }
    return ltl_check_launch("decode_attn");
}

int ltl_decode_attn(const void* qkv, void* kcache, void* vcache, void* out,
                    const int32_t* pos, int B, int H, int hd, int ctx, float scale, int dtype,
                    int splits, float* scratch, const float2* cs_table, int interleaved, int use_rope,
                    int* err, cudaStream_t s, const float* qkv_parts, int nparts)
{
    if (use_rope && !cs_table) return ltl_fail(LTL_ERR_NULL, "decode_attn: missing angle table");
    if (nparts > 0 && (!qkv_parts || !aligned16(qkv_parts) || (H * hd) % 4))
        return ltl_fail(LTL_ERR_ARG, "decode_attn: partial sums need a 16-byte aligned buffer and a width that is a multiple of 4");
    if (nparts > 0) qkv = qkv_parts;                          // the stored q | k | v row is not read
    if (!qkv || !kcache || !vcache || !out || !pos) return ltl_fail(LTL_ERR_NULL, "decode_attn: null pointer");
    if (B <= 0 || H <= 0) return ltl_fail(LTL_ERR_SHAPE, "decode_attn: bad shape");
    if (B > 65535 || splits > 65535) return ltl_fail(LTL_ERR_SHAPE, "decode_attn: grid too large");
    if (splits < 1) splits = 1;
    if (splits > 1 && !scratch) return ltl_fail(LTL_ERR_NULL, "decode_attn: split-KV needs scratch");
    if (!aligned16(qkv) || !aligned16(kcache) || !aligned16(vcache))
        return ltl_fail(LTL_ERR_ARG, "decode_attn: operands must be 16-byte aligned");
#define DA(TT, HH) return launch_decode_attn<TT, HH>(qkv, kcache, vcache, out, pos, B, H, ctx, scale, splits, scratch, cs_table, interleaved, use_rope, err, s, qkv_parts, nparts < 0 ? 0 : nparts)
    if (dtype == LTL_F32) {
        if (hd == 16) DA(float, 16);
        if (hd == 32) DA(float, 32);
        if (hd == 64) DA(float, 64);
        if (hd == 128) DA(float, 128);
    } else if (dtype == LTL_BF16) {
        if (hd == 16) DA(bf16, 16);
        if (hd == 32) DA(bf16, 32);
        if (hd == 64) DA(bf16, 64);
        if (hd == 128) DA(bf16, 128);
    } else return ltl_fail(LTL_ERR_DTYPE, "decode_attn: dtype %d", dtype);
#undef DA
    return ltl_fail(LTL_ERR_UNSUPPORTED, "decode_attn: head_dim %d not in {16,32,64,128}", hd);
}

// ------------------------------------------------------------------------------------------
__global__ void pick_advance_kernel(const float* __restrict__ logits, int V, int32_t* __restrict__ next,
                                    int32_t* __restrict__ out_ids, int out_stride,
                                    int32_t* __restrict__ count, int32_t* __restrict__ pos,
                                    int32_t* __restrict__ hist, int hist_stride, int hist_base)
{
    __shared__ float red_v[32];
    __shared__ int red_i[32];
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x;
    const float* row = logits + (size_t)b * V;
    float best = -INFINITY;
    int bi = 0x7FFFFFFF;
    if ((V & 3) == 0 && (reinterpret_cast<uintptr_t>(row) & 15) == 0) {
        for (int i = threadIdx.x * 4; i < V; i += blockDim.x * 4) {      // ascending per thread: first maximum wins
            const float4 q = *reinterpret_cast<const float4*>(row + i);
            if (q.x > best) { best = q.x; bi = i; }
            if (q.y > best) { best = q.y; bi = i + 1; }
            if (q.z > best) { best = q.z; bi = i + 2; }
            if (q.w > best) { best = q.w; bi = i + 3; }
        }
    } else {
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            const float v = row[i];
            if (v > best) { best = v; bi = i; }
        }
    }
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
        if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (lane == 0) { red_v[wid] = best; red_i[wid] = bi; }
    __syncthreads();
    if (wid == 0) {
        best = lane < nw ? red_v[lane] : -INFINITY;
        bi = lane < nw ? red_i[lane] : 0x7FFFFFFF;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, o);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, bi, o);
            if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
        }
        if (lane == 0) {
            if (bi == 0x7FFFFFFF) bi = 0;
            next[b] = bi;
            const int c = count[b];
            if (out_ids && c < out_stride) out_ids[(size_t)b * out_stride + c] = bi;
            if (hist && hist_base + c < hist_stride) hist[(size_t)b * hist_stride + hist_base + c] = bi;
            count[b] = c + 1;
            pos[b] += 1;
        }
    }
}

int ltl_pick_advance(const float* logits, int B, int V, int32_t* next, int32_t* out_ids,
                     int out_stride, int32_t* count, int32_t* pos, int32_t* hist, int hist_stride,
                     int hist_base, cudaStream_t s)
{
    if (!logits || !next || !count || !pos) return ltl_fail(LTL_ERR_NULL, "pick_advance: null pointer");
    if (B <= 0) return LTL_OK;
    LTL_CUDA("pick_advance launch", ltl_launch(pick_advance_kernel, dim3(B), dim3(V >= 4096 ? 1024 : 256), 0, s, ltl_pdl_enabled(), logits, V, next, out_ids, out_stride, count, pos, hist, hist_stride, hist_base));
    return ltl_check_launch("pick_advance");
}

// ------------------------------------------------------------------------------------------
// Sampling beyond greedy on the device (rule: ai/optim/lmtrain.lua:1364-1436).
//   temperature <= 0            -> argmax (pick_advance_kernel)
//   top_k in [1, 128]           -> the k largest logits in descending order (ties: lower index first), softmax at the
//                                  temperature over them, optional nucleus cut-off top_p inside that set, then the
//                                  first candidate whose cumulative weight reaches u * norm
//   top_k = 0 and top_p = 0     -> the same walk over the whole row in index order
// u is a counter-based uniform in [0, 1) with 24 bits: splitmix64(seed, sequence, position), so a generation is
// reproducible and independent of launch geometry.  One CTA per row.
// ------------------------------------------------------------------------------------------
namespace samp {
constexpr int MAXK = 128, EQCAP = 1024;
__host__ __device__ inline uint64_t mix64(uint64_t z)
{
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
__host__ __device__ inline float uniform24(uint64_t seed, uint32_t row, uint32_t counter)
{
    const uint64_t h = mix64(mix64(seed ^ ((uint64_t)row << 32)) ^ counter);
    return (float)(h >> 40) * (1.0f / 16777216.0f);
}
__device__ __forceinline__ uint32_t order_key(float x)       // larger float -> larger unsigned
{
    const uint32_t u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
}  // namespace samp

// ---- general rule: any top_k, nucleus over the whole row -------------------------------------------------------
// The reference sorts the row (or keeps an ordered top-k list) and walks it in descending order accumulating softmax
// weights (ai/optim/lmtrain.lua:1377-1436).  Nothing is sorted here.  The k-th largest key comes from a radix select;
// weights are taken as 40-bit fixed point (integer sums do not depend on the order of the atomics, so a draw is
// reproducible), and "the first candidate, in descending order, at which the running sum reaches tau" is found by a
// second radix descent over the keys, byte by byte, on per-bucket weight sums.  Equal values rank by index (lower
// first), as the reference's insertion pass leaves them.
namespace samp {
__device__ __forceinline__ float key_value(unsigned key)
{
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7FFFFFFFu) : ~key);
}
__device__ __forceinline__ unsigned long long weight_q(float x, float mx, float invT)
{
    return __float2ull_rz(expf((x - mx) * invT) * 1099511627776.0f);      // 2^40
}
// Index of the j-th (1-based, ascending index) element whose key equals K; -1 if there are fewer.  cnt: blockDim.x ints.
__device__ int nth_with_key(const float* __restrict__ row, int V, unsigned K, int j, int* cnt, int* s_out)
{
    const int tid = threadIdx.x, nt = blockDim.x;
    const int chunk = (V + nt - 1) / nt, i0 = min(V, tid * chunk), i1 = min(V, i0 + chunk);
    int c = 0;
    for (int i = i0; i < i1; ++i) c += order_key(row[i]) == K;
    __syncthreads();
    cnt[tid] = c;
    __syncthreads();
    if (tid == 0) {
        int acc = 0, owner = -1, res = -1;
        for (int t = 0; t < nt; ++t) { if (acc + cnt[t] >= j) { owner = t; break; } acc += cnt[t]; }
        if (owner >= 0 && j >= 1) {
            const int a = min(V, owner * chunk), b = min(V, a + chunk);
            for (int i = a; i < b; ++i) if (order_key(row[i]) == K && ++acc == j) { res = i; break; }
        }
        *s_out = res;
    }
    __syncthreads();
    return *s_out;
}
}  // namespace samp

// Key of the k-th largest element of the row (1 <= k <= V): radix select, most significant byte first.
__device__ unsigned select_kth_key(const float* __restrict__ row, int V, int k, unsigned* hist, unsigned* s_prefix, unsigned* s_need)
{
    using namespace samp;
    const int tid = threadIdx.x, nt = blockDim.x;
    __syncthreads();
    if (tid == 0) { *s_prefix = 0; *s_need = (unsigned)k; }
    for (int pass = 0; pass < 4; ++pass) {
        const int shift = 24 - 8 * pass;
        for (int i = tid; i < 256; i += nt) hist[i] = 0;
        __syncthreads();
        const unsigned prefix = *s_prefix, himask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
        for (int i = tid; i < V; i += nt) {
            const unsigned key = order_key(row[i]);
            if ((key & himask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
        }
        __syncthreads();
        if (tid == 0) {
            unsigned need = *s_need;
            int bkt = 255;
            for (; bkt > 0; --bkt) { if (hist[bkt] >= need) break; need -= hist[bkt]; }
            *s_prefix = prefix | ((unsigned)bkt << shift);
            *s_need = need;
        }
        __syncthreads();
    }
    return *s_prefix;
}

__device__ int sample_row_general(const float* __restrict__ row, int V, float temperature, int top_k, float top_p, float u)
{
    using namespace samp;
    __shared__ unsigned hist[256];
    __shared__ unsigned long long mass[256];
    __shared__ int cnt[1024];
    __shared__ float red[33];
    __shared__ unsigned s_prefix, s_need, s_ngt;
    __shared__ unsigned long long s_total, s_acc;
    __shared__ int s_idx;
    const int tid = threadIdx.x, nt = blockDim.x;
    const float invT = 1.0f / temperature;
    float mxl = -INFINITY;
    for (int i = tid; i < V; i += nt) mxl = fmaxf(mxl, row[i]);
    const float mx = block_max(mxl, red);
    // candidate set: the k largest (ties at the k-th value: lowest indices), or the whole row
    unsigned kth = 0u;
    int tie_cut = V;
    if (top_k > 0 && top_k < V) {
        kth = select_kth_key(row, V, top_k, hist, &s_prefix, &s_need);
        if (tid == 0) s_ngt = 0;
        __syncthreads();
        unsigned c = 0;
        for (int i = tid; i < V; i += nt) c += order_key(row[i]) > kth;
        if (c) atomicAdd(&s_ngt, c);
        __syncthreads();
        tie_cut = nth_with_key(row, V, kth, top_k - (int)s_ngt, cnt, &s_idx);
        if (tie_cut < 0) tie_cut = V;
    }
    auto in_set = [&](unsigned key, int i) { return key > kth || (key == kth && i <= tie_cut); };
    if (tid == 0) s_total = 0ull;
    __syncthreads();
    {
        unsigned long long t = 0ull;
        for (int i = tid; i < V; i += nt) { const float x = row[i]; if (in_set(order_key(x), i)) t += weight_q(x, mx, invT); }
        if (t) atomicAdd(&s_total, t);
    }
    __syncthreads();
    // Descending walk to the first candidate at which the running sum reaches tau (1 <= tau <= sum of the set): returns
    // its index, leaves the running sum including that candidate in s_acc.
    auto crossing = [&](unsigned long long tau) -> int {
        __syncthreads();
        if (tid == 0) { s_prefix = 0u; s_acc = 0ull; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int i = tid; i < 256; i += nt) mass[i] = 0ull;
            __syncthreads();
            const unsigned prefix = s_prefix, himask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
            for (int i = tid; i < V; i += nt) {
                const float x = row[i];
                const unsigned key = order_key(x);
                if ((key & himask) == prefix && in_set(key, i)) {
                    const unsigned long long w = weight_q(x, mx, invT);
                    if (w) atomicAdd(&mass[(key >> shift) & 255u], w);
                }
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long acc = s_acc;
                int bkt = 255;
                for (; bkt > 0; --bkt) { if (acc + mass[bkt] >= tau) break; acc += mass[bkt]; }
                s_prefix = prefix | ((unsigned)bkt << shift);
                s_acc = acc;
            }
            __syncthreads();
        }
        const unsigned key = s_prefix;
        unsigned long long w = weight_q(key_value(key), mx, invT);
        if (w == 0ull) w = 1ull;
        const unsigned long long acc = s_acc;
        const unsigned long long j = tau > acc ? (tau - acc + w - 1ull) / w : 1ull;
        const int idx = nth_with_key(row, V, key, (int)j, cnt, &s_idx);
        if (tid == 0) s_acc = acc + j * w;
        __syncthreads();
        return idx;
    };
    unsigned long long norm = s_total;
    if (norm == 0ull) norm = 1ull;
    if (top_p > 0.0f && top_p < 1.0f) {
        unsigned long long tau = (unsigned long long)ceil((double)top_p * (double)norm);
        if (tau < 1ull) tau = 1ull;
        if (tau > norm) tau = norm;
        (void)crossing(tau);
        norm = s_acc;                                    // weight of the nucleus: everything down to the candidate that closed it
    }
    unsigned long long tau = (unsigned long long)ceil((double)u * (double)norm);
    if (tau < 1ull) tau = 1ull;
    if (tau > norm) tau = norm;
    int pick = crossing(tau);
    if (pick < 0) {                                       // cannot happen for finite logits; fall back to the largest
        float best = -INFINITY; int bi = 0;
        if (tid == 0) { for (int i = 0; i < V; ++i) if (row[i] > best) { best = row[i]; bi = i; } s_idx = bi; }
        __syncthreads();
        pick = s_idx;
    }
    return pick;
}

// Returns the sampled index of one row (valid in thread 0).  blockDim.x threads, a multiple of 32, at most 1024.
__device__ int sample_row(const float* __restrict__ row, int V, float temperature, int top_k, float top_p, float u)
{
    using namespace samp;
    __shared__ unsigned hist[256];
    __shared__ float cand_v[MAXK];
    __shared__ int cand_i[MAXK];
    __shared__ int eq_i[EQCAP];
    __shared__ float sorted_v[MAXK];
    __shared__ int sorted_i[MAXK];
    __shared__ unsigned s_prefix, s_need, s_ngt, s_neq;
    __shared__ float red[33];
    __shared__ float scan[1024];
    __shared__ int s_pick;
    const int tid = threadIdx.x, nt = blockDim.x;
    const float invT = 1.0f / temperature;
    const bool nucleus = top_p > 0.0f && top_p < 1.0f;
    if ((top_k > MAXK && top_k < V) || (nucleus && !(top_k > 0 && top_k < V)))
        return sample_row_general(row, V, temperature, top_k, top_p, u);
    if (top_k > 0 && top_k < V) {
        const int k = top_k < MAXK ? top_k : MAXK;
        // radix select, most significant byte first: key of the k-th largest element
        if (tid == 0) { s_prefix = 0; s_need = (unsigned)k; }
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int i = tid; i < 256; i += nt) hist[i] = 0;
            __syncthreads();
            const unsigned prefix = s_prefix, himask = pass == 0 ? 0u : (0xFFFFFFFFu << (shift + 8));
            for (int i = tid; i < V; i += nt) {
                const unsigned key = order_key(row[i]);
                if ((key & himask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned need = s_need;
                int bkt = 255;
                for (; bkt > 0; --bkt) { if (hist[bkt] >= need) break; need -= hist[bkt]; }
                s_prefix = prefix | ((unsigned)bkt << shift);
                s_need = need;                           // how many of the bucket's elements are still wanted
            }
            __syncthreads();
        }
        const unsigned kth = s_prefix;
        if (tid == 0) { s_ngt = 0; s_neq = 0; }
        __syncthreads();
        for (int i = tid; i < V; i += nt) {
            const float x = row[i];
            const unsigned key = order_key(x);
            if (key > kth) { const unsigned slot = atomicAdd(&s_ngt, 1u); if (slot < (unsigned)MAXK) { cand_v[slot] = x; cand_i[slot] = i; } }
            else if (key == kth) { const unsigned slot = atomicAdd(&s_neq, 1u); if (slot < (unsigned)EQCAP) eq_i[slot] = i; }
        }
        __syncthreads();
        const int ngt = min((int)s_ngt, k), neq = min((int)s_neq, EQCAP), want_eq = min(k - ngt, neq);
        // the elements equal to the k-th value with the lowest indices complete the set
        for (int e = tid; e < neq; e += nt) {
            int rank = 0;
            for (int o = 0; o < neq; ++o) rank += eq_i[o] < eq_i[e];
            if (rank < want_eq) { cand_v[ngt + rank] = row[eq_i[e]]; cand_i[ngt + rank] = eq_i[e]; }
        }
        __syncthreads();
        const int n = ngt + want_eq;
        // order: value descending, index ascending (rank sort over at most 128 candidates)
        for (int e = tid; e < n; e += nt) {
            int rank = 0;
            for (int o = 0; o < n; ++o) rank += (cand_v[o] > cand_v[e]) || (cand_v[o] == cand_v[e] && cand_i[o] < cand_i[e]);
            sorted_v[rank] = cand_v[e]; sorted_i[rank] = cand_i[e];
        }
        __syncthreads();
        if (tid == 0) {
            const float mx = sorted_v[0];
            float sum = 0.0f;
            for (int r = 0; r < n; ++r) { cand_v[r] = expf((sorted_v[r] - mx) * invT); sum += cand_v[r]; }
            int limit = n;
            if (top_p > 0.0f && top_p < 1.0f) {
                float acc = 0.0f;
                for (int r = 0; r < n; ++r) { acc += cand_v[r] / sum; if (acc >= top_p) { limit = r + 1; break; } }
            }
            float norm = 0.0f;
            for (int r = 0; r < limit; ++r) norm += cand_v[r];
            const float target = u * norm;
            float acc = 0.0f;
            int pick = sorted_i[limit - 1];
            for (int r = 0; r < limit; ++r) { acc += cand_v[r]; if (acc >= target) { pick = sorted_i[r]; break; } }
            s_pick = pick;
        }
        __syncthreads();
        return s_pick;
    }
    // whole row in index order: contiguous chunk per thread, block scan of the chunk sums
    const int chunk = (V + nt - 1) / nt, i0 = tid * chunk, i1 = min(V, i0 + chunk);
    float mx = -INFINITY;
    for (int i = i0; i < i1; ++i) mx = fmaxf(mx, row[i]);
    mx = block_max(mx, red);
    float local = 0.0f;
    for (int i = i0; i < i1; ++i) local += expf((row[i] - mx) * invT);
    scan[tid] = local;
    __syncthreads();
    if (tid == 0) {
        float total = 0.0f;
        for (int t = 0; t < nt; ++t) total += scan[t];
        const float target = u * total;
        float acc = 0.0f;
        int owner = nt - 1;
        for (int t = 0; t < nt; ++t) { if (acc + scan[t] >= target) { owner = t; break; } acc += scan[t]; }
        while (owner > 0 && owner * chunk >= V) --owner;
        int pick = min(V, (owner + 1) * chunk) - 1;
        for (int i = owner * chunk; i < min(V, (owner + 1) * chunk); ++i) {
            acc += expf((row[i] - mx) * invT);
            if (acc >= target) { pick = i; break; }
        }
        s_pick = pick;
    }
    __syncthreads();
    return s_pick;
}

__global__ void __launch_bounds__(1024)
sample_advance_kernel(const float* __restrict__ logits, int V, int32_t* __restrict__ next, int32_t* __restrict__ out_ids,
                      int out_stride, int32_t* __restrict__ count, int32_t* __restrict__ pos, int32_t* __restrict__ hist,
                      int hist_stride, int hist_base, float temperature, int top_k, float top_p, unsigned long long seed,
                      int stop_id, int32_t* __restrict__ done, int slot0)
{
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.x;
    const float u = samp::uniform24(seed, (uint32_t)(slot0 + b), (uint32_t)pos[b]);
    int pick = sample_row(logits + (size_t)b * V, V, temperature, top_k, top_p, u);
    if (threadIdx.x == 0) {
        if (done && stop_id >= 0) {
            if (done[b]) pick = stop_id;                 // a finished sequence keeps emitting its stop token
            else if (pick == stop_id) done[b] = 1;
        }
        next[b] = pick;
        const int c = count[b];
        if (out_ids && c < out_stride) out_ids[(size_t)b * out_stride + c] = pick;
        if (hist && hist_base + c < hist_stride) hist[(size_t)b * hist_stride + hist_base + c] = pick;
        count[b] = c + 1;
        pos[b] += 1;
    }
}

// One sampled index per row with explicit counters (the position of the row in its sequence): the rule of the
// generation loop as an immediate op.
__global__ void __launch_bounds__(1024)
sample_rows_kernel(const float* __restrict__ logits, int V, float temperature, int top_k, float top_p,
                   unsigned long long seed, const int32_t* __restrict__ counters, int32_t* __restrict__ out)
{
    const int b = blockIdx.x;
    const float u = samp::uniform24(seed, (uint32_t)b, (uint32_t)(counters ? counters[b] : 0));
    const int pick = sample_row(logits + (size_t)b * V, V, temperature, top_k, top_p, u);
    if (threadIdx.x == 0) out[b] = pick;
}

static int check_sampling(float temperature, int top_k, float top_p, int V)
{
    (void)top_p; (void)V;
    if (!(temperature > 0.0f)) return ltl_fail(LTL_ERR_ARG, "sample: temperature must be positive (use the greedy pick otherwise)");
    if (top_k < 0) return ltl_fail(LTL_ERR_ARG, "sample: top_k %d is negative", top_k);
    return LTL_OK;
}

int ltl_sample_advance(const float* logits, int B, int V, int32_t* next, int32_t* out_ids, int out_stride, int32_t* count,
                       int32_t* pos, int32_t* hist, int hist_stride, int hist_base, float temperature, int top_k, float top_p,
                       uint64_t seed, int stop_id, int32_t* done, int slot0, cudaStream_t s)
{
    if (!logits || !next || !count || !pos) return ltl_fail(LTL_ERR_NULL, "sample_advance: null pointer");
    LTL_TRY(check_sampling(temperature, top_k, top_p, V));
    if (B <= 0) return LTL_OK;
    LTL_CUDA("sample_advance launch", ltl_launch(sample_advance_kernel, dim3(B), dim3(V >= 4096 ? 1024 : 256), 0, s, ltl_pdl_enabled(),
                                                 logits, V, next, out_ids, out_stride, count, pos, hist, hist_stride, hist_base,
                                                 temperature, top_k, top_p, (unsigned long long)seed, stop_id, done, slot0));
    return ltl_check_launch("sample_advance");
}

int ltl_sample_rows(const float* logits, int rows, int V, float temperature, int top_k, float top_p, uint64_t seed,
                    const int32_t* counters, int32_t* out, cudaStream_t s)
{
    if (!logits || !out) return ltl_fail(LTL_ERR_NULL, "sample_rows: null pointer");
    if (rows < 0 || V <= 0) return ltl_fail(LTL_ERR_SHAPE, "sample_rows: bad shape %dx%d", rows, V);
    LTL_TRY(check_sampling(temperature, top_k, top_p, V));
    if (rows == 0) return LTL_OK;
    sample_rows_kernel<<<rows, V >= 4096 ? 1024 : 256, 0, s>>>(logits, V, temperature, top_k, top_p, (unsigned long long)seed, counters, out);
    return ltl_check_launch("sample_rows");
}

__global__ void fill_i32_kernel(int32_t* p, int n, int32_t v)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}
int ltl_fill_i32(int32_t* p, int n, int32_t value, cudaStream_t s)
{
    if (!p) return ltl_fail(LTL_ERR_NULL, "fill_i32: null pointer");
    if (n <= 0) return LTL_OK;
    fill_i32_kernel<<<(n + 255) / 256, 256, 0, s>>>(p, n, value);
    return ltl_check_launch("fill_i32");
}

__global__ void count_correct_kernel(const int32_t* __restrict__ pred, const int32_t* __restrict__ tgt,
                                     int n, float* __restrict__ correct)
{
    __shared__ float red[33];
    float c = 0.0f;
    for (int i = threadIdx.x; i < n; i += blockDim.x)
        if (tgt[i] >= 0 && pred[i] == tgt[i]) c += 1.0f;
    c = block_sum(c, red);
    if (threadIdx.x == 0) correct[0] += c;
}
int ltl_count_correct(const int32_t* pred, const int32_t* tgt, int n, float* correct, cudaStream_t s)
{
    if (!pred || !tgt || !correct) return ltl_fail(LTL_ERR_NULL, "count_correct: null pointer");
    count_correct_kernel<<<1, 1024, 0, s>>>(pred, tgt, n, correct);
    return ltl_check_launch("count_correct");
}

__global__ void gather_last_rows_kernel(const float* __restrict__ x, float* __restrict__ out, int T_,
                                        int cols, int last)
{
    const int b = blockIdx.x;
    const float* src = x + ((size_t)b * T_ + last) * cols;
    for (int c = threadIdx.x; c < cols; c += blockDim.x) out[(size_t)b * cols + c] = src[c];
}
int ltl_gather_last_rows(const float* x, float* out, int B, int T, int cols, int last, cudaStream_t s)
{
    if (!x || !out) return ltl_fail(LTL_ERR_NULL, "gather_last_rows: null pointer");
    if (B <= 0) return LTL_OK;
    gather_last_rows_kernel<<<B, 256, 0, s>>>(x, out, T, cols, last);
    return ltl_check_launch("gather_last_rows");
}
