// Kernels that exist only inside the token loop: embedding gather into the fp32 residual
// stream, RMSNorm from the fp32 stream into the GEMM input type, RoPE + KV-cache append,
// decode attention over the device-resident KV cache, greedy pick + position advance.
//
// KV cache layout: K and V are separate arrays [B, H, ctx, hd]; all positions of one
// (sequence, head) are contiguous, so decode attention streams each head's keys and values
// front to back with 16-byte loads.  The reference has no device KV cache (its GPU model
// re-runs a full forward per token, ai/gpu/gpu_transformer.lua:677); the semantics follow the
// CPU model's step() (ai/nn/transformer.lua:297-434).
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

// ------------------------------------------------------------------------------------------
// RoPE of the new token's q and k, and append of k, v to the cache at pos[b].
template <typename T>
__global__ void rope_append_kernel(T* __restrict__ qkv, T* __restrict__ kc, T* __restrict__ vc,
                                   const int32_t* __restrict__ pos, int B, int H, int hd, int ctx,
                                   const float2* __restrict__ cs, int interleaved, int use_rope,
                                   int* __restrict__ err)
{
    const int pairs = hd >> 1;
    const int n = B * H * pairs;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    const int p = idx % pairs, h = (idx / pairs) % H, b = idx / (pairs * H);
    const int D = H * hd;
    const int ps = pos[b];
    if (ps < 0 || ps >= ctx) { if (err) *err = 1; return; }
    float c = 1.0f, sn = 0.0f;
    if (use_rope) { const float2 t = cs[(size_t)ps * pairs + p]; c = t.x; sn = t.y; }
    const int i0 = interleaved ? 2 * p : p, i1 = interleaved ? 2 * p + 1 : p + pairs;
    T* row = qkv + (size_t)b * 3 * D + (size_t)h * hd;
    const float q0 = Cvt<T>::ld(row, i0), q1 = Cvt<T>::ld(row, i1);
    Cvt<T>::st(row, i0, q0 * c - q1 * sn);
    Cvt<T>::st(row, i1, q1 * c + q0 * sn);
    const float k0 = Cvt<T>::ld(row + D, i0), k1 = Cvt<T>::ld(row + D, i1);
    const size_t co = (((size_t)b * H + h) * ctx + ps) * hd;
    Cvt<T>::st(kc, co + i0, k0 * c - k1 * sn);
    Cvt<T>::st(kc, co + i1, k1 * c + k0 * sn);
    vc[co + i0] = row[2 * D + i0];
    vc[co + i1] = row[2 * D + i1];
}

int ltl_rope_append(void* qkv, void* kcache, void* vcache, const int32_t* pos, int B, int H, int hd,
                    int ctx, const float2* cs_table, int interleaved, int use_rope, int dtype,
                    int* err, cudaStream_t s)
{
    if (!qkv || !kcache || !vcache || !pos) return ltl_fail(LTL_ERR_NULL, "rope_append: null pointer");
    if (use_rope && !cs_table) return ltl_fail(LTL_ERR_NULL, "rope_append: missing angle table");
    const int n = B * H * (hd / 2);
    if (n <= 0) return LTL_OK;
    if (dtype == LTL_F32) rope_append_kernel<float><<<(n + 255) / 256, 256, 0, s>>>((float*)qkv, (float*)kcache, (float*)vcache, pos, B, H, hd, ctx, cs_table, interleaved, use_rope, err);
    else if (dtype == LTL_BF16) rope_append_kernel<bf16><<<(n + 255) / 256, 256, 0, s>>>((bf16*)qkv, (bf16*)kcache, (bf16*)vcache, pos, B, H, hd, ctx, cs_table, interleaved, use_rope, err);
    else return ltl_fail(LTL_ERR_DTYPE, "rope_append: dtype %d", dtype);
    return ltl_check_launch("rope_append");
}

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

int ltl_kv_store(const void* qkv, void* kcache, void* vcache, int B, int T, int H, int hd, int ctx,
                 int dtype, cudaStream_t s)
{
    if (!qkv || !kcache || !vcache) return ltl_fail(LTL_ERR_NULL, "kv_store: null pointer");
    if (T > ctx) return ltl_fail(LTL_ERR_SHAPE, "kv_store: %d positions exceed the cache (%d)", T, ctx);
    const uint64_t n = (uint64_t)B * T * H * hd;
    if (n == 0) return LTL_OK;
    unsigned grid = (unsigned)((n + 255) / 256);
    const unsigned cap = (unsigned)ltl_sm_count() * 16;
    if (grid > cap) grid = cap;
    if (dtype == LTL_F32) kv_store_kernel<float><<<grid, 256, 0, s>>>((const float*)qkv, (float*)kcache, (float*)vcache, B, T, H, hd, ctx);
    else if (dtype == LTL_BF16) kv_store_kernel<bf16><<<grid, 256, 0, s>>>((const bf16*)qkv, (bf16*)kcache, (bf16*)vcache, B, T, H, hd, ctx);
    else return ltl_fail(LTL_ERR_DTYPE, "kv_store: dtype %d", dtype);
    return ltl_check_launch("kv_store");
}

// ------------------------------------------------------------------------------------------
// Decode attention.  One CTA (128 threads) per (head, sequence, split).  A key of hd elements
// is covered by GL = hd * sizeof(T) / 16 lanes, each holding one 16-byte packet; the 128 / GL
// lane groups of the CTA walk the keys round-robin, four keys in flight per group, each group
// keeping its own online-softmax state; the groups are merged through shared memory.
// Bytes per (sequence, head): 2 * n * hd * sizeof(T) read once - HBM-bound.
// ------------------------------------------------------------------------------------------
template <typename T, int HD>
__global__ void __launch_bounds__(128)
decode_attn_kernel(const T* __restrict__ qkv, const T* __restrict__ kc, const T* __restrict__ vc,
                   T* __restrict__ out, const int32_t* __restrict__ pos, int H, int ctx, float scale,
                   int splits, float* __restrict__ scratch)
{
    constexpr int N = Vec16<T>::N;
    constexpr int GL = HD / N;           // lanes per key
    constexpr int NG = 128 / GL;         // key groups per CTA
    constexpr int U = 4;                 // keys in flight per group
    static_assert(GL >= 1 && GL <= 32 && (GL & (GL - 1)) == 0, "head_dim / packet must be a power of two <= 32");
    __shared__ float sm_m[NG], sm_l[NG];
    __shared__ float sm_acc[NG][HD + 1];
    const int h = blockIdx.x, b = blockIdx.y, z = blockIdx.z;
    const int D = H * HD;
    const int g = threadIdx.x / GL, r = threadIdx.x % GL;
    int n = pos[b] + 1;
    if (n > ctx) n = ctx;
    if (n < 0) n = 0;
    const int chunk = (n + splits - 1) / splits;
    const int kbeg = z * chunk, kend = min(n, kbeg + chunk);

    float q[N];
    ld16<T>(qkv + (size_t)b * 3 * D + (size_t)h * HD + r * N, q);
#pragma unroll
    for (int i = 0; i < N; ++i) q[i] *= scale;
    const T* kb = kc + ((size_t)b * H + h) * ctx * HD + r * N;
    const T* vb = vc + ((size_t)b * H + h) * ctx * HD + r * N;

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

size_t ltl_decode_attn_scratch_floats(int B, int H, int hd, int splits)
{
    return splits > 1 ? (size_t)B * H * splits * (hd + 2) : 0;
}

template <typename T, int HD>
static int launch_decode_attn(const void* qkv, const void* kc, const void* vc, void* out,
                              const int32_t* pos, int B, int H, int ctx, float scale, int splits,
                              float* scratch, cudaStream_t s)
{
    dim3 grid(H, B, splits);
    decode_attn_kernel<T, HD><<<grid, 128, 0, s>>>((const T*)qkv, (const T*)kc, (const T*)vc, (T*)out,
                                                   pos, H, ctx, scale, splits, scratch);
    if (splits > 1) {
        dim3 g2(H, B);
        decode_attn_combine_kernel<T, HD><<<g2, HD < 32 ? 32 : HD, 0, s>>>(scratch, (T*)out, H, splits);
    }
    return ltl_check_launch("decode_attn");
}

int ltl_decode_attn(const void* qkv, const void* kcache, const void* vcache, void* out,
                    const int32_t* pos, int B, int H, int hd, int ctx, float scale, int dtype,
                    int splits, float* scratch, cudaStream_t s)
{
    if (!qkv || !kcache || !vcache || !out || !pos) return ltl_fail(LTL_ERR_NULL, "decode_attn: null pointer");
    if (B <= 0 || H <= 0) return ltl_fail(LTL_ERR_SHAPE, "decode_attn: bad shape");
    if (B > 65535 || splits > 65535) return ltl_fail(LTL_ERR_SHAPE, "decode_attn: grid too large");
    if (splits < 1) splits = 1;
    if (splits > 1 && !scratch) return ltl_fail(LTL_ERR_NULL, "decode_attn: split-KV needs scratch");
    if (!aligned16(qkv) || !aligned16(kcache) || !aligned16(vcache))
        return ltl_fail(LTL_ERR_ARG, "decode_attn: operands must be 16-byte aligned");
#define DA(TT, HH) return launch_decode_attn<TT, HH>(qkv, kcache, vcache, out, pos, B, H, ctx, scale, splits, scratch, s)
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
                                    int32_t* __restrict__ count, int32_t* __restrict__ pos)
{
    __shared__ float red_v[32];
    __shared__ int red_i[32];
    const int b = blockIdx.x;
    const float* row = logits + (size_t)b * V;
    float best = -INFINITY;
    int bi = 0x7FFFFFFF;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = row[i];
        if (v > best) { best = v; bi = i; }
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
            count[b] = c + 1;
            pos[b] += 1;
        }
    }
}

int ltl_pick_advance(const float* logits, int B, int V, int32_t* next, int32_t* out_ids,
                     int out_stride, int32_t* count, int32_t* pos, cudaStream_t s)
{
    if (!logits || !next || !count || !pos) return ltl_fail(LTL_ERR_NULL, "pick_advance: null pointer");
    if (B <= 0) return LTL_OK;
    pick_advance_kernel<<<B, 256, 0, s>>>(logits, V, next, out_ids, out_stride, count, pos);
    return ltl_check_launch("pick_advance");
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
