// Causal multi-head self-attention over packed q|k|v rows, forward and backward, without
// ever writing the [T, T] score matrix to HBM.
//
// The reference materialises S = QK^T per sequence, runs a separate masked softmax over
// [B*H*T, T] and then P V (ai/gpu/gpu_transformer.lua:338-358), and keeps P for the backward
// (:437-470).  Here one kernel streams 32-key tiles through shared memory with an online
// softmax (running max / sum per query row), and the backward recomputes P from the saved
// log-sum-exp.  HBM traffic drops from O(T^2) to O(T * hd) per head.
//
// Work mapping: one CTA = 16 query rows (or 16 key rows in the dK/dV kernel; 8 at head_dim
// 128) of one (sequence, head); 4 warps, each warp owns 4 (2) rows; inside a tile lane j owns key j for the
// dot products and output dims {lane, lane+32, ...} for the accumulations.  All math fp32.
#include "ops.h"

namespace {

constexpr int KT = 32;            // keys (or queries) per shared-memory tile
// Rows per warp: 4 (16 rows per CTA), 2 for head_dim 128 so that the tiles fit in 48 KB.
template <int HD> struct Rows { static constexpr int RPW = HD >= 128 ? 2 : 4; static constexpr int QB = 4 * RPW; };

template <typename T, int HD>
__device__ __forceinline__ void load_tile(float (*dst)[HD + 1], const T* __restrict__ src, int row0,
                                          int nrows_total, long long row_stride, int tile_rows)
{
    // tile_rows x HD elements, converted to fp32; rows beyond nrows_total are zero.
    for (int idx = threadIdx.x; idx < tile_rows * HD; idx += blockDim.x) {
        const int r = idx / HD, d = idx - r * HD;
        const int gr = row0 + r;
        dst[r][d] = gr < nrows_total ? Cvt<T>::ld(src, (size_t)(gr * row_stride + d)) : 0.0f;
    }
}

// ---------------------------------------------------------------------------------------
// forward
// ---------------------------------------------------------------------------------------
template <typename T, int HD>
__global__ void __launch_bounds__(128)
attn_fwd_kernel(const T* __restrict__ qkv, T* __restrict__ out, float* __restrict__ lse,
                int T_, int H, float scale, int causal)
{
    constexpr int RPW = Rows<HD>::RPW, QB = Rows<HD>::QB;
    constexpr int DPL = (HD + 31) / 32;
    __shared__ float Ks[KT][HD + 1];
    __shared__ float Vs[KT][HD + 1];
    __shared__ __align__(16) float Qs[QB][HD];
    const int D = H * HD, D3 = 3 * D;
    const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * QB;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* base = qkv + (size_t)b * T_ * D3 + h * HD;

    for (int idx = threadIdx.x; idx < QB * HD; idx += blockDim.x) {
        const int r = idx / HD, d = idx - r * HD;
        Qs[r][d] = (q0 + r < T_) ? Cvt<T>::ld(base, (size_t)(q0 + r) * D3 + d) : 0.0f;
    }
    float m[RPW], l[RPW], acc[RPW][DPL];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        m[r] = -INFINITY; l[r] = 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[r][i] = 0.0f;
    }
    const int qlast = min(q0 + QB, T_) - 1;
    const int kend = causal ? qlast + 1 : T_;
    for (int k0 = 0; k0 < kend; k0 += KT) {
        __syncthreads();
        load_tile<T, HD>(Ks, base + D, k0, T_, D3, KT);
        load_tile<T, HD>(Vs, base + 2 * D, k0, T_, D3, KT);
        __syncthreads();
        float s[RPW];
#pragma unroll
        for (int r = 0; r < RPW; ++r) s[r] = 0.0f;
#pragma unroll 4
        for (int d = 0; d < HD; d += 4) {
            const float k0v = Ks[lane][d], k1v = Ks[lane][d + 1], k2v = Ks[lane][d + 2], k3v = Ks[lane][d + 3];
#pragma unroll
            for (int r = 0; r < RPW; ++r) {
                const float4 q = *reinterpret_cast<const float4*>(&Qs[warp * RPW + r][d]);
                s[r] = fmaf(q.x, k0v, fmaf(q.y, k1v, fmaf(q.z, k2v, fmaf(q.w, k3v, s[r]))));
            }
        }
        const int kj = k0 + lane;
        float p[RPW];
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            const int qrow = q0 + warp * RPW + r;
            const bool valid = kj < T_ && qrow < T_ && (!causal || kj <= qrow);
            const float sv = valid ? s[r] * scale : -INFINITY;
            const float mn = fmaxf(m[r], warp_max(sv));
            const float corr = (m[r] == -INFINITY) ? 0.0f : expf(m[r] - mn);
            p[r] = valid ? expf(sv - mn) : 0.0f;
            l[r] = l[r] * corr + warp_sum(p[r]);
            m[r] = mn;
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[r][i] *= corr;
        }
        for (int jj = 0; jj < KT; ++jj) {
            float pj[RPW];
#pragma unroll
            for (int r = 0; r < RPW; ++r) pj[r] = __shfl_sync(0xFFFFFFFFu, p[r], jj);
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int d = lane + 32 * i;
                const float v = d < HD ? Vs[jj][d] : 0.0f;
#pragma unroll
                for (int r = 0; r < RPW; ++r) acc[r][i] = fmaf(pj[r], v, acc[r][i]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        const int qrow = q0 + warp * RPW + r;
        if (qrow >= T_) continue;
        const float inv = l[r] > 0.0f ? 1.0f / l[r] : 0.0f;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = lane + 32 * i;
            if (d < HD) Cvt<T>::st(out, ((size_t)b * T_ + qrow) * D + h * HD + d, acc[r][i] * inv);
        }
        if (lane == 0 && lse) lse[((size_t)b * H + h) * T_ + qrow] = m[r] + logf(fmaxf(l[r], 1e-30f));
    }
}

// ---------------------------------------------------------------------------------------
// backward, part 0: delta[b,h,t] = sum_d dO[t,d] * O[t,d]   (= sum_j dP_tj P_tj)
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void attn_delta_kernel(const T* __restrict__ out, const T* __restrict__ dout,
                                  float* __restrict__ delta, int B, int T_, int H, int HD)
{
    const int w = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (w >= B * T_ * H) return;
    const int h = w % H, row = w / H;              // row = b*T + t
    const size_t off = (size_t)row * H * HD + (size_t)h * HD;
    float acc = 0.0f;
    for (int d = lane; d < HD; d += 32) acc = fmaf(Cvt<T>::ld(out, off + d), Cvt<T>::ld(dout, off + d), acc);
    acc = warp_sum(acc);
    if (lane == 0) {
        const int b = row / T_, t = row - b * T_;
        delta[((size_t)b * H + h) * T_ + t] = acc;
    }
}

// ---------------------------------------------------------------------------------------
// backward, part 1: dQ.  Same walk as the forward; P is rebuilt from lse.
//   dS_ij = P_ij (dP_ij - delta_i) * scale ;  dQ_i = sum_j dS_ij K_j
// ---------------------------------------------------------------------------------------
template <typename T, int HD>
__global__ void __launch_bounds__(128)
attn_bwd_dq_kernel(const T* __restrict__ qkv, const T* __restrict__ dout, const float* __restrict__ lse,
                   const float* __restrict__ delta, T* __restrict__ dqkv, int T_, int H, float scale,
                   int causal)
{
    constexpr int RPW = Rows<HD>::RPW, QB = Rows<HD>::QB;
    constexpr int DPL = (HD + 31) / 32;
    __shared__ float Ks[KT][HD + 1];
    __shared__ float Vs[KT][HD + 1];
    __shared__ __align__(16) float Qs[QB][HD];
    __shared__ __align__(16) float Os[QB][HD];      // dO rows
    const int D = H * HD, D3 = 3 * D;
    const int b = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * QB;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* base = qkv + (size_t)b * T_ * D3 + h * HD;
    const T* dob = dout + (size_t)b * T_ * D + h * HD;
    for (int idx = threadIdx.x; idx < QB * HD; idx += blockDim.x) {
        const int r = idx / HD, d = idx - r * HD;
        const bool ok = q0 + r < T_;
        Qs[r][d] = ok ? Cvt<T>::ld(base, (size_t)(q0 + r) * D3 + d) : 0.0f;
        Os[r][d] = ok ? Cvt<T>::ld(dob, (size_t)(q0 + r) * D + d) : 0.0f;
    }
    float ls[RPW], dl[RPW], acc[RPW][DPL];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        const int qrow = q0 + warp * RPW + r;
        const size_t si = ((size_t)b * H + h) * T_ + min(qrow, T_ - 1);
        ls[r] = lse[si]; dl[r] = delta[si];
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[r][i] = 0.0f;
    }
    const int qlast = min(q0 + QB, T_) - 1;
    const int kend = causal ? qlast + 1 : T_;
    for (int k0 = 0; k0 < kend; k0 += KT) {
        __syncthreads();
        load_tile<T, HD>(Ks, base + D, k0, T_, D3, KT);
        load_tile<T, HD>(Vs, base + 2 * D, k0, T_, D3, KT);
        __syncthreads();
        float s[RPW], dp[RPW];
#pragma unroll
        for (int r = 0; r < RPW; ++r) { s[r] = 0.0f; dp[r] = 0.0f; }
#pragma unroll 4
        for (int d = 0; d < HD; d += 4) {
            const float k0v = Ks[lane][d], k1v = Ks[lane][d + 1], k2v = Ks[lane][d + 2], k3v = Ks[lane][d + 3];
            const float v0 = Vs[lane][d], v1 = Vs[lane][d + 1], v2 = Vs[lane][d + 2], v3 = Vs[lane][d + 3];
#pragma unroll
            for (int r = 0; r < RPW; ++r) {
                const float4 q = *reinterpret_cast<const float4*>(&Qs[warp * RPW + r][d]);
                const float4 o = *reinterpret_cast<const float4*>(&Os[warp * RPW + r][d]);
                s[r] = fmaf(q.x, k0v, fmaf(q.y, k1v, fmaf(q.z, k2v, fmaf(q.w, k3v, s[r]))));
                dp[r] = fmaf(o.x, v0, fmaf(o.y, v1, fmaf(o.z, v2, fmaf(o.w, v3, dp[r]))));
            }
        }
        const int kj = k0 + lane;
        float ds[RPW];
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            const int qrow = q0 + warp * RPW + r;
            const bool valid = kj < T_ && qrow < T_ && (!causal || kj <= qrow);
            const float p = valid ? expf(s[r] * scale - ls[r]) : 0.0f;
            ds[r] = p * (dp[r] - dl[r]) * scale;
        }
        for (int jj = 0; jj < KT; ++jj) {
            float dj[RPW];
#pragma unroll
            for (int r = 0; r < RPW; ++r) dj[r] = __shfl_sync(0xFFFFFFFFu, ds[r], jj);
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int d = lane + 32 * i;
                const float kv = d < HD ? Ks[jj][d] : 0.0f;
#pragma unroll
                for (int r = 0; r < RPW; ++r) acc[r][i] = fmaf(dj[r], kv, acc[r][i]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        const int qrow = q0 + warp * RPW + r;
        if (qrow >= T_) continue;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = lane + 32 * i;
            if (d < HD) Cvt<T>::st(dqkv, ((size_t)b * T_ + qrow) * D3 + h * HD + d, acc[r][i]);
        }
    }
}

// ---------------------------------------------------------------------------------------
// backward, part 2: dK and dV.  One CTA = 16 key rows; query tiles of 32 stream through.
//   dV_j = sum_i P_ij dO_i ;  dK_j = sum_i dS_ij Q_i
// ---------------------------------------------------------------------------------------
template <typename T, int HD>
__global__ void __launch_bounds__(128)
attn_bwd_dkv_kernel(const T* __restrict__ qkv, const T* __restrict__ dout, const float* __restrict__ lse,
                    const float* __restrict__ delta, T* __restrict__ dqkv, int T_, int H, float scale,
                    int causal)
{
    constexpr int RPW = Rows<HD>::RPW, QB = Rows<HD>::QB;
    constexpr int DPL = (HD + 31) / 32;
    __shared__ float Qt[KT][HD + 1];
    __shared__ float Ot[KT][HD + 1];                // dO tile
    __shared__ __align__(16) float Kr[QB][HD];
    __shared__ __align__(16) float Vr[QB][HD];
    __shared__ float lt[KT], dt[KT];
    const int D = H * HD, D3 = 3 * D;
    const int b = blockIdx.z, h = blockIdx.y, j0 = blockIdx.x * QB;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* base = qkv + (size_t)b * T_ * D3 + h * HD;
    const T* dob = dout + (size_t)b * T_ * D + h * HD;
    for (int idx = threadIdx.x; idx < QB * HD; idx += blockDim.x) {
        const int r = idx / HD, d = idx - r * HD;
        const bool ok = j0 + r < T_;
        Kr[r][d] = ok ? Cvt<T>::ld(base + D, (size_t)(j0 + r) * D3 + d) : 0.0f;
        Vr[r][d] = ok ? Cvt<T>::ld(base + 2 * D, (size_t)(j0 + r) * D3 + d) : 0.0f;
    }
    float dk[RPW][DPL], dv[RPW][DPL];
#pragma unroll
    for (int r = 0; r < RPW; ++r)
#pragma unroll
        for (int i = 0; i < DPL; ++i) { dk[r][i] = 0.0f; dv[r][i] = 0.0f; }
    const int istart = causal ? (j0 / KT) * KT : 0;   // first query tile that can see key j0
    for (int i0 = istart; i0 < T_; i0 += KT) {
        __syncthreads();
        load_tile<T, HD>(Qt, base, i0, T_, D3, KT);
        load_tile<T, HD>(Ot, dob, i0, T_, D, KT);
        if (threadIdx.x < KT) {
            const int qi = min(i0 + (int)threadIdx.x, T_ - 1);
            lt[threadIdx.x] = lse[((size_t)b * H + h) * T_ + qi];
            dt[threadIdx.x] = delta[((size_t)b * H + h) * T_ + qi];
        }
        __syncthreads();
        float s[RPW], dp[RPW];
#pragma unroll
        for (int r = 0; r < RPW; ++r) { s[r] = 0.0f; dp[r] = 0.0f; }
#pragma unroll 4
        for (int d = 0; d < HD; d += 4) {
            const float q0v = Qt[lane][d], q1v = Qt[lane][d + 1], q2v = Qt[lane][d + 2], q3v = Qt[lane][d + 3];
            const float o0 = Ot[lane][d], o1 = Ot[lane][d + 1], o2 = Ot[lane][d + 2], o3 = Ot[lane][d + 3];
#pragma unroll
            for (int r = 0; r < RPW; ++r) {
                const float4 k = *reinterpret_cast<const float4*>(&Kr[warp * RPW + r][d]);
                const float4 v = *reinterpret_cast<const float4*>(&Vr[warp * RPW + r][d]);
                s[r] = fmaf(k.x, q0v, fmaf(k.y, q1v, fmaf(k.z, q2v, fmaf(k.w, q3v, s[r]))));
                dp[r] = fmaf(v.x, o0, fmaf(v.y, o1, fmaf(v.z, o2, fmaf(v.w, o3, dp[r]))));
            }
        }
        const int qi = i0 + lane;
        float p[RPW], ds[RPW];
#pragma unroll
        for (int r = 0; r < RPW; ++r) {
            const int kj = j0 + warp * RPW + r;
            const bool valid = qi < T_ && kj < T_ && (!causal || kj <= qi);
            p[r] = valid ? expf(s[r] * scale - lt[lane]) : 0.0f;
            ds[r] = p[r] * (dp[r] - dt[lane]) * scale;
        }
        for (int ii = 0; ii < KT; ++ii) {
            float pi[RPW], di[RPW];
#pragma unroll
            for (int r = 0; r < RPW; ++r) {
                pi[r] = __shfl_sync(0xFFFFFFFFu, p[r], ii);
                di[r] = __shfl_sync(0xFFFFFFFFu, ds[r], ii);
            }
#pragma unroll
            for (int i = 0; i < DPL; ++i) {
                const int d = lane + 32 * i;
                const float ov = d < HD ? Ot[ii][d] : 0.0f;
                const float qv = d < HD ? Qt[ii][d] : 0.0f;
#pragma unroll
                for (int r = 0; r < RPW; ++r) {
                    dv[r][i] = fmaf(pi[r], ov, dv[r][i]);
                    dk[r][i] = fmaf(di[r], qv, dk[r][i]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
        const int kj = j0 + warp * RPW + r;
        if (kj >= T_) continue;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int d = lane + 32 * i;
            if (d < HD) {
                const size_t o = ((size_t)b * T_ + kj) * D3 + h * HD + d;
                Cvt<T>::st(dqkv, o + D, dk[r][i]);
                Cvt<T>::st(dqkv, o + 2 * D, dv[r][i]);
            }
        }
    }
}

template <typename T, int HD>
int launch_fwd(const void* qkv, void* out, float* lse, int B, int T_, int H, float scale, int causal, cudaStream_t s)
{
    dim3 grid((T_ + Rows<HD>::QB - 1) / Rows<HD>::QB, H, B);
    attn_fwd_kernel<T, HD><<<grid, 128, 0, s>>>((const T*)qkv, (T*)out, lse, T_, H, scale, causal);
    return ltl_check_launch("attn_fwd");
}
template <typename T, int HD>
int launch_bwd(const void* qkv, const void* out, const void* dout, const float* lse, float* delta,
               void* dqkv, int B, int T_, int H, float scale, int causal, cudaStream_t s)
{
    const int nw = B * T_ * H;
    attn_delta_kernel<T><<<(nw * 32 + 255) / 256, 256, 0, s>>>((const T*)out, (const T*)dout, delta, B, T_, H, HD);
    dim3 grid((T_ + Rows<HD>::QB - 1) / Rows<HD>::QB, H, B);
    attn_bwd_dq_kernel<T, HD><<<grid, 128, 0, s>>>((const T*)qkv, (const T*)dout, lse, delta, (T*)dqkv, T_, H, scale, causal);
    attn_bwd_dkv_kernel<T, HD><<<grid, 128, 0, s>>>((const T*)qkv, (const T*)dout, lse, delta, (T*)dqkv, T_, H, scale, causal);
    return ltl_check_launch("attn_bwd");
}

}  // namespace

#define ATTN_DISPATCH(FN, ...)                                                              \
    do {                                                                                    \
        if (dtype == LTL_F32) {                                                             \
            if (hd == 16) return FN<float, 16>(__VA_ARGS__);                                \
            if (hd == 32) return FN<float, 32>(__VA_ARGS__);                                \
            if (hd == 64) return FN<float, 64>(__VA_ARGS__);                                \
            if (hd == 128) return FN<float, 128>(__VA_ARGS__);                              \
        } else if (dtype == LTL_BF16) {                                                     \
            if (hd == 16) return FN<bf16, 16>(__VA_ARGS__);                                 \
            if (hd == 32) return FN<bf16, 32>(__VA_ARGS__);                                 \
            if (hd == 64) return FN<bf16, 64>(__VA_ARGS__);                                 \
            if (hd == 128) return FN<bf16, 128>(__VA_ARGS__);                               \
        } else return ltl_fail(LTL_ERR_DTYPE, "attention: dtype %d not supported", dtype);  \
        return ltl_fail(LTL_ERR_UNSUPPORTED, "attention: head_dim %d not in {16,32,64,128}", hd); \
    } while (0)

int ltl_attn_fwd(const void* qkv, void* out, float* lse, int B, int T, int H, int hd, float scale,
                 int causal, int dtype, cudaStream_t s)
{
    if (!qkv || !out) return ltl_fail(LTL_ERR_NULL, "attn_fwd: null pointer");
    if (B <= 0 || T <= 0 || H <= 0) return ltl_fail(LTL_ERR_SHAPE, "attn_fwd: bad shape");
    if (B > 65535 || H > 65535) return ltl_fail(LTL_ERR_SHAPE, "attn_fwd: grid too large");
    ATTN_DISPATCH(launch_fwd, qkv, out, lse, B, T, H, scale, causal, s);
}

// delta[b, h, t] = sum_d dO[t, d] O[t, d], the row term of the softmax backward.
int ltl_attn_delta(const void* out, const void* dout, float* delta, int B, int T, int H, int hd, int dtype, cudaStream_t s)
{
    const int nw = B * T * H;
    if (dtype == LTL_F32) attn_delta_kernel<float><<<(nw * 32 + 255) / 256, 256, 0, s>>>((const float*)out, (const float*)dout, delta, B, T, H, hd);
    else if (dtype == LTL_BF16) attn_delta_kernel<bf16><<<(nw * 32 + 255) / 256, 256, 0, s>>>((const bf16*)out, (const bf16*)dout, delta, B, T, H, hd);
    else return ltl_fail(LTL_ERR_DTYPE, "attn_delta: dtype %d", dtype);
    return ltl_check_launch("attn_delta");
}

int ltl_attn_bwd(const void* qkv, const void* out, const void* dout, const float* lse, float* delta,
                 void* dqkv, int B, int T, int H, int hd, float scale, int causal, int dtype,
                 cudaStream_t s)
{
    if (!qkv || !out || !dout || !lse || !delta || !dqkv) return ltl_fail(LTL_ERR_NULL, "attn_bwd: null pointer");
    if (B <= 0 || T <= 0 || H <= 0) return ltl_fail(LTL_ERR_SHAPE, "attn_bwd: bad shape");
    if (B > 65535 || H > 65535) return ltl_fail(LTL_ERR_SHAPE, "attn_bwd: grid too large");
    ATTN_DISPATCH(launch_bwd, qkv, out, dout, lse, delta, dqkv, B, T, H, scale, causal, s);
}
