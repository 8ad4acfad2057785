// Bandwidth-bound kernels of the token loop: RMSNorm fwd/bwd, masked softmax fwd/bwd,
// SwiGLU fwd/bwd, RoPE, embedding gather / scatter-add, fused cross-entropy (+argmax),
// row argmax, norm / clip / sum reductions, element-wise ops, AdamW and SGD.
//
// Design: every kernel moves 16-byte packets per thread (4 fp32 or 8 bf16/f16), row
// reductions are warp shuffles, a row that fits in registers is read from HBM exactly
// once.  The roofline that bounds all of them is HBM bandwidth.  Shapes that break the
// 16-byte rules (odd widths, unaligned bases) take a scalar kernel with the same math.
#include "ops.h"

#define DISPATCH_T(dt, ...)                                                          \
    do {                                                                             \
        if ((dt) == LTL_F32) { typedef float T; __VA_ARGS__; }                       \
        else if ((dt) == LTL_BF16) { typedef bf16 T; __VA_ARGS__; }                  \
        else if ((dt) == LTL_F16) { typedef __half T; __VA_ARGS__; }                 \
        else return ltl_fail(LTL_ERR_DTYPE, "unknown dtype %d", (int)(dt));          \
    } while (0)

#define DISPATCH_CH(ch, ...)                                                         \
    do {                                                                             \
        if ((ch) <= 1) { constexpr int CH = 1; __VA_ARGS__; }                        \
        else if ((ch) <= 2) { constexpr int CH = 2; __VA_ARGS__; }                   \
        else if ((ch) <= 4) { constexpr int CH = 4; __VA_ARGS__; }                   \
        else if ((ch) <= 8) { constexpr int CH = 8; __VA_ARGS__; }                   \
        else { constexpr int CH = 16; __VA_ARGS__; }                                 \
    } while (0)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static inline unsigned grid1d(uint64_t work_items, int block, int per_sm = 16)
{
    uint64_t g = (work_items + block - 1) / block;
    const uint64_t cap = (uint64_t)ltl_sm_count() * per_sm;
    if (g > cap) g = cap;
    if (g < 1) g = 1;
    return (unsigned)g;
}
constexpr int ROW_WARPS = 4;   // warps per CTA in the warp-per-row kernels
constexpr int MAX_CH = 16;

// Can a row of `cols` elements of `esz` bytes be held by one warp in registers?
static inline int row_chunks(int cols, size_t esz)
{
    const int n = (int)(16 / esz);
    if (cols % n) return 0;
    const int ch = (cols / n + 31) / 32;
    return ch <= MAX_CH ? ch : 0;
}

// ------------------------------------------------------------------------------------------
// RMSNorm forward: y = x * rsqrt(mean(x^2) + eps) * w
// (reference kernel: cuda/luaTL_core.cu:1092; CPU: ai/core/tensor2.lua:609)
// ------------------------------------------------------------------------------------------
template <typename T, int CH>
__global__ void __launch_bounds__(ROW_WARPS * 32)
rmsnorm_warp_kernel(const T* __restrict__ x, const T* __restrict__ w, T* __restrict__ out,
                    int rows, int cols, float eps)
{
    constexpr int N = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
    if (row >= rows) return;
    const T* xr = x + (size_t)row * cols;
    float v[CH][N];
    float ss = 0.0f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int e = (c * 32 + lane) * N;
        if (e < cols) {
            ld16<T>(xr + e, v[c]);
#pragma unroll
            for (int i = 0; i < N; ++i) ss = fmaf(v[c][i], v[c][i], ss);
        }
    }
    ss = warp_sum(ss);
    const float sc = 1.0f / sqrtf(ss / (float)cols + eps);
    T* orow = out + (size_t)row * cols;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int e = (c * 32 + lane) * N;
        if (e < cols) {
            float g[N];
            if (w) ld16<T>(w + e, g);
#pragma unroll
            for (int i = 0; i < N; ++i) v[c][i] = v[c][i] * sc * (w ? g[i] : 1.0f);
            st16<T>(orow + e, v[c]);
        }
    }
}

template <typename T>
__global__ void rmsnorm_block_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                     T* __restrict__ out, int rows, int cols, float eps)
{
    __shared__ float red[33];
    const T* xr = x + (size_t)blockIdx.x * cols;
    T* orow = out + (size_t)blockIdx.x * cols;
    float ss = 0.0f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        const float v = Cvt<T>::ld(xr, i);
        ss = fmaf(v, v, ss);
    }
    ss = block_sum(ss, red);
    const float sc = 1.0f / sqrtf(ss / (float)cols + eps);
    for (int i = threadIdx.x; i < cols; i += blockDim.x)
        Cvt<T>::st(orow, i, Cvt<T>::ld(xr, i) * sc * (w ? Cvt<T>::ld(w, i) : 1.0f));
}

int ltl_rmsnorm(const void* x, const void* w, void* out, int rows, int cols, float eps,
                int dtype, cudaStream_t s)
{
    if (!x || !out) return ltl_fail(LTL_ERR_NULL, "rmsnorm: null pointer");
    if (rows < 0 || cols <= 0) return ltl_fail(LTL_ERR_SHAPE, "rmsnorm: bad shape %dx%d", rows, cols);
    if (rows == 0) return LTL_OK;
    const int ch = row_chunks(cols, ltl_dtype_size(dtype));
    const bool vec = ch && aligned16(x) && aligned16(out) && (!w || aligned16(w));
    DISPATCH_T(dtype, {
        if (vec) {
            DISPATCH_CH(ch, rmsnorm_warp_kernel<T, CH><<<(rows + ROW_WARPS - 1) / ROW_WARPS,
                             ROW_WARPS * 32, 0, s>>>((const T*)x, (const T*)w, (T*)out, rows, cols, eps));
        } else {
            rmsnorm_block_kernel<T><<<rows, 256, 0, s>>>((const T*)x, (const T*)w, (T*)out, rows, cols, eps);
        }
    });
    return ltl_check_launch("rmsnorm");
}

// ------------------------------------------------------------------------------------------
// RMSNorm backward (reference: cuda/luaTL_train.cu:489; CPU: ai/core/tensor2.lua:641)
//   dx_i = s*g_i*dy_i - x_i * s^3/N * sum_j dy_j g_j x_j ;  dgamma_i += sum_rows dy_i x_i s
// dgamma is reduced without atomics: every warp keeps the partial sums of the columns it
// owns in registers while it walks its rows, writes one partial row to scratch, and a
// second kernel adds the partial rows into dgamma in a fixed order.
// ------------------------------------------------------------------------------------------
template <typename T, int CH>
__global__ void __launch_bounds__(ROW_WARPS * 32)
rmsnorm_bwd_warp_kernel(const T* __restrict__ x, const T* __restrict__ g,
                        const T* __restrict__ dy, T* __restrict__ dx,
                        float* __restrict__ partial, int rows, int cols, float eps)
{
    constexpr int N = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const int wglobal = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
    const int wtotal = gridDim.x * ROW_WARPS;
    float gam[CH][N], dg[CH][N];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int e = (c * 32 + lane) * N;
#pragma unroll
        for (int i = 0; i < N; ++i) { gam[c][i] = 1.0f; dg[c][i] = 0.0f; }
        if (g && e < cols) ld16<T>(g + e, gam[c]);
    }
    for (int row = wglobal; row < rows; row += wtotal) {
        const T* xr = x + (size_t)row * cols;
        const T* dyr = dy + (size_t)row * cols;
        float xv[CH][N], dv[CH][N];
        float ss = 0.0f, dot = 0.0f;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const int e = (c * 32 + lane) * N;
            if (e < cols) {
                ld16<T>(xr + e, xv[c]);
                ld16<T>(dyr + e, dv[c]);
#pragma unroll
                for (int i = 0; i < N; ++i) {
                    ss = fmaf(xv[c][i], xv[c][i], ss);
                    dot = fmaf(dv[c][i] * gam[c][i], xv[c][i], dot);
                }
            }
        }
        ss = warp_sum(ss);
        dot = warp_sum(dot);
        const float sc = 1.0f / sqrtf(ss / (float)cols + eps);
        const float coef = sc * sc * sc / (float)cols * dot;
        T* dxr = dx + (size_t)row * cols;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const int e = (c * 32 + lane) * N;
            if (e < cols) {
                float o[N];
#pragma unroll
                for (int i = 0; i < N; ++i) {
                    o[i] = sc * gam[c][i] * dv[c][i] - coef * xv[c][i];
                    dg[c][i] = fmaf(dv[c][i] * xv[c][i], sc, dg[c][i]);
                }
                st16<T>(dxr + e, o);
            }
        }
    }
    if (partial) {
        float* pr = partial + (size_t)wglobal * cols;
#pragma unroll
        for (int c = 0; c < CH; ++c) {
            const int e = (c * 32 + lane) * N;
            if (e < cols) {
#pragma unroll
                for (int i = 0; i < N; i += 4)
                    *reinterpret_cast<float4*>(pr + e + i) =
                        make_float4(dg[c][i], dg[c][i + 1], dg[c][i + 2], dg[c][i + 3]);
            }
        }
    }
}

// dgamma[c] += sum_p partial[p][c]; 32 columns per CTA, 8 row slices per column.
__global__ void colsum_partials_kernel(const float* __restrict__ partial, int nparts, int cols,
                                       float* __restrict__ out)
{
    __shared__ float red[8][33];
    const int c = blockIdx.x * 32 + (threadIdx.x & 31);
    const int slice = threadIdx.x >> 5;
    float acc = 0.0f;
    if (c < cols)
        for (int p = slice; p < nparts; p += 8) acc += partial[(size_t)p * cols + c];
    red[slice][threadIdx.x & 31] = acc;
    __syncthreads();
    if (slice == 0 && c < cols) {
        float t = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) t += red[i][threadIdx.x];
        out[c] += t;
    }
}

template <typename T>
__global__ void rmsnorm_bwd_block_kernel(const T* __restrict__ x, const T* __restrict__ g,
                                         const T* __restrict__ dy, T* __restrict__ dx,
                                         float* __restrict__ dgamma, int rows, int cols, float eps)
{
    __shared__ float red[33];
    const size_t base = (size_t)blockIdx.x * cols;
    float ss = 0.0f, dot = 0.0f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        const float v = Cvt<T>::ld(x, base + i);
        ss = fmaf(v, v, ss);
        dot += Cvt<T>::ld(dy, base + i) * (g ? Cvt<T>::ld(g, i) : 1.0f) * v;
    }
    ss = block_sum(ss, red);
    dot = block_sum(dot, red);
    const float sc = 1.0f / sqrtf(ss / (float)cols + eps);
    const float coef = sc * sc * sc / (float)cols * dot;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        const float xi = Cvt<T>::ld(x, base + i), dyi = Cvt<T>::ld(dy, base + i);
        Cvt<T>::st(dx, base + i, sc * (g ? Cvt<T>::ld(g, i) : 1.0f) * dyi - coef * xi);
        if (dgamma) atomicAdd(&dgamma[i], dyi * xi * sc);
    }
}

static inline int rmsnorm_bwd_grid(int rows)
{
    int g = (rows + ROW_WARPS * 4 - 1) / (ROW_WARPS * 4);   // at least 4 rows per warp
    const int cap = ltl_sm_count() * 2;
    if (g > cap) g = cap;
    return g < 1 ? 1 : g;
}
size_t ltl_rmsnorm_bwd_scratch_floats(int cols)
{
    return (size_t)ltl_sm_count() * 2 * ROW_WARPS * (size_t)cols;
}

// The operand tests of the launcher below, without the scratch: does this call take the warp-per-row kernel?
static bool rmsnorm_bwd_takes_warp_kernel(const void* x, const void* gamma, const void* dy, const void* dx, int cols, int dtype)
{
    return row_chunks(cols, ltl_dtype_size(dtype)) && aligned16(x) && aligned16(dy) && aligned16(dx) &&
           (!gamma || aligned16(gamma));
}

int ltl_rmsnorm_bwd(const void* x, const void* gamma, const void* dy, void* dx, float* dgamma,
                    int rows, int cols, float eps, int dtype, float* scratch, cudaStream_t s)
{
    if (!x || !dy || !dx) return ltl_fail(LTL_ERR_NULL, "rmsnorm_bwd: null pointer");
    if (rows < 0 || cols <= 0) return ltl_fail(LTL_ERR_SHAPE, "rmsnorm_bwd: bad shape %dx%d", rows, cols);
    if (rows == 0) return LTL_OK;
    const int ch = row_chunks(cols, ltl_dtype_size(dtype));
    const bool vec = ch && aligned16(x) && aligned16(dy) && aligned16(dx) &&
                     (!gamma || aligned16(gamma)) && (!dgamma || (scratch && aligned16(scratch)));
    const int grid = rmsnorm_bwd_grid(rows);
    DISPATCH_T(dtype, {
        if (vec) {
            DISPATCH_CH(ch, rmsnorm_bwd_warp_kernel<T, CH><<<grid, ROW_WARPS * 32, 0, s>>>(
                (const T*)x, (const T*)gamma, (const T*)dy, (T*)dx, dgamma ? scratch : nullptr,
                rows, cols, eps));
            if (dgamma)
                colsum_partials_kernel<<<(cols + 31) / 32, 256, 0, s>>>(scratch, grid * ROW_WARPS,
                                                                        cols, dgamma);
        } else {
            rmsnorm_bwd_block_kernel<T><<<rows, 256, 0, s>>>((const T*)x, (const T*)gamma,
                (const T*)dy, (T*)dx, dgamma, rows, cols, eps);
        }
    });
    return ltl_check_launch("rmsnorm_bwd");
}

// RMSNorm backward for wide fp32 rows fused with what follows it in the mixed-precision backward: the input
// gradient is ADDED to the residual-stream gradient (res += dx, in place) and the updated row is also written as
// bf16 (the next GEMMs' operand).  A persistent grid of 256-thread CTAs walks the rows; a thread owns CHT 16-byte
// chunks of every row (x, dy, gamma and its share of dgamma stay in registers: 32 floats at 2048 columns against
// 256 in the warp-per-row kernel), the two row sums cross the CTA through shared memory, and every CTA leaves one
// partial dgamma row in scratch for colsum_partials_kernel.
template <int CHT>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_res_kernel(const float* __restrict__ x, const float* __restrict__ g, const float* __restrict__ dy,
                       float* __restrict__ res, bf16* __restrict__ res_bf16, float* __restrict__ partial,
                       int rows, int cols, float eps)
{
    __shared__ float red[2][8];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float4 gam[CHT], dg[CHT];
#pragma unroll
    for (int c = 0; c < CHT; ++c) {
        const int e = (c * 256 + tid) * 4;
        gam[c] = (g && e < cols) ? *reinterpret_cast<const float4*>(g + e) : make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        dg[c] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    for (int row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t base = (size_t)row * cols;
        float4 xv[CHT], dv[CHT], rv[CHT];
        float ss = 0.0f, dot = 0.0f;
#pragma unroll
        for (int c = 0; c < CHT; ++c) {
            const int e = (c * 256 + tid) * 4;
            xv[c] = dv[c] = rv[c] = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
            if (e < cols) {
                xv[c] = *reinterpret_cast<const float4*>(x + base + e);
                dv[c] = *reinterpret_cast<const float4*>(dy + base + e);
                rv[c] = *reinterpret_cast<const float4*>(res + base + e);
            }
            ss += xv[c].x * xv[c].x + xv[c].y * xv[c].y + xv[c].z * xv[c].z + xv[c].w * xv[c].w;
            dot += dv[c].x * gam[c].x * xv[c].x + dv[c].y * gam[c].y * xv[c].y + dv[c].z * gam[c].z * xv[c].z + dv[c].w * gam[c].w * xv[c].w;
        }
        ss = warp_sum(ss);
        dot = warp_sum(dot);
        __syncthreads();                                  // the previous row's sums have been read
        if (lane == 0) { red[0][warp] = ss; red[1][warp] = dot; }
        __syncthreads();
        ss = 0.0f; dot = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) { ss += red[0][w]; dot += red[1][w]; }
        const float sc = 1.0f / sqrtf(ss / (float)cols + eps);
        const float coef = sc * sc * sc / (float)cols * dot;
#pragma unroll
        for (int c = 0; c < CHT; ++c) {
            const int e = (c * 256 + tid) * 4;
            if (e < cols) {
                float4 o;
                o.x = rv[c].x + (sc * gam[c].x * dv[c].x - coef * xv[c].x);
                o.y = rv[c].y + (sc * gam[c].y * dv[c].y - coef * xv[c].y);
                o.z = rv[c].z + (sc * gam[c].z * dv[c].z - coef * xv[c].z);
                o.w = rv[c].w + (sc * gam[c].w * dv[c].w - coef * xv[c].w);
                dg[c].x = fmaf(dv[c].x * xv[c].x, sc, dg[c].x); dg[c].y = fmaf(dv[c].y * xv[c].y, sc, dg[c].y);
                dg[c].z = fmaf(dv[c].z * xv[c].z, sc, dg[c].z); dg[c].w = fmaf(dv[c].w * xv[c].w, sc, dg[c].w);
                *reinterpret_cast<float4*>(res + base + e) = o;
                if (res_bf16) {
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
                    uint2 pk;
                    pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                    pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(res_bf16 + base + e) = pk;
                }
            }
        }
    }
    if (partial) {
        float* pr = partial + (size_t)blockIdx.x * cols;
#pragma unroll
        for (int c = 0; c < CHT; ++c) {
            const int e = (c * 256 + tid) * 4;
            if (e < cols) *reinterpret_cast<float4*>(pr + e) = dg[c];
        }
    }
}

// res += rmsnorm_bwd(x, gamma, dy); res_bf16 = bf16(res) (optional); dgamma += ... (optional, needs scratch of
// ltl_rmsnorm_bwd_scratch_floats(cols)).  fp32, cols a multiple of 4 and at most 4096.
int ltl_rmsnorm_bwd_residual(const float* x, const float* gamma, const float* dy, float* res, bf16* res_bf16, float* dgamma,
                             int rows, int cols, float eps, float* scratch, cudaStream_t s)
{
    if (!x || !dy || !res) return ltl_fail(LTL_ERR_NULL, "rmsnorm_bwd_residual: null pointer");
    if (rows < 0 || cols <= 0 || cols % 4 || cols > 4096) return ltl_fail(LTL_ERR_SHAPE, "rmsnorm_bwd_residual: bad shape %dx%d", rows, cols);
    if (!aligned16(x) || !aligned16(dy) || !aligned16(res) || (gamma && !aligned16(gamma)) || (res_bf16 && !aligned16(res_bf16)) ||
        (dgamma && (!scratch || !aligned16(scratch))))
        return ltl_fail(LTL_ERR_ARG, "rmsnorm_bwd_residual: operands must be 16-byte aligned (and scratch given with dgamma)");
    if (rows == 0) return LTL_OK;
    int grid = 2 * ltl_sm_count();
    if (grid > rows) grid = rows;
    float* partial = dgamma ? scratch : nullptr;
    const int cht = (cols + 1023) / 1024;
    if (cht <= 1) rmsnorm_bwd_res_kernel<1><<<grid, 256, 0, s>>>(x, gamma, dy, res, res_bf16, partial, rows, cols, eps);
    else if (cht == 2) rmsnorm_bwd_res_kernel<2><<<grid, 256, 0, s>>>(x, gamma, dy, res, res_bf16, partial, rows, cols, eps);
    else rmsnorm_bwd_res_kernel<4><<<grid, 256, 0, s>>>(x, gamma, dy, res, res_bf16, partial, rows, cols, eps);
    if (dgamma) colsum_partials_kernel<<<(cols + 31) / 32, 256, 0, s>>>(scratch, grid, cols, dgamma);
    return ltl_check_launch("rmsnorm_bwd_residual");
}

// ------------------------------------------------------------------------------------------
// Masked softmax forward / backward (reference: cuda/luaTL_train.cu:545,589).
//   v = x*scale + bias ; columns > (row % group) + mask_offset are masked when causal.
// ------------------------------------------------------------------------------------------
template <typename T, int CH>
__global__ void __launch_bounds__(ROW_WARPS * 32)
softmax_warp_kernel(const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ out,
                    int rows, int cols, float scale, int causal, int group, int mask_offset)
{
    constexpr int N = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lrow = group > 0 ? row % group : row;
    const int limit = causal ? lrow + mask_offset : cols - 1;
    const T* xr = x + (size_t)row * cols;
    float v[CH][N];
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int e = (c * 32 + lane) * N;
        if (e < cols) {
            ld16<T>(xr + e, v[c]);
            float b[N];
            if (bias) ld16<T>(bias + e, b);
#pragma unroll
            for (int i = 0; i < N; ++i) {
                v[c][i] = (e + i <= limit) ? v[c][i] * scale + (bias ? b[i] : 0.0f) : -INFINITY;
                mx = fmaxf(mx, v[c][i]);
            }
        }
    }
    mx = warp_max(mx);
    const float base = (mx == -INFINITY) ? 0.0f : mx;
    float sum = 0.0f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int e = (c * 32 + lane) * N;
        if (e < cols) {
#pragma unroll
            for (int i = 0; i < N; ++i) {
                v[c][i] = (e + i <= limit) ? __expf(v[c][i] - base) : 0.0f;
                sum += v[c][i];
            }
        }
    }
    sum = warp_sum(sum);
    const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
    T* orow = out + (size_t)row * cols;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int e = (c * 32 + lane) * N;
        if (e < cols) {
#pragma unroll
            for (int i = 0; i < N; ++i) v[c][i] *= inv;
            st16<T>(orow + e, v[c]);
        }
    }
}

// Wide rows (more than four 16-byte packets per lane of a warp): one CTA of TH threads per row, PT packets per
// thread (two, so that a thread has 32 bytes in flight).  The warp-per-row form keeps 64 values per lane in registers there, which leaves 16 warps per SM and
// the loads of a row exposed (34 % of DRAM throughput at 2048 columns); this form runs at full occupancy.
template <typename T, int PT, int TH>
__global__ void __launch_bounds__(TH)
softmax_cta_kernel(const T* __restrict__ x, const T* __restrict__ bias, T* __restrict__ out,
                   int rows, int cols, float scale, int causal, int group, int mask_offset)
{
    constexpr int N = Vec16<T>::N;
    __shared__ float red[33];
    const int row = blockIdx.x;
    const int lrow = group > 0 ? row % group : row;
    const int limit = causal ? lrow + mask_offset : cols - 1;
    const T* xr = x + (size_t)row * cols;
    float v[PT][N];
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < PT; ++c) {
        const int e = (c * TH + threadIdx.x) * N;
        if (e < cols) {
            ld16<T>(xr + e, v[c]);
            float b[N];
            if (bias) ld16<T>(bias + e, b);
#pragma unroll
            for (int i = 0; i < N; ++i) {
                v[c][i] = (e + i <= limit) ? v[c][i] * scale + (bias ? b[i] : 0.0f) : -INFINITY;
                mx = fmaxf(mx, v[c][i]);
            }
        }
    }
    mx = block_max(mx, red);
    const float base = (mx == -INFINITY) ? 0.0f : mx;
    float sum = 0.0f;
#pragma unroll
    for (int c = 0; c < PT; ++c) {
        const int e = (c * TH + threadIdx.x) * N;
        if (e < cols) {
#pragma unroll
            for (int i = 0; i < N; ++i) {
                v[c][i] = (e + i <= limit) ? __expf(v[c][i] - base) : 0.0f;
                sum += v[c][i];
            }
        }
    }
    sum = block_sum(sum, red);
    const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
    T* orow = out + (size_t)row * cols;
#pragma unroll
    for (int c = 0; c < PT; ++c) {
        const int e = (c * TH + threadIdx.x) * N;
        if (e < cols) {
#pragma unroll
            for (int i = 0; i < N; ++i) v[c][i] *= inv;
            st16<T>(orow + e, v[c]);
        }
    }
}

template <typename T>
__global__ void softmax_block_kernel(const T* __restrict__ x, const T* __restrict__ bias,
                                     T* __restrict__ out, int rows, int cols, float scale,
                                     int causal, int group, int mask_offset)
{
    __shared__ float red[33];
    const int row = blockIdx.x;
    const int lrow = group > 0 ? row % group : row;
    const int limit = causal ? lrow + mask_offset : cols - 1;
    const size_t base_i = (size_t)row * cols;
    float mx = -INFINITY;
    for (int i = threadIdx.x; i < cols; i += blockDim.x)
        if (i <= limit)
            mx = fmaxf(mx, Cvt<T>::ld(x, base_i + i) * scale + (bias ? Cvt<T>::ld(bias, i) : 0.0f));
    mx = block_max(mx, red);
    const float base = (mx == -INFINITY) ? 0.0f : mx;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x)
        if (i <= limit)
            sum += expf(Cvt<T>::ld(x, base_i + i) * scale + (bias ? Cvt<T>::ld(bias, i) : 0.0f) - base);
    sum = block_sum(sum, red);
    const float inv = sum > 0.0f ? 1.0f / sum : 0.0f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        float e = 0.0f;
        if (i <= limit)
            e = expf(Cvt<T>::ld(x, base_i + i) * scale + (bias ? Cvt<T>::ld(bias, i) : 0.0f) - base) * inv;
        Cvt<T>::st(out, base_i + i, e);
    }
}

int ltl_softmax(const void* x, const void* bias, void* out, int rows, int cols, float scale,
                int causal, int group, int mask_offset, int dtype, cudaStream_t s)
{
    if (!x || !out) return ltl_fail(LTL_ERR_NULL, "softmax: null pointer");
    if (rows < 0 || cols <= 0) return ltl_fail(LTL_ERR_SHAPE, "softmax: bad shape %dx%d", rows, cols);
    if (rows == 0) return LTL_OK;
    const int ch = row_chunks(cols, ltl_dtype_size(dtype));
    const bool vec = ch && aligned16(x) && aligned16(out) && (!bias || aligned16(bias));
    DISPATCH_T(dtype, {
        if (vec && ch > 4) {
            // ch packets per lane of a warp = 32 ch packets per row: two per thread of a 128- or 256-thread CTA
            if (ch <= 8) softmax_cta_kernel<T, 2, 128><<<rows, 128, 0, s>>>((const T*)x, (const T*)bias, (T*)out, rows, cols, scale, causal, group, mask_offset);
            else softmax_cta_kernel<T, 2, 256><<<rows, 256, 0, s>>>((const T*)x, (const T*)bias, (T*)out, rows, cols, scale, causal, group, mask_offset);
        } else if (vec) {
            DISPATCH_CH(ch, softmax_warp_kernel<T, CH><<<(rows + ROW_WARPS - 1) / ROW_WARPS,
                ROW_WARPS * 32, 0, s>>>((const T*)x, (const T*)bias, (T*)out, rows, cols, scale,
                                        causal, group, mask_offset));
        } else {
            // The block kernel re-reads x after writing out: not safe in place.
            if (x == out) return ltl_fail(LTL_ERR_UNSUPPORTED,
                "softmax: in-place needs 16-byte aligned rows of at most %d elements", 32 * MAX_CH * 4);
            softmax_block_kernel<T><<<rows, 256, 0, s>>>((const T*)x, (const T*)bias, (T*)out, rows,
                                                         cols, scale, causal, group, mask_offset);
        }
    });
    return ltl_check_launch("softmax");
}

template <typename T, int CH>
__global__ void __launch_bounds__(ROW_WARPS * 32)
softmax_bwd_warp_kernel(const T* __restrict__ y, const T* __restrict__ dy, T* __restrict__ dx,
                        int rows, int cols, float scale, int causal, int group, int mask_offset)
{
    constexpr int N = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * ROW_WARPS + (threadIdx.x >> 5);
    if (row >= rows) return;
    const int lrow = group > 0 ? row % group : row;
    const int limit = causal ? lrow + mask_offset : cols - 1;
    const size_t base = (size_t)row * cols;
    float yv[CH][N], dv[CH][N];
    float dot = 0.0f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int e = (c * 32 + lane) * N;
        if (e < cols) {
            ld16<T>(y + base + e, yv[c]);
            ld16<T>(dy + base + e, dv[c]);
#pragma unroll
            for (int i = 0; i < N; ++i)
                if (e + i <= limit) dot = fmaf(dv[c][i], yv[c][i], dot);
        }
    }
    dot = warp_sum(dot);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int e = (c * 32 + lane) * N;
        if (e < cols) {
            float o[N];
#pragma unroll
            for (int i = 0; i < N; ++i)
                o[i] = (e + i <= limit) ? scale * yv[c][i] * (dv[c][i] - dot) : 0.0f;
            st16<T>(dx + base + e, o);
        }
    }
}

template <typename T>
__global__ void softmax_bwd_block_kernel(const T* __restrict__ y, const T* __restrict__ dy,
                                         T* __restrict__ dx, int rows, int cols, float scale,
                                         int causal, int group, int mask_offset)
{
    __shared__ float red[33];
    const int row = blockIdx.x;
    const int lrow = group > 0 ? row % group : row;
    const int limit = causal ? lrow + mask_offset : cols - 1;
    const size_t base = (size_t)row * cols;
    float dot = 0.0f;
    for (int i = threadIdx.x; i < cols; i += blockDim.x)
        if (i <= limit) dot += Cvt<T>::ld(dy, base + i) * Cvt<T>::ld(y, base + i);
    dot = block_sum(dot, red);   // every read of dy happens before the barrier inside
    for (int i = threadIdx.x; i < cols; i += blockDim.x) {
        float v = 0.0f;
        if (i <= limit) v = scale * Cvt<T>::ld(y, base + i) * (Cvt<T>::ld(dy, base + i) - dot);
        Cvt<T>::st(dx, base + i, v);
    }
}

int ltl_softmax_bwd(const void* y, const void* dy, void* dx, int rows, int cols, float scale,
                    int causal, int group, int mask_offset, int dtype, cudaStream_t s)
{
    if (!y || !dy || !dx) return ltl_fail(LTL_ERR_NULL, "softmax_bwd: null pointer");
    if (rows < 0 || cols <= 0) return ltl_fail(LTL_ERR_SHAPE, "softmax_bwd: bad shape %dx%d", rows, cols);
    if (rows == 0) return LTL_OK;
    const int ch = row_chunks(cols, ltl_dtype_size(dtype));
    const bool vec = ch && aligned16(y) && aligned16(dy) && aligned16(dx);
    DISPATCH_T(dtype, {
        if (vec) {
            DISPATCH_CH(ch, softmax_bwd_warp_kernel<T, CH><<<(rows + ROW_WARPS - 1) / ROW_WARPS,
                ROW_WARPS * 32, 0, s>>>((const T*)y, (const T*)dy, (T*)dx, rows, cols, scale, causal,
                                        group, mask_offset));
        } else {
            softmax_bwd_block_kernel<T><<<rows, 256, 0, s>>>((const T*)y, (const T*)dy, (T*)dx, rows,
                                                             cols, scale, causal, group, mask_offset);
        }
    });
    return ltl_check_launch("softmax_bwd");
}

// ------------------------------------------------------------------------------------------
// SwiGLU: out = silu(a) * b on strided rows (reference: cuda/luaTL_train.cu:647,666)
// ------------------------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void swiglu_fwd_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                  T* __restrict__ o, int rows, int cols, int lda, int ldb, int ldo)
{
    constexpr int N = VEC ? Vec16<T>::N : 1;
    const int cpr = cols / N;
    const uint64_t n = (uint64_t)rows * cpr;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (uint64_t)gridDim.x * blockDim.x) {
        const int r = (int)(idx / cpr);
        const int c = (int)(idx - (uint64_t)r * cpr) * N;
        if (VEC) {
            float av[Vec16<T>::N], bv[Vec16<T>::N];
            ld16<T>(a + (size_t)r * lda + c, av);
            ld16<T>(b + (size_t)r * ldb + c, bv);
#pragma unroll
            for (int i = 0; i < Vec16<T>::N; ++i) av[i] = silu_f(av[i]) * bv[i];
            st16<T>(o + (size_t)r * ldo + c, av);
        } else {
            Cvt<T>::st(o, (size_t)r * ldo + c,
                       silu_f(Cvt<T>::ld(a, (size_t)r * lda + c)) * Cvt<T>::ld(b, (size_t)r * ldb + c));
        }
    }
}

template <typename T, bool VEC>
__global__ void swiglu_bwd_kernel(const T* __restrict__ a, const T* __restrict__ b,
                                  const T* __restrict__ dout, T* __restrict__ da,
                                  T* __restrict__ db, int rows, int cols, int lda, int ldb, int ldo)
{
    constexpr int N = VEC ? Vec16<T>::N : 1;
    const int cpr = cols / N;
    const uint64_t n = (uint64_t)rows * cpr;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (uint64_t)gridDim.x * blockDim.x) {
        const int r = (int)(idx / cpr);
        const int c = (int)(idx - (uint64_t)r * cpr) * N;
        if (VEC) {
            float av[Vec16<T>::N], bv[Vec16<T>::N], gv[Vec16<T>::N], oa[Vec16<T>::N], ob[Vec16<T>::N];
            ld16<T>(a + (size_t)r * lda + c, av);
            ld16<T>(b + (size_t)r * ldb + c, bv);
            ld16<T>(dout + (size_t)r * ldo + c, gv);
#pragma unroll
            for (int i = 0; i < Vec16<T>::N; ++i) {
                oa[i] = gv[i] * bv[i] * silu_grad_f(av[i]);
                ob[i] = gv[i] * silu_f(av[i]);
            }
            if (da) st16<T>(da + (size_t)r * lda + c, oa);
            if (db) st16<T>(db + (size_t)r * ldb + c, ob);
        } else {
            const float av = Cvt<T>::ld(a, (size_t)r * lda + c), bv = Cvt<T>::ld(b, (size_t)r * ldb + c);
            const float go = Cvt<T>::ld(dout, (size_t)r * ldo + c);
            if (da) Cvt<T>::st(da, (size_t)r * lda + c, go * bv * silu_grad_f(av));
            if (db) Cvt<T>::st(db, (size_t)r * ldb + c, go * silu_f(av));
        }
    }
}

int ltl_swiglu_fwd(const void* a, const void* b, void* out, int rows, int cols, int lda, int ldb,
                   int ldo, int dtype, cudaStream_t s)
{
    if (!a || !b || !out) return ltl_fail(LTL_ERR_NULL, "swiglu: null pointer");
    if (rows < 0 || cols < 0) return ltl_fail(LTL_ERR_SHAPE, "swiglu: bad shape %dx%d", rows, cols);
    if (rows == 0 || cols == 0) return LTL_OK;
    const int n = (int)(16 / ltl_dtype_size(dtype));
    const bool vec = cols % n == 0 && lda % n == 0 && ldb % n == 0 && ldo % n == 0 &&
                     aligned16(a) && aligned16(b) && aligned16(out);
    const uint64_t work = (uint64_t)rows * (vec ? cols / n : cols);
    DISPATCH_T(dtype, {
        if (vec) swiglu_fwd_kernel<T, true><<<grid1d(work, 256), 256, 0, s>>>((const T*)a, (const T*)b, (T*)out, rows, cols, lda, ldb, ldo);
        else swiglu_fwd_kernel<T, false><<<grid1d(work, 256), 256, 0, s>>>((const T*)a, (const T*)b, (T*)out, rows, cols, lda, ldb, ldo);
    });
    return ltl_check_launch("swiglu_fwd");
}

int ltl_swiglu_bwd(const void* a, const void* b, const void* dout, void* da, void* db, int rows,
                   int cols, int lda, int ldb, int ldo, int dtype, cudaStream_t s)
{
    if (!a || !b || !dout) return ltl_fail(LTL_ERR_NULL, "swiglu_bwd: null pointer");
    if (rows < 0 || cols < 0) return ltl_fail(LTL_ERR_SHAPE, "swiglu_bwd: bad shape %dx%d", rows, cols);
    if (rows == 0 || cols == 0) return LTL_OK;
    const int n = (int)(16 / ltl_dtype_size(dtype));
    const bool vec = cols % n == 0 && lda % n == 0 && ldb % n == 0 && ldo % n == 0 && aligned16(a) &&
                     aligned16(b) && aligned16(dout) && (!da || aligned16(da)) && (!db || aligned16(db));
    const uint64_t work = (uint64_t)rows * (vec ? cols / n : cols);
    DISPATCH_T(dtype, {
        if (vec) swiglu_bwd_kernel<T, true><<<grid1d(work, 256), 256, 0, s>>>((const T*)a, (const T*)b, (const T*)dout, (T*)da, (T*)db, rows, cols, lda, ldb, ldo);
        else swiglu_bwd_kernel<T, false><<<grid1d(work, 256), 256, 0, s>>>((const T*)a, (const T*)b, (const T*)dout, (T*)da, (T*)db, rows, cols, lda, ldb, ldo);
    });
    return ltl_check_launch("swiglu_bwd");
}

// ------------------------------------------------------------------------------------------
// RoPE, in place (reference: cuda/luaTL_train.cu:719).  Half-split pairs (p, p + hd/2) by
// default, interleaved pairs (2p, 2p+1) on request; inverse negates the sine (= backward).
// Angles come from a (cos, sin) table when one is given, else pos * theta^(-2p/hd) inline.
// ------------------------------------------------------------------------------------------
__global__ void rope_table_kernel(float2* __restrict__ table, int npos, int hd, float theta)
{
    const int pairs = hd >> 1;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= npos * pairs) return;
    const int p = idx % pairs, pos = idx / pairs;
    const double freq = pow((double)theta, -2.0 * (double)p / (double)hd);
    double sn, cs;
    sincos((double)pos * freq, &sn, &cs);
    table[idx] = make_float2((float)cs, (float)sn);
}

int ltl_rope_table(float2* table, int npos, int head_dim, float theta, cudaStream_t s)
{
    if (!table) return ltl_fail(LTL_ERR_NULL, "rope_table: null pointer");
    const int n = npos * (head_dim / 2);
    if (n <= 0) return LTL_OK;
    rope_table_kernel<<<(n + 255) / 256, 256, 0, s>>>(table, npos, head_dim, theta);
    return ltl_check_launch("rope_table");
}

__device__ __forceinline__ void rope_angle(int pos, int p, int hd, float theta,
                                           const float2* __restrict__ table, int table_rows,
                                           float& c, float& sn)
{
    if (table && pos >= 0 && pos < table_rows) {
        const float2 cs = table[(size_t)pos * (hd >> 1) + p];
        c = cs.x; sn = cs.y;
    } else {
        const float freq = powf(theta, -2.0f * (float)p / (float)hd);
        sincosf((float)pos * freq, &sn, &c);
    }
}

// VEC: half-split layout, one thread rotates Vec16<T>::N consecutive pairs.
template <typename T, bool VEC>
__global__ void rope_kernel(T* __restrict__ x, const int32_t* __restrict__ pos_ids, int rows,
                            int heads, int hd, int row_stride, int pos_offset, float theta,
                            int interleaved, int inverse, const float2* __restrict__ table,
                            int table_rows)
{
    constexpr int N = VEC ? Vec16<T>::N : 1;
    const int pairs = hd >> 1;
    const int ppr = pairs / N;                       // packets per (row, head)
    const uint64_t n = (uint64_t)rows * heads * ppr;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (uint64_t)gridDim.x * blockDim.x) {
        const int p = (int)(idx % ppr) * N;
        const int hh = (int)((idx / ppr) % heads);
        const int r = (int)(idx / ((uint64_t)ppr * heads));
        const int pos = pos_ids ? pos_ids[r] : r + pos_offset;
        const size_t base = (size_t)r * row_stride + (size_t)hh * hd;
        if (VEC) {
            float x0[Vec16<T>::N], x1[Vec16<T>::N], y0[Vec16<T>::N], y1[Vec16<T>::N];
            ld16<T>(x + base + p, x0);
            ld16<T>(x + base + p + pairs, x1);
#pragma unroll
            for (int i = 0; i < Vec16<T>::N; ++i) {
                float c, sn;
                rope_angle(pos, p + i, hd, theta, table, table_rows, c, sn);
                if (inverse) sn = -sn;
                y0[i] = x0[i] * c - x1[i] * sn;
                y1[i] = x1[i] * c + x0[i] * sn;
            }
            st16<T>(x + base + p, y0);
            st16<T>(x + base + p + pairs, y1);
        } else {
            float c, sn;
            rope_angle(pos, p, hd, theta, table, table_rows, c, sn);
            if (inverse) sn = -sn;
            const size_t i0 = interleaved ? base + 2 * p : base + p;
            const size_t i1 = interleaved ? base + 2 * p + 1 : base + p + pairs;
            const float a0 = Cvt<T>::ld(x, i0), a1 = Cvt<T>::ld(x, i1);
            Cvt<T>::st(x, i0, a0 * c - a1 * sn);
            Cvt<T>::st(x, i1, a1 * c + a0 * sn);
        }
    }
}

// Half-split layout without a table: the angle depends on (position, pair) only, so one thread computes
// the sines and cosines of Vec16<T>::N pairs once and rotates those pairs in every head of its row
// (the per-element powf + sincosf made the per-head form bound by the SM, not by memory).
template <typename T>
__global__ void rope_heads_kernel(T* __restrict__ x, const int32_t* __restrict__ pos_ids, int rows,
                                  int heads, int hd, int row_stride, int pos_offset, float theta, int inverse)
{
    constexpr int N = Vec16<T>::N;
    const int pairs = hd >> 1;
    const int ppr = pairs / N;                       // packets per row (of one head)
    const uint64_t n = (uint64_t)rows * ppr;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (uint64_t)gridDim.x * blockDim.x) {
        const int p = (int)(idx % ppr) * N;
        const int r = (int)(idx / ppr);
        const int pos = pos_ids ? pos_ids[r] : r + pos_offset;
        float c[N], sn[N];
#pragma unroll
        for (int i = 0; i < N; ++i) {
            rope_angle(pos, p + i, hd, theta, nullptr, 0, c[i], sn[i]);
            if (inverse) sn[i] = -sn[i];
        }
        T* xr = x + (size_t)r * row_stride + p;
#pragma unroll 4
        for (int hh = 0; hh < heads; ++hh) {
            float x0[N], x1[N], y0[N], y1[N];
            ld16<T>(xr + (size_t)hh * hd, x0);
            ld16<T>(xr + (size_t)hh * hd + pairs, x1);
#pragma unroll
            for (int i = 0; i < N; ++i) {
                y0[i] = x0[i] * c[i] - x1[i] * sn[i];
                y1[i] = x1[i] * c[i] + x0[i] * sn[i];
            }
            st16<T>(xr + (size_t)hh * hd, y0);
            st16<T>(xr + (size_t)hh * hd + pairs, y1);
        }
    }
}

int ltl_rope(void* x, const int32_t* pos_ids, int rows, int heads, int head_dim, int row_stride,
             int pos_offset, float theta, int interleaved, int inverse, int dtype,
             const float2* cs_table, int table_rows, cudaStream_t s)
{
    if (!x) return ltl_fail(LTL_ERR_NULL, "rope: null pointer");
    if (head_dim & 1) return ltl_fail(LTL_ERR_ARG, "rope: head_dim must be even");
    if (rows < 0 || heads <= 0 || head_dim <= 0)
        return ltl_fail(LTL_ERR_SHAPE, "rope: bad shape rows=%d heads=%d head_dim=%d", rows, heads, head_dim);
    if (rows == 0) return LTL_OK;
    const int n = (int)(16 / ltl_dtype_size(dtype));
    const int pairs = head_dim / 2;
    const bool vec = !interleaved && pairs % n == 0 && row_stride % n == 0 && aligned16(x);
    const uint64_t work = (uint64_t)rows * heads * (vec ? pairs / n : pairs);
    DISPATCH_T(dtype, {
        if (vec && !cs_table && heads >= 4 && (uint64_t)rows * (pairs / n) >= 4096)
            rope_heads_kernel<T><<<grid1d((uint64_t)rows * (pairs / n), 128), 128, 0, s>>>((T*)x, pos_ids, rows, heads, head_dim, row_stride, pos_offset, theta, inverse);
        else if (vec) rope_kernel<T, true><<<grid1d(work, 256), 256, 0, s>>>((T*)x, pos_ids, rows, heads, head_dim, row_stride, pos_offset, theta, interleaved, inverse, cs_table, table_rows);
        else rope_kernel<T, false><<<grid1d(work, 256), 256, 0, s>>>((T*)x, pos_ids, rows, heads, head_dim, row_stride, pos_offset, theta, interleaved, inverse, cs_table, table_rows);
    });
    return ltl_check_launch("rope");
}

// ------------------------------------------------------------------------------------------
// Embedding gather (bit-exact row copies; an id outside [0, vocab) yields a zero row) and
// scatter-add of the gradient (reference: cuda/luaTL_train.cu:771,790).
// ------------------------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void embed_fwd_kernel(const int32_t* __restrict__ ids, const T* __restrict__ table,
                                 T* __restrict__ out, int rows, int dim, int vocab)
{
    constexpr int N = VEC ? Vec16<T>::N : 1;
    const int ppr = dim / N;
    const uint64_t n = (uint64_t)rows * ppr;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (uint64_t)gridDim.x * blockDim.x) {
        const int r = (int)(idx / ppr);
        const int c = (int)(idx - (uint64_t)r * ppr) * N;
        const int t = ids[r];
        const bool ok = t >= 0 && t < vocab;
        if (VEC) {
            uint4 q = make_uint4(0, 0, 0, 0);
            if (ok) q = *reinterpret_cast<const uint4*>(table + (size_t)t * dim + c);
            *reinterpret_cast<uint4*>(out + (size_t)r * dim + c) = q;
        } else {
            out[(size_t)r * dim + c] = ok ? table[(size_t)t * dim + c] : T(0.0f);
        }
    }
}

template <typename T>
__global__ void embed_bwd_kernel(const int32_t* __restrict__ ids, const T* __restrict__ dout,
                                 float* __restrict__ dtable, int rows, int dim, int vocab, float scale)
{
    const uint64_t n = (uint64_t)rows * dim;
    for (uint64_t idx = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < n;
         idx += (uint64_t)gridDim.x * blockDim.x) {
        const int r = (int)(idx / dim);
        const int c = (int)(idx - (uint64_t)r * dim);
        const int t = ids[r];
        if (t < 0 || t >= vocab) continue;
        atomicAdd(&dtable[(size_t)t * dim + c], scale * Cvt<T>::ld(dout, (size_t)r * dim + c));
    }
}

int ltl_embed_fwd(const int32_t* ids, const void* table, void* out, int rows, int dim, int vocab,
                  int dtype, cudaStream_t s)
{
    if (!ids || !table || !out) return ltl_fail(LTL_ERR_NULL, "embed_fwd: null pointer");
    if (rows < 0 || dim <= 0 || vocab <= 0) return ltl_fail(LTL_ERR_SHAPE, "embed_fwd: bad shape");
    if (rows == 0) return LTL_OK;
    const int n = (int)(16 / ltl_dtype_size(dtype));
    const bool vec = dim % n == 0 && aligned16(table) && aligned16(out);
    const uint64_t work = (uint64_t)rows * (vec ? dim / n : dim);
    DISPATCH_T(dtype, {
        if (vec) embed_fwd_kernel<T, true><<<grid1d(work, 256), 256, 0, s>>>(ids, (const T*)table, (T*)out, rows, dim, vocab);
        else embed_fwd_kernel<T, false><<<grid1d(work, 256), 256, 0, s>>>(ids, (const T*)table, (T*)out, rows, dim, vocab);
    });
    return ltl_check_launch("embed_fwd");
}

int ltl_embed_bwd(const int32_t* ids, const void* dout, float* dtable, int rows, int dim,
                  int vocab, float scale, int dtype, cudaStream_t s)
{
    if (!ids || !dout || !dtable) return ltl_fail(LTL_ERR_NULL, "embed_bwd: null pointer");
    if (rows < 0 || dim <= 0 || vocab <= 0) return ltl_fail(LTL_ERR_SHAPE, "embed_bwd: bad shape");
    if (rows == 0) return LTL_OK;
    DISPATCH_T(dtype, embed_bwd_kernel<T><<<grid1d((uint64_t)rows * dim, 256), 256, 0, s>>>(
        ids, (const T*)dout, dtable, rows, dim, vocab, scale));
    return ltl_check_launch("embed_bwd");
}

// ------------------------------------------------------------------------------------------
// Arg-max helpers: ties resolve to the lowest index (reference: cuda/luaTL_train.cu:1000,1014;
// CPU greedy pick: ai/optim/lmtrain.lua:1365-1371, first strict maximum).
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ void argmax_merge(float& v, int& i, float ov, int oi)
{
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
}
// red_v/red_i: 32 entries each.  Result valid in every thread.
__device__ __forceinline__ void block_argmax(float& v, int& i, float* red_v, int* red_i)
{
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        argmax_merge(v, i, __shfl_xor_sync(0xFFFFFFFFu, v, o), __shfl_xor_sync(0xFFFFFFFFu, i, o));
    __syncthreads();
    if (lane == 0) { red_v[wid] = v; red_i[wid] = i; }
    __syncthreads();
    v = lane < nw ? red_v[lane] : -INFINITY;
    i = lane < nw ? red_i[lane] : 0x7FFFFFFF;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1)
        argmax_merge(v, i, __shfl_xor_sync(0xFFFFFFFFu, v, o), __shfl_xor_sync(0xFFFFFFFFu, i, o));
    if (i == 0x7FFFFFFF) i = 0;   // every value was NaN or -inf
}

template <typename T, bool VEC>
__global__ void argmax_rows_kernel(const T* __restrict__ x, int32_t* __restrict__ out, int rows, int cols)
{
    __shared__ float red_v[32];
    __shared__ int red_i[32];
    const T* xr = x + (size_t)blockIdx.x * cols;
    float best = -INFINITY;
    int bi = 0x7FFFFFFF;
    if (VEC) {
        constexpr int N = Vec16<T>::N;
        for (int e = threadIdx.x * N; e < cols; e += blockDim.x * N) {
            float v[N];
            ld16<T>(xr + e, v);
#pragma unroll
            for (int i = 0; i < N; ++i) if (v[i] > best) { best = v[i]; bi = e + i; }
        }
    } else {
        for (int i = threadIdx.x; i < cols; i += blockDim.x) {
            const float v = Cvt<T>::ld(xr, i);
            if (v > best) { best = v; bi = i; }
        }
    }
    block_argmax(best, bi, red_v, red_i);
    if (threadIdx.x == 0) out[blockIdx.x] = bi;
}

int ltl_argmax_rows(const void* x, int32_t* out, int rows, int cols, int dtype, cudaStream_t s)
{
    if (!x || !out) return ltl_fail(LTL_ERR_NULL, "argmax: null pointer");
    if (rows < 0 || cols <= 0) return ltl_fail(LTL_ERR_SHAPE, "argmax: bad shape %dx%d", rows, cols);
    if (rows == 0) return LTL_OK;
    const int n = (int)(16 / ltl_dtype_size(dtype));
    const bool vec = cols % n == 0 && aligned16(x);
    DISPATCH_T(dtype, {
        if (vec) argmax_rows_kernel<T, true><<<rows, 256, 0, s>>>((const T*)x, out, rows, cols);
        else argmax_rows_kernel<T, false><<<rows, 256, 0, s>>>((const T*)x, out, rows, cols);
    });
    return ltl_check_launch("argmax");
}

// ------------------------------------------------------------------------------------------
// Fused softmax + cross-entropy + dlogits (+ optional argmax), one CTA per row
// (reference: cuda/luaTL_train.cu:837).  The row is staged once in shared memory as fp32
// (rows up to 50 000 logits), so HBM sees one read and, with dlogits, one write.
//   loss_r = lse - x_t ; dlogits = gscale * (softmax - onehot) ; ignored row -> 0 / zeros.
// ------------------------------------------------------------------------------------------
constexpr int CE_SMEM_MAX_V = 50000;

template <typename T, bool CACHE>
__global__ void ce_kernel(const T* __restrict__ logits, const int32_t* __restrict__ targets,
                          float* __restrict__ losses, T* __restrict__ dlogits,
                          int32_t* __restrict__ pred, int rows, int V, int ignore_index, float gscale)
{
    extern __shared__ float rowbuf[];
    __shared__ float red[33];
    __shared__ float red_v[32];
    __shared__ int red_i[32];
    const int r = blockIdx.x;
    const T* lr = logits + (size_t)r * V;
    T* dr = dlogits ? dlogits + (size_t)r * V : nullptr;
    const int t = targets[r];
    const bool ignored = t < 0 || t >= V || t == ignore_index;
    if (ignored && !pred) {
        if (threadIdx.x == 0 && losses) losses[r] = 0.0f;
        if (dr) for (int i = threadIdx.x; i < V; i += blockDim.x) Cvt<T>::st(dr, i, 0.0f);
        return;
    }
    float best = -INFINITY;
    int bi = 0x7FFFFFFF;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float v = Cvt<T>::ld(lr, i);
        if (CACHE) rowbuf[i] = v;
        if (v > best) { best = v; bi = i; }
    }
    block_argmax(best, bi, red_v, red_i);
    if (pred && threadIdx.x == 0) pred[r] = bi;
    if (ignored) {
        if (threadIdx.x == 0 && losses) losses[r] = 0.0f;
        if (dr) for (int i = threadIdx.x; i < V; i += blockDim.x) Cvt<T>::st(dr, i, 0.0f);
        return;
    }
    const float mx = best;
    float sum = 0.0f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float e = expf((CACHE ? rowbuf[i] : Cvt<T>::ld(lr, i)) - mx);
        if (CACHE) rowbuf[i] = e;
        sum += e;
    }
    const float xt = Cvt<T>::ld(lr, t);   // read before dlogits may overwrite the row
    sum = block_sum(sum, red);
    const float ssum = fmaxf(sum, 1e-30f);
    if (threadIdx.x == 0 && losses) losses[r] = logf(ssum) + mx - xt;
    if (dr) {
        const float inv = 1.0f / ssum;
        for (int i = threadIdx.x; i < V; i += blockDim.x) {
            float p = (CACHE ? rowbuf[i] : expf(Cvt<T>::ld(lr, i) - mx)) * inv;
            if (i == t) p -= 1.0f;
            Cvt<T>::st(dr, i, gscale * p);
        }
    }
}

// fp32 rows of up to 32768 logits (a multiple of 4): the row lives in registers (NV float4 per thread, 1024
// threads), so the logits are read once with 16-byte loads, never staged in shared memory, and dlogits is written
// from the registers.  Same results as ce_kernel up to the rounding of the fast exponential.
template <int NV>
__global__ void __launch_bounds__(1024)
ce_reg_kernel(const float* __restrict__ logits, const int32_t* __restrict__ targets, float* __restrict__ losses,
              float* __restrict__ dlogits, bf16* __restrict__ dlogits_bf16, int32_t* __restrict__ pred, int rows, int V,
              int ignore_index, float gscale)
{
    __shared__ float red[33];
    __shared__ float red_v[32];
    __shared__ int red_i[32];
    const int r = blockIdx.x;
    const float* lr = logits + (size_t)r * V;
    float* dr = dlogits ? dlogits + (size_t)r * V : nullptr;
    bf16* db = dlogits_bf16 ? dlogits_bf16 + (size_t)r * V : nullptr;
    const int t = targets[r];
    const bool ignored = t < 0 || t >= V || t == ignore_index;
    if (ignored && !pred) {
        if (threadIdx.x == 0 && losses) losses[r] = 0.0f;
        if (dr) for (int i = threadIdx.x * 4; i < V; i += blockDim.x * 4) *reinterpret_cast<float4*>(dr + i) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (db) for (int i = threadIdx.x * 4; i < V; i += blockDim.x * 4) *reinterpret_cast<uint2*>(db + i) = make_uint2(0u, 0u);
        return;
    }
    float4 v[NV];
    float best = -INFINITY;
    int bi = 0x7FFFFFFF;
#pragma unroll
    for (int c = 0; c < NV; ++c) {
        const int i = (c * 1024 + threadIdx.x) * 4;
        v[c] = i < V ? *reinterpret_cast<const float4*>(lr + i) : make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
        if (v[c].x > best) { best = v[c].x; bi = i; }
        if (v[c].y > best) { best = v[c].y; bi = i + 1; }
        if (v[c].z > best) { best = v[c].z; bi = i + 2; }
        if (v[c].w > best) { best = v[c].w; bi = i + 3; }
    }
    block_argmax(best, bi, red_v, red_i);
    if (pred && threadIdx.x == 0) pred[r] = bi;
    if (ignored) {
        if (threadIdx.x == 0 && losses) losses[r] = 0.0f;
        if (dr) for (int i = threadIdx.x * 4; i < V; i += blockDim.x * 4) *reinterpret_cast<float4*>(dr + i) = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (db) for (int i = threadIdx.x * 4; i < V; i += blockDim.x * 4) *reinterpret_cast<uint2*>(db + i) = make_uint2(0u, 0u);
        return;
    }
    const float mx = best;
    float sum = 0.0f;
#pragma unroll
    for (int c = 0; c < NV; ++c) {
        v[c].x = __expf(v[c].x - mx); v[c].y = __expf(v[c].y - mx); v[c].z = __expf(v[c].z - mx); v[c].w = __expf(v[c].w - mx);
        sum += (v[c].x + v[c].y) + (v[c].z + v[c].w);
    }
    const float xt = lr[t];               // read before dlogits may overwrite the row
    sum = block_sum(sum, red);
    const float ssum = fmaxf(sum, 1e-30f);
    if (threadIdx.x == 0 && losses) losses[r] = logf(ssum) + mx - xt;
    if (dr || db) {
        const float k = gscale / ssum;
#pragma unroll
        for (int c = 0; c < NV; ++c) {
            const int i = (c * 1024 + threadIdx.x) * 4;
            if (i < V) {
                float4 p = make_float4(v[c].x * k, v[c].y * k, v[c].z * k, v[c].w * k);
                if (t == i) p.x -= gscale; else if (t == i + 1) p.y -= gscale; else if (t == i + 2) p.z -= gscale; else if (t == i + 3) p.w -= gscale;
                if (dr) *reinterpret_cast<float4*>(dr + i) = p;
                if (db) {
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(p.x, p.y), hi = __floats2bfloat162_rn(p.z, p.w);
                    uint2 pk;
                    pk.x = *reinterpret_cast<const uint32_t*>(&lo);
                    pk.y = *reinterpret_cast<const uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(db + i) = pk;
                }
            }
        }
    }
}

bool ltl_cross_entropy_bf16_grad_supported(const void* logits, int vocab)
{
    return vocab % 4 == 0 && vocab >= 4096 && vocab <= 32768 && aligned16(logits);
}
// fp32 logits in, loss / argmax out, the gradient written as bf16 only (the operand of the backward's GEMMs).
int ltl_cross_entropy_bf16_grad(const float* logits, const int32_t* targets, float* losses, bf16* dlogits_bf16, int32_t* pred,
                                int rows, int vocab, int ignore_index, float grad_scale, cudaStream_t s)
{
    if (!logits || !targets || !dlogits_bf16) return ltl_fail(LTL_ERR_NULL, "cross_entropy: null pointer");
    if (!ltl_cross_entropy_bf16_grad_supported(logits, vocab) || (reinterpret_cast<uintptr_t>(dlogits_bf16) & 7))
        return ltl_fail(LTL_ERR_UNSUPPORTED, "cross_entropy: bf16 gradient output needs a vocabulary of 4096 .. 32768, a multiple of 4");
    if (rows <= 0) return LTL_OK;
    const int nv = (vocab + 4095) / 4096;
#define CE_REG(NVV) ce_reg_kernel<NVV><<<rows, 1024, 0, s>>>(logits, targets, losses, nullptr, dlogits_bf16, pred, rows, vocab, ignore_index, grad_scale)
    if (nv <= 2) CE_REG(2); else if (nv <= 4) CE_REG(4); else CE_REG(8);
#undef CE_REG
    return ltl_check_launch("cross_entropy");
}

int ltl_cross_entropy(const void* logits, const int32_t* targets, float* losses, void* dlogits,
                      int32_t* pred, int rows, int vocab, int ignore_index, float grad_scale,
                      int dtype, cudaStream_t s)
{
    if (!logits || !targets) return ltl_fail(LTL_ERR_NULL, "cross_entropy: null pointer");
    if (rows < 0 || vocab <= 0) return ltl_fail(LTL_ERR_SHAPE, "cross_entropy: bad shape %dx%d", rows, vocab);
    if (rows == 0) return LTL_OK;
    if (dtype == LTL_F32 && vocab % 4 == 0 && vocab >= 4096 && vocab <= 32768 && aligned16(logits) && (!dlogits || aligned16(dlogits))) {
        const int nv = (vocab + 4095) / 4096;
#define CE_REG(NVV) ce_reg_kernel<NVV><<<rows, 1024, 0, s>>>((const float*)logits, targets, losses, (float*)dlogits, nullptr, pred, rows, vocab, ignore_index, grad_scale)
        if (nv <= 2) CE_REG(2); else if (nv <= 4) CE_REG(4); else CE_REG(8);
#undef CE_REG
        return ltl_check_launch("cross_entropy");
    }
    const bool cache = vocab <= CE_SMEM_MAX_V;
    const int threads = vocab >= 8192 ? 1024 : (vocab >= 1024 ? 512 : 256);
    const size_t smem = cache ? (size_t)vocab * sizeof(float) : 0;
    DISPATCH_T(dtype, {
        if (cache) {
            if (smem > 48 * 1024)
                LTL_CUDA("cross_entropy attr", cudaFuncSetAttribute(ce_kernel<T, true>,
                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            ce_kernel<T, true><<<rows, threads, smem, s>>>((const T*)logits, targets, losses,
                (T*)dlogits, pred, rows, vocab, ignore_index, grad_scale);
        } else {
            ce_kernel<T, false><<<rows, threads, 0, s>>>((const T*)logits, targets, losses,
                (T*)dlogits, pred, rows, vocab, ignore_index, grad_scale);
        }
    });
    return ltl_check_launch("cross_entropy");
}

// ------------------------------------------------------------------------------------------
// Reductions, clipping (reference: cuda/luaTL_train.cu:921,947,969)
// ------------------------------------------------------------------------------------------
template <typename T>
__global__ void l2sq_kernel(const T* __restrict__ x, uint64_t n, float* __restrict__ out, int vec)
{
    __shared__ float red[33];
    constexpr int N = Vec16<T>::N;
    float acc = 0.0f;
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nt = (uint64_t)gridDim.x * blockDim.x;
    uint64_t done = 0;
    if (vec) {
        const uint64_t np = n / N;
        for (uint64_t p = tid; p < np; p += nt) {
            float v[N];
            ld16<T>(x + p * N, v);
#pragma unroll
            for (int i = 0; i < N; ++i) acc = fmaf(v[i], v[i], acc);
        }
        done = np * N;
    }
    for (uint64_t i = done + tid; i < n; i += nt) {
        const float v = Cvt<T>::ld(x, i);
        acc = fmaf(v, v, acc);
    }
    acc = block_sum(acc, red);
    if (threadIdx.x == 0) atomicAdd(out, acc);
}

int ltl_l2_accum(const void* x, uint64_t n, float* out, int dtype, cudaStream_t s)
{
    if (!x || !out) return ltl_fail(LTL_ERR_NULL, "l2_accum: null pointer");
    if (n == 0) return LTL_OK;
    const int N = (int)(16 / ltl_dtype_size(dtype));
    DISPATCH_T(dtype, l2sq_kernel<T><<<grid1d((n + N - 1) / N, 256, 4), 256, 0, s>>>(
        (const T*)x, n, out, aligned16(x) ? 1 : 0));
    return ltl_check_launch("l2_accum");
}

template <typename T>
__global__ void clip_kernel(T* __restrict__ x, uint64_t n, const float* __restrict__ nsq, float max_norm)
{
    const float nrm = sqrtf(fmaxf(nsq[0], 0.0f));
    float f = 1.0f;
    if (max_norm > 0.0f && nrm > max_norm) f = max_norm / (nrm + 1e-6f);
    if (f == 1.0f) return;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (uint64_t)gridDim.x * blockDim.x)
        Cvt<T>::st(x, i, Cvt<T>::ld(x, i) * f);
}

int ltl_clip_by_nsq(void* x, uint64_t n, const float* nsq, float max_norm, int dtype, cudaStream_t s)
{
    if (!x || !nsq) return ltl_fail(LTL_ERR_NULL, "clip: null pointer");
    if (n == 0) return LTL_OK;
    DISPATCH_T(dtype, clip_kernel<T><<<grid1d(n, 256), 256, 0, s>>>((T*)x, n, nsq, max_norm));
    return ltl_check_launch("clip");
}

__global__ void sum_f32_kernel(const float* __restrict__ x, uint64_t n, float* __restrict__ out, float scale)
{
    __shared__ float red[33];
    float acc = 0.0f;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (uint64_t)gridDim.x * blockDim.x)
        acc += x[i];
    acc = block_sum(acc, red);
    if (threadIdx.x == 0) atomicAdd(out, acc * scale);
}

int ltl_sum_f32(const float* x, uint64_t n, float* out, float scale, cudaStream_t s)
{
    if (!x || !out) return ltl_fail(LTL_ERR_NULL, "sum_f32: null pointer");
    if (n == 0) return LTL_OK;
    // One CTA up to 64 Ki elements keeps the sum order fixed (losses of one batch).
    const unsigned grid = n <= 65536 ? 1u : grid1d(n, 1024, 2);
    sum_f32_kernel<<<grid, 1024, 0, s>>>(x, n, out, scale);
    return ltl_check_launch("sum_f32");
}

// ------------------------------------------------------------------------------------------
// Element-wise family (opcode numbering: ai/gpu/luaTL.lua:200-205)
// ------------------------------------------------------------------------------------------
__device__ __forceinline__ float gelu_f(float x)
{
    const float t = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.0f + tanhf(t));
}
__device__ __forceinline__ float gelu_grad_f(float x)
{
    const float t = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    const float th = tanhf(t);
    const float dt = 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * x * x);
    return 0.5f * (1.0f + th) + 0.5f * x * (1.0f - th * th) * dt;
}
__device__ __forceinline__ float ew_apply(int op, float a, float b, float alpha, float beta)
{
    switch (op) {
        case 0:  return a;                                  // COPY
        case 1:  return alpha * a + beta * b;               // ADD
        case 2:  return alpha * a - beta * b;               // SUB
        case 3:  return alpha * a * b;                      // MUL
        case 4:  return alpha * a / (b + 1e-20f);           // DIV
        case 5:  return alpha * a + beta;                   // SCALE
        case 6:  return alpha * a + b;                      // AXPY
        case 7:  return alpha;                              // FILL
        case 8:  return fmaxf(a, 0.0f);                     // RELU
        case 9:  return gelu_f(a);                          // GELU
        case 10: return silu_f(a);                          // SILU
        case 11: return tanhf(a);                           // TANH
        case 12: return 1.0f / (1.0f + expf(-a));           // SIGMOID
        case 13: return expf(a);                            // EXP
        case 14: return sqrtf(fmaxf(a, 0.0f));              // SQRT
        case 15: return rsqrtf(fmaxf(a, 1e-20f));           // RSQRT
        case 16: return -a;                                 // NEG
        case 17: return 1.0f / (a + 1e-20f);                // RECIP
        case 18: return fabsf(a);                           // ABS
        case 19: return fminf(fmaxf(a, alpha), beta);       // CLAMP
        case 20: return a > 0.0f ? b : 0.0f;                // DRELU
        case 21: return b * silu_grad_f(a);                 // DSILU
        case 22: return b * gelu_grad_f(a);                 // DGELU
        default: return a;
    }
}

template <typename T>
__global__ void ew_kernel(const T* __restrict__ A, const T* __restrict__ B, T* __restrict__ C,
                          uint64_t n, int op, float alpha, float beta, int vec)
{
    constexpr int N = Vec16<T>::N;
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nt = (uint64_t)gridDim.x * blockDim.x;
    uint64_t done = 0;
    if (vec) {
        const uint64_t np = n / N;
        for (uint64_t p = tid; p < np; p += nt) {
            float a[N], b[N];
#pragma unroll
            for (int i = 0; i < N; ++i) { a[i] = 0.0f; b[i] = 0.0f; }
            if (A) ld16<T>(A + p * N, a);
            if (B) ld16<T>(B + p * N, b);
#pragma unroll
            for (int i = 0; i < N; ++i) a[i] = ew_apply(op, a[i], b[i], alpha, beta);
            st16<T>(C + p * N, a);
        }
        done = np * N;
    }
    for (uint64_t i = done + tid; i < n; i += nt)
        Cvt<T>::st(C, i, ew_apply(op, A ? Cvt<T>::ld(A, i) : 0.0f, B ? Cvt<T>::ld(B, i) : 0.0f, alpha, beta));
}

int ltl_elementwise(const void* a, const void* b, void* c, uint64_t n, int dtype, int op,
                    float alpha, float beta, cudaStream_t s)
{
    if (!c) return ltl_fail(LTL_ERR_NULL, "elementwise: null output");
    if (op < 0 || op > 22) return ltl_fail(LTL_ERR_ARG, "elementwise: unknown op %d", op);
    if (!a && op != 7) return ltl_fail(LTL_ERR_NULL, "elementwise: op %d needs input A", op);
    if (n == 0) return LTL_OK;
    const int N = (int)(16 / ltl_dtype_size(dtype));
    const int vec = (aligned16(c) && (!a || aligned16(a)) && (!b || aligned16(b))) ? 1 : 0;
    DISPATCH_T(dtype, ew_kernel<T><<<grid1d((n + N - 1) / N, 256), 256, 0, s>>>(
        (const T*)a, (const T*)b, (T*)c, n, op, alpha, beta, vec));
    return ltl_check_launch("elementwise");
}

template <typename TS, typename TD>
__global__ void cast_kernel(const TS* __restrict__ src, TD* __restrict__ dst, uint64_t n)
{
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (uint64_t)gridDim.x * blockDim.x)
        Cvt<TD>::st(dst, i, Cvt<TS>::ld(src, i));
}

int ltl_cast(const void* src, int sd, void* dst, int dd, uint64_t n, cudaStream_t s)
{
    if (!src || !dst) return ltl_fail(LTL_ERR_NULL, "cast: null pointer");
    if (n == 0) return LTL_OK;
    const unsigned g = grid1d(n, 256);
#define CAST_CASE(SD, TS, DD, TD) \
    if (sd == SD && dd == DD) { cast_kernel<TS, TD><<<g, 256, 0, s>>>((const TS*)src, (TD*)dst, n); return ltl_check_launch("cast"); }
    CAST_CASE(LTL_F32, float, LTL_F32, float) CAST_CASE(LTL_F32, float, LTL_BF16, bf16)
    CAST_CASE(LTL_F32, float, LTL_F16, __half) CAST_CASE(LTL_BF16, bf16, LTL_F32, float)
    CAST_CASE(LTL_F16, __half, LTL_F32, float) CAST_CASE(LTL_BF16, bf16, LTL_BF16, bf16)
    CAST_CASE(LTL_F16, __half, LTL_F16, __half) CAST_CASE(LTL_BF16, bf16, LTL_F16, __half)
    CAST_CASE(LTL_F16, __half, LTL_BF16, bf16)
#undef CAST_CASE
    return ltl_fail(LTL_ERR_DTYPE, "cast: unsupported dtype pair %d -> %d", sd, dd);
}

__global__ void transpose_to_bf16_kernel(const float* __restrict__ in, bf16* __restrict__ out,
                                         int rows, int cols, int half)
{
    __shared__ float tile[32][33];
    const int x = blockIdx.x * 32 + threadIdx.x, y0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += 8)
        tile[j][threadIdx.x] = (y0 + j < rows && x < cols) ? in[(size_t)(y0 + j) * cols + x] : 0.0f;
    __syncthreads();
    const int ox = y0 + threadIdx.x;               // column in out = row in in
    for (int j = threadIdx.y; j < 32; j += 8) {
        const int oy = blockIdx.x * 32 + j;        // row in out = column in in
        if (oy < cols && ox < rows) {
            const int orow = half > 0 ? (oy < half ? 2 * oy : 2 * (oy - half) + 1) : oy;
            out[(size_t)orow * rows + ox] = __float2bfloat16_rn(tile[threadIdx.x][j]);
        }
    }
}

int ltl_transpose_to_bf16(const float* in, bf16* out, int rows, int cols, int interleave_half, cudaStream_t s)
{
    if (!in || !out) return ltl_fail(LTL_ERR_NULL, "transpose_to_bf16: null pointer");
    if (rows <= 0 || cols <= 0) return LTL_OK;
    dim3 grid((cols + 31) / 32, (rows + 31) / 32), block(32, 8);
    transpose_to_bf16_kernel<<<grid, block, 0, s>>>(in, out, rows, cols, interleave_half);
    return ltl_check_launch("transpose_to_bf16");
}

// out[C, R] (bf16) = in[R, C]^T for an fp32 or bf16 input: 64 x 64 tiles through shared memory, two
// elements per thread on both sides, so that reads and writes are 128-byte segments per warp.  The
// backward's weight-gradient GEMMs take both operands with the token dimension contiguous.
template <typename TI>
__global__ void __launch_bounds__(256)
transpose_any_to_bf16_kernel(const TI* __restrict__ in, bf16* __restrict__ out, int rows, int cols)
{
    __shared__ float tile[64][65];
    const int r0 = blockIdx.y * 64, c0 = blockIdx.x * 64;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;          // 32 x 8
    for (int j = ty; j < 64; j += 8) {
        const int r = r0 + j, c = c0 + 2 * tx;
        float a = 0.0f, b = 0.0f;
        if (r < rows) {
            if (c + 1 < cols && (cols & 1) == 0) {
                if (sizeof(TI) == 4) { const float2 v = *reinterpret_cast<const float2*>(in + (size_t)r * cols + c); a = v.x; b = v.y; }
                else { const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(in + (size_t)r * cols + c); a = __low2float(v); b = __high2float(v); }
            } else {
                if (c < cols) a = Cvt<TI>::ld(in, (size_t)r * cols + c);
                if (c + 1 < cols) b = Cvt<TI>::ld(in, (size_t)r * cols + c + 1);
            }
        }
        tile[j][2 * tx] = a; tile[j][2 * tx + 1] = b;
    }
    __syncthreads();
    for (int j = ty; j < 64; j += 8) {
        const int oc = c0 + j, orr = r0 + 2 * tx;                   // out row = input column
        if (oc >= cols) continue;
        const float a = tile[2 * tx][j], b = tile[2 * tx + 1][j];
        if (orr + 1 < rows && (rows & 1) == 0) {
            *reinterpret_cast<__nv_bfloat162*>(out + (size_t)oc * rows + orr) = __floats2bfloat162_rn(a, b);
        } else {
            if (orr < rows) out[(size_t)oc * rows + orr] = __float2bfloat16_rn(a);
            if (orr + 1 < rows) out[(size_t)oc * rows + orr + 1] = __float2bfloat16_rn(b);
        }
    }
}

int ltl_transpose_any_to_bf16(const void* in, int in_dtype, bf16* out, int rows, int cols, cudaStream_t s)
{
    if (!in || !out) return ltl_fail(LTL_ERR_NULL, "transpose: null pointer");
    if (rows <= 0 || cols <= 0) return LTL_OK;
    dim3 grid((cols + 63) / 64, (rows + 63) / 64);
    if (grid.y > 65535) return ltl_fail(LTL_ERR_SHAPE, "transpose: %d rows exceed the grid", rows);
    if (in_dtype == LTL_F32) transpose_any_to_bf16_kernel<float><<<grid, 256, 0, s>>>((const float*)in, out, rows, cols);
    else if (in_dtype == LTL_BF16) transpose_any_to_bf16_kernel<bf16><<<grid, 256, 0, s>>>((const bf16*)in, out, rows, cols);
    else return ltl_fail(LTL_ERR_DTYPE, "transpose: input dtype %d", in_dtype);
    return ltl_check_launch("transpose");
}

// ------------------------------------------------------------------------------------------
// Optimisers.  AdamW as the reference's GPU path (cuda/luaTL_core.cu:1348; bias correction
// cuda/luaTL_train.cu:1428-1431); SGD as the reference's CPU path
// (ai/optim/optim2.lua:93-99: p -= lr * (g + wd * p)) with the GPU path's clip factor
// (cuda/luaTL_train.cu:950-952) folded in.
// ------------------------------------------------------------------------------------------
template <typename TG>
__global__ void adamw_kernel(float* __restrict__ w, const TG* __restrict__ g, float* __restrict__ m,
                             float* __restrict__ v, TG* __restrict__ w_lp, uint64_t n, float lr,
                             float beta1, float beta2, float eps, float wd, float bc1, float bc2, float clip)
{
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (uint64_t)gridDim.x * blockDim.x) {
        float gr = Cvt<TG>::ld(g, i);
        if (clip > 0.0f) gr = fminf(fmaxf(gr, -clip), clip);
        const float mi = beta1 * m[i] + (1.0f - beta1) * gr;
        const float vi = beta2 * v[i] + (1.0f - beta2) * gr * gr;
        m[i] = mi; v[i] = vi;
        float wi = w[i];
        wi -= lr * wd * wi;
        wi -= lr * (mi * bc1) / (sqrtf(vi * bc2) + eps);
        w[i] = wi;
        if (w_lp) Cvt<TG>::st(w_lp, i, wi);
    }
}

int ltl_adamw(float* w, const void* g, float* m, float* v, void* w_lp, uint64_t n, int grad_dtype,
              float lr, float beta1, float beta2, float eps, float wd, int step, float clip, cudaStream_t s)
{
    if (!w || !g || !m || !v) return ltl_fail(LTL_ERR_NULL, "adamw: null pointer");
    if (n == 0) return LTL_OK;
    if (step < 1) step = 1;
    const float bc1 = 1.0f / (1.0f - powf(beta1, (float)step));
    const float bc2 = 1.0f / (1.0f - powf(beta2, (float)step));
    DISPATCH_T(grad_dtype, adamw_kernel<T><<<grid1d(n, 256), 256, 0, s>>>(w, (const T*)g, m, v,
        (T*)w_lp, n, lr, beta1, beta2, eps, wd, bc1, bc2, clip));
    return ltl_check_launch("adamw");
}

__global__ void sgd_kernel(float* __restrict__ w, const float* __restrict__ g, bf16* __restrict__ w_lp,
                           uint64_t n, float lr, float wd, const float* __restrict__ nsq,
                           float max_norm, int vec)
{
    float f = 1.0f;
    if (nsq && max_norm > 0.0f) {
        const float nrm = sqrtf(fmaxf(nsq[0], 0.0f));
        if (nrm > max_norm) f = max_norm / (nrm + 1e-6f);
    }
    const uint64_t tid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint64_t nt = (uint64_t)gridDim.x * blockDim.x;
    uint64_t done = 0;
    if (vec) {
        const uint64_t np = n / 4;
        for (uint64_t p = tid; p < np; p += nt) {
            float4 wv = reinterpret_cast<float4*>(w)[p];
            const float4 gv = reinterpret_cast<const float4*>(g)[p];
            wv.x -= lr * (f * gv.x + wd * wv.x);
            wv.y -= lr * (f * gv.y + wd * wv.y);
            wv.z -= lr * (f * gv.z + wd * wv.z);
            wv.w -= lr * (f * gv.w + wd * wv.w);
            reinterpret_cast<float4*>(w)[p] = wv;
            if (w_lp) {
                reinterpret_cast<__nv_bfloat162*>(w_lp)[2 * p] = __floats2bfloat162_rn(wv.x, wv.y);
                reinterpret_cast<__nv_bfloat162*>(w_lp)[2 * p + 1] = __floats2bfloat162_rn(wv.z, wv.w);
            }
        }
        done = np * 4;
    }
    for (uint64_t i = done + tid; i < n; i += nt) {
        const float wi = w[i] - lr * (f * g[i] + wd * w[i]);
        w[i] = wi;
        if (w_lp) w_lp[i] = __float2bfloat16_rn(wi);
    }
}

int ltl_sgd(float* w, const float* g, bf16* w_lp, uint64_t n, float lr, float wd, const float* nsq,
            float max_norm, cudaStream_t s)
{
    if (!w || !g) return ltl_fail(LTL_ERR_NULL, "sgd: null pointer");
    if (n == 0) return LTL_OK;
    const int vec = aligned16(w) && aligned16(g) && (!w_lp || (reinterpret_cast<uintptr_t>(w_lp) & 7u) == 0);
    sgd_kernel<<<grid1d((n + 3) / 4, 256), 256, 0, s>>>(w, g, w_lp, n, lr, wd, nsq, max_norm, vec);
    return ltl_check_launch("sgd");
}

// ------------------------------------------------------------------------------------------
// Whole-model optimizer launches: one kernel over the flat parameter buffer.
//   * weight decay applies everywhere except inside the `nodecay` ranges (the gain vectors; sorted [begin, end) pairs,
//     every boundary a multiple of 4 so that a 16-byte packet never straddles one), looked up by binary search in
//     shared memory;
//   * `loss` (optional) is the step's loss on the device: a non-finite value turns the launch into a no-op, which is
//     the reference's "skip the update when the loss is not finite" (ai/gpu/gpu_transformer.lua:653-660) without a
//     host round trip in the middle of the step.
// ------------------------------------------------------------------------------------------
constexpr int OPT_MAX_RANGES = 1024;

__device__ __forceinline__ bool in_ranges(const long long* r, int npairs, long long e)
{
    int lo = 0, hi = npairs;                  // first pair with end > e
    while (lo < hi) { const int mid = (lo + hi) >> 1; if (r[2 * mid + 1] > e) hi = mid; else lo = mid + 1; }
    return lo < npairs && r[2 * lo] <= e;
}

__global__ void __launch_bounds__(256)
sgd_flat_kernel(float* __restrict__ w, const float* __restrict__ g, uint64_t n, const long long* __restrict__ nodecay,
                int npairs, const float* __restrict__ loss, const float* __restrict__ nsq, float lr, float wd,
                float max_norm)
{
    extern __shared__ long long rng[];
    if (loss && !isfinite(loss[0])) return;
    for (int i = threadIdx.x; i < 2 * npairs; i += blockDim.x) rng[i] = nodecay[i];
    __syncthreads();
    float f = 1.0f;
    if (nsq && max_norm > 0.0f) {
        const float nrm = sqrtf(fmaxf(nsq[0], 0.0f));
        if (nrm > max_norm) f = max_norm / (nrm + 1e-6f);
    }
    const uint64_t np4 = n / 4, nt = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t p = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; p < np4; p += nt) {
        const float d = (wd != 0.0f && !in_ranges(rng, npairs, (long long)(4 * p))) ? wd : 0.0f;
        float4 wv = reinterpret_cast<float4*>(w)[p];
        const float4 gv = reinterpret_cast<const float4*>(g)[p];
        wv.x -= lr * (f * gv.x + d * wv.x);
        wv.y -= lr * (f * gv.y + d * wv.y);
        wv.z -= lr * (f * gv.z + d * wv.z);
        wv.w -= lr * (f * gv.w + d * wv.w);
        reinterpret_cast<float4*>(w)[p] = wv;
    }
    for (uint64_t i = np4 * 4 + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nt) {
        const float d = (wd != 0.0f && !in_ranges(rng, npairs, (long long)i)) ? wd : 0.0f;
        w[i] -= lr * (f * g[i] + d * w[i]);
    }
}

__global__ void __launch_bounds__(256)
adamw_flat_kernel(float* __restrict__ w, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                  uint64_t n, const long long* __restrict__ nodecay, int npairs, const float* __restrict__ loss,
                  float lr, float beta1, float beta2, float eps, float wd, float bc1, float bc2)
{
    extern __shared__ long long rng[];
    if (loss && !isfinite(loss[0])) return;
    for (int i = threadIdx.x; i < 2 * npairs; i += blockDim.x) rng[i] = nodecay[i];
    __syncthreads();
    const uint64_t np4 = n / 4, nt = (uint64_t)gridDim.x * blockDim.x;
    // element-wise arithmetic exactly as adamw_kernel above
    auto upd = [&](float& wi, float gr, float& mi, float& vi, float d) {
        mi = beta1 * mi + (1.0f - beta1) * gr;
        vi = beta2 * vi + (1.0f - beta2) * gr * gr;
        wi -= lr * d * wi;
        wi -= lr * (mi * bc1) / (sqrtf(vi * bc2) + eps);
    };
    for (uint64_t p = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; p < np4; p += nt) {
        const float d = (wd != 0.0f && !in_ranges(rng, npairs, (long long)(4 * p))) ? wd : 0.0f;
        float4 wv = reinterpret_cast<float4*>(w)[p], mv = reinterpret_cast<float4*>(m)[p], vv = reinterpret_cast<float4*>(v)[p];
        const float4 gv = reinterpret_cast<const float4*>(g)[p];
        upd(wv.x, gv.x, mv.x, vv.x, d); upd(wv.y, gv.y, mv.y, vv.y, d);
        upd(wv.z, gv.z, mv.z, vv.z, d); upd(wv.w, gv.w, mv.w, vv.w, d);
        reinterpret_cast<float4*>(w)[p] = wv; reinterpret_cast<float4*>(m)[p] = mv; reinterpret_cast<float4*>(v)[p] = vv;
    }
    for (uint64_t i = np4 * 4 + (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += nt) {
        const float d = (wd != 0.0f && !in_ranges(rng, npairs, (long long)i)) ? wd : 0.0f;
        upd(w[i], g[i], m[i], v[i], d);
    }
}

int ltl_opt_ranges_ok(const long long* host_pairs, int npairs, const void* w, const void* g)
{
    if (npairs < 0 || npairs > OPT_MAX_RANGES || !aligned16(w) || !aligned16(g)) return 0;
    for (int i = 0; i < 2 * npairs; ++i) if (host_pairs[i] % 4) return 0;
    return 1;
}

int ltl_sgd_flat(float* w, const float* g, uint64_t n, const long long* d_nodecay, int npairs, const float* loss,
                 const float* nsq, float lr, float wd, float max_norm, cudaStream_t s)
{
    if (!w || !g) return ltl_fail(LTL_ERR_NULL, "sgd: null pointer");
    if (n == 0) return LTL_OK;
    sgd_flat_kernel<<<grid1d((n + 3) / 4, 256), 256, (size_t)npairs * 16, s>>>(w, g, n, d_nodecay, npairs, loss, nsq, lr, wd,
                                                                              max_norm);
    return ltl_check_launch("sgd");
}

int ltl_adamw_flat(float* w, const float* g, float* m, float* v, uint64_t n, const long long* d_nodecay, int npairs,
                   const float* loss, float lr, float beta1, float beta2, float eps, float wd, int step, cudaStream_t s)
{
    if (!w || !g || !m || !v) return ltl_fail(LTL_ERR_NULL, "adamw: null pointer");
    if (n == 0) return LTL_OK;
    if (step < 1) step = 1;
    const float bc1 = 1.0f / (1.0f - powf(beta1, (float)step));
    const float bc2 = 1.0f / (1.0f - powf(beta2, (float)step));
    adamw_flat_kernel<<<grid1d((n + 3) / 4, 256), 256, (size_t)npairs * 16, s>>>(w, g, m, v, n, d_nodecay, npairs, loss, lr,
                                                                                beta1, beta2, eps, wd, bc1, bc2);
    return ltl_check_launch("adamw");
}

// ------------------------------------------------------------------------------------------
// RMSNorm backward without any allocation.
//
// Who needs it: code that may not call cudaMalloc when it wants a gradient - a host that has
// handed all device memory to its own arena and forbids further driver allocations, or a
// latency-critical loop that cannot afford the implicit device synchronisation of
// cudaMalloc / cudaFree.  luaTL_rmsnorm_bwd takes its dgamma scratch (one partial row per warp)
// from a workspace the library grows with cudaMalloc on demand; this entry point uses a fixed
// array in the library's own device image instead.
//
// The array costs RMSNORM_BWD_STATIC_FLOATS * 4 bytes (4.6 MB) on every GPU that loads the
// library, from load until exit.  The kernel overwrites every partial row it later sums, so
// nothing in the array has to be cleared between calls; but all calls share it, so two calls
// that overlap on the GPU (different streams, or another host thread) race on it.
// ------------------------------------------------------------------------------------------
constexpr size_t RMSNORM_BWD_STATIC_FLOATS = (size_t)1184 * 1024;   // 148 SMs * 2 CTAs * 4 warps rows of <= 1024 columns
static __device__ __align__(256) float g_rmsnorm_bwd_static[RMSNORM_BWD_STATIC_FLOATS];

extern "C" int luaTL_rmsnorm_bwd_noalloc(const void* x, const void* gamma, const void* dy, void* dx, float* dgamma,
                                         int rows, int cols, float eps, int dtype)
{
    LTL_TRY(ltl_require_init("rmsnorm_bwd_noalloc"));
    // In host code the array's name is only a handle: the device address has to be asked for, once
    // per device, with that device current.  The first call on a device does it (so make that first
    // call outside of any stream capture).
    static float* dev_ptr[64] = { nullptr };
    int dev = -1;
    LTL_CUDA("cudaGetDevice", cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return ltl_fail(LTL_ERR_ARG, "rmsnorm_bwd_noalloc: device ordinal %d not supported", dev);
    // The library's stream belongs to the device luaTL_init bound; a caller that has made another device current
    // would get this array's address on one GPU and a stream of another.
    if (dev != ltl_bound_device())
        return ltl_fail(LTL_ERR_ARG, "rmsnorm_bwd_noalloc: current device %d is not the device the library was initialised on (%d)",
                        dev, ltl_bound_device());
    if (!dev_ptr[dev]) {
        float* p = nullptr;
        LTL_CUDA("cudaGetSymbolAddress(rmsnorm_bwd scratch)", cudaGetSymbolAddress((void**)&p, g_rmsnorm_bwd_static));
        if (!p) return ltl_fail(LTL_ERR_CUDA, "rmsnorm_bwd_noalloc: the static scratch has no device address");
        dev_ptr[dev] = p;
    }
    // Only the warp-per-row kernel leaves dgamma partials in scratch; shapes that take the CTA-per-row kernel
    // (row width not a whole number of 16-byte packets per lane, or operands off a 16-byte boundary) need none.
    const bool wants_scratch = dgamma && cols > 0 && rmsnorm_bwd_takes_warp_kernel(x, gamma, dy, dx, cols, dtype);
    if (wants_scratch && ltl_rmsnorm_bwd_scratch_floats(cols) > RMSNORM_BWD_STATIC_FLOATS)
        return ltl_fail(LTL_ERR_CAPACITY, "rmsnorm_bwd_noalloc: %d columns need %zu scratch floats, the static scratch holds %zu "
                        "(at most %zu columns on this GPU); use luaTL_rmsnorm_bwd for wider rows", cols,
                        ltl_rmsnorm_bwd_scratch_floats(cols), RMSNORM_BWD_STATIC_FLOATS,
                        RMSNORM_BWD_STATIC_FLOATS / ((size_t)ltl_sm_count() * 2 * ROW_WARPS));
    cudaStream_t s = ltl_default_stream();
    LTL_TRY(ltl_rmsnorm_bwd(x, gamma, dy, dx, dgamma, rows, cols, eps, dtype, dev_ptr[dev], s));
    return ltl_sync_stream("rmsnorm_bwd_noalloc");      // waits unless luaTL_set_deferred(1) is in force
}
