// Shared plumbing of the B200 backend: status codes, the error buffer behind
// luaTL_get_last_error(), dtype tags, reductions and 128-bit access helpers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

// Status codes and dtype tags are part of the ABI the LuaJIT shim reads
// (reference: cuda/luaTL_core.cu:108-118, ai/gpu/luaTL.lua:193-218).
enum {
    LTL_OK = 0, LTL_ERR_NULL = -1, LTL_ERR_SHAPE = -2, LTL_ERR_DTYPE = -3, LTL_ERR_CUDA = -4,
    LTL_ERR_OOM = -5, LTL_ERR_ARG = -6, LTL_ERR_CAPACITY = -7, LTL_ERR_UNSUPPORTED = -8
};
enum { LTL_F32 = 0, LTL_F16 = 1, LTL_BF16 = 2 };

int  ltl_fail(int status, const char* fmt, ...);   // records the message, returns status
int  ltl_cuda_fail(const char* ctx, cudaError_t e);
int  ltl_check_launch(const char* ctx);            // cudaGetLastError -> status
int  ltl_require_init(const char* ctx);            // LTL_ERR_CUDA unless luaTL_init succeeded
cudaStream_t ltl_default_stream();
int  ltl_bound_device();              // the device luaTL_init bound
int  ltl_sync_stream(const char* ctx);   // launch check + wait for the library stream (no wait in deferred mode)
bool ltl_pdl_enabled();               // programmatic dependent launch for the decode-step kernels
void ltl_pdl_set(bool on);
int  ltl_sm_count();

#define LTL_CUDA(ctx, call)                                               \
    do {                                                                  \
        cudaError_t _e = (call);                                          \
        if (_e != cudaSuccess) return ltl_cuda_fail((ctx), _e);           \
    } while (0)
#define LTL_TRY(call)                                                     \
    do { int _s = (call); if (_s != LTL_OK) return _s; } while (0)

static inline size_t ltl_dtype_size(int dt) { return dt == LTL_F32 ? 4 : 2; }

#ifdef __CUDACC__

typedef __nv_bfloat16 bf16;

// Programmatic dependent launch.  A kernel launched with the attribute may start while its
// predecessor in the stream is still running: it must call pdl_wait() before it reads anything the
// predecessor wrote or writes anything the predecessor reads.  pdl_trigger() lets the successor
// start its own prologue early.  Both are no-ops for a plain launch.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
static inline cudaError_t ltl_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                     bool pdl, Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at; cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename T> struct Cvt;
template <> struct Cvt<float> {
    static __device__ __forceinline__ float ld(const float* p, size_t i) { return p[i]; }
    static __device__ __forceinline__ void  st(float* p, size_t i, float v) { p[i] = v; }
};
template <> struct Cvt<__half> {
    static __device__ __forceinline__ float ld(const __half* p, size_t i) { return __half2float(p[i]); }
    static __device__ __forceinline__ void  st(__half* p, size_t i, float v) { p[i] = __float2half_rn(v); }
};
template <> struct Cvt<bf16> {
    static __device__ __forceinline__ float ld(const bf16* p, size_t i) { return __bfloat162float(p[i]); }
    static __device__ __forceinline__ void  st(bf16* p, size_t i, float v) { p[i] = __float2bfloat16_rn(v); }
};

// A 16-byte packet of T viewed as floats: N = 4 (fp32) or 8 (16-bit types).
template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

template <typename T>
__device__ __forceinline__ void ld16(const T* p, float (&v)[Vec16<T>::N]);
template <>
__device__ __forceinline__ void ld16<float>(const float* p, float (&v)[4])
{
    const float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
}
template <>
__device__ __forceinline__ void ld16<bf16>(const bf16* p, float (&v)[8])
{
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = { q.x, q.y, q.z, q.w };
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        v[2 * i]     = __uint_as_float(w[i] << 16);
        v[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
    }
}
template <>
__device__ __forceinline__ void ld16<__half>(const __half* p, float (&v)[8])
{
    const uint4 q = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&q);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
}

template <typename T>
__device__ __forceinline__ void st16(T* p, const float (&v)[Vec16<T>::N]);
template <>
__device__ __forceinline__ void st16<float>(float* p, const float (&v)[4])
{
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
template <>
__device__ __forceinline__ void st16<bf16>(bf16* p, const float (&v)[8])
{
    uint4 q;
    __nv_bfloat162 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    q = *reinterpret_cast<uint4*>(h);
    *reinterpret_cast<uint4*>(p) = q;
}
template <>
__device__ __forceinline__ void st16<__half>(__half* p, const float (&v)[8])
{
    __half2 h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<uint4*>(h);
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
// Block-wide sum / max, result broadcast to every thread. `red` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* red)
{
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : 0.0f;
    return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float* red)
{
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : -INFINITY;
    return warp_max(t);
}

// Two floats rounded to bf16, the first in the low half (the lower address).
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi)
{
    const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&t);
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_grad_f(float x)
{
    const float s = 1.0f / (1.0f + expf(-x));
    return s * (1.0f + x * (1.0f - s));
}

#endif  // __CUDACC__
