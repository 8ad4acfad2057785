// Runtime, device pool, tensors and the one-shot math entry points of luaTL.so.
// Signatures and behaviour follow the reference's FFI surface (ai/gpu/luaTL.lua:66-167,
// ai/gpu/luaTL_train.lua:27-89); the implementation is this library's own.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include <map>
#include <unordered_map>
#include <vector>

#include "../../include/luatl_b200.h"
#include "ops.h"

// ------------------------------------------------------------------------------------------
// error plumbing
// ------------------------------------------------------------------------------------------
static char g_err[1024] = { 0 };
static int g_has_err = 0;
static int g_verbose = 0;
static int g_initialized = 0;
static int g_device = 0;
static int g_bound_once = 0;
static int g_sm_count = 148;
static uint64_t g_epoch = 1;
static char g_devname[320] = { 0 };
static cudaStream_t g_stream = nullptr;

int ltl_fail(int status, const char* fmt, ...)
{
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    g_has_err = 1;
    if (g_verbose) fprintf(stderr, "[luaTL] %s\n", g_err);
    return status;
}
int ltl_cuda_fail(const char* ctx, cudaError_t e)
{
    return ltl_fail(e == cudaErrorMemoryAllocation ? LTL_ERR_OOM : LTL_ERR_CUDA,
                    "%s failed: %s (cuda error %d)", ctx, cudaGetErrorString(e), (int)e);
}
int ltl_check_launch(const char* ctx)
{
    const cudaError_t e = cudaGetLastError();
    return e == cudaSuccess ? LTL_OK : ltl_cuda_fail(ctx, e);
}
int ltl_require_init(const char* ctx)
{
    if (g_initialized) return LTL_OK;
    return ltl_fail(LTL_ERR_CUDA, "%s: luaTL_init has not succeeded (no CUDA device bound); "
                    "this backend has no CPU fallback", ctx);
}
cudaStream_t ltl_default_stream() { return g_stream; }
int ltl_bound_device() { return g_device; }
static bool g_pdl = false;
bool ltl_pdl_enabled() { return g_pdl; }
void ltl_pdl_set(bool on) { g_pdl = on; }
int ltl_sm_count() { return g_sm_count; }

static bool g_deferred = false;          // luaTL_set_deferred(1): immediate ops do not wait for the stream
static cudaEvent_t g_timer[2] = { nullptr, nullptr };

static int sync_stream(const char* ctx)
{
    LTL_TRY(ltl_check_launch(ctx));
    if (g_deferred) return LTL_OK;
    LTL_CUDA(ctx, cudaStreamSynchronize(g_stream));
    return LTL_OK;
}
int ltl_sync_stream(const char* ctx) { return sync_stream(ctx); }

// ------------------------------------------------------------------------------------------
// caching device pool: power-of-two classes below 1 MiB, 1 MiB granules above
// ------------------------------------------------------------------------------------------
struct luaTL_pool_s {
    int device = 0;
    std::unordered_map<void*, size_t> live;             // ptr -> class bytes, handed out
    std::unordered_map<void*, size_t> owned;            // every block cudaMalloc'ed by this pool
    std::map<size_t, std::vector<void*>> free_lists;
    luaTL_pool_stats_t st = {};
};
static luaTL_pool_t* g_pool = nullptr;
static std::vector<luaTL_pool_t*> g_extra_pools;      // made by luaTL_pool_create, freed with the library

static size_t size_class(size_t bytes)
{
    if (bytes < 256) bytes = 256;
    if (bytes <= (1u << 20)) {
        size_t c = 256;
        while (c < bytes) c <<= 1;
        return c;
    }
    const size_t g = 1u << 20;
    return (bytes + g - 1) / g * g;
}

static void pool_trim(luaTL_pool_t* P)
{
    for (auto& kv : P->free_lists)
        for (void* p : kv.second) {
            cudaFree(p);
            P->owned.erase(p);
            P->st.bytes_reserved -= kv.first;
            P->st.n_cuda_free++;
            P->st.block_count--;
        }
    P->free_lists.clear();
    P->st.free_block_count = 0;
    P->st.n_trim++;
}

static void* pool_alloc(luaTL_pool_t* P, size_t bytes)
{
    const size_t cls = size_class(bytes);
    P->st.n_alloc++;
    void* p = nullptr;
    auto it = P->free_lists.find(cls);
    if (it != P->free_lists.end() && !it->second.empty()) {
        p = it->second.back();
        it->second.pop_back();
        P->st.n_cache_hit++;
        P->st.free_block_count--;
    } else {
        P->st.n_cache_miss++;
        cudaError_t e = cudaMalloc(&p, cls);
        if (e != cudaSuccess) {            // give the cache back and retry once
            cudaGetLastError();
            pool_trim(P);
            e = cudaMalloc(&p, cls);
        }
        if (e != cudaSuccess) {
            cudaGetLastError();
            ltl_fail(LTL_ERR_OOM, "device pool: cudaMalloc of %zu bytes failed: %s", cls, cudaGetErrorString(e));
            return nullptr;
        }
        P->owned[p] = cls;
        P->st.n_cuda_malloc++;
        P->st.bytes_reserved += cls;
        P->st.block_count++;
    }
    P->live[p] = cls;
    P->st.bytes_in_use += cls;
    if (P->st.bytes_in_use > P->st.peak_in_use) P->st.peak_in_use = P->st.bytes_in_use;
    return p;
}

static void pool_free(luaTL_pool_t* P, void* p)
{
    auto it = P->live.find(p);
    if (it == P->live.end()) return;       // double free or foreign pointer: ignore
    const size_t cls = it->second;
    P->live.erase(it);
    P->free_lists[cls].push_back(p);
    P->st.bytes_in_use -= cls;
    P->st.free_block_count++;
    P->st.n_free++;
}

// Library workspace for kernels that need scratch (grown outside of any graph capture).
static float* g_ws = nullptr;
static size_t g_ws_floats = 0;
static int* g_tickets = nullptr;         // tile tickets of luaTL_gemm_bf16_resid
static size_t g_tickets_cap = 0;
static float* workspace(size_t floats)
{
    if (floats <= g_ws_floats) return g_ws;
    cudaStreamSynchronize(g_stream);
    if (g_ws) cudaFree(g_ws);
    g_ws = nullptr; g_ws_floats = 0;
    if (cudaMalloc(&g_ws, floats * sizeof(float)) != cudaSuccess) {
        cudaGetLastError();
        ltl_fail(LTL_ERR_OOM, "workspace: cudaMalloc of %zu bytes failed", floats * sizeof(float));
        return nullptr;
    }
    g_ws_floats = floats;
    return g_ws;
}

extern "C" {

// ------------------------------------------------------------------------------------------
// runtime
// ------------------------------------------------------------------------------------------
const char* luaTL_version(void) { return "luaTL-b200 0.1.0 (sm_100a)"; }
const char* luaTL_train_version(void) { return "luaTL-train b200 0.1.0"; }
void luaTL_set_verbose(int on) { g_verbose = on; }
uint64_t luaTL_epoch(void) { return g_epoch; }
const char* luaTL_device_name(void) { return g_devname; }
const char* luaTL_get_last_error(void) { return g_err; }
int luaTL_has_error(void) { return g_has_err; }
void luaTL_clear_error(void) { g_err[0] = 0; g_has_err = 0; cudaGetLastError(); }

int luaTL_init(int device)
{
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count <= 0) {
        cudaGetLastError();
        ltl_fail(LTL_ERR_CUDA, "luaTL_init: no CUDA device (%s)", e == cudaSuccess ? "count is 0" : cudaGetErrorString(e));
        return 0;
    }
    if (device < 0 || device >= count) {
        ltl_fail(LTL_ERR_ARG, "luaTL_init: device %d out of range (0..%d)", device, count - 1);
        return 0;
    }
    if (g_initialized && device == g_device) return count;
    // One device per process: kernel attributes, cached tensor maps and the streams held by live models and Programs
    // all belong to the device bound first (the reference binds device 0 once, ai/gpu/luatl_adapter.lua:12).
    if (g_bound_once && device != g_device) {
        ltl_fail(LTL_ERR_UNSUPPORTED, "luaTL_init: this process is bound to device %d; one device per process "
                 "(start one process per GPU)", g_device);
        return 0;
    }
    if ((e = cudaSetDevice(device)) != cudaSuccess) { ltl_cuda_fail("cudaSetDevice", e); return 0; }
    if ((e = cudaFree(0)) != cudaSuccess) { ltl_cuda_fail("context creation", e); return 0; }
    cudaDeviceProp prop;
    if ((e = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) { ltl_cuda_fail("cudaGetDeviceProperties", e); return 0; }
    if (prop.major < 10) {
        ltl_fail(LTL_ERR_UNSUPPORTED, "luaTL_init: device %s is sm_%d%d; this library is built for sm_100a only",
                 prop.name, prop.major, prop.minor);
        return 0;
    }
    snprintf(g_devname, sizeof(g_devname), "%s", prop.name);
    g_sm_count = prop.multiProcessorCount > 0 ? prop.multiProcessorCount : 148;
    if ((e = cudaStreamCreateWithFlags(&g_stream, cudaStreamNonBlocking)) != cudaSuccess) { ltl_cuda_fail("cudaStreamCreate", e); return 0; }
    g_device = device;
    g_bound_once = 1;
    g_pool = new luaTL_pool_s();
    g_pool->device = device;
    g_initialized = 1;
    return count;
}

void luaTL_shutdown(void)
{
    if (!g_initialized) return;
    cudaDeviceSynchronize();
    if (g_pool) {
        for (auto& kv : g_pool->owned) cudaFree(kv.first);
        delete g_pool;
        g_pool = nullptr;
    }
    for (luaTL_pool_t* P : g_extra_pools) {
        for (auto& kv : P->owned) cudaFree(kv.first);
        delete P;
    }
    g_extra_pools.clear();
    if (g_ws) { cudaFree(g_ws); g_ws = nullptr; g_ws_floats = 0; }
    if (g_tickets) { cudaFree(g_tickets); g_tickets = nullptr; g_tickets_cap = 0; }
    if (g_stream) { cudaStreamDestroy(g_stream); g_stream = nullptr; }
    g_initialized = 0;
}
void luaTL_shutdown_safe(void) { g_epoch++; luaTL_shutdown(); }
void luaTL_finalize(void) { g_epoch++; luaTL_shutdown(); }

int luaTL_sync(void)
{
    LTL_TRY(ltl_require_init("sync"));
    LTL_CUDA("sync", cudaDeviceSynchronize());
    return LTL_OK;
}

int luaTL_get_devinfo(int device, luaTL_devinfo_t* d)
{
    if (!d) return ltl_fail(LTL_ERR_NULL, "get_devinfo: null output");
    cudaDeviceProp p;
    LTL_CUDA("cudaGetDeviceProperties", cudaGetDeviceProperties(&p, device));
    memset(d, 0, sizeof(*d));
    d->device = device; d->major = p.major; d->minor = p.minor; d->mp_count = p.multiProcessorCount;
    d->warp_size = p.warpSize; d->max_threads_per_block = p.maxThreadsPerBlock;
    d->max_threads_per_mp = p.maxThreadsPerMultiProcessor; d->max_blocks_per_mp = p.maxBlocksPerMultiProcessor;
    d->regs_per_block = p.regsPerBlock; d->regs_per_mp = p.regsPerMultiprocessor;
    int v = 0;
    cudaDeviceGetAttribute(&v, cudaDevAttrClockRate, device); d->clock_khz = v;
    cudaDeviceGetAttribute(&v, cudaDevAttrMemoryClockRate, device); d->memory_clock_khz = v;
    cudaDeviceGetAttribute(&v, cudaDevAttrGlobalMemoryBusWidth, device); d->memory_bus_width = v;
    d->l2_cache_size = p.l2CacheSize; d->concurrent_kernels = p.concurrentKernels;
    d->async_engines = p.asyncEngineCount; d->unified_addressing = p.unifiedAddressing;
    d->cooperative_launch = p.cooperativeLaunch; d->has_tensor_cores = p.major >= 7;
    d->has_fp16 = 1; d->has_bf16 = p.major >= 8; d->ecc_enabled = p.ECCEnabled; d->integrated = p.integrated;
    d->cores_per_mp = 128;
    d->shared_mem_per_block = p.sharedMemPerBlockOptin; d->shared_mem_per_mp = p.sharedMemPerMultiprocessor;
    size_t fb = 0, tb = 0;
    if (cudaMemGetInfo(&fb, &tb) == cudaSuccess) { d->free_global_mem = fb; d->total_global_mem = tb; }
    d->peak_mem_bandwidth_gbs = (double)d->memory_clock_khz * 1e-6 * (d->memory_bus_width / 8.0) * 2.0;
    d->peak_fp32_gflops = 2.0 * d->cores_per_mp * d->mp_count * (double)d->clock_khz * 1e-6;
    d->peak_fp16_gflops = d->peak_fp32_gflops * 8.0;
    snprintf(d->name, sizeof(d->name), "%s", p.name);
    return LTL_OK;
}

int luaTL_mem_info(uint64_t* freeb, uint64_t* totalb)
{
    LTL_TRY(ltl_require_init("mem_info"));
    size_t f = 0, t = 0;
    LTL_CUDA("cudaMemGetInfo", cudaMemGetInfo(&f, &t));
    if (freeb) *freeb = f;
    if (totalb) *totalb = t;
    return LTL_OK;
}

// ------------------------------------------------------------------------------------------
// pool and tensors
// ------------------------------------------------------------------------------------------
luaTL_pool_t* luaTL_default_pool(void) { return g_pool; }

// cuda/luaTL_core.cu:1818-1838: a second caching pool with its own statistics; the default pool cannot be destroyed.
luaTL_pool_t* luaTL_pool_create(int device)
{
    if (ltl_require_init("pool_create") != LTL_OK) return nullptr;
    if (device >= 0 && device != g_device) {
        ltl_fail(LTL_ERR_ARG, "pool_create: device %d is not the device this process is bound to (%d)", device, g_device);
        return nullptr;
    }
    luaTL_pool_t* P = new luaTL_pool_s();
    P->device = g_device;
    g_extra_pools.push_back(P);
    return P;
}
void luaTL_pool_destroy(luaTL_pool_t* P)
{
    if (!P || P == g_pool) return;
    for (size_t i = 0; i < g_extra_pools.size(); ++i)
        if (g_extra_pools[i] == P) {
            g_extra_pools.erase(g_extra_pools.begin() + i);
            if (g_initialized) { cudaDeviceSynchronize(); for (auto& kv : P->owned) cudaFree(kv.first); }
            delete P;
            cudaGetLastError();
            return;
        }
}

void* luaTL_tensor_alloc(luaTL_pool_t* P, uint64_t bytes)
{
    if (ltl_require_init("tensor_alloc") != LTL_OK) return nullptr;
    if (!P) P = g_pool;
    return pool_alloc(P, (size_t)bytes);
}
void luaTL_tensor_free(luaTL_pool_t* P, void* ptr)
{
    if (!g_initialized || !ptr) return;
    if (!P) P = g_pool;
    pool_free(P, ptr);
}
void luaTL_pool_trim(luaTL_pool_t* P)
{
    if (!g_initialized) return;
    if (!P) P = g_pool;
    cudaDeviceSynchronize();
    pool_trim(P);
}
int luaTL_pool_get_stats(luaTL_pool_t* P, luaTL_pool_stats_t* out)
{
    if (!out) return ltl_fail(LTL_ERR_NULL, "pool_get_stats: null output");
    LTL_TRY(ltl_require_init("pool_get_stats"));
    if (!P) P = g_pool;
    *out = P->st;
    return LTL_OK;
}
int luaTL_pool_owns(luaTL_pool_t* P, void* ptr)
{
    if (!g_initialized) return 0;
    if (!P) P = g_pool;
    return P->owned.count(ptr) ? 1 : 0;
}

int luaTL_tensor_init(luaTL_tensor_t* t, int rows, int cols, int dtype, luaTL_pool_t* P)
{
    if (!t) return ltl_fail(LTL_ERR_NULL, "tensor_init: null tensor");
    LTL_TRY(ltl_require_init("tensor_init"));
    if (rows <= 0 || cols <= 0) return ltl_fail(LTL_ERR_SHAPE, "tensor_init: bad shape %dx%d", rows, cols);
    if (dtype < 0 || dtype > 2) return ltl_fail(LTL_ERR_DTYPE, "tensor_init: unknown dtype %d", dtype);
    if (!P) P = g_pool;
    const uint64_t n = (uint64_t)rows * (uint64_t)cols;
    const uint64_t bytes = n * ltl_dtype_size(dtype);
    void* p = pool_alloc(P, (size_t)bytes);
    if (!p) return LTL_ERR_OOM;
    LTL_CUDA("tensor_init memset", cudaMemsetAsync(p, 0, bytes, g_stream));
    t->data = p; t->nelem = n; t->nbytes = bytes; t->rows = rows; t->cols = cols; t->dtype = dtype;
    t->owns = 1; t->pool = P; t->device = g_device; t->flags = 0;
    return sync_stream("tensor_init");
}
int luaTL_tensor_wrap(luaTL_tensor_t* t, void* data, int rows, int cols, int dtype)
{
    if (!t || !data) return ltl_fail(LTL_ERR_NULL, "tensor_wrap: null pointer");
    if (rows <= 0 || cols <= 0) return ltl_fail(LTL_ERR_SHAPE, "tensor_wrap: bad shape %dx%d", rows, cols);
    if (dtype < 0 || dtype > 2) return ltl_fail(LTL_ERR_DTYPE, "tensor_wrap: unknown dtype %d", dtype);
    t->data = data; t->nelem = (uint64_t)rows * cols; t->nbytes = t->nelem * ltl_dtype_size(dtype);
    t->rows = rows; t->cols = cols; t->dtype = dtype; t->owns = 0; t->pool = nullptr;
    t->device = g_device; t->flags = 0;
    return LTL_OK;
}
void luaTL_tensor_release(luaTL_tensor_t* t)
{
    if (!t) return;
    if (t->owns && t->data && g_initialized && g_pool) {
        luaTL_pool_t* P = (luaTL_pool_t*)(t->pool ? t->pool : g_pool);
        bool alive = P == g_pool;
        for (luaTL_pool_t* q : g_extra_pools) alive = alive || q == P;
        if (alive) pool_free(P, t->data);
    }
    t->data = nullptr; t->owns = 0; t->nelem = 0; t->nbytes = 0;
}
void luaTL_tensor_release_safe(luaTL_tensor_t* t)
{
    if (!t) return;
    if (!g_initialized || !g_pool) { t->data = nullptr; t->owns = 0; return; }
    luaTL_tensor_release(t);
}
int luaTL_tensor_view(luaTL_tensor_t* dst, const luaTL_tensor_t* src, int row_off, int rows, int cols)
{
    if (!dst || !src || !src->data) return ltl_fail(LTL_ERR_NULL, "tensor_view: null pointer");
    if (row_off < 0 || rows <= 0 || cols <= 0 ||
        (uint64_t)row_off * src->cols + (uint64_t)rows * cols > src->nelem)
        return ltl_fail(LTL_ERR_SHAPE, "tensor_view: %dx%d at row %d exceeds %dx%d", rows, cols, row_off, src->rows, src->cols);
    *dst = *src;
    dst->data = (char*)src->data + (size_t)row_off * src->cols * ltl_dtype_size(src->dtype);
    dst->rows = rows; dst->cols = cols; dst->nelem = (uint64_t)rows * cols;
    dst->nbytes = dst->nelem * ltl_dtype_size(src->dtype); dst->owns = 0;
    return LTL_OK;
}
int luaTL_tensor_zero(luaTL_tensor_t* t)
{
    if (!t || !t->data) return ltl_fail(LTL_ERR_NULL, "tensor_zero: null tensor");
    LTL_TRY(ltl_require_init("tensor_zero"));
    LTL_CUDA("tensor_zero", cudaMemsetAsync(t->data, 0, t->nbytes, g_stream));
    return sync_stream("tensor_zero");
}

static int upload_as(void* dev, int dtype, const float* host, uint64_t n)
{
    if (dtype == LTL_F32) {
        LTL_CUDA("upload", cudaMemcpyAsync(dev, host, n * 4, cudaMemcpyHostToDevice, g_stream));
        return sync_stream("upload");
    }
    void* tmp = pool_alloc(g_pool, n * 4);
    if (!tmp) return LTL_ERR_OOM;
    cudaError_t e = cudaMemcpyAsync(tmp, host, n * 4, cudaMemcpyHostToDevice, g_stream);
    int st = e == cudaSuccess ? ltl_cast(tmp, LTL_F32, dev, dtype, n, g_stream) : ltl_cuda_fail("upload", e);
    if (st == LTL_OK) st = sync_stream("upload");
    pool_free(g_pool, tmp);
    return st;
}
static int download_as(const void* dev, int dtype, float* host, uint64_t n)
{
    if (dtype == LTL_F32) {
        LTL_CUDA("download", cudaMemcpyAsync(host, dev, n * 4, cudaMemcpyDeviceToHost, g_stream));
        return sync_stream("download");
    }
    void* tmp = pool_alloc(g_pool, n * 4);
    if (!tmp) return LTL_ERR_OOM;
    int st = ltl_cast(dev, dtype, tmp, LTL_F32, n, g_stream);
    if (st == LTL_OK) {
        cudaError_t e = cudaMemcpyAsync(host, tmp, n * 4, cudaMemcpyDeviceToHost, g_stream);
        st = e == cudaSuccess ? sync_stream("download") : ltl_cuda_fail("download", e);
    }
    pool_free(g_pool, tmp);
    return st;
}

int luaTL_tensor_upload(luaTL_tensor_t* t, const float* host, uint64_t nelem)
{
    if (!t || !t->data || !host) return ltl_fail(LTL_ERR_NULL, "tensor_upload: null pointer");
    LTL_TRY(ltl_require_init("tensor_upload"));
    if (nelem > t->nelem) return ltl_fail(LTL_ERR_SHAPE, "tensor_upload: %llu elements into a tensor of %llu",
                                          (unsigned long long)nelem, (unsigned long long)t->nelem);
    if (nelem == 0) return LTL_OK;
    return upload_as(t->data, t->dtype, host, nelem);
}
int luaTL_tensor_download(const luaTL_tensor_t* t, float* host, uint64_t nelem)
{
    if (!t || !t->data || !host) return ltl_fail(LTL_ERR_NULL, "tensor_download: null pointer");
    LTL_TRY(ltl_require_init("tensor_download"));
    if (nelem > t->nelem) return ltl_fail(LTL_ERR_SHAPE, "tensor_download: %llu elements from a tensor of %llu",
                                          (unsigned long long)nelem, (unsigned long long)t->nelem);
    if (nelem == 0) return LTL_OK;
    return download_as(t->data, t->dtype, host, nelem);
}
int luaTL_tensor_copy(const luaTL_tensor_t* src, luaTL_tensor_t* dst)
{
    if (!src || !dst || !src->data || !dst->data) return ltl_fail(LTL_ERR_NULL, "tensor_copy: null pointer");
    LTL_TRY(ltl_require_init("tensor_copy"));
    if (src->nelem != dst->nelem) return ltl_fail(LTL_ERR_SHAPE, "tensor_copy: element counts differ");
    if (src->dtype == dst->dtype)
        LTL_CUDA("tensor_copy", cudaMemcpyAsync(dst->data, src->data, src->nbytes, cudaMemcpyDeviceToDevice, g_stream));
    else
        LTL_TRY(ltl_cast(src->data, src->dtype, dst->data, dst->dtype, src->nelem, g_stream));
    return sync_stream("tensor_copy");
}
int luaTL_tensor_cast(const luaTL_tensor_t* src, luaTL_tensor_t* dst) { return luaTL_tensor_copy(src, dst); }

int luaTL_gpu_copy(const float* src, float* dst, uint64_t nelem)
{
    if (!src || !dst) return ltl_fail(LTL_ERR_NULL, "gpu_copy: null pointer");
    LTL_TRY(ltl_require_init("gpu_copy"));
    LTL_CUDA("gpu_copy", cudaMemcpyAsync(dst, src, nelem * 4, cudaMemcpyDeviceToDevice, g_stream));
    return sync_stream("gpu_copy");
}
int luaTL_gpu_zero(float* p, uint64_t nelem)
{
    if (!p) return ltl_fail(LTL_ERR_NULL, "gpu_zero: null pointer");
    LTL_TRY(ltl_require_init("gpu_zero"));
    LTL_CUDA("gpu_zero", cudaMemsetAsync(p, 0, nelem * 4, g_stream));
    return sync_stream("gpu_zero");
}
int luaTL_upload_i32(void* dev, const int32_t* host, uint64_t n)
{
    if (!dev || !host) return ltl_fail(LTL_ERR_NULL, "upload_i32: null pointer");
    LTL_TRY(ltl_require_init("upload_i32"));
    LTL_CUDA("upload_i32", cudaMemcpyAsync(dev, host, n * 4, cudaMemcpyHostToDevice, g_stream));
    return sync_stream("upload_i32");
}
int luaTL_download_i32(const void* dev, int32_t* host, uint64_t n)
{
    if (!dev || !host) return ltl_fail(LTL_ERR_NULL, "download_i32: null pointer");
    LTL_TRY(ltl_require_init("download_i32"));
    LTL_CUDA("download_i32", cudaMemcpyAsync(host, dev, n * 4, cudaMemcpyDeviceToHost, g_stream));
    return sync_stream("download_i32");
}
int luaTL_download_f32(const void* dev, float* host, uint64_t n)
{
    if (!dev || !host) return ltl_fail(LTL_ERR_NULL, "download_f32: null pointer");
    LTL_TRY(ltl_require_init("download_f32"));
    LTL_CUDA("download_f32", cudaMemcpyAsync(host, dev, n * 4, cudaMemcpyDeviceToHost, g_stream));
    return sync_stream("download_f32");
}

// ------------------------------------------------------------------------------------------
// one-shot math: enqueue on the library stream, synchronise, report
// ------------------------------------------------------------------------------------------
#define ONE_SHOT(ctx, call)                         \
    do {                                            \
        LTL_TRY(ltl_require_init(ctx));             \
        LTL_TRY(call);                              \
        return sync_stream(ctx);                    \
    } while (0)

int luaTL_gemm_ex(const void* A, const void* B, void* C, const void* bias, const void* gamma,
                  const float* rowscale, int M, int N, int K, int dtype,
                  long long a_rs, long long a_cs, long long b_rs, long long b_cs,
                  long long c_rs, long long c_cs, long long a_bs, long long b_bs, long long c_bs,
                  int batch, float alpha, float beta, float eps, int pre_op, int post_op)
{
    GemmDesc g = { A, B, C, bias, nullptr, M, N, K, batch < 1 ? 1 : batch, a_rs, a_cs, b_rs, b_cs, c_rs, c_cs,
                   a_bs, b_bs, c_bs, alpha, beta, post_op, dtype, dtype, dtype, pre_op, gamma, rowscale, eps };
    ONE_SHOT("gemm_ex", ltl_gemm_simt(g, g_stream));
}
int luaTL_gemm(const void* A, const void* B, void* C, const void* bias, const void* gamma,
               const float* rowscale, int M, int N, int K, int dtype, float alpha, float beta,
               float eps, int pre_op, int post_op)
{
    return luaTL_gemm_ex(A, B, C, bias, gamma, rowscale, M, N, K, dtype, K, 1, N, 1, N, 1, 0, 0, 0, 1,
                         alpha, beta, eps, pre_op, post_op);
}
int luaTL_rmsnorm(const void* x, const void* w, void* out, int rows, int cols, float eps, int dtype)
{
    ONE_SHOT("rmsnorm", ltl_rmsnorm(x, w, out, rows, cols, eps, dtype, g_stream));
}
int luaTL_rmsnorm_bwd(const void* x, const void* gamma, const void* dy, void* dx, float* dgamma,
                      int rows, int cols, float eps, int dtype)
{
    LTL_TRY(ltl_require_init("rmsnorm_bwd"));
    float* ws = nullptr;
    if (dgamma && cols > 0) {
        ws = workspace(ltl_rmsnorm_bwd_scratch_floats(cols));
        if (!ws) return LTL_ERR_OOM;
    }
    LTL_TRY(ltl_rmsnorm_bwd(x, gamma, dy, dx, dgamma, rows, cols, eps, dtype, ws, g_stream));
    return sync_stream("rmsnorm_bwd");
}
int luaTL_softmax(const void* x, const void* bias, void* out, int rows, int cols, float scale,
                  int causal, int mask_offset, int dtype)
{
    ONE_SHOT("softmax", ltl_softmax(x, bias, out, rows, cols, scale, causal, 0, mask_offset, dtype, g_stream));
}
int luaTL_softmax_ex(const void* x, const void* bias, void* out, int rows, int cols, float scale,
                     int causal, int group, int mask_offset, int dtype)
{
    ONE_SHOT("softmax_ex", ltl_softmax(x, bias, out, rows, cols, scale, causal, group, mask_offset, dtype, g_stream));
}
int luaTL_softmax_bwd(const void* y, const void* dy, void* dx, int rows, int cols, float scale,
                      int causal, int group, int mask_offset, int dtype)
{
    ONE_SHOT("softmax_bwd", ltl_softmax_bwd(y, dy, dx, rows, cols, scale, causal, group, mask_offset, dtype, g_stream));
}
int luaTL_swiglu_fwd(const void* a, const void* b, void* out, int rows, int cols, int lda, int ldb, int ldo, int dtype)
{
    ONE_SHOT("swiglu_fwd", ltl_swiglu_fwd(a, b, out, rows, cols, lda, ldb, ldo, dtype, g_stream));
}
int luaTL_swiglu_bwd(const void* a, const void* b, const void* dout, void* da, void* db, int rows,
                     int cols, int lda, int ldb, int ldo, int dtype)
{
    ONE_SHOT("swiglu_bwd", ltl_swiglu_bwd(a, b, dout, da, db, rows, cols, lda, ldb, ldo, dtype, g_stream));
}
int luaTL_rope(void* x, const void* pos_ids, int rows, int heads, int head_dim, int row_stride,
               int pos_offset, float theta, int interleaved, int inverse, int dtype)
{
    ONE_SHOT("rope", ltl_rope(x, (const int32_t*)pos_ids, rows, heads, head_dim, row_stride, pos_offset, theta,
                              interleaved, inverse, dtype, nullptr, 0, g_stream));
}
int luaTL_embed_fwd(const void* ids, const void* table, void* out, int rows, int dim, int vocab, int dtype)
{
    ONE_SHOT("embed_fwd", ltl_embed_fwd((const int32_t*)ids, table, out, rows, dim, vocab, dtype, g_stream));
}
int luaTL_embed_bwd(const void* ids, const void* dout, float* dtable, int rows, int dim, int vocab, float scale, int dtype)
{
    ONE_SHOT("embed_bwd", ltl_embed_bwd((const int32_t*)ids, dout, dtable, rows, dim, vocab, scale, dtype, g_stream));
}
int luaTL_cross_entropy(const void* logits, const void* targets, float* losses, void* dlogits,
                        int rows, int vocab, int ignore_index, float grad_scale, int dtype)
{
    ONE_SHOT("cross_entropy", ltl_cross_entropy(logits, (const int32_t*)targets, losses, dlogits, nullptr, rows,
                                                vocab, ignore_index, grad_scale, dtype, g_stream));
}
int luaTL_l2_accum(const void* x, uint64_t n, float* out, int dtype)
{
    ONE_SHOT("l2_accum", ltl_l2_accum(x, n, out, dtype, g_stream));
}
int luaTL_clip_by_nsq(void* x, uint64_t n, const float* nsq, float max_norm, int dtype)
{
    ONE_SHOT("clip_by_nsq", ltl_clip_by_nsq(x, n, nsq, max_norm, dtype, g_stream));
}
int luaTL_sum_f32(const float* x, uint64_t n, float* out, float scale)
{
    ONE_SHOT("sum_f32", ltl_sum_f32(x, n, out, scale, g_stream));
}
int luaTL_argmax_rows(const void* x, void* out_i32, int rows, int cols, int dtype)
{
    ONE_SHOT("argmax_rows", ltl_argmax_rows(x, (int32_t*)out_i32, rows, cols, dtype, g_stream));
}
int luaTL_elementwise(const void* A, const void* B, void* C, uint64_t n, int dtype, int op, float alpha, float beta)
{
    ONE_SHOT("elementwise", ltl_elementwise(A, B, C, n, dtype, op, alpha, beta, g_stream));
}
int luaTL_adamw(float* w, const void* g, float* m, float* v, void* w_lp, uint64_t n, int grad_dtype,
                float lr, float beta1, float beta2, float eps, float wd, int step, float clip)
{
    ONE_SHOT("adamw", ltl_adamw(w, g, m, v, w_lp, n, grad_dtype, lr, beta1, beta2, eps, wd, step, clip, g_stream));
}
int luaTL_gemm_bf16_tc(const void* A, const void* B, void* C, const void* R, int M, int N, int K, int c_dtype, int tile_n)
{
    LTL_TRY(ltl_require_init("gemm_bf16_tc"));
    LTL_TRY(ltl_gemm_tc(A, B, C, R, M, N, K, c_dtype, tile_n & 0xFFFF, (tile_n >> 16) & 3, (tile_n >> 20) & 0xFF, g_stream));
    LTL_TRY(sync_stream("gemm_bf16_tc"));
    return g_deferred ? LTL_OK : ltl_gemm_tc_check(g_stream);      // deferred: luaTL_timer_stop reads the flag
}
// Immediate ops normally return after the stream has drained (the reference's contract).  Deferred mode lets a
// caller queue many of them back to back; luaTL_sync or luaTL_timer_stop waits.  Errors of queued kernels then
// surface at that wait.
void luaTL_set_deferred(int on) { g_deferred = on != 0; }
int luaTL_timer_start(void)
{
    LTL_TRY(ltl_require_init("timer_start"));
    for (int i = 0; i < 2; ++i)
        if (!g_timer[i]) LTL_CUDA("timer_start", cudaEventCreate(&g_timer[i]));
    LTL_CUDA("timer_start", cudaEventRecord(g_timer[0], g_stream));
    return LTL_OK;
}
int luaTL_timer_stop(float* ms)
{
    LTL_TRY(ltl_require_init("timer_stop"));
    if (!ms || !g_timer[1]) return ltl_fail(LTL_ERR_ARG, "timer_stop: no result pointer, or timer_start was not called");
    LTL_CUDA("timer_stop", cudaEventRecord(g_timer[1], g_stream));
    LTL_CUDA("timer_stop", cudaStreamSynchronize(g_stream));
    LTL_CUDA("timer_stop", cudaEventElapsedTime(ms, g_timer[0], g_timer[1]));
    return ltl_gemm_tc_check(g_stream);
}
int luaTL_rmsnorm_bwd_residual(const float* x, const float* gamma, const float* dy, float* res, void* res_bf16, float* dgamma,
                               int rows, int cols, float eps)
{
    LTL_TRY(ltl_require_init("rmsnorm_bwd_residual"));
    float* scratch = nullptr;
    if (dgamma) {
        scratch = workspace(ltl_rmsnorm_bwd_scratch_floats(cols));
        if (!scratch) return LTL_ERR_OOM;
    }
    LTL_TRY(ltl_rmsnorm_bwd_residual(x, gamma, dy, res, (bf16*)res_bf16, dgamma, rows, cols, eps, scratch, g_stream));
    return sync_stream("rmsnorm_bwd_residual");
}
int luaTL_sample_rows(const float* logits, int rows, int vocab, float temperature, int top_k, float top_p, uint64_t seed,
                      const int32_t* counters, int32_t* out)
{
    ONE_SHOT("sample_rows", ltl_sample_rows(logits, rows, vocab, temperature, top_k, top_p, seed, counters, out, g_stream));
}
int luaTL_gemm_bf16_tc_xty(const void* X, const void* Y, float* C, int M, int N, int K, int ksplit)
{
    LTL_TRY(ltl_require_init("gemm_bf16_tc_xty"));
    LTL_TRY(ltl_gemm_tc_xty(X, Y, C, M, N, K, ksplit, g_stream));
    LTL_TRY(sync_stream("gemm_bf16_tc_xty"));
    return ltl_gemm_tc_check(g_stream);
}
int luaTL_gemm_bf16_rows(const void* A, const void* B, void* C, int M, int N, int K, int c_dtype, int epilogue, int ksplit)
{
    ONE_SHOT("gemm_bf16_rows", ltl_gemm_rows(A, B, C, M, N, K, c_dtype, epilogue, ksplit, g_stream));
}
// Arrival counters of the fused residual GEMMs for the immediate entry point: one per output tile, zero at rest.
static int* abi_tickets(size_t n)
{
    if (n > g_tickets_cap) {
        cudaStreamSynchronize(g_stream);
        if (g_tickets) cudaFree(g_tickets);
        g_tickets = nullptr; g_tickets_cap = 0;
        if (cudaMalloc(&g_tickets, n * sizeof(int)) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        // on the library stream (a non-blocking stream is not ordered after the legacy stream's memset)
        if (cudaMemsetAsync(g_tickets, 0, n * sizeof(int), g_stream) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        g_tickets_cap = n;
    }
    return g_tickets;
}
int luaTL_gemm_bf16_resid(const void* A, const void* B, float* slices, float* x, const float* gain, void* h, float* ssq,
                          int M, int N, int K, int ksplit, int impl)
{
    LTL_TRY(ltl_require_init("gemm_bf16_resid"));
    if (N <= 0 || M <= 0) return ltl_fail(LTL_ERR_SHAPE, "gemm_bf16_resid: bad shape %dx%d", M, N);
    int* tickets = abi_tickets((size_t)((M + 127) / 128) * ((N + 31) / 32));
    if (!tickets) return ltl_fail(LTL_ERR_OOM, "gemm_bf16_resid: tile tickets");
    LtlGemmFuse f = {};
    f.x = x; f.gain = gain; f.h = h; f.ssq_out = ssq; f.counters = tickets;
    if (impl == 1) LTL_TRY(ltl_gemm_rows(A, B, slices, M, N, K, LTL_F32, 3, ksplit < 1 ? 1 : ksplit, g_stream, &f));
    else LTL_TRY(ltl_gemm_tc(A, B, slices, nullptr, M, N, K, LTL_F32, 32, 3, ksplit < 1 ? 1 : ksplit, g_stream, &f));
    LTL_TRY(sync_stream("gemm_bf16_resid"));
    return impl == 1 ? LTL_OK : ltl_gemm_tc_check(g_stream);
}
int luaTL_gemm_bf16_rowscale(const void* A, const void* B, void* C, const float* ssq, int ssq_tiles, float eps, int M, int N, int K,
                             int c_dtype, int epilogue, int impl)
{
    LTL_TRY(ltl_require_init("gemm_bf16_rowscale"));
    if (!ssq || ssq_tiles < 1) return ltl_fail(LTL_ERR_ARG, "gemm_bf16_rowscale: ssq [M][ssq_tiles] is needed");
    LtlGemmFuse f = {};
    f.ssq_in = ssq; f.ssq_tiles = ssq_tiles; f.inv_dim = 1.0f / (float)K; f.eps = eps;
    if (impl == 1) LTL_TRY(ltl_gemm_rows(A, B, C, M, N, K, c_dtype, epilogue, 1, g_stream, &f));
    else LTL_TRY(ltl_gemm_tc(A, B, C, nullptr, M, N, K, c_dtype, 0, epilogue, 1, g_stream, &f));
    LTL_TRY(sync_stream("gemm_bf16_rowscale"));
    return impl == 1 ? LTL_OK : ltl_gemm_tc_check(g_stream);
}
int luaTL_gemm_bf16_tc_time(const void* A, const void* B, void* C, int M, int N, int K, int c_dtype, int tile_n,
                            int iters, float* ms_per_launch)
{
    LTL_TRY(ltl_require_init("gemm_bf16_tc_time"));
    if (!ms_per_launch || iters < 1) return ltl_fail(LTL_ERR_ARG, "gemm_bf16_tc_time: iters >= 1 and a result pointer are needed");
    cudaEvent_t e0, e1;
    LTL_CUDA("event", cudaEventCreate(&e0));
    LTL_CUDA("event", cudaEventCreate(&e1));
    int rc = LTL_OK;
    for (int i = 0; i < 2 && rc == LTL_OK; ++i)          // warm-up (tensor maps, attributes)
        rc = ltl_gemm_tc(A, B, C, nullptr, M, N, K, c_dtype, tile_n & 0xFFFF, (tile_n >> 16) & 3, (tile_n >> 20) & 0xFF, g_stream);
    cudaEventRecord(e0, g_stream);
    for (int i = 0; i < iters && rc == LTL_OK; ++i)
        rc = ltl_gemm_tc(A, B, C, nullptr, M, N, K, c_dtype, tile_n & 0xFFFF, (tile_n >> 16) & 3, (tile_n >> 20) & 0xFF, g_stream);
    cudaEventRecord(e1, g_stream);
    const cudaError_t se = cudaStreamSynchronize(g_stream);
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    if (rc != LTL_OK) return rc;
    if (se != cudaSuccess) return ltl_cuda_fail("gemm_bf16_tc_time", se);
    *ms_per_launch = ms / (float)iters;
    return ltl_gemm_tc_check(g_stream);
}
// Fused causal attention over a packed qkv [B*T, 3*H*hd] (q | k | v per row).  impl: 0 = choose, 1 = CUDA cores,
// 2 = tensor cores (bf16, head_dim 64 / 128, T a multiple of 8).
int luaTL_attention_fwd(const void* qkv, void* out, float* lse, int B, int T, int H, int hd, float scale, int causal,
                        int dtype, int impl)
{
    LTL_TRY(ltl_require_init("attention_fwd"));
    const bool tc_ok = ltl_attn_tc_supported(T, H, hd, dtype);
    if (impl == 2 && !tc_ok) return ltl_fail(LTL_ERR_UNSUPPORTED, "attention_fwd: the tensor-core kernel needs bf16, head_dim 64 or 128 and T %% 8 == 0");
    if (impl == 2 || (impl == 0 && tc_ok)) {
        LTL_TRY(ltl_attn_fwd_tc(qkv, out, lse, B, T, H, hd, scale, causal, g_stream));
        LTL_TRY(sync_stream("attention_fwd"));
        return ltl_gemm_tc_check(g_stream);
    }
    ONE_SHOT("attention_fwd", ltl_attn_fwd(qkv, out, lse, B, T, H, hd, scale, causal, dtype, g_stream));
}
// Backward of luaTL_attention_fwd: dqkv [B*T, 3*H*hd] from out, dout [B*T, H*hd] and lse [B*H*T].
int luaTL_attention_bwd(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv, int B, int T,
                        int H, int hd, float scale, int causal, int dtype, int impl)
{
    LTL_TRY(ltl_require_init("attention_bwd"));
    const bool tc_ok = ltl_attn_tc_supported(T, H, hd, dtype);
    if (impl == 2 && !tc_ok) return ltl_fail(LTL_ERR_UNSUPPORTED, "attention_bwd: the tensor-core kernels need bf16, head_dim 64 or 128 and T %% 8 == 0");
    const bool tc = impl == 2 || (impl == 0 && tc_ok);
    float* delta = nullptr;
    LTL_CUDA("attention_bwd scratch", cudaMalloc(&delta, (size_t)B * H * T * 4));
    int rc = tc ? ltl_attn_bwd_tc(qkv, out, dout, lse, delta, dqkv, B, T, H, hd, scale, causal, g_stream)
                : ltl_attn_bwd(qkv, out, dout, lse, delta, dqkv, B, T, H, hd, scale, causal, dtype, g_stream);
    if (rc == LTL_OK) rc = sync_stream("attention_bwd");
    cudaFree(delta);
    LTL_TRY(rc);
    return tc ? ltl_gemm_tc_check(g_stream) : LTL_OK;
}
int luaTL_gemm_tf32_tc(const float* A, const float* B, float* C, const float* R, int M, int N, int K, int accumulate, int ksplit)
{
    LTL_TRY(ltl_require_init("gemm_tf32_tc"));
    LTL_TRY(ltl_gemm_tf32(A, B, C, R, M, N, K, accumulate, ksplit, g_stream));
    LTL_TRY(sync_stream("gemm_tf32_tc"));
    return g_deferred ? LTL_OK : ltl_gemm_tc_check(g_stream);
}
int luaTL_sgd(float* w, const float* g, uint64_t n, float lr, float wd, const float* nsq, float max_norm)
{
    ONE_SHOT("sgd", ltl_sgd(w, g, nullptr, n, lr, wd, nsq, max_norm, g_stream));
}

}  // extern "C"
