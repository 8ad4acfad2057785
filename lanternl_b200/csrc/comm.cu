// Data-parallel gradient exchange: one NCCL all-reduce (sum) over the flat gradient buffer,
// between the backward and the optimizer kernel.  The reference is single-GPU and has no
// collective at all; this is the one exchange step data-parallel training needs.
//
// NCCL is resolved at run time (dlopen of libnccl.so.2) so that the library loads on hosts
// without it; only the calls below need it.  One communicator per process, one process per GPU.
//
// Failure handling.  A rank that never reaches the exchange would leave every other rank waiting inside the
// collective for ever.  The host therefore never blocks on a stream that carries a collective: it polls the stream
// (cudaStreamQuery) and the communicator's asynchronous error state (ncclCommGetAsyncError) until the work is done, an
// error is reported or a time limit passes (luaTL_comm_set_timeout, default 120 s, LUATL_COMM_TIMEOUT_MS); on error or
// expiry the communicator is aborted (ncclCommAbort ends its kernels), the entry point returns LUATL_ERR_CUDA and the
// process can report and leave - it does not fall back to anything.  The wait loop takes its three operations as
// function pointers, so its logic is tested on the CPU against fakes (luaTL_comm_selftest_wait).
#include <dlfcn.h>
#include <stdlib.h>
#include <string.h>
#include <sys/stat.h>
#include <time.h>

#include "../../include/luatl_b200.h"
#include "common.cuh"

namespace {

typedef struct { char internal[128]; } nccl_uid;
typedef void* nccl_comm;
typedef int (*fn_get_uid)(nccl_uid*);
typedef int (*fn_init_rank)(nccl_comm*, int, nccl_uid, int);
typedef int (*fn_allreduce)(const void*, void*, size_t, int, int, nccl_comm, cudaStream_t);
typedef int (*fn_destroy)(nccl_comm);
typedef int (*fn_abort)(nccl_comm);
typedef int (*fn_async_err)(nccl_comm, int*);
typedef const char* (*fn_errstr)(int);

void* g_lib = nullptr;
fn_get_uid p_get_uid = nullptr;
fn_init_rank p_init_rank = nullptr;
fn_allreduce p_allreduce = nullptr;
fn_destroy p_destroy = nullptr;
fn_errstr p_errstr = nullptr;
fn_abort p_abort = nullptr;            // optional (older libraries): without it the communicator is only dropped
fn_async_err p_async_err = nullptr;
nccl_comm g_comm = nullptr;
int g_world = 1, g_rank = 0;
int g_timeout_ms = -1;                 // -1: LUATL_COMM_TIMEOUT_MS or 120 s

// The three things the wait loop does, as callbacks: is the work done (0 = yes, 1 = not yet, < 0 = error), has the
// communicator reported an asynchronous error (0 = no), and tear the communicator down.
struct WaitOps {
    int (*done)(void* ctx);
    int (*async_error)(void* ctx);
    void (*abort)(void* ctx);
};

double now_ms()
{
    timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec * 1e3 + ts.tv_nsec * 1e-6;
}

// Returns LTL_OK once done() says so; LTL_ERR_CUDA after abort() when done() fails, async_error() reports one or
// `timeout_ms` passes first.
int wait_bounded(const WaitOps& ops, void* ctx, int timeout_ms, const char* what)
{
    const double t0 = now_ms();
    long polls = 0;
    for (;;) {
        const int d = ops.done(ctx);
        if (d == 0) return LTL_OK;
        if (d < 0) { ops.abort(ctx); return ltl_fail(LTL_ERR_CUDA, "comm: %s failed on the device; communicator aborted", what); }
        const int ae = ops.async_error(ctx);
        if (ae != 0) {
            ops.abort(ctx);
            return ltl_fail(LTL_ERR_CUDA, "comm: %s: the communicator reported asynchronous error %d; communicator aborted", what, ae);
        }
        const double el = now_ms() - t0;
        if (el > (double)timeout_ms) {
            ops.abort(ctx);
            return ltl_fail(LTL_ERR_CUDA, "comm: %s did not finish within %d ms (a rank did not arrive?); communicator aborted",
                            what, timeout_ms);
        }
        // back off: spin for the first polls (a step's tail is microseconds away), then sleep 50 us between polls
        if (++polls > 200) { timespec ts = { 0, 50000 }; nanosleep(&ts, nullptr); }
    }
}

int effective_timeout_ms()
{
    if (g_timeout_ms >= 0) return g_timeout_ms;
    const char* e = getenv("LUATL_COMM_TIMEOUT_MS");
    const int v = e ? atoi(e) : 0;
    return v > 0 ? v : 120000;
}

// the real operations: a CUDA stream and the NCCL communicator
int real_done(void* ctx)
{
    const cudaError_t e = cudaStreamQuery((cudaStream_t)ctx);
    if (e == cudaSuccess) return 0;
    if (e == cudaErrorNotReady) { cudaGetLastError(); return 1; }
    return -1;
}
int real_async_error(void*)
{
    if (!g_comm || !p_async_err) return 0;
    int st = 0;
    if (p_async_err(g_comm, &st) != 0) return -1;
    return (st == 0 || st == 7 /* ncclInProgress */) ? 0 : st;
}
void real_abort(void*)
{
    if (g_comm) { if (p_abort) p_abort(g_comm); g_comm = nullptr; }
    g_world = 1; g_rank = 0;
}

int load_nccl()
{
    if (g_lib) return LTL_OK;
    const char* names[] = { "libnccl.so.2", "libnccl.so" };
    for (const char* n : names) { g_lib = dlopen(n, RTLD_NOW | RTLD_GLOBAL); if (g_lib) break; }
    if (!g_lib) return ltl_fail(LTL_ERR_UNSUPPORTED, "comm: libnccl.so.2 not found (%s)", dlerror());
    p_get_uid = (fn_get_uid)dlsym(g_lib, "ncclGetUniqueId");
    p_init_rank = (fn_init_rank)dlsym(g_lib, "ncclCommInitRank");
    p_allreduce = (fn_allreduce)dlsym(g_lib, "ncclAllReduce");
    p_destroy = (fn_destroy)dlsym(g_lib, "ncclCommDestroy");
    p_errstr = (fn_errstr)dlsym(g_lib, "ncclGetErrorString");
    p_abort = (fn_abort)dlsym(g_lib, "ncclCommAbort");
    p_async_err = (fn_async_err)dlsym(g_lib, "ncclCommGetAsyncError");
    if (!p_get_uid || !p_init_rank || !p_allreduce || !p_destroy)
        return ltl_fail(LTL_ERR_UNSUPPORTED, "comm: NCCL symbols missing in libnccl.so.2");
    return LTL_OK;
}

int nccl_fail(const char* ctx, int rc)
{
    return ltl_fail(LTL_ERR_CUDA, "%s failed: %s (nccl error %d)", ctx, p_errstr ? p_errstr(rc) : "?", rc);
}

}  // namespace

int ltl_comm_world() { return g_comm ? g_world : 1; }

// Wait for `s` (a stream that carries, or waits for, a collective) without ever blocking past the time limit.
int ltl_comm_wait(cudaStream_t s, const char* what)
{
    if (!g_comm) { LTL_CUDA(what, cudaStreamSynchronize(s)); return LTL_OK; }
    const WaitOps ops = { real_done, real_async_error, real_abort };
    return wait_bounded(ops, (void*)s, effective_timeout_ms(), what);
}

int ltl_comm_allreduce(float* dev, uint64_t n, cudaStream_t s)
{
    if (!g_comm) return ltl_fail(LTL_ERR_ARG, "comm: all-reduce without a communicator (call luaTL_comm_init)");
    const int rc = p_allreduce(dev, dev, (size_t)n, /*ncclFloat32*/ 7, /*ncclSum*/ 0, g_comm, s);
    return rc == 0 ? LTL_OK : nccl_fail("ncclAllReduce", rc);
}

extern "C" {

int luaTL_comm_unique_id(char* id128)
{
    if (!id128) return ltl_fail(LTL_ERR_NULL, "comm_unique_id: null buffer");
    LTL_TRY(load_nccl());
    nccl_uid u;
    const int rc = p_get_uid(&u);
    if (rc != 0) return nccl_fail("ncclGetUniqueId", rc);
    memcpy(id128, u.internal, 128);
    return LTL_OK;
}

int luaTL_comm_init(const char* id128, int world, int rank)
{
    if (!id128) return ltl_fail(LTL_ERR_NULL, "comm_init: null id");
    if (world < 1 || rank < 0 || rank >= world) return ltl_fail(LTL_ERR_ARG, "comm_init: rank %d of %d", rank, world);
    LTL_TRY(ltl_require_init("comm_init"));
    LTL_TRY(load_nccl());
    if (g_comm) { p_destroy(g_comm); g_comm = nullptr; }
    nccl_uid u;
    memcpy(u.internal, id128, 128);
    const int rc = p_init_rank(&g_comm, world, u, rank);
    if (rc != 0) { g_comm = nullptr; return nccl_fail("ncclCommInitRank", rc); }
    g_world = world; g_rank = rank;
    return LTL_OK;
}

int luaTL_comm_world(void) { return ltl_comm_world(); }

int luaTL_comm_allreduce_f32(float* dev, uint64_t n)
{
    if (!dev) return ltl_fail(LTL_ERR_NULL, "comm_allreduce: null pointer");
    LTL_TRY(ltl_comm_allreduce(dev, n, ltl_default_stream()));
    return ltl_comm_wait(ltl_default_stream(), "all-reduce");
}

void luaTL_comm_set_timeout(int ms) { g_timeout_ms = ms; }

// Self-test of the wait loop against fakes, for hosts without a GPU.  The "collective" is done when the file
// `arrive_path` exists (another process creates it when it reaches the exchange; NULL: never); the fake communicator
// reports `async_error` (0: none) from the `error_after`-th poll on.  Returns what the real wait would: 0, or
// LUATL_ERR_CUDA with the abort recorded in *aborted.
struct FakeCtx { const char* path; int async_error, error_after, polls, aborted; };
static int fake_done(void* c)
{
    FakeCtx* f = (FakeCtx*)c;
    f->polls++;
    struct stat st;
    return (f->path && stat(f->path, &st) == 0) ? 0 : 1;
}
static int fake_async_error(void* c) { FakeCtx* f = (FakeCtx*)c; return (f->async_error && f->polls >= f->error_after) ? f->async_error : 0; }
static void fake_abort(void* c) { ((FakeCtx*)c)->aborted = 1; }
int luaTL_comm_selftest_wait(const char* arrive_path, int timeout_ms, int async_error, int error_after, int* aborted)
{
    FakeCtx f = { arrive_path, async_error, error_after, 0, 0 };
    const WaitOps ops = { fake_done, fake_async_error, fake_abort };
    const int rc = wait_bounded(ops, &f, timeout_ms, "all-reduce");
    if (aborted) *aborted = f.aborted;
    return rc;
}

void luaTL_comm_destroy(void)
{
    if (g_comm && p_destroy) p_destroy(g_comm);
    g_comm = nullptr; g_world = 1; g_rank = 0;
}

}  // extern "C"
