// Data-parallel gradient exchange: one NCCL all-reduce (sum) over the flat gradient buffer,
// between the backward and the optimizer kernel.  The reference is single-GPU and has no
// collective at all; this is the one exchange step data-parallel training needs.
//
// NCCL is resolved at run time (dlopen of libnccl.so.2) so that the library loads on hosts
// without it; only the calls below need it.  One communicator per process, one process per GPU.
#include <dlfcn.h>
#include <string.h>

#include "../../include/luatl_b200.h"
#include "common.cuh"

namespace {

typedef struct { char internal[128]; } nccl_uid;
typedef void* nccl_comm;
typedef int (*fn_get_uid)(nccl_uid*);
typedef int (*fn_init_rank)(nccl_comm*, int, nccl_uid, int);
typedef int (*fn_allreduce)(const void*, void*, size_t, int, int, nccl_comm, cudaStream_t);
typedef int (*fn_destroy)(nccl_comm);
typedef const char* (*fn_errstr)(int);

void* g_lib = nullptr;
fn_get_uid p_get_uid = nullptr;
fn_init_rank p_init_rank = nullptr;
fn_allreduce p_allreduce = nullptr;
fn_destroy p_destroy = nullptr;
fn_errstr p_errstr = nullptr;
nccl_comm g_comm = nullptr;
int g_world = 1, g_rank = 0;

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
    LTL_CUDA("comm_allreduce sync", cudaStreamSynchronize(ltl_default_stream()));
    return LTL_OK;
}

void luaTL_comm_destroy(void)
{
    if (g_comm && p_destroy) p_destroy(g_comm);
    g_comm = nullptr; g_world = 1; g_rank = 0;
}

}  // extern "C"
