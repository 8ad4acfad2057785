// Program: the wide command buffer the LuaJIT host fills field by field, its interpreter and
// the CUDA-graph capture / replay around it.  Behaviour follows the reference
// (cuda/luaTL_train.cu:1346-1712): ops run in order on the Program's own non-blocking stream,
// a failing op stops the run with "prog_run: op i (opcode k) failed: ...", bit 0 of `flags`
// asks for a stream synchronise at the end, SYNC ops are skipped while capturing.
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "../../include/luatl_b200.h"
#include "ops.h"

#include <unordered_map>

// Scratch of a Program's ops (the dgamma partials of RMSNORM_BWD).  Every Program owns its buffer: a captured graph
// carries the pointer as a kernel argument, so it must not move when another Program or an immediate call needs more,
// and Programs run on their own streams, so a shared buffer would race.  luaTL_prog_t is laid out by the host
// language, hence the side table.  The buffer grows only in prog_run / prog_capture (never inside a capture); growing
// drops the Program's captured graph.
struct ProgScratch { float* p = nullptr; size_t floats = 0; };
static std::unordered_map<const luaTL_prog_t*, ProgScratch> g_prog_scratch;

static void free_scratch(const luaTL_prog_t* P)
{
    auto it = g_prog_scratch.find(P);
    if (it == g_prog_scratch.end()) return;
    if (it->second.p) cudaFree(it->second.p);
    g_prog_scratch.erase(it);
}

static int prepare_scratch(luaTL_prog_t* P, float** ws)
{
    size_t need = 0;
    for (int i = 0; i < P->count; ++i) {
        const luaTL_op_t* c = &P->ops[i];
        if (c->op == LUATL_P_RMSNORM_BWD && c->p4 && c->i1 > 0) {
            const size_t n = ltl_rmsnorm_bwd_scratch_floats(c->i1);
            if (n > need) need = n;
        }
    }
    *ws = nullptr;
    if (!need) return LTL_OK;
    ProgScratch& sc = g_prog_scratch[P];
    if (need > sc.floats) {
        cudaStreamSynchronize((cudaStream_t)P->stream);
        luaTL_prog_graph_free(P);                      // the old pointer is baked into the captured nodes
        if (sc.p) cudaFree(sc.p);
        sc.p = nullptr; sc.floats = 0;
        if (cudaMalloc(&sc.p, need * sizeof(float)) != cudaSuccess) {
            cudaGetLastError();
            return ltl_fail(LTL_ERR_OOM, "prog: cudaMalloc of %zu scratch bytes failed", need * sizeof(float));
        }
        sc.floats = need;
    }
    *ws = sc.p;
    return LTL_OK;
}

static int exec_op(const luaTL_op_t* c, float* ws, cudaStream_t s)
{
    switch (c->op) {
    case LUATL_P_NOP: return LTL_OK;
    case LUATL_P_GEMM: {
        if (c->i0 <= 0 || c->i1 <= 0 || c->i2 <= 0) return ltl_fail(LTL_ERR_SHAPE, "gemm: bad shape %dx%dx%d", c->i0, c->i1, c->i2);
        // p4 = gamma, p5 = rowscale, f2 = eps of the RMSNorm prologue (cuda/luaTL_train.cu:1353-1359)
        GemmDesc g = { c->p0, c->p1, c->p2, c->p3, nullptr, c->i0, c->i1, c->i2, c->i3 > 0 ? c->i3 : 1,
                       c->s0, c->s1, c->s2, c->s3, c->s4, c->s5, c->s6, c->s7, c->s8, c->f0, c->f1, c->act,
                       c->dtype, c->dtype, c->dtype, c->pre, c->p4, (const float*)c->p5, c->f2 };
        return ltl_gemm_simt(g, s);
    }
    case LUATL_P_EW:
        if (c->n == 0) return LTL_OK;
        return ltl_elementwise(c->p0, c->p1, c->p2, c->n, c->dtype, c->i0, c->f0, c->f1, s);
    case LUATL_P_RMSNORM:
        return ltl_rmsnorm(c->p0, c->p1, c->p2, c->i0, c->i1, c->f0, c->dtype, s);
    case LUATL_P_RMSNORM_BWD:
        return ltl_rmsnorm_bwd(c->p0, c->p1, c->p2, c->p3, (float*)c->p4, c->i0, c->i1, c->f0, c->dtype, ws, s);
    case LUATL_P_SOFTMAX:
        return ltl_softmax(c->p0, c->p1, c->p2, c->i0, c->i1, c->f0, c->i2, c->i3, c->i4, c->dtype, s);
    case LUATL_P_SOFTMAX_BWD:
        return ltl_softmax_bwd(c->p0, c->p1, c->p2, c->i0, c->i1, c->f0, c->i2, c->i3, c->i4, c->dtype, s);
    case LUATL_P_SWIGLU:
        return ltl_swiglu_fwd(c->p0, c->p1, c->p2, c->i0, c->i1, c->i2, c->i3, c->i4, c->dtype, s);
    case LUATL_P_SWIGLU_BWD:
        return ltl_swiglu_bwd(c->p0, c->p1, c->p2, c->p3, c->p4, c->i0, c->i1, c->i2, c->i3, c->i4, c->dtype, s);
    case LUATL_P_ROPE:
        return ltl_rope(c->p0, (const int32_t*)c->p1, c->i0, c->i1, c->i2, c->i3 > 0 ? c->i3 : c->i1 * c->i2,
                        c->i4, c->f0, c->i5, c->i6, c->dtype, nullptr, 0, s);
    case LUATL_P_EMBED:
        return ltl_embed_fwd((const int32_t*)c->p0, c->p1, c->p2, c->i0, c->i1, c->i2, c->dtype, s);
    case LUATL_P_EMBED_BWD:
        return ltl_embed_bwd((const int32_t*)c->p0, c->p1, (float*)c->p2, c->i0, c->i1, c->i2, c->f0, c->dtype, s);
    case LUATL_P_CE:
        return ltl_cross_entropy(c->p0, (const int32_t*)c->p1, (float*)c->p2, c->p3, nullptr, c->i0, c->i1,
                                 c->i2, c->f0, c->dtype, s);
    case LUATL_P_L2:
        if (c->n == 0) return LTL_OK;
        return ltl_l2_accum(c->p0, c->n, (float*)c->p2, c->dtype, s);
    case LUATL_P_CLIP:
        if (c->n == 0) return LTL_OK;
        return ltl_clip_by_nsq(c->p2, c->n, (const float*)c->p1, c->f0, c->dtype, s);
    case LUATL_P_ADAMW:
        if (c->n == 0) return LTL_OK;
        return ltl_adamw((float*)c->p0, c->p1, (float*)c->p2, (float*)c->p3, c->p4, c->n, c->dtype, c->f0,
                         c->f1, c->f2, c->f3, c->f4, c->i0, c->f5, s);
    case LUATL_P_SGD:      // w=p0 g=p1 nsq=p2 (optional); lr=f0 wd=f1 max_norm=f2
        if (c->n == 0) return LTL_OK;
        return ltl_sgd((float*)c->p0, (const float*)c->p1, nullptr, c->n, c->f0, c->f1, (const float*)c->p2, c->f2, s);
    case LUATL_P_ZERO:
        if (!c->p2 || c->n == 0) return LTL_OK;
        LTL_CUDA("cudaMemsetAsync", cudaMemsetAsync(c->p2, 0, (size_t)c->n, s));
        return LTL_OK;
    case LUATL_P_COPY:
        if (!c->p0 || !c->p2 || c->n == 0) return LTL_OK;
        LTL_CUDA("cudaMemcpyAsync", cudaMemcpyAsync(c->p2, c->p0, (size_t)c->n, cudaMemcpyDeviceToDevice, s));
        return LTL_OK;
    case LUATL_P_CAST:
        return ltl_cast(c->p0, c->i0, c->p2, c->i1, c->n, s);
    case LUATL_P_ARGMAX:
        return ltl_argmax_rows(c->p0, (int32_t*)c->p2, c->i0, c->i1, c->dtype, s);
    case LUATL_P_SUM:
        if (c->n == 0) return LTL_OK;
        return ltl_sum_f32((const float*)c->p0, c->n, (float*)c->p2, c->f0, s);
    case LUATL_P_SYNC:
        LTL_CUDA("cudaStreamSynchronize", cudaStreamSynchronize(s));
        return LTL_OK;
    case LUATL_P_REDUCE_COLS:      // out[c] = f0 * sum_r x[r, c] + f1 * out[c]; s0 = row stride (0: cols)
        return ltl_reduce_cols(c->p0, (float*)c->p2, c->i0, c->i1, c->s0 > 0 ? c->s0 : c->i1, c->f0, c->f1, c->dtype, s);
    case LUATL_P_TRANSPOSE:
        return ltl_transpose(c->p0, c->p2, c->i0, c->i1, c->dtype, s);
    case LUATL_P_BCAST_ADD:
        return ltl_bcast_add(c->p0, c->p1, c->p2, c->i0, c->i1, c->f0, c->dtype, s);
    case LUATL_P_GATHER:
        return ltl_gather_rows(c->p0, (const int32_t*)c->p1, c->p2, c->i0, c->i1, c->i2, c->dtype, s);
    case LUATL_P_ROWRMS:
        return ltl_row_rms(c->p0, (float*)c->p2, c->i0, c->i1, c->s0 > 0 ? c->s0 : c->i1, c->s1 > 0 ? c->s1 : 1, c->f0,
                           c->dtype, s);
    default:
        return ltl_fail(LTL_ERR_ARG, "prog: unknown opcode %d", c->op);
    }
}

static void read_timing(luaTL_prog_t* P)
{
    if (!P->timing || !P->ev_start || !P->ev_stop) return;
    float ms = 0.0f;
    if (cudaEventElapsedTime(&ms, (cudaEvent_t)P->ev_start, (cudaEvent_t)P->ev_stop) == cudaSuccess)
        P->last_ms = (double)ms;
    else
        cudaGetLastError();
}

extern "C" {

luaTL_prog_t* luaTL_prog_create(int capacity, int timing)
{
    if (ltl_require_init("prog_create") != LTL_OK) return nullptr;
    if (capacity <= 0) capacity = 4096;
    luaTL_prog_t* P = (luaTL_prog_t*)calloc(1, sizeof(luaTL_prog_t));
    luaTL_op_t* ops = (luaTL_op_t*)calloc((size_t)capacity, sizeof(luaTL_op_t));
    cudaStream_t s = nullptr;
    if (!P || !ops || cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess) {
        free(P); free(ops);
        cudaGetLastError();
        ltl_fail(LTL_ERR_OOM, "prog_create: could not allocate %d ops and a stream", capacity);
        return nullptr;
    }
    P->ops = ops; P->capacity = capacity; P->stream = s; P->owns_stream = 1;
    P->timing = timing ? 1 : 0; P->flags = 1; P->last_ms = -1.0;
    if (P->timing) {
        cudaEvent_t a = nullptr, b = nullptr;
        cudaEventCreate(&a); cudaEventCreate(&b);
        P->ev_start = a; P->ev_stop = b;
    }
    return P;
}

void luaTL_prog_graph_free(luaTL_prog_t* P)
{
    if (!P) return;
    if (P->graph_exec) { cudaGraphExecDestroy((cudaGraphExec_t)P->graph_exec); P->graph_exec = nullptr; }
    if (P->graph) { cudaGraphDestroy((cudaGraph_t)P->graph); P->graph = nullptr; }
    P->captured = 0;
    cudaGetLastError();
}

void luaTL_prog_destroy(luaTL_prog_t* P)
{
    if (!P) return;
    if (P->stream) cudaStreamSynchronize((cudaStream_t)P->stream);
    luaTL_prog_graph_free(P);
    free_scratch(P);
    if (P->ev_start) cudaEventDestroy((cudaEvent_t)P->ev_start);
    if (P->ev_stop) cudaEventDestroy((cudaEvent_t)P->ev_stop);
    if (P->stream && P->owns_stream) cudaStreamDestroy((cudaStream_t)P->stream);
    free(P->ops);
    free(P);
    cudaGetLastError();
}

void luaTL_prog_reset(luaTL_prog_t* P)
{
    if (P) { P->count = 0; P->status = LTL_OK; }
}

int luaTL_prog_push(luaTL_prog_t* P, const luaTL_op_t* op)
{
    if (!P || !op) return ltl_fail(LTL_ERR_NULL, "prog_push: null pointer");
    if (P->count >= P->capacity) return ltl_fail(LTL_ERR_CAPACITY, "prog_push: program full (%d)", P->capacity);
    P->ops[P->count++] = *op;
    return LTL_OK;
}

static int finish_run(luaTL_prog_t* P, cudaStream_t s, const char* what)
{
    if (P->timing && P->ev_stop) cudaEventRecord((cudaEvent_t)P->ev_stop, s);
    if (P->flags & 1) {
        const cudaError_t e = cudaStreamSynchronize(s);
        if (e != cudaSuccess) { P->status = ltl_cuda_fail(what, e); return P->status; }
        read_timing(P);
    }
    P->total_runs++;
    P->total_ops += (uint64_t)P->count;
    P->status = LTL_OK;
    return LTL_OK;
}

int luaTL_prog_run(luaTL_prog_t* P)
{
    if (!P) return ltl_fail(LTL_ERR_NULL, "prog_run: null program");
    if (P->count <= 0) { P->status = LTL_OK; return LTL_OK; }
    if (P->count > P->capacity) {
        P->status = ltl_fail(LTL_ERR_CAPACITY, "prog_run: count %d > capacity %d", P->count, P->capacity);
        return P->status;
    }
    float* ws = nullptr;
    if ((P->status = prepare_scratch(P, &ws)) != LTL_OK) return P->status;
    cudaStream_t s = (cudaStream_t)P->stream;
    if (P->timing && P->ev_start) cudaEventRecord((cudaEvent_t)P->ev_start, s);
    for (int i = 0; i < P->count; ++i) {
        const int rc = exec_op(&P->ops[i], ws, s);
        if (rc != LTL_OK) {
            char inner[768];
            snprintf(inner, sizeof(inner), "%s", luaTL_get_last_error());
            ltl_fail(rc, "prog_run: op %d (opcode %d) failed: %s", i, P->ops[i].op, inner);
            P->status = rc;
            cudaStreamSynchronize(s);
            cudaGetLastError();
            return rc;
        }
    }
    return finish_run(P, s, "prog_run: stream sync");
}

int luaTL_prog_capture(luaTL_prog_t* P)
{
    if (!P) return ltl_fail(LTL_ERR_NULL, "prog_capture: null program");
    if (P->count <= 0) return ltl_fail(LTL_ERR_ARG, "prog_capture: empty program");
    luaTL_prog_graph_free(P);
    float* ws = nullptr;
    LTL_TRY(prepare_scratch(P, &ws));
    cudaStream_t s = (cudaStream_t)P->stream;
    LTL_CUDA("cudaStreamSynchronize(pre-capture)", cudaStreamSynchronize(s));
    LTL_CUDA("cudaStreamBeginCapture", cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    P->capturing = 1;
    int rc = LTL_OK;
    for (int i = 0; i < P->count && rc == LTL_OK; ++i) {
        if (P->ops[i].op == LUATL_P_SYNC) continue;
        rc = exec_op(&P->ops[i], ws, s);
    }
    cudaGraph_t g = nullptr;
    const cudaError_t e2 = cudaStreamEndCapture(s, &g);
    P->capturing = 0;
    if (rc != LTL_OK) { if (g) cudaGraphDestroy(g); cudaGetLastError(); return rc; }
    if (e2 != cudaSuccess) return ltl_cuda_fail("cudaStreamEndCapture", e2);
    cudaGraphExec_t ge = nullptr;
    const cudaError_t e3 = cudaGraphInstantiate(&ge, g, 0);
    if (e3 != cudaSuccess) { cudaGraphDestroy(g); return ltl_cuda_fail("cudaGraphInstantiate", e3); }
    P->graph = g; P->graph_exec = ge; P->captured = 1;
    return LTL_OK;
}

int luaTL_prog_replay(luaTL_prog_t* P)
{
    if (!P) return ltl_fail(LTL_ERR_NULL, "prog_replay: null program");
    if (!P->captured || !P->graph_exec) return luaTL_prog_run(P);
    cudaStream_t s = (cudaStream_t)P->stream;
    if (P->timing && P->ev_start) cudaEventRecord((cudaEvent_t)P->ev_start, s);
    const cudaError_t e = cudaGraphLaunch((cudaGraphExec_t)P->graph_exec, s);
    if (e != cudaSuccess) { P->status = ltl_cuda_fail("cudaGraphLaunch", e); return P->status; }
    return finish_run(P, s, "graph sync");
}

int luaTL_prog_wait(luaTL_prog_t* P)
{
    if (!P || !P->stream) return ltl_fail(LTL_ERR_NULL, "prog_wait: null program");
    LTL_CUDA("cudaStreamSynchronize", cudaStreamSynchronize((cudaStream_t)P->stream));
    read_timing(P);
    return LTL_OK;
}

}  // extern "C"
