// The device-resident language model: flat parameter / gradient buffers, the training step
// (forward, cross-entropy, backward, optimizer), the KV-cache prefill and the greedy decode
// loop replayed as one CUDA graph per token.
//
// What it replaces: the op lists the reference's Lua host queues per step
// (ai/gpu/gpu_transformer.lua:309-391 forward, :393-488 backward, :490-517 optimizer) and its
// cache-less generate (ai/gpu/gpu_transformer.lua:677 re-runs a full [B, T] forward per
// token).  Decode semantics follow the CPU model's step() (ai/nn/transformer.lua:297-434) and
// the cache branch of generate (ai/optim/lmtrain.lua:1499-1519).
//
// Differences in structure (not in math): attention is one fused kernel per layer instead of
// 2B batched GEMMs and a [B*H*T, T] softmax; residual adds ride in the GEMM epilogue instead
// of a copy + beta = 1; all gradients live in one flat buffer (one memset, one all-reduce,
// one optimizer launch).
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <map>
#include <vector>

#include "../../include/luatl_b200.h"
#include "ops.h"

int ltl_comm_world();
int ltl_comm_allreduce(float* dev, uint64_t n, cudaStream_t s);
int ltl_comm_wait(cudaStream_t s, const char* what);

namespace {

struct TensorInfo { char name[32]; int rows, cols; int64_t off; int decay; int is_matrix; };
struct LayerOff { int64_t ln1, wqkv, wo, ln2, w13, w2; };

// Activation set.  layered = 1 keeps one copy per layer (needed by the backward).
struct Act {
    int rows_cap = 0, layered = 0;
    float* res = nullptr;        // layered: [(L+1), rows, D]; else [rows, D]
    float* mid = nullptr;        // layered only: [L, rows, D]
    void *h1 = nullptr, *qkv = nullptr, *attn = nullptr, *h2 = nullptr, *h13 = nullptr, *hs = nullptr;
    float* lse = nullptr;        // layered only: [L, B*H*T]
    void* hf = nullptr;          // [rows, D]
    float* logits = nullptr;     // [logit_rows, V]
    int logit_rows = 0;
    int32_t* posids = nullptr;   // [rows]
    int posids_T = -1, posids_rows = -1;
};

struct GraphEntry { cudaGraph_t g = nullptr; cudaGraphExec_t ge = nullptr; int64_t launches = 0;
                    const void* out = nullptr; int out_stride = 0;
                    const void* hist = nullptr; int hist_stride = 0, hist_base = 0; };

}  // namespace

struct luaTL_lm_s {
    luaTL_lm_config_t c;
    int D, H, hd, F, V, L, T, B, adt, splits;
    float scale;
    std::vector<TensorInfo> tens;
    std::vector<LayerOff> lo;
    int64_t np, off_emb, off_lnf, off_head;
    float *W = nullptr, *G = nullptr, *M1 = nullptr, *M2 = nullptr;
    bf16* Wb = nullptr;          // bf16 mirror, matrices transposed to [out, in]
    bf16* Wm = nullptr;          // second bf16 mirror for the backward: the other orientation of every matrix
    int mirror_dirty = 1;
    // fp32 model on the tensor cores (luaTL_lm_set_tf32): every matrix transposed to [out, in] in fp32 (the K-major B operand
    // of the forward products), and scratch for the transposed activations of the weight-gradient products
    int tf32 = 0;
    float* Wt = nullptr;
    float *tA = nullptr, *tB = nullptr;
    size_t tA_floats = 0, tB_floats = 0;
    int train_tc = 0;            // bf16 model that has been asked to train: mixed-precision step
    // sampling of the generation loop (temperature <= 0: greedy); captured decode graphs are specific to these values
    struct Sampling { float temperature = 0.0f; int top_k = 0; float top_p = 0.0f; uint64_t seed = 0; int stop_id = -1; } samp;
    int32_t* d_done = nullptr;   // per sequence: the stop token has been emitted
    // data-parallel gradient exchange overlapped with the backward: a layer's slice of the flat gradient is reduced
    // on its own stream as soon as that layer's backward has finished
    cudaStream_t comm_s = nullptr;
    cudaEvent_t ev_grad = nullptr, ev_comm = nullptr;
    int overlap_comm = 1;        // LUATL_OVERLAP_COMM=0: one all-reduce after the backward
    int attn_tc = 1;             // tensor-core attention where the shape allows (LUATL_ATTN_TC=0 turns it off)
    // mixed-precision backward scratch (bf16): activation gradients
    bf16 *b_dres = nullptr, *b_dhs = nullptr, *b_dh13 = nullptr, *b_dattn = nullptr, *b_dqkv = nullptr, *b_dl = nullptr;
    cudaStream_t s = nullptr;
    float2* rope_tab = nullptr;
    Act train, infer, dec;
    // backward scratch
    float *dres = nullptr, *dbr = nullptr, *dhf = nullptr, *dh1 = nullptr, *dqkv = nullptr,
          *dattn = nullptr, *dh2 = nullptr, *dh13 = nullptr, *dhs = nullptr, *delta = nullptr;
    float* losses = nullptr;
    int32_t *d_ids = nullptr, *d_tgt = nullptr, *d_pred = nullptr;
    float* ws = nullptr;         // rmsnorm_bwd partials, split-KV partials
    size_t ws_floats = 0;
    // decode state
    int nseq_cap = 0;
    void *kc = nullptr, *vc = nullptr;
    int32_t *d_pos = nullptr, *d_count = nullptr, *d_next = nullptr, *d_hist = nullptr, *d_win = nullptr,
            *d_prompt = nullptr, *d_out = nullptr;
    int hist_cap = 0, prompt_cap = 0, out_cap = 0;
    int* d_err = nullptr;
    float* xlast = nullptr;
    float* part = nullptr;       // split-K partial sums of the decode GEMMs [8][nseq_cap][D]
    float* part_q = nullptr;     // split-K partial sums of the QKV projection of the decode step [8][nseq_cap][3 D]
    float* ssq[2] = { nullptr, nullptr };   // per-row sums of squares by 32-column tile [nseq_cap][D / 32] (fused residual GEMMs)
    int* tile_tickets = nullptr; // arrival counters of the fused residual GEMMs, one per output tile, zero between launches
    unsigned* chain_bar = nullptr;   // grid barrier words of the chain kernel (arrivals, generation)
    int use_chain = 0, chain_pdl = 1;
    std::map<int, GraphEntry> graphs;
    cudaEvent_t ev[4] = { nullptr, nullptr, nullptr, nullptr };
    float prefill_ms = 0, decode_ms = 0;
    int64_t launches = 0;
    int adam_alloc = 0;
    // whole-model optimizer launch: element ranges without weight decay (the gains), on the device
    long long* d_nodecay = nullptr;
    int n_nodecay = 0, flat_opt = 0;
    // captured forward + loss + backward of the training step (luaTL_lm_set_graph)
    struct StepGraph { cudaGraph_t g = nullptr; cudaGraphExec_t ge = nullptr; int valid = 0, accumulate = 0;
                       const int32_t *ids = nullptr, *tgt = nullptr; int64_t launches = 0; } step_graph;
    int graph_steps = 0, warm_steps = 0;
    int use_tc = 1, fuse_swiglu = 0, use_pdl = 1, rows_gemm = 1, fuse_norm = 0;
    // two-halves decode loop (see generate_halves): second stream, its activation set and split-K scratch, fork / join
    // events, and the two captured steps (full: both halves; tail: the last step)
    int halves = 0, halves_min = 128;
    int split_qkv = 1;           // LUATL_DECODE_SPLIT_QKV=0: the QKV projection of small batches in one piece (A/B aid)
    int pref_rows = -1;          // rows per (sequence, head) of the decode step's L2 prefetch rider; -1: by batch size
    cudaStream_t s2 = nullptr;
    Act dec2;
    float* part2 = nullptr;
    int half_cap = 0;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    GraphEntry hgraph[2];
    int hgraph_nseq = 0;
};

namespace {

typedef luaTL_lm_s LM;

int dalloc(void** p, size_t bytes, const char* what)
{
    if (bytes == 0) bytes = 16;
    const cudaError_t e = cudaMalloc(p, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        *p = nullptr;
        return ltl_fail(LTL_ERR_OOM, "lm: cudaMalloc of %zu bytes for %s failed: %s", bytes, what, cudaGetErrorString(e));
    }
    return LTL_OK;
}
#define DALLOC(ptr, bytes, what) LTL_TRY(dalloc((void**)&(ptr), (bytes), (what)))

void add_tensor(LM* m, const char* name, int rows, int cols, int decay, int is_matrix)
{
    TensorInfo t;
    memset(&t, 0, sizeof(t));
    snprintf(t.name, sizeof(t.name), "%s", name);
    t.rows = rows; t.cols = cols; t.off = m->np; t.decay = decay; t.is_matrix = is_matrix;
    m->np += (int64_t)rows * cols;
    m->tens.push_back(t);
}

void layout_params(LM* m)
{
    char nm[32];
    m->np = 0;
    m->off_emb = 0;
    add_tensor(m, "tok_emb", m->V, m->D, 1, 0);
    m->lo.resize(m->L);
    for (int l = 0; l < m->L; ++l) {
        LayerOff& o = m->lo[l];
        snprintf(nm, sizeof(nm), "l%d.ln1", l + 1);  o.ln1 = m->np;  add_tensor(m, nm, 1, m->D, 0, 0);
        snprintf(nm, sizeof(nm), "l%d.wqkv", l + 1); o.wqkv = m->np; add_tensor(m, nm, m->D, 3 * m->D, 1, 1);
        snprintf(nm, sizeof(nm), "l%d.wo", l + 1);   o.wo = m->np;   add_tensor(m, nm, m->D, m->D, 1, 1);
        snprintf(nm, sizeof(nm), "l%d.ln2", l + 1);  o.ln2 = m->np;  add_tensor(m, nm, 1, m->D, 0, 0);
        snprintf(nm, sizeof(nm), "l%d.w13", l + 1);  o.w13 = m->np;  add_tensor(m, nm, m->D, 2 * m->F, 1, 1);
        snprintf(nm, sizeof(nm), "l%d.w2", l + 1);   o.w2 = m->np;   add_tensor(m, nm, m->F, m->D, 1, 1);
    }
    m->off_lnf = m->np;
    add_tensor(m, "lnf", 1, m->D, 0, 0);
    m->off_head = -1;
    if (!m->c.tie) { m->off_head = m->np; add_tensor(m, "head", m->D, m->V, 1, 1); }
}

size_t esz(int dt) { return ltl_dtype_size(dt); }

int alloc_act(LM* m, Act& a, int rows, int layered, int logit_rows)
{
    if (a.rows_cap >= rows && a.layered == layered && a.logit_rows >= logit_rows) return LTL_OK;
    if (a.rows_cap != 0) return ltl_fail(LTL_ERR_CAPACITY, "lm: activation set sized for %d rows, %d requested", a.rows_cap, rows);
    const size_t D = m->D, F = m->F, V = m->V, L = m->L, R = rows, e = esz(m->adt), nl = layered ? L : 1;
    DALLOC(a.res, (layered ? L + 1 : 1) * R * D * 4, "residual stream");
    if (layered) DALLOC(a.mid, L * R * D * 4, "mid residual");
    DALLOC(a.h1, nl * R * D * e, "h1");
    DALLOC(a.qkv, nl * R * 3 * D * e, "qkv");
    DALLOC(a.attn, nl * R * D * e, "attn");
    DALLOC(a.h2, nl * R * D * e, "h2");
    DALLOC(a.h13, nl * R * 2 * F * e, "h13");
    DALLOC(a.hs, nl * R * F * e, "hs");
    if (layered) DALLOC(a.lse, L * R * (size_t)m->H * 4, "lse");
    DALLOC(a.hf, R * D * e, "hf");
    DALLOC(a.logits, (size_t)logit_rows * V * 4, "logits");
    DALLOC(a.posids, R * 4, "position ids");
    a.rows_cap = rows; a.layered = layered; a.logit_rows = logit_rows;
    return LTL_OK;
}

void free_act(Act& a)
{
    cudaFree(a.res); cudaFree(a.mid); cudaFree(a.h1); cudaFree(a.qkv); cudaFree(a.attn); cudaFree(a.h2);
    cudaFree(a.h13); cudaFree(a.hs); cudaFree(a.lse); cudaFree(a.hf); cudaFree(a.logits); cudaFree(a.posids);
    a = Act();
}

__global__ void posids_kernel(int32_t* p, int rows, int T) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < rows) p[i] = i % T;
}

void drop_graphs(LM* m);

// Grows the scratch buffer.  Captured decode graphs carry the old pointer as a kernel argument (the split-KV
// partials of decode attention), so they are dropped together with the buffer they point into.
int ensure_ws(LM* m, size_t floats)
{
    if (floats <= m->ws_floats) return LTL_OK;
    LTL_CUDA("lm workspace sync", cudaStreamSynchronize(m->s));
    drop_graphs(m);
    cudaFree(m->ws); m->ws = nullptr; m->ws_floats = 0;
    DALLOC(m->ws, floats * 4, "workspace");
    m->ws_floats = floats;
    return LTL_OK;
}

bool use_attn_tc(const LM* m, int T)
{
    return m->attn_tc && m->use_tc && m->adt == LTL_BF16 && m->c.causal && ltl_attn_tc_supported(T, m->H, m->hd, LTL_BF16);
}

// bf16 mirror: matrices transposed to [out, in] (K contiguous, the layout the tensor-core
// GEMM wants for its B operand), tok_emb and gains cast in place.
int sync_mirror(LM* m)
{
    if (m->adt == LTL_F32 && m->tf32 && m->mirror_dirty) {
        if (!m->Wt) DALLOC(m->Wt, (size_t)m->np * 4, "transposed fp32 weights");
        for (const TensorInfo& t : m->tens)
            if (t.is_matrix) LTL_TRY(ltl_transpose(m->W + t.off, m->Wt + t.off, t.rows, t.cols, LTL_F32, m->s));
        m->mirror_dirty = 0;
        return LTL_OK;
    }
    if (m->adt != LTL_BF16 || !m->mirror_dirty) return LTL_OK;
    for (const TensorInfo& t : m->tens) {
        if (t.is_matrix) {
            // w13 [D, 2F]: with the fused SwiGLU epilogue its mirror rows alternate gate_j / up_j
            const int half = (m->fuse_swiglu && t.cols == 2 * m->F && t.rows == m->D && strstr(t.name, "w13")) ? m->F : 0;
            LTL_TRY(ltl_transpose_to_bf16(m->W + t.off, m->Wb + t.off, t.rows, t.cols, half, m->s));
            if (m->Wm) LTL_TRY(ltl_cast(m->W + t.off, LTL_F32, m->Wm + t.off, LTL_BF16, (uint64_t)t.rows * t.cols, m->s));
        } else {
            LTL_TRY(ltl_cast(m->W + t.off, LTL_F32, m->Wb + t.off, LTL_BF16, (uint64_t)t.rows * t.cols, m->s));
            // tok_emb [V, D] is read as [out = V, in = D] by the tied head: its other orientation is the transpose
            if (m->Wm && t.off == m->off_emb && t.rows == m->V)
                LTL_TRY(ltl_transpose_any_to_bf16(m->W + t.off, LTL_F32, m->Wm + t.off, t.rows, t.cols, m->s));
        }
    }
    m->mirror_dirty = 0;
    return LTL_OK;
}

// C[M, Nout] = A[M, K] * Wt (+ R).  Weight `w_off` is [K, Nout] row-major in the fp32 master
// and [Nout, K] in the bf16 mirror.  transposed_master = 1: the master itself is [Nout, K]
// (tok_emb used as the tied head).
int wgemm(LM* m, const void* A, int M, int K, int64_t w_off, int Nout, void* C, int c_dt, const void* R,
          int transposed_master, int epi = 0)
{
    GemmDesc g;
    memset(&g, 0, sizeof(g));
    g.A = A; g.C = C; g.R = R; g.M = M; g.N = Nout; g.K = K; g.batch = 1;
    g.a_rs = K; g.a_cs = 1; g.c_rs = Nout; g.c_cs = 1;
    g.alpha = 1.0f; g.beta = 0.0f; g.a_dtype = m->adt; g.b_dtype = m->adt; g.c_dtype = c_dt;
    m->launches++;
    if (m->adt == LTL_F32) {
        if (m->tf32 && m->Wt && c_dt == LTL_F32 && !epi) {
            // tensor cores: B = the weight as [Nout, K] (the transposed mirror, or tok_emb itself as the tied head)
            const float* Bt = transposed_master ? m->W + w_off : m->Wt + w_off;
            if (ltl_gemm_tf32_supported(A, Bt, C, M, Nout, K))
                return ltl_gemm_tf32((const float*)A, Bt, (float*)C, (const float*)R, M, Nout, K, 0, 1, m->s);
        }
        g.B = m->W + w_off;
        if (transposed_master) { g.b_rs = 1; g.b_cs = K; } else { g.b_rs = Nout; g.b_cs = 1; }
    } else {
        g.B = m->Wb + w_off;
        g.b_rs = 1; g.b_cs = K;
        // bf16: activations [M, K] and the mirrored weight [Nout, K] are both K-major -> tensor cores
        if (m->use_tc && ltl_gemm_tc_supported(A, g.B, M, Nout, K))
            return ltl_gemm_tc(A, g.B, C, R, M, Nout, K, c_dt, 0, epi, 1, m->s);
        if (epi) return ltl_fail(LTL_ERR_UNSUPPORTED, "lm: fused SwiGLU needs the tensor-core GEMM");
    }
    return ltl_gemm_simt(g, m->s);
}

// Scratch of the transposed operands (grown outside of any capture: the first training step sizes it).
int ensure_tscratch(LM* m, size_t a_floats, size_t b_floats)
{
    if (a_floats > m->tA_floats) {
        LTL_CUDA("scratch sync", cudaStreamSynchronize(m->s));
        cudaFree(m->tA); m->tA = nullptr; m->tA_floats = 0;
        DALLOC(m->tA, a_floats * 4, "transposed A operand");
        m->tA_floats = a_floats;
    }
    if (b_floats > m->tB_floats) {
        LTL_CUDA("scratch sync", cudaStreamSynchronize(m->s));
        cudaFree(m->tB); m->tB = nullptr; m->tB_floats = 0;
        DALLOC(m->tB, b_floats * 4, "transposed B operand");
        m->tB_floats = b_floats;
    }
    return LTL_OK;
}

// Generic fp32 strided GEMM used by the backward.
int sgemm(LM* m, const float* A, long long a_rs, long long a_cs, const float* B, long long b_rs, long long b_cs,
          float* C, int M, int N, int K, float beta)
{
    m->launches++;
    if (m->tf32 && (beta == 0.0f || beta == 1.0f)) {
        // Tensor cores want both operands with the contraction index contiguous.  An operand given the other way round
        // (dW = X^T dY reads token-major activations down their rows) is transposed into scratch first.
        const bool a_k = a_cs == 1 && a_rs == K, a_mn = a_rs == 1 && a_cs == M;
        const bool b_k = b_rs == 1 && b_cs == K, b_mn = b_cs == 1 && b_rs == N;
        if ((a_k || a_mn) && (b_k || b_mn) && K % 4 == 0 && M % 4 == 0 && N % 4 == 0) {
            const float *Ak = A, *Bk = B;
            if (a_mn) {
                LTL_TRY(ensure_tscratch(m, (size_t)M * K, 0));
                LTL_TRY(ltl_transpose(A, m->tA, K, M, LTL_F32, m->s));       // stored [K, M] -> [M, K]
                Ak = m->tA;
                m->launches++;
            }
            if (b_mn) {
                LTL_TRY(ensure_tscratch(m, 0, (size_t)N * K));
                LTL_TRY(ltl_transpose(B, m->tB, K, N, LTL_F32, m->s));       // stored [K, N] -> [N, K]
                Bk = m->tB;
                m->launches++;
            }
            if (ltl_gemm_tf32_supported(Ak, Bk, C, M, N, K))
                return ltl_gemm_tf32(Ak, Bk, C, nullptr, M, N, K, beta == 1.0f ? 1 : 0, 0, m->s);
        }
    }
    GemmDesc g;
    memset(&g, 0, sizeof(g));
    g.A = A; g.B = B; g.C = C; g.M = M; g.N = N; g.K = K; g.batch = 1;
    g.a_rs = a_rs; g.a_cs = a_cs; g.b_rs = b_rs; g.b_cs = b_cs; g.c_rs = N; g.c_cs = 1;
    g.alpha = 1.0f; g.beta = beta;
    return ltl_gemm_simt(g, m->s);
}

inline char* layer_ptr(void* base, const Act& a, int l, size_t elems_per_layer, size_t e)
{
    return (char*)base + (a.layered ? (size_t)l * elems_per_layer * e : 0);
}

enum { MODE_TRAIN = 0, MODE_PREFILL = 1 };

// Forward over nseq sequences of T tokens (ids on the device).  TRAIN: keep every layer's
// activations and produce logits for all rows.  PREFILL: single activation set, K/V stored
// in the cache, logits only for the last position of each sequence.
int forward(LM* m, Act& a, const int32_t* d_ids, int nseq, int T, int mode)
{
    const int D = m->D, F = m->F, V = m->V, L = m->L, H = m->H, hd = m->hd, adt = m->adt;
    const int rows = nseq * T;
    const size_t e = esz(adt);
    if (rows > a.rows_cap) return ltl_fail(LTL_ERR_CAPACITY, "lm forward: %d rows exceed the buffers (%d)", rows, a.rows_cap);
    if (T > m->T) return ltl_fail(LTL_ERR_SHAPE, "lm forward: %d tokens exceed max_seq %d", T, m->T);
    LTL_TRY(sync_mirror(m));
    if (a.posids_T != T || a.posids_rows != rows) {
        posids_kernel<<<(rows + 255) / 256, 256, 0, m->s>>>(a.posids, rows, T);
        a.posids_T = T; a.posids_rows = rows;
    }
    const size_t RD = (size_t)a.rows_cap * D;
    const void* table = adt == LTL_F32 ? (const void*)(m->W + m->off_emb) : (const void*)(m->Wb + m->off_emb);
    LTL_TRY(ltl_lm_embed(d_ids, table, adt, a.res, rows, D, V, m->s));
    m->launches++;
    for (int l = 0; l < L; ++l) {
        const LayerOff& o = m->lo[l];
        float* xin = a.layered ? a.res + (size_t)l * RD : a.res;
        float* mid = a.layered ? a.mid + (size_t)l * RD : a.res;
        float* xout = a.layered ? a.res + (size_t)(l + 1) * RD : a.res;
        void* h1 = layer_ptr(a.h1, a, l, RD, e);
        void* qkv = layer_ptr(a.qkv, a, l, 3 * RD, e);
        void* attn = layer_ptr(a.attn, a, l, RD, e);
        void* h2 = layer_ptr(a.h2, a, l, RD, e);
        void* h13 = layer_ptr(a.h13, a, l, (size_t)a.rows_cap * 2 * F, e);
        void* hs = layer_ptr(a.hs, a, l, (size_t)a.rows_cap * F, e);
        float* lse = a.layered ? a.lse + (size_t)l * a.rows_cap * H : nullptr;

        LTL_TRY(ltl_lm_rmsnorm(xin, m->W + o.ln1, h1, adt, rows, D, m->c.eps, m->s));
        LTL_TRY(wgemm(m, h1, rows, D, o.wqkv, 3 * D, qkv, adt, nullptr, 0));
        if (m->c.use_rope)
            LTL_TRY(ltl_rope(qkv, a.posids, rows, 2 * H, hd, 3 * D, 0, m->c.rope_base, m->c.rope_interleaved, 0,
                             adt, m->rope_tab, m->T, m->s));
        if (use_attn_tc(m, T)) {
            LTL_TRY(ltl_attn_fwd_tc(qkv, attn, lse, nseq, T, H, hd, m->scale, 1, m->s));
            m->launches++;
        } else {
            LTL_TRY(ltl_attn_fwd(qkv, attn, lse, nseq, T, H, hd, m->scale, m->c.causal, adt, m->s));
        }
        if (mode == MODE_PREFILL) {
            const size_t cl = (size_t)m->nseq_cap * H * m->T * hd * e;
            LTL_TRY(ltl_kv_store(qkv, (char*)m->kc + l * cl, (char*)m->vc + l * cl, nseq, T, H, hd, m->T, adt, m->s));
            m->launches++;
        }
        LTL_TRY(wgemm(m, attn, rows, D, o.wo, D, mid, LTL_F32, xin, 0));
        LTL_TRY(ltl_lm_rmsnorm(mid, m->W + o.ln2, h2, adt, rows, D, m->c.eps, m->s));
        if (m->fuse_swiglu) {
            LTL_TRY(wgemm(m, h2, rows, D, o.w13, 2 * F, hs, adt, nullptr, 0, 1));
            m->launches += 4;
        } else {
            LTL_TRY(wgemm(m, h2, rows, D, o.w13, 2 * F, h13, adt, nullptr, 0));
            LTL_TRY(ltl_swiglu_fwd(h13, (char*)h13 + (size_t)F * e, hs, rows, F, 2 * F, 2 * F, F, adt, m->s));
            m->launches += 5;
        }
        LTL_TRY(wgemm(m, hs, rows, F, o.w2, D, xout, LTL_F32, mid, 0));
    }
    const float* xf = a.layered ? a.res + (size_t)L * RD : a.res;
    int lrows = rows;
    if (mode == MODE_PREFILL) {
        LTL_TRY(ltl_gather_last_rows(xf, m->xlast, nseq, T, D, T - 1, m->s));
        xf = m->xlast; lrows = nseq;
        m->launches++;
    }
    if (lrows > a.logit_rows) return ltl_fail(LTL_ERR_CAPACITY, "lm forward: %d logit rows exceed the buffer (%d)", lrows, a.logit_rows);
    LTL_TRY(ltl_lm_rmsnorm(xf, m->W + m->off_lnf, a.hf, adt, lrows, D, m->c.eps, m->s));
    m->launches++;
    if (m->c.tie) LTL_TRY(wgemm(m, a.hf, lrows, D, m->off_emb, V, a.logits, LTL_F32, nullptr, 1));
    else LTL_TRY(wgemm(m, a.hf, lrows, D, m->off_head, V, a.logits, LTL_F32, nullptr, 0));
    return LTL_OK;
}

int alloc_backward(LM* m)
{
    if (m->dres) return LTL_OK;
    const size_t R = (size_t)m->B * m->T, D = m->D, F = m->F;
    DALLOC(m->dres, R * D * 4, "dres"); DALLOC(m->dbr, R * D * 4, "dbr"); DALLOC(m->dhf, R * D * 4, "dhf");
    DALLOC(m->dh1, R * D * 4, "dh1"); DALLOC(m->dqkv, R * 3 * D * 4, "dqkv"); DALLOC(m->dattn, R * D * 4, "dattn");
    DALLOC(m->dh2, R * D * 4, "dh2"); DALLOC(m->dh13, R * 2 * F * 4, "dh13"); DALLOC(m->dhs, R * F * 4, "dhs");
    DALLOC(m->delta, R * m->H * 4, "delta");
    return LTL_OK;
}

// Backward of the fp32 model; dlogits already sits in a.logits.  Gradients accumulate into G.
int backward(LM* m, Act& a, const int32_t* d_ids, int nseq, int T)
{
    const int D = m->D, F = m->F, V = m->V, L = m->L, H = m->H, hd = m->hd;
    const int rows = nseq * T;
    const size_t RD = (size_t)a.rows_cap * D;
    float* W = m->W; float* G = m->G;
    const float* dl = a.logits;
    const float* hf = (const float*)a.hf;
    LTL_TRY(ensure_ws(m, ltl_rmsnorm_bwd_scratch_floats(D)));
    if (m->c.tie) {
        LTL_TRY(sgemm(m, dl, 1, V, hf, D, 1, G + m->off_emb, V, D, rows, 1.0f));       // dEmb += dl^T hf
        LTL_TRY(sgemm(m, dl, V, 1, W + m->off_emb, D, 1, m->dhf, rows, D, V, 0.0f));   // dhf = dl emb
    } else {
        LTL_TRY(sgemm(m, hf, 1, D, dl, V, 1, G + m->off_head, D, V, rows, 1.0f));      // dHead += hf^T dl
        LTL_TRY(sgemm(m, dl, V, 1, W + m->off_head, 1, V, m->dhf, rows, D, V, 0.0f));  // dhf = dl head^T
    }
    LTL_TRY(ltl_rmsnorm_bwd(a.res + (size_t)L * RD, W + m->off_lnf, m->dhf, m->dres, G + m->off_lnf, rows, D,
                            m->c.eps, LTL_F32, m->ws, m->s));
    m->launches += 2;
    for (int l = L - 1; l >= 0; --l) {
        const LayerOff& o = m->lo[l];
        const float* xin = a.res + (size_t)l * RD;
        const float* mid = a.mid + (size_t)l * RD;
        const float* h1 = (const float*)a.h1 + (size_t)l * RD;
        const float* qkv = (const float*)a.qkv + (size_t)l * 3 * RD;
        const float* attn = (const float*)a.attn + (size_t)l * RD;
        const float* h2 = (const float*)a.h2 + (size_t)l * RD;
        const float* h13 = (const float*)a.h13 + (size_t)l * a.rows_cap * 2 * F;
        const float* hs = (const float*)a.hs + (size_t)l * a.rows_cap * F;
        const float* lse = a.lse + (size_t)l * a.rows_cap * H;

        // feed-forward
        LTL_TRY(sgemm(m, m->dres, D, 1, W + o.w2, 1, D, m->dhs, rows, F, D, 0.0f));          // dhs = dres W2^T
        LTL_TRY(sgemm(m, hs, 1, F, m->dres, D, 1, G + o.w2, F, D, rows, 1.0f));              // dW2 += hs^T dres
        LTL_TRY(ltl_swiglu_bwd(h13, h13 + F, m->dhs, m->dh13, m->dh13 + F, rows, F, 2 * F, 2 * F, F, LTL_F32, m->s));
        LTL_TRY(sgemm(m, h2, 1, D, m->dh13, 2 * F, 1, G + o.w13, D, 2 * F, rows, 1.0f));     // dW13 += h2^T dh13
        LTL_TRY(sgemm(m, m->dh13, 2 * F, 1, W + o.w13, 1, 2 * F, m->dh2, rows, D, 2 * F, 0.0f));
        LTL_TRY(ltl_rmsnorm_bwd(mid, W + o.ln2, m->dh2, m->dbr, G + o.ln2, rows, D, m->c.eps, LTL_F32, m->ws, m->s));
        LTL_TRY(ltl_elementwise(m->dres, m->dbr, m->dres, (uint64_t)rows * D, LTL_F32, 6, 1.0f, 0.0f, m->s));
        // attention
        LTL_TRY(sgemm(m, m->dres, D, 1, W + o.wo, 1, D, m->dattn, rows, D, D, 0.0f));        // dattn = dres Wo^T
        LTL_TRY(sgemm(m, attn, 1, D, m->dres, D, 1, G + o.wo, D, D, rows, 1.0f));            // dWo += attn^T dres
        LTL_TRY(ltl_attn_bwd(qkv, attn, m->dattn, lse, m->delta, m->dqkv, nseq, T, H, hd, m->scale, m->c.causal,
                             LTL_F32, m->s));
        if (m->c.use_rope)
            LTL_TRY(ltl_rope(m->dqkv, a.posids, rows, 2 * H, hd, 3 * D, 0, m->c.rope_base, m->c.rope_interleaved, 1,
                             LTL_F32, m->rope_tab, m->T, m->s));
        LTL_TRY(sgemm(m, h1, 1, D, m->dqkv, 3 * D, 1, G + o.wqkv, D, 3 * D, rows, 1.0f));    // dWqkv += h1^T dqkv
        LTL_TRY(sgemm(m, m->dqkv, 3 * D, 1, W + o.wqkv, 1, 3 * D, m->dh1, rows, D, 3 * D, 0.0f));
        LTL_TRY(ltl_rmsnorm_bwd(xin, W + o.ln1, m->dh1, m->dbr, G + o.ln1, rows, D, m->c.eps, LTL_F32, m->ws, m->s));
        LTL_TRY(ltl_elementwise(m->dres, m->dbr, m->dres, (uint64_t)rows * D, LTL_F32, 6, 1.0f, 0.0f, m->s));
        m->launches += 12;
    }
    LTL_TRY(ltl_embed_bwd(d_ids, m->dres, G + m->off_emb, rows, D, V, 1.0f, LTL_F32, m->s));
    m->launches++;
    return LTL_OK;
}

// ---------------- mixed-precision backward (bf16 model) ----------------------------------------
// The saved activations are bf16, the residual stream and its gradient fp32, the weight gradients fp32.
// Every contraction runs on the tensor-core GEMM, which takes both operands with the contraction
// dimension contiguous:
//   dX[R, in]  = dY[R, out] . W[in, out]^T     B = the second weight mirror (Wm, master orientation)
//   dW[in, out] += X[R, in]^T . dY[R, out]      both operands MN-major (read as they lie, no transpose),
//                                               accumulated into G by the split-K atomic epilogue.
int alloc_backward_tc(LM* m)
{
    if (m->b_dres) return LTL_OK;
    const size_t R = (size_t)m->B * m->T, D = m->D, F = m->F, V = m->V;
    if (!m->dres) {
        DALLOC(m->dres, R * D * 4, "dres"); DALLOC(m->dbr, R * D * 4, "dbr"); DALLOC(m->dhf, R * D * 4, "dhf");
        DALLOC(m->dh1, R * D * 4, "dh1"); DALLOC(m->dh2, R * D * 4, "dh2"); DALLOC(m->delta, R * m->H * 4, "delta");
    }
    DALLOC(m->b_dres, R * D * 2, "dres bf16"); DALLOC(m->b_dhs, R * F * 2, "dhs bf16");
    DALLOC(m->b_dh13, R * 2 * F * 2, "dh13 bf16"); DALLOC(m->b_dattn, R * D * 2, "dattn bf16");
    DALLOC(m->b_dqkv, R * 3 * D * 2, "dqkv bf16"); DALLOC(m->b_dl, R * V * 2, "dlogits bf16");
    return LTL_OK;
}

// dW[wr, wc] += X^T . dY with X [R, wr] and dY [R, wc] bf16: both operands are read as they lie (MN-major).
int dw_gemm(LM* m, const void* X, int wr, const void* dY, int wc, float* dW, int R)
{
    m->launches++;
    return ltl_gemm_tc_xty(X, dY, dW, wr, wc, R, ltl_gemm_tc_plan_accum(wr, wc, R, 128), m->s);
}
// dX[R, n_in] = dY[R, n_out] . Wt^T with Wt = the mirror that holds the weight as [n_in, n_out].
int dx_gemm(LM* m, const bf16* dY, int n_out, const bf16* Wt, int n_in, void* dX, int dx_dt, int R)
{
    m->launches++;
    return ltl_gemm_tc(dY, Wt, dX, nullptr, R, n_in, n_out, dx_dt, 0, 0, 1, m->s);
}

// Queues an all-reduce of G[off, off + count) on the communication stream, after everything queued so far on the
// compute stream (the kernels that produced that slice).
int reduce_slice(LM* m, int64_t off, int64_t count)
{
    if (!m->comm_s) {
        LTL_CUDA("comm stream", cudaStreamCreateWithFlags(&m->comm_s, cudaStreamNonBlocking));
        LTL_CUDA("comm event", cudaEventCreateWithFlags(&m->ev_grad, cudaEventDisableTiming));
        LTL_CUDA("comm event", cudaEventCreateWithFlags(&m->ev_comm, cudaEventDisableTiming));
    }
    LTL_CUDA("comm record", cudaEventRecord(m->ev_grad, m->s));
    LTL_CUDA("comm wait", cudaStreamWaitEvent(m->comm_s, m->ev_grad, 0));
    return ltl_comm_allreduce(m->G + off, (uint64_t)count, m->comm_s);
}

int backward_tc(LM* m, Act& a, const int32_t* d_ids, int nseq, int T, bool dl_in_bf16, bool overlap_allreduce)
{
    const int D = m->D, F = m->F, V = m->V, L = m->L, H = m->H, hd = m->hd;
    const int rows = nseq * T;
    const size_t RD = (size_t)a.rows_cap * D;
    float* W = m->W; float* G = m->G;
    LTL_TRY(ensure_ws(m, ltl_rmsnorm_bwd_scratch_floats(D)));
    // head: dlogits (fp32, in a.logits) -> bf16, unless the loss kernel already wrote it there
    if (!dl_in_bf16) LTL_TRY(ltl_cast(a.logits, LTL_F32, m->b_dl, LTL_BF16, (uint64_t)rows * V, m->s));
    if (m->c.tie) {
        LTL_TRY(dw_gemm(m, m->b_dl, V, a.hf, D, G + m->off_emb, rows));         // dEmb += dl^T hf
        LTL_TRY(dx_gemm(m, m->b_dl, V, m->Wm + m->off_emb, D, m->dhf, LTL_F32, rows));              // dhf = dl emb
    } else {
        LTL_TRY(dw_gemm(m, a.hf, D, m->b_dl, V, G + m->off_head, rows));        // dHead += hf^T dl
        LTL_TRY(dx_gemm(m, m->b_dl, V, m->Wm + m->off_head, D, m->dhf, LTL_F32, rows));             // dhf = dl head^T
    }
    LTL_TRY(ltl_rmsnorm_bwd(a.res + (size_t)L * RD, W + m->off_lnf, m->dhf, m->dres, G + m->off_lnf, rows, D,
                            m->c.eps, LTL_F32, m->ws, m->s));
    m->launches += 2;
    if (overlap_allreduce) LTL_TRY(reduce_slice(m, m->off_lnf, m->np - m->off_lnf));      // lnf (and an untied head): final
    for (int l = L - 1; l >= 0; --l) {
        const LayerOff& o = m->lo[l];
        const float* xin = a.res + (size_t)l * RD;
        const float* mid = a.mid + (size_t)l * RD;
        const bf16* h1 = (const bf16*)a.h1 + (size_t)l * RD;
        const bf16* qkv = (const bf16*)a.qkv + (size_t)l * 3 * RD;
        const bf16* attn = (const bf16*)a.attn + (size_t)l * RD;
        const bf16* h2 = (const bf16*)a.h2 + (size_t)l * RD;
        const bf16* h13 = (const bf16*)a.h13 + (size_t)l * a.rows_cap * 2 * F;
        const bf16* hs = (const bf16*)a.hs + (size_t)l * a.rows_cap * F;
        const float* lse = a.lse + (size_t)l * a.rows_cap * H;

        // feed-forward (the bf16 copy of dres is left by the previous layer's last kernel)
        if (l == L - 1) LTL_TRY(ltl_cast(m->dres, LTL_F32, m->b_dres, LTL_BF16, (uint64_t)rows * D, m->s));
        LTL_TRY(dx_gemm(m, m->b_dres, D, m->Wm + o.w2, F, m->b_dhs, LTL_BF16, rows));               // dhs = dres W2^T
        LTL_TRY(dw_gemm(m, hs, F, m->b_dres, D, G + o.w2, rows));               // dW2 += hs^T dres
        LTL_TRY(ltl_swiglu_bwd(h13, h13 + F, m->b_dhs, m->b_dh13, m->b_dh13 + F, rows, F, 2 * F, 2 * F, F, LTL_BF16, m->s));
        LTL_TRY(dw_gemm(m, h2, D, m->b_dh13, 2 * F, G + o.w13, rows));          // dW13 += h2^T dh13
        LTL_TRY(dx_gemm(m, m->b_dh13, 2 * F, m->Wm + o.w13, D, m->dh2, LTL_F32, rows));             // dh2 = dh13 W13^T
        // dres += rmsnorm_bwd(...) and its bf16 copy for the GEMMs below, in one kernel when the row width allows
        const bool fused_norm = D % 4 == 0 && D <= 4096;
        if (fused_norm) {
            LTL_TRY(ltl_rmsnorm_bwd_residual(mid, W + o.ln2, m->dh2, m->dres, m->b_dres, G + o.ln2, rows, D, m->c.eps, m->ws, m->s));
        } else {
            LTL_TRY(ltl_rmsnorm_bwd(mid, W + o.ln2, m->dh2, m->dbr, G + o.ln2, rows, D, m->c.eps, LTL_F32, m->ws, m->s));
            LTL_TRY(ltl_elementwise(m->dres, m->dbr, m->dres, (uint64_t)rows * D, LTL_F32, 6, 1.0f, 0.0f, m->s));
            LTL_TRY(ltl_cast(m->dres, LTL_F32, m->b_dres, LTL_BF16, (uint64_t)rows * D, m->s));
        }
        // attention
        LTL_TRY(dx_gemm(m, m->b_dres, D, m->Wm + o.wo, D, m->b_dattn, LTL_BF16, rows));             // dattn = dres Wo^T
        LTL_TRY(dw_gemm(m, attn, D, m->b_dres, D, G + o.wo, rows));             // dWo += attn^T dres
        if (use_attn_tc(m, T)) {
            LTL_TRY(ltl_attn_bwd_tc(qkv, attn, m->b_dattn, lse, m->delta, m->b_dqkv, nseq, T, H, hd, m->scale, 1, m->s));
            m->launches += 3;
        } else {
            LTL_TRY(ltl_attn_bwd(qkv, attn, m->b_dattn, lse, m->delta, m->b_dqkv, nseq, T, H, hd, m->scale, m->c.causal,
                                 LTL_BF16, m->s));
        }
        if (m->c.use_rope)
            LTL_TRY(ltl_rope(m->b_dqkv, a.posids, rows, 2 * H, hd, 3 * D, 0, m->c.rope_base, m->c.rope_interleaved, 1,
                             LTL_BF16, m->rope_tab, m->T, m->s));
        LTL_TRY(dw_gemm(m, h1, D, m->b_dqkv, 3 * D, G + o.wqkv, rows));         // dWqkv += h1^T dqkv
        LTL_TRY(dx_gemm(m, m->b_dqkv, 3 * D, m->Wm + o.wqkv, D, m->dh1, LTL_F32, rows));            // dh1 = dqkv Wqkv^T
        if (fused_norm) {
            LTL_TRY(ltl_rmsnorm_bwd_residual(xin, W + o.ln1, m->dh1, m->dres, l > 0 ? m->b_dres : nullptr, G + o.ln1, rows, D,
                                             m->c.eps, m->ws, m->s));
        } else {
            LTL_TRY(ltl_rmsnorm_bwd(xin, W + o.ln1, m->dh1, m->dbr, G + o.ln1, rows, D, m->c.eps, LTL_F32, m->ws, m->s));
            LTL_TRY(ltl_elementwise(m->dres, m->dbr, m->dres, (uint64_t)rows * D, LTL_F32, 6, 1.0f, 0.0f, m->s));
            if (l > 0) LTL_TRY(ltl_cast(m->dres, LTL_F32, m->b_dres, LTL_BF16, (uint64_t)rows * D, m->s));
        }
        m->launches += 10;
        if (overlap_allreduce) {                         // this layer's slice [ln1 .. end of w2] is final
            const int64_t end = l + 1 < L ? m->lo[l + 1].ln1 : m->off_lnf;
            LTL_TRY(reduce_slice(m, o.ln1, end - o.ln1));
        }
    }
    LTL_TRY(ltl_embed_bwd(d_ids, m->dres, G + m->off_emb, rows, D, V, 1.0f, LTL_F32, m->s));
    m->launches++;
    if (overlap_allreduce) {
        // the embedding (it also holds the tied head's gradient) and the loss / accuracy tail come last; the compute
        // stream then waits for the communication stream before the optimizer reads G
        LTL_TRY(reduce_slice(m, m->off_emb, m->lo[0].ln1 - m->off_emb));
        LTL_TRY(reduce_slice(m, m->np, 2));
        LTL_CUDA("comm record", cudaEventRecord(m->ev_comm, m->comm_s));
        LTL_CUDA("comm wait", cudaStreamWaitEvent(m->s, m->ev_comm, 0));
    }
    return LTL_OK;
}

int count_valid(const int32_t* tgt, int n, int V)
{
    int v = 0;
    for (int i = 0; i < n; ++i) if (tgt[i] >= 0 && tgt[i] < V) ++v;
    return v;
}

int ensure_train(LM* m)
{
    const int rows = m->B * m->T;
    LTL_TRY(alloc_act(m, m->train, rows, 1, rows));
    if (!m->losses) {
        DALLOC(m->losses, (size_t)rows * 4, "losses");
        DALLOC(m->d_ids, (size_t)rows * 4, "ids");
        DALLOC(m->d_tgt, (size_t)rows * 4, "targets");
        DALLOC(m->d_pred, (size_t)rows * 4, "predictions");
    }
    return LTL_OK;
}

// tail of G: [np] loss accumulator, [np+1] correct count, [np+2] grad norm^2, [np+3] spare
int loss_and_grad(LM* m, const int32_t* d_ids, const int32_t* d_tgt, int valid_global, int want_grad, int accumulate = 0,
                  bool overlap_allreduce = false)
{
    const int rows = m->B * m->T;
    Act& a = m->train;
    const float gs = 1.0f / (float)(valid_global < 1 ? 1 : valid_global);
    if (!accumulate) LTL_CUDA("zero gradients", cudaMemsetAsync(m->G, 0, (size_t)(m->np + 4) * 4, m->s));
    LTL_TRY(forward(m, a, d_ids, m->B, m->T, MODE_TRAIN));
    // Mixed precision: the gradient of the logits is only ever read as a bf16 GEMM operand, so CE writes it as such.
    const bool dl_bf16 = want_grad && m->adt == LTL_BF16 && ltl_cross_entropy_bf16_grad_supported(a.logits, m->V);
    if (dl_bf16) {
        LTL_TRY(alloc_backward_tc(m));
        LTL_TRY(ltl_cross_entropy_bf16_grad(a.logits, d_tgt, m->losses, m->b_dl, m->d_pred, rows, m->V, -1, gs, m->s));
    } else {
        LTL_TRY(ltl_cross_entropy(a.logits, d_tgt, m->losses, want_grad ? a.logits : nullptr, m->d_pred, rows, m->V,
                                  -1, gs, LTL_F32, m->s));
    }
    LTL_TRY(ltl_sum_f32(m->losses, rows, m->G + m->np, gs, m->s));
    LTL_TRY(ltl_count_correct(m->d_pred, d_tgt, rows, m->G + m->np + 1, m->s));
    m->launches += 4;
    if (want_grad && m->adt == LTL_BF16) {
        LTL_TRY(alloc_backward_tc(m));
        LTL_TRY(backward_tc(m, a, d_ids, m->B, m->T, dl_bf16, overlap_allreduce));
    } else if (want_grad) {
        LTL_TRY(alloc_backward(m));
        LTL_TRY(backward(m, a, d_ids, m->B, m->T));
    }
    return LTL_OK;
}

void drop_step_graph(LM* m);
void drop_graphs(LM* m)
{
    drop_step_graph(m);
    for (auto& kv : m->graphs) {
        if (kv.second.ge) cudaGraphExecDestroy(kv.second.ge);
        if (kv.second.g) cudaGraphDestroy(kv.second.g);
    }
    m->graphs.clear();
    for (GraphEntry& ge : m->hgraph) {
        if (ge.ge) cudaGraphExecDestroy(ge.ge);
        if (ge.g) cudaGraphDestroy(ge.g);
        ge = GraphEntry();
    }
    m->hgraph_nseq = 0;
}

// A bf16 model asked to train: from now on the feed-forward keeps gate|up (the backward needs them), so the
// fused SwiGLU epilogue and its interleaved weight mirror are dropped, and the second mirror is kept.
int enter_train_tc(LM* m)
{
    if (m->train_tc) return LTL_OK;
    if (!m->use_tc) return ltl_fail(LTL_ERR_UNSUPPORTED, "lm train_step: the bf16 training step needs the tensor-core GEMM");
    if (m->D % 8 || m->F % 8 || m->V % 8)
        return ltl_fail(LTL_ERR_SHAPE, "lm train_step: the bf16 training step needs dim, ffn and vocab to be multiples of 8 "
                        "(got %d, %d, %d)", m->D, m->F, m->V);
    LTL_CUDA("sync", cudaStreamSynchronize(m->s));
    drop_graphs(m);
    DALLOC(m->Wm, (size_t)m->np * 2, "second bf16 weight mirror");
    m->fuse_swiglu = 0;
    m->mirror_dirty = 1;
    m->train_tc = 1;
    return LTL_OK;
}

// The forward + loss + backward of a step as one CUDA graph (what the reference's Model:capture() does for its p_step
// Program, ai/gpu/gpu_transformer.lua:714-733): captured on the first eligible step after a warm step, replayed while
// the denominator of the loss - baked into the CE and sum kernels as an argument - and the buffers are the same (the
// reference's replay rule, ai/gpu/gpu_transformer.lua:643).  The optimizer stays outside: its scalars change per step.
void drop_step_graph(LM* m)
{
    if (m->step_graph.ge) cudaGraphExecDestroy(m->step_graph.ge);
    if (m->step_graph.g) cudaGraphDestroy(m->step_graph.g);
    m->step_graph = LM::StepGraph();
}

int loss_and_grad_graphed(LM* m, const int32_t* d_ids, const int32_t* d_tgt, int valid, int accumulate)
{
    LM::StepGraph& sg = m->step_graph;
    if (sg.ge && (sg.valid != valid || sg.accumulate != accumulate || sg.ids != d_ids || sg.tgt != d_tgt)) drop_step_graph(m);
    if (sg.ge) {
        LTL_TRY(sync_mirror(m));                        // the bf16 mirrors follow the master outside the graph
        LTL_CUDA("step graph launch", cudaGraphLaunch(sg.ge, m->s));
        m->launches += sg.launches;
        return LTL_OK;
    }
    if (m->warm_steps < 2)                              // lazy allocations (activations, scratch, mirrors) must be warm
        return loss_and_grad(m, d_ids, d_tgt, valid, 1, accumulate, false);
    LTL_TRY(sync_mirror(m));
    LTL_CUDA("pre-capture sync", cudaStreamSynchronize(m->s));
    const int64_t before = m->launches;
    LTL_CUDA("begin capture", cudaStreamBeginCapture(m->s, cudaStreamCaptureModeThreadLocal));
    const int rc = loss_and_grad(m, d_ids, d_tgt, valid, 1, accumulate, false);
    cudaGraph_t g = nullptr;
    const cudaError_t ce = cudaStreamEndCapture(m->s, &g);
    if (rc != LTL_OK) { if (g) cudaGraphDestroy(g); cudaGetLastError(); return rc; }
    if (ce != cudaSuccess) return ltl_cuda_fail("end capture", ce);
    cudaGraphExec_t gx = nullptr;
    const cudaError_t ie = cudaGraphInstantiate(&gx, g, 0);
    if (ie != cudaSuccess) { cudaGraphDestroy(g); return ltl_cuda_fail("graph instantiate", ie); }
    sg.g = g; sg.ge = gx; sg.valid = valid; sg.accumulate = accumulate; sg.ids = d_ids; sg.tgt = d_tgt;
    sg.launches = m->launches - before;
    LTL_CUDA("step graph launch", cudaGraphLaunch(sg.ge, m->s));      // the capture itself executed nothing
    return LTL_OK;
}

int train_step_dev(LM* m, const int32_t* d_ids, const int32_t* d_tgt, const luaTL_lm_train_args_t* a,
                   luaTL_lm_result_t* out, int valid_local)
{
    if (a->optimizer != 0 && a->optimizer != 1) return ltl_fail(LTL_ERR_ARG, "lm train_step: unknown optimizer %d", a->optimizer);
    if (m->adt == LTL_BF16) LTL_TRY(enter_train_tc(m));
    LTL_TRY(ensure_train(m));
    const int world = ltl_comm_world();
    const int valid = a->valid_global > 0 ? a->valid_global : valid_local;
    m->launches = 0;
    LTL_CUDA("event", cudaEventRecord(m->ev[0], m->s));
    // Mixed-precision models exchange the gradient slice by slice under the backward of the step's last micro-batch
    // (a layer's slice is final once that backward has passed the layer).
    const bool exchange = world > 1 && !a->skip_allreduce;
    const bool overlap = exchange && m->adt == LTL_BF16 && m->overlap_comm;
    if (m->graph_steps && !overlap) LTL_TRY(loss_and_grad_graphed(m, d_ids, d_tgt, valid, a->accumulate));
    else LTL_TRY(loss_and_grad(m, d_ids, d_tgt, valid, 1, a->accumulate, overlap));
    if (exchange && !overlap) LTL_TRY(ltl_comm_allreduce(m->G, (uint64_t)m->np + 2, m->s));
    // The loss stays on the device until the end of the step: the optimizer kernels read it there and do nothing when
    // it is not finite (never apply a non-finite update, ai/gpu/gpu_transformer.lua:653-660) - no host round trip
    // between the backward and the update.
    const float* d_loss = m->G + m->np;
    const int need_norm = !a->no_update && a->clip_norm > 0.0f;
    if (!a->no_update) {
        float* nsq = m->G + m->np + 2;
        if (need_norm) { LTL_TRY(ltl_l2_accum(m->G, (uint64_t)m->np, nsq, LTL_F32, m->s)); m->launches++; }
        if (a->optimizer == 1 && !m->adam_alloc) {
            DALLOC(m->M1, (size_t)m->np * 4, "adam m"); DALLOC(m->M2, (size_t)m->np * 4, "adam v");
            LTL_CUDA("adam zero", cudaMemsetAsync(m->M1, 0, (size_t)m->np * 4, m->s));
            LTL_CUDA("adam zero", cudaMemsetAsync(m->M2, 0, (size_t)m->np * 4, m->s));
            m->adam_alloc = 1;
        }
        // AdamW clips the gradient in place first (cuda/luaTL_train.cu:947-952), SGD folds the factor into its update.
        if (a->optimizer == 1 && need_norm) { LTL_TRY(ltl_clip_by_nsq(m->G, (uint64_t)m->np, nsq, a->clip_norm, LTL_F32, m->s)); m->launches++; }
        if (m->flat_opt) {
            if (a->optimizer == 0)
                LTL_TRY(ltl_sgd_flat(m->W, m->G, (uint64_t)m->np, m->d_nodecay, m->n_nodecay, d_loss, need_norm ? nsq : nullptr,
                                     a->lr, a->weight_decay, a->clip_norm, m->s));
            else
                LTL_TRY(ltl_adamw_flat(m->W, m->G, m->M1, m->M2, (uint64_t)m->np, m->d_nodecay, m->n_nodecay, d_loss, a->lr,
                                       a->beta1, a->beta2, a->adam_eps, a->weight_decay, a->step, m->s));
            m->launches++;
        } else {
            // Parameter offsets off a 16-byte boundary (never the case for dim % 8 == 0): one launch per tensor, and the
            // finite test has to come to the host first.
            float l0 = 0.0f;
            LTL_CUDA("loss download", cudaMemcpyAsync(&l0, d_loss, 4, cudaMemcpyDeviceToHost, m->s));
            LTL_CUDA("loss sync", cudaStreamSynchronize(m->s));
            if (isfinite(l0))
                for (const TensorInfo& t : m->tens) {
                    const float wd = t.decay ? a->weight_decay : 0.0f;
                    if (a->optimizer == 0)
                        LTL_TRY(ltl_sgd(m->W + t.off, m->G + t.off, nullptr, (uint64_t)t.rows * t.cols, a->lr, wd,
                                        need_norm ? nsq : nullptr, a->clip_norm, m->s));
                    else
                        LTL_TRY(ltl_adamw(m->W + t.off, m->G + t.off, m->M1 + t.off, m->M2 + t.off, nullptr, (uint64_t)t.rows * t.cols,
                                          LTL_F32, a->lr, a->beta1, a->beta2, a->adam_eps, wd, a->step, 0.0f, m->s));
                    m->launches++;
                }
        }
        m->mirror_dirty = 1;
    }
    float tail[4] = { 0, 0, 0, 0 };
    LTL_CUDA("loss download", cudaMemcpyAsync(tail, m->G + m->np, need_norm ? 12 : 8, cudaMemcpyDeviceToHost, m->s));
    LTL_CUDA("event", cudaEventRecord(m->ev[1], m->s));
    // a step that exchanged gradients is waited for with a time limit (a rank that never arrives must not hang this one)
    if (exchange) LTL_TRY(ltl_comm_wait(m->s, "training step with gradient all-reduce"));
    else LTL_CUDA("step sync", cudaStreamSynchronize(m->s));
    m->warm_steps++;
    const int finite = isfinite(tail[0]) ? 1 : 0;
    const float gnorm = (finite && tail[2] > 0.0f) ? sqrtf(tail[2]) : 0.0f;
    if (out) {
        out->loss = tail[0]; out->grad_norm = gnorm; out->correct = (int)(tail[1] + 0.5f);
        out->valid = valid; out->finite = finite;
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, m->ev[0], m->ev[1]);
        out->step_ms = ms;
    }
    return LTL_OK;
}

// ---------------- decode -----------------------------------------------------------------
int ensure_decode(LM* m, int nseq, int n_prompt, int n_new)
{
    if (m->c.decode_batch <= 0) return ltl_fail(LTL_ERR_ARG, "lm: created with decode_batch = 0 (no KV cache)");
    if (nseq > m->c.decode_batch) return ltl_fail(LTL_ERR_CAPACITY, "lm: %d sequences exceed decode_batch %d", nseq, m->c.decode_batch);
    const size_t e = esz(m->adt);
    if (!m->kc) {
        m->nseq_cap = m->c.decode_batch;
        const size_t cache = (size_t)m->L * m->nseq_cap * m->H * m->T * m->hd * e;
        DALLOC(m->kc, cache, "K cache"); DALLOC(m->vc, cache, "V cache");
        DALLOC(m->d_pos, (size_t)m->nseq_cap * 4, "positions"); DALLOC(m->d_count, (size_t)m->nseq_cap * 4, "counts");
        DALLOC(m->d_next, (size_t)m->nseq_cap * 4, "next tokens"); DALLOC(m->d_err, 4, "error flag");
        DALLOC(m->d_done, (size_t)m->nseq_cap * 4, "stop flags");
        DALLOC(m->d_win, (size_t)m->nseq_cap * m->T * 4, "window ids");
        DALLOC(m->xlast, (size_t)m->nseq_cap * m->D * 4, "last rows");
        DALLOC(m->part, (size_t)8 * m->nseq_cap * m->D * 4, "split-K partial sums");
        DALLOC(m->part_q, (size_t)8 * m->nseq_cap * 3 * m->D * 4, "split-K partial sums of q | k | v");
        {
            const size_t tiles = (size_t)(m->D + 31) / 32, ntick = ((size_t)m->nseq_cap / 128 + 1) * tiles;
            DALLOC(m->ssq[0], (size_t)m->nseq_cap * tiles * 4, "row sums of squares");
            DALLOC(m->ssq[1], (size_t)m->nseq_cap * tiles * 4, "row sums of squares");
            DALLOC(m->tile_tickets, ntick * 4, "tile tickets");
            LTL_CUDA("memset", cudaMemsetAsync(m->tile_tickets, 0, ntick * 4, m->s));
            DALLOC(m->chain_bar, 16, "chain barrier");
            LTL_CUDA("memset", cudaMemsetAsync(m->chain_bar, 0, 16, m->s));
        }
        LTL_CUDA("memset", cudaMemsetAsync(m->d_pos, 0, (size_t)m->nseq_cap * 4, m->s));
        LTL_CUDA("memset", cudaMemsetAsync(m->d_count, 0, (size_t)m->nseq_cap * 4, m->s));
        LTL_CUDA("memset", cudaMemsetAsync(m->d_err, 0, 4, m->s));
        LTL_TRY(alloc_act(m, m->dec, m->nseq_cap, 0, m->nseq_cap));
        int sp = m->c.kv_splits;
        if (sp <= 0) {
            // One CTA per (sequence, head) once that gives every SM one: a second slice would add the combine
            // launch to every layer of a step that is bound by launch latency.  Fewer: slice the cache to two CTAs per SM.
            const int ctas = m->nseq_cap * m->H, sms = ltl_sm_count();
            const char* e = getenv("LUATL_KV_SPLITS");
            sp = e ? atoi(e) : (ctas >= sms ? 1 : (2 * sms + ctas - 1) / ctas);
            if (sp > 16) sp = 16;
            if (sp < 1) sp = 1;
        }
        m->splits = sp;
        LTL_TRY(ensure_ws(m, ltl_decode_attn_scratch_floats(m->nseq_cap, m->H, m->hd, sp) + 16));
    }
    if (n_prompt > 0) {
        // Window of the prefill: the prompt, or the whole context once generation can fill it.
        const int T = (n_prompt + n_new > m->T) ? m->T : n_prompt;
        if (m->infer.rows_cap < nseq * T) {
            if (m->infer.rows_cap) { LTL_CUDA("sync", cudaStreamSynchronize(m->s)); free_act(m->infer); }
            LTL_TRY(alloc_act(m, m->infer, nseq * T, 0, m->nseq_cap));
        }
        const int hist = n_prompt + n_new;
        if (m->hist_cap < m->nseq_cap * hist) {
            LTL_CUDA("sync", cudaStreamSynchronize(m->s));
            cudaFree(m->d_hist);
            DALLOC(m->d_hist, (size_t)m->nseq_cap * hist * 4, "token history");
            m->hist_cap = m->nseq_cap * hist;
        }
    }
    return LTL_OK;
}

// Greedy pick, or the sampled one when a temperature is set; both advance the sequence state on the device.
int pick_next(LM* m, const float* logits, int nseq, int slot0, int32_t* d_out, int out_stride, int32_t* hist, int hist_stride,
              int hist_base, cudaStream_t st)
{
    if (m->samp.temperature > 0.0f)
        return ltl_sample_advance(logits, nseq, m->V, m->d_next + slot0, d_out, out_stride, m->d_count + slot0, m->d_pos + slot0,
                                  hist, hist_stride, hist_base, m->samp.temperature, m->samp.top_k, m->samp.top_p, m->samp.seed,
                                  m->samp.stop_id, m->d_done ? m->d_done + slot0 : nullptr, slot0, st);
    return ltl_pick_advance(logits, nseq, m->V, m->d_next + slot0, d_out, out_stride, m->d_count + slot0, m->d_pos + slot0,
                            hist, hist_stride, hist_base, st);
}

// Decode step of the bf16 tensor-core path.  The two residual GEMMs of a layer (attention output
// and FFN down projection: N = D, few tiles) run split-K so that every SM pulls weights; their
// fp32 partial sums are added to the residual stream, in a fixed order, by the RMSNorm kernel that
// follows anyway (2 + 7 L launches per step; the default), or - fused form, LUATL_DECODE_FUSE_NORM=1 - by the
// last-arriving CTA of the GEMM itself, with the normalisation factor applied by the next GEMM's epilogue (2 + 5 L).
// cx (optional): the activation set, split-K scratch and stream of the step, and a window [op_lo, op_hi) of its launch
// sequence (numbered 0 = embed, 1 + 7 l .. 7 + 7 l = the seven launches of layer l, then head and pick) - what the
// two-halves generation loop uses to issue half a batch on its own stream and to cut a step after an attention kernel.
struct DecCtx { Act* a; float* part; cudaStream_t s; int op_lo, op_hi; };

int decode_step_split(LM* m, int nseq, int slot0, const int32_t* d_tok, int32_t* d_out, int out_stride, int pick,
                      int32_t* hist, int hist_stride, int hist_base, const DecCtx* cx = nullptr)
{
    const int D = m->D, F = m->F, V = m->V, L = m->L, H = m->H, hd = m->hd;
    const size_t e = 2;
    Act& a = cx ? *cx->a : m->dec;
    float* const part = cx ? cx->part : m->part;
    const cudaStream_t st = cx ? cx->s : m->s;
    const int op_lo = cx ? cx->op_lo : 0, op_hi = cx ? cx->op_hi : 0x7FFFFFFF;
    int opi = 0;
    auto on = [&]() { const bool r = opi >= op_lo && opi < op_hi; ++opi; return r; };
    float* x = a.res;
    const int32_t* pos = m->d_pos + slot0;
    const size_t cl = (size_t)m->nseq_cap * H * m->T * hd * e;
    const size_t cslot = (size_t)slot0 * H * m->T * hd * e;
    // Every kernel of the step is launched with programmatic stream serialization: each calls
    // griddepcontrol.wait before touching anything a kernel of the step writes, so only launch latency and
    // prologues overlap (the GEMMs also request their weights ahead of the wait: no kernel of the step writes them, and
    // what does write them - the mirror kernels after an optimizer step or a parameter upload - is separated from this
    // chain by a fully ordered operation: the token upload of a single step, or the prefill of a generation).
    struct PdlScope { bool prev; PdlScope(bool on) : prev(ltl_pdl_enabled()) { ltl_pdl_set(on); } ~PdlScope() { ltl_pdl_set(prev); } } pdl(m->use_pdl);
    // L2 prefetch rider on the second reduce of a layer: the first rows of every (sequence, head) slab of the next attention
    // kernel's cache are asked into L2 while the products run, so that kernel's first tiles arrive without the HBM ramp.
    // Measured per pass of 511 steps: 256 sequences 255.2 -> 246.3 ms with 38 rows (20 MB per layer), 251.1 with 76;
    // 128 sequences 185.7 -> 182.4 with 38 rows, 185.1 with 76; no gain at 64 sequences and fewer, where the products
    // slow down under the extra traffic by as much as the attention kernel gains.  LUATL_KV_PREFETCH_ROWS overrides.
    const int pref_rows = m->pref_rows >= 0 ? m->pref_rows : (nseq * H >= 1024 ? 40 : 0);
    int bn_o, s_o, bn_d, s_d;
    ltl_gemm_tc_plan_split(nseq, D, D, &bn_o, &s_o);
    ltl_gemm_tc_plan_split(nseq, D, F, &bn_d, &s_d);
    // Up to 32 sequences the step uses the few-row mma.sync kernel (weights prefetched ahead of the dependency wait):
    // a 128-row tcgen05 tile would be at most a quarter full and every GEMM is bound by the latency of its launch.
    // Measured per pass of 512 steps: 8 sequences 126 -> 103 ms, 16: 130 -> 112 ms, 32: 134 -> 131 ms; at 64 the
    // tcgen05 tiles win (152 vs 176 ms: four row tiles per warp and a 64 KB activation stage per CTA).
    const bool rows = m->rows_gemm && nseq <= 32 && ltl_gemm_rows_supported(a.h1, m->Wb, nseq, D, D, 1) &&
                      ltl_gemm_rows_supported(a.hs, m->Wb, nseq, D, F, 8);
    // Few rows: the QKV projection is split over K as well (every CTA then stages a quarter of the activation rows) and
    // the attention kernel adds the slices when it fetches q | k | v of its (sequence, head).  Measured per pass of 511
    // steps: 32 sequences 123.7 -> 118.7 ms (the projection 3.9 -> 2.8 us in a chain), 16 sequences 111.8 -> 110.3; not
    // with the cache cut in more than three slices (8 sequences: 102.0 -> 102.9, every slice's CTA adds the partial sums).
    int s_q = 1, bn_q = 0;
    const bool parts_ok = (!cx || cx->a == &m->dec) && m->split_qkv && m->part_q && m->splits <= 3 && ltl_decode_attn_takes_parts(hd, LTL_BF16);
    if (rows) {
        s_o = ltl_gemm_rows_plan_split(D, D, 8);
        s_d = ltl_gemm_rows_plan_split(D, F, 8);
        if (parts_ok && ltl_gemm_rows_supported(a.h1, m->Wb, nseq, 3 * D, D, 8)) s_q = ltl_gemm_rows_plan_split(3 * D, D, 8);
    } else if (parts_ok && m->split_qkv >= 2) {
        // tcgen05 tiles (LUATL_DECODE_SPLIT_QKV=2, off): the projection gets faster in a chain (4.5 -> 3.7 us at 128 rows) but the
        // attention kernel, whose every CTA then adds three slices, loses more: 128 sequences 185.6 -> 188.3 ms per pass, 64: 148.0 -> 146.7
        ltl_gemm_tc_plan_split(nseq, 3 * D, D, &bn_q, &s_q);
        if (s_q <= 1) { s_q = 1; bn_q = 0; }
    }
    auto gemm = [&](const void* A, const bf16* Wt, void* C, int N, int K, int c_dt, int bn, int epi, int ks,
                    const LtlGemmFuse* fz = nullptr) -> int {
        if (rows) return ltl_gemm_rows(A, Wt, C, nseq, N, K, c_dt, epi, ks, st, fz);
        return ltl_gemm_tc(A, Wt, C, nullptr, nseq, N, K, c_dt, bn, epi, ks, st, fz);
    };
    if (on()) {
        LTL_TRY(ltl_lm_embed_rmsnorm(d_tok, m->Wb + m->off_emb, LTL_BF16, x, m->W + m->lo[0].ln1, a.h1, LTL_BF16, nseq, D, V,
                                     m->c.eps, st));
        m->launches++;
    }
    // Fused form: the split-K reduce, the residual add and the gain of the next RMSNorm ride in the residual GEMM
    // (its last-arriving CTA per tile), the normalisation factor of a row is applied by the epilogue of the GEMM that
    // consumes it (a per-row scale commutes with the product): 5 launches per layer instead of 7.  Optional, see create.
    const bool fuse = !cx && m->fuse_norm && D % 32 == 0 && m->ssq[0] && m->tile_tickets;
    const int tiles = D / 32;
    auto resid = [&](const float* gain, void* h, int which) {
        LtlGemmFuse f = {};
        f.x = x; f.gain = gain; f.h = h; f.ssq_out = m->ssq[which]; f.counters = m->tile_tickets;
        return f;
    };
    auto scale_by = [&](int which) {
        LtlGemmFuse f = {};
        f.ssq_in = m->ssq[which]; f.ssq_tiles = tiles; f.inv_dim = 1.0f / (float)D; f.eps = m->c.eps;
        return f;
    };
    for (int l = 0; l < L; ++l) {
        const LayerOff& o = m->lo[l];
        void* kcl = (char*)m->kc + l * cl + cslot;
        void* vcl = (char*)m->vc + l * cl + cslot;
        const bool last = l + 1 == L;
        const float* next_gain = m->W + (last ? m->off_lnf : m->lo[l + 1].ln1);
        void* next_h = last ? a.hf : a.h1;
        if (fuse) {
            const LtlGemmFuse in1 = scale_by(1), in0 = scale_by(0);
            const LtlGemmFuse ro = resid(m->W + o.ln2, a.h2, 0), rd = resid(next_gain, next_h, 1);
            LTL_TRY(gemm(a.h1, m->Wb + o.wqkv, a.qkv, 3 * D, D, LTL_BF16, 0, 0, 1, l > 0 ? &in1 : nullptr));
            LTL_TRY(ltl_decode_attn(a.qkv, kcl, vcl, a.attn, pos, nseq, H, hd, m->T, m->scale, LTL_BF16, m->splits, m->ws,
                                    m->rope_tab, m->c.rope_interleaved, m->c.use_rope, m->d_err, m->s));
            LTL_TRY(gemm(a.attn, m->Wb + o.wo, m->part, D, D, LTL_F32, bn_o, 3, s_o, &ro));
            LTL_TRY(gemm(a.h2, m->Wb + o.w13, a.hs, 2 * F, D, LTL_BF16, 0, 1, 1, &in0));
            LTL_TRY(gemm(a.hs, m->Wb + o.w2, m->part, D, F, LTL_F32, bn_d, 3, s_d, &rd));
            m->launches += 5 + (m->splits > 1 ? 1 : 0);
            continue;
        }
        if (on()) {
            if (s_q > 1) LTL_TRY(gemm(a.h1, m->Wb + o.wqkv, m->part_q, 3 * D, D, LTL_F32, bn_q, 0, s_q));
            else LTL_TRY(gemm(a.h1, m->Wb + o.wqkv, a.qkv, 3 * D, D, LTL_BF16, 0, 0, 1));
            m->launches++;
        }
        if (on()) {
            LTL_TRY(ltl_decode_attn(a.qkv, kcl, vcl, a.attn, pos, nseq, H, hd, m->T, m->scale, LTL_BF16, m->splits, m->ws,
                                    m->rope_tab, m->c.rope_interleaved, m->c.use_rope, m->d_err, st,
                                    s_q > 1 ? m->part_q : nullptr, s_q > 1 ? s_q : 0));
            m->launches += 1 + (m->splits > 1 ? 1 : 0);
        }
        if (on()) { LTL_TRY(gemm(a.attn, m->Wb + o.wo, part, D, D, LTL_F32, bn_o, 0, s_o)); m->launches++; }
        if (on()) { LTL_TRY(ltl_lm_residual_rmsnorm(x, part, s_o, m->W + o.ln2, a.h2, LTL_BF16, nseq, D, m->c.eps, st)); m->launches++; }
        if (on()) { LTL_TRY(gemm(a.h2, m->Wb + o.w13, a.hs, 2 * F, D, LTL_BF16, 0, 1, 1)); m->launches++; }
        if (on()) { LTL_TRY(gemm(a.hs, m->Wb + o.w2, part, D, F, LTL_F32, bn_d, 0, s_d)); m->launches++; }
        if (on()) {
            const int ln = last ? 0 : l + 1;          // after the last layer: layer 0 of the next step, one row longer
            const LtlKvPrefetch pf = { (char*)m->kc + ln * cl + cslot, (char*)m->vc + ln * cl + cslot, pos, H, m->T, (int)(hd * e), nseq,
                                       last ? 1 : 0, pref_rows };
            LTL_TRY(ltl_lm_residual_rmsnorm(x, part, s_d, next_gain, next_h, LTL_BF16, nseq, D, m->c.eps, st,
                                            pref_rows > 0 ? &pf : nullptr));
            m->launches++;
        }
    }
    if (on()) {
        const LtlGemmFuse in1 = scale_by(1);
        LTL_TRY(gemm(a.hf, m->Wb + (m->c.tie ? m->off_emb : m->off_head), a.logits, V, D, LTL_F32, 0, 0, 1, fuse ? &in1 : nullptr));
        m->launches++;
    }
    if (pick && on()) {
        LTL_TRY(pick_next(m, a.logits, nseq, slot0, d_out, out_stride, hist, hist_stride, hist_base, st));
        m->launches++;
    }
    return LTL_OK;
}

// Decode step with the chain kernel: one launch gathers the embedding and forms layer 0's q | k | v; every layer is then the
// attention kernel and ONE cooperative launch that runs Wo (+ residual), RMSNorm + W13 + SwiGLU, W2 (+ residual) and RMSNorm +
// the next layer's QKV (after the last layer: the lm_head) with grid barriers in between: 2 + 2 L launches per step
// instead of 2 + 7 L.
int decode_step_chain(LM* m, int nseq, int slot0, const int32_t* d_tok, int32_t* d_out, int out_stride, int pick,
                      int32_t* hist, int hist_stride, int hist_base)
{
    const int D = m->D, F = m->F, V = m->V, L = m->L, H = m->H, hd = m->hd;
    const size_t e = 2;
    Act& a = m->dec;
    float* x = a.res;
    const int32_t* pos = m->d_pos + slot0;
    const size_t cl = (size_t)m->nseq_cap * H * m->T * hd * e;
    const size_t cslot = (size_t)slot0 * H * m->T * hd * e;
    struct PdlScope { bool prev; PdlScope(bool on) : prev(ltl_pdl_enabled()) { ltl_pdl_set(on); } ~PdlScope() { ltl_pdl_set(prev); } } pdl(m->use_pdl);
    LtlChainDesc d;
    memset(&d, 0, sizeof(d));
    d.M = nseq; d.eps = m->c.eps; d.tok = d_tok; d.vocab = V; d.x = x; d.bar = m->chain_bar; d.err = m->d_err; d.allow_pdl = m->chain_pdl;
    d.nphases = 1;
    d.ph[0] = LtlChainPhase{ 2, 2, 3 * D, D, m->Wb + m->off_emb, m->W + m->lo[0].ln1, m->Wb + m->lo[0].wqkv, a.qkv };
    LTL_TRY(ltl_decode_chain(d, m->s));
    m->launches++;
    const bf16* head = m->Wb + (m->c.tie ? m->off_emb : m->off_head);
    for (int l = 0; l < L; ++l) {
        const LayerOff& o = m->lo[l];
        void* kcl = (char*)m->kc + l * cl + cslot;
        void* vcl = (char*)m->vc + l * cl + cslot;
        const bool last = l + 1 == L;
        LTL_TRY(ltl_decode_attn(a.qkv, kcl, vcl, a.attn, pos, nseq, H, hd, m->T, m->scale, LTL_BF16, m->splits, m->ws,
                                m->rope_tab, m->c.rope_interleaved, m->c.use_rope, m->d_err, m->s));
        d.nphases = 4;
        d.ph[0] = LtlChainPhase{ 0, 0, D, D, a.attn, nullptr, m->Wb + o.wo, x };
        d.ph[1] = LtlChainPhase{ 1, 1, 2 * F, D, x, m->W + o.ln2, m->Wb + o.w13, a.hs };
        d.ph[2] = LtlChainPhase{ 0, 0, D, F, a.hs, nullptr, m->Wb + o.w2, x };
        if (last) d.ph[3] = LtlChainPhase{ 1, 3, V, D, x, m->W + m->off_lnf, head, a.logits };
        else d.ph[3] = LtlChainPhase{ 1, 2, 3 * D, D, x, m->W + m->lo[l + 1].ln1, m->Wb + m->lo[l + 1].wqkv, a.qkv };
        LTL_TRY(ltl_decode_chain(d, m->s));
        m->launches += 2 + (m->splits > 1 ? 1 : 0);
    }
    if (pick) {
        LTL_TRY(pick_next(m, a.logits, nseq, slot0, d_out, out_stride, hist, hist_stride, hist_base, m->s));
        m->launches++;
    }
    return LTL_OK;
}

// One token for every sequence: consumes d_next / d_pos, appends K/V, picks the next token.
// Everything it reads that changes between steps lives in device memory, so the launch
// sequence can be captured once and replayed.
int decode_step(LM* m, int nseq, int slot0, const int32_t* d_tok, int32_t* d_out, int out_stride, int pick,
                int32_t* hist = nullptr, int hist_stride = 0, int hist_base = 0)
{
    const int D = m->D, F = m->F, V = m->V, L = m->L, H = m->H, hd = m->hd, adt = m->adt;
    if (m->fuse_swiglu && m->use_chain && !m->fuse_norm && m->chain_bar && ltl_decode_chain_supported(D, F, V))
        return decode_step_chain(m, nseq, slot0, d_tok, d_out, out_stride, pick, hist, hist_stride, hist_base);
    if (m->fuse_swiglu && ltl_gemm_tc_supported(m->dec.h1, m->Wb, nseq, D, D) && F % 8 == 0 && D % 8 == 0)
        return decode_step_split(m, nseq, slot0, d_tok, d_out, out_stride, pick, hist, hist_stride, hist_base);
    const size_t e = esz(adt);
    Act& a = m->dec;
    float* x = a.res;
    const void* table = adt == LTL_F32 ? (const void*)(m->W + m->off_emb) : (const void*)(m->Wb + m->off_emb);
    const int32_t* pos = m->d_pos + slot0;
    LTL_TRY(ltl_lm_embed(d_tok, table, adt, x, nseq, D, V, m->s));
    m->launches++;
    const size_t cl = (size_t)m->nseq_cap * H * m->T * hd * e;       // bytes per layer of cache
    const size_t cslot = (size_t)slot0 * H * m->T * hd * e;
    for (int l = 0; l < L; ++l) {
        const LayerOff& o = m->lo[l];
        void* kcl = (char*)m->kc + l * cl + cslot;
        void* vcl = (char*)m->vc + l * cl + cslot;
        LTL_TRY(ltl_lm_rmsnorm(x, m->W + o.ln1, a.h1, adt, nseq, D, m->c.eps, m->s));
        LTL_TRY(wgemm(m, a.h1, nseq, D, o.wqkv, 3 * D, a.qkv, adt, nullptr, 0));
        LTL_TRY(ltl_decode_attn(a.qkv, kcl, vcl, a.attn, pos, nseq, H, hd, m->T, m->scale, adt, m->splits, m->ws,
                                m->rope_tab, m->c.rope_interleaved, m->c.use_rope, m->d_err, m->s));
        LTL_TRY(wgemm(m, a.attn, nseq, D, o.wo, D, x, LTL_F32, x, 0));
        LTL_TRY(ltl_lm_rmsnorm(x, m->W + o.ln2, a.h2, adt, nseq, D, m->c.eps, m->s));
        if (m->fuse_swiglu) {
            LTL_TRY(wgemm(m, a.h2, nseq, D, o.w13, 2 * F, a.hs, adt, nullptr, 0, 1));
        } else {
            LTL_TRY(wgemm(m, a.h2, nseq, D, o.w13, 2 * F, a.h13, adt, nullptr, 0));
            LTL_TRY(ltl_swiglu_fwd(a.h13, (char*)a.h13 + (size_t)F * e, a.hs, nseq, F, 2 * F, 2 * F, F, adt, m->s));
            m->launches++;
        }
        LTL_TRY(wgemm(m, a.hs, nseq, F, o.w2, D, x, LTL_F32, x, 0));
        m->launches += 3 + (m->splits > 1 ? 1 : 0);
    }
    LTL_TRY(ltl_lm_rmsnorm(x, m->W + m->off_lnf, a.hf, adt, nseq, D, m->c.eps, m->s));
    if (m->c.tie) LTL_TRY(wgemm(m, a.hf, nseq, D, m->off_emb, V, a.logits, LTL_F32, nullptr, 1));
    else LTL_TRY(wgemm(m, a.hf, nseq, D, m->off_head, V, a.logits, LTL_F32, nullptr, 0));
    m->launches++;
    if (pick) {
        LTL_TRY(pick_next(m, a.logits, nseq, slot0, d_out, out_stride, hist, hist_stride, hist_base, m->s));
        m->launches++;
    }
    return LTL_OK;
}

__global__ void window_kernel(const int32_t* __restrict__ hist, int hist_stride, int len, int32_t* __restrict__ win,
                              int W, int nseq)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nseq * W) return;
    const int b = i / W, t = i - b * W;
    win[i] = hist[(size_t)b * hist_stride + (len - W) + t];
}
__global__ void copy_prompt_kernel(const int32_t* __restrict__ prompts, int n_prompt, int32_t* __restrict__ hist,
                                   int hist_stride, int nseq)
{
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nseq * n_prompt) return;
    const int b = i / n_prompt, t = i - b * n_prompt;
    hist[(size_t)b * hist_stride + t] = prompts[i];
}

// Prefill the cache from the last min(len, max_seq) tokens of the history and pick a token.
int prefill_and_pick(LM* m, int nseq, int len, int hist_stride, int hist_base, int32_t* d_out, int out_stride)
{
    const int Wn = len < m->T ? len : m->T;
    window_kernel<<<(nseq * Wn + 255) / 256, 256, 0, m->s>>>(m->d_hist, hist_stride, len, m->d_win, Wn, nseq);
    LTL_TRY(ltl_check_launch("window"));
    LTL_TRY(forward(m, m->infer, m->d_win, nseq, Wn, MODE_PREFILL));
    LTL_TRY(ltl_fill_i32(m->d_pos, nseq, Wn - 1, m->s));
    LTL_TRY(pick_next(m, m->infer.logits, nseq, 0, d_out, out_stride, m->d_hist, hist_stride, hist_base, m->s));
    m->launches += 3;
    return LTL_OK;
}

// The decode loop of a large batch as two halves, half a layer out of phase.
//
// A decode step is a chain of 2 + 7 L dependent launches: the attention kernels stream the KV cache (bound by HBM), the
// launches between them are products over L2-resident weights, each a few microseconds of launch and memory latency that
// leave HBM idle.  Here the batch is cut in two halves with their own activations; half A runs on the model's stream,
// half B on a second one, and one captured graph per step holds both branches:
//     branch A:  [Wo ... of layer 0, layers 1 .. L-1, head, pick] of step k, then [embed, QKV, attention of layer 0] of step k + 1
//     branch B:  the whole of step k
// so that when the graph starts A enters the products after an attention kernel while B is about to enter one, and the
// two stay in antiphase for the L layers of the step: one half's cache streaming runs under the other's latency chain.
// For the two to share an SM the attention kernel runs as a fixed number of CTAs per SM that walk the (sequence, head)
// items, and the GEMM CTAs take a shallow ring (ltl_decode_attn_shape, ltl_gemm_tc_set_lean).  No kernel waits on
// another: the only cross-branch edges are the fork and the join of the graph.
struct HalvesShape {
    HalvesShape(int ctas, int stages) { ltl_gemm_tc_set_lean(1); ltl_decode_attn_shape(ctas, stages); }
    ~HalvesShape() { ltl_gemm_tc_set_lean(0); ltl_decode_attn_shape(0, 0); }
};

bool halves_eligible(LM* m, int nseq, int n_prompt, int n_new)
{
    return m->halves && nseq >= m->halves_min && (nseq % 2) == 0 && n_prompt + n_new <= m->T && m->splits == 1 &&
           m->adt == LTL_BF16 && m->use_tc && m->fuse_swiglu && !m->use_chain && !m->fuse_norm && m->F % 8 == 0 && m->D % 8 == 0 &&
           ltl_gemm_tc_supported(m->dec.h1, m->Wb, nseq / 2, m->D, m->D) && n_new >= 4;
}

int ensure_halves(LM* m, int nh)
{
    if (!m->s2) LTL_CUDA("second stream", cudaStreamCreateWithFlags(&m->s2, cudaStreamNonBlocking));
    if (!m->ev_fork) LTL_CUDA("fork event", cudaEventCreateWithFlags(&m->ev_fork, cudaEventDisableTiming));
    if (!m->ev_join) LTL_CUDA("join event", cudaEventCreateWithFlags(&m->ev_join, cudaEventDisableTiming));
    if (m->half_cap < nh) {
        LTL_CUDA("sync", cudaStreamSynchronize(m->s));
        LTL_CUDA("sync", cudaStreamSynchronize(m->s2));
        drop_graphs(m);
        free_act(m->dec2);
        if (m->part2) { cudaFree(m->part2); m->part2 = nullptr; }
        m->half_cap = 0;
        LTL_TRY(alloc_act(m, m->dec2, nh, 0, nh));
        DALLOC(m->part2, (size_t)8 * nh * m->D * 4, "split-K partial sums of the second half");
        m->half_cap = nh;
    }
    return LTL_OK;
}

// Decode steps 1 .. n_new - 1 after the prefill (which picked token 0).  Leaves everything ordered on m->s.
int generate_halves(LM* m, int nseq, int n_prompt, int n_new, int32_t* d_out, int hs)
{
    const int nh = nseq / 2, L = m->L;
    LTL_TRY(ensure_halves(m, nh));
    static const int attn_ctas = [] { const char* e = getenv("LUATL_HALVES_ATTN_CTAS"); return e && atoi(e) > 0 ? atoi(e) : 4; }();
    static const int attn_stages = [] { const char* e = getenv("LUATL_HALVES_ATTN_STAGES"); return e && atoi(e) > 0 ? atoi(e) : 2; }();
    HalvesShape shape(attn_ctas, attn_stages);
    static const int cut = [] { const char* e = getenv("LUATL_HALVES_CUT"); return e ? atoi(e) : 3; }();   // 3: embed, QKV and attention of layer 0 (0: halves in phase, A/B aid)
    const int all = 0x7FFFFFFF;
    auto piece = [&](int h, cudaStream_t st, int lo, int hi) -> int {
        DecCtx cx = { h ? &m->dec2 : &m->dec, h ? m->part2 : m->part, st, lo, hi };
        return decode_step_split(m, nh, h * nh, m->d_next + h * nh, d_out + (size_t)h * nh * n_new, n_new, 1,
                                 m->d_hist + (size_t)h * nh * hs, hs, n_prompt, &cx);
    };
    int steps = n_new - 1;
    GraphEntry& full = m->hgraph[0];
    GraphEntry& tail = m->hgraph[1];
    if (full.ge && (m->hgraph_nseq != nseq || full.out != d_out || full.out_stride != n_new || full.hist != m->d_hist ||
                    full.hist_stride != hs || full.hist_base != n_prompt)) {
        for (GraphEntry& ge : m->hgraph) {
            if (ge.ge) cudaGraphExecDestroy(ge.ge);
            if (ge.g) cudaGraphDestroy(ge.g);
            ge = GraphEntry();
        }
    }
    if (!full.ge) {
        // First use: one step eagerly, both halves in turn on the model's stream (a real step), then the two captures.
        const int64_t before = m->launches;
        LTL_TRY(piece(0, m->s, 0, all));
        LTL_TRY(piece(1, m->s, 0, all));
        const int64_t per_step = m->launches - before;
        --steps;
        LTL_CUDA("pre-capture sync", cudaStreamSynchronize(m->s));
        LTL_CUDA("pre-capture sync", cudaStreamSynchronize(m->s2));
        for (int which = 0; which < 2; ++which) {
            const int64_t b0 = m->launches;
            LTL_CUDA("begin capture", cudaStreamBeginCapture(m->s, cudaStreamCaptureModeThreadLocal));
            int rc = LTL_OK;
            cudaError_t ce = cudaEventRecord(m->ev_fork, m->s);
            if (ce == cudaSuccess) ce = cudaStreamWaitEvent(m->s2, m->ev_fork, 0);
            if (ce == cudaSuccess) {
                rc = piece(0, m->s, cut, all);
                if (rc == LTL_OK && which == 0) rc = piece(0, m->s, 0, cut);
                if (rc == LTL_OK) rc = piece(1, m->s2, 0, all);
                ce = cudaEventRecord(m->ev_join, m->s2);
                if (ce == cudaSuccess) ce = cudaStreamWaitEvent(m->s, m->ev_join, 0);
            }
            cudaGraph_t g = nullptr;
            const cudaError_t ee = cudaStreamEndCapture(m->s, &g);
            const int64_t captured = m->launches - b0;
            m->launches = b0;                     // the captured copy did not execute
            if (rc != LTL_OK) { if (g) cudaGraphDestroy(g); cudaGetLastError(); return rc; }
            if (ce != cudaSuccess) { if (g) cudaGraphDestroy(g); return ltl_cuda_fail("capture of the two-halves step", ce); }
            if (ee != cudaSuccess) return ltl_cuda_fail("end capture", ee);
            cudaGraphExec_t gx = nullptr;
            const cudaError_t ie = cudaGraphInstantiate(&gx, g, 0);
            if (ie != cudaSuccess) { cudaGraphDestroy(g); return ltl_cuda_fail("graph instantiate", ie); }
            GraphEntry& ge = m->hgraph[which];
            ge.g = g; ge.ge = gx; ge.launches = captured; ge.out = d_out; ge.out_stride = n_new;
            ge.hist = m->d_hist; ge.hist_stride = hs; ge.hist_base = n_prompt;
        }
        (void)per_step;
        m->hgraph_nseq = nseq;
    }
    if (steps <= 0) return LTL_OK;
    // Half A's head start, then steps - 1 full graphs and the tail.
    LTL_TRY(piece(0, m->s, 0, cut));
    for (int k = 0; k + 1 < steps; ++k) {
        LTL_CUDA("graph launch", cudaGraphLaunch(full.ge, m->s));
        m->launches += full.launches;
    }
    LTL_CUDA("graph launch", cudaGraphLaunch(tail.ge, m->s));
    m->launches += tail.launches;
    return LTL_OK;
}

int generate_dev(LM* m, const int32_t* d_prompts, int nseq, int n_prompt, int n_new, int32_t* d_out,
                 luaTL_lm_result_t* timing)
{
    if (nseq <= 0 || n_prompt <= 0 || n_new <= 0) return ltl_fail(LTL_ERR_SHAPE, "lm generate: nseq, n_prompt and n_new must be positive");
    LTL_TRY(ensure_decode(m, nseq, n_prompt, n_new));
    LTL_TRY(sync_mirror(m));
    const int hs = n_prompt + n_new;
    m->launches = 0;
    LTL_CUDA("event", cudaEventRecord(m->ev[0], m->s));
    LTL_CUDA("memset", cudaMemsetAsync(m->d_count, 0, (size_t)nseq * 4, m->s));
    LTL_CUDA("memset", cudaMemsetAsync(m->d_err, 0, 4, m->s));
    LTL_CUDA("memset", cudaMemsetAsync(m->d_done, 0, (size_t)nseq * 4, m->s));
    copy_prompt_kernel<<<(nseq * n_prompt + 255) / 256, 256, 0, m->s>>>(d_prompts, n_prompt, m->d_hist, hs, nseq);
    LTL_TRY(ltl_check_launch("copy_prompt"));
    LTL_TRY(prefill_and_pick(m, nseq, n_prompt, hs, n_prompt, d_out, n_new));
    LTL_CUDA("event", cudaEventRecord(m->ev[1], m->s));
    int len = n_prompt;                     // tokens in the history before the one just picked
    int cached = n_prompt < m->T ? n_prompt : m->T;   // tokens in the cache
    const bool halves = halves_eligible(m, nseq, n_prompt, n_new);
    if (halves) LTL_TRY(generate_halves(m, nseq, n_prompt, n_new, d_out, hs));
    for (int step = 1; step < n_new && !halves; ++step) {
        ++len;                                // the pick that produced d_next also appended it to the history
        if (cached >= m->T) {
            // cache full: rebuild it from the last max_seq tokens (ai/optim/lmtrain.lua:1511-1515)
            LTL_TRY(prefill_and_pick(m, nseq, len, hs, n_prompt, d_out, n_new));
            cached = m->T;
            continue;
        }
        GraphEntry& ge = m->graphs[nseq];
        if (ge.ge && (ge.out != d_out || ge.out_stride != n_new || ge.hist != m->d_hist || ge.hist_stride != hs ||
                      ge.hist_base != n_prompt)) {   // captured for other buffers
            cudaGraphExecDestroy(ge.ge); cudaGraphDestroy(ge.g);
            ge = GraphEntry();
        }
        if (!ge.ge) {
            // First use: run the step eagerly (it is a real step), then capture a copy for replay.
            const int64_t before = m->launches;
            LTL_TRY(decode_step(m, nseq, 0, m->d_next, d_out, n_new, 1, m->d_hist, hs, n_prompt));
            const int64_t per_step = m->launches - before;
            ++cached;
            LTL_CUDA("pre-capture sync", cudaStreamSynchronize(m->s));
            LTL_CUDA("begin capture", cudaStreamBeginCapture(m->s, cudaStreamCaptureModeThreadLocal));
            const int rc = decode_step(m, nseq, 0, m->d_next, d_out, n_new, 1, m->d_hist, hs, n_prompt);
            cudaGraph_t g = nullptr;
            const cudaError_t ce = cudaStreamEndCapture(m->s, &g);
            m->launches -= per_step;        // the captured copy did not execute
            if (rc != LTL_OK) { if (g) cudaGraphDestroy(g); cudaGetLastError(); return rc; }
            if (ce != cudaSuccess) return ltl_cuda_fail("end capture", ce);
            cudaGraphExec_t gx = nullptr;
            const cudaError_t ie = cudaGraphInstantiate(&gx, g, 0);
            if (ie != cudaSuccess) { cudaGraphDestroy(g); return ltl_cuda_fail("graph instantiate", ie); }
            ge.g = g; ge.ge = gx; ge.launches = per_step; ge.out = d_out; ge.out_stride = n_new;
            ge.hist = m->d_hist; ge.hist_stride = hs; ge.hist_base = n_prompt;
            continue;
        }
        LTL_CUDA("graph launch", cudaGraphLaunch(ge.ge, m->s));
        m->launches += ge.launches;
        ++cached;
    }
    LTL_CUDA("event", cudaEventRecord(m->ev[2], m->s));
    int err = 0;
    LTL_CUDA("error flag", cudaMemcpyAsync(&err, m->d_err, 4, cudaMemcpyDeviceToHost, m->s));
    LTL_CUDA("generate sync", cudaStreamSynchronize(m->s));
    if (err == 3) {
        cudaMemsetAsync(m->chain_bar, 0, 16, m->s);               // the barrier words may be mid-count: start clean next time
        cudaStreamSynchronize(m->s);
        return ltl_fail(LTL_ERR_CUDA, "lm generate: a grid barrier of the decode chain kernel ran out of polls");
    }
    if (err) return ltl_fail(LTL_ERR_CAPACITY, "lm generate: a position left the KV cache");
    if (m->adt == LTL_BF16 && m->use_tc) LTL_TRY(ltl_gemm_tc_check(m->s));
    cudaEventElapsedTime(&m->prefill_ms, m->ev[0], m->ev[1]);
    cudaEventElapsedTime(&m->decode_ms, m->ev[1], m->ev[2]);
    if (timing) {
        memset(timing, 0, sizeof(*timing));
        timing->step_ms = m->prefill_ms + m->decode_ms;
        timing->valid = nseq * n_new;
        timing->finite = 1;
    }
    return LTL_OK;
}

}  // namespace

extern "C" {

luaTL_lm_t* luaTL_lm_create(const luaTL_lm_config_t* cfg)
{
    if (ltl_require_init("lm_create") != LTL_OK) return nullptr;
    if (!cfg) { ltl_fail(LTL_ERR_NULL, "lm_create: null config"); return nullptr; }
    const luaTL_lm_config_t& c = *cfg;
    if (c.vocab < 1 || c.dim < 1 || c.layers < 1 || c.heads < 1 || c.ffn < 1 || c.max_seq < 1 || c.batch < 0) {
        ltl_fail(LTL_ERR_ARG, "lm_create: vocab, dim, layers, heads, ffn and max_seq must be positive integers");
        return nullptr;
    }
    if (c.dim % c.heads) { ltl_fail(LTL_ERR_ARG, "lm_create: dim (%d) must be divisible by heads (%d)", c.dim, c.heads); return nullptr; }
    const int hd = c.dim / c.heads;
    if (hd & 1) { ltl_fail(LTL_ERR_ARG, "lm_create: head_dim (dim/heads = %d) must be even for RoPE", hd); return nullptr; }
    if (hd != 16 && hd != 32 && hd != 64 && hd != 128) {
        ltl_fail(LTL_ERR_UNSUPPORTED, "lm_create: head_dim %d not in {16, 32, 64, 128}", hd); return nullptr;
    }
    if (c.dim % 8 || c.ffn % 8) { ltl_fail(LTL_ERR_UNSUPPORTED, "lm_create: dim and ffn must be multiples of 8"); return nullptr; }
    if (c.dtype != LTL_F32 && c.dtype != LTL_BF16) { ltl_fail(LTL_ERR_DTYPE, "lm_create: dtype must be f32 or bf16"); return nullptr; }
    LM* m = new LM();
    m->c = c;
    m->D = c.dim; m->H = c.heads; m->hd = hd; m->F = c.ffn; m->V = c.vocab; m->L = c.layers; m->T = c.max_seq;
    m->B = c.batch; m->adt = c.dtype; m->splits = 1;
    m->scale = 1.0f / sqrtf((float)hd);
    m->s = ltl_default_stream();
    {   // LUATL_DISABLE_TC=1 routes the bf16 GEMMs through the CUDA-core kernel (A/B comparison)
        const char* e = getenv("LUATL_DISABLE_TC");
        m->use_tc = !(e && e[0] == '1');
        m->fuse_swiglu = m->use_tc && m->adt == LTL_BF16;
        const char* p = getenv("LUATL_PDL");
        m->use_pdl = !(p && p[0] == '0');
        const char* at = getenv("LUATL_ATTN_TC");
        m->attn_tc = !(at && at[0] == '0');
        const char* rg = getenv("LUATL_DECODE_ROWS_GEMM");          // 0: tcgen05 tiles at every batch size (A/B comparison)
        m->rows_gemm = !(rg && rg[0] == '0');
        // LUATL_DECODE_FUSE_NORM=1: split-K reduce + residual inside the GEMM (last-arriving CTA per tile), RMSNorm factor
        // in the next GEMM's epilogue.  Off by default: measured slower than the reduce + RMSNorm kernel of its own
        // (256 sequences 263.6 -> 302.4 ms per pass, 32: 136.9 -> 153.7, 8: 102.9 -> 107.7) - with programmatic
        // dependent launch that kernel is already resident when its input lands, so it costs one memory round trip,
        // while the fence + ticket + reduction of the fused form add three to the GEMM's critical path.
        const char* fn = getenv("LUATL_DECODE_FUSE_NORM");
        m->fuse_norm = fn && fn[0] == '1';
        // LUATL_DECODE_CHAIN=1: the products of a layer between two attention kernels as ONE cooperative launch with grid
        // barriers (decode_chain.cu), 2 + 2 L launches per step instead of 2 + 7 L.  Off by default: measured slower at every
        // shard size (256 sequences 253.9 -> 387.6 ms per pass of 511 steps, 32 sequences 131.8 -> 183.6 ms).  A phase of that
        // kernel costs about 6 us - panel load, product, epilogue, fence + arrival + poll of the barrier are five dependent
        // L2 round trips - against about 4.3 us for a stand-alone kernel launched with programmatic dependent launch, whose
        // prologue and weight fetch run under its predecessor's tail.  LUATL_CHAIN_PDL=0: the chain kernel waits for the whole
        // of its predecessor instead of starting under its tail.
        const char* ch = getenv("LUATL_DECODE_CHAIN");
        m->use_chain = ch && ch[0] == '1';
        const char* cp = getenv("LUATL_CHAIN_PDL");
        m->chain_pdl = !(cp && cp[0] == '0');
        // LUATL_DECODE_HALVES=1: batches of at least LUATL_DECODE_HALVES_MIN (128) sequences are generated as two halves on
        // two streams, half a layer out of phase (generate_halves).
        const char* hv = getenv("LUATL_DECODE_HALVES");
        m->halves = hv && hv[0] == '1';
        const char* hm = getenv("LUATL_DECODE_HALVES_MIN");
        if (hm && atoi(hm) >= 2) m->halves_min = atoi(hm);
        const char* sq = getenv("LUATL_DECODE_SPLIT_QKV");
        m->split_qkv = sq ? atoi(sq) : 1;          // 0: never, 1: few-row kernel only, 2: tcgen05 tiles too
        const char* pm = getenv("LUATL_KV_PREFETCH_ROWS");
        m->pref_rows = pm ? atoi(pm) : -1;
        const char* oc = getenv("LUATL_OVERLAP_COMM");
        m->overlap_comm = !(oc && oc[0] == '0');
    }
    layout_params(m);
    int rc = LTL_OK;
    auto A = [&](void** p, size_t bytes, const char* what) { if (rc == LTL_OK) rc = dalloc(p, bytes, what); };
    A((void**)&m->W, (size_t)m->np * 4, "parameters");
    A((void**)&m->G, (size_t)(m->np + 4) * 4, "gradients");
    if (m->adt == LTL_BF16) A((void**)&m->Wb, (size_t)m->np * 2, "bf16 weights");
    A((void**)&m->rope_tab, (size_t)m->T * (hd / 2) * sizeof(float2), "rope table");
    for (int i = 0; i < 4 && rc == LTL_OK; ++i)
        if (cudaEventCreate(&m->ev[i]) != cudaSuccess) rc = ltl_fail(LTL_ERR_CUDA, "lm_create: cudaEventCreate failed");
    if (rc == LTL_OK) {
        std::vector<long long> nd;
        for (const TensorInfo& t : m->tens) if (!t.decay) { nd.push_back(t.off); nd.push_back(t.off + (long long)t.rows * t.cols); }
        m->n_nodecay = (int)nd.size() / 2;
        A((void**)&m->d_nodecay, nd.size() * sizeof(long long), "no-decay ranges");
        if (rc == LTL_OK && !nd.empty() &&
            cudaMemcpyAsync(m->d_nodecay, nd.data(), nd.size() * sizeof(long long), cudaMemcpyHostToDevice, m->s) != cudaSuccess)
            rc = ltl_fail(LTL_ERR_CUDA, "lm_create: upload of the no-decay ranges failed");
        if (rc == LTL_OK && cudaStreamSynchronize(m->s) != cudaSuccess) rc = ltl_fail(LTL_ERR_CUDA, "lm_create: sync failed");
        m->flat_opt = rc == LTL_OK && ltl_opt_ranges_ok(nd.data(), m->n_nodecay, m->W, m->G);
    }
    if (rc == LTL_OK) rc = ltl_rope_table(m->rope_tab, m->T, hd, c.rope_base, m->s);
    if (rc == LTL_OK && cudaMemsetAsync(m->W, 0, (size_t)m->np * 4, m->s) != cudaSuccess) rc = ltl_fail(LTL_ERR_CUDA, "lm_create: memset failed");
    if (rc == LTL_OK && cudaMemsetAsync(m->G, 0, (size_t)(m->np + 4) * 4, m->s) != cudaSuccess) rc = ltl_fail(LTL_ERR_CUDA, "lm_create: memset failed");
    if (rc == LTL_OK && cudaStreamSynchronize(m->s) != cudaSuccess) rc = ltl_fail(LTL_ERR_CUDA, "lm_create: sync failed");
    if (rc != LTL_OK) { luaTL_lm_destroy(m); return nullptr; }
    return m;
}

void luaTL_lm_destroy(luaTL_lm_t* m)
{
    if (!m) return;
    cudaDeviceSynchronize();
    drop_graphs(m);
    free_act(m->train); free_act(m->infer); free_act(m->dec); free_act(m->dec2);
    if (m->part2) cudaFree(m->part2);
    if (m->ev_fork) cudaEventDestroy(m->ev_fork);
    if (m->ev_join) cudaEventDestroy(m->ev_join);
    if (m->s2) cudaStreamDestroy(m->s2);
    void* ptrs[] = { m->W, m->G, m->M1, m->M2, m->Wb, m->rope_tab, m->dres, m->dbr, m->dhf, m->dh1, m->dqkv, m->dattn,
                     m->dh2, m->dh13, m->dhs, m->delta, m->losses, m->d_ids, m->d_tgt, m->d_pred, m->ws, m->kc, m->vc,
                     m->d_pos, m->d_count, m->d_next, m->d_hist, m->d_win, m->d_prompt, m->d_out, m->d_err, m->xlast, m->part, m->part_q,
                     m->Wm, m->d_done, m->d_nodecay, m->chain_bar, m->Wt, m->tA, m->tB, m->ssq[0], m->ssq[1], m->tile_tickets, m->b_dres, m->b_dhs, m->b_dh13, m->b_dattn, m->b_dqkv, m->b_dl };
    for (void* p : ptrs) if (p) cudaFree(p);
    for (int i = 0; i < 4; ++i) if (m->ev[i]) cudaEventDestroy(m->ev[i]);
    if (m->ev_grad) cudaEventDestroy(m->ev_grad);
    if (m->ev_comm) cudaEventDestroy(m->ev_comm);
    if (m->comm_s) cudaStreamDestroy(m->comm_s);
    cudaGetLastError();
    delete m;
}

int64_t luaTL_lm_nparams(const luaTL_lm_t* m) { return m ? m->np : 0; }
int luaTL_lm_ntensors(const luaTL_lm_t* m) { return m ? (int)m->tens.size() : 0; }
int luaTL_lm_tensor_info(const luaTL_lm_t* m, int i, char* name32, int32_t* rows, int32_t* cols, int64_t* offset, int32_t* decay)
{
    if (!m) return ltl_fail(LTL_ERR_NULL, "lm_tensor_info: null model");
    if (i < 0 || i >= (int)m->tens.size()) return ltl_fail(LTL_ERR_ARG, "lm_tensor_info: no parameter %d", i);
    const TensorInfo& t = m->tens[i];
    if (name32) memcpy(name32, t.name, 32);
    if (rows) *rows = t.rows;
    if (cols) *cols = t.cols;
    if (offset) *offset = t.off;
    if (decay) *decay = t.decay;
    return LTL_OK;
}

static int check_range(const luaTL_lm_t* m, int64_t offset, int64_t count, const void* host, const char* ctx)
{
    if (!m || !host) return ltl_fail(LTL_ERR_NULL, "%s: null pointer", ctx);
    if (offset < 0 || count < 0 || offset + count > m->np)
        return ltl_fail(LTL_ERR_SHAPE, "%s: range %lld..%lld outside the %lld parameters", ctx, (long long)offset,
                        (long long)(offset + count), (long long)m->np);
    return LTL_OK;
}
int luaTL_lm_write_params(luaTL_lm_t* m, int64_t offset, int64_t count, const float* host)
{
    LTL_TRY(check_range(m, offset, count, host, "lm_write_params"));
    LTL_CUDA("lm_write_params", cudaMemcpyAsync(m->W + offset, host, (size_t)count * 4, cudaMemcpyHostToDevice, m->s));
    LTL_CUDA("lm_write_params", cudaStreamSynchronize(m->s));
    m->mirror_dirty = 1;
    return LTL_OK;
}
int luaTL_lm_read_params(luaTL_lm_t* m, int64_t offset, int64_t count, float* host)
{
    LTL_TRY(check_range(m, offset, count, host, "lm_read_params"));
    LTL_CUDA("lm_read_params", cudaMemcpyAsync(host, m->W + offset, (size_t)count * 4, cudaMemcpyDeviceToHost, m->s));
    LTL_CUDA("lm_read_params", cudaStreamSynchronize(m->s));
    return LTL_OK;
}
int luaTL_lm_read_grads(luaTL_lm_t* m, int64_t offset, int64_t count, float* host)
{
    LTL_TRY(check_range(m, offset, count, host, "lm_read_grads"));
    LTL_CUDA("lm_read_grads", cudaMemcpyAsync(host, m->G + offset, (size_t)count * 4, cudaMemcpyDeviceToHost, m->s));
    LTL_CUDA("lm_read_grads", cudaStreamSynchronize(m->s));
    return LTL_OK;
}
float* luaTL_lm_params_device(luaTL_lm_t* m) { if (m) m->mirror_dirty = 1; return m ? m->W : nullptr; }
float* luaTL_lm_grads_device(luaTL_lm_t* m) { return m ? m->G : nullptr; }

int luaTL_lm_train_step_dev(luaTL_lm_t* m, const int32_t* d_ids, const int32_t* d_targets,
                            const luaTL_lm_train_args_t* a, luaTL_lm_result_t* out)
{
    if (!m || !d_ids || !d_targets || !a) return ltl_fail(LTL_ERR_NULL, "lm_train_step_dev: null pointer");
    if (m->B < 1) return ltl_fail(LTL_ERR_ARG, "lm_train_step: model created with batch = 0");
    if (a->valid_global <= 0) return ltl_fail(LTL_ERR_ARG, "lm_train_step_dev: valid_global must be given for device-resident targets");
    return train_step_dev(m, d_ids, d_targets, a, out, a->valid_global);
}

// Host-side contract of the id / target blocks, shared by the training and the evaluation step: inputs inside the
// vocabulary, targets inside it or negative (ignored).
static int check_tokens(const luaTL_lm_t* m, const int32_t* ids, const int32_t* targets, int rows, const char* ctx)
{
    for (int i = 0; i < rows; ++i)
        if (ids[i] < 0 || ids[i] >= m->V || targets[i] >= m->V)
            return ltl_fail(LTL_ERR_ARG, "%s: token out of range at row %d (input %d, target %d, vocab %d)",
                            ctx, i, ids[i], targets[i], m->V);
    return LTL_OK;
}

int luaTL_lm_train_step(luaTL_lm_t* m, const int32_t* ids, const int32_t* targets,
                        const luaTL_lm_train_args_t* a, luaTL_lm_result_t* out)
{
    if (!m || !ids || !targets || !a) return ltl_fail(LTL_ERR_NULL, "lm_train_step: null pointer");
    if (m->B < 1) return ltl_fail(LTL_ERR_ARG, "lm_train_step: model created with batch = 0");
    LTL_TRY(ensure_train(m));
    const int rows = m->B * m->T;
    LTL_TRY(check_tokens(m, ids, targets, rows, "lm_train_step"));
    LTL_CUDA("ids upload", cudaMemcpyAsync(m->d_ids, ids, (size_t)rows * 4, cudaMemcpyHostToDevice, m->s));
    LTL_CUDA("targets upload", cudaMemcpyAsync(m->d_tgt, targets, (size_t)rows * 4, cudaMemcpyHostToDevice, m->s));
    return train_step_dev(m, m->d_ids, m->d_tgt, a, out, count_valid(targets, rows, m->V));
}

int luaTL_lm_eval_step(luaTL_lm_t* m, const int32_t* ids, const int32_t* targets, luaTL_lm_result_t* out)
{
    if (!m || !ids || !targets) return ltl_fail(LTL_ERR_NULL, "lm_eval_step: null pointer");
    if (m->B < 1) return ltl_fail(LTL_ERR_ARG, "lm_eval_step: model created with batch = 0");
    LTL_TRY(ensure_train(m));
    const int rows = m->B * m->T;
    LTL_TRY(check_tokens(m, ids, targets, rows, "lm_eval_step"));
    LTL_CUDA("ids upload", cudaMemcpyAsync(m->d_ids, ids, (size_t)rows * 4, cudaMemcpyHostToDevice, m->s));
    LTL_CUDA("targets upload", cudaMemcpyAsync(m->d_tgt, targets, (size_t)rows * 4, cudaMemcpyHostToDevice, m->s));
    const int valid = count_valid(targets, rows, m->V);
    m->launches = 0;
    LTL_CUDA("event", cudaEventRecord(m->ev[0], m->s));
    LTL_TRY(loss_and_grad(m, m->d_ids, m->d_tgt, valid, 0));
    LTL_CUDA("event", cudaEventRecord(m->ev[1], m->s));
    float tail[2] = { 0, 0 };
    LTL_CUDA("loss download", cudaMemcpyAsync(tail, m->G + m->np, 8, cudaMemcpyDeviceToHost, m->s));
    LTL_CUDA("eval sync", cudaStreamSynchronize(m->s));
    if (out) {
        memset(out, 0, sizeof(*out));
        out->loss = tail[0]; out->correct = (int)(tail[1] + 0.5f); out->valid = valid; out->finite = isfinite(tail[0]) ? 1 : 0;
        cudaEventElapsedTime(&out->step_ms, m->ev[0], m->ev[1]);
    }
    return LTL_OK;
}

int luaTL_lm_forward(luaTL_lm_t* m, const int32_t* ids, int nseq, int ntok, float* logits_host, int last_only)
{
    if (!m || !ids || !logits_host) return ltl_fail(LTL_ERR_NULL, "lm_forward: null pointer");
    if (m->B < 1) return ltl_fail(LTL_ERR_ARG, "lm_forward: model created with batch = 0");
    if (nseq < 1 || nseq > m->B || ntok < 1 || ntok > m->T)
        return ltl_fail(LTL_ERR_SHAPE, "lm_forward: %d sequences x %d tokens outside batch %d x max_seq %d", nseq, ntok, m->B, m->T);
    LTL_TRY(ensure_train(m));
    const int rows = nseq * ntok;
    for (int i = 0; i < rows; ++i)
        if (ids[i] < 0 || ids[i] >= m->V) return ltl_fail(LTL_ERR_ARG, "lm_forward: token %d out of range at row %d", ids[i], i);
    LTL_CUDA("ids upload", cudaMemcpyAsync(m->d_ids, ids, (size_t)rows * 4, cudaMemcpyHostToDevice, m->s));
    m->launches = 0;
    LTL_TRY(forward(m, m->train, m->d_ids, nseq, ntok, MODE_TRAIN));
    if (last_only)
        LTL_CUDA("logits download", cudaMemcpyAsync(logits_host, m->train.logits + (size_t)(ntok - 1) * m->V, (size_t)m->V * 4,
                                                    cudaMemcpyDeviceToHost, m->s));
    else
        LTL_CUDA("logits download", cudaMemcpyAsync(logits_host, m->train.logits, (size_t)rows * m->V * 4,
                                                    cudaMemcpyDeviceToHost, m->s));
    LTL_CUDA("forward sync", cudaStreamSynchronize(m->s));
    return LTL_OK;
}

int luaTL_lm_state_reset(luaTL_lm_t* m)
{
    if (!m) return ltl_fail(LTL_ERR_NULL, "lm_state_reset: null model");
    LTL_TRY(ensure_decode(m, 1, 0, 0));
    LTL_CUDA("memset", cudaMemsetAsync(m->d_pos, 0, (size_t)m->nseq_cap * 4, m->s));
    LTL_CUDA("memset", cudaMemsetAsync(m->d_count, 0, (size_t)m->nseq_cap * 4, m->s));
    LTL_CUDA("memset", cudaMemsetAsync(m->d_err, 0, 4, m->s));
    LTL_CUDA("state_reset sync", cudaStreamSynchronize(m->s));
    return LTL_OK;
}

int luaTL_lm_slot_reset(luaTL_lm_t* m, int slot)
{
    if (!m) return ltl_fail(LTL_ERR_NULL, "lm_slot_reset: null model");
    LTL_TRY(ensure_decode(m, 1, 0, 0));
    if (slot < 0 || slot >= m->nseq_cap) return ltl_fail(LTL_ERR_ARG, "lm_slot_reset: slot %d outside 0..%d", slot, m->nseq_cap - 1);
    LTL_CUDA("memset", cudaMemsetAsync(m->d_pos + slot, 0, 4, m->s));
    LTL_CUDA("memset", cudaMemsetAsync(m->d_count + slot, 0, 4, m->s));
    LTL_CUDA("slot_reset sync", cudaStreamSynchronize(m->s));
    return LTL_OK;
}

int luaTL_lm_state_len(luaTL_lm_t* m, int slot)
{
    if (!m || !m->d_pos || slot < 0 || slot >= m->nseq_cap) return -1;
    int v = -1;
    if (cudaMemcpyAsync(&v, m->d_pos + slot, 4, cudaMemcpyDeviceToHost, m->s) != cudaSuccess) return -1;
    if (cudaStreamSynchronize(m->s) != cudaSuccess) return -1;
    return v;
}

int luaTL_lm_step(luaTL_lm_t* m, int slot, int32_t id, float* logits_host)
{
    if (!m || !logits_host) return ltl_fail(LTL_ERR_NULL, "lm_step: null pointer");
    LTL_TRY(ensure_decode(m, 1, 0, 0));
    if (slot < 0 || slot >= m->nseq_cap) return ltl_fail(LTL_ERR_ARG, "lm_step: slot %d outside 0..%d", slot, m->nseq_cap - 1);
    if (id < 0 || id >= m->V) return ltl_fail(LTL_ERR_ARG, "lm_step: token id out of range: %d", id);
    const int len = luaTL_lm_state_len(m, slot);
    if (len < 0) return ltl_fail(LTL_ERR_CUDA, "lm_step: could not read the state length");
    if (len >= m->T) return ltl_fail(LTL_ERR_CAPACITY, "lm_step: context is full (%d tokens)", m->T);
    LTL_TRY(sync_mirror(m));
    LTL_CUDA("token upload", cudaMemcpyAsync(m->d_next + slot, &id, 4, cudaMemcpyHostToDevice, m->s));
    const int sp = m->splits;
    LTL_TRY(decode_step(m, 1, slot, m->d_next + slot, nullptr, 0, 1));
    m->splits = sp;
    LTL_CUDA("logits download", cudaMemcpyAsync(logits_host, m->dec.logits, (size_t)m->V * 4, cudaMemcpyDeviceToHost, m->s));
    LTL_CUDA("lm_step sync", cudaStreamSynchronize(m->s));
    return LTL_OK;
}

int luaTL_lm_generate_dev(luaTL_lm_t* m, const int32_t* d_prompts, int nseq, int n_prompt, int n_new,
                          int32_t* d_out, luaTL_lm_result_t* timing)
{
    if (!m || !d_prompts || !d_out) return ltl_fail(LTL_ERR_NULL, "lm_generate_dev: null pointer");
    return generate_dev(m, d_prompts, nseq, n_prompt, n_new, d_out, timing);
}

int luaTL_lm_generate(luaTL_lm_t* m, const int32_t* prompts, int nseq, int n_prompt, int n_new,
                      int32_t* out, luaTL_lm_result_t* timing)
{
    if (!m || !prompts || !out) return ltl_fail(LTL_ERR_NULL, "lm_generate: null pointer");
    if (nseq <= 0 || n_prompt <= 0 || n_new <= 0) return ltl_fail(LTL_ERR_SHAPE, "lm_generate: nseq, n_prompt and n_new must be positive");
    for (int i = 0; i < nseq * n_prompt; ++i)
        if (prompts[i] < 0 || prompts[i] >= m->V) return ltl_fail(LTL_ERR_ARG, "lm_generate: token %d out of range at %d", prompts[i], i);
    if (m->prompt_cap < nseq * n_prompt) {
        cudaStreamSynchronize(m->s);
        cudaFree(m->d_prompt);
        DALLOC(m->d_prompt, (size_t)nseq * n_prompt * 4, "prompts");
        m->prompt_cap = nseq * n_prompt;
    }
    if (m->out_cap < nseq * n_new) {
        cudaStreamSynchronize(m->s);
        cudaFree(m->d_out);
        DALLOC(m->d_out, (size_t)nseq * n_new * 4, "generated ids");
        m->out_cap = nseq * n_new;
    }
    LTL_CUDA("prompt upload", cudaMemcpyAsync(m->d_prompt, prompts, (size_t)nseq * n_prompt * 4, cudaMemcpyHostToDevice, m->s));
    LTL_TRY(generate_dev(m, m->d_prompt, nseq, n_prompt, n_new, m->d_out, timing));
    LTL_CUDA("ids download", cudaMemcpyAsync(out, m->d_out, (size_t)nseq * n_new * 4, cudaMemcpyDeviceToHost, m->s));
    LTL_CUDA("generate sync", cudaStreamSynchronize(m->s));
    return LTL_OK;
}

int luaTL_lm_set_sampling(luaTL_lm_t* m, float temperature, int top_k, float top_p, uint64_t seed, int stop_id)
{
    if (!m) return ltl_fail(LTL_ERR_NULL, "lm_set_sampling: null model");
    if (temperature > 0.0f && top_k < 0) return ltl_fail(LTL_ERR_ARG, "lm_set_sampling: top_k %d is negative", top_k);
    if (stop_id >= m->V) return ltl_fail(LTL_ERR_ARG, "lm_set_sampling: stop token %d outside the vocabulary", stop_id);
    LM::Sampling n;
    n.temperature = temperature > 0.0f ? temperature : 0.0f; n.top_k = top_k; n.top_p = top_p; n.seed = seed; n.stop_id = stop_id;
    const LM::Sampling& o = m->samp;
    if (n.temperature != o.temperature || n.top_k != o.top_k || n.top_p != o.top_p || n.seed != o.seed || n.stop_id != o.stop_id) {
        LTL_CUDA("sync", cudaStreamSynchronize(m->s));
        drop_graphs(m);                                  // captured decode steps carry the old values as kernel arguments
        m->samp = n;
    }
    return LTL_OK;
}

int luaTL_lm_set_graph(luaTL_lm_t* m, int on)
{
    if (!m) return ltl_fail(LTL_ERR_NULL, "lm_set_graph: null model");
    if (!on && m->graph_steps) { LTL_CUDA("sync", cudaStreamSynchronize(m->s)); drop_step_graph(m); }
    m->graph_steps = on ? 1 : 0;
    return LTL_OK;
}
int luaTL_lm_graph_ready(const luaTL_lm_t* m) { return m && m->step_graph.ge ? 1 : 0; }

int luaTL_lm_set_tf32(luaTL_lm_t* m, int on)
{
    if (!m) return ltl_fail(LTL_ERR_NULL, "lm_set_tf32: null model");
    if (m->adt != LTL_F32) return ltl_fail(LTL_ERR_UNSUPPORTED, "lm_set_tf32: only fp32 models have an exact and a TF32 path (bf16 models always use the tensor cores)");
    if ((on != 0) == (m->tf32 != 0)) return LTL_OK;
    LTL_CUDA("sync", cudaStreamSynchronize(m->s));
    drop_graphs(m);                                       // captured steps hold the other path's kernels
    m->tf32 = on ? 1 : 0;
    m->mirror_dirty = 1;
    return LTL_OK;
}

int luaTL_lm_time_decode_attn(luaTL_lm_t* m, int nseq, int cache_len, int iters, float* ms_per_launch)
{
    if (!m || !ms_per_launch) return ltl_fail(LTL_ERR_NULL, "lm_time_decode_attn: null pointer");
    if (nseq < 1 || iters < 1 || cache_len < 0 || cache_len >= m->T)
        return ltl_fail(LTL_ERR_ARG, "lm_time_decode_attn: need 0 <= cache_len < max_seq, nseq >= 1, iters >= 1");
    LTL_TRY(ensure_decode(m, nseq, 0, 0));
    const size_t e = esz(m->adt);
    const size_t cl = (size_t)m->nseq_cap * m->H * m->T * m->hd * e;
    LTL_TRY(ltl_fill_i32(m->d_pos, nseq, cache_len, m->s));
    auto round = [&]() -> int {
        for (int l = 0; l < m->L; ++l)
            LTL_TRY(ltl_decode_attn(m->dec.qkv, (char*)m->kc + l * cl, (char*)m->vc + l * cl, m->dec.attn, m->d_pos, nseq,
                                    m->H, m->hd, m->T, m->scale, m->adt, m->splits, m->ws, m->rope_tab,
                                    m->c.rope_interleaved, m->c.use_rope, m->d_err, m->s));
        return LTL_OK;
    };
    for (int w = 0; w < 3; ++w) LTL_TRY(round());
    LTL_CUDA("event", cudaEventRecord(m->ev[0], m->s));
    for (int i = 0; i < iters; ++i) LTL_TRY(round());
    LTL_CUDA("event", cudaEventRecord(m->ev[1], m->s));
    LTL_CUDA("sync", cudaStreamSynchronize(m->s));
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, m->ev[0], m->ev[1]);
    *ms_per_launch = ms / (float)(iters * m->L);
    LTL_CUDA("memset", cudaMemsetAsync(m->d_pos, 0, (size_t)m->nseq_cap * 4, m->s));
    LTL_CUDA("memset", cudaMemsetAsync(m->d_err, 0, 4, m->s));
    LTL_CUDA("sync", cudaStreamSynchronize(m->s));
    return LTL_OK;
}

// Measurement aid: what each launch of the decode step costs inside a dependent chain.  Every launch kind of the step
// (the product path's own launch code, windowed) is captured 60 times back to back into a CUDA graph - programmatic
// dependent launch as in the step - and replayed; us[i] = microseconds per launch:
//   0 embed + RMSNorm   1 QKV   2 Wo (split-K)   3 reduce + RMSNorm   4 W13 + SwiGLU   5 W2 (split-K)
//   6 reduce + RMSNorm (+ prefetch rider)   7 lm_head   8 pick   9 one layer's chain Wo .. next QKV (six launches, total)
// Attention is left out (luaTL_lm_time_decode_attn times it over a cache larger than L2).
int luaTL_lm_time_decode_launches(luaTL_lm_t* m, int nseq, int cache_len, int reps, float* us, int n)
{
    if (!m || !us) return ltl_fail(LTL_ERR_NULL, "lm_time_decode_launches: null pointer");
    if (nseq < 1 || reps < 1 || n < 10 || cache_len < 0 || cache_len >= m->T)
        return ltl_fail(LTL_ERR_ARG, "lm_time_decode_launches: need nseq >= 1, reps >= 1, 0 <= cache_len < max_seq and room for 10 values");
    LTL_TRY(ensure_decode(m, nseq, 0, 0));
    if (!(m->adt == LTL_BF16 && m->use_tc && m->fuse_swiglu && m->F % 8 == 0 && m->D % 8 == 0 &&
          ltl_gemm_tc_supported(m->dec.h1, m->Wb, nseq, m->D, m->D)))
        return ltl_fail(LTL_ERR_UNSUPPORTED, "lm_time_decode_launches: the model does not decode on the bf16 tensor-core path");
    LTL_TRY(sync_mirror(m));
    LTL_TRY(ltl_fill_i32(m->d_pos, nseq, cache_len, m->s));
    const int L = m->L, CH = 60;
    const int lo[10] = { 0, 1, 3, 4, 5, 6, 7, 1 + 7 * L, 2 + 7 * L, 3 };
    const int hi[10] = { 1, 2, 4, 5, 6, 7, 8, 2 + 7 * L, 3 + 7 * L, L >= 2 ? 9 : 8 };
    const int64_t keep = m->launches;
    int rc = LTL_OK;
    for (int i = 0; i < 10 && rc == LTL_OK; ++i) {
        const DecCtx cx = { &m->dec, m->part, m->s, lo[i], hi[i] };
        auto issue = [&]() { return decode_step_split(m, nseq, 0, m->d_next, nullptr, 0, 1, nullptr, 0, 0, &cx); };
        const int per = i == 9 ? CH / 6 : CH;            // graph launches of (hi - lo) kernels each
        if ((rc = issue()) != LTL_OK) break;             // first use of a shape sets kernel attributes: outside the capture
        LTL_CUDA("pre-capture sync", cudaStreamSynchronize(m->s));
        LTL_CUDA("begin capture", cudaStreamBeginCapture(m->s, cudaStreamCaptureModeThreadLocal));
        for (int k = 0; k < per && rc == LTL_OK; ++k) rc = issue();
        cudaGraph_t g = nullptr;
        const cudaError_t ce = cudaStreamEndCapture(m->s, &g);
        if (rc != LTL_OK) { if (g) cudaGraphDestroy(g); cudaGetLastError(); break; }
        if (ce != cudaSuccess) { rc = ltl_cuda_fail("end capture", ce); break; }
        cudaGraphExec_t gx = nullptr;
        const cudaError_t ie = cudaGraphInstantiate(&gx, g, 0);
        if (ie != cudaSuccess) { cudaGraphDestroy(g); rc = ltl_cuda_fail("graph instantiate", ie); break; }
        cudaError_t e = cudaSuccess;
        for (int w = 0; w < 3 && e == cudaSuccess; ++w) e = cudaGraphLaunch(gx, m->s);
        if (e == cudaSuccess) e = cudaEventRecord(m->ev[0], m->s);
        for (int r = 0; r < reps && e == cudaSuccess; ++r) e = cudaGraphLaunch(gx, m->s);
        if (e == cudaSuccess) e = cudaEventRecord(m->ev[1], m->s);
        if (e == cudaSuccess) e = cudaStreamSynchronize(m->s);
        cudaGraphExecDestroy(gx); cudaGraphDestroy(g);
        if (e != cudaSuccess) { rc = ltl_cuda_fail("lm_time_decode_launches", e); break; }
        float ms = 0.0f;
        cudaEventElapsedTime(&ms, m->ev[0], m->ev[1]);
        us[i] = ms * 1000.0f / (float)(reps * per);      // slot 9: per pass over the layer's chain
    }
    m->launches = keep;
    cudaMemsetAsync(m->d_pos, 0, (size_t)m->nseq_cap * 4, m->s);
    cudaMemsetAsync(m->d_count, 0, (size_t)m->nseq_cap * 4, m->s);
    cudaMemsetAsync(m->d_err, 0, 4, m->s);
    cudaStreamSynchronize(m->s);
    if (rc == LTL_OK) rc = ltl_gemm_tc_check(m->s);
    return rc;
}

int luaTL_lm_last_timing(luaTL_lm_t* m, float* prefill_ms, float* decode_ms, int64_t* launches)
{
    if (!m) return ltl_fail(LTL_ERR_NULL, "lm_last_timing: null model");
    if (prefill_ms) *prefill_ms = m->prefill_ms;
    if (decode_ms) *decode_ms = m->decode_ms;
    if (launches) *launches = m->launches;
    return LTL_OK;
}

}  // extern "C"
