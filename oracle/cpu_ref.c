/*
 * CPU oracle for the lanternl language-model token loop.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C with double
 * arithmetic (Lua numbers are doubles), the reference's CPU implementation of
 * the path.  It is called only by the tests, by the smoke check and by the
 * CPU-baseline leg of the benchmark.  The product library never links or
 * calls it.
 *
 * What each function follows (paths inside the reference project):
 *   ora_forward        ai/nn/transformer.lua:228-257 (forward), :196-226
 *                      (_attention), ai/core/tensor2.lua:609-634 (rmsnorm),
 *                      :332-383 (softmax_rows, causal), :410-446 (rope),
 *                      :572-590 (embed), :272-291 (silu)
 *   ora_loss_grad      ai/core/tensor2.lua:809-882 (cross_entropy + backward),
 *                      :641-666 (rmsnorm bwd), :388-408 (softmax bwd),
 *                      :451-473 (rope bwd), :592-607 (embed bwd),
 *                      :293-303 (silu bwd); loss/grad normalisation follows
 *                      ai/gpu/gpu_transformer.lua:546-553 (1/valid over the
 *                      whole batch), targets < 0 ignored as in
 *                      cuda/luaTL_train.cu:849-854
 *   ora_sgd            ai/optim/optim2.lua:72-102 (no momentum branch)
 *   ora_grad_norm      ai/optim/optim2.lua:27-38
 *   ora_step           ai/nn/transformer.lua:297-434 (KV-cache decode step)
 *   ora_greedy         ai/optim/lmtrain.lua:1364-1371 (pick_token, greedy:
 *                      first strict maximum) and :1499-1519 (cache branch of
 *                      generate, including the re-prefill when the state is
 *                      full)
 *
 * Two deliberate parameters bridge the reference's CPU and GPU models, which
 * are not the same function:
 *   - weights are taken in the GPU model's layout (fused wqkv [D,3D] and
 *     w13 [D,2F]; ai/gpu/gpu_transformer.lua:224-239).  A fused product is
 *     the column concatenation of the separate products of
 *     transformer.lua:197-199, so nothing changes numerically.
 *   - rope_interleaved = 1 rotates pairs (2k, 2k+1) as tensor2.lua:432-438
 *     does; 0 rotates pairs (k, k + hd/2) as cuda/luaTL_train.cu:742-750
 *     does.
 *
 * Parity pinning: the reference ships no golden vectors for the whole path.
 * The op-level known answers it does ship (tests/core_test.lua:31-57,86-92;
 * tests/test.lua sections 8-10,13) are checked in tests/test_oracle.py, and
 * whole-path outputs are pinned against the reference's own compiled CUDA
 * kernels (oracle/ref_driver.py) on the GPU box and against the fixtures
 * under tests/golden/ that were generated from them.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

typedef struct {
    int32_t vocab, dim, layers, heads, ffn, max_seq, tie, rope_interleaved;
    double  eps, rope_base;
    int32_t act_bf16, pad_;
} ora_cfg;

/* act_bf16 = 1 models the bf16 configuration: every activation that the reference's kernels
 * would STORE in a bf16 tensor (its TAcc<bf16> store, cuda/luaTL_core.cu bf16 traits) is rounded
 * to bfloat16 (nearest even) where it is stored - the normed GEMM inputs, q|k|v before and after
 * RoPE (the K/V cache holds these), the attention output, the gate|up projection and the SwiGLU
 * output.  The residual stream, the accumulations and the logits stay in full precision. */
static double rbf(double x)
{
    float f = (float)x;
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7F800000u) == 0x7F800000u) return x;
    u = (u + 0x7FFFu + ((u >> 16) & 1u)) & 0xFFFF0000u;
    memcpy(&f, &u, 4);
    return (double)f;
}
static void round_bf16(const ora_cfg *c, double *x, int64_t n)
{
    if (!c->act_bf16) return;
    for (int64_t i = 0; i < n; ++i) x[i] = rbf(x[i]);
}

typedef struct {
    const double *emb, *lnf, *head;
    const double *ln1, *wqkv, *wo, *ln2, *w13, *w2; /* of the current layer */
} ora_w;

static int64_t layer_elems(const ora_cfg *c)
{
    const int64_t D = c->dim, F = c->ffn;
    return D + D * 3 * D + D * D + D + D * 2 * F + F * D;
}

int64_t ora_nparams(const ora_cfg *c)
{
    const int64_t D = c->dim, V = c->vocab;
    return V * D + c->layers * layer_elems(c) + D + (c->tie ? 0 : D * V);
}

/* Offsets of tensor `which` (0 ln1, 1 wqkv, 2 wo, 3 ln2, 4 w13, 5 w2) of layer l. */
static int64_t layer_off(const ora_cfg *c, int l, int which)
{
    const int64_t D = c->dim, F = c->ffn, V = c->vocab;
    int64_t o = V * D + (int64_t)l * layer_elems(c);
    const int64_t sz[6] = { D, D * 3 * D, D * D, D, D * 2 * F, F * D };
    for (int i = 0; i < which; ++i) o += sz[i];
    return o;
}
static int64_t lnf_off(const ora_cfg *c)
{
    return (int64_t)c->vocab * c->dim + (int64_t)c->layers * layer_elems(c);
}

/* 1 where weight decay applies (matrices), 0 on the norm gains
 * (ai/gpu/gpu_transformer.lua:224-239). */
void ora_decay_mask(const ora_cfg *c, uint8_t *mask)
{
    const int64_t n = ora_nparams(c);
    memset(mask, 1, (size_t)n);
    for (int l = 0; l < c->layers; ++l) {
        memset(mask + layer_off(c, l, 0), 0, (size_t)c->dim);
        memset(mask + layer_off(c, l, 3), 0, (size_t)c->dim);
    }
    memset(mask + lnf_off(c), 0, (size_t)c->dim);
}

/* ---- small dense helpers (row-major, double) ---- */

/* C[M,N] (+)= A[M,K] B[K,N]; loop order i-k-j with the skip-zero shortcut of
 * ai/core/matrix.lua:514-539. */
static void mm(const double *A, const double *B, double *C, int M, int K, int N, int acc)
{
    for (int i = 0; i < M; ++i) {
        double *c = C + (int64_t)i * N;
        if (!acc) for (int j = 0; j < N; ++j) c[j] = 0.0;
        for (int k = 0; k < K; ++k) {
            const double a = A[(int64_t)i * K + k];
            if (a == 0.0) continue;
            const double *b = B + (int64_t)k * N;
            for (int j = 0; j < N; ++j) c[j] += a * b[j];
        }
    }
}
/* C[M,N] (+)= A[M,K] B[N,K]^T   (ai/core/matrix.lua:597-627 matmul_nt) */
static void mm_nt(const double *A, const double *B, double *C, int M, int K, int N, int acc)
{
    for (int i = 0; i < M; ++i)
        for (int j = 0; j < N; ++j) {
            double s = 0.0;
            const double *a = A + (int64_t)i * K, *b = B + (int64_t)j * K;
            for (int k = 0; k < K; ++k) s += a[k] * b[k];
            if (acc) C[(int64_t)i * N + j] += s; else C[(int64_t)i * N + j] = s;
        }
}
/* C[K,N] += A[M,K]^T B[M,N]   (ai/core/matrix.lua:629-660 matmul_tn) */
static void mm_tn_acc(const double *A, const double *B, double *C, int M, int K, int N)
{
    for (int i = 0; i < M; ++i)
        for (int k = 0; k < K; ++k) {
            const double a = A[(int64_t)i * K + k];
            if (a == 0.0) continue;
            const double *b = B + (int64_t)i * N;
            double *c = C + (int64_t)k * N;
            for (int j = 0; j < N; ++j) c[j] += a * b[j];
        }
}

static void rmsnorm_rows(const double *x, const double *w, double *y, double *inv,
                         int rows, int cols, double eps)
{
    for (int i = 0; i < rows; ++i) {
        const double *xr = x + (int64_t)i * cols;
        double ss = 0.0;
        for (int j = 0; j < cols; ++j) ss += xr[j] * xr[j];
        const double r = 1.0 / sqrt(ss / cols + eps);
        if (inv) inv[i] = r;
        for (int j = 0; j < cols; ++j) y[(int64_t)i * cols + j] = xr[j] * r * w[j];
    }
}

static void rmsnorm_bwd_rows(const double *x, const double *w, const double *inv,
                             const double *g, double *xg, double *wg, int rows, int cols)
{
    for (int i = 0; i < rows; ++i) {
        const double *xr = x + (int64_t)i * cols, *gr = g + (int64_t)i * cols;
        const double r = inv[i];
        double dot = 0.0;
        for (int j = 0; j < cols; ++j) dot += gr[j] * w[j] * xr[j];
        const double coef = dot * r * r * r / cols;
        for (int j = 0; j < cols; ++j) {
            xg[(int64_t)i * cols + j] += gr[j] * w[j] * r - xr[j] * coef;
            wg[j] += gr[j] * xr[j] * r;
        }
    }
}

static double sigmoid_stable(double v)
{
    if (v >= 0) return 1.0 / (1.0 + exp(-v));
    const double z = exp(v);
    return z / (1.0 + z);
}

/* In-place rotary embedding of one [T, hd] head slice living inside a wider
 * row (row stride `ld`).  inverse = transpose rotation (the backward). */
static void rope_head(double *x, int T, int hd, int ld, int pos0, double base,
                      int interleaved, int inverse)
{
    const int np = hd / 2;
    for (int t = 0; t < T; ++t) {
        double *xr = x + (int64_t)t * ld;
        for (int k = 0; k < np; ++k) {
            const double invf = 1.0 / pow(base, (2.0 * k) / hd);
            const double ang = (double)(pos0 + t) * invf;
            const double c = cos(ang);
            const double s = inverse ? -sin(ang) : sin(ang);
            const int i0 = interleaved ? 2 * k : k;
            const int i1 = interleaved ? 2 * k + 1 : k + np;
            const double x0 = xr[i0], x1 = xr[i1];
            xr[i0] = x0 * c - x1 * s;
            xr[i1] = x0 * s + x1 * c;
        }
    }
}

static void set_layer(const ora_cfg *c, const double *P, int l, ora_w *w)
{
    w->ln1 = P + layer_off(c, l, 0);
    w->wqkv = P + layer_off(c, l, 1);
    w->wo = P + layer_off(c, l, 2);
    w->ln2 = P + layer_off(c, l, 3);
    w->w13 = P + layer_off(c, l, 4);
    w->w2 = P + layer_off(c, l, 5);
}

/* Saved activations of one sequence (needed by the backward). */
typedef struct {
    double *res;   /* [L+1][T*D]  residual stream entering layer l (res[L] = output) */
    double *mid;   /* [L][T*D] */
    double *h1, *h2;            /* [L][T*D] */
    double *inv1, *inv2;        /* [L][T] */
    double *qkv;   /* [L][T*3D] after rope */
    double *pr;    /* [L][H*T*T] */
    double *ctx;   /* [L][T*D] */
    double *h13;   /* [L][T*2F] */
    double *hs;    /* [L][T*F] */
    double *hf, *invf;          /* [T*D], [T] */
} ora_act;

static ora_act act_alloc(const ora_cfg *c, int T)
{
    const int64_t L = c->layers, D = c->dim, F = c->ffn, H = c->heads;
    ora_act a;
    a.res = (double *)calloc((size_t)((L + 1) * T * D), 8);
    a.mid = (double *)calloc((size_t)(L * T * D), 8);
    a.h1 = (double *)calloc((size_t)(L * T * D), 8);
    a.h2 = (double *)calloc((size_t)(L * T * D), 8);
    a.inv1 = (double *)calloc((size_t)(L * T), 8);
    a.inv2 = (double *)calloc((size_t)(L * T), 8);
    a.qkv = (double *)calloc((size_t)(L * T * 3 * D), 8);
    a.pr = (double *)calloc((size_t)(L * H * T * T), 8);
    a.ctx = (double *)calloc((size_t)(L * T * D), 8);
    a.h13 = (double *)calloc((size_t)(L * T * 2 * F), 8);
    a.hs = (double *)calloc((size_t)(L * T * F), 8);
    a.hf = (double *)calloc((size_t)(T * D), 8);
    a.invf = (double *)calloc((size_t)T, 8);
    return a;
}
static void act_free(ora_act *a)
{
    free(a->res); free(a->mid); free(a->h1); free(a->h2); free(a->inv1); free(a->inv2);
    free(a->qkv); free(a->pr); free(a->ctx); free(a->h13); free(a->hs); free(a->hf);
    free(a->invf);
}

/* Forward of ONE sequence of T tokens (ids 0-indexed). logits [T,V]. */
static void forward_seq(const ora_cfg *c, const double *P, const int32_t *ids, int T,
                        ora_act *a, double *logits)
{
    const int D = c->dim, H = c->heads, hd = D / H, F = c->ffn, V = c->vocab, L = c->layers;
    const double scale = 1.0 / sqrt((double)hd);
    double *sc = (double *)malloc((size_t)T * T * 8);
    double *qh = (double *)malloc((size_t)T * hd * 8);
    double *kh = (double *)malloc((size_t)T * hd * 8);
    double *vh = (double *)malloc((size_t)T * hd * 8);
    double *oh = (double *)malloc((size_t)T * hd * 8);
    double *tmp = (double *)malloc((size_t)T * D * 8);

    for (int t = 0; t < T; ++t) {
        const int id = ids[t];
        for (int j = 0; j < D; ++j)
            a->res[(int64_t)t * D + j] = (id >= 0 && id < V) ? P[(int64_t)id * D + j] : 0.0;
    }
    for (int l = 0; l < L; ++l) {
        ora_w w; set_layer(c, P, l, &w);
        const double *xin = a->res + (int64_t)l * T * D;
        double *mid = a->mid + (int64_t)l * T * D;
        double *xout = a->res + (int64_t)(l + 1) * T * D;
        double *h1 = a->h1 + (int64_t)l * T * D, *h2 = a->h2 + (int64_t)l * T * D;
        double *qkv = a->qkv + (int64_t)l * T * 3 * D;
        double *ctx = a->ctx + (int64_t)l * T * D;
        double *h13 = a->h13 + (int64_t)l * T * 2 * F;
        double *hs = a->hs + (int64_t)l * T * F;

        rmsnorm_rows(xin, w.ln1, h1, a->inv1 + (int64_t)l * T, T, D, c->eps);
        round_bf16(c, h1, (int64_t)T * D);
        mm(h1, w.wqkv, qkv, T, D, 3 * D, 0);
        round_bf16(c, qkv, (int64_t)T * 3 * D);
        for (int h = 0; h < H; ++h) {
            rope_head(qkv + h * hd, T, hd, 3 * D, 0, c->rope_base, c->rope_interleaved, 0);
            rope_head(qkv + D + h * hd, T, hd, 3 * D, 0, c->rope_base, c->rope_interleaved, 0);
        }
        round_bf16(c, qkv, (int64_t)T * 3 * D);
        for (int h = 0; h < H; ++h) {
            for (int t = 0; t < T; ++t)
                for (int j = 0; j < hd; ++j) {
                    qh[t * hd + j] = qkv[(int64_t)t * 3 * D + h * hd + j];
                    kh[t * hd + j] = qkv[(int64_t)t * 3 * D + D + h * hd + j];
                    vh[t * hd + j] = qkv[(int64_t)t * 3 * D + 2 * D + h * hd + j];
                }
            mm_nt(qh, kh, sc, T, hd, T, 0);
            double *pr = a->pr + ((int64_t)l * H + h) * T * T;
            for (int i = 0; i < T; ++i) {
                const int n = i + 1;           /* causal limit */
                double mx = -INFINITY;
                for (int j = 0; j < n; ++j) {
                    sc[i * T + j] *= scale;
                    if (sc[i * T + j] > mx) mx = sc[i * T + j];
                }
                double sum = 0.0;
                for (int j = 0; j < n; ++j) {
                    const double e = exp(sc[i * T + j] - mx);
                    pr[i * T + j] = e; sum += e;
                }
                const double inv = 1.0 / sum;
                for (int j = 0; j < n; ++j) pr[i * T + j] *= inv;
                for (int j = n; j < T; ++j) pr[i * T + j] = 0.0;
            }
            mm(pr, vh, oh, T, T, hd, 0);
            for (int t = 0; t < T; ++t)
                for (int j = 0; j < hd; ++j) ctx[(int64_t)t * D + h * hd + j] = oh[t * hd + j];
        }
        round_bf16(c, ctx, (int64_t)T * D);
        mm(ctx, w.wo, tmp, T, D, D, 0);
        for (int64_t i = 0; i < (int64_t)T * D; ++i) mid[i] = xin[i] + tmp[i];

        rmsnorm_rows(mid, w.ln2, h2, a->inv2 + (int64_t)l * T, T, D, c->eps);
        round_bf16(c, h2, (int64_t)T * D);
        mm(h2, w.w13, h13, T, D, 2 * F, 0);
        round_bf16(c, h13, (int64_t)T * 2 * F);
        for (int t = 0; t < T; ++t)
            for (int j = 0; j < F; ++j) {
                const double g = h13[(int64_t)t * 2 * F + j], u = h13[(int64_t)t * 2 * F + F + j];
                hs[(int64_t)t * F + j] = g * sigmoid_stable(g) * u;
            }
        round_bf16(c, hs, (int64_t)T * F);
        mm(hs, w.w2, tmp, T, F, D, 0);
        for (int64_t i = 0; i < (int64_t)T * D; ++i) xout[i] = mid[i] + tmp[i];
    }
    rmsnorm_rows(a->res + (int64_t)L * T * D, P + lnf_off(c), a->hf, a->invf, T, D, c->eps);
    round_bf16(c, a->hf, (int64_t)T * D);
    if (c->tie) mm_nt(a->hf, P, logits, T, D, V, 0);
    else        mm(a->hf, P + lnf_off(c) + D, logits, T, D, V, 0);

    free(sc); free(qh); free(kh); free(vh); free(oh); free(tmp);
}

/* logits [B*T, V] for B independent sequences of T tokens each. */
int ora_forward(const ora_cfg *c, const double *P, const int32_t *ids, int B, int T,
                double *logits)
{
    #pragma omp parallel for schedule(dynamic)
    for (int b = 0; b < B; ++b) {
        ora_act a = act_alloc(c, T);
        forward_seq(c, P, ids + (int64_t)b * T, T, &a, logits + (int64_t)b * T * c->vocab);
        act_free(&a);
    }
    return 0;
}

/* Backward of one sequence given dlogits [T,V]; accumulates into G (size nparams). */
static void backward_seq(const ora_cfg *c, const double *P, const int32_t *ids, int T,
                         const ora_act *a, const double *dlogits, double *G)
{
    const int D = c->dim, H = c->heads, hd = D / H, F = c->ffn, V = c->vocab, L = c->layers;
    const double scale = 1.0 / sqrt((double)hd);
    double *dres = (double *)calloc((size_t)T * D, 8);
    double *dhf = (double *)calloc((size_t)T * D, 8);
    double *dhs = (double *)malloc((size_t)T * F * 8);
    double *dh13 = (double *)malloc((size_t)T * 2 * F * 8);
    double *dh = (double *)malloc((size_t)T * D * 8);
    double *dctx = (double *)malloc((size_t)T * D * 8);
    double *dqkv = (double *)malloc((size_t)T * 3 * D * 8);
    double *dpr = (double *)malloc((size_t)T * T * 8);
    double *qh = (double *)malloc((size_t)T * hd * 8), *kh = (double *)malloc((size_t)T * hd * 8);
    double *vh = (double *)malloc((size_t)T * hd * 8), *doh = (double *)malloc((size_t)T * hd * 8);
    double *dqh = (double *)malloc((size_t)T * hd * 8), *dkh = (double *)malloc((size_t)T * hd * 8);
    double *dvh = (double *)malloc((size_t)T * hd * 8);

    /* head */
    if (c->tie) {
        /* logits = hf emb^T : demb += dlogits^T hf ; dhf = dlogits emb */
        mm_tn_acc(dlogits, a->hf, G, T, V, D);
        mm(dlogits, P, dhf, T, V, D, 0);
    } else {
        const double *Wh = P + lnf_off(c) + D;
        mm_tn_acc(a->hf, dlogits, G + lnf_off(c) + D, T, D, V);
        mm_nt(dlogits, Wh, dhf, T, V, D, 0);
    }
    rmsnorm_bwd_rows(a->res + (int64_t)L * T * D, P + lnf_off(c), a->invf, dhf, dres,
                     G + lnf_off(c), T, D);

    for (int l = L - 1; l >= 0; --l) {
        ora_w w; set_layer(c, P, l, &w);
        const double *xin = a->res + (int64_t)l * T * D;
        const double *mid = a->mid + (int64_t)l * T * D;
        const double *h1 = a->h1 + (int64_t)l * T * D, *h2 = a->h2 + (int64_t)l * T * D;
        const double *qkv = a->qkv + (int64_t)l * T * 3 * D;
        const double *ctx = a->ctx + (int64_t)l * T * D;
        const double *h13 = a->h13 + (int64_t)l * T * 2 * F;
        const double *hs = a->hs + (int64_t)l * T * F;

        /* xout = mid + hs W2 */
        mm_nt(dres, w.w2, dhs, T, D, F, 0);
        mm_tn_acc(hs, dres, G + layer_off(c, l, 5), T, F, D);
        for (int t = 0; t < T; ++t)
            for (int j = 0; j < F; ++j) {
                const double g = h13[(int64_t)t * 2 * F + j], u = h13[(int64_t)t * 2 * F + F + j];
                const double s = sigmoid_stable(g), go = dhs[(int64_t)t * F + j];
                dh13[(int64_t)t * 2 * F + j] = go * u * (s * (1.0 + g * (1.0 - s)));
                dh13[(int64_t)t * 2 * F + F + j] = go * g * s;
            }
        mm_tn_acc(h2, dh13, G + layer_off(c, l, 4), T, D, 2 * F);
        mm_nt(dh13, w.w13, dh, T, 2 * F, D, 0);
        /* dres (grad wrt mid) += rmsnorm_bwd(dh) */
        rmsnorm_bwd_rows(mid, w.ln2, a->inv2 + (int64_t)l * T, dh, dres,
                         G + layer_off(c, l, 3), T, D);

        /* mid = xin + ctx Wo */
        mm_nt(dres, w.wo, dctx, T, D, D, 0);
        mm_tn_acc(ctx, dres, G + layer_off(c, l, 2), T, D, D);
        for (int h = 0; h < H; ++h) {
            const double *pr = a->pr + ((int64_t)l * H + h) * T * T;
            for (int t = 0; t < T; ++t)
                for (int j = 0; j < hd; ++j) {
                    qh[t * hd + j] = qkv[(int64_t)t * 3 * D + h * hd + j];
                    kh[t * hd + j] = qkv[(int64_t)t * 3 * D + D + h * hd + j];
                    vh[t * hd + j] = qkv[(int64_t)t * 3 * D + 2 * D + h * hd + j];
                    doh[t * hd + j] = dctx[(int64_t)t * D + h * hd + j];
                }
            mm_nt(doh, vh, dpr, T, hd, T, 0);             /* dP = dO V^T */
            memset(dvh, 0, (size_t)T * hd * 8);
            mm_tn_acc(pr, doh, dvh, T, T, hd);            /* dV = P^T dO */
            for (int i = 0; i < T; ++i) {                 /* dS = P (dP - dot) * scale */
                const int n = i + 1;
                double dot = 0.0;
                for (int j = 0; j < n; ++j) dot += dpr[i * T + j] * pr[i * T + j];
                for (int j = 0; j < n; ++j)
                    dpr[i * T + j] = scale * pr[i * T + j] * (dpr[i * T + j] - dot);
                for (int j = n; j < T; ++j) dpr[i * T + j] = 0.0;
            }
            mm(dpr, kh, dqh, T, T, hd, 0);                /* dQ = dS K */
            memset(dkh, 0, (size_t)T * hd * 8);
            mm_tn_acc(dpr, qh, dkh, T, T, hd);            /* dK = dS^T Q */
            rope_head(dqh, T, hd, hd, 0, c->rope_base, c->rope_interleaved, 1);
            rope_head(dkh, T, hd, hd, 0, c->rope_base, c->rope_interleaved, 1);
            for (int t = 0; t < T; ++t)
                for (int j = 0; j < hd; ++j) {
                    dqkv[(int64_t)t * 3 * D + h * hd + j] = dqh[t * hd + j];
                    dqkv[(int64_t)t * 3 * D + D + h * hd + j] = dkh[t * hd + j];
                    dqkv[(int64_t)t * 3 * D + 2 * D + h * hd + j] = dvh[t * hd + j];
                }
        }
        mm_tn_acc(h1, dqkv, G + layer_off(c, l, 1), T, D, 3 * D);
        mm_nt(dqkv, w.wqkv, dh, T, 3 * D, D, 0);
        rmsnorm_bwd_rows(xin, w.ln1, a->inv1 + (int64_t)l * T, dh, dres,
                         G + layer_off(c, l, 0), T, D);
    }
    for (int t = 0; t < T; ++t) {
        const int id = ids[t];
        if (id < 0 || id >= V) continue;
        for (int j = 0; j < D; ++j) G[(int64_t)id * D + j] += dres[(int64_t)t * D + j];
    }
    free(dres); free(dhf); free(dhs); free(dh13); free(dh); free(dctx); free(dqkv); free(dpr);
    free(qh); free(kh); free(vh); free(doh); free(dqh); free(dkh); free(dvh);
}

/*
 * Forward + cross-entropy + full backward over a [B,T] block.
 * targets < 0 are padding: loss 0, no gradient.  loss = sum / valid,
 * dlogits = (softmax - onehot) / valid, valid = number of non-padding rows
 * (at least 1).  Outputs (any may be NULL): grads[nparams], loss[1],
 * logits[B*T*V], pred[B*T] (first strict maximum, 0-indexed), losses[B*T].
 */
int ora_loss_grad(const ora_cfg *c, const double *P, const int32_t *ids, const int32_t *tgt,
                  int B, int T, double *grads, double *loss, double *logits_out,
                  int32_t *pred, double *losses_out)
{
    const int V = c->vocab;
    const int64_t np = ora_nparams(c);
    int valid = 0;
    for (int64_t r = 0; r < (int64_t)B * T; ++r) if (tgt[r] >= 0 && tgt[r] < V) ++valid;
    if (valid < 1) valid = 1;
    const double gs = 1.0 / valid;
    double total = 0.0;
    if (grads) memset(grads, 0, (size_t)np * 8);

    #pragma omp parallel for schedule(dynamic)
    for (int b = 0; b < B; ++b) {
        ora_act a = act_alloc(c, T);
        double *lg = (double *)malloc((size_t)T * V * 8);
        double *G = grads ? (double *)calloc((size_t)np, 8) : NULL;
        const int32_t *idb = ids + (int64_t)b * T, *tb = tgt + (int64_t)b * T;
        forward_seq(c, P, idb, T, &a, lg);
        if (logits_out) memcpy(logits_out + (int64_t)b * T * V, lg, (size_t)T * V * 8);
        double lsum = 0.0;
        for (int t = 0; t < T; ++t) {
            double *row = lg + (int64_t)t * V;
            int best = 0; double bv = -INFINITY;
            for (int j = 0; j < V; ++j) if (row[j] > bv) { bv = row[j]; best = j; }
            if (pred) pred[(int64_t)b * T + t] = best;
            const int y = tb[t];
            if (y < 0 || y >= V) {
                if (losses_out) losses_out[(int64_t)b * T + t] = 0.0;
                for (int j = 0; j < V; ++j) row[j] = 0.0;
                continue;
            }
            double sum = 0.0;
            for (int j = 0; j < V; ++j) sum += exp(row[j] - bv);
            const double li = (bv + log(sum)) - row[y];
            if (losses_out) losses_out[(int64_t)b * T + t] = li;
            lsum += li;
            const double inv = 1.0 / sum;
            for (int j = 0; j < V; ++j) {
                double p = exp(row[j] - bv) * inv;
                if (j == y) p -= 1.0;
                row[j] = p * gs;
            }
        }
        if (G) backward_seq(c, P, idb, T, &a, lg, G);
        #pragma omp critical
        {
            total += lsum;
            if (G) for (int64_t i = 0; i < np; ++i) grads[i] += G[i];
        }
        free(G); free(lg); act_free(&a);
    }
    if (loss) *loss = total * gs;
    return valid;
}

double ora_grad_norm(const double *g, int64_t n)
{
    double s = 0.0;
    for (int64_t i = 0; i < n; ++i) s += g[i] * g[i];
    return sqrt(s);
}

/* p -= lr * (g + wd * p); wd only where mask != 0 (mask may be NULL = everywhere). */
void ora_sgd(double *p, const double *g, const uint8_t *mask, int64_t n, double lr, double wd)
{
    for (int64_t i = 0; i < n; ++i) {
        double gk = g[i];
        if (wd != 0.0 && (!mask || mask[i])) gk += wd * p[i];
        p[i] -= lr * gk;
    }
}

/* ---- KV-cache decode ---- */

typedef struct {
    int32_t n, cap;
    double *k, *v;        /* [L][cap*D] */
    double *buf;          /* scratch */
} ora_state;

ora_state *ora_state_new(const ora_cfg *c)
{
    ora_state *s = (ora_state *)calloc(1, sizeof(ora_state));
    s->cap = c->max_seq;
    s->k = (double *)calloc((size_t)c->layers * s->cap * c->dim, 8);
    s->v = (double *)calloc((size_t)c->layers * s->cap * c->dim, 8);
    s->buf = (double *)calloc((size_t)(8 * c->dim + 3 * c->ffn + c->max_seq + 16), 8);
    return s;
}
void ora_state_reset(ora_state *s) { s->n = 0; }
int  ora_state_len(const ora_state *s) { return s->n; }
void ora_state_free(ora_state *s) { if (s) { free(s->k); free(s->v); free(s->buf); free(s); } }

static void vecmat(const double *x, const double *W, int fin, int fout, int ldw, double *out)
{
    for (int j = 0; j < fout; ++j) out[j] = 0.0;
    for (int i = 0; i < fin; ++i) {
        const double xv = x[i];
        if (xv == 0.0) continue;
        const double *w = W + (int64_t)i * ldw;
        for (int j = 0; j < fout; ++j) out[j] += xv * w[j];
    }
}

/* One token through the model with the per-layer K/V appended at position
 * state->n.  Returns -1 when the context is full or the id is out of range. */
int ora_step(const ora_cfg *c, const double *P, ora_state *st, int id, double *logits)
{
    const int D = c->dim, H = c->heads, hd = D / H, F = c->ffn, V = c->vocab;
    const int pos = st->n;
    if (pos >= c->max_seq || id < 0 || id >= V) return -1;
    const double scale = 1.0 / sqrt((double)hd);
    double *x = st->buf, *h = x + D, *qkv = h + D, *ctx = qkv + 3 * D, *o = ctx + D;
    double *gu = o + D, *hsv = gu + 2 * F, *att = hsv + F;

    for (int j = 0; j < D; ++j) x[j] = P[(int64_t)id * D + j];
    for (int l = 0; l < c->layers; ++l) {
        ora_w w; set_layer(c, P, l, &w);
        rmsnorm_rows(x, w.ln1, h, NULL, 1, D, c->eps);
        round_bf16(c, h, D);
        vecmat(h, w.wqkv, D, 3 * D, 3 * D, qkv);
        round_bf16(c, qkv, 3 * D);
        for (int hh = 0; hh < H; ++hh) {
            rope_head(qkv + hh * hd, 1, hd, 3 * D, pos, c->rope_base, c->rope_interleaved, 0);
            rope_head(qkv + D + hh * hd, 1, hd, 3 * D, pos, c->rope_base, c->rope_interleaved, 0);
        }
        round_bf16(c, qkv, 3 * D);
        double *kc = st->k + (int64_t)l * st->cap * D, *vc = st->v + (int64_t)l * st->cap * D;
        for (int j = 0; j < D; ++j) {
            kc[(int64_t)pos * D + j] = qkv[D + j];
            vc[(int64_t)pos * D + j] = qkv[2 * D + j];
        }
        const int n = pos + 1;
        for (int hh = 0; hh < H; ++hh) {
            const int off = hh * hd;
            double mx = -INFINITY;
            for (int t = 0; t < n; ++t) {
                double s = 0.0;
                for (int j = 0; j < hd; ++j) s += qkv[off + j] * kc[(int64_t)t * D + off + j];
                s *= scale; att[t] = s;
                if (s > mx) mx = s;
            }
            double sum = 0.0;
            for (int t = 0; t < n; ++t) { att[t] = exp(att[t] - mx); sum += att[t]; }
            const double inv = 1.0 / sum;
            for (int j = 0; j < hd; ++j) ctx[off + j] = 0.0;
            for (int t = 0; t < n; ++t) {
                const double wt = att[t] * inv;
                if (wt == 0.0) continue;
                for (int j = 0; j < hd; ++j) ctx[off + j] += wt * vc[(int64_t)t * D + off + j];
            }
        }
        round_bf16(c, ctx, D);
        vecmat(ctx, w.wo, D, D, D, o);
        for (int j = 0; j < D; ++j) x[j] += o[j];
        rmsnorm_rows(x, w.ln2, h, NULL, 1, D, c->eps);
        round_bf16(c, h, D);
        vecmat(h, w.w13, D, 2 * F, 2 * F, gu);
        round_bf16(c, gu, 2 * F);
        for (int j = 0; j < F; ++j) hsv[j] = gu[j] * sigmoid_stable(gu[j]) * gu[F + j];
        round_bf16(c, hsv, F);
        vecmat(hsv, w.w2, F, D, D, o);
        for (int j = 0; j < D; ++j) x[j] += o[j];
    }
    rmsnorm_rows(x, P + lnf_off(c), h, NULL, 1, D, c->eps);
    round_bf16(c, h, D);
    if (c->tie) {
        for (int r = 0; r < V; ++r) {
            double s = 0.0;
            const double *e = P + (int64_t)r * D;
            for (int j = 0; j < D; ++j) s += h[j] * e[j];
            logits[r] = s;
        }
    } else {
        vecmat(h, P + lnf_off(c) + D, D, V, V, logits);
    }
    st->n = pos + 1;
    return 0;
}

static int pick_greedy(const double *row, int n)
{
    int best = 0; double bv = -INFINITY;
    for (int j = 0; j < n; ++j) if (row[j] > bv) { bv = row[j]; best = j; }
    return best;
}

/*
 * Greedy generation with the KV cache for B independent sequences.
 * prompts [B, n_prompt] (0-indexed ids); out [B, n_new].  When the state is
 * full it is rebuilt from the last max_seq tokens, as the reference's
 * generate does.  last_logits (may be NULL) receives, per sequence, the
 * logits that produced the FIRST generated token ([B, V]).
 */
int ora_greedy(const ora_cfg *c, const double *P, const int32_t *prompts, int B, int n_prompt,
               int n_new, int32_t *out, double *first_logits)
{
    const int V = c->vocab, ctxmax = c->max_seq;
    int rc = 0;
    #pragma omp parallel for schedule(dynamic)
    for (int b = 0; b < B; ++b) {
        ora_state *st = ora_state_new(c);
        double *lg = (double *)malloc((size_t)V * 8);
        int32_t *tok = (int32_t *)malloc((size_t)(n_prompt + n_new) * 4);
        int ntok = n_prompt;
        memcpy(tok, prompts + (int64_t)b * n_prompt, (size_t)n_prompt * 4);
        int first = ntok - ctxmax; if (first < 0) first = 0;
        for (int i = first; i < ntok; ++i) if (ora_step(c, P, st, tok[i], lg)) rc = -1;
        if (first_logits) memcpy(first_logits + (int64_t)b * V, lg, (size_t)V * 8);
        for (int s = 0; s < n_new; ++s) {
            const int nx = pick_greedy(lg, V);
            tok[ntok++] = nx;
            out[(int64_t)b * n_new + s] = nx;
            if (s == n_new - 1) break;
            if (st->n >= ctxmax) {
                ora_state_reset(st);
                int lo = ntok - ctxmax; if (lo < 0) lo = 0;
                for (int i = lo; i < ntok; ++i) if (ora_step(c, P, st, tok[i], lg)) rc = -1;
            } else if (ora_step(c, P, st, nx, lg)) rc = -1;
        }
        free(tok); free(lg); ora_state_free(st);
    }
    return rc;
}

/* ---- op-level restatements used by the known-answer tests ---- */

/* Row softmax with optional causal limit (row i keeps columns <= i + offset). */
void ora_softmax_rows(const double *x, double *y, int rows, int cols, int causal, int offset)
{
    for (int i = 0; i < rows; ++i) {
        int n = cols;
        if (causal) { n = i + 1 + offset; if (n > cols) n = cols; if (n < 1) n = 1; }
        double mx = -INFINITY;
        for (int j = 0; j < n; ++j) if (x[(int64_t)i * cols + j] > mx) mx = x[(int64_t)i * cols + j];
        if (mx == -INFINITY || mx != mx) mx = 0.0;
        double sum = 0.0;
        for (int j = 0; j < n; ++j) {
            const double e = exp(x[(int64_t)i * cols + j] - mx);
            y[(int64_t)i * cols + j] = e; sum += e;
        }
        if (!(sum > 0)) sum = 1.0;
        for (int j = 0; j < n; ++j) y[(int64_t)i * cols + j] /= sum;
        for (int j = n; j < cols; ++j) y[(int64_t)i * cols + j] = 0.0;
    }
}

/* Mean cross-entropy over rows whose target != ignore (targets 0-indexed). */
double ora_cross_entropy(const double *x, const int32_t *tgt, int rows, int cols, int ignore)
{
    double total = 0.0; int counted = 0;
    for (int i = 0; i < rows; ++i) {
        if (tgt[i] == ignore) continue;
        const double *r = x + (int64_t)i * cols;
        double mx = -INFINITY, sum = 0.0;
        for (int j = 0; j < cols; ++j) if (r[j] > mx) mx = r[j];
        for (int j = 0; j < cols; ++j) sum += exp(r[j] - mx);
        total += (mx + log(sum)) - r[tgt[i]];
        ++counted;
    }
    if (counted == 0) counted = 1;
    return total / counted;
}

void ora_matmul(const double *A, const double *B, double *C, int M, int K, int N)
{
    mm(A, B, C, M, K, N, 0);
}

void ora_rmsnorm(const double *x, const double *w, double *y, int rows, int cols, double eps)
{
    rmsnorm_rows(x, w, y, NULL, rows, cols, eps);
}

void ora_rope(double *x, int rows, int heads, int hd, int pos0, double base, int interleaved,
              int inverse)
{
    for (int h = 0; h < heads; ++h)
        rope_head(x + h * hd, rows, hd, heads * hd, pos0, base, interleaved, inverse);
}
