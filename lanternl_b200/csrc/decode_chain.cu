// The part of a decode step between two attention kernels as ONE cooperative launch.
//
// A decode step of the bf16 model is a chain of small dependent products on [sequences, dim] activations:
//   attention -> Wo (+ residual) -> RMSNorm -> W13 + SwiGLU -> W2 (+ residual) -> RMSNorm -> QKV of the next layer
// (or the lm_head after the last layer).  As separate kernels each link costs a dependent launch (about 4 us here even
// with programmatic dependent launch) whatever its size, and 51 of them were 40 % of a step at 256 sequences and 80 %
// at 32.  This kernel runs the four products of a layer in one launch: a fixed grid of CTAs (at most one per SM, all
// resident: a cooperative launch) walks the output tiles of a phase, meets at a grid barrier in L2, and goes on to the
// next phase; a layer then costs two launches (attention, chain) instead of seven.
//
//   * The products are too small for bytes or flops to matter (a phase moves 0.5 .. 3 MB of L2-resident weights and
//     0.07 .. 0.4 GFLOP): what counts is the number of dependent memory round trips.  A tile therefore fetches its whole
//     A panel [BM, K] and B panel [BN, K] with one wave of cp.async (one round trip), computes from shared memory with
//     mma.sync.m16n8k16 (bf16, fp32 accumulate; operands through ldmatrix from rows padded by 16 bytes, conflict free),
//     and writes its epilogue.  The B panel of a CTA's first tile of the NEXT phase - weights, which no phase writes -
//     is requested before the barrier, so it arrives while the CTA waits.
//   * RMSNorm is folded into the A load of the product that consumes it: the tile reads its rows of the fp32 residual
//     stream, normalises them (row sum by warp shuffle, the expression of the stand-alone kernel: x * rsqrt * gain,
//     rounded to bf16) straight into the A panel.  Tiles of the same row block repeat this (L2 reads), which is cheaper
//     than a phase of its own.
//   * Residual products add into the fp32 stream in place; every element is owned by one thread (no split-K, no atomics),
//     so results do not depend on scheduling.
//   * The first launch of a step has no attention before it: its only phase gathers the embedding rows (into the stream)
//     in the A load of layer 0's QKV product.
//
// Grid barrier: a counter and a generation word in global memory.  A CTA reads the generation, arrives with one atomic;
// the last arrival resets the counter and bumps the generation (release), the others poll it (acquire).  Polling is
// bounded: a CTA that gives up raises the error word and goes on, so the kernel always terminates; the host then reports
// LUATL_ERR_CUDA and resets the barrier.  All CTAs are co-resident by construction (cooperative launch, grid <= SMs).
#include <string.h>

#include "common.cuh"
#include "ops.h"

namespace {

constexpr int CH_THREADS = 256;                 // 8 warps
constexpr int CH_PAD = 8;                       // bf16 elements of padding per panel row (16 bytes)
constexpr int CH_A_BYTES = 94 * 1024;           // A panel region; the B panel region follows it
constexpr int CH_B_BYTES = 94 * 1024;
constexpr unsigned CH_SPIN = 1u << 24;          // barrier polls before a CTA gives up (tens of milliseconds)

enum { EPI_RESID = 0, EPI_SWIGLU = 1, EPI_BF16 = 2, EPI_F32 = 3 };
enum { A_BF16 = 0, A_NORM = 1, A_EMBED = 2 };

struct Phase {
    int a_kind, epi;
    int N, K;                   // output columns (rows of B), contraction length
    const void* a;              // A_BF16: bf16 [M, K]; A_NORM: fp32 x [M, K]; A_EMBED: bf16 table [vocab, K]
    const float* gain;          // A_NORM / A_EMBED: [K]
    const bf16* b;              // [N, K], K contiguous
    void* out;                  // EPI_RESID: fp32 x [M, N]; EPI_SWIGLU: bf16 [M, N/2]; EPI_BF16 / EPI_F32: [M, N]
    int tile;                   // 0: 16x64, 1: 16x32, 2: 32x64, 3: 32x32, 4: 64x64
};

struct ChainParams {
    int M, nphases;
    float eps;
    const int32_t* tok;         // A_EMBED: token ids [M]
    int vocab;
    float* x;                   // A_EMBED: the residual stream the gathered rows are written to
    unsigned* bar;              // [0] arrivals, [1] generation
    int* err;
    Phase ph[4];
};

__device__ __forceinline__ void cp16(void* dst, const void* src)
{
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], const void* p)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0, %1}, [%2];"
                 : "=r"(r[0]), "=r"(r[1]) : "r"((uint32_t)__cvta_generic_to_shared(p)));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2])
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Reusable grid barrier (see the header).  Returns false when the wait ran out.
__device__ bool grid_barrier(unsigned* bar, int* err)
{
    __shared__ int ok_s;
    __syncthreads();
    if (threadIdx.x == 0) {
        bool ok = true;
        unsigned gen;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(gen) : "l"(bar + 1) : "memory");
        __threadfence();                                          // this CTA's writes of the phase are visible device-wide
        const unsigned arrived = atomicAdd(bar, 1u);
        if (arrived == gridDim.x - 1) {
            atomicExch(bar, 0u);
            __threadfence();
            asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(bar + 1), "r"(gen + 1u) : "memory");
        } else {
            unsigned now = gen, polls = 0;
            do {
                asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(now) : "l"(bar + 1) : "memory");
                if (now != gen) break;
                __nanosleep(32);
            } while (++polls < CH_SPIN);
            if (now == gen) { ok = false; if (err) atomicExch(err, 3); }
        }
        ok_s = ok ? 1 : 0;
    }
    __syncthreads();
    return ok_s != 0;
}

// Tile shapes: WM x WN warps (8 in all, or 4 working), every warp 16 rows x NT n8 tiles.
template <int WM_, int WN_, int NT_> struct Shape { static constexpr int WM = WM_, WN = WN_, NT = NT_, BM = 16 * WM_, BN = 8 * NT_ * WN_; };
typedef Shape<1, 8, 1> S16x64;
typedef Shape<1, 4, 1> S16x32;
typedef Shape<2, 4, 2> S32x64;
typedef Shape<2, 4, 1> S32x32;
typedef Shape<4, 2, 4> S64x64;

__host__ __device__ inline void tile_dims(int tile, int& bm, int& bn)
{
    switch (tile) {
    case 0: bm = 16; bn = 64; break;
    case 1: bm = 16; bn = 32; break;
    case 2: bm = 32; bn = 64; break;
    case 3: bm = 32; bn = 32; break;
    default: bm = 64; bn = 64; break;
    }
}

// B panel of tile column block n0: rows n0 .. n0 + BN - 1 of W [N, K] (rows past N are zero filled).
__device__ __forceinline__ void load_b_panel(unsigned char* sB, const bf16* W, int N, int K, int n0, int BN)
{
    const int pitch = (K + CH_PAD) * 2, per_row = K / 8;
    for (int i = threadIdx.x; i < BN * per_row; i += CH_THREADS) {
        const int r = i / per_row, p = i - r * per_row;
        unsigned char* dst = sB + r * pitch + p * 16;
        if (n0 + r < N) cp16(dst, W + (size_t)(n0 + r) * K + p * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
}

// A panel, bf16 source.
__device__ __forceinline__ void load_a_bf16(unsigned char* sA, const bf16* A, int M, int K, int m0, int BM)
{
    const int pitch = (K + CH_PAD) * 2, per_row = K / 8;
    for (int i = threadIdx.x; i < BM * per_row; i += CH_THREADS) {
        const int r = i / per_row, p = i - r * per_row;
        unsigned char* dst = sA + r * pitch + p * 16;
        if (m0 + r < M) cp16(dst, A + (size_t)(m0 + r) * K + p * 8);
        else *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
    }
}

// A panel from the fp32 residual stream, normalised (RMSNorm with gain) and rounded to bf16.  A warp takes RB rows at a time
// and issues the loads of all of them before it reduces any (one memory round trip per RB rows); NJ = float4 packets per
// lane and row (K <= 128 * NJ).  With `tok` the rows are first gathered from the bf16 embedding table and, when write_x is
// set, written to the stream.
template <int NJ, int RB>
__device__ __forceinline__ void load_a_norm_t(unsigned char* sA, const float* x, const float* gain, int M, int K, int m0, int BM,
                                              float eps, const int32_t* tok, const bf16* table, int vocab, float* xout, bool write_x)
{
    const int pitch = (K + CH_PAD) * 2, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    constexpr int NW = CH_THREADS / 32;
    for (int rb = warp * RB; rb < BM; rb += NW * RB) {
        float4 v[RB][NJ];
#pragma unroll
        for (int i = 0; i < RB; ++i) {
            const int row = m0 + rb + i;
            const bool live = rb + i < BM && row < M;
            int t = 0;
            bool okid = true;
            if (tok && live) { t = tok[row]; okid = t >= 0 && t < vocab; }
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const int c = lane * 4 + 128 * j;
                float4 q = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
                if (live && c < K) {
                    if (tok) {
                        if (okid) {
                            const uint2 raw = *reinterpret_cast<const uint2*>(table + (size_t)t * K + c);
                            q = make_float4(__uint_as_float(raw.x << 16), __uint_as_float(raw.x & 0xFFFF0000u),
                                            __uint_as_float(raw.y << 16), __uint_as_float(raw.y & 0xFFFF0000u));
                        }
                    } else {
                        q = __ldcg(reinterpret_cast<const float4*>(x + (size_t)row * K + c));
                    }
                }
                v[i][j] = q;
            }
        }
#pragma unroll
        for (int i = 0; i < RB; ++i) {
            if (rb + i >= BM) continue;
            const int row = m0 + rb + i;
            unsigned char* dst = sA + (rb + i) * pitch;
            float ss = 0.0f;
#pragma unroll
            for (int j = 0; j < NJ; ++j) ss = fmaf(v[i][j].x, v[i][j].x, fmaf(v[i][j].y, v[i][j].y, fmaf(v[i][j].z, v[i][j].z, fmaf(v[i][j].w, v[i][j].w, ss))));
            ss = warp_sum(ss);
            const float sc = 1.0f / sqrtf(ss / (float)K + eps);
#pragma unroll
            for (int j = 0; j < NJ; ++j) {
                const int c = lane * 4 + 128 * j;
                if (c >= K) continue;
                uint2 pk = make_uint2(0u, 0u);
                if (row < M) {
                    const float4 g = *reinterpret_cast<const float4*>(gain + c);
                    pk.x = pack_bf16x2(v[i][j].x * sc * g.x, v[i][j].y * sc * g.y);
                    pk.y = pack_bf16x2(v[i][j].z * sc * g.z, v[i][j].w * sc * g.w);
                    if (tok && write_x) *reinterpret_cast<float4*>(xout + (size_t)row * K + c) = v[i][j];
                }
                *reinterpret_cast<uint2*>(dst + c * 2) = pk;
            }
        }
    }
}

__device__ __forceinline__ void load_a_norm(unsigned char* sA, const float* x, const float* gain, int M, int K, int m0, int BM,
                                            float eps, const int32_t* tok, const bf16* table, int vocab, float* xout, bool write_x)
{
    if (K <= 512) load_a_norm_t<4, 4>(sA, x, gain, M, K, m0, BM, eps, tok, table, vocab, xout, write_x);
    else if (K <= 1024) load_a_norm_t<8, 2>(sA, x, gain, M, K, m0, BM, eps, tok, table, vocab, xout, write_x);
    else load_a_norm_t<16, 1>(sA, x, gain, M, K, m0, BM, eps, tok, table, vocab, xout, write_x);
}

// One output tile from the panels in shared memory, and its epilogue.
template <class S>
__device__ __forceinline__ void compute_tile(const unsigned char* sA, const unsigned char* sB, const Phase& ph, int M, int m0, int n0)
{
    const int K = ph.K, N = ph.N, pitch = (K + CH_PAD) * 2;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (warp >= S::WM * S::WN) return;
    const int wm = warp / S::WN, wn = warp % S::WN;
    float acc[S::NT][4];
#pragma unroll
    for (int t = 0; t < S::NT; ++t) { acc[t][0] = 0.0f; acc[t][1] = 0.0f; acc[t][2] = 0.0f; acc[t][3] = 0.0f; }
    // ldmatrix row addresses: A x4 = (rows 0-7, k 0-7), (rows 8-15, k 0-7), (rows 0-7, k 8-15), (rows 8-15, k 8-15)
    const unsigned char* ap = sA + (wm * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * pitch + (lane >> 4) * 16;
    // B x2 = (n rows 0-7, k 0-7), (n rows 0-7, k 8-15); lanes 16-31 repeat valid addresses
    const unsigned char* bp = sB + (wn * S::NT * 8 + (lane & 7)) * pitch + ((lane >> 3) & 1) * 16;
#pragma unroll 4
    for (int k0 = 0; k0 < K; k0 += 16) {
        uint32_t a[4];
        ldsm_x4(a, ap + k0 * 2);
#pragma unroll
        for (int t = 0; t < S::NT; ++t) {
            uint32_t b[2];
            ldsm_x2(b, bp + t * 8 * pitch + k0 * 2);
            mma16816(acc[t], a, b);
        }
    }
    // accumulator fragment: c0, c1 = (row g, columns 2t, 2t + 1), c2, c3 = (row g + 8, same columns)
    const int g = lane >> 2, tq = lane & 3;
#pragma unroll
    for (int t = 0; t < S::NT; ++t) {
        const int n = n0 + (wn * S::NT + t) * 8 + 2 * tq;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = m0 + wm * 16 + g + 8 * h;
            if (row >= M || n >= N) continue;
            const float v0 = acc[t][2 * h], v1 = acc[t][2 * h + 1];
            if (ph.epi == EPI_RESID) {
                float2* p = reinterpret_cast<float2*>(reinterpret_cast<float*>(ph.out) + (size_t)row * N + n);
                float2 o = __ldcg(p);                             // written by another CTA in an earlier phase: read from L2
                o.x += v0; o.y += v1;
                *p = o;
            } else if (ph.epi == EPI_SWIGLU) {
                // interleaved (gate, up) rows of B; both rounded to bf16 first, as a stored gate|up tensor would be
                const float gt = __bfloat162float(__float2bfloat16_rn(v0)), up = __bfloat162float(__float2bfloat16_rn(v1));
                reinterpret_cast<bf16*>(ph.out)[(size_t)row * (N >> 1) + (n >> 1)] = __float2bfloat16_rn(silu_f(gt) * up);
            } else if (ph.epi == EPI_BF16) {
                *reinterpret_cast<uint32_t*>(reinterpret_cast<bf16*>(ph.out) + (size_t)row * N + n) = pack_bf16x2(v0, v1);
            } else {
                *reinterpret_cast<float2*>(reinterpret_cast<float*>(ph.out) + (size_t)row * N + n) = make_float2(v0, v1);
            }
        }
    }
}

__device__ __forceinline__ void dispatch_tile(int tile, const unsigned char* sA, const unsigned char* sB, const Phase& ph, int M, int m0, int n0)
{
    switch (tile) {
    case 0: compute_tile<S16x64>(sA, sB, ph, M, m0, n0); break;
    case 1: compute_tile<S16x32>(sA, sB, ph, M, m0, n0); break;
    case 2: compute_tile<S32x64>(sA, sB, ph, M, m0, n0); break;
    case 3: compute_tile<S32x32>(sA, sB, ph, M, m0, n0); break;
    default: compute_tile<S64x64>(sA, sB, ph, M, m0, n0); break;
    }
}

// Work of CTA `cta` in a phase: row block cta % nt_m, column blocks cta / nt_m, + the CTAs of that row block, ... - a CTA
// stays on one row block, so its A panel (and a normalisation, where the load has one) is built once per phase.
struct Assign { int mb, n_first, n_stride, nt_n, bm, bn; };
__device__ __forceinline__ Assign assign(const Phase& ph, int M, int cta, int G)
{
    Assign a;
    tile_dims(ph.tile, a.bm, a.bn);
    const int nt_m = (M + a.bm - 1) / a.bm;
    a.nt_n = (ph.N + a.bn - 1) / a.bn;
    a.mb = cta % nt_m;
    a.n_first = cta / nt_m;
    a.n_stride = (G - a.mb + nt_m - 1) / nt_m;                   // CTAs that share this row block
    return a;
}

__global__ void __launch_bounds__(CH_THREADS, 1)
decode_chain_kernel(const ChainParams P)
{
    extern __shared__ __align__(128) unsigned char ch_smem[];
    unsigned char* sA = ch_smem;
    unsigned char* sB = ch_smem + CH_A_BYTES;
    const int G = gridDim.x, cta = blockIdx.x;
    // first B panel: weights, needed whatever the predecessor kernel is still doing
    bool b_ready = false;
    {
        const Assign a = assign(P.ph[0], P.M, cta, G);
        if (a.n_first < a.nt_n) { load_b_panel(sB, P.ph[0].b, P.ph[0].N, P.ph[0].K, a.n_first * a.bn, a.bn); b_ready = true; }
    }
    pdl_trigger();
    pdl_wait();
    for (int p = 0; p < P.nphases; ++p) {
        const Phase& ph = P.ph[p];
        const Assign a = assign(ph, P.M, cta, G);
        const int m0 = a.mb * a.bm;
        if (a.n_first < a.nt_n) {
            if (ph.a_kind == A_BF16) load_a_bf16(sA, reinterpret_cast<const bf16*>(ph.a), P.M, ph.K, m0, a.bm);
            else if (ph.a_kind == A_NORM) load_a_norm(sA, reinterpret_cast<const float*>(ph.a), ph.gain, P.M, ph.K, m0, a.bm, P.eps,
                                                      nullptr, nullptr, 0, nullptr, false);
            else load_a_norm(sA, nullptr, ph.gain, P.M, ph.K, m0, a.bm, P.eps, P.tok, reinterpret_cast<const bf16*>(ph.a), P.vocab,
                             P.x, a.n_first == 0);
        }
        for (int nb = a.n_first; nb < a.nt_n; nb += a.n_stride) {
            const int n0 = nb * a.bn;
            if (!b_ready) load_b_panel(sB, ph.b, ph.N, ph.K, n0, a.bn);
            b_ready = false;
            cp_wait_all();
            __syncthreads();
            dispatch_tile(ph.tile, sA, sB, ph, P.M, m0, n0);
            __syncthreads();                                     // the B panel is free again
        }
        if (p + 1 < P.nphases) {
            // request this CTA's first B panel of the next phase, then meet the others
            const Phase& nx = P.ph[p + 1];
            const Assign na = assign(nx, P.M, cta, G);
            if (na.n_first < na.nt_n) { load_b_panel(sB, nx.b, nx.N, nx.K, na.n_first * na.bn, na.bn); b_ready = true; }
            grid_barrier(P.bar, P.err);
        }
    }
    cp_wait_all();
}

int pick_tile(int M, int K)
{
    // the panels of a tile must fit: (BM + BN) * (K + 8) * 2 bytes in the two 94 KB regions
    const bool wide = (size_t)64 * (K + CH_PAD) * 2 <= (size_t)CH_A_BYTES;       // K <= 743
    if (wide) return M <= 16 ? 0 : (M <= 32 ? 2 : 4);
    return M <= 16 ? 1 : 3;
}

}  // namespace

bool ltl_decode_chain_supported(int D, int F, int V)
{
    // panels: 32 rows of the longest contraction must fit a region; fragments want K % 16 == 0; the norm loader holds a row
    // in registers (K <= 2048) and reads float4 (K % 4 == 0); SwiGLU and the paired stores want even widths
    const int kmax = D > F ? D : F;
    return (size_t)32 * (kmax + CH_PAD) * 2 <= (size_t)CH_A_BYTES && D % 16 == 0 && F % 16 == 0 && D <= 2048 && V % 2 == 0;
}

int ltl_decode_chain_grid()
{
    static int grid = 0;
    if (grid) return grid;
    cudaFuncSetAttribute(decode_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, CH_A_BYTES + CH_B_BYTES);
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_chain_kernel, CH_THREADS, CH_A_BYTES + CH_B_BYTES) != cudaSuccess ||
        per_sm < 1) {
        cudaGetLastError();
        return 0;
    }
    grid = ltl_sm_count();
    return grid;
}

// One launch: up to four phases (see LtlChainDesc).  Cooperative, so that every CTA of the grid is resident while the
// CTAs wait for each other at the barriers.
int ltl_decode_chain(const LtlChainDesc& d, cudaStream_t s)
{
    if (d.nphases < 1 || d.nphases > 4) return ltl_fail(LTL_ERR_ARG, "decode_chain: %d phases", d.nphases);
    if (!d.bar) return ltl_fail(LTL_ERR_NULL, "decode_chain: no barrier words");
    const int grid_max = ltl_decode_chain_grid();
    if (grid_max < 1) return ltl_fail(LTL_ERR_CUDA, "decode_chain: the kernel does not fit an SM");
    ChainParams P;
    memset(&P, 0, sizeof(P));
    P.M = d.M; P.nphases = d.nphases; P.eps = d.eps; P.tok = d.tok; P.vocab = d.vocab; P.x = d.x; P.bar = d.bar; P.err = d.err;
    int most = 1;
    for (int i = 0; i < d.nphases; ++i) {
        const LtlChainPhase& q = d.ph[i];
        Phase& ph = P.ph[i];
        if (!q.a || !q.b || !q.out || q.N < 2 || q.K < 16 || (q.K % 16) || (q.N & 1))
            return ltl_fail(LTL_ERR_ARG, "decode_chain: phase %d: bad operands (N=%d K=%d)", i, q.N, q.K);
        if ((q.a_kind == A_NORM || q.a_kind == A_EMBED) && (!q.gain || q.K > 2048 || (q.K % 4)))
            return ltl_fail(LTL_ERR_ARG, "decode_chain: phase %d: the normalising load needs a gain and K <= 2048", i);
        if (q.a_kind == A_EMBED && (!d.tok || !d.x)) return ltl_fail(LTL_ERR_NULL, "decode_chain: the gathering load needs ids and the stream");
        ph.a_kind = q.a_kind; ph.epi = q.epi; ph.N = q.N; ph.K = q.K; ph.a = q.a; ph.gain = q.gain; ph.b = (const bf16*)q.b; ph.out = q.out;
        ph.tile = pick_tile(d.M, q.K);
        int bm, bn;
        tile_dims(ph.tile, bm, bn);
        if ((size_t)bm * (q.K + CH_PAD) * 2 > (size_t)CH_A_BYTES || (size_t)bn * (q.K + CH_PAD) * 2 > (size_t)CH_B_BYTES)
            return ltl_fail(LTL_ERR_UNSUPPORTED, "decode_chain: phase %d: K = %d does not fit the panels", i, q.K);
        const int tiles = ((d.M + bm - 1) / bm) * ((q.N + bn - 1) / bn);
        if (tiles > most) most = tiles;
    }
    const int grid = most < grid_max ? most : grid_max;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid); cfg.blockDim = dim3(CH_THREADS); cfg.dynamicSmemBytes = CH_A_BYTES + CH_B_BYTES; cfg.stream = s;
    cudaLaunchAttribute at[2];
    at[0].id = cudaLaunchAttributeCooperative;
    at[0].val.cooperative = 1;
    at[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    cfg.numAttrs = (ltl_pdl_enabled() && d.allow_pdl) ? 2 : 1;
    LTL_CUDA("decode_chain launch", cudaLaunchKernelEx(&cfg, decode_chain_kernel, P));
    return ltl_check_launch("decode_chain");
}
