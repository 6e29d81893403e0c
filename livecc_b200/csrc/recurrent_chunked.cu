// Sequence-parallel form of the gated linear recurrence for prompt portions:
//     St <- diag(a_t) St + k_t (sc_t u_t)^T ,  y_t = St^T (cs c_t) + skip * u_t          (St: N x P per head, fp32)
// The rows of a call are cut into blocks of CL = 64 tokens (counted from row 0 of the call; the carried state enters
// block 0). With b_t = sum of log a over the rows of the block up to and including t:
//     y_t   = sum_n cs c_t[n] exp(b_t[n]) S_in[n, :]  +  sum_{s <= t} M[t, s] u_s  + skip u_t
//     M[t,s]= cs sc_s sum_n c_t[n] k_s[n] exp(b_t[n] - b_s[n])                       (every exponent is <= 0)
//     S_out = diag(exp(b_last)) S_in + sum_s (k_s * exp(b_last - b_s)) (sc_s u_s)^T
// Five launches: block-local cumulative log decays, M, the blocks' own state contributions, a short sequential pass
// over blocks that turns them into the state entering each block, and the outputs. All arithmetic is fp32 on the
// CUDA cores (the recurrence's operands are fp32 by the models' precision rules); the three products are register-
// tiled 64 x 64 tiles whose operands are formed (decay factors applied) while they are staged into shared memory.
#include <math.h>

#include <algorithm>

#include "common.cuh"
#include "launch.h"
#include "seqmix.h"

namespace lcc {
namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }

__device__ __forceinline__ bool seq_done(const SeqPos& p) { return p.finished && *p.finished; }

constexpr int CL = 64;          // tokens per block
constexpr int TS = 64;          // output tile edge
constexpr int KS = 16;          // depth of a staged operand slice
constexpr int PAD = TS + 4;

struct Tile {
    float a[KS][PAD];
    float b[KS][PAD];
};

// Stage one KS-deep slice of both operands: fa(r, kk) / fb(r, kk) give element (tile row or column r, depth kk) or 0
// outside the problem. KC: consecutive threads walk the depth index (operands contiguous along it), else the row index.
template <bool KC_A, bool KC_B, typename FA, typename FB>
__device__ __forceinline__ void stage(Tile& sh, FA fa, FB fb) {
#pragma unroll
    for (int i = 0; i < TS * KS / 256; ++i) {
        const int e = threadIdx.x + i * 256;
        { const int r = KC_A ? e / KS : e % TS, kk = KC_A ? e % KS : e / TS; sh.a[kk][r] = fa(r, kk); }
        { const int r = KC_B ? e / KS : e % TS, kk = KC_B ? e % KS : e / TS; sh.b[kk][r] = fb(r, kk); }
    }
}

__device__ __forceinline__ void fma_slice(const Tile& sh, int tm, int tn, float (&acc)[4][4]) {
#pragma unroll
    for (int kk = 0; kk < KS; ++kk) {
        const float4 av = *reinterpret_cast<const float4*>(&sh.a[kk][tm]);
        const float4 bv = *reinterpret_cast<const float4*>(&sh.b[kk][tn]);
        const float a[4] = {av.x, av.y, av.z, av.w}, b[4] = {bv.x, bv.y, bv.z, bv.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
}

struct ChunkArgs {
    const void* k; int ld_k;
    const void* c; int ld_c;
    const void* u; int ld_u;
    float* la;                 // [S, heads * NV] log decays, replaced by their block-local cumulative sums
    const float* sc;           // [S, heads] or null
    const float* skip;         // [heads] or null
    float cs;
    float* state;              // [heads, P, N]
    float* y; int ld_y;
    float* ws_m;               // [blocks, heads, CL, CL]
    float* ws_s;               // [blocks, heads, P, N]
    int row0;                  // first row of this pass
    int S;                     // rows of this pass
    int heads, heads_per_group, N, P, NV;   // NV = N (a decay per key channel) or 1 (a decay per head)
};

// ---- 1: block-local cumulative sums of the log decays ---------------------------------------------------------------
__global__ void chunk_cumsum_kernel(ChunkArgs a, SeqPos pos) {
    if (seq_done(pos)) return;
    const int col = blockIdx.y * blockDim.x + threadIdx.x, ncol = a.heads * a.NV;
    if (col >= ncol) return;
    const int t0 = blockIdx.x * CL, len = min(CL, a.S - t0);
    float* p = a.la + (size_t)(a.row0 + t0) * ncol + col;
    float acc = 0.f;
    for (int tb = 0; tb < len; tb += 16) {     // 16 independent loads in flight, then the running sum in row order
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = tb + i < len ? p[(size_t)(tb + i) * ncol] : 0.f;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            acc += v[i];
            if (tb + i < len) p[(size_t)(tb + i) * ncol] = acc;
        }
    }
}

// ---- 2: M[t, s] -------------------------------------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) chunk_weights_kernel(ChunkArgs a, SeqPos pos) {
    if (seq_done(pos)) return;
    __shared__ float sc_[KS][PAD], sk_[KS][PAD], sb_[KS][PAD];
    // a decay per head: the product c k^T is the same for every head of a group, so a CTA forms it once per group and
    // writes one decayed copy per head; a decay per key channel: one CTA per head
    const int blk = blockIdx.x, g = VEC ? blockIdx.y / a.heads_per_group : blockIdx.y;
    const int h_first = VEC ? blockIdx.y : g * a.heads_per_group, h_count = VEC ? 1 : a.heads_per_group;
    const int h = h_first;
    const int t0 = blk * CL, len = min(CL, a.S - t0);
    const int N = a.N, ncol = a.heads * a.NV;
    const int ty = threadIdx.x / 16, tx = threadIdx.x % 16, tm = ty * 4, tn = tx * 4;
    const T* gc = (const T*)a.c + (size_t)(a.row0 + t0) * a.ld_c + (size_t)g * N;
    const T* gk = (const T*)a.k + (size_t)(a.row0 + t0) * a.ld_k + (size_t)g * N;
    const float* gb = a.la + (size_t)(a.row0 + t0) * ncol + (size_t)h * a.NV;
    const bool live = tn <= tm + 3;            // tiles wholly above the diagonal stay zero
    float acc[4][4] = {};
    for (int n0 = 0; n0 < N; n0 += KS) {
        __syncthreads();
#pragma unroll
        for (int i = 0; i < CL * KS / 256; ++i) {
            const int e = threadIdx.x + i * 256, r = e / KS, kk = e % KS, n = n0 + kk;
            const bool ok = r < len && n < N;
            sc_[kk][r] = ok ? ldf(gc + (size_t)r * a.ld_c + n) : 0.f;
            sk_[kk][r] = ok ? ldf(gk + (size_t)r * a.ld_k + n) : 0.f;
            if (VEC) sb_[kk][r] = ok ? gb[(size_t)r * ncol + n] : 0.f;
        }
        __syncthreads();
        if (!live) continue;
#pragma unroll 4
        for (int kk = 0; kk < KS; ++kk) {
            float cv[4], kv[4], bt[4], bs[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { cv[i] = sc_[kk][tm + i]; kv[i] = sk_[kk][tn + i]; }
            if (VEC) {
#pragma unroll
                for (int i = 0; i < 4; ++i) { bt[i] = sb_[kk][tm + i]; bs[i] = sb_[kk][tn + i]; }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (VEC) acc[i][j] = fmaf(cv[i] * kv[j], expf(fminf(bt[i] - bs[j], 0.f)), acc[i][j]);
                    else acc[i][j] = fmaf(cv[i], kv[j], acc[i][j]);
                }
        }
    }
    for (int hh = h_first; hh < h_first + h_count; ++hh) {
        float* out = a.ws_m + ((size_t)blk * a.heads + hh) * CL * CL;
        const float* hb = a.la + (size_t)(a.row0 + t0) * ncol + (size_t)hh * a.NV;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int t = tm + i;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int s = tn + j;
                float v = 0.f;
                if (s <= t && t < len) {
                    v = acc[i][j] * a.cs * (a.sc ? a.sc[(size_t)(a.row0 + t0 + s) * a.heads + hh] : 1.f);
                    if (!VEC) v *= expf(fminf(hb[(size_t)t * ncol] - hb[(size_t)s * ncol], 0.f));
                }
                out[t * CL + s] = v;
            }
        }
    }
}

// ---- 3: a block's own contribution to the state, stored [p][n] ----------------------------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) chunk_state_kernel(ChunkArgs a, SeqPos pos) {
    if (seq_done(pos)) return;
    __shared__ Tile sh;
    const int blk = blockIdx.x / a.heads, h = blockIdx.x % a.heads, g = h / a.heads_per_group;
    const int p0 = blockIdx.y * TS, n0 = blockIdx.z * TS;
    const int t0 = blk * CL, len = min(CL, a.S - t0);
    const int N = a.N, P = a.P, ncol = a.heads * a.NV;
    const T* gu = (const T*)a.u + (size_t)(a.row0 + t0) * a.ld_u + (size_t)h * P;
    const T* gk = (const T*)a.k + (size_t)(a.row0 + t0) * a.ld_k + (size_t)g * N;
    const float* gb = a.la + (size_t)(a.row0 + t0) * ncol + (size_t)h * a.NV;
    const float* gsc = a.sc ? a.sc + (size_t)(a.row0 + t0) * a.heads + h : nullptr;
    const float* blast = gb + (size_t)(len - 1) * ncol;
    const int tm = (threadIdx.x / 16) * 4, tn = (threadIdx.x % 16) * 4;
    __shared__ float rowf[CL];     // per row: the step scale, and in the per-head case the decay from the row to the block's end
    if (threadIdx.x < CL) {
        const int s = threadIdx.x;
        float f = 0.f;
        if (s < len) {
            f = gsc ? gsc[(size_t)s * a.heads] : 1.f;
            if (!VEC) f *= expf(fminf(blast[0] - gb[(size_t)s * ncol], 0.f));
        }
        rowf[s] = f;
    }
    float acc[4][4] = {};
    for (int s0 = 0; s0 < len; s0 += KS) {
        __syncthreads();
        stage<false, false>(sh,
            [&](int r, int kk) { const int s = s0 + kk, p = p0 + r;
                                 return (s < len && p < P) ? ldf(gu + (size_t)s * a.ld_u + p) * rowf[s] : 0.f; },
            [&](int r, int kk) { const int s = s0 + kk, n = n0 + r;
                                 if (s >= len || n >= N) return 0.f;
                                 const float kv = ldf(gk + (size_t)s * a.ld_k + n);
                                 return VEC ? kv * expf(fminf(blast[n] - gb[(size_t)s * ncol + n], 0.f)) : kv; });
        __syncthreads();
        fma_slice(sh, tm, tn, acc);
    }
    float* out = a.ws_s + ((size_t)blk * a.heads + h) * P * N;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int p = p0 + tm + i;
        if (p >= P) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tn + j;
            if (n < N) out[(size_t)p * N + n] = acc[i][j];
        }
    }
}

// ---- 4: contributions -> the state that enters each block; the state after the last block goes back to the slot -----
template <bool VEC>
__global__ void chunk_prefix_kernel(ChunkArgs a, int nblocks, SeqPos pos) {
    if (seq_done(pos)) return;
    const size_t per = (size_t)a.heads * a.P * a.N;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= per) return;
    const int n = (int)(idx % a.N), h = (int)(idx / ((size_t)a.P * a.N));
    const int ncol = a.heads * a.NV;
    float st = a.state[idx];
    for (int b0 = 0; b0 < nblocks; b0 += 8) {  // 8 blocks' loads in flight together; the chain over blocks runs in registers
        float d[8], e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int b = b0 + i;
            if (b < nblocks) {
                const int tlast = min((b + 1) * CL, a.S) - 1;
                d[i] = a.ws_s[(size_t)b * per + idx];
                e[i] = a.la[(size_t)(a.row0 + tlast) * ncol + (size_t)h * a.NV + (VEC ? n : 0)];
            }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int b = b0 + i;
            if (b < nblocks) {
                a.ws_s[(size_t)b * per + idx] = st;
                st = fmaf(expf(e[i]), st, d[i]);
            }
        }
    }
    a.state[idx] = st;
}

// ---- 5: outputs ---------------------------------------------------------------------------------------------------------
template <typename T, bool VEC>
__global__ void __launch_bounds__(256) chunk_output_kernel(ChunkArgs a, SeqPos pos) {
    if (seq_done(pos)) return;
    __shared__ Tile sh;
    const int blk = blockIdx.x / a.heads, h = blockIdx.x % a.heads, g = h / a.heads_per_group;
    const int p0 = blockIdx.y * TS;
    const int t0 = blk * CL, len = min(CL, a.S - t0);
    const int N = a.N, P = a.P, ncol = a.heads * a.NV;
    const T* gu = (const T*)a.u + (size_t)(a.row0 + t0) * a.ld_u + (size_t)h * P;
    const T* gc = (const T*)a.c + (size_t)(a.row0 + t0) * a.ld_c + (size_t)g * N;
    const float* gb = a.la + (size_t)(a.row0 + t0) * ncol + (size_t)h * a.NV;
    const float* sin = a.ws_s + ((size_t)blk * a.heads + h) * P * N;
    const float* gm = a.ws_m + ((size_t)blk * a.heads + h) * CL * CL;
    const int tm = (threadIdx.x / 16) * 4, tn = (threadIdx.x % 16) * 4;
    float acc[4][4] = {};
    for (int n0 = 0; n0 < N; n0 += KS) {       // the entering state, seen through the decayed queries
        __syncthreads();
        stage<true, true>(sh,
            [&](int r, int kk) { const int n = n0 + kk;
                                 if (r >= len || n >= N) return 0.f;
                                 return a.cs * ldf(gc + (size_t)r * a.ld_c + n) * expf(gb[(size_t)r * ncol + (VEC ? n : 0)]); },
            [&](int r, int kk) { const int n = n0 + kk, p = p0 + r;
                                 return (n < N && p < P) ? sin[(size_t)p * N + n] : 0.f; });
        __syncthreads();
        fma_slice(sh, tm, tn, acc);
    }
    for (int s0 = 0; s0 < len; s0 += KS) {     // the block's own rows
        __syncthreads();
        stage<true, false>(sh,
            [&](int r, int kk) { const int s = s0 + kk; return s < len ? gm[r * CL + s] : 0.f; },
            [&](int r, int kk) { const int s = s0 + kk, p = p0 + r;
                                 return (s < len && p < P) ? ldf(gu + (size_t)s * a.ld_u + p) : 0.f; });
        __syncthreads();
        fma_slice(sh, tm, tn, acc);
    }
    const float skip = a.skip ? a.skip[h] : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int t = tm + i;
        if (t >= len) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int p = p0 + tn + j;
            if (p < P) a.y[(size_t)(a.row0 + t0 + t) * a.ld_y + (size_t)h * P + p] = acc[i][j] + skip * ldf(gu + (size_t)t * a.ld_u + p);
        }
    }
}

template <typename T, bool VEC>
int run_chunked(const ScanArgs& s, SeqPos pos, cudaStream_t st) {
    const size_t per_block = (size_t)s.heads * ((size_t)CL * CL + (size_t)s.P * s.N);
    const int max_blocks = (int)std::min<size_t>(s.ws_floats / per_block, 1 << 20);
    if (max_blocks < 1) return -3;
    ChunkArgs a{};
    a.k = s.k; a.ld_k = s.ld_k; a.c = s.c; a.ld_c = s.ld_c; a.u = s.u; a.ld_u = s.ld_u;
    a.la = s.a; a.sc = s.sc; a.skip = s.skip; a.cs = s.cs; a.state = s.state; a.y = s.y; a.ld_y = s.ld_y;
    a.heads = s.heads; a.heads_per_group = s.heads_per_group; a.N = s.N; a.P = s.P; a.NV = VEC ? s.N : 1;
    const size_t per_state = (size_t)s.heads * s.P * s.N;
    for (int row0 = 0; row0 < s.S; row0 += max_blocks * CL) {
        const int rows = std::min(s.S - row0, max_blocks * CL), nb = (rows + CL - 1) / CL;
        a.row0 = row0; a.S = rows;
        a.ws_m = s.ws; a.ws_s = s.ws + (size_t)nb * s.heads * CL * CL;
        const int ncol = a.heads * a.NV;
        count_launch();
        chunk_cumsum_kernel<<<dim3(nb, (ncol + 127) / 128), 128, 0, st>>>(a, pos);
        count_launch();
        chunk_weights_kernel<T, VEC><<<dim3(nb, VEC ? s.heads : s.heads / s.heads_per_group), 256, 0, st>>>(a, pos);
        count_launch();
        chunk_state_kernel<T, VEC><<<dim3(nb * s.heads, (s.P + TS - 1) / TS, (s.N + TS - 1) / TS), 256, 0, st>>>(a, pos);
        count_launch();
        chunk_prefix_kernel<VEC><<<(unsigned)((per_state + 255) / 256), 256, 0, st>>>(a, nb, pos);
        count_launch();
        chunk_output_kernel<T, VEC><<<dim3(nb * s.heads, (s.P + TS - 1) / TS), 256, 0, st>>>(a, pos);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

}  // namespace

size_t gated_scan_ws_floats(int S, int heads, int N, int P) {
    const size_t nb = std::min<size_t>(((size_t)(S > 0 ? S : 1) + CL - 1) / CL, kScanMaxBlocks);
    return nb * (size_t)heads * ((size_t)CL * CL + (size_t)P * N);
}

int gated_scan_chunked(const ScanArgs& a, SeqPos pos, cudaStream_t s) {
    if (!a.ws) return -2;
    if (a.dt == DT_F32) return a.vec_decay ? run_chunked<float, true>(a, pos, s) : run_chunked<float, false>(a, pos, s);
    return a.vec_decay ? run_chunked<bf16, true>(a, pos, s) : run_chunked<bf16, false>(a, pos, s);
}

}  // namespace lcc
