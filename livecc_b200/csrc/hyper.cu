// Pre-norm residual blocks on several residual streams (hyper-connections). Between two sublayers one kernel does what
// three row passes would: the write of the finished sublayer (x_t <- sum_s mix[s][t] x_s + out[t] y), the read of the
// next one (u = sum_s in[s] x_s) and its RMS norm. Streams, sums and norms are fp32; y and the normed row are in the
// model's storage type.
#include <math.h>

#include "common.cuh"
#include "launch.h"
#include "seqmix.h"

namespace lcc {
namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void stf(T* p, float v);
template <> __device__ __forceinline__ void stf<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void stf<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

constexpr int kMaxStreams = 8, kMaxTop = 8;

// Where the finished sublayer's output row comes from: a plain row y, or (a routed feed-forward) the weighted sum of the
// chosen experts' rows plus the gated shared expert's row, formed here instead of in a kernel of its own.
template <typename T>
struct YSource {
    const T* y; int ld_y;
    const T* eo; int ld_eo; const int* pos; const float* weight; int top;
    const T* so; int ld_so; const float* gate;
};

template <typename T>
__device__ __forceinline__ float y_value(const YSource<T>& s, int r, int c) {
    if (s.y) return ldf(s.y + (size_t)r * s.ld_y + c);
    float acc = 0.f;
    for (int k = 0; k < s.top; ++k)
        acc = fmaf(s.weight[(size_t)r * s.top + k], ldf(s.eo + (size_t)s.pos[(size_t)r * s.top + k] * s.ld_eo + c), acc);
    if (s.so) acc = fmaf(s.gate[r], ldf(s.so + (size_t)r * s.ld_so + c), acc);
    return acc;
}

// One CTA per row; a thread owns columns threadIdx.x, +256, ... of every stream. Rows of up to 256 * E columns (E > 0, with
// N > 0 streams known at compile time) are loaded whole before anything is computed, so that all of a thread's loads are in
// flight together; other shapes walk the columns one by one. Sums run over the streams in ascending order in both forms,
// so a row's result does not depend on the form or the batch.
template <typename T, int N, int E>
__global__ void __launch_bounds__(256) hyper_boundary_kernel(float* __restrict__ xs, int n_rt, YSource<T> src,
                                                             const float* __restrict__ prev, const float* __restrict__ next,
                                                             const float* __restrict__ w, float eps, T* __restrict__ xa,
                                                             float* __restrict__ sum_out, int W) {
    __shared__ float red[32];
    constexpr bool FAST = N > 0 && E > 0;
    const int n = N > 0 ? N : n_rt;
    const int r = blockIdx.x;
    const bool has_y = src.y || src.eo;
    float* x = xs + (size_t)r * n * W;
    float mix[kMaxStreams * kMaxStreams], ov[kMaxStreams], in[kMaxStreams];
    for (int i = 0; i < n; ++i) {
        ov[i] = has_y ? prev[n + i] : 0.f;
        in[i] = next ? next[i] : 0.f;
        for (int j = 0; j < n; ++j) mix[i * n + j] = has_y ? prev[2 * n + i * n + j] : 0.f;
    }
    float ss = 0.f;
    if (FAST) {
        constexpr int NN = N > 0 ? N : 1, EE = E > 0 ? E : 1;
        float xv[NN][EE], yv[EE], u[EE];
        // the routed rows: positions and weights once per row
        int pk[kMaxTop];
        float wk[kMaxTop];
        const bool routed = !src.y && src.eo;
        const float gs = (routed && src.so) ? src.gate[r] : 0.f;
        if (routed) {
#pragma unroll
            for (int k = 0; k < kMaxTop; ++k) {
                pk[k] = k < src.top ? src.pos[(size_t)r * src.top + k] : 0;
                wk[k] = k < src.top ? src.weight[(size_t)r * src.top + k] : 0.f;
            }
        }
#pragma unroll
        for (int e = 0; e < EE; ++e) {
            const int c = threadIdx.x + e * 256;
            const bool ok = c < W;
#pragma unroll
            for (int i = 0; i < NN; ++i) xv[i][e] = ok ? x[(size_t)i * W + c] : 0.f;
            yv[e] = 0.f;
            if (ok && src.y) yv[e] = ldf(src.y + (size_t)r * src.ld_y + c);
        }
        if (routed) {
#pragma unroll
            for (int k = 0; k < kMaxTop; ++k) {
                if (k < src.top) {
#pragma unroll
                    for (int e = 0; e < EE; ++e) {
                        const int c = threadIdx.x + e * 256;
                        if (c < W) yv[e] = fmaf(wk[k], ldf(src.eo + (size_t)pk[k] * src.ld_eo + c), yv[e]);
                    }
                }
            }
            if (src.so) {
#pragma unroll
                for (int e = 0; e < EE; ++e) {
                    const int c = threadIdx.x + e * 256;
                    if (c < W) yv[e] = fmaf(gs, ldf(src.so + (size_t)r * src.ld_so + c), yv[e]);
                }
            }
        }
#pragma unroll
        for (int e = 0; e < EE; ++e) {
            const int c = threadIdx.x + e * 256;
            if (c >= W) { u[e] = 0.f; continue; }
            float nw[NN];
            if (has_y) {
#pragma unroll
                for (int t = 0; t < NN; ++t) {
                    float acc = 0.f;
#pragma unroll
                    for (int i = 0; i < NN; ++i) acc = fmaf(mix[i * NN + t], xv[i][e], acc);
                    nw[t] = fmaf(ov[t], yv[e], acc);
                    x[(size_t)t * W + c] = nw[t];
                }
            } else {
#pragma unroll
                for (int i = 0; i < NN; ++i) nw[i] = xv[i][e];
            }
            if (sum_out) {
                float sm = 0.f;
#pragma unroll
                for (int i = 0; i < NN; ++i) sm += nw[i];
                sum_out[(size_t)r * W + c] = sm;
            }
            float uu = 0.f;
#pragma unroll
            for (int i = 0; i < NN; ++i) uu = fmaf(in[i], nw[i], uu);
            u[e] = uu;
            ss = fmaf(uu, uu, ss);
        }
        if (!w) return;
        ss = block_sum(ss, red);
        const float rn = 1.f / sqrtf(ss / (float)W + eps);
#pragma unroll
        for (int e = 0; e < EE; ++e) {
            const int c = threadIdx.x + e * 256;
            if (c < W) stf(xa + (size_t)r * W + c, u[e] * rn * w[c]);
        }
        return;
    }
    // the general form: any stream count, any width, top above kMaxTop
    for (int c = threadIdx.x; c < W; c += 256) {
        float old[kMaxStreams], nw[kMaxStreams];
        for (int i = 0; i < n; ++i) old[i] = x[(size_t)i * W + c];
        if (has_y) {
            const float yv = y_value(src, r, c);
            for (int t = 0; t < n; ++t) {
                float acc = 0.f;
                for (int i = 0; i < n; ++i) acc = fmaf(mix[i * n + t], old[i], acc);
                nw[t] = fmaf(ov[t], yv, acc);
                x[(size_t)t * W + c] = nw[t];
            }
        } else {
            for (int i = 0; i < n; ++i) nw[i] = old[i];
        }
        if (sum_out) {
            float sm = 0.f;
            for (int i = 0; i < n; ++i) sm += nw[i];
            sum_out[(size_t)r * W + c] = sm;
        }
        if (w) {
            float u = 0.f;
            for (int i = 0; i < n; ++i) u = fmaf(in[i], nw[i], u);
            ss = fmaf(u, u, ss);
        }
    }
    if (!w) return;
    ss = block_sum(ss, red);
    const float rn = 1.f / sqrtf(ss / (float)W + eps);
    for (int c = threadIdx.x; c < W; c += 256) {
        float u = 0.f;
        for (int i = 0; i < n; ++i) u = fmaf(in[i], x[(size_t)i * W + c], u);   // the streams this thread has just written
        stf(xa + (size_t)r * W + c, u * rn * w[c]);
    }
}

template <typename T>
int launch_boundary(float* xs, int n, const YSource<T>& src, const float* prev, const float* next, const float* w, float eps,
                    void* xa, float* sum_out, int S, int W, cudaStream_t s) {
    const int per = (W + 255) / 256;
    const bool top_ok = src.y || !src.eo || src.top <= kMaxTop;
    count_launch();
#define LCC_HB(N, E) hyper_boundary_kernel<T, N, E><<<S, 256, 0, s>>>(xs, n, src, prev, next, w, eps, (T*)xa, sum_out, W)
#define LCC_HB_E(N)                                                                                                        \
    do {                                                                                                                   \
        if (per <= 4 && top_ok) LCC_HB(N, 4); else if (per <= 8 && top_ok) LCC_HB(N, 8); else if (per <= 16 && top_ok) LCC_HB(N, 16); else LCC_HB(0, 0); \
    } while (0)
    if (n == 1) LCC_HB_E(1);
    else if (n == 2) LCC_HB_E(2);
    else if (n == 4) LCC_HB_E(4);
    else LCC_HB(0, 0);
#undef LCC_HB_E
#undef LCC_HB
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

}  // namespace

int hyper_boundary(int dt, float* xs, int n, const void* y, int ld_y, const float* prev, const float* next, const float* w,
                   float eps, void* xa, float* sum_out, int S, int W, cudaStream_t s, const MoeCombine* mc) {
    const bool has_y = y || mc;
    if (!xs || n < 1 || n > kMaxStreams || S < 1 || W < 1 || (has_y && !prev) || (w && (!next || !xa)) || (y && mc)) return -2;
    if (mc && (!mc->eo || !mc->pos || !mc->weight || mc->top < 1 || (mc->so && !mc->gate))) return -2;
    if (!has_y && !w && !sum_out) return 0;
    if (dt == DT_F32) {
        YSource<float> src{(const float*)y, ld_y, nullptr, 0, nullptr, nullptr, 0, nullptr, 0, nullptr};
        if (mc) src = YSource<float>{nullptr, 0, (const float*)mc->eo, mc->ld_eo, mc->pos, mc->weight, mc->top, (const float*)mc->so, mc->ld_so, mc->gate};
        return launch_boundary<float>(xs, n, src, prev, next, w, eps, xa, sum_out, S, W, s);
    }
    YSource<bf16> src{(const bf16*)y, ld_y, nullptr, 0, nullptr, nullptr, 0, nullptr, 0, nullptr};
    if (mc) src = YSource<bf16>{nullptr, 0, (const bf16*)mc->eo, mc->ld_eo, mc->pos, mc->weight, mc->top, (const bf16*)mc->so, mc->ld_so, mc->gate};
    return launch_boundary<bf16>(xs, n, src, prev, next, w, eps, xa, sum_out, S, W, s);
}

}  // namespace lcc
