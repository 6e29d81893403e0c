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

constexpr int kMaxStreams = 8;

// One CTA per row; a thread owns columns threadIdx.x, +256, ... of every stream. Rows of up to 256 * E columns keep the
// read value u in registers between the sum of squares and the store (E = 0: recomputed from the streams just written,
// by the thread that wrote them). Sums run over the streams in ascending order, so a row's result does not depend on the batch.
template <typename T, int N, int E>
__global__ void __launch_bounds__(256) hyper_boundary_kernel(float* __restrict__ xs, int n_rt, const T* __restrict__ y, int ld_y,
                                                             const float* __restrict__ prev, const float* __restrict__ next,
                                                             const float* __restrict__ w, float eps, T* __restrict__ xa,
                                                             float* __restrict__ sum_out, int W) {
    __shared__ float red[32];
    const int n = N > 0 ? N : n_rt;
    const int r = blockIdx.x;
    float* x = xs + (size_t)r * n * W;
    float mix[kMaxStreams * kMaxStreams], ov[kMaxStreams], in[kMaxStreams];
    for (int i = 0; i < n; ++i) {
        ov[i] = y ? prev[n + i] : 0.f;
        in[i] = next ? next[i] : 0.f;
        for (int j = 0; j < n; ++j) mix[i * n + j] = y ? prev[2 * n + i * n + j] : 0.f;
    }
    constexpr int EN = E > 0 ? E : 1;
    float uc[EN];
    float ss = 0.f;
    int e = 0;
    for (int c = threadIdx.x; c < W; c += 256, ++e) {
        float old[kMaxStreams], nw[kMaxStreams];
        for (int i = 0; i < n; ++i) old[i] = x[(size_t)i * W + c];
        if (y) {
            const float yv = ldf(y + (size_t)r * ld_y + c);
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
            if (E > 0) uc[e < EN ? e : 0] = u;
        }
    }
    if (!w) return;
    ss = block_sum(ss, red);
    const float rn = 1.f / sqrtf(ss / (float)W + eps);
    e = 0;
    for (int c = threadIdx.x; c < W; c += 256, ++e) {
        float u;
        if (E > 0) {
            u = uc[e < EN ? e : 0];
        } else {
            u = 0.f;
            for (int i = 0; i < n; ++i) u = fmaf(in[i], x[(size_t)i * W + c], u);
        }
        stf(xa + (size_t)r * W + c, u * rn * w[c]);
    }
}

}  // namespace

int hyper_boundary(int dt, float* xs, int n, const void* y, int ld_y, const float* prev, const float* next, const float* w,
                   float eps, void* xa, float* sum_out, int S, int W, cudaStream_t s) {
    if (!xs || n < 1 || n > kMaxStreams || S < 1 || W < 1 || (y && !prev) || (w && (!next || !xa))) return -2;
    if (!y && !w && !sum_out) return 0;
    count_launch();
    const int per = (W + 255) / 256;
#define LCC_HB(N, E)                                                                                                       \
    do {                                                                                                                   \
        if (dt == DT_F32)                                                                                                  \
            hyper_boundary_kernel<float, N, E><<<S, 256, 0, s>>>(xs, n, (const float*)y, ld_y, prev, next, w, eps, (float*)xa, sum_out, W); \
        else                                                                                                               \
            hyper_boundary_kernel<bf16, N, E><<<S, 256, 0, s>>>(xs, n, (const bf16*)y, ld_y, prev, next, w, eps, (bf16*)xa, sum_out, W); \
    } while (0)
#define LCC_HB_E(N)                                                                                                        \
    do {                                                                                                                   \
        if (per <= 4) LCC_HB(N, 4); else if (per <= 16) LCC_HB(N, 16); else LCC_HB(N, 0);                                   \
    } while (0)
    // the unrolled stream count changes neither the order of a sum nor its operands
    if (n == 1) LCC_HB_E(1);
    else if (n == 2) LCC_HB_E(2);
    else if (n == 4) LCC_HB_E(4);
    else LCC_HB_E(0);
#undef LCC_HB_E
#undef LCC_HB
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

}  // namespace lcc
