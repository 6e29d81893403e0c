// General-shape linear layers: C[M,N] = A[M,K] x W[N,K]^T (+ bias), fp32 accumulation, bf16 or fp32 storage.
// Two CUDA-core kernels cover every shape the tensor-core GEMM (gemm_tcgen05.cu) does not take: ragged N or K, fp32
// storage (true fp32 FMAs, no reduced-precision matrix mode), and the few-row case of a decode step, where the
// weight matrix is streamed once and every row of A is multiplied against it (HBM-bound).
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

constexpr int BM = 64, BN = 64, BK = 16;

// 64 x 64 output tile per CTA, 256 threads x (4 x 4) accumulators, k-slices of 16 staged in shared memory as fp32.
template <typename T, typename TC>
__global__ void __launch_bounds__(256) linear_tile_kernel(const T* __restrict__ A, int lda, const T* __restrict__ W, int ldw,
                                                          const float* __restrict__ bias, TC* __restrict__ C, int ldc, int M,
                                                          int N, int K) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += BK) {
        // 64 rows x 16 k per operand = 1024 elements, 4 per thread; consecutive threads read consecutive k (coalesced)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int e = tid + i * 256, r = e / BK, k = e % BK;
            const int gm = m0 + r, gn = n0 + r, gk = k0 + k;
            As[k][r] = (gm < M && gk < K) ? ldf(A + (size_t)gm * lda + gk) : 0.f;
            Ws[k][r] = (gn < N && gk < K) ? ldf(W + (size_t)gn * ldw + gk) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < BK; ++k) {
            float a[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = As[k][tm + i]; w[i] = Ws[k][tn + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int gm = m0 + tm + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tn + j;
            if (gn < N) stf(C + (size_t)gm * ldc + gn, acc[i][j] + (bias ? bias[gn] : 0.f));
        }
    }
}

// Few rows (M <= 8), the shape of a decode step: the weight matrix is streamed once (HBM-bound). A warp owns WR output
// columns (2 for wide matrices; 1, in CTAs of 2 warps, when N is small, so that every SM still has enough loads in
// flight) and keeps WR x WU independent 16-byte non-allocating loads of their weight rows in flight per lane before it
// touches the activations (which stay in L1); lanes stride over k and keep one accumulator per (column, row of A), so
// the order of a column's sum does not depend on WR or M. Scalar loads when K or a row start is not 16-byte aligned.
constexpr int kRowsMax = 8;
constexpr int WU = 4;
template <typename T> struct Vec16;
template <> struct Vec16<bf16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void unpack(const uint4& u, float (&v)[8]) {
        const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
    }
};
template <> struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void unpack(const uint4& u, float (&v)[4]) {
        v[0] = __uint_as_float(u.x); v[1] = __uint_as_float(u.y); v[2] = __uint_as_float(u.z); v[3] = __uint_as_float(u.w);
    }
};

template <typename T, typename TC, bool VEC, int WR>
__global__ void __launch_bounds__(256) linear_rows_kernel(const T* __restrict__ A, int lda, const T* __restrict__ W, int ldw,
                                                          const float* __restrict__ bias, TC* __restrict__ C, int ldc, int M,
                                                          int N, int K) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = (blockIdx.x * (blockDim.x >> 5) + warp) * WR;
    if (n0 >= N) return;
    float acc[WR][kRowsMax];
#pragma unroll
    for (int r = 0; r < WR; ++r)
#pragma unroll
        for (int m = 0; m < kRowsMax; ++m) acc[r][m] = 0.f;
    if (VEC) {
        constexpr int V = Vec16<T>::N;
        const T* w[WR];
#pragma unroll
        for (int r = 0; r < WR; ++r) w[r] = W + (size_t)min(n0 + r, N - 1) * ldw;
        for (int kb = lane * V; kb < K; kb += 32 * V * WU) {
            uint4 wq[WR][WU];
#pragma unroll
            for (int r = 0; r < WR; ++r)
#pragma unroll
                for (int u = 0; u < WU; ++u) {
                    const int k = kb + u * 32 * V;
                    wq[r][u] = k < K ? ld_stream16(w[r] + k) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
            for (int u = 0; u < WU; ++u) {
                const int k = min(kb + u * 32 * V, K - V);      // past the end the weights are zero; keep the address valid
                float wv[WR][V];
#pragma unroll
                for (int r = 0; r < WR; ++r) Vec16<T>::unpack(wq[r][u], wv[r]);
#pragma unroll
                for (int m = 0; m < kRowsMax; ++m) {
                    if (m < M) {
                        float av[V];
                        Vec16<T>::unpack(__ldg(reinterpret_cast<const uint4*>(A + (size_t)m * lda + k)), av);
#pragma unroll
                        for (int r = 0; r < WR; ++r)
#pragma unroll
                            for (int i = 0; i < V; ++i) acc[r][m] = fmaf(av[i], wv[r][i], acc[r][m]);
                    }
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
#pragma unroll
            for (int r = 0; r < WR; ++r) {
                const float wv = ldf(W + (size_t)min(n0 + r, N - 1) * ldw + k);
#pragma unroll
                for (int m = 0; m < kRowsMax; ++m)
                    if (m < M) acc[r][m] = fmaf(ldf(A + (size_t)m * lda + k), wv, acc[r][m]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < WR; ++r) {
        const int n = n0 + r;
#pragma unroll
        for (int m = 0; m < kRowsMax; ++m) {
            if (m < M) {
                const float v = warp_sum(acc[r][m]);
                if (lane == 0 && n < N) stf(C + (size_t)m * ldc + n, v + (bias ? bias[n] : 0.f));
            }
        }
    }
}

template <typename T, typename TC>
int launch_linear(const void* A, int lda, const void* W, int ldw, const float* bias, void* C, int ldc, int M, int N, int K,
                  cudaStream_t s) {
    if (M <= kRowsMax) {
        constexpr int V = Vec16<T>::N;
        const bool vec = (K % V) == 0 && (lda % V) == 0 && (ldw % V) == 0 && ((uintptr_t)A % 16) == 0 && ((uintptr_t)W % 16) == 0;
        count_launch();
#define LCC_ROWS(VECB, WRN, WARPS)                                                                                         \
    linear_rows_kernel<T, TC, VECB, WRN><<<(N + WARPS * WRN - 1) / (WARPS * WRN), WARPS * 32, 0, s>>>((const T*)A, lda, (const T*)W, \
                                                                                                      ldw, bias, (TC*)C, ldc, M, N, K)
        if (N >= 8192) {
            if (vec) LCC_ROWS(true, 2, 8); else LCC_ROWS(false, 2, 8);
        } else {
            if (vec) LCC_ROWS(true, 1, 2); else LCC_ROWS(false, 1, 2);
        }
#undef LCC_ROWS
    } else {
        dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
        count_launch();
        linear_tile_kernel<T, TC><<<grid, 256, 0, s>>>((const T*)A, lda, (const T*)W, ldw, bias, (TC*)C, ldc, M, N, K);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

}  // namespace

int linear_any(int dt, const void* A, int lda, const void* W, int ldw, const float* bias, void* C, int ldc, bool c_f32,
               int M, int N, int K, cudaStream_t s) {
    if (!A || !W || !C || M < 1 || N < 1 || K < 1 || lda < K || ldw < K || ldc < N) return -2;
    if (dt == DT_F32) return launch_linear<float, float>(A, lda, W, ldw, bias, C, ldc, M, N, K, s);
    if (c_f32) return launch_linear<bf16, float>(A, lda, W, ldw, bias, C, ldc, M, N, K, s);
    return launch_linear<bf16, bf16>(A, lda, W, ldw, bias, C, ldc, M, N, K, s);
}

}  // namespace lcc
