// Chunk-local attention over a paged K/V cache with arbitrary head sizes:
//   * q/k RMS norm over the whole projection (all heads at once) and the append of k, v to the pages,
//   * attention of new rows over the keys of their own chunk (chunks counted from position 0 of the sequence) with a
//     softmax sink: p_j = exp(s_j) / (1 + sum_j exp(s_j)), and a per-head sigmoid output gate.
// Scores, weights and the accumulation are fp32; K and V pages hold the model's storage type.
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

__device__ __forceinline__ int seq_past(const SeqPos& p, int) { return p.kv_len ? *p.kv_len : p.past; }
__device__ __forceinline__ bool seq_done(const SeqPos& p) { return p.finished && *p.finished; }

// One CTA per new row.
template <typename T>
__global__ void __launch_bounds__(256) qk_norm_kv_append_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ qn_w,
                                                                const float* __restrict__ kn_w, float eps, float* __restrict__ q_out,
                                                                T* __restrict__ k_pages, T* __restrict__ v_pages,
                                                                const int* __restrict__ page_table, int page_size, int S, int Hq,
                                                                int G, int D, int DV, SeqPos pos) {
    if (seq_done(pos)) return;
    __shared__ float red[32];
    const int t = blockIdx.x;
    const int p = seq_past(pos, S) + t;
    const T* row = proj + (size_t)t * ld;
    const int nq = Hq * D, nk = G * D, nv = G * DV;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float v = ldf(row + i); sq = fmaf(v, v, sq); }
    for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float v = ldf(row + nq + i); sk = fmaf(v, v, sk); }
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    const float rq = 1.f / sqrtf(sq / (float)nq + eps), rk = 1.f / sqrtf(sk / (float)nk + eps);
    for (int i = threadIdx.x; i < nq; i += blockDim.x) q_out[(size_t)t * nq + i] = ldf(row + i) * rq * qn_w[i];
    const int page = page_table[p / page_size], slot = p % page_size;
    for (int i = threadIdx.x; i < nk; i += blockDim.x) {
        const int g = i / D, d = i % D;
        stf(k_pages + (((size_t)page * G + g) * page_size + slot) * D + d, ldf(row + nq + i) * rk * kn_w[i]);
    }
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const int g = i / DV, d = i % DV;
        v_pages[(((size_t)page * G + g) * page_size + slot) * DV + d] = row[nq + nk + i];
    }
}

// One CTA per (new row, query head). Scores of the row's chunk go to shared memory (fp32), then the weights, then
// thread c accumulates output channel c over the keys.
template <typename T>
__global__ void __launch_bounds__(128) attn_chunk_sink_kernel(const float* __restrict__ q, const T* __restrict__ k_pages,
                                                              const T* __restrict__ v_pages, const int* __restrict__ page_table,
                                                              int page_size, const T* __restrict__ gate, int ld_gate,
                                                              T* __restrict__ out, int ld_out, int S, int Hq, int G, int D, int DV,
                                                              int chunk, float scale, SeqPos pos) {
    if (seq_done(pos)) return;
    extern __shared__ float sm[];
    __shared__ float red[32];
    const int t = blockIdx.x, h = blockIdx.y;
    const int g = h / (Hq / G);
    const int p = seq_past(pos, S) + t;
    const int start = chunk > 0 ? (p / chunk) * chunk : 0;
    const int nkeys = p - start + 1;
    float* sq = sm;           // [D]
    float* sc = sm + D;       // [nkeys]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int i = threadIdx.x; i < D; i += blockDim.x) sq[i] = q[((size_t)t * Hq + h) * D + i];
    __syncthreads();
    // scores: one warp per key, lanes over the head dimension
    float mx = 0.f;  // the sink's score
    for (int jk = warp; jk < nkeys; jk += nwarps) {
        const int pj = start + jk;
        const T* kr = k_pages + (((size_t)page_table[pj / page_size] * G + g) * page_size + pj % page_size) * D;
        float acc = 0.f;
        for (int d = lane; d < D; d += 32) acc = fmaf(sq[d], ldf(kr + d), acc);
        acc = warp_sum(acc) * scale;
        if (lane == 0) sc[jk] = acc;
        mx = fmaxf(mx, acc);
    }
    mx = warp_max(mx);
    __syncthreads();
    if (lane == 0) red[warp] = mx;
    __syncthreads();
    mx = red[0];
    for (int i = 1; i < nwarps; ++i) mx = fmaxf(mx, red[i]);
    float sum = 0.f;
    for (int jk = threadIdx.x; jk < nkeys; jk += blockDim.x) {
        const float e = expf(sc[jk] - mx);
        sc[jk] = e;
        sum += e;
    }
    sum = block_sum(sum, red);   // contains the barrier that publishes sc[]
    const float inv = 1.f / (expf(-mx) + sum);
    float gv = 1.f;
    if (gate) gv = 1.f / (1.f + expf(-ldf(gate + (size_t)t * ld_gate + h)));
    for (int c = threadIdx.x; c < DV; c += blockDim.x) {
        float acc = 0.f;
        for (int jk = 0; jk < nkeys; ++jk) {
            const int pj = start + jk;
            const T* vr = v_pages + (((size_t)page_table[pj / page_size] * G + g) * page_size + pj % page_size) * DV;
            acc = fmaf(sc[jk], ldf(vr + c), acc);
        }
        stf(out + (size_t)t * ld_out + (size_t)h * DV + c, acc * inv * gv);
    }
}

}  // namespace

int qk_norm_kv_append(int dt, const void* proj, int ld, const float* qn_w, const float* kn_w, float eps, float* q_out,
                      void* k_pages, void* v_pages, const int* page_table, int page_size, int S, int Hq, int G, int D,
                      int DV, SeqPos pos, cudaStream_t s) {
    if (!proj || !qn_w || !kn_w || !q_out || !k_pages || !v_pages || !page_table || S < 1 || Hq < 1 || G < 1 || D < 1 ||
        DV < 1 || page_size < 1)
        return -2;
    count_launch();
    if (dt == DT_F32)
        qk_norm_kv_append_kernel<float><<<S, 256, 0, s>>>((const float*)proj, ld, qn_w, kn_w, eps, q_out, (float*)k_pages,
                                                          (float*)v_pages, page_table, page_size, S, Hq, G, D, DV, pos);
    else
        qk_norm_kv_append_kernel<bf16><<<S, 256, 0, s>>>((const bf16*)proj, ld, qn_w, kn_w, eps, q_out, (bf16*)k_pages,
                                                         (bf16*)v_pages, page_table, page_size, S, Hq, G, D, DV, pos);
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

int attn_chunk_sink(int dt, const float* q, const void* k_pages, const void* v_pages, const int* page_table,
                    int page_size, const void* gate, int ld_gate, void* out, int ld_out, int S, int Hq, int G, int D,
                    int DV, int chunk, float scale, SeqPos pos, cudaStream_t s) {
    if (!q || !k_pages || !v_pages || !page_table || !out || S < 1 || Hq < 1 || G < 1 || Hq % G || D < 1 || DV < 1)
        return -2;
    // shared memory holds one score per key of the longest window a row of this call can have
    int max_keys = chunk;
    if (chunk <= 0) {
        if (pos.kv_len) return -3;  // plain causal attention needs the host-side length to size the score buffer
        max_keys = pos.past + S;
    }
    const size_t smem = sizeof(float) * ((size_t)D + (size_t)max_keys);
    if (smem > 200 * 1024) return -3;
    dim3 grid(S, Hq);
    count_launch();
    if (dt == DT_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attn_chunk_sink_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attn_chunk_sink_kernel<float><<<grid, 128, smem, s>>>(q, (const float*)k_pages, (const float*)v_pages, page_table,
                                                              page_size, (const float*)gate, ld_gate, (float*)out, ld_out, S, Hq,
                                                              G, D, DV, chunk, scale, pos);
    } else {
        if (smem > 48 * 1024) cudaFuncSetAttribute(attn_chunk_sink_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        attn_chunk_sink_kernel<bf16><<<grid, 128, smem, s>>>(q, (const bf16*)k_pages, (const bf16*)v_pages, page_table,
                                                             page_size, (const bf16*)gate, ld_gate, (bf16*)out, ld_out, S, Hq, G,
                                                             D, DV, chunk, scale, pos);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

}  // namespace lcc
