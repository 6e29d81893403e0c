// Rotary positions in the rotate-half layout on slices of a projection, written as fp32 for a recurrence that keeps
// its operands in fp32. Positions, angles, cos and sin are fp32 (full-range sinf / cosf, no fast-math).
#include <math.h>

#include "common.cuh"
#include "launch.h"
#include "seqmix.h"

namespace lcc {
namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p);
template <> __device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ldf<bf16>(const bf16* p) { return __bfloat162float(*p); }

__device__ __forceinline__ int seq_past(const SeqPos& p) { return p.kv_len ? *p.kv_len : p.past; }
__device__ __forceinline__ bool seq_done(const SeqPos& p) { return p.finished && *p.finished; }

struct Segs { RotarySegment s[4]; int n; };

// gridDim.y CTAs per row (several when the call has few rows, so that a decode step's single row is not one CTA's serial
// walk); together their threads walk the output channels of every segment.
template <typename T>
__global__ void __launch_bounds__(256) rotary_pack_kernel(const T* __restrict__ in, int ld_in, float* __restrict__ out, int ld_out,
                                                          Segs segs, const float* __restrict__ inv_freq, float mag,
                                                          const float* __restrict__ fill, float* __restrict__ fill_out, int fill_n,
                                                          SeqPos pos) {
    if (seq_done(pos)) return;
    const int t = blockIdx.x;
    const float p = (float)(seq_past(pos) + t);
    const T* row = in + (size_t)t * ld_in;
    float* orow = out + (size_t)t * ld_out;
    for (int si = 0; si < segs.n; ++si) {
        const RotarySegment sg = segs.s[si];
        const int n = sg.heads * sg.dim, half = sg.rot_dims / 2;
        for (int i = threadIdx.x + blockIdx.y * blockDim.x; i < n; i += blockDim.x * gridDim.y) {
            const int d = i % sg.dim, hb = i - d;
            const int r = d - sg.rot_off;
            float v = ldf(row + sg.col_in + i);
            if (r >= 0 && r < sg.rot_dims) {
                const int j = r < half ? r : r - half;
                const float ang = p * inv_freq[j];
                const float c = cosf(ang) * mag, s = sinf(ang) * mag;
                const float other = ldf(row + sg.col_in + hb + sg.rot_off + (r < half ? r + half : r - half));
                v = r < half ? v * c - other * s : v * c + other * s;
            }
            orow[sg.col_out + i] = v * sg.scale;
        }
    }
    if (fill_out && blockIdx.y == 0)
        for (int i = threadIdx.x; i < fill_n; i += blockDim.x) fill_out[(size_t)t * fill_n + i] = fill[i];
}

}  // namespace

int rotary_pack_f32(int dt, const void* in, int ld_in, float* out, int ld_out, const RotarySegment* seg, int n_seg,
                    const float* inv_freq, float mag, const float* fill, float* fill_out, int fill_n, int S, SeqPos pos,
                    cudaStream_t s) {
    if (!in || !out || !seg || n_seg < 1 || n_seg > 4 || S < 1 || (fill_out && (!fill || fill_n < 1))) return -2;
    Segs g{};
    g.n = n_seg;
    for (int i = 0; i < n_seg; ++i) {
        g.s[i] = seg[i];
        if (seg[i].rot_dims < 0 || (seg[i].rot_dims & 1) || seg[i].rot_off < 0 || seg[i].rot_off + seg[i].rot_dims > seg[i].dim ||
            (seg[i].rot_dims > 0 && !inv_freq))
            return -2;
    }
    count_launch();
    const dim3 S_grid(S, S < 32 ? 8 : 1);
    if (dt == DT_F32)
        rotary_pack_kernel<float><<<S_grid, 256, 0, s>>>((const float*)in, ld_in, out, ld_out, g, inv_freq, mag, fill, fill_out, fill_n, pos);
    else
        rotary_pack_kernel<bf16><<<S_grid, 256, 0, s>>>((const bf16*)in, ld_in, out, ld_out, g, inv_freq, mag, fill, fill_out, fill_n, pos);
    return cudaGetLastError() == cudaSuccess ? 0 : -100;
}

}  // namespace lcc
