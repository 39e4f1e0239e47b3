// Rotary attention inputs and the embedding with learned positions.
//
//   embed_pos        x[t] = E[token[t]] * scale + P[position[t]]            -> fp32 residual stream
//   rot_prep         splits qkv[T, H*d + G*d + G*e]; rotates the first rot_dims entries of every q and k head as interleaved pairs
//                    (2i, 2i + 1) by position * freq[i]; optionally divides each head by its root mean square (no weight);
//                    writes q[T, H*d], k[T, G*d], v[T, G*e] token-major and, for tokens with a ring row, k and v into the ring
//   kv_scatter       k[T, G*d], v[T, G*e] -> ring rows cache_rows[t] (after a prompt's attention has read the old ring)
//
// The angle is position * freq[i] in double precision (frequencies come from the host in float64): an fp32 product at
// position 1000 is already off by 6e-5 rad.  Rotation and norm are fp32; the results are stored in the storage type.
#pragma once
#include "hybrid_common.cuh"

namespace mbh {

template <typename T>
__global__ void embed_pos_kernel(const int64_t* __restrict__ tok, const int* __restrict__ positions, const T* __restrict__ E, const T* __restrict__ P,
                                 float scale, float* __restrict__ x, int D) {
    const T* row = E + (size_t)tok[blockIdx.x] * D;
    const T* prow = P + (size_t)positions[blockIdx.x] * D;
    float* o = x + (size_t)blockIdx.x * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = to_f(row[i]) * scale + to_f(prow[i]);
}

struct RotPrepArgs {
    const void* qkv;        // [T, H*d + G*d + G*e]
    const double* freq;     // [rot_dims / 2] angle per position step of pair i
    const int* positions;   // [T]
    const int* cache_rows;  // [T] ring row or -1; null: nothing goes to the ring in this call
    void* q_out;            // [T, H*d]
    void* k_out; void* v_out;   // [T, G*d] / [T, G*e], or null
    void* ring_k; void* ring_v; // [rows, G, d] / [rows, G, e]
    int H, G, d, e, rot_dims;
    int unit_norm;          // divide every rotated q and k head by sqrt(mean(x^2) + eps)
    float eps;
};

constexpr int RP_MAXP = 4;  // pairs per lane: head sizes up to 256

// grid (T, groups of heads), a warp per head
template <typename T>
__global__ void __launch_bounds__(128) rot_prep_kernel(RotPrepArgs a) {
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int Nq = a.H * a.d, Nk = a.G * a.d, Nv = a.G * a.e;
    const T* row = static_cast<const T*>(a.qkv) + (size_t)t * (Nq + Nk + Nv);
    const int pos = a.positions[t];
    const int crow = a.cache_rows ? a.cache_rows[t] : -1;
    const int half = a.d >> 1;  // pairs; an odd last entry passes unchanged
    for (int h = blockIdx.y * nw + warp; h < a.H + a.G; h += gridDim.y * nw) {
        const bool is_q = h < a.H;
        const T* src = row + (is_q ? h * a.d : Nq + (h - a.H) * a.d);
        float u[RP_MAXP], v[RP_MAXP], ss = 0.f;
#pragma unroll
        for (int r = 0; r < RP_MAXP; ++r) {
            const int pi = lane + 32 * r;
            u[r] = v[r] = 0.f;
            if (pi < half) {
                float x0 = to_f(src[2 * pi]), x1 = to_f(src[2 * pi + 1]);
                if (2 * pi + 1 < a.rot_dims) {
                    double sn, cs;
                    sincos((double)pos * a.freq[pi], &sn, &cs);
                    const float c = (float)cs, s = (float)sn;
                    const float y0 = x0 * c - x1 * s, y1 = x1 * c + x0 * s;
                    x0 = y0; x1 = y1;
                }
                u[r] = x0; v[r] = x1;
                ss = fmaf(x0, x0, fmaf(x1, x1, ss));
            }
        }
        float last = 0.f;
        if ((a.d & 1) && lane == 0) { last = to_f(src[a.d - 1]); ss = fmaf(last, last, ss); }
        ss = warp_sum(ss);
        const float inv = a.unit_norm ? 1.f / sqrtf(ss / (float)a.d + a.eps) : 1.f;
        T* dst0 = is_q ? static_cast<T*>(a.q_out) + (size_t)t * Nq + h * a.d
                       : (a.k_out ? static_cast<T*>(a.k_out) + (size_t)t * Nk + (h - a.H) * a.d : nullptr);
        T* dst1 = (!is_q && crow >= 0) ? static_cast<T*>(a.ring_k) + (size_t)crow * Nk + (h - a.H) * a.d : nullptr;
#pragma unroll
        for (int r = 0; r < RP_MAXP; ++r) {
            const int pi = lane + 32 * r;
            if (pi < half) {
                const T y0 = from_f<T>(u[r] * inv), y1 = from_f<T>(v[r] * inv);
                if (dst0) { dst0[2 * pi] = y0; dst0[2 * pi + 1] = y1; }
                if (dst1) { dst1[2 * pi] = y0; dst1[2 * pi + 1] = y1; }
            }
        }
        if ((a.d & 1) && lane == 0) {
            if (dst0) dst0[a.d - 1] = from_f<T>(last * inv);
            if (dst1) dst1[a.d - 1] = from_f<T>(last * inv);
        }
    }
    const T* vsrc = row + Nq + Nk;
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < Nv; i += gridDim.y * blockDim.x) {
        if (a.v_out) static_cast<T*>(a.v_out)[(size_t)t * Nv + i] = vsrc[i];
        if (crow >= 0) static_cast<T*>(a.ring_v)[(size_t)crow * Nv + i] = vsrc[i];
    }
}

template <typename T>
__global__ void kv_scatter_kernel(const T* __restrict__ k, const T* __restrict__ v, const int* __restrict__ cache_rows, T* __restrict__ ring_k,
                                  T* __restrict__ ring_v, int Nk, int Nv) {
    const int t = blockIdx.x, crow = cache_rows[t];
    if (crow < 0) return;
    for (int i = threadIdx.x; i < Nk; i += blockDim.x) ring_k[(size_t)crow * Nk + i] = k[(size_t)t * Nk + i];
    for (int i = threadIdx.x; i < Nv; i += blockDim.x) ring_v[(size_t)crow * Nv + i] = v[(size_t)t * Nv + i];
}

}  // namespace mbh
