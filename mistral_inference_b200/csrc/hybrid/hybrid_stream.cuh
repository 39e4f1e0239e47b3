// Steps on the fp32 residual stream of designs whose sublayers read the stream itself and are normed on the way back:
//
//   canon_conv        h[t] = x[t] + sum_j w[:, j] * x[t - taps + 1 + j]: a causal convolution over time on every channel, added to
//                     its own input; what lies before the sequence's start is zero.  The last taps - 1 inputs of each sequence are
//                     carried in the cache (fp32), so a prompt portion or a decode step continues where the last call stopped
//   canon_state       writes those last taps - 1 inputs back after the convolution has read the old ones
//   canon_conv_step   both for one token per sequence (a decode step), one launch
//   rmsnorm_add       acc[t] += y[t] / sqrt(mean(y[t]^2) + eps) * w: the norm of a sublayer's OUTPUT, added to the stream in fp32;
//                     optionally followed by the depth average: out[t] = sum_j c[j] * X_j[t] over the layer results X_0 .. X_(n-1)
//                     kept one after the other (X_(n-1) is acc itself, just updated)
//   depth_mix         the depth average alone
#pragma once
#include "hybrid_common.cuh"

namespace mbh {

struct CanonArgs {
    const float* x;        // [T, D] the stream
    const void* w;         // [D, taps] storage type
    float* state;          // sequence in slot s: state + s * state_stride + state_off, [taps - 1, D]
    int state_stride, state_off;
    const int* q_start;    // [B + 1]
    const int* seqpos;     // [B] tokens before this call (0: nothing before, whatever the slot holds)
    const int* slots;      // [B]
    void* h;               // [T, D] storage type
    int B, D, taps;
};

// grid (T, blocks of channels)
template <typename T>
__global__ void canon_conv_kernel(CanonArgs a) {
    const int t = blockIdx.x;
    int b = 0;
    while (b + 1 < a.B && a.q_start[b + 1] <= t) ++b;
    const int i = t - a.q_start[b], back = a.taps - 1;
    const bool has_state = a.seqpos[b] > 0;
    const float* st = a.state + (size_t)a.slots[b] * a.state_stride + a.state_off;
    const T* W = static_cast<const T*>(a.w);
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < a.D; c += gridDim.y * blockDim.x) {
        const float xc = a.x[(size_t)t * a.D + c];
        float acc = 0.f;
        for (int j = 0; j < a.taps; ++j) {
            const int src = i - back + j;  // index within this call's tokens of the sequence
            float v;
            if (src >= 0) v = a.x[(size_t)(a.q_start[b] + src) * a.D + c];
            else v = has_state ? st[(size_t)(back + src) * a.D + c] : 0.f;
            acc = fmaf(to_f(W[(size_t)c * a.taps + j]), v, acc);
        }
        static_cast<T*>(a.h)[(size_t)t * a.D + c] = from_f<T>(xc + acc);
    }
}

// Prompts: a CTA takes CANON_TILE consecutive tokens and 4 * blockDim channels; a thread owns 4 adjacent channels (one 16-byte load
// of the stream per token) and walks the tile's tokens with the last TAPS - 1 inputs in registers, so the stream is read once (plus
// TAPS - 1 rows where a tile or a sequence starts).  Needs D % 4 == 0.  grid (ceil(T / CANON_TILE), ceil(D / (4 * blockDim)))
constexpr int CANON_TILE = 16;

template <typename T> __device__ __forceinline__ void store4(T* p, const float* v);
template <> __device__ __forceinline__ void store4<float>(float* p, const float* v) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
template <> __device__ __forceinline__ void store4<bf16>(bf16* p, const float* v) {
    __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t*>(&lo); u.y = *reinterpret_cast<uint32_t*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
}

template <typename T, int TAPS>
__global__ void __launch_bounds__(128) canon_conv_tiled_kernel(CanonArgs a, int T_total) {
    constexpr int BACK = TAPS - 1;
    const int c = (blockIdx.y * blockDim.x + threadIdx.x) * 4;
    if (c >= a.D) return;
    const int t0 = blockIdx.x * CANON_TILE, t1 = min(t0 + CANON_TILE, T_total);
    float w[4][TAPS];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
        for (int j = 0; j < TAPS; ++j) w[u][j] = to_f(static_cast<const T*>(a.w)[(size_t)(c + u) * TAPS + j]);
    float4 win[BACK > 0 ? BACK : 1];
    int b = 0;
    while (b + 1 < a.B && a.q_start[b + 1] <= t0) ++b;
    int seq_end = a.q_start[b + 1];
    bool fresh = true;  // the window must be (re)loaded: first token of the tile, or of a sequence
    for (int t = t0; t < t1; ++t) {
        if (t >= seq_end) {
            while (b + 1 < a.B && a.q_start[b + 1] <= t) ++b;
            seq_end = a.q_start[b + 1];
            fresh = true;
        }
        if (fresh) {
            const int i = t - a.q_start[b];
            const bool has_state = a.seqpos[b] > 0;
            const float* st = a.state + (size_t)a.slots[b] * a.state_stride + a.state_off;
#pragma unroll
            for (int j = 0; j < BACK; ++j) {
                const int src = i - BACK + j;
                if (src >= 0) win[j] = *reinterpret_cast<const float4*>(a.x + (size_t)(a.q_start[b] + src) * a.D + c);
                else if (has_state) win[j] = *reinterpret_cast<const float4*>(st + (size_t)(BACK + src) * a.D + c);
                else win[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
            fresh = false;
        }
        const float4 xc = *reinterpret_cast<const float4*>(a.x + (size_t)t * a.D + c);
        float o[4] = {xc.x, xc.y, xc.z, xc.w};
#pragma unroll
        for (int j = 0; j < BACK; ++j) {
            o[0] = fmaf(w[0][j], win[j].x, o[0]); o[1] = fmaf(w[1][j], win[j].y, o[1]);
            o[2] = fmaf(w[2][j], win[j].z, o[2]); o[3] = fmaf(w[3][j], win[j].w, o[3]);
        }
        o[0] = fmaf(w[0][BACK], xc.x, o[0]); o[1] = fmaf(w[1][BACK], xc.y, o[1]);
        o[2] = fmaf(w[2][BACK], xc.z, o[2]); o[3] = fmaf(w[3][BACK], xc.w, o[3]);
        store4<T>(static_cast<T*>(a.h) + (size_t)t * a.D + c, o);
#pragma unroll
        for (int j = 0; j + 1 < BACK; ++j) win[j] = win[j + 1];
        if (BACK > 0) win[BACK - 1] = xc;
    }
}

// grid (B, blocks of channels); a thread moves one channel's entries in rising order, reading only entries it has not yet written
__global__ void canon_state_kernel(CanonArgs a) {
    const int b = blockIdx.x, back = a.taps - 1;
    const int len = a.q_start[b + 1] - a.q_start[b];
    if (len <= 0) return;
    const bool has_state = a.seqpos[b] > 0;
    float* st = a.state + (size_t)a.slots[b] * a.state_stride + a.state_off;
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < a.D; c += gridDim.y * blockDim.x)
        for (int j = 0; j < back; ++j) {
            const int src = len - back + j;
            float v;
            if (src >= 0) v = a.x[(size_t)(a.q_start[b] + src) * a.D + c];
            else v = has_state ? st[(size_t)(j + len) * a.D + c] : 0.f;
            st[(size_t)j * a.D + c] = v;
        }
}

// one token per sequence (token b belongs to sequence b): convolution and state shift in one launch.  grid (B, blocks of channels)
template <typename T>
__global__ void canon_conv_step_kernel(CanonArgs a) {
    const int b = blockIdx.x, back = a.taps - 1;
    const bool has_state = a.seqpos[b] > 0;
    float* st = a.state + (size_t)a.slots[b] * a.state_stride + a.state_off;
    const T* W = static_cast<const T*>(a.w);
    for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < a.D; c += gridDim.y * blockDim.x) {
        const float xc = a.x[(size_t)b * a.D + c];
        float acc = to_f(W[(size_t)c * a.taps + back]) * xc;
        for (int j = 0; j < back; ++j) {
            const float v = has_state ? st[(size_t)j * a.D + c] : 0.f;
            acc = fmaf(to_f(W[(size_t)c * a.taps + j]), v, acc);
            if (j > 0) st[(size_t)(j - 1) * a.D + c] = v;
        }
        if (back > 0) st[(size_t)(back - 1) * a.D + c] = xc;
        static_cast<T*>(a.h)[(size_t)b * a.D + c] = from_f<T>(xc + acc);
    }
}

struct NormAddArgs {
    const float* y;        // [T, D] sublayer output
    const void* w;         // [D] storage type
    float* acc;            // [T, D] the stream, updated in place
    int D;
    float eps;
    const float* stack;    // depth average: X_j = stack + j * stack_stride, j < n - 1; X_(n-1) = acc.  null: none
    size_t stack_stride;
    const void* coef;      // [n] storage type
    int n;
    float* out;            // [T, D]
};

// grid (rows, column blocks): with one column block a CTA takes a whole row; a decode step's few rows are spread over several CTAs,
// each of which sums the squares of the whole row (a few KB from L2) and then updates its own slice of the columns
template <typename T>
__global__ void rmsnorm_add_kernel(NormAddArgs a) {
    __shared__ float red[32];
    const size_t row = (size_t)blockIdx.x * a.D;
    const float* r = a.y + row;
    float ss = 0.f;
    for (int i = threadIdx.x; i < a.D; i += blockDim.x) ss = fmaf(r[i], r[i], ss);
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)a.D + a.eps);
    const T* w = static_cast<const T*>(a.w);
    const T* cf = static_cast<const T*>(a.coef);
    const int per = (a.D + gridDim.y - 1) / gridDim.y, c0 = blockIdx.y * per, c1 = min(a.D, c0 + per);
    for (int i = c0 + threadIdx.x; i < c1; i += blockDim.x) {
        const float v = a.acc[row + i] + r[i] * inv * to_f(w[i]);
        a.acc[row + i] = v;
        if (a.stack) {
            float m = 0.f;
            for (int j = 0; j + 1 < a.n; ++j) m = fmaf(to_f(cf[j]), a.stack[(size_t)j * a.stack_stride + row + i], m);
            a.out[row + i] = fmaf(to_f(cf[a.n - 1]), v, m);
        }
    }
}

// out[i] = sum_j coef[j] * stack[j * stride + i], i < count
template <typename T>
__global__ void depth_mix_kernel(const float* __restrict__ stack, size_t stride, const T* __restrict__ coef, int n, float* __restrict__ out, size_t count) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float m = 0.f;
    for (int j = 0; j < n; ++j) m = fmaf(to_f(coef[j]), stack[(size_t)j * stride + i], m);
    out[i] = m;
}

}  // namespace mbh
