// Mixture-of-experts feed-forward of layered decoders.
//
//   moe_route         fp32 router: z = W_r h, s = softmax(z) over all n routed outputs (the last n_identity of them are identity
//                     experts: output = input); choice = s + correction; the n outputs form `groups` equal groups of
//                     neighbours, a group scores its largest choice, only the best `keep` groups stay eligible; the `top`
//                     largest eligible choices are taken, each weighted by its s (not renormalised).  Ties go to the lower index.
//                     Writes the dense weights [T, n] (0 where not chosen) and the chosen (index, weight) pairs [T, top].
//   moe_gateup_sparse / moe_down_sparse   few tokens (decode): one CTA column per (token, chosen expert) streams only that
//                     expert's rows: act = silu(W_gate h) * (W_up h), then y = sum_k w_k W_down[e_k] act_k + (identity weights) h
//   rows_axpy         y[t] += (sum of the identity weights of t) * h[t]       (after the dense, masked form for prompts)
//
// Weights are packed: w13 [E * 2 * ff, width] with rows (2c, 2c + 1) = (gate_c, up_c) of each expert in turn; w2 [width, E * ff]
// with expert e's down projection in columns e*ff .. (e+1)*ff - 1.  Prompts run the dense form through the Linear kernels:
// every expert on every token, the SwiGLU epilogue multiplying by the token's routing weight of the column's expert.
#pragma once
#include "hybrid_common.cuh"

namespace mbh {

struct MoeRouteArgs {
    const void* h;            // [T, width]
    const void* w_router;     // [n, width]
    const void* correction;   // [n] or null
    float* dense;             // [T, n]
    int* idx;                 // [T, top]
    float* wsel;              // [T, top]
    int width, n, groups, keep, top;
    int score;                // 0: softmax over the outputs; 1: sigmoid of each output
    float scale;              // the weights (dense and wsel) are the chosen scores times this
};

// (value, index) argmax over a warp; the lower index wins a tie
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, v, o);
        const int oi = __shfl_xor_sync(0xffffffffu, i, o);
        if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
    }
}

// dot product of two rows of K elements over a warp (16-byte loads when both rows allow it); every lane gets the sum
template <typename T>
__device__ __forceinline__ float warp_dot(const T* __restrict__ w, const T* __restrict__ x, int K, int lane) {
    constexpr int V = Vec<T>::N;
    float acc = 0.f;
    if (K % V == 0 && ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(x)) % 16 == 0)) {
        for (int k = lane * V; k < K; k += 32 * V) {
            float wv[V], xv[V];
            Vec<T>::load(w + k, wv);
            Vec<T>::load(x + k, xv);
#pragma unroll
            for (int i = 0; i < V; ++i) acc = fmaf(wv[i], xv[i], acc);
        }
    } else {
        for (int k = lane; k < K; k += 32) acc = fmaf(to_f(w[k]), to_f(x[k]), acc);
    }
    return warp_sum(acc);
}

constexpr int MOE_ROUTE_THREADS = 256;

// one CTA per token; shared memory: z[n] | choice[n] | gbest[groups] | kept[groups]
template <typename T>
__global__ void __launch_bounds__(MOE_ROUTE_THREADS) moe_route_kernel(MoeRouteArgs a) {
    extern __shared__ float sm[];
    float* z = sm;
    float* ch = sm + a.n;
    float* gb = sm + 2 * a.n;
    float* kept = gb + a.groups;
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const T* h = static_cast<const T*>(a.h) + (size_t)t * a.width;
    const T* W = static_cast<const T*>(a.w_router);
    for (int e = warp; e < a.n; e += nw) {
        const float acc = warp_dot<T>(W + (size_t)e * a.width, h, a.width, lane);
        if (lane == 0) z[e] = acc;
    }
    __syncthreads();
    if (warp != 0) return;
    float sum = 1.f;
    if (a.score == 1) {
        for (int e = lane; e < a.n; e += 32) z[e] = sigmoid_exact(z[e]);
    } else {
        float mx = -INFINITY;
        for (int e = lane; e < a.n; e += 32) mx = fmaxf(mx, z[e]);
        mx = warp_max(mx);
        sum = 0.f;
        for (int e = lane; e < a.n; e += 32) { const float p = expf(z[e] - mx); z[e] = p; sum += p; }
        sum = warp_sum(sum);
    }
    const T* corr = static_cast<const T*>(a.correction);
    for (int e = lane; e < a.n; e += 32) {
        const float s = z[e] / sum;
        z[e] = s;
        ch[e] = s + (corr ? to_f(corr[e]) : 0.f);
        a.dense[(size_t)t * a.n + e] = 0.f;
    }
    __syncwarp();
    if (a.groups > 1 && a.keep < a.groups) {
        const int gs = a.n / a.groups;
        for (int g = lane; g < a.groups; g += 32) {
            float b = -INFINITY;
            for (int e = g * gs; e < (g + 1) * gs; ++e) b = fmaxf(b, ch[e]);
            gb[g] = b;
            kept[g] = 0.f;
        }
        __syncwarp();
        // take the best `keep` groups one at a time; then drop the experts of the others
        for (int k = 0; k < a.keep; ++k) {
            float v = -INFINITY; int gi = 0x7fffffff;
            for (int g = lane; g < a.groups; g += 32)
                if (kept[g] == 0.f && (gi == 0x7fffffff || gb[g] > v)) { v = gb[g]; gi = g; }
            warp_argmax(v, gi);
            if (lane == 0 && gi != 0x7fffffff) kept[gi] = 1.f;
            __syncwarp();
        }
        for (int e = lane; e < a.n; e += 32)
            if (kept[e / gs] == 0.f) ch[e] = -INFINITY;
        __syncwarp();
    }
    for (int k = 0; k < a.top; ++k) {
        float v = -INFINITY; int ei = 0x7fffffff;
        for (int e = lane; e < a.n; e += 32)
            if (ch[e] > v) { v = ch[e]; ei = e; }
        warp_argmax(v, ei);
        if (ei == 0x7fffffff) ei = 0;  // fewer eligible outputs than `top` (a configuration error): weight 0 below
        if (lane == 0) {
            const float w = (v == -INFINITY) ? 0.f : z[ei] * a.scale;
            a.idx[(size_t)t * a.top + k] = ei;
            a.wsel[(size_t)t * a.top + k] = w;
            if (v != -INFINITY) { a.dense[(size_t)t * a.n + ei] = w; ch[ei] = -INFINITY; }
        }
        __syncwarp();
    }
}

struct MoeSparseArgs {
    const void* h;            // [T, width]
    const void* w13;          // [E * 2 * ff, width]
    const void* w2;           // [width, E * ff]
    const int* idx;           // [T, top]
    const float* wsel;        // [T, top]
    void* act;                // [T * top, ff]
    float* y32;               // [T, width]
    int width, ff, E, top;
    int glu;                  // 0: silu(gate) * up, the routing weight multiplies the expert's OUTPUT; 1: the weight multiplies the
    float limit, alpha;       //    expert's INPUT: g = min(w gate, limit), u = clamp(w up, +-limit), act = g sigmoid(alpha g) (u + 1);
                              // 2: experts without a gate, act = max(W_up h, 0)^2, w13 = [E * ff, width] plain rows, weight on the OUTPUT
    int accumulate;           // y32 += the experts' sum (y32 is the residual stream) instead of y32 = it
};

constexpr int MOE_WARPS = 8;

// grid (ceil(ff / MOE_WARPS), T * top): a warp per hidden unit of the chosen expert
template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32) moe_gateup_sparse_kernel(MoeSparseArgs a) {
    const int slot = blockIdx.y, t = slot / a.top, e = a.idx[slot];
    if (e >= a.E) return;  // identity expert: no weights
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, c = blockIdx.x * MOE_WARPS + warp;
    if (c >= a.ff) return;
    const T* h = static_cast<const T*>(a.h) + (size_t)t * a.width;
    if (a.glu == 2) {
        const float u = rnd<T>(warp_dot<T>(static_cast<const T*>(a.w13) + ((size_t)e * a.ff + c) * a.width, h, a.width, lane));
        if (lane == 0) { const float r = fmaxf(u, 0.f); static_cast<T*>(a.act)[(size_t)slot * a.ff + c] = from_f<T>(r * r); }
        return;
    }
    const T* wg = static_cast<const T*>(a.w13) + ((size_t)e * a.ff + c) * 2 * a.width;
    float g = rnd<T>(warp_dot<T>(wg, h, a.width, lane)), u = rnd<T>(warp_dot<T>(wg + a.width, h, a.width, lane));
    if (lane != 0) return;
    float act;
    if (a.glu == 1) {
        const float w = a.wsel[slot];
        g = fminf(g * w, a.limit);
        u = fminf(fmaxf(u * w, -a.limit), a.limit);
        act = g * sigmoid_exact(a.alpha * g) * (u + 1.f);
    } else {
        act = g * sigmoid_exact(g) * u;
    }
    static_cast<T*>(a.act)[(size_t)slot * a.ff + c] = from_f<T>(act);
}

// grid (ceil(width / MOE_WARPS), T): a warp per output column, summing the token's chosen experts in slot order
template <typename T>
__global__ void __launch_bounds__(MOE_WARPS * 32) moe_down_sparse_kernel(MoeSparseArgs a) {
    const int t = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n = blockIdx.x * MOE_WARPS + warp;
    if (n >= a.width) return;
    const T* wrow = static_cast<const T*>(a.w2) + (size_t)n * a.E * a.ff;
    float acc = 0.f;
    for (int k = 0; k < a.top; ++k) {
        const int slot = t * a.top + k, e = a.idx[slot];
        const float w = a.glu == 1 ? 1.f : a.wsel[slot];
        if (e >= a.E) acc += w * to_f(static_cast<const T*>(a.h)[(size_t)t * a.width + n]);
        else acc += w * rnd<T>(warp_dot<T>(wrow + (size_t)e * a.ff, static_cast<const T*>(a.act) + (size_t)slot * a.ff, a.ff, lane));
    }
    if (lane == 0) {
        if (a.accumulate) a.y32[(size_t)t * a.width + n] += acc;
        else a.y32[(size_t)t * a.width + n] = acc;
    }
}

// y[t, :] += (sum of dense[t, first .. n - 1]) * h[t, :]
template <typename T>
__global__ void rows_axpy_kernel(float* __restrict__ y, const T* __restrict__ h, const float* __restrict__ dense, int n, int first, int D) {
    const int t = blockIdx.x;
    float w = 0.f;
    for (int e = first; e < n; ++e) w += dense[(size_t)t * n + e];
    if (w == 0.f) return;
    for (int i = threadIdx.x; i < D; i += blockDim.x) y[(size_t)t * D + i] += w * to_f(h[(size_t)t * D + i]);
}

}  // namespace mbh
