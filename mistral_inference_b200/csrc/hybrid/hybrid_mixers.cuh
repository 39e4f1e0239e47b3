// Token mixers of the layered decoder and the elementwise steps around them.
//
//   embed_scale       x[t] = E[token[t]] * scale                       -> fp32 residual stream
//   rmsnorm_f32       y = x / sqrt(mean(x^2) + eps) * w                 fp32 in, storage type out
//   layernorm_f32     y = (x - mean) / sqrt(var + eps) * w + b          fp32 in; storage type out, or added to the residual stream
//   attn_prep         per-head RMS norm of q and k (shared weight), query temperature by position, value mixing with an
//                     earlier layer's values, scatter of k and v into the layer's cache ring
//   whole_norm_prep   RMS norm of a token's whole query and whole key projection (weights of that size), k and v to the ring
//   attn_bias         causal softmax attention over the ring with a per-(distance, head) additive bias, GQA, separate
//                     key and value sizes; one kernel for prompts, prompt portions and decode; optionally a sliding window and
//                     sigmoid weights instead of the softmax (every visible key weighs sigmoid(score), nothing is normalised)
//   lightning_scan    decayed linear attention S <- a S + k v^T, o = S^T q with the fp32 state carried in the cache
//   gated_headnorm    y = rms(o over all heads) * w * sigmoid(g)
#pragma once
#include "hybrid_common.cuh"

namespace mbh {

// ------------------------------------------------------------------------------------------------ embedding, norm
template <typename T, bool ADD = false>
__global__ void embed_scale_kernel(const int64_t* __restrict__ tok, const T* __restrict__ E, float scale, float* __restrict__ x, int D) {
    const T* row = E + (size_t)tok[blockIdx.x] * D;
    float* o = x + (size_t)blockIdx.x * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float v = to_f(row[i]) * scale;
        o[i] = ADD ? o[i] + v : v;
    }
}

// Layer norm of one fp32 row per CTA; the variance is the mean of the squared deviations (second pass over the row, which the
// first pass left in L1).  ADD: acc[t] += norm(x[t]) in fp32 (the norm after a sublayer, added to the residual stream);
// otherwise y[t] = norm(x[t]) in the storage type.  b may be null.
template <typename T, bool ADD>
__global__ void layernorm_f32_kernel(const float* __restrict__ x, const T* __restrict__ w, const T* __restrict__ b, T* __restrict__ y,
                                     float* __restrict__ acc, int D, float eps) {
    __shared__ float red[32];
    const float* r = x + (size_t)blockIdx.x * D;
    float s = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) s += r[i];
    const float mean = block_sum(s, red) / (float)D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) { const float dlt = r[i] - mean; ss = fmaf(dlt, dlt, ss); }
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)D + eps);
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
        const float v = (r[i] - mean) * inv * to_f(w[i]) + (b ? to_f(b[i]) : 0.f);
        if (ADD) acc[(size_t)blockIdx.x * D + i] += v;
        else y[(size_t)blockIdx.x * D + i] = from_f<T>(v);
    }
}

template <typename T>
__global__ void rmsnorm_f32_kernel(const float* __restrict__ x, const T* __restrict__ w, T* __restrict__ y, int D, float eps) {
    __shared__ float red[32];
    const float* r = x + (size_t)blockIdx.x * D;
    float ss = 0.f;
    for (int i = threadIdx.x; i < D; i += blockDim.x) ss = fmaf(r[i], r[i], ss);
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)D + eps);
    T* o = y + (size_t)blockIdx.x * D;
    for (int i = threadIdx.x; i < D; i += blockDim.x) o[i] = from_f<T>(r[i] * inv * to_f(w[i]));
}

// ------------------------------------------------------------------------------------------------ attention: q/k/v preparation
struct AttnPrepArgs {
    const void* qkv;       // [T, H*d + G*d + G*e] projections with bias
    const void* qnorm; const void* knorm;   // [d] each, or null (no norm)
    const int* positions;  // [T]
    const int* cache_rows; // [T] flat ring row (slot * W + pos % W) or -1
    void* q_out;           // [T, H*d]
    void* cache_k; void* cache_v;  // [rows, G, d] / [rows, G, e]
    void* v_first;         // [T, G*e]: written when vmix_mode == 1, read when == 2
    const void* vmix;      // scalar lambda (storage type), vmix_mode == 2
    int vmix_mode;
    int H, G, d, e;
    float eps, temp_coef; int temp_every;  // temperature 1 + coef * ln(floor((p + 1) / every) + 1); every == 0: none
};

template <typename T>
__global__ void attn_prep_kernel(AttnPrepArgs a) {
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int Nq = a.H * a.d, Nk = a.G * a.d, Nv = a.G * a.e;
    const T* row = static_cast<const T*>(a.qkv) + (size_t)t * (Nq + Nk + Nv);
    const int pos = a.positions[t];
    const int crow = a.cache_rows ? a.cache_rows[t] : -1;
    float temp = 1.f;
    if (a.temp_every > 0) temp = 1.f + a.temp_coef * logf((float)((pos + 1) / a.temp_every + 1));
    for (int h = warp; h < a.H + a.G; h += nw) {
        const bool is_q = h < a.H;
        const T* src = row + (is_q ? h * a.d : Nq + (h - a.H) * a.d);
        const T* nwgt = static_cast<const T*>(is_q ? a.qnorm : a.knorm);
        float ss = 0.f;
        for (int i = lane; i < a.d; i += 32) { float v = to_f(src[i]); ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        const float inv = nwgt ? 1.f / sqrtf(ss / (float)a.d + a.eps) : 1.f;
        T* dst;
        if (is_q) dst = static_cast<T*>(a.q_out) + (size_t)t * Nq + h * a.d;
        else { if (crow < 0) continue; dst = static_cast<T*>(a.cache_k) + (size_t)crow * Nk + (h - a.H) * a.d; }
        for (int i = lane; i < a.d; i += 32) {
            float v = to_f(src[i]) * inv * (nwgt ? to_f(nwgt[i]) : 1.f);
            if (is_q) v = rnd<T>(v) * temp;
            dst[i] = from_f<T>(v);
        }
    }
    const T* vsrc = row + Nq + Nk;
    T* vf = static_cast<T*>(a.v_first) + (size_t)t * Nv;
    const float lam = a.vmix_mode == 2 ? to_f(*static_cast<const T*>(a.vmix)) : 0.f;
    for (int i = threadIdx.x; i < Nv; i += blockDim.x) {
        float v = to_f(vsrc[i]);
        if (a.vmix_mode == 1) vf[i] = vsrc[i];
        else if (a.vmix_mode == 2) v = (1.f - lam) * v + lam * to_f(vf[i]);
        if (crow >= 0) static_cast<T*>(a.cache_v)[(size_t)crow * Nv + i] = from_f<T>(v);
    }
}

// ------------------------------------------------------------------------------------------------ attention: norm over the whole projection
struct WholeNormPrepArgs {
    const void* qkv;       // [T, H*d + G*d + G*e] projections with bias
    const void* qnorm;     // [H*d] weight of the RMS norm over ALL query entries of a token (not per head)
    const void* knorm;     // [G*d] the same for the keys
    const int* cache_rows; // [T] ring row or -1; null: nothing goes to the ring in this call
    void* q_out;           // [T, H*d]
    void* k_out; void* v_out;   // [T, G*d] / [T, G*e] token-major, or null
    void* ring_k; void* ring_v; // [rows, G, d] / [rows, G, e]
    int Nq, Nk, Nv;
    float eps;
};

// one token per CTA: q <- rms_norm(q) * qnorm and k <- rms_norm(k) * knorm over the whole projections; no rotation
template <typename T>
__global__ void __launch_bounds__(256) whole_norm_prep_kernel(WholeNormPrepArgs a) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    const T* row = static_cast<const T*>(a.qkv) + (size_t)t * (a.Nq + a.Nk + a.Nv);
    const int crow = a.cache_rows ? a.cache_rows[t] : -1;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < a.Nq; i += blockDim.x) { const float v = to_f(row[i]); sq = fmaf(v, v, sq); }
    for (int i = threadIdx.x; i < a.Nk; i += blockDim.x) { const float v = to_f(row[a.Nq + i]); sk = fmaf(v, v, sk); }
    sq = block_sum(sq, red);
    sk = block_sum(sk, red);
    const float iq = 1.f / sqrtf(sq / (float)a.Nq + a.eps), ik = 1.f / sqrtf(sk / (float)a.Nk + a.eps);
    const T* wq = static_cast<const T*>(a.qnorm);
    const T* wk = static_cast<const T*>(a.knorm);
    for (int i = threadIdx.x; i < a.Nq; i += blockDim.x)
        static_cast<T*>(a.q_out)[(size_t)t * a.Nq + i] = from_f<T>(to_f(row[i]) * iq * to_f(wq[i]));
    for (int i = threadIdx.x; i < a.Nk; i += blockDim.x) {
        const T v = from_f<T>(to_f(row[a.Nq + i]) * ik * to_f(wk[i]));
        if (a.k_out) static_cast<T*>(a.k_out)[(size_t)t * a.Nk + i] = v;
        if (crow >= 0) static_cast<T*>(a.ring_k)[(size_t)crow * a.Nk + i] = v;
    }
    const T* vsrc = row + a.Nq + a.Nk;
    for (int i = threadIdx.x; i < a.Nv; i += blockDim.x) {
        if (a.v_out) static_cast<T*>(a.v_out)[(size_t)t * a.Nv + i] = vsrc[i];
        if (crow >= 0) static_cast<T*>(a.ring_v)[(size_t)crow * a.Nv + i] = vsrc[i];
    }
}

// ------------------------------------------------------------------------------------------------ attention core
struct AttnArgs {
    const void* q;          // [T, H*d]
    const void* cache_k; const void* cache_v;
    const float* bias_tab;  // [n_tab, H] additive bias by distance; distances >= n_tab use row n_tab - 1
    int n_tab;
    const int* positions;   // [T]
    const int* q_start;     // [B + 1]
    const int* slots;       // [B] physical cache row block of each sequence
    void* out;              // [T, H*e]
    int T, B, W, H, G, d, e;
    float scale;
    int splits;             // CTAs per (token, head) along the keys; > 1: partial (max, sum, acc) go to `scratch`
    float* scratch;         // [T*H, splits, 2 + e] fp32
    int k_pitch, v_pitch;   // elements per ring row of keys / values; 0: G*d / G*e.  (A latent ring is one row per token that both
                            // pointers address: its first e entries are the value.)  bias_tab may be null: no bias.
    int window;             // > 0: a token at position p sees keys p - window + 1 .. p only (sliding window); 0: every key up to p
    const void* own_k; const void* own_v;  // prompts over a ring shorter than the sequence: keys / values of THIS call's tokens, token-major
                            // [T, G*d] / [T, G*e]; key j >= seqpos[b] is row q_start[b] + j - seqpos[b] there, older keys are in the ring
                            // (which this call's tokens are written to only after attention).  null: every key is in the ring.
    const int* seqpos;      // [B] tokens cached before this call (with own_k)
    int chunk;              // keys per warp and step, at most AT_CHUNK (0: AT_CHUNK).  A short ring read by few (token, head) pairs -- a decode
                            // step of a small batch over a sliding window -- is spread over more CTAs with a smaller chunk
    int sigmoid;            // 1: the weight of a visible key is sigmoid(score), not normalised over the keys (no softmax): partial results
                            // simply add, so the running maximum stays 0 and the sum is never divided by
};

// where key / value j of a sequence lives: this call's own rows, or the ring
template <typename T>
struct KeySource {
    const T* ring; const T* own; size_t ring_pitch, own_pitch; int W, own_from;
    __device__ __forceinline__ const T* row(int j) const {
        return j >= own_from ? own + (size_t)(j - own_from) * own_pitch : ring + (size_t)(j % W) * ring_pitch;
    }
};

constexpr int AT_WARPS = 4, AT_CHUNK = 128, AT_MAXR = 8, AT_MAXR_WIDE = 16;  // e <= 32 * MAXR

// `splits` CTAs per (token, head); their warps take alternate chunks of AT_CHUNK keys (scores: lanes over keys, a whole key row
// per lane; values: every lane owns ceil(e / 32) adjacent value columns) with a running (max, sum); the warps' partial results
// are merged through shared memory, the CTAs' (decode: few queries, long contexts) by attn_merge_kernel.
template <typename T, int MAXR = AT_MAXR>
__global__ void __launch_bounds__(AT_WARPS * 32) attn_bias_kernel(AttnArgs a) {
    extern __shared__ __align__(16) float sm[];
    const int t = blockIdx.x / a.H, h = blockIdx.x % a.H, g = h / (a.H / a.G);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* qs = sm;                                  // [d]
    float* sc = sm + a.d + warp * AT_CHUNK;          // [AT_CHUNK] per warp
    float* mrg = sm + a.d + AT_WARPS * AT_CHUNK;     // [AT_WARPS][2 + 32 * MAXR]
    int b = 0;
    while (b + 1 < a.B && a.q_start[b + 1] <= t) ++b;
    const int pos = a.positions[t], n = pos + 1;
    const T* q = static_cast<const T*>(a.q) + ((size_t)t * a.H + h) * a.d;
    for (int i = threadIdx.x; i < a.d; i += blockDim.x) qs[i] = to_f(q[i]) * a.scale;
    __syncthreads();
    const size_t base = (size_t)a.slots[b] * a.W;
    const size_t ks = a.k_pitch ? (size_t)a.k_pitch : (size_t)a.G * a.d, vs = a.v_pitch ? (size_t)a.v_pitch : (size_t)a.G * a.e;
    const int own_from = a.own_k ? a.seqpos[b] : 0x7fffffff;
    const size_t own_row = a.own_k ? (size_t)a.q_start[b] : 0;
    const KeySource<T> Ksrc{static_cast<const T*>(a.cache_k) + base * ks + (size_t)g * a.d,
                            static_cast<const T*>(a.own_k) + own_row * a.G * a.d + (size_t)g * a.d, ks, (size_t)a.G * a.d, a.W, own_from};
    const KeySource<T> Vsrc{static_cast<const T*>(a.cache_v) + base * vs + (size_t)g * a.e,
                            static_cast<const T*>(a.own_v) + own_row * a.G * a.e + (size_t)g * a.e, vs, (size_t)a.G * a.e, a.W, own_from};
    constexpr int V = Vec<T>::N;
    const bool vec_ok = (a.d % V == 0) && (ks % V == 0) && (reinterpret_cast<uintptr_t>(a.cache_k) % 16 == 0)
                        && (!a.own_k || reinterpret_cast<uintptr_t>(a.own_k) % 16 == 0);
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;  // first visible key
    float m = a.sigmoid ? 0.f : -INFINITY, l = 0.f, acc[MAXR];
#pragma unroll
    for (int r = 0; r < MAXR; ++r) acc[r] = 0.f;
    const int cpl = (a.e + 31) / 32;  // value columns per lane: lane * cpl .. + cpl - 1
    const int CH = a.chunk > 0 ? a.chunk : AT_CHUNK;
    for (int c0 = lo + (blockIdx.y * AT_WARPS + warp) * CH; c0 < n; c0 += a.splits * AT_WARPS * CH) {
        const int cn = min(CH, n - c0);
        float cmax = -INFINITY;
        for (int jj = lane; jj < cn; jj += 32) {
            const int j = c0 + jj;
            const T* kr = Ksrc.row(j);
            float s = 0.f;
            if (vec_ok) {
                for (int i = 0; i < a.d; i += V) {
                    float kv[V];
                    Vec<T>::load(kr + i, kv);
#pragma unroll
                    for (int u = 0; u < V; u += 4) {  // q from shared memory four at a time (qs is 16-byte aligned, i % 4 == 0)
                        const float4 q4 = *reinterpret_cast<const float4*>(qs + i + u);
                        s = fmaf(q4.x, kv[u], s); s = fmaf(q4.y, kv[u + 1], s); s = fmaf(q4.z, kv[u + 2], s); s = fmaf(q4.w, kv[u + 3], s);
                    }
                }
            } else {
                for (int i = 0; i < a.d; ++i) s = fmaf(qs[i], to_f(kr[i]), s);
            }
            if (a.bias_tab) s += a.bias_tab[(size_t)min(pos - j, a.n_tab - 1) * a.H + h];
            sc[jj] = s;
            cmax = fmaxf(cmax, s);
        }
        cmax = warp_max(cmax);
        const float m_new = a.sigmoid ? 0.f : fmaxf(m, cmax);
        const float corr = a.sigmoid ? 1.f : (m == -INFINITY) ? 0.f : expf(m - m_new);
        float psum = 0.f;
        for (int jj = lane; jj < cn; jj += 32) { float p = a.sigmoid ? sigmoid_exact(sc[jj]) : expf(sc[jj] - m_new); sc[jj] = p; psum += p; }
        psum = warp_sum(psum);
        l = l * corr + psum;
        m = m_new;
        __syncwarp();
#pragma unroll
        for (int r = 0; r < MAXR; ++r) acc[r] *= corr;
        {
            const int vo = lane * cpl;
            int jj = 0;
            for (; jj + 4 <= cn; jj += 4) {
                const T* r0 = Vsrc.row(c0 + jj) + vo;
                const T* r1 = Vsrc.row(c0 + jj + 1) + vo;
                const T* r2 = Vsrc.row(c0 + jj + 2) + vo;
                const T* r3 = Vsrc.row(c0 + jj + 3) + vo;
                const float w0 = sc[jj], w1 = sc[jj + 1], w2 = sc[jj + 2], w3 = sc[jj + 3];
#pragma unroll
                for (int r = 0; r < MAXR; ++r)
                    if (r < cpl && lane * cpl + r < a.e)
                        acc[r] += w0 * to_f(r0[r]) + w1 * to_f(r1[r]) + w2 * to_f(r2[r]) + w3 * to_f(r3[r]);
            }
            for (; jj < cn; ++jj) {
                const T* r0 = Vsrc.row(c0 + jj) + vo;
                const float w0 = sc[jj];
#pragma unroll
                for (int r = 0; r < MAXR; ++r)
                    if (r < cpl && lane * cpl + r < a.e) acc[r] = fmaf(w0, to_f(r0[r]), acc[r]);
            }
        }
        __syncwarp();
    }
    // merge the warps
    float* mine = mrg + warp * (2 + 32 * MAXR);
    if (lane == 0) { mine[0] = m; mine[1] = l; }
#pragma unroll
    for (int r = 0; r < MAXR; ++r) mine[2 + r * 32 + lane] = acc[r];
    __syncthreads();
    if (warp == 0) {
        float M = -INFINITY;
        for (int w = 0; w < AT_WARPS; ++w) M = fmaxf(M, mrg[w * (2 + 32 * MAXR)]);
        float L = 0.f, o[MAXR];
#pragma unroll
        for (int r = 0; r < MAXR; ++r) o[r] = 0.f;
        for (int w = 0; w < AT_WARPS; ++w) {
            const float* p = mrg + w * (2 + 32 * MAXR);
            if (p[0] == -INFINITY) continue;
            const float f = expf(p[0] - M);
            L += p[1] * f;
#pragma unroll
            for (int r = 0; r < MAXR; ++r) o[r] = fmaf(p[2 + r * 32 + lane], f, o[r]);
        }
        if (a.splits > 1) {
            float* part = a.scratch + ((size_t)blockIdx.x * a.splits + blockIdx.y) * (2 + a.e);
            if (lane == 0) { part[0] = M; part[1] = L; }
#pragma unroll
            for (int r = 0; r < MAXR; ++r)
                if (r < cpl && lane * cpl + r < a.e) part[2 + lane * cpl + r] = o[r];
        } else {
            T* out = static_cast<T*>(a.out) + ((size_t)t * a.H + h) * a.e;
#pragma unroll
            for (int r = 0; r < MAXR; ++r)
                if (r < cpl && lane * cpl + r < a.e) out[lane * cpl + r] = from_f<T>(a.sigmoid ? o[r] : o[r] / L);
        }
    }
}

// out[t, h, :] from the `splits` (at most AT_MAX_SPLITS) partial results of attn_bias_kernel: the splits' weights exp(m_s - M) are
// computed once into shared memory, then every thread sums ONE value column over the splits (coalesced over the columns, four
// loads in flight).  grid (token * head, blocks of blockDim columns)
constexpr int AT_MAX_SPLITS = 64;
template <typename T>
__global__ void attn_merge_kernel(const float* __restrict__ scratch, T* __restrict__ out, int splits, int e, int sigmoid = 0) {
    __shared__ float f[AT_MAX_SPLITS];
    __shared__ float red[32];
    const float* part = scratch + (size_t)blockIdx.x * splits * (2 + e);
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, part[(size_t)s * (2 + e)]);
    float lpart = 0.f;
    for (int s = threadIdx.x; s < splits; s += blockDim.x) {
        const float m = part[(size_t)s * (2 + e)];
        const float w = (m == -INFINITY) ? 0.f : expf(m - M);
        f[s] = w;
        lpart += w * part[(size_t)s * (2 + e) + 1];
    }
    const float L = sigmoid ? 1.f : block_sum(lpart, red);  // its barriers also publish f[]
    if (sigmoid) __syncthreads();
    const int c = blockIdx.y * blockDim.x + threadIdx.x;
    if (c >= e) return;
    const float* col = part + 2 + c;
    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
    int s = 0;
    for (; s + 4 <= splits; s += 4) {
        o0 = fmaf(col[(size_t)s * (2 + e)], f[s], o0);
        o1 = fmaf(col[(size_t)(s + 1) * (2 + e)], f[s + 1], o1);
        o2 = fmaf(col[(size_t)(s + 2) * (2 + e)], f[s + 2], o2);
        o3 = fmaf(col[(size_t)(s + 3) * (2 + e)], f[s + 3], o3);
    }
    for (; s < splits; ++s) o0 = fmaf(col[(size_t)s * (2 + e)], f[s], o0);
    out[(size_t)blockIdx.x * e + c] = from_f<T>(((o0 + o1) + (o2 + o3)) / L);
}

// ------------------------------------------------------------------------------------------------ lightning attention
struct LightningArgs {
    const void* qkvg;      // [T, 2*H*d + 2*H*e]: q | k | v (activated) | g
    float* state;          // [slots, H, d, e] fp32
    const float* decay;    // [H]
    const int* q_start;    // [B + 1]
    const int* seqpos;     // [B] tokens before this call (0: the state starts at zero)
    const int* slots;      // [B]
    float* o;              // [T, H*e] fp32
    int B, H, d, e;
};

constexpr int LS_TB = 16, LS_THREADS = 128;

// One CTA of LS_THREADS threads per (sequence, head, block of LS_THREADS value columns); thread c owns column c of the state:
// DMAX registers.  Keys and queries of LS_TB tokens at a time go through shared memory; the next LS_TB tokens are fetched into
// registers while the current ones are consumed, so the scan does not wait for global memory.  Sequential in t, exact in fp32.
template <typename T, int DMAX>
__global__ void __launch_bounds__(LS_THREADS) lightning_scan_kernel(LightningArgs a) {
    constexpr int R = 2 * LS_TB * DMAX / LS_THREADS;  // staged values per thread and tile
    __shared__ __align__(16) float ks[LS_TB][DMAX], qs[LS_TB][DMAX];
    const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
    const int c = blockIdx.y * LS_THREADS + threadIdx.x;
    const bool live = c < a.e;
    const int t0 = a.q_start[b], t1 = a.q_start[b + 1];
    const int stride = 2 * a.H * a.d + 2 * a.H * a.e;
    const T* X = static_cast<const T*>(a.qkvg);
    float* st = a.state + (((size_t)a.slots[b] * a.H + h) * a.d) * a.e;
    const float dec = a.decay[h];
    float S[DMAX], pre[R];
    const bool fresh = a.seqpos[b] == 0;
#pragma unroll
    for (int i = 0; i < DMAX; ++i) S[i] = (live && !fresh && i < a.d) ? st[(size_t)i * a.e + c] : 0.f;

    auto fetch = [&](int tb) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int idx = threadIdx.x + r * LS_THREADS;
            const int tt = idx / (2 * DMAX), rem = idx % (2 * DMAX), which = rem / DMAX, i = rem % DMAX;
            const bool ok = tb + tt < t1 && i < a.d;
            pre[r] = ok ? to_f(X[(size_t)(tb + tt) * stride + (which ? a.H * a.d : 0) + h * a.d + i]) : 0.f;
        }
    };
    fetch(t0);
    for (int tb = t0; tb < t1; tb += LS_TB) {
        const int nt = min(LS_TB, t1 - tb);
        __syncthreads();
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int idx = threadIdx.x + r * LS_THREADS;
            const int tt = idx / (2 * DMAX), rem = idx % (2 * DMAX), which = rem / DMAX, i = rem % DMAX;
            (which ? ks : qs)[tt][i] = pre[r];
        }
        __syncthreads();
        if (tb + LS_TB < t1) fetch(tb + LS_TB);
        if (live) {
            const T* vcol = X + 2 * a.H * a.d + h * a.e + c;
            float vn = to_f(vcol[(size_t)tb * stride]);
            for (int tt = 0; tt < nt; ++tt) {
                const float v = vn;
                if (tt + 1 < nt) vn = to_f(vcol[(size_t)(tb + tt + 1) * stride]);  // in flight while this token is consumed
                float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;  // four chains: the sum over i is not one dependent chain of DMAX FMAs
#pragma unroll
                for (int i = 0; i < DMAX; i += 4) {
                    const float4 k4 = *reinterpret_cast<const float4*>(&ks[tt][i]);
                    const float4 q4 = *reinterpret_cast<const float4*>(&qs[tt][i]);
                    S[i] = fmaf(dec, S[i], k4.x * v);         o0 = fmaf(S[i], q4.x, o0);
                    S[i + 1] = fmaf(dec, S[i + 1], k4.y * v); o1 = fmaf(S[i + 1], q4.y, o1);
                    S[i + 2] = fmaf(dec, S[i + 2], k4.z * v); o2 = fmaf(S[i + 2], q4.z, o2);
                    S[i + 3] = fmaf(dec, S[i + 3], k4.w * v); o3 = fmaf(S[i + 3], q4.w, o3);
                }
                a.o[(size_t)(tb + tt) * a.H * a.e + h * a.e + c] = (o0 + o1) + (o2 + o3);
            }
        }
    }
    if (live) {
#pragma unroll
        for (int i = 0; i < DMAX; ++i)
            if (i < a.d) st[(size_t)i * a.e + c] = S[i];
    }
}

// y[t, :] = o[t, :] / sqrt(mean(o[t]^2) + eps) * w * sigmoid(g[t, :]); g lives at column `g_off` of rows of pitch `g_pitch`
template <typename T>
__global__ void gated_headnorm_kernel(const float* __restrict__ o, const T* __restrict__ w, const T* __restrict__ g, int g_pitch, int g_off,
                                      T* __restrict__ y, int N, float eps) {
    __shared__ float red[32];
    const float* r = o + (size_t)blockIdx.x * N;
    const T* gr = g + (size_t)blockIdx.x * g_pitch + g_off;
    float ss = 0.f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) ss = fmaf(r[i], r[i], ss);
    ss = block_sum(ss, red);
    const float inv = 1.f / sqrtf(ss / (float)N + eps);
    for (int i = threadIdx.x; i < N; i += blockDim.x)
        y[(size_t)blockIdx.x * N + i] = from_f<T>(r[i] * inv * to_f(w[i]) * sigmoid_exact(to_f(gr[i])));
}

}  // namespace mbh
