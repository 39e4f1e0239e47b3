// Linear attention with data-dependent gates: one scan kernel for every recurrence of the form
//
//     S_t = diag(a_t) S_(t-1) + b_t v_t^T,    o_t = S_t^T q_t          per head, S [d, e] fp32, carried in the cache
//
// and the small kernels that turn a layer's projections into (q, a, b) and its raw output into the next Linear's input.
//
//   gated_scan       the recurrence; with `ones` the state has one more column whose value is 1 for every token: the normaliser
//                    n_t = a_t n_(t-1) + b_t.  It does not get a thread column of its own (at 128 value columns that would be a second
//                    CTA with one live thread): thread i of the first column block carries n[i] beside its state column and writes
//                    n_t[i] q_t[i] per token; scan_post sums them to n_t . q_t
//                    Long prompts run chunk-parallel, still exactly this recurrence in fp32: every chunk of `chunk_len` tokens first
//                    runs from a zero state (GS_LOCAL: its own contribution L_c), chunk_decay multiplies each channel's a_t over the
//                    chunk (A_c), scan_combine walks the chunks in order, S_c = A_c S_(c-1) + L_c, leaving each chunk's START state
//                    in the scratch and the last one in the cache, and the chunks then run again from their start states for the
//                    outputs (GS_OUTPUT).  Twice the arithmetic on chunk-count times the CTAs.
//   hgrn2_gates      f = l + (1 - l) sigmoid(f_pre): a = f, b = 1 - f (the forget gate also decides what is written)
//   mlstm_m / mlstm_qab   exponential input and forget gates kept in range by a running maximum m (m_0 = 0):
//                    i = cap tanh(i_pre / cap), f = logsigmoid(cap tanh(f_pre / cap)), m_t = max(f + m_(t-1), i),
//                    a = exp(f + m_(t-1) - m_t) (one number per head), b = exp(i - m_t) k, q scaled; also exp(-m_t) per token
//   retention_qab    a fixed decay per head and rotated queries and keys: the first rot_dims entries of each head turn by
//                    position * freq[i], entry i paired with entry i + rot_dims / 2; a = decay[h], b = rotated k * kscale
//   gla_qab          a decay per key channel from a projection z: a = sigmoid(z)^(1 / tau) = exp(logsigmoid(z) / tau), q scaled, b = k
//   scan_post        o / (max(|n . q|, exp(-m)) + 1e-6) when there is a normaliser; every head divided by its root mean square;
//                    times a weight (per head column, one set shared by the heads, or none) and an optional gate (sigmoid or SiLU)
//
// Everything here is fp32 except the projections that are read and the activations that are written.
#pragma once
#include "hybrid_common.cuh"

namespace mbh {

struct GatedScanArgs {
    const float* qab;      // [T, 3, H*d]: q | a | b
    const void* v;         // storage type: value (t, h, c) at v[t * v_pitch + v_off + h*e + c]
    int v_pitch, v_off;
    float* state;          // [slots, state_stride]; head h's matrix [d, e + ones] starts at h * d * (e + ones)
    int state_stride;
    const int* q_start;    // [B + 1]
    const int* seqpos;     // [B] tokens before this call (0: the state starts at zero)
    const int* slots;      // [B]
    float* o;              // [T, H * e]
    float* nq;             // with `ones`: [T, H * d], n_t[i] * q_t[i]
    int B, H, d, e, ones;
    int chunk_len;         // chunk-parallel modes: tokens per chunk (blockIdx.z is the chunk); whole mode: unused
    float* scratch;        // [B*H, chunks, d, e + ones] chunk-local states, then chunk start states
    float* aprod;          // [B*H, chunks, d] product of a_t over each chunk
    int key_blocks;        // key sizes above 128: the keys are split into blocks of 128 over CTAs (grid.y = column blocks * key_blocks),
                           // whose partial outputs are summed into a zeroed o with atomic adds
};

enum { GS_WHOLE = 0, GS_LOCAL = 1, GS_OUTPUT = 2 };

constexpr int GS_THREADS = 128;

// One CTA per (sequence, head, block of GS_THREADS state columns); thread c owns column c of the state in DMAX registers.
// q, a, b of GS_TB tokens at a time go through shared memory, the next tile is fetched into registers meanwhile (fewer tokens
// per tile at the largest key size, where the state alone takes 128 registers, and fewer again with the normaliser).
template <typename T, int DMAX, int GS_TB, int MODE, bool ONES, bool SPLIT = false>
__global__ void __launch_bounds__(GS_THREADS) gated_scan_kernel(GatedScanArgs p) {
    constexpr int R = 3 * GS_TB * DMAX / GS_THREADS;
    __shared__ __align__(16) float qs[GS_TB][DMAX], as[GS_TB][DMAX], bs[GS_TB][DMAX];
    const int b = blockIdx.x / p.H, h = blockIdx.x % p.H;
    // SPLIT (key sizes above DMAX): this CTA's keys are i0 .. i0 + DMAX - 1, its outputs partial sums
    const int ncb = SPLIT ? gridDim.y / p.key_blocks : gridDim.y, i0 = SPLIT ? (blockIdx.y / ncb) * DMAX : 0;
    const int c = (blockIdx.y % ncb) * GS_THREADS + threadIdx.x;
    const int ec = p.e + p.ones;
    const bool live = c < p.e;
    // the normaliser entry this thread carries: key i0 + threadIdx.x, in the first column block only
    const bool nrm = ONES && (blockIdx.y % ncb) == 0 && threadIdx.x < DMAX && i0 + (int)threadIdx.x < p.d;
    int t0 = p.q_start[b], t1 = p.q_start[b + 1];
    const int Hd = p.H * p.d;
    float* st = p.state + (size_t)p.slots[b] * p.state_stride + (size_t)h * p.d * ec;
    if (MODE != GS_WHOLE) {  // this CTA's chunk of the sequence; its state lives in the scratch
        t0 += blockIdx.z * p.chunk_len;
        t1 = min(t1, t0 + p.chunk_len);
        if (t0 >= t1) return;
        st = p.scratch + ((size_t)blockIdx.x * gridDim.z + blockIdx.z) * p.d * ec;
    }
    float S[DMAX], pre[R];
    const bool fresh = MODE == GS_LOCAL || (MODE == GS_WHOLE && p.seqpos[b] == 0);
#pragma unroll
    for (int i = 0; i < DMAX; ++i) S[i] = (live && !fresh && i0 + i < p.d) ? st[(size_t)(i0 + i) * ec + c] : 0.f;
    float nst = (nrm && !fresh) ? st[(size_t)(i0 + threadIdx.x) * ec + p.e] : 0.f;

    auto fetch = [&](int tb) {
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int idx = threadIdx.x + r * GS_THREADS;
            const int tt = idx / (3 * DMAX), rem = idx % (3 * DMAX), which = rem / DMAX, i = rem % DMAX;
            const bool ok = tb + tt < t1 && i0 + i < p.d;
            pre[r] = ok ? p.qab[((size_t)(tb + tt) * 3 + which) * Hd + h * p.d + i0 + i] : 0.f;
        }
    };
    fetch(t0);
    const T* vcol = static_cast<const T*>(p.v) + p.v_off + h * p.e + (live ? c : 0);
    for (int tb = t0; tb < t1; tb += GS_TB) {
        const int nt = min(GS_TB, t1 - tb);
        __syncthreads();
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const int idx = threadIdx.x + r * GS_THREADS;
            const int tt = idx / (3 * DMAX), rem = idx % (3 * DMAX), which = rem / DMAX, i = rem % DMAX;
            (which == 0 ? qs : which == 1 ? as : bs)[tt][i] = pre[r];
        }
        __syncthreads();
        if (tb + GS_TB < t1) fetch(tb + GS_TB);
        if (ONES && nrm) {
            const int i = threadIdx.x % DMAX;  // = threadIdx.x; the modulo keeps the shared-memory index in range for the compiler
            for (int tt = 0; tt < nt; ++tt) {
                nst = fmaf(as[tt][i], nst, bs[tt][i]);
                if (MODE != GS_LOCAL) p.nq[(size_t)(tb + tt) * Hd + h * p.d + i0 + i] = nst * qs[tt][i];
            }
        }
        if (live) {
            float vn = to_f(vcol[(size_t)tb * p.v_pitch]);
            for (int tt = 0; tt < nt; ++tt) {
                const float v = vn;
                if (tt + 1 < nt) vn = to_f(vcol[(size_t)(tb + tt + 1) * p.v_pitch]);
                float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
                for (int i = 0; i < DMAX; i += 4) {
                    const float4 a4 = *reinterpret_cast<const float4*>(&as[tt][i]);
                    const float4 b4 = *reinterpret_cast<const float4*>(&bs[tt][i]);
                    const float4 q4 = *reinterpret_cast<const float4*>(&qs[tt][i]);
                    S[i] = fmaf(a4.x, S[i], b4.x * v);         o0 = fmaf(S[i], q4.x, o0);
                    S[i + 1] = fmaf(a4.y, S[i + 1], b4.y * v); o1 = fmaf(S[i + 1], q4.y, o1);
                    S[i + 2] = fmaf(a4.z, S[i + 2], b4.z * v); o2 = fmaf(S[i + 2], q4.z, o2);
                    S[i + 3] = fmaf(a4.w, S[i + 3], b4.w * v); o3 = fmaf(S[i + 3], q4.w, o3);
                }
                if (MODE != GS_LOCAL) {
                    float* dst = &p.o[(size_t)(tb + tt) * p.H * p.e + h * p.e + c];
                    if (SPLIT) atomicAdd(dst, (o0 + o1) + (o2 + o3));
                    else *dst = (o0 + o1) + (o2 + o3);
                }
            }
        }
    }
    // the state goes back through a pointer the compiler cannot see before this point: otherwise it computes the DMAX store addresses
    // ahead of the token loop and keeps them in registers beside the state (spills at 128 keys)
    asm volatile("" : "+l"(st));
    if (live && MODE != GS_OUTPUT) {
#pragma unroll
        for (int i = 0; i < DMAX; ++i)
            if (i0 + i < p.d) st[(size_t)(i0 + i) * ec + c] = S[i];
    }
    if (ONES && nrm && MODE != GS_OUTPUT) st[(size_t)(i0 + threadIdx.x) * ec + p.e] = nst;
}

// aprod[(b, h), chunk, i] = product of a_t[h, i] over the chunk's tokens.  grid (B*H, chunks), threads over i
__global__ void chunk_decay_kernel(GatedScanArgs p) {
    const int b = blockIdx.x / p.H, h = blockIdx.x % p.H;
    const int t0 = p.q_start[b] + blockIdx.y * p.chunk_len, t1 = min(p.q_start[b + 1], t0 + p.chunk_len);
    const int Hd = p.H * p.d;
    for (int i = threadIdx.x; i < p.d; i += blockDim.x) {
        float a0 = 1.f, a1 = 1.f;
        int t = t0;
        for (; t + 1 < t1; t += 2) {
            a0 *= p.qab[((size_t)t * 3 + 1) * Hd + h * p.d + i];
            a1 *= p.qab[((size_t)(t + 1) * 3 + 1) * Hd + h * p.d + i];
        }
        if (t < t1) a0 *= p.qab[((size_t)t * 3 + 1) * Hd + h * p.d + i];
        p.aprod[((size_t)blockIdx.x * gridDim.y + blockIdx.y) * p.d + i] = a0 * a1;
    }
}

// One thread per state element (i, column): walks the sequence's chunks in order, S <- A_c[i] S + L_c, replacing L_c in the scratch
// by the state the chunk STARTS from and writing the last state to the cache.  grid (B*H, ceil(d * ec / blockDim)), `chunks` = grid.z
// of the scan launches
__global__ void scan_combine_kernel(GatedScanArgs p, int chunks) {
    const int b = blockIdx.x / p.H, h = blockIdx.x % p.H, ec = p.e + p.ones;
    const int idx = blockIdx.y * blockDim.x + threadIdx.x;
    if (idx >= p.d * ec) return;
    const int i = idx / ec;
    const int len = p.q_start[b + 1] - p.q_start[b], n = (len + p.chunk_len - 1) / p.chunk_len;
    float* st = p.state + (size_t)p.slots[b] * p.state_stride + (size_t)h * p.d * ec + idx;
    float S = p.seqpos[b] == 0 ? 0.f : *st;
    for (int c = 0; c < n; ++c) {
        float* L = p.scratch + ((size_t)blockIdx.x * chunks + c) * p.d * ec + idx;
        const float l = *L;
        *L = S;
        S = fmaf(p.aprod[((size_t)blockIdx.x * chunks + c) * p.d + i], S, l);
    }
    if (n > 0) *st = S;
}

// ------------------------------------------------------------------------------------------------ HGRN2 gates
struct Hgrn2GateArgs {
    const void* qfv;     // [T, 2*H*d + H*e]: silu(q) | f_pre (bias added) | v
    const void* lower;   // [H*d] lower bound of the forget gate
    float* qab;          // [T, 3, H*d]
    int Hd, pitch;
};

template <typename T>
__global__ void hgrn2_gates_kernel(Hgrn2GateArgs p) {
    const int t = blockIdx.x;  // grid (T, blocks of blockDim entries): a decode step has few tokens but thousands of entries
    const T* row = static_cast<const T*>(p.qfv) + (size_t)t * p.pitch;
    float* out = p.qab + (size_t)t * 3 * p.Hd;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < p.Hd; j += gridDim.y * blockDim.x) {
        const float l = to_f(static_cast<const T*>(p.lower)[j]);
        const float f = l + (1.f - l) * sigmoid_exact(to_f(row[p.Hd + j]));
        out[j] = to_f(row[j]);
        out[p.Hd + j] = f;
        out[2 * p.Hd + j] = 1.f - f;
    }
}

// ------------------------------------------------------------------------------------------------ mLSTM gates
struct MlstmGateArgs {
    const void* qkvg;    // [T, pitch]: q | k | v | g
    const float* gif;    // [T, 2H] fp32: i_pre | f_pre (bias added)
    float* gates;        // [T, H, 3]: a (decay), s (input scale), exp(-m_t)
    float* qab;          // [T, 3, H*d]
    float* state;        // m of head h of a sequence at state[slot * state_stride + m_off + h]
    int state_stride, m_off;
    const int* q_start; const int* seqpos; const int* slots;
    int H, d, pitch;
    float cap, qscale;
};

__device__ __forceinline__ float logsigmoid_exact(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// One warp per (sequence, head): lanes take 32 tokens' gates at a time, the running maximum goes through them in order.
template <typename T>
__global__ void __launch_bounds__(32) mlstm_m_kernel(MlstmGateArgs p) {
    const int b = blockIdx.x / p.H, h = blockIdx.x % p.H, lane = threadIdx.x;
    const int t0 = p.q_start[b], t1 = p.q_start[b + 1];
    float* mst = p.state + (size_t)p.slots[b] * p.state_stride + p.m_off + h;
    float m = p.seqpos[b] == 0 ? 0.f : *mst;
    const float* G = p.gif;
    for (int tb = t0; tb < t1; tb += 32) {
        const int t = tb + lane;
        float ig = 0.f, fg = 0.f;
        if (t < t1) {
            ig = p.cap * tanhf(G[(size_t)t * 2 * p.H + h] / p.cap);
            fg = logsigmoid_exact(p.cap * tanhf(G[(size_t)t * 2 * p.H + p.H + h] / p.cap));
        }
        float m_prev = 0.f, m_mine = 0.f;
        const int nt = min(32, t1 - tb);
        for (int s = 0; s < nt; ++s) {
            const float fs = __shfl_sync(0xffffffffu, fg, s), is = __shfl_sync(0xffffffffu, ig, s);
            const float mn = fmaxf(fs + m, is);
            if (lane == s) { m_prev = m; m_mine = mn; }
            m = mn;
        }
        if (t < t1) {
            float* g = p.gates + ((size_t)t * p.H + h) * 3;
            g[0] = expf(fg + m_prev - m_mine);
            g[1] = expf(ig - m_mine);
            g[2] = expf(-m_mine);
        }
    }
    if (lane == 0) *mst = m;
}

template <typename T>
__global__ void mlstm_qab_kernel(MlstmGateArgs p) {
    const int t = blockIdx.x, Hd = p.H * p.d;
    const T* row = static_cast<const T*>(p.qkvg) + (size_t)t * p.pitch;
    float* out = p.qab + (size_t)t * 3 * Hd;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < Hd; j += gridDim.y * blockDim.x) {
        const float* g = p.gates + ((size_t)t * p.H + j / p.d) * 3;
        out[j] = to_f(row[j]) * p.qscale;
        out[Hd + j] = g[0];
        out[2 * Hd + j] = g[1] * to_f(row[Hd + j]);
    }
}

// ------------------------------------------------------------------------------------------------ retention and GLA gates
struct RetentionQabArgs {
    const void* qk;        // [T, pitch]: q (H*d) | k (H*d) | ...
    const double* freq;    // [rot_dims / 2]
    const float* decay;    // [H]
    const int* positions;  // [T]
    float* qab;            // [T, 3, H*d]
    int H, d, pitch, rot_dims;
    float kscale;
};

// grid (T, blocks of blockDim entries); a thread per (head, entry of the first half of the rotated part or unrotated entry)
template <typename T>
__global__ void retention_qab_kernel(RetentionQabArgs p) {
    const int t = blockIdx.x, Hd = p.H * p.d, half = p.rot_dims >> 1;
    const T* row = static_cast<const T*>(p.qk) + (size_t)t * p.pitch;
    float* out = p.qab + (size_t)t * 3 * Hd;
    const int pos = p.positions[t];
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < Hd; j += gridDim.y * blockDim.x) {
        const int h = j / p.d, i = j % p.d;
        out[Hd + j] = p.decay[h];
        if (i >= p.rot_dims) {
            out[j] = to_f(row[j]);
            out[2 * Hd + j] = to_f(row[Hd + j]) * p.kscale;
        } else if (i < half) {
            double sn, cs;
            sincos((double)pos * p.freq[i], &sn, &cs);
            const float c = (float)cs, s = (float)sn;
            const float qu = to_f(row[j]), qv = to_f(row[j + half]), ku = to_f(row[Hd + j]), kv = to_f(row[Hd + j + half]);
            out[j] = qu * c - qv * s;
            out[j + half] = qv * c + qu * s;
            out[2 * Hd + j] = (ku * c - kv * s) * p.kscale;
            out[2 * Hd + j + half] = (kv * c + ku * s) * p.kscale;
        }
    }
}

struct GlaQabArgs {
    const void* qk;        // [T, pitch]: q (H*d) | k (H*d) | ...
    const float* z;        // [T, H*d] fp32 decay projection (bias added)
    float* qab;            // [T, 3, H*d]
    int Hd, pitch;
    float qscale, inv_tau;
};

template <typename T>
__global__ void gla_qab_kernel(GlaQabArgs p) {
    const int t = blockIdx.x;
    const T* row = static_cast<const T*>(p.qk) + (size_t)t * p.pitch;
    float* out = p.qab + (size_t)t * 3 * p.Hd;
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < p.Hd; j += gridDim.y * blockDim.x) {
        out[j] = to_f(row[j]) * p.qscale;
        out[p.Hd + j] = expf(logsigmoid_exact(p.z[(size_t)t * p.Hd + j]) * p.inv_tau);
        out[2 * p.Hd + j] = to_f(row[p.Hd + j]);
    }
}

// ------------------------------------------------------------------------------------------------ after the scan
struct ScanPostArgs {
    const float* o;        // [T, H * e]
    const float* nq;       // with `ones`: [T, H * d], summed over d to n_t . q_t
    int d;
    const float* gates;    // [T, H, 3] (exp(-m_t) in entry 2) with `ones`, else null
    const void* w;         // weight: [H*e] (w_per_head) or [e] shared by the heads; null: none
    int w_per_head;
    const void* gate;      // gate at gate[t * g_pitch + g_off + h*e + c], or null
    int g_pitch, g_off;
    int gate_act;          // 0: times sigmoid(gate); 1: times gate * sigmoid(gate)
    void* y;               // [T, H*e]
    int H, e, ones;
    float eps;
};

// grid (T, groups of heads), a warp per head
template <typename T>
__global__ void __launch_bounds__(128) scan_post_kernel(ScanPostArgs p) {
    const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    for (int h = blockIdx.y * nw + warp; h < p.H; h += gridDim.y * nw) {
        const float* o = p.o + ((size_t)t * p.H + h) * p.e;
        float den = 1.f;
        if (p.ones) {
            float nq = 0.f;
            for (int i = lane; i < p.d; i += 32) nq += p.nq[((size_t)t * p.H + h) * p.d + i];
            den = fmaxf(fabsf(warp_sum(nq)), p.gates[((size_t)t * p.H + h) * 3 + 2]) + 1e-6f;
        }
        float ss = 0.f;
        for (int c = lane; c < p.e; c += 32) { const float v = o[c] / den; ss = fmaf(v, v, ss); }
        ss = warp_sum(ss);
        const float inv = 1.f / sqrtf(ss / (float)p.e + p.eps);
        const T* w = p.w ? static_cast<const T*>(p.w) + (p.w_per_head ? h * p.e : 0) : nullptr;
        const T* g = p.gate ? static_cast<const T*>(p.gate) + (size_t)t * p.g_pitch + p.g_off + h * p.e : nullptr;
        T* y = static_cast<T*>(p.y) + ((size_t)t * p.H + h) * p.e;
        for (int c = lane; c < p.e; c += 32) {
            float v = o[c] / den * inv * (w ? to_f(w[c]) : 1.f);
            if (g) { const float gv = to_f(g[c]); v *= p.gate_act ? gv * sigmoid_exact(gv) : sigmoid_exact(gv); }
            y[c] = from_f<T>(v);
        }
    }
}

}  // namespace mbh
