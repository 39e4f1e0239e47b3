// Prompt attention with the distance bias on tensor cores (bf16 storage): flash-style, one CTA per (64-query tile, head).
//
// Four warps, 16 queries each.  Per tile of 64 keys: K rows and V (transposed) are staged in shared memory from the layer's
// ring; S = Q K^T with mma.sync.m16n8k16 (Q fragments stay in registers); score = S * scale + bias[min(distance, n_tab - 1), h],
// causal mask, running (max, sum) per query row in fp32; P is rounded to bf16 and multiplies V on the tensor cores with fp32
// accumulators.  Query tiles never straddle two sequences; positions inside a tile are consecutive.
// With AttnArgs::sigmoid the weights are sigmoid(score) (fp32, then bf16 for P V) and nothing is normalised.
#pragma once
#include "hybrid_mixers.cuh"

namespace mbh {

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float quad_max(float v) {
    v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 1));
    return fmaxf(v, __shfl_xor_sync(0xffffffffu, v, 2));
}
__device__ __forceinline__ float quad_sum(float v) {
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    return v + __shfl_xor_sync(0xffffffffu, v, 2);
}

constexpr int FA_BQ = 64, FA_BK = 64;

template <int D, int E>
__global__ void __launch_bounds__(128) attn_bias_flash_kernel(AttnArgs a) {
    constexpr int KP = D + 8, VP = FA_BK + 8;
    __shared__ __align__(16) bf16 Ks[FA_BK][KP];
    __shared__ __align__(16) bf16 Vt[E][VP];
    const int h = blockIdx.y, g = h / (a.H / a.G);
    int tile = blockIdx.x, b = 0, t0 = 0;
    for (; b < a.B; ++b) {
        const int len = a.q_start[b + 1] - a.q_start[b], nt = (len + FA_BQ - 1) / FA_BQ;
        if (tile < nt) { t0 = a.q_start[b] + tile * FA_BQ; break; }
        tile -= nt;
    }
    if (b == a.B) return;
    const int t_end = a.q_start[b + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    const int r0 = t0 + warp * 16 + gid, r1 = r0 + 8;
    const bool v0 = r0 < t_end, v1 = r1 < t_end;
    const int pos_first = a.positions[t0];
    const int p0 = v0 ? pos_first + (r0 - t0) : -1, p1 = v1 ? pos_first + (r1 - t0) : -1;
    const int pos_last = pos_first + (min(t0 + FA_BQ, t_end) - 1 - t0);
    const int pos_warp_last = pos_first + (min(t0 + warp * 16 + 16, t_end) - 1 - t0);  // below pos_first + warp*16 when the warp has no row

    const bf16* Q = static_cast<const bf16*>(a.q);
    uint32_t qf[D / 16][4];
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        const int col = ks * 16 + tig * 2;
        const bf16* q0 = Q + ((size_t)r0 * a.H + h) * D + col;
        const bf16* q1 = Q + ((size_t)r1 * a.H + h) * D + col;
        qf[ks][0] = v0 ? *reinterpret_cast<const uint32_t*>(q0) : 0u;
        qf[ks][1] = v1 ? *reinterpret_cast<const uint32_t*>(q1) : 0u;
        qf[ks][2] = v0 ? *reinterpret_cast<const uint32_t*>(q0 + 8) : 0u;
        qf[ks][3] = v1 ? *reinterpret_cast<const uint32_t*>(q1 + 8) : 0u;
    }
    float o[E / 8][4];
#pragma unroll
    for (int ne = 0; ne < E / 8; ++ne) o[ne][0] = o[ne][1] = o[ne][2] = o[ne][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const size_t base = (size_t)a.slots[b] * a.W;
    const size_t kstride = (size_t)a.G * D, vstride = (size_t)a.G * E;
    const int own_from = a.own_k ? a.seqpos[b] : 0x7fffffff;
    const size_t own_row = a.own_k ? (size_t)a.q_start[b] : 0;
    const KeySource<bf16> Ksrc{static_cast<const bf16*>(a.cache_k) + base * kstride + (size_t)g * D,
                               static_cast<const bf16*>(a.own_k) + own_row * kstride + (size_t)g * D, kstride, kstride, a.W, own_from};
    const KeySource<bf16> Vsrc{static_cast<const bf16*>(a.cache_v) + base * vstride + (size_t)g * E,
                               static_cast<const bf16*>(a.own_v) + own_row * vstride + (size_t)g * E, vstride, vstride, a.W, own_from};
    // sliding window: the first key any row of this tile sees; key tiles below it are skipped
    const int j_lo = a.window > 0 ? max(0, pos_first - a.window + 1) : 0;
    const int w0 = a.window > 0 ? a.window : 0x40000000;  // row at position p sees keys j with p - j < w0
    const float* bias = a.bias_tab ? a.bias_tab + h : nullptr;  // null: no bias
    const int last_tab = a.n_tab - 1;

    for (int j0 = (j_lo / FA_BK) * FA_BK; j0 <= pos_last; j0 += FA_BK) {
        __syncthreads();
        for (int c = threadIdx.x; c < FA_BK * (D / 8); c += 128) {
            const int r = c / (D / 8), kc = (c % (D / 8)) * 8, j = j0 + r;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (j <= pos_last && j >= j_lo) v = *reinterpret_cast<const uint4*>(Ksrc.row(j) + kc);
            *reinterpret_cast<uint4*>(&Ks[r][kc]) = v;
        }
        for (int c = threadIdx.x; c < FA_BK * (E / 8); c += 128) {
            const int r = c % FA_BK, ec = (c / FA_BK) * 8, j = j0 + r;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (j <= pos_last && j >= j_lo) v = *reinterpret_cast<const uint4*>(Vsrc.row(j) + ec);
            const bf16* pv = reinterpret_cast<const bf16*>(&v);
#pragma unroll
            for (int i = 0; i < 8; ++i) Vt[ec + i][r] = pv[i];
        }
        __syncthreads();
        if (j0 > pos_warp_last) continue;  // every key of this tile is in the future of this warp's rows (the barriers above are kept)

        float s[8][4];
#pragma unroll
        for (int nt = 0; nt < 8; ++nt) s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks)
#pragma unroll
            for (int nt = 0; nt < 8; ++nt) {
                const bf16* p = &Ks[nt * 8 + gid][ks * 16 + tig * 2];
                mma_bf16(s[nt], qf[ks], *reinterpret_cast<const uint32_t*>(p), *reinterpret_cast<const uint32_t*>(p + 8));
            }
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const int j = j0 + nt * 8 + tig * 2 + c;
                const float x0 = (j <= p0 && p0 - j < w0) ? s[nt][c] * a.scale + (bias ? bias[(size_t)min(p0 - j, last_tab) * a.H] : 0.f) : -INFINITY;
                const float x1 = (j <= p1 && p1 - j < w0) ? s[nt][2 + c] * a.scale + (bias ? bias[(size_t)min(p1 - j, last_tab) * a.H] : 0.f) : -INFINITY;
                s[nt][c] = x0; s[nt][2 + c] = x1;
                mx0 = fmaxf(mx0, x0); mx1 = fmaxf(mx1, x1);
            }
        if (a.sigmoid) {  // weights sigmoid(score), 0 where masked; nothing to rescale
#pragma unroll
            for (int nt = 0; nt < 8; ++nt)
#pragma unroll
                for (int c = 0; c < 4; ++c) s[nt][c] = s[nt][c] == -INFINITY ? 0.f : __fdividef(1.f, 1.f + __expf(-s[nt][c]));  // rounded to bf16 just below
        }
        const float mn0 = a.sigmoid ? 0.f : fmaxf(m0, quad_max(mx0)), mn1 = a.sigmoid ? 0.f : fmaxf(m1, quad_max(mx1));
        const float c0 = (a.sigmoid || mn0 == -INFINITY) ? 1.f : expf(m0 - mn0), c1 = (a.sigmoid || mn1 == -INFINITY) ? 1.f : expf(m1 - mn1);
        float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 8; ++nt)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const float e0 = a.sigmoid ? s[nt][c] : (mn0 == -INFINITY) ? 0.f : expf(s[nt][c] - mn0);
                const float e1 = a.sigmoid ? s[nt][2 + c] : (mn1 == -INFINITY) ? 0.f : expf(s[nt][2 + c] - mn1);
                s[nt][c] = e0; s[nt][2 + c] = e1;
                ps0 += e0; ps1 += e1;
            }
        l0 = l0 * c0 + ps0; l1 = l1 * c1 + ps1;  // per-thread partial sums; the quad is reduced at the end (same factors in a quad)
        m0 = mn0; m1 = mn1;
#pragma unroll
        for (int ne = 0; ne < E / 8; ++ne) { o[ne][0] *= c0; o[ne][1] *= c0; o[ne][2] *= c1; o[ne][3] *= c1; }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
            uint32_t pa[4] = {pack_bf16(s[2 * kk][0], s[2 * kk][1]), pack_bf16(s[2 * kk][2], s[2 * kk][3]),
                              pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]), pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3])};
#pragma unroll
            for (int ne = 0; ne < E / 8; ++ne) {
                const bf16* p = &Vt[ne * 8 + gid][kk * 16 + tig * 2];
                mma_bf16(o[ne], pa, *reinterpret_cast<const uint32_t*>(p), *reinterpret_cast<const uint32_t*>(p + 8));
            }
        }
    }
    l0 = quad_sum(l0); l1 = quad_sum(l1);
    if (a.sigmoid) l0 = l1 = 1.f;
    bf16* out = static_cast<bf16*>(a.out);
#pragma unroll
    for (int ne = 0; ne < E / 8; ++ne) {
        const int col = ne * 8 + tig * 2;
        if (v0) *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)r0 * a.H + h) * E + col) = __floats2bfloat162_rn(o[ne][0] / l0, o[ne][1] / l0);
        if (v1) *reinterpret_cast<__nv_bfloat162*>(out + ((size_t)r1 * a.H + h) * E + col) = __floats2bfloat162_rn(o[ne][2] / l1, o[ne][3] / l1);
    }
}

// true when a (D, E) instantiation exists; launches it
inline bool launch_attn_flash(const AttnArgs& a, int n_tiles, cudaStream_t st) {
    dim3 grid(n_tiles, a.H);
#define MBH_FA(DD, EE) if (a.d == DD && a.e == EE) { attn_bias_flash_kernel<DD, EE><<<grid, 128, 0, st>>>(a); return true; }
    MBH_FA(32, 32) MBH_FA(64, 32) MBH_FA(64, 64) MBH_FA(128, 64) MBH_FA(64, 128) MBH_FA(128, 128) MBH_FA(96, 64) MBH_FA(192, 128)
#undef MBH_FA
    return false;
}

}  // namespace mbh
