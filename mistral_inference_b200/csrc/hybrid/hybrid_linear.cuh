// Linear layers of any shape, y = x W^T (+ b), W stored [N, K] row-major, with the layer's next elementwise step as epilogue.
//
//   EPI_STORE     out[M, N]    = act(acc + b)   act = SiLU on columns < n_act, identity elsewhere
//   EPI_RESIDUAL  resid[M, N] += acc + b        fp32 residual stream, in place
//   EPI_GLU       out[M, N/2]: rows of W interleaved (2c = gate, 2c + 1 = up):
//                 g = min(gate, limit), u = clamp(up, +-limit), out = g * sigmoid(alpha * g) * (u + 1); with rowscale (as for
//                 EPI_SWIGLU) gate and up are multiplied by rowscale[m, c / rs_group] BEFORE the clamps: experts whose INPUT is
//                 scaled by the routing weight, run densely (weight 0 gives exactly 0)
//   EPI_F32       out32[M, N]  = acc + b        (logits); with limit > 0: limit * tanh((acc + b) / limit), a soft cap
//   EPI_RESIDUAL_SCALED  resid[M, N] += alpha * (acc + b)    (one of several sublayers that are summed with fixed weights)
//   EPI_SWIGLU    out[M, N/2]: interleaved rows as for EPI_GLU: out = silu(gate) * up * rowscale[m, c / rs_group]
//                 (rowscale fp32 [M, rs_pitch] or null: a mixture of experts run densely, every expert's hidden units scaled by
//                 the token's routing weight, 0 for an expert that the token did not choose)
//   EPI_RELU2     out[M, N]    = max(acc, 0)^2 * rowscale[m, n / rs_group]   (plain rows, no gate; rowscale as for EPI_SWIGLU)
//
// In bf16 mode the Linear's own output is rounded to bf16 before the epilogue's arithmetic (the rounding point of a bf16
// Linear); accumulation is fp32 in both modes.
//
// Kernels: `linear_tiled_mma` (bf16) and `linear_tiled_fma` (fp32) for prompts, any shape; `linear_skinny` (M <= 8 rows, FMA,
// one warp per pair of weight rows) and `linear_skinny_mma` (bf16, 3..8 rows, tensor cores) for decode: every weight byte is read
// once with 16-byte loads; `linear_epilogue_kernel` applies the epilogues to the output of another GEMM (the main library's
// tcgen05 GEMM takes the large aligned bf16 Linears of prompts, see _abi_hybrid.linear).
#pragma once
#include "hybrid_common.cuh"

namespace mbh {

enum { EPI_STORE = 0, EPI_RESIDUAL = 1, EPI_GLU = 2, EPI_F32 = 3, EPI_SWIGLU = 4, EPI_RESIDUAL_SCALED = 5, EPI_RELU2 = 6 };

struct LinearArgs {
    const void* x; const void* w; const void* bias;
    void* out; float* out32;  // out: storage type; out32: fp32 residual (EPI_RESIDUAL) or logits (EPI_F32)
    int M, N, K;
    int epi, n_act;
    float limit, alpha;
    const float* rowscale; int rs_pitch, rs_group;  // EPI_SWIGLU
};

template <typename T>
__device__ __forceinline__ void epilogue_pair(const LinearArgs& a, int m, int n, float v0, float v1, bool has1) {
    // (m, n) and (m, n + 1); n is even
    const T* bias = static_cast<const T*>(a.bias);
    if (bias) { v0 += to_f(bias[n]); if (has1) v1 += to_f(bias[n + 1]); }
    if (a.epi != EPI_F32) { v0 = rnd<T>(v0); v1 = rnd<T>(v1); }
    switch (a.epi) {
    case EPI_STORE: {
        T* o = static_cast<T*>(a.out) + (size_t)m * a.N + n;
        if (n < a.n_act) v0 = v0 * sigmoid_exact(v0);
        o[0] = from_f<T>(v0);
        if (has1) { if (n + 1 < a.n_act) v1 = v1 * sigmoid_exact(v1); o[1] = from_f<T>(v1); }
        break; }
    case EPI_RESIDUAL: {
        float* o = a.out32 + (size_t)m * a.N + n;
        o[0] += v0;
        if (has1) o[1] += v1;
        break; }
    case EPI_RESIDUAL_SCALED: {
        float* o = a.out32 + (size_t)m * a.N + n;
        o[0] += a.alpha * v0;
        if (has1) o[1] += a.alpha * v1;
        break; }
    case EPI_GLU: {
        if (!has1) break;
        if (a.rowscale) { const float rs = a.rowscale[(size_t)m * a.rs_pitch + (n >> 1) / a.rs_group]; v0 *= rs; v1 *= rs; }
        float g = fminf(v0, a.limit), u = fminf(fmaxf(v1, -a.limit), a.limit);
        static_cast<T*>(a.out)[(size_t)m * (a.N >> 1) + (n >> 1)] = from_f<T>(g * sigmoid_exact(a.alpha * g) * (u + 1.f));
        break; }
    case EPI_SWIGLU: {
        if (!has1) break;
        const int c = n >> 1;
        float v = v0 * sigmoid_exact(v0) * v1;
        if (a.rowscale) v *= a.rowscale[(size_t)m * a.rs_pitch + c / a.rs_group];
        static_cast<T*>(a.out)[(size_t)m * (a.N >> 1) + c] = from_f<T>(v);
        break; }
    case EPI_RELU2: {
        T* o = static_cast<T*>(a.out) + (size_t)m * a.N + n;
        v0 = fmaxf(v0, 0.f); v1 = fmaxf(v1, 0.f);
        v0 *= v0; v1 *= v1;
        if (a.rowscale) {
            v0 *= a.rowscale[(size_t)m * a.rs_pitch + n / a.rs_group];
            if (has1) v1 *= a.rowscale[(size_t)m * a.rs_pitch + (n + 1) / a.rs_group];
        }
        o[0] = from_f<T>(v0);
        if (has1) o[1] = from_f<T>(v1);
        break; }
    default: {
        float* o = a.out32 + (size_t)m * a.N + n;
        if (a.limit > 0.f) { v0 = a.limit * tanhf(v0 / a.limit); v1 = a.limit * tanhf(v1 / a.limit); }
        o[0] = v0;
        if (has1) o[1] = v1;
        break; }
    }
}

// ------------------------------------------------------------------------------------------------ tiled, FMA (fp32 mode)
constexpr int LT_BM = 64, LT_BN = 64, LT_BK = 16, LT_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(LT_THREADS) linear_tiled_fma(LinearArgs a) {
    __shared__ float As[LT_BK][LT_BM + 4];
    __shared__ float Ws[LT_BK][LT_BN + 4];
    const T* X = static_cast<const T*>(a.x);
    const T* W = static_cast<const T*>(a.w);
    const int m0 = blockIdx.y * LT_BM, n0 = blockIdx.x * LT_BN;
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    float acc[4][4] = {};
    const int lr = tid >> 2, lc = (tid & 3) * 4;  // loader: row lr of the tile, 4 consecutive k
    for (int k0 = 0; k0 < a.K; k0 += LT_BK) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int k = k0 + lc + i;
            int m = m0 + lr, n = n0 + lr;
            As[lc + i][lr] = (m < a.M && k < a.K) ? to_f(X[(size_t)m * a.K + k]) : 0.f;
            Ws[lc + i][lr] = (n < a.N && k < a.K) ? to_f(W[(size_t)n * a.K + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < LT_BK; ++k) {
            float av[4], wv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { av[i] = As[k][ty * 4 + i]; wv[i] = Ws[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int m = m0 + ty * 4 + i;
        if (m >= a.M) continue;
#pragma unroll
        for (int j = 0; j < 4; j += 2) {
            int n = n0 + tx * 4 + j;
            if (n < a.N) epilogue_pair<T>(a, m, n, acc[i][j], acc[i][j + 1], n + 1 < a.N);
        }
    }
}

// ------------------------------------------------------------------------------------------------ tiled, tensor cores (bf16 mode)
// 128 x 128 output tile, 8 warps as 2 (m) x 4 (n): each warp 64 x 32 = 4 x 4 mma.sync.m16n8k16 tiles, K step 32.
constexpr int MM_BM = 128, MM_BN = 128, MM_BK = 32, MM_THREADS = 256, MM_LD = MM_BK + 8;  // row pitch 40 bf16 = 80 B: conflict-free fragments

__global__ void __launch_bounds__(MM_THREADS) linear_tiled_mma(LinearArgs a) {
    __shared__ __align__(16) bf16 As[2][MM_BM][MM_LD];
    __shared__ __align__(16) bf16 Ws[2][MM_BN][MM_LD];
    const bf16* X = static_cast<const bf16*>(a.x);
    const bf16* W = static_cast<const bf16*>(a.w);
    const int m0 = blockIdx.y * MM_BM, n0 = blockIdx.x * MM_BN;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = (warp >> 2) * 64, wn = (warp & 3) * 32;
    const int gid = lane >> 2, tig = lane & 3;
    const bool vec_ok = (a.K % 8 == 0) && ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W)) % 16 == 0);
    float acc[4][4][4] = {};

    // loader: 128 rows x 32 k = 512 chunks of 8 bf16 per operand, 2 per thread
    auto load_tile = [&](int buf, int k0) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            int chunk = tid + c * MM_THREADS, r = chunk >> 2, kc = (chunk & 3) * 8;
            int k = k0 + kc;
            uint4 va = make_uint4(0, 0, 0, 0), vw = make_uint4(0, 0, 0, 0);
            if (vec_ok) {
                if (m0 + r < a.M && k < a.K) va = *reinterpret_cast<const uint4*>(X + (size_t)(m0 + r) * a.K + k);
                if (n0 + r < a.N && k < a.K) vw = *reinterpret_cast<const uint4*>(W + (size_t)(n0 + r) * a.K + k);
            } else {
                bf16* pa = reinterpret_cast<bf16*>(&va);
                bf16* pw = reinterpret_cast<bf16*>(&vw);
                for (int i = 0; i < 8; ++i) {
                    if (m0 + r < a.M && k + i < a.K) pa[i] = X[(size_t)(m0 + r) * a.K + k + i];
                    if (n0 + r < a.N && k + i < a.K) pw[i] = W[(size_t)(n0 + r) * a.K + k + i];
                }
            }
            *reinterpret_cast<uint4*>(&As[buf][r][kc]) = va;
            *reinterpret_cast<uint4*>(&Ws[buf][r][kc]) = vw;
        }
    };

    const int nk = (a.K + MM_BK - 1) / MM_BK;
    load_tile(0, 0);
    __syncthreads();
    for (int kt = 0; kt < nk; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < nk) load_tile(buf ^ 1, (kt + 1) * MM_BK);
#pragma unroll
        for (int ks = 0; ks < MM_BK; ks += 16) {
            uint32_t af[4][4], bfr[4][2];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const bf16* p = &As[buf][wm + i * 16 + gid][ks + tig * 2];
                af[i][0] = *reinterpret_cast<const uint32_t*>(p);
                af[i][1] = *reinterpret_cast<const uint32_t*>(p + 8 * MM_LD);
                af[i][2] = *reinterpret_cast<const uint32_t*>(p + 8);
                af[i][3] = *reinterpret_cast<const uint32_t*>(p + 8 * MM_LD + 8);
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const bf16* p = &Ws[buf][wn + j * 8 + gid][ks + tig * 2];
                bfr[j][0] = *reinterpret_cast<const uint32_t*>(p);
                bfr[j][1] = *reinterpret_cast<const uint32_t*>(p + 8);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                                 : "+f"(acc[i][j][0]), "+f"(acc[i][j][1]), "+f"(acc[i][j][2]), "+f"(acc[i][j][3])
                                 : "r"(af[i][0]), "r"(af[i][1]), "r"(af[i][2]), "r"(af[i][3]), "r"(bfr[j][0]), "r"(bfr[j][1]));
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int n = n0 + wn + j * 8 + tig * 2;
            if (n >= a.N) continue;
            int m = m0 + wm + i * 16 + gid;
            if (m < a.M) epilogue_pair<bf16>(a, m, n, acc[i][j][0], acc[i][j][1], n + 1 < a.N);
            if (m + 8 < a.M) epilogue_pair<bf16>(a, m + 8, n, acc[i][j][2], acc[i][j][3], n + 1 < a.N);
        }
}

// ------------------------------------------------------------------------------------------------ skinny (decode)
constexpr int SK_MAX_M = 8, SK_WARPS = 8;

// R weight rows per warp (R even: gate/up pairs stay together); more rows per warp = fewer re-reads of x per weight byte
template <typename T, int MM, int R>
__global__ void __launch_bounds__(SK_WARPS * 32) linear_skinny(LinearArgs a) {
    const T* X = static_cast<const T*>(a.x);
    const T* W = static_cast<const T*>(a.w);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = (blockIdx.x * SK_WARPS + warp) * R;
    if (n >= a.N) return;
    const T* wr[R];
#pragma unroll
    for (int r = 0; r < R; ++r) wr[r] = W + (size_t)min(n + r, a.N - 1) * a.K;
    float acc[R][MM];
#pragma unroll
    for (int r = 0; r < R; ++r)
#pragma unroll
        for (int m = 0; m < MM; ++m) acc[r][m] = 0.f;
    constexpr int V = Vec<T>::N;
    const bool vec_ok = (a.K % V == 0) && ((reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(W)) % 16 == 0);
    if (vec_ok) {
        for (int k = lane * V; k < a.K; k += 32 * V) {
            float wv[R][V], xv[V];
#pragma unroll
            for (int r = 0; r < R; ++r) Vec<T>::load(wr[r] + k, wv[r]);
#pragma unroll
            for (int m = 0; m < MM; ++m) {
                if (m < a.M) {
                    Vec<T>::load(X + (size_t)m * a.K + k, xv);
#pragma unroll
                    for (int r = 0; r < R; ++r)
#pragma unroll
                        for (int i = 0; i < V; ++i) acc[r][m] = fmaf(wv[r][i], xv[i], acc[r][m]);
                }
            }
        }
    } else {
        for (int k = lane; k < a.K; k += 32) {
            float wv[R];
#pragma unroll
            for (int r = 0; r < R; ++r) wv[r] = to_f(wr[r][k]);
#pragma unroll
            for (int m = 0; m < MM; ++m)
                if (m < a.M) {
                    const float xv = to_f(X[(size_t)m * a.K + k]);
#pragma unroll
                    for (int r = 0; r < R; ++r) acc[r][m] = fmaf(wv[r], xv, acc[r][m]);
                }
        }
    }
#pragma unroll
    for (int m = 0; m < MM; ++m)
#pragma unroll
        for (int r = 0; r < R; r += 2) {
            const float s0 = warp_sum(acc[r][m]), s1 = warp_sum(acc[r + 1][m]);
            if (lane == 0 && m < a.M && n + r < a.N) epilogue_pair<T>(a, m, n + r, s0, s1, n + r + 1 < a.N);
        }
}

// ------------------------------------------------------------------------------------------------ skinny on tensor cores (bf16, 3..8 rows)
// y^T = W x^T: the 16 weight rows of a CTA are the M side of m16n8k16 tiles, the (up to 8) tokens the N side, so a decode batch
// costs one tensor-core instruction per 16 x 16 weights instead of 8 FMAs per weight.  The CTA's warps split K; every lane
// loads 16 contiguous bytes of two weight rows and of one token's activations per step -- the k order inside a step is
// permuted identically for both operands, which a dot product does not notice.  Needs K % 8 == 0 and 16-byte aligned rows.
constexpr int SKM_WARPS = 8;

__global__ void __launch_bounds__(SKM_WARPS * 32) linear_skinny_mma(LinearArgs a) {
    __shared__ float part[SKM_WARPS][16][9];
    const bf16* X = static_cast<const bf16*>(a.x);
    const bf16* W = static_cast<const bf16*>(a.w);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, gid = lane >> 2, tig = lane & 3;
    const int n0 = blockIdx.x * 16;
    const bf16* wa = W + (size_t)min(n0 + gid, a.N - 1) * a.K;
    const bf16* wb = W + (size_t)min(n0 + gid + 8, a.N - 1) * a.K;
    const bool xrow = gid < a.M;
    const bf16* xr = X + (size_t)(xrow ? gid : 0) * a.K;
    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4  // four steps of loads in flight per warp: the kernel waits on global memory, not on the tensor pipe
    for (int kb = warp * 32; kb < a.K; kb += SKM_WARPS * 32) {
        const int k = kb + tig * 8;
        uint4 va = make_uint4(0, 0, 0, 0), vb = va, vx = va;
        if (k < a.K) {
            va = *reinterpret_cast<const uint4*>(wa + k);
            vb = *reinterpret_cast<const uint4*>(wb + k);
            if (xrow) vx = *reinterpret_cast<const uint4*>(xr + k);
        }
        const uint32_t a0[4] = {va.x, vb.x, va.y, vb.y}, a1[4] = {va.z, vb.z, va.w, vb.w};
        mma_bf16(c, a0, vx.x, vx.y);
        mma_bf16(c, a1, vx.z, vx.w);
    }
    part[warp][gid][tig * 2] = c[0]; part[warp][gid][tig * 2 + 1] = c[1];
    part[warp][gid + 8][tig * 2] = c[2]; part[warp][gid + 8][tig * 2 + 1] = c[3];
    __syncthreads();
    if (threadIdx.x < 64) {
        const int m = threadIdx.x & 7, r = (threadIdx.x >> 3) * 2, n = n0 + r;
        if (m < a.M && n < a.N) {
            float s0 = 0.f, s1 = 0.f;
#pragma unroll
            for (int w = 0; w < SKM_WARPS; ++w) { s0 += part[w][r][m]; s1 += part[w][r + 1][m]; }
            epilogue_pair<bf16>(a, m, n, s0, s1, n + 1 < a.N);
        }
    }
}

// The epilogues alone, over a Linear output y[M, N] (storage type, N even) that another GEMM produced
template <typename T>
__global__ void linear_epilogue_kernel(LinearArgs a, const T* __restrict__ y) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t pairs = (size_t)a.M * (a.N >> 1);
    if (idx >= pairs) return;
    const int m = (int)(idx / (a.N >> 1)), n = (int)(idx % (a.N >> 1)) * 2;
    epilogue_pair<T>(a, m, n, to_f(y[(size_t)m * a.N + n]), to_f(y[(size_t)m * a.N + n + 1]), true);
}

template <typename T>
inline cudaError_t launch_linear(const LinearArgs& a, cudaStream_t st) {
    if (a.M <= 0 || a.N <= 0) return cudaSuccess;
    if constexpr (sizeof(T) == 2) {
        if (a.M > 2 && a.M <= 8 && a.K % 8 == 0 && (reinterpret_cast<uintptr_t>(a.x) | reinterpret_cast<uintptr_t>(a.w)) % 16 == 0) {
            linear_skinny_mma<<<(a.N + 15) / 16, SKM_WARPS * 32, 0, st>>>(a);
            return cudaGetLastError();
        }
    }
    if (a.M <= SK_MAX_M) {
        dim3 grid2((a.N + 2 * SK_WARPS - 1) / (2 * SK_WARPS));  // two rows per warp measured faster than four at M = 8
        if (a.M <= 1) linear_skinny<T, 1, 2><<<grid2, SK_WARPS * 32, 0, st>>>(a);
        else if (a.M <= 2) linear_skinny<T, 2, 2><<<grid2, SK_WARPS * 32, 0, st>>>(a);
        else if (a.M <= 4) linear_skinny<T, 4, 2><<<grid2, SK_WARPS * 32, 0, st>>>(a);
        else linear_skinny<T, 8, 2><<<grid2, SK_WARPS * 32, 0, st>>>(a);
    } else if constexpr (sizeof(T) == 2) {
        dim3 grid((a.N + MM_BN - 1) / MM_BN, (a.M + MM_BM - 1) / MM_BM);
        linear_tiled_mma<<<grid, MM_THREADS, 0, st>>>(a);
    } else {
        dim3 grid((a.N + LT_BN - 1) / LT_BN, (a.M + LT_BM - 1) / LT_BM);
        linear_tiled_fma<T><<<grid, LT_THREADS, 0, st>>>(a);
    }
    return cudaGetLastError();
}

}  // namespace mbh
