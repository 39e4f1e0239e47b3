// C ABI of libmb200_hybrid.so: the kernels of layered decoders (per-layer mixer kinds, fp32 residual stream, bf16 or fp32
// storage).  Declarations: include/mistral_b200_hybrid.h.  `dt` selects the storage type of activations and weights:
// 0 = bf16, 1 = fp32.  Every call returns 0 or a CUDA error code; mbh_last_error() gives the text.
#include "hybrid_linear.cuh"
#include "hybrid_mixers.cuh"
#include "hybrid_attn_flash.cuh"
#include "hybrid_latent.cuh"
#include "hybrid_moe.cuh"
#include "hybrid_rotary.cuh"
#include "hybrid_gated_scan.cuh"
#include "hybrid_stream.cuh"
#include "../../../include/mistral_b200_hybrid.h"

#include <stdio.h>

using namespace mbh;

static thread_local char g_err[256] = "";

static int fail(cudaError_t e, const char* what) {
    snprintf(g_err, sizeof(g_err), "%s: %s", what, cudaGetErrorString(e));
    return (int)e;
}
static int bad(const char* what) {
    snprintf(g_err, sizeof(g_err), "%s", what);
    return -1;
}
#define DISPATCH(dt, ...)                                   \
    do {                                                    \
        if ((dt) == 0) { using ST = bf16; __VA_ARGS__; }     \
        else if ((dt) == 1) { using ST = float; __VA_ARGS__; } \
        else return bad("dt must be 0 (bf16) or 1 (fp32)"); \
    } while (0)

template <typename T>
static cudaError_t launch_lightning(const LightningArgs& a, cudaStream_t st) {
    const int threads = LS_THREADS;
    dim3 grid(a.B * a.H, (a.e + threads - 1) / threads);
    if (a.d <= 32) lightning_scan_kernel<T, 32><<<grid, threads, 0, st>>>(a);
    else if (a.d <= 64) lightning_scan_kernel<T, 64><<<grid, threads, 0, st>>>(a);
    else lightning_scan_kernel<T, 128><<<grid, threads, 0, st>>>(a);
    return cudaGetLastError();
}


// key size -> registers per state column; tokens per shared-memory tile chosen so that nothing spills
template <typename T, int MODE>
static void launch_gated_scan_mode(const GatedScanArgs& a, dim3 grid, cudaStream_t st) {
    if (a.ones) {
        if (a.d <= 32) gated_scan_kernel<T, 32, 16, MODE, true><<<grid, GS_THREADS, 0, st>>>(a);
        else if (a.d <= 64) gated_scan_kernel<T, 64, 16, MODE, true><<<grid, GS_THREADS, 0, st>>>(a);
        else if (a.d <= 128) gated_scan_kernel<T, 128, 8, MODE, true><<<grid, GS_THREADS, 0, st>>>(a);
        else gated_scan_kernel<T, 128, 8, MODE, true, true><<<grid, GS_THREADS, 0, st>>>(a);
    } else {
        if (a.d <= 32) gated_scan_kernel<T, 32, 16, MODE, false><<<grid, GS_THREADS, 0, st>>>(a);
        else if (a.d <= 64) gated_scan_kernel<T, 64, 16, MODE, false><<<grid, GS_THREADS, 0, st>>>(a);
        else if (a.d <= 128) gated_scan_kernel<T, 128, 8, MODE, false><<<grid, GS_THREADS, 0, st>>>(a);
        else gated_scan_kernel<T, 128, 8, MODE, false, true><<<grid, GS_THREADS, 0, st>>>(a);
    }
}

template <typename T>
static cudaError_t launch_gated_scan(const GatedScanArgs& a, cudaStream_t st) {
    dim3 grid(a.B * a.H, (a.e + GS_THREADS - 1) / GS_THREADS * a.key_blocks);
    launch_gated_scan_mode<T, GS_WHOLE>(a, grid, st);
    return cudaGetLastError();
}

template <typename T, int MODE>
static void launch_gated_scan_chunks(const GatedScanArgs& a, int chunks, cudaStream_t st) {
    dim3 grid(a.B * a.H, (a.e + GS_THREADS - 1) / GS_THREADS * a.key_blocks, chunks);
    launch_gated_scan_mode<T, MODE>(a, grid, st);
}

// long prompts: chunk-local states, decay products, the walk over the chunks, then the outputs from each chunk's start state
template <typename T>
static cudaError_t launch_gated_scan_chunked(const GatedScanArgs& a, int chunks, cudaStream_t st) {
    launch_gated_scan_chunks<T, GS_LOCAL>(a, chunks, st);
    chunk_decay_kernel<<<dim3(a.B * a.H, chunks), 128, 0, st>>>(a);
    const int elems = a.d * (a.e + a.ones);
    scan_combine_kernel<<<dim3(a.B * a.H, (elems + 255) / 256), 256, 0, st>>>(a, chunks);
    launch_gated_scan_chunks<T, GS_OUTPUT>(a, chunks, st);
    return cudaGetLastError();
}

template <typename T> static void run_mlstm_gates(const MlstmGateArgs& a, int64_t B, int64_t T_, cudaStream_t st) {
    mlstm_m_kernel<T><<<(unsigned)(B * a.H), 32, 0, st>>>(a);
    const unsigned jb = T_ < 512 ? (unsigned)((a.H * a.d + 255) / 256) : 1u;
    mlstm_qab_kernel<T><<<dim3((unsigned)T_, jb), 256, 0, st>>>(a);
}
template <typename T> static void run_embed(const void* tokens, const void* table, float scale, void* x32, int64_t T_, int64_t D, cudaStream_t st) {
    embed_scale_kernel<T><<<(unsigned)T_, 128, 0, st>>>((const int64_t*)tokens, (const T*)table, scale, (float*)x32, (int)D);
}
template <typename T> static void run_embed_add(const void* tokens, const void* table, float scale, void* x32, int64_t T_, int64_t D, cudaStream_t st) {
    embed_scale_kernel<T, true><<<(unsigned)T_, 128, 0, st>>>((const int64_t*)tokens, (const T*)table, scale, (float*)x32, (int)D);
}
template <typename T> static void run_layernorm(const void* x32, const void* w, const void* b, void* y, void* acc32, int64_t T_, int64_t D, float eps,
                                                cudaStream_t st) {
    const int threads = D >= 1024 ? 256 : 128;
    if (acc32) layernorm_f32_kernel<T, true><<<(unsigned)T_, threads, 0, st>>>((const float*)x32, (const T*)w, (const T*)b, nullptr, (float*)acc32, (int)D, eps);
    else layernorm_f32_kernel<T, false><<<(unsigned)T_, threads, 0, st>>>((const float*)x32, (const T*)w, (const T*)b, (T*)y, nullptr, (int)D, eps);
}
template <typename T> static void run_attn_wide(const AttnArgs& a, size_t smem, cudaStream_t st) {
    attn_bias_kernel<T, AT_MAXR_WIDE><<<dim3((unsigned)(a.T * a.H), (unsigned)a.splits), AT_WARPS * 32, smem, st>>>(a);
    if (a.splits > 1) attn_merge_kernel<T><<<dim3((unsigned)(a.T * a.H), (unsigned)((a.e + 127) / 128)), 128, 0, st>>>(a.scratch, (T*)a.out, a.splits, a.e, a.sigmoid);
}
template <typename T> static void run_moe_sparse(const MoeSparseArgs& a, int64_t T_, cudaStream_t st) {
    moe_gateup_sparse_kernel<T><<<dim3((unsigned)((a.ff + MOE_WARPS - 1) / MOE_WARPS), (unsigned)(T_ * a.top)), MOE_WARPS * 32, 0, st>>>(a);
    moe_down_sparse_kernel<T><<<dim3((unsigned)((a.width + MOE_WARPS - 1) / MOE_WARPS), (unsigned)T_), MOE_WARPS * 32, 0, st>>>(a);
}
template <typename T> static void run_rmsnorm(const void* x32, const void* w, void* y, int64_t T_, int64_t D, float eps, cudaStream_t st) {
    rmsnorm_f32_kernel<T><<<(unsigned)T_, D >= 1024 ? 256 : 128, 0, st>>>((const float*)x32, (const T*)w, (T*)y, (int)D, eps);
}
template <typename T> static void run_epilogue(const LinearArgs& a, const void* y, cudaStream_t st) {
    const size_t pairs = (size_t)a.M * (a.N >> 1);
    linear_epilogue_kernel<T><<<(unsigned)((pairs + 255) / 256), 256, 0, st>>>(a, (const T*)y);
}
template <typename T> static void run_prep(const AttnPrepArgs& a, int64_t T_, cudaStream_t st) { attn_prep_kernel<T><<<(unsigned)T_, 128, 0, st>>>(a); }
template <typename T> static void run_attn(const AttnArgs& a, size_t smem, cudaStream_t st) {
    attn_bias_kernel<T><<<dim3((unsigned)(a.T * a.H), (unsigned)a.splits), AT_WARPS * 32, smem, st>>>(a);
    if (a.splits > 1) attn_merge_kernel<T><<<dim3((unsigned)(a.T * a.H), (unsigned)((a.e + 127) / 128)), 128, 0, st>>>(a.scratch, (T*)a.out, a.splits, a.e, a.sigmoid);
}
template <typename T> static void run_headnorm(const void* o32, const void* w, const void* g, int64_t g_pitch, int64_t g_off, void* y, int64_t T_,
                                               int64_t N, float eps, cudaStream_t st) {
    gated_headnorm_kernel<T><<<(unsigned)T_, 128, 0, st>>>((const float*)o32, (const T*)w, (const T*)g, (int)g_pitch, (int)g_off, (T*)y, (int)N, eps);
}

template <typename T, int HPW> static cudaError_t run_latent_decode(const LatentDecodeArgs& a, void* out, size_t smem, cudaStream_t st) {
    cudaError_t e = cudaFuncSetAttribute(attn_latent_decode_kernel<T, HPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e) return e;
    attn_latent_decode_kernel<T, HPW><<<dim3((unsigned)a.B, (unsigned)a.splits), LD_WARPS * 32, smem, st>>>(a);
    attn_merge_kernel<T><<<dim3((unsigned)(a.B * a.H), (unsigned)((a.kv_rank + 127) / 128)), 128, 0, st>>>(a.scratch, (T*)out, a.splits, a.kv_rank);
    return cudaGetLastError();
}
template <typename T> static cudaError_t launch_latent_decode(const LatentDecodeArgs& a, void* out, cudaStream_t st) {
    const int d = a.kv_rank + a.rot_dim, kp = d + (sizeof(T) == 2 ? 2 : 1);
    const size_t smem = sizeof(float) * ((size_t)a.H * d + (size_t)a.H * LD_KT) + sizeof(T) * (size_t)LD_KT * kp;
    if (smem > 220 * 1024) return cudaErrorInvalidValue;
    if (a.H <= LD_WARPS) return run_latent_decode<T, 1>(a, out, smem, st);
    if (a.H <= 2 * LD_WARPS) return run_latent_decode<T, 2>(a, out, smem, st);
    return run_latent_decode<T, 4>(a, out, smem, st);
}

extern "C" {

int mbh_abi_version(void) { return MBH_ABI_VERSION; }
const char* mbh_last_error(void) { return g_err; }

int mbh_embed_scale(const void* tokens, const void* table, float scale, void* x32, int64_t T, int64_t D, int dt, void* stream) {
    if (T == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, run_embed<ST>(tokens, table, scale, x32, T, D, st));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_embed_scale") : 0;
}

int mbh_rmsnorm(const void* x32, const void* w, void* y, int64_t T, int64_t D, float eps, int dt, void* stream) {
    if (T == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, run_rmsnorm<ST>(x32, w, y, T, D, eps, st));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_rmsnorm") : 0;
}

int mbh_linear(const void* x, const void* w, const void* bias, void* out, void* out32, int64_t M, int64_t N, int64_t K, int epi, int64_t n_act,
               float limit, float alpha, int dt, void* stream) {
    if ((epi < 0 || epi > 3) && epi != EPI_RESIDUAL_SCALED) return bad("mbh_linear: unknown epilogue");  // EPI_SWIGLU: mbh_linear_swiglu
    if (epi == EPI_GLU && (N & 1)) return bad("mbh_linear: the gated epilogue needs interleaved (even) rows");
    LinearArgs a{x, w, bias, out, (float*)out32, (int)M, (int)N, (int)K, epi, (int)n_act, limit, alpha};
    cudaError_t e = cudaSuccess;
    DISPATCH(dt, e = launch_linear<ST>(a, (cudaStream_t)stream));
    return e ? fail(e, "mbh_linear") : 0;
}

int mbh_linear_epilogue(const void* y, const void* bias, void* out, void* out32, int64_t M, int64_t N, int epi, int64_t n_act, float limit, float alpha,
                        int dt, void* stream) {
    if (((epi < 0 || epi > 3) && epi != EPI_RESIDUAL_SCALED) || (N & 1)) return bad("mbh_linear_epilogue: unknown epilogue or odd N");
    if (M == 0) return 0;
    LinearArgs a{nullptr, nullptr, bias, out, (float*)out32, (int)M, (int)N, 0, epi, (int)n_act, limit, alpha};
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, run_epilogue<ST>(a, y, st));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_linear_epilogue") : 0;
}

int mbh_attn_prep(const void* qkv, const void* qnorm, const void* knorm, const void* positions, const void* cache_rows, void* q_out, void* cache_k,
                  void* cache_v, void* v_first, const void* vmix, int vmix_mode, int64_t T, int64_t H, int64_t G, int64_t d, int64_t e, float eps,
                  float temp_coef, int64_t temp_every, int dt, void* stream) {
    if (T == 0) return 0;
    AttnPrepArgs a{qkv, qnorm, knorm, (const int*)positions, (const int*)cache_rows, q_out, cache_k, cache_v, v_first, vmix, vmix_mode,
                   (int)H, (int)G, (int)d, (int)e, eps, temp_coef, (int)temp_every};
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, run_prep<ST>(a, T, st));
    cudaError_t err = cudaGetLastError();
    return err ? fail(err, "mbh_attn_prep") : 0;
}

int mbh_attn_bias(const void* q, const void* cache_k, const void* cache_v, const void* bias_tab, int64_t n_tab, const void* positions,
                  const void* q_start, const void* slots, void* out, int64_t T, int64_t B, int64_t W, int64_t H, int64_t G, int64_t d, int64_t e,
                  float scale, int64_t n_tiles, int64_t splits, void* scratch, int dt, void* stream) {
    return mbh_attn_window(q, cache_k, cache_v, bias_tab, n_tab, positions, q_start, slots, out, T, B, W, H, G, d, e, scale, n_tiles, splits, scratch,
                           0, nullptr, nullptr, nullptr, 0, 0, dt, stream);
}

int mbh_attn_window(const void* q, const void* cache_k, const void* cache_v, const void* bias_tab, int64_t n_tab, const void* positions,
                    const void* q_start, const void* slots, void* out, int64_t T, int64_t B, int64_t W, int64_t H, int64_t G, int64_t d, int64_t e,
                    float scale, int64_t n_tiles, int64_t splits, void* scratch, int64_t window, const void* own_k, const void* own_v,
                    const void* seqpos, int64_t chunk, int weights, int dt, void* stream) {
    if (T == 0) return 0;
    if (weights != 0 && weights != 1) return bad("mbh_attn_window: weights are 0 (softmax) or 1 (sigmoid)");
    if (chunk < 0 || chunk > AT_CHUNK) return bad("mbh_attn_window: chunk is 0 (default) or 1 .. 128 keys");
    if (e > 32 * AT_MAXR) return bad("mbh_attn_bias: value size above 256");
    if (H % G) return bad("mbh_attn_bias: heads must be a multiple of kv heads");
    if (splits > AT_MAX_SPLITS) return bad("mbh_attn_bias: at most 64 splits");
    if (window < 0 || (!own_k != !own_v) || (own_k && !seqpos)) return bad("mbh_attn_window: window >= 0; own keys, own values and seqpos come together");
    AttnArgs a{q, cache_k, cache_v, (const float*)bias_tab, (int)n_tab, (const int*)positions, (const int*)q_start, (const int*)slots, out,
               (int)T, (int)B, (int)W, (int)H, (int)G, (int)d, (int)e, scale, (int)(splits > 1 && scratch ? splits : 1), (float*)scratch, 0, 0,
               (int)window, own_k, own_v, (const int*)seqpos, (int)chunk, weights};
    const size_t smem = sizeof(float) * ((size_t)d + AT_WARPS * AT_CHUNK + AT_WARPS * (2 + 32 * AT_MAXR));
    cudaStream_t st = (cudaStream_t)stream;
    // prompts in bf16: the tensor-core kernel, when the caller counted the 64-query tiles and the sizes are instantiated
    if (dt == 0 && n_tiles > 0 && launch_attn_flash(a, (int)n_tiles, st)) {
        cudaError_t ferr = cudaGetLastError();
        return ferr ? fail(ferr, "mbh_attn_bias (flash)") : 0;
    }
    DISPATCH(dt, run_attn<ST>(a, smem, st));
    cudaError_t err = cudaGetLastError();
    return err ? fail(err, "mbh_attn_bias") : 0;
}

int mbh_lightning_scan(const void* qkvg, void* state, const void* decay, const void* q_start, const void* seqpos, const void* slots, void* o32,
                       int64_t B, int64_t H, int64_t d, int64_t e, int dt, void* stream) {
    if (B == 0) return 0;
    if (d > 128) return bad("mbh_lightning_scan: key size above 128");
    LightningArgs a{qkvg, (float*)state, (const float*)decay, (const int*)q_start, (const int*)seqpos, (const int*)slots, (float*)o32,
                    (int)B, (int)H, (int)d, (int)e};
    cudaError_t err = cudaSuccess;
    DISPATCH(dt, err = launch_lightning<ST>(a, (cudaStream_t)stream));
    return err ? fail(err, "mbh_lightning_scan") : 0;
}

int mbh_gated_headnorm(const void* o32, const void* w, const void* g, int64_t g_pitch, int64_t g_off, void* y, int64_t T, int64_t N, float eps,
                       int dt, void* stream) {
    if (T == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, run_headnorm<ST>(o32, w, g, g_pitch, g_off, y, T, N, eps, st));
    cudaError_t err = cudaGetLastError();
    return err ? fail(err, "mbh_gated_headnorm") : 0;
}

int mbh_embed_add(const void* tokens, const void* table, float scale, void* x32, int64_t T, int64_t D, int dt, void* stream) {
    if (T == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, run_embed_add<ST>(tokens, table, scale, x32, T, D, st));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_embed_add") : 0;
}

int mbh_layernorm(const void* x32, const void* w, const void* b, void* y, void* acc32, int64_t T, int64_t D, float eps, int dt, void* stream) {
    if (T == 0) return 0;
    if (!y == !acc32) return bad("mbh_layernorm: exactly one of y and acc32");
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, run_layernorm<ST>(x32, w, b, y, acc32, T, D, eps, st));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_layernorm") : 0;
}

int mbh_linear_swiglu(const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K, const void* rowscale, int64_t rs_pitch,
                      int64_t rs_group, int dt, void* stream) {
    if (N & 1) return bad("mbh_linear_swiglu: the gated epilogue needs interleaved (even) rows");
    if (rowscale && rs_group <= 0) return bad("mbh_linear_swiglu: rs_group must be positive");
    LinearArgs a{x, w, nullptr, out, nullptr, (int)M, (int)N, (int)K, EPI_SWIGLU, 0, 0.f, 0.f, (const float*)rowscale, (int)rs_pitch, (int)rs_group};
    cudaError_t e = cudaSuccess;
    DISPATCH(dt, e = launch_linear<ST>(a, (cudaStream_t)stream));
    return e ? fail(e, "mbh_linear_swiglu") : 0;
}

int mbh_swiglu_epilogue(const void* y, void* out, int64_t M, int64_t N, const void* rowscale, int64_t rs_pitch, int64_t rs_group, int dt,
                        void* stream) {
    if (N & 1) return bad("mbh_swiglu_epilogue: odd N");
    if (rowscale && rs_group <= 0) return bad("mbh_swiglu_epilogue: rs_group must be positive");
    if (M == 0) return 0;
    LinearArgs a{nullptr, nullptr, nullptr, out, nullptr, (int)M, (int)N, 0, EPI_SWIGLU, 0, 0.f, 0.f, (const float*)rowscale, (int)rs_pitch, (int)rs_group};
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, run_epilogue<ST>(a, y, st));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_swiglu_epilogue") : 0;
}

int mbh_latent_prep(const void* y, const void* qnorm, const void* cnorm, const void* freq, const void* positions, const void* cache_rows, void* cq,
                    void* ring, int64_t T, int64_t pitch, int64_t q_rank, int64_t kv_rank, int64_t rot_dim, int64_t rot_dims, float eps, float mag,
                    int dt, void* stream) {
    if (T == 0) return 0;
    if (rot_dims > rot_dim || (rot_dims & 1)) return bad("mbh_latent_prep: rot_dims must be even and at most rot_dim");
    LatentPrepArgs a{y, qnorm, cnorm, (const double*)freq, (const int*)positions, (const int*)cache_rows, cq, ring,
                     (int)q_rank, (int)kv_rank, (int)rot_dim, (int)rot_dims, (int)pitch, eps, mag};
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, latent_prep_kernel<ST><<<(unsigned)T, 128, 0, st>>>(a));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_latent_prep") : 0;
}

int mbh_latent_absorb(const void* q, const void* w_uk, const void* freq, const void* positions, void* qa, int64_t T, int64_t H, int64_t dn,
                      int64_t rot_dim, int64_t rot_dims, int64_t kv_rank, float mag, int dt, void* stream) {
    if (T == 0) return 0;
    if (rot_dims > rot_dim || (rot_dims & 1)) return bad("mbh_latent_absorb: rot_dims must be even and at most rot_dim");
    LatentAbsorbArgs a{q, w_uk, (const double*)freq, (const int*)positions, qa, (int)H, (int)dn, (int)rot_dim, (int)rot_dims, (int)kv_rank, mag};
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, latent_absorb_kernel<ST><<<dim3((unsigned)(T * H), (unsigned)(w_uk ? (kv_rank + 127) / 128 : 1)), 128, sizeof(float) * (size_t)dn, st>>>(a));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_latent_absorb") : 0;
}

int mbh_latent_expand(const void* kn, const void* v, const void* ring, const void* positions, const void* cache_rows, const void* q_start, void* kfull,
                      void* vfull, int64_t T, int64_t B, int64_t Wt, int64_t H, int64_t dn, int64_t rot_dim, int64_t dv, int64_t kv_rank, int dt,
                      void* stream) {
    if (T == 0) return 0;
    LatentExpandArgs a{kn, v, ring, (const int*)positions, (const int*)cache_rows, (const int*)q_start, kfull, vfull,
                       (int)B, (int)Wt, (int)H, (int)dn, (int)rot_dim, (int)dv, (int)kv_rank};
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, latent_expand_kernel<ST><<<(unsigned)T, 128, 0, st>>>(a));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_latent_expand") : 0;
}

int mbh_head_gate(void* out, const void* gate, int64_t g_pitch, int64_t g_off, int64_t T, int64_t H, int64_t dv, int dt, void* stream) {
    if (T == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, head_gate_kernel<ST><<<(unsigned)T, 256, 0, st>>>((ST*)out, (const ST*)gate, (int)g_pitch, (int)g_off, (int)H, (int)dv));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_head_gate") : 0;
}

int mbh_attn_latent(const void* qa, const void* ring, const void* positions, const void* q_start, const void* slots, void* o_lat, int64_t T,
                    int64_t B, int64_t W, int64_t H, int64_t kv_rank, int64_t rot_dim, float scale, int64_t splits, void* scratch, int dt,
                    void* stream) {
    if (T == 0) return 0;
    if (kv_rank > 32 * AT_MAXR_WIDE) return bad("mbh_attn_latent: latent size above 512");
    if (splits > AT_MAX_SPLITS) return bad("mbh_attn_latent: at most 64 splits");
    const int d = (int)(kv_rank + rot_dim);
    AttnArgs a{qa, ring, ring, nullptr, 0, (const int*)positions, (const int*)q_start, (const int*)slots, o_lat,
               (int)T, (int)B, (int)W, (int)H, 1, d, (int)kv_rank, scale, (int)(splits > 1 && scratch ? splits : 1), (float*)scratch, d, d};
    const bool wide = kv_rank > 32 * AT_MAXR;
    const size_t smem = sizeof(float) * ((size_t)d + AT_WARPS * AT_CHUNK + AT_WARPS * (2 + 32 * (wide ? AT_MAXR_WIDE : AT_MAXR)));
    cudaStream_t st = (cudaStream_t)stream;
    if (wide) DISPATCH(dt, run_attn_wide<ST>(a, smem, st));
    else DISPATCH(dt, run_attn<ST>(a, smem, st));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_attn_latent") : 0;
}

int mbh_attn_latent_decode(const void* qa, const void* ring, const void* positions, const void* slots, void* o_lat, int64_t B, int64_t W, int64_t H,
                           int64_t kv_rank, int64_t rot_dim, float scale, int64_t splits, void* scratch, int dt, void* stream) {
    if (B == 0) return 0;
    if (H > 4 * LD_WARPS || kv_rank > 32 * LD_CPL) return bad("mbh_attn_latent_decode: at most 32 heads and a latent of 512");
    if (splits < 1 || splits > AT_MAX_SPLITS || !scratch) return bad("mbh_attn_latent_decode: needs 1 <= splits <= 64 and scratch");
    LatentDecodeArgs a{qa, ring, (const int*)positions, (const int*)slots, (float*)scratch, (int)B, (int)W, (int)H, (int)kv_rank, (int)rot_dim, scale,
                       (int)splits};
    cudaError_t e = cudaSuccess;
    DISPATCH(dt, e = launch_latent_decode<ST>(a, o_lat, (cudaStream_t)stream));
    return e ? fail(e, "mbh_attn_latent_decode") : 0;
}

int mbh_latent_vup(const void* o_lat, const void* w_uv, const void* gate, int64_t g_pitch, int64_t g_off, void* out, int64_t T, int64_t H,
                   int64_t dv, int64_t kv_rank, int dt, void* stream) {
    if (T == 0) return 0;
    LatentVupArgs a{o_lat, w_uv, gate, out, (int)H, (int)dv, (int)kv_rank, (int)g_pitch, (int)g_off};
    cudaStream_t st = (cudaStream_t)stream;
    // few tokens: a CTA per four value columns, so that a decode step fills the GPU; prompts: one CTA per (token, head)
    const unsigned vblocks = (T * H < 2048) ? (unsigned)((dv + 3) / 4) : 1u;
    DISPATCH(dt, latent_vup_kernel<ST><<<dim3((unsigned)(T * H), vblocks), 128, sizeof(float) * (size_t)kv_rank, st>>>(a));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_latent_vup") : 0;
}

int mbh_moe_route(const void* h, const void* w_router, const void* correction, void* dense, void* idx, void* wsel, int64_t T, int64_t width,
                  int64_t n, int64_t groups, int64_t keep, int64_t top, int score, float scale, int dt, void* stream) {
    if (T == 0) return 0;
    if (groups < 1 || n % groups || keep < 1 || keep > groups) return bad("mbh_moe_route: groups must divide the routed outputs, 1 <= keep <= groups");
    if (top < 1 || top > n / groups * keep) return bad("mbh_moe_route: top exceeds the eligible outputs");
    const size_t smem = sizeof(float) * (size_t)(2 * n + 2 * groups);
    if (smem > 48 * 1024) return bad("mbh_moe_route: too many routed outputs");
    if (score != 0 && score != 1) return bad("mbh_moe_route: score is 0 (softmax) or 1 (sigmoid)");
    MoeRouteArgs a{h, w_router, correction, (float*)dense, (int*)idx, (float*)wsel, (int)width, (int)n, (int)groups, (int)keep, (int)top, score, scale};
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, moe_route_kernel<ST><<<(unsigned)T, MOE_ROUTE_THREADS, smem, st>>>(a));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_moe_route") : 0;
}

int mbh_moe_sparse(const void* h, const void* w13, const void* w2, const void* idx, const void* wsel, void* act, void* y32, int64_t T, int64_t width,
                   int64_t ff, int64_t E, int64_t top, int glu, float limit, float alpha, int accumulate, int dt, void* stream) {
    if (T == 0) return 0;
    MoeSparseArgs a{h, w13, w2, (const int*)idx, (const float*)wsel, act, (float*)y32, (int)width, (int)ff, (int)E, (int)top, glu, limit, alpha, accumulate};
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, run_moe_sparse<ST>(a, T, st));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_moe_sparse") : 0;
}

int mbh_rows_axpy(void* y32, const void* h, const void* dense, int64_t T, int64_t n, int64_t first, int64_t D, int dt, void* stream) {
    if (T == 0 || first >= n) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, rows_axpy_kernel<ST><<<(unsigned)T, 128, 0, st>>>((float*)y32, (const ST*)h, (const float*)dense, (int)n, (int)first, (int)D));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_rows_axpy") : 0;
}

int mbh_linear_glu(const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K, float limit, float alpha, const void* rowscale,
                   int64_t rs_pitch, int64_t rs_group, int dt, void* stream) {
    if (N & 1) return bad("mbh_linear_glu: the gated epilogue needs interleaved (even) rows");
    if (rowscale && rs_group <= 0) return bad("mbh_linear_glu: rs_group must be positive");
    LinearArgs a{x, w, nullptr, out, nullptr, (int)M, (int)N, (int)K, EPI_GLU, 0, limit, alpha, (const float*)rowscale, (int)rs_pitch, (int)rs_group};
    cudaError_t e = cudaSuccess;
    DISPATCH(dt, e = launch_linear<ST>(a, (cudaStream_t)stream));
    return e ? fail(e, "mbh_linear_glu") : 0;
}

int mbh_glu_epilogue(const void* y, void* out, int64_t M, int64_t N, float limit, float alpha, const void* rowscale, int64_t rs_pitch, int64_t rs_group,
                     int dt, void* stream) {
    if (N & 1) return bad("mbh_glu_epilogue: odd N");
    if (rowscale && rs_group <= 0) return bad("mbh_glu_epilogue: rs_group must be positive");
    if (M == 0) return 0;
    LinearArgs a{nullptr, nullptr, nullptr, out, nullptr, (int)M, (int)N, 0, EPI_GLU, 0, limit, alpha, (const float*)rowscale, (int)rs_pitch, (int)rs_group};
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, run_epilogue<ST>(a, y, st));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_glu_epilogue") : 0;
}

int mbh_embed_pos(const void* tokens, const void* positions, const void* table, const void* pos_table, float scale, void* x32, int64_t T, int64_t D,
                  int dt, void* stream) {
    if (T == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, embed_pos_kernel<ST><<<(unsigned)T, 128, 0, st>>>((const int64_t*)tokens, (const int*)positions, (const ST*)table, (const ST*)pos_table,
                                                                    scale, (float*)x32, (int)D));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_embed_pos") : 0;
}

int mbh_rot_prep(const void* qkv, const void* freq, const void* positions, const void* cache_rows, void* q_out, void* k_out, void* v_out, void* ring_k,
                 void* ring_v, int64_t T, int64_t H, int64_t G, int64_t d, int64_t e, int64_t rot_dims, int unit_norm, float eps, int dt, void* stream) {
    if (T == 0) return 0;
    if (d > 64 * RP_MAXP) return bad("mbh_rot_prep: head size above 256");
    if (rot_dims > d || (rot_dims & 1)) return bad("mbh_rot_prep: rot_dims must be even and at most the head size");
    if (!k_out != !v_out) return bad("mbh_rot_prep: k_out and v_out come together");
    if (cache_rows && (!ring_k || !ring_v)) return bad("mbh_rot_prep: ring rows without a ring");
    RotPrepArgs a{qkv, (const double*)freq, (const int*)positions, (const int*)cache_rows, q_out, k_out, v_out, ring_k, ring_v,
                  (int)H, (int)G, (int)d, (int)e, (int)rot_dims, unit_norm, eps};
    cudaStream_t st = (cudaStream_t)stream;
    // few tokens (decode): the heads of a token are spread over CTAs; prompts: one CTA per token
    const unsigned hb = T < 512 ? (unsigned)((H + G + 3) / 4) : 1u;
    DISPATCH(dt, rot_prep_kernel<ST><<<dim3((unsigned)T, hb), 128, 0, st>>>(a));
    cudaError_t err = cudaGetLastError();
    return err ? fail(err, "mbh_rot_prep") : 0;
}

int mbh_kv_scatter(const void* k, const void* v, const void* cache_rows, void* ring_k, void* ring_v, int64_t T, int64_t Nk, int64_t Nv, int dt,
                   void* stream) {
    if (T == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, kv_scatter_kernel<ST><<<(unsigned)T, 128, 0, st>>>((const ST*)k, (const ST*)v, (const int*)cache_rows, (ST*)ring_k, (ST*)ring_v, (int)Nk,
                                                                    (int)Nv));
    cudaError_t err = cudaGetLastError();
    return err ? fail(err, "mbh_kv_scatter") : 0;
}

int mbh_gated_scan(const void* qab, const void* v, int64_t v_pitch, int64_t v_off, void* state, int64_t state_stride, const void* q_start,
                   const void* seqpos, const void* slots, void* o32, void* nq, int64_t T, int64_t B, int64_t H, int64_t d, int64_t e,
                   int ones, int64_t chunk_len, int64_t chunks, void* scratch, int dt, void* stream) {
    if (B == 0 || T == 0) return 0;
    if (!ones != !nq) return bad("mbh_gated_scan: the normaliser column and its output come together");
    if (d > 2048) return bad("mbh_gated_scan: key size above 2048");
    if (chunks > 1 && (chunk_len < 1 || !scratch || chunks > 65535)) return bad("mbh_gated_scan: chunks need a length and scratch");
    const int ec = (int)e + (ones ? 1 : 0);
    GatedScanArgs a{(const float*)qab, v, (int)v_pitch, (int)v_off, (float*)state, (int)state_stride, (const int*)q_start, (const int*)seqpos,
                    (const int*)slots, (float*)o32, (float*)nq, (int)B, (int)H, (int)d, (int)e, ones ? 1 : 0, (int)chunk_len, (float*)scratch,
                    scratch ? (float*)scratch + (size_t)B * H * chunks * d * ec : nullptr, (int)((d + 127) / 128)};
    cudaError_t err = cudaSuccess;
    if (a.key_blocks > 1) {  // the key blocks' CTAs add their partial outputs
        err = cudaMemsetAsync(o32, 0, sizeof(float) * (size_t)T * H * e, (cudaStream_t)stream);
        if (err) return fail(err, "mbh_gated_scan");
    }
    if (chunks > 1) DISPATCH(dt, err = launch_gated_scan_chunked<ST>(a, (int)chunks, (cudaStream_t)stream));
    else DISPATCH(dt, err = launch_gated_scan<ST>(a, (cudaStream_t)stream));
    return err ? fail(err, "mbh_gated_scan") : 0;
}

int mbh_hgrn2_gates(const void* qfv, const void* lower, void* qab, int64_t T, int64_t Hd, int64_t pitch, int dt, void* stream) {
    if (T == 0) return 0;
    Hgrn2GateArgs a{qfv, lower, (float*)qab, (int)Hd, (int)pitch};
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned jb = T < 512 ? (unsigned)((Hd + 255) / 256) : 1u;
    DISPATCH(dt, hgrn2_gates_kernel<ST><<<dim3((unsigned)T, jb), 256, 0, st>>>(a));
    cudaError_t err = cudaGetLastError();
    return err ? fail(err, "mbh_hgrn2_gates") : 0;
}

int mbh_mlstm_gates(const void* qkvg, const void* gif, void* gates, void* qab, void* state, int64_t state_stride, int64_t m_off, const void* q_start,
                    const void* seqpos, const void* slots, int64_t T, int64_t B, int64_t H, int64_t d, int64_t pitch, float cap, float qscale, int dt,
                    void* stream) {
    if (T == 0) return 0;
    MlstmGateArgs a{qkvg, (const float*)gif, (float*)gates, (float*)qab, (float*)state, (int)state_stride, (int)m_off, (const int*)q_start, (const int*)seqpos,
                    (const int*)slots, (int)H, (int)d, (int)pitch, cap, qscale};
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, run_mlstm_gates<ST>(a, B, T, st));
    cudaError_t err = cudaGetLastError();
    return err ? fail(err, "mbh_mlstm_gates") : 0;
}

int mbh_scan_post(const void* o32, const void* nq, int64_t d, const void* gates, const void* w, int w_per_head, const void* gate, int64_t g_pitch,
                  int64_t g_off, int gate_act, void* y, int64_t T, int64_t H, int64_t e, int ones, float eps, int dt, void* stream) {
    if (T == 0) return 0;
    if (ones && (!gates || !nq)) return bad("mbh_scan_post: a normaliser needs its products and the gates");
    ScanPostArgs a{(const float*)o32, (const float*)nq, (int)d, (const float*)gates, w, w_per_head, gate, (int)g_pitch, (int)g_off, gate_act, y, (int)H, (int)e, ones ? 1 : 0, eps};
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned hb = T < 512 ? (unsigned)((H + 3) / 4) : 1u;
    DISPATCH(dt, scan_post_kernel<ST><<<dim3((unsigned)T, hb), 128, 0, st>>>(a));
    cudaError_t err = cudaGetLastError();
    return err ? fail(err, "mbh_scan_post") : 0;
}

int mbh_canon_conv(const void* x32, const void* w, void* state, int64_t state_stride, int64_t state_off, const void* q_start, const void* seqpos,
                   const void* slots, void* h, int64_t T, int64_t B, int64_t D, int64_t taps, int one_each, int dt, void* stream) {
    if (T == 0) return 0;
    if (taps < 1) return bad("mbh_canon_conv: at least one tap");
    if (one_each && T != B) return bad("mbh_canon_conv: one token per sequence means T == B");
    CanonArgs a{(const float*)x32, w, (float*)state, (int)state_stride, (int)state_off, (const int*)q_start, (const int*)seqpos, (const int*)slots, h,
                (int)B, (int)D, (int)taps};
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned cb = (unsigned)((D + 255) / 256);
    if (one_each) {
        DISPATCH(dt, canon_conv_step_kernel<ST><<<dim3((unsigned)B, cb), 256, 0, st>>>(a));
    } else {
        // the tiled kernel for the usual few taps and channel counts it can load four at a time; the plain one for everything else
        const bool tiled = taps <= 8 && D % 4 == 0 && (reinterpret_cast<uintptr_t>(x32) | reinterpret_cast<uintptr_t>(h) | reinterpret_cast<uintptr_t>(state)) % 16 == 0
                           && (state_stride % 4 == 0) && (state_off % 4 == 0);
        if (tiled) {
            const dim3 grid((unsigned)((T + CANON_TILE - 1) / CANON_TILE), (unsigned)((D / 4 + 127) / 128));
#define MBH_CANON(TP) case TP: DISPATCH(dt, canon_conv_tiled_kernel<ST, TP><<<grid, 128, 0, st>>>(a, (int)T)); break;
            switch ((int)taps) { MBH_CANON(1) MBH_CANON(2) MBH_CANON(3) MBH_CANON(4) MBH_CANON(5) MBH_CANON(6) MBH_CANON(7) MBH_CANON(8) }
#undef MBH_CANON
        } else {
            DISPATCH(dt, canon_conv_kernel<ST><<<dim3((unsigned)T, cb), 256, 0, st>>>(a));
        }
        if (taps > 1) canon_state_kernel<<<dim3((unsigned)B, cb), 256, 0, st>>>(a);
    }
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_canon_conv") : 0;
}

int mbh_rmsnorm_add(const void* y32, const void* w, void* acc32, int64_t T, int64_t D, float eps, const void* stack, int64_t stack_stride,
                    const void* coef, int64_t n, void* out32, int dt, void* stream) {
    if (T == 0) return 0;
    if (stack && (!coef || !out32 || n < 1)) return bad("mbh_rmsnorm_add: the depth average needs coefficients and an output");
    NormAddArgs a{(const float*)y32, w, (float*)acc32, (int)D, eps, (const float*)stack, (size_t)stack_stride, coef, (int)n, (float*)out32};
    cudaStream_t st = (cudaStream_t)stream;
    const int threads = D >= 1024 ? 256 : 128;
    const unsigned cb = T <= 32 ? (unsigned)((D + 2 * threads - 1) / (2 * threads)) : 1u;  // few rows: two columns per thread, many CTAs
    DISPATCH(dt, rmsnorm_add_kernel<ST><<<dim3((unsigned)T, cb), threads, 0, st>>>(a));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_rmsnorm_add") : 0;
}

int mbh_depth_mix(const void* stack, int64_t stack_stride, const void* coef, int64_t n, void* out32, int64_t count, int dt, void* stream) {
    if (count == 0) return 0;
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, depth_mix_kernel<ST><<<(unsigned)((count + 255) / 256), 256, 0, st>>>((const float*)stack, (size_t)stack_stride, (const ST*)coef, (int)n,
                                                                                         (float*)out32, (size_t)count));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_depth_mix") : 0;
}

int mbh_retention_qab(const void* qk, int64_t pitch, const void* freq, const void* decay, const void* positions, void* qab, int64_t T, int64_t H,
                      int64_t d, int64_t rot_dims, float kscale, int dt, void* stream) {
    if (T == 0) return 0;
    if (rot_dims < 0 || rot_dims > d || (rot_dims & 1)) return bad("mbh_retention_qab: the rotation covers an even number of a head's entries");
    RetentionQabArgs a{qk, (const double*)freq, (const float*)decay, (const int*)positions, (float*)qab, (int)H, (int)d, (int)pitch, (int)rot_dims, kscale};
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned jb = T < 512 ? (unsigned)((H * d + 255) / 256) : 1u;
    DISPATCH(dt, retention_qab_kernel<ST><<<dim3((unsigned)T, jb), 256, 0, st>>>(a));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_retention_qab") : 0;
}

int mbh_gla_qab(const void* qk, int64_t pitch, const void* z32, void* qab, int64_t T, int64_t Hd, float qscale, float inv_tau, int dt, void* stream) {
    if (T == 0) return 0;
    GlaQabArgs a{qk, (const float*)z32, (float*)qab, (int)Hd, (int)pitch, qscale, inv_tau};
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned jb = T < 512 ? (unsigned)((Hd + 255) / 256) : 1u;
    DISPATCH(dt, gla_qab_kernel<ST><<<dim3((unsigned)T, jb), 256, 0, st>>>(a));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_gla_qab") : 0;
}

int mbh_whole_norm_prep(const void* qkv, const void* qnorm, const void* knorm, const void* cache_rows, void* q_out, void* k_out, void* v_out,
                        void* ring_k, void* ring_v, int64_t T, int64_t Nq, int64_t Nk, int64_t Nv, float eps, int dt, void* stream) {
    if (T == 0) return 0;
    if (cache_rows && (!ring_k || !ring_v)) return bad("mbh_whole_norm_prep: ring rows without a ring");
    WholeNormPrepArgs a{qkv, qnorm, knorm, (const int*)cache_rows, q_out, k_out, v_out, ring_k, ring_v, (int)Nq, (int)Nk, (int)Nv, eps};
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, whole_norm_prep_kernel<ST><<<(unsigned)T, 256, 0, st>>>(a));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_whole_norm_prep") : 0;
}

int mbh_linear_relu2(const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K, const void* rowscale, int64_t rs_pitch,
                     int64_t rs_group, int dt, void* stream) {
    if (rowscale && rs_group <= 0) return bad("mbh_linear_relu2: rs_group must be positive");
    LinearArgs a{x, w, nullptr, out, nullptr, (int)M, (int)N, (int)K, EPI_RELU2, 0, 0.f, 0.f, (const float*)rowscale, (int)rs_pitch, (int)rs_group};
    cudaError_t e = cudaSuccess;
    DISPATCH(dt, e = launch_linear<ST>(a, (cudaStream_t)stream));
    return e ? fail(e, "mbh_linear_relu2") : 0;
}

int mbh_relu2_epilogue(const void* y, void* out, int64_t M, int64_t N, const void* rowscale, int64_t rs_pitch, int64_t rs_group, int dt,
                       void* stream) {
    if (M == 0 || N == 0) return 0;
    if (N & 1) return bad("mbh_relu2_epilogue: N must be even");
    if (rowscale && rs_group <= 0) return bad("mbh_relu2_epilogue: rs_group must be positive");
    LinearArgs a{nullptr, nullptr, nullptr, out, nullptr, (int)M, (int)N, 0, EPI_RELU2, 0, 0.f, 0.f, (const float*)rowscale, (int)rs_pitch, (int)rs_group};
    cudaStream_t st = (cudaStream_t)stream;
    DISPATCH(dt, run_epilogue<ST>(a, y, st));
    cudaError_t e = cudaGetLastError();
    return e ? fail(e, "mbh_relu2_epilogue") : 0;
}

}  // extern "C"
