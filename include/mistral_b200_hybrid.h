/* C ABI of libmb200_hybrid.so: kernels of layered decoders (a list of layers, each with its own kind of token mixer),
 * with an fp32 residual stream and bf16 or fp32 storage of activations and weights.
 *
 * Conventions: pointers are device pointers; `dt` = 0 (bf16) or 1 (fp32) is the storage type of every `void*` activation
 * and weight operand; index tensors are int32 unless said otherwise; `stream` is a cudaStream_t.  Every call returns 0 or
 * an error code and leaves the text in mbh_last_error().  No call synchronises or allocates.
 */
#ifndef MISTRAL_B200_HYBRID_H
#define MISTRAL_B200_HYBRID_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MBH_ABI_VERSION 4

int mbh_abi_version(void);
const char* mbh_last_error(void);

/* x32[t, :] = table[tokens[t], :] * scale.  tokens: int64 [T]; table [V, D]; x32: fp32 [T, D]. */
int mbh_embed_scale(const void* tokens, const void* table, float scale, void* x32, int64_t T, int64_t D, int dt, void* stream);

/* y[t, :] = x32[t, :] / sqrt(mean(x32[t]^2) + eps) * w.  x32 fp32 [T, D] (the residual stream); y, w: storage type. */
int mbh_rmsnorm(const void* x32, const void* w, void* y, int64_t T, int64_t D, float eps, int dt, void* stream);

/* Linear x[M, K] W[N, K]^T (+ bias[N]) with an epilogue:
 *   0  out[M, N] = act(.)      SiLU on columns < n_act, identity elsewhere
 *   1  out32[M, N] += .        in-place add into the fp32 residual stream
 *   2  out[M, N/2]             rows of W interleaved (2c gate, 2c+1 up): g = min(gate, limit), u = clamp(up, -limit, limit),
 *                              out = g * sigmoid(alpha * g) * (u + 1)
 *   3  out32[M, N] = .         fp32 result (logits); with limit > 0: limit * tanh(. / limit)
 *   5  out32[M, N] += alpha * .  the residual add of epilogue 1 with a fixed weight
 * Any M, N, K.  M <= 8 runs the weight-streaming kernel, larger M the tiled one (tensor cores for bf16). */
int mbh_linear(const void* x, const void* w, const void* bias, void* out, void* out32, int64_t M, int64_t N, int64_t K, int epi, int64_t n_act,
               float limit, float alpha, int dt, void* stream);

/* The epilogues of mbh_linear alone, applied to y[M, N] (storage type, N even) that another GEMM produced. */
int mbh_linear_epilogue(const void* y, const void* bias, void* out, void* out32, int64_t M, int64_t N, int epi, int64_t n_act, float limit, float alpha,
                        int dt, void* stream);

/* Splits qkv[T, H*d + G*d + G*e]; RMS-norms every q and k head over d with the shared weights qnorm / knorm [d] (null: no
 * norm); multiplies q at position p by 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1) (temp_every = 0: no temperature);
 * value mixing: vmix_mode 0 none, 1 copy v to v_first[T, G*e], 2 v <- (1 - *vmix) v + *vmix v_first; then scatters k and v to
 * row cache_rows[t] of cache_k [rows, G, d] / cache_v [rows, G, e] (-1: not cached) and writes q_out [T, H*d]. */
int mbh_attn_prep(const void* qkv, const void* qnorm, const void* knorm, const void* positions, const void* cache_rows, void* q_out, void* cache_k,
                  void* cache_v, void* v_first, const void* vmix, int vmix_mode, int64_t T, int64_t H, int64_t G, int64_t d, int64_t e, float eps,
                  float temp_coef, int64_t temp_every, int dt, void* stream);

/* Causal softmax attention of q[T, H*d] over the ring: token t of sequence b (q_start[B+1]) at position positions[t] sees keys
 * 0..position of cache block slots[b] (W rows each, key j in row j % W); score = q.k * scale + bias_tab[min(distance, n_tab-1), h]
 * (fp32 [n_tab, H]; null: no bias).  out [T, H*e].
 * n_tiles > 0 (prompts): the number of 64-query tiles, sum over sequences of ceil(len / 64); with bf16 storage and key/value
 * sizes among {32, 64, 128} the tensor-core kernel runs (P rounded to bf16 before P V).  n_tiles = 0: the exact fp32 kernel,
 * with `splits` > 1 CTAs per (token, head) along the keys (decode) and their partial results in scratch (fp32 [T*H, splits, 2 + e]). */
int mbh_attn_bias(const void* q, const void* cache_k, const void* cache_v, const void* bias_tab, int64_t n_tab, const void* positions,
                  const void* q_start, const void* slots, void* out, int64_t T, int64_t B, int64_t W, int64_t H, int64_t G, int64_t d, int64_t e,
                  float scale, int64_t n_tiles, int64_t splits, void* scratch, int dt, void* stream);

/* Decayed linear attention.  qkvg [T, 2*H*d + 2*H*e] = q | k | v | gate; per head S <- decay[h] S + k v^T, o = S^T q, fp32;
 * state fp32 [slots, H, d, e] is read (unless seqpos[b] == 0: starts at zero) and written back; o32 fp32 [T, H*e]. */
int mbh_lightning_scan(const void* qkvg, void* state, const void* decay, const void* q_start, const void* seqpos, const void* slots, void* o32,
                       int64_t B, int64_t H, int64_t d, int64_t e, int dt, void* stream);

/* y[t, :] = rms_norm(o32[t, :N]; eps) * w * sigmoid(g[t * g_pitch + g_off + :N]). */
int mbh_gated_headnorm(const void* o32, const void* w, const void* g, int64_t g_pitch, int64_t g_off, void* y, int64_t T, int64_t N, float eps,
                       int dt, void* stream);

/* x32[t, :] += table[tokens[t], :] * scale (the embedding added again to the residual stream). */
int mbh_embed_add(const void* tokens, const void* table, float scale, void* x32, int64_t T, int64_t D, int dt, void* stream);

/* Layer norm of fp32 rows x32 [T, D]: (x - mean) / sqrt(var + eps) * w + b, var = mean of the squared deviations; b may be null.
 * Exactly one of y (storage type [T, D]: y = norm) and acc32 (fp32 [T, D]: acc32 += norm, in fp32) is given. */
int mbh_layernorm(const void* x32, const void* w, const void* b, void* y, void* acc32, int64_t T, int64_t D, float eps, int dt, void* stream);

/* Linear with interleaved gate/up rows (as epilogue 2 of mbh_linear) and out[M, N/2] = silu(gate) * up * rowscale[m, c / rs_group];
 * rowscale: fp32 [M, rs_pitch] or null (no scaling).  mbh_swiglu_epilogue applies the same to y[M, N] of another GEMM. */
int mbh_linear_swiglu(const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K, const void* rowscale, int64_t rs_pitch,
                      int64_t rs_group, int dt, void* stream);
int mbh_swiglu_epilogue(const void* y, void* out, int64_t M, int64_t N, const void* rowscale, int64_t rs_pitch, int64_t rs_group, int dt,
                        void* stream);

/* Latent attention, input side.  y [T, pitch] = [query latent (q_rank) | key/value latent (kv_rank) | shared rotated key part
 * (rot_dim) | ...].  cq [T, q_rank] = rms_norm(query latent) * qnorm; ring row cache_rows[t] (-1: not cached) of ring
 * [rows, kv_rank + rot_dim] = [rms_norm(kv latent) * cnorm | rot(key part)].  rot: the pairs (2i, 2i+1), i < rot_dims / 2, turn by
 * positions[t] * freq[i] (freq: float64 [rot_dims / 2]), cos and sin times mag; entries from rot_dims on pass unchanged. */
int mbh_latent_prep(const void* y, const void* qnorm, const void* cnorm, const void* freq, const void* positions, const void* cache_rows, void* cq,
                    void* ring, int64_t T, int64_t pitch, int64_t q_rank, int64_t kv_rank, int64_t rot_dim, int64_t rot_dims, float eps, float mag,
                    int dt, void* stream);

/* q [T, H, dn + rot_dim] -> qa [T, H, kv_rank + rot_dim] = [W_uk[h]^T q[:dn] | rot(q[dn:])], w_uk [H * dn, kv_rank].
 * w_uk null: no folding, qa [T, H, dn + rot_dim] = [q[:dn] | rot(q[dn:])]. */
int mbh_latent_absorb(const void* q, const void* w_uk, const void* freq, const void* positions, void* qa, int64_t T, int64_t H, int64_t dn,
                      int64_t rot_dim, int64_t rot_dims, int64_t kv_rank, float mag, int dt, void* stream);

/* Keys and values per head of whole prompts, for ordinary multi-head attention (mbh_attn_bias with bias_tab null): token t at
 * position p of sequence b goes to row b * Wt + p of kfull [B * Wt, H, dn + rot_dim] = [kn[t, h] | rotated key part of ring row
 * cache_rows[t]] and vfull [B * Wt, H, dv] = v[t, h].  kn [T, H * dn], v [T, H * dv]. */
int mbh_latent_expand(const void* kn, const void* v, const void* ring, const void* positions, const void* cache_rows, const void* q_start, void* kfull,
                      void* vfull, int64_t T, int64_t B, int64_t Wt, int64_t H, int64_t dn, int64_t rot_dim, int64_t dv, int64_t kv_rank, int dt,
                      void* stream);

/* out [T, H, dv] *= sigmoid(gate[t * g_pitch + g_off + h]), in place. */
int mbh_head_gate(void* out, const void* gate, int64_t g_pitch, int64_t g_off, int64_t T, int64_t H, int64_t dv, int dt, void* stream);

/* Causal softmax attention of qa over latent rows: score = qa . ring row * scale, value = the row's first kv_rank entries;
 * o_lat [T, H, kv_rank].  Ring addressing, splits and scratch as mbh_attn_bias (exact fp32 kernel, one key/value head). */
int mbh_attn_latent(const void* qa, const void* ring, const void* positions, const void* q_start, const void* slots, void* o_lat, int64_t T,
                    int64_t B, int64_t W, int64_t H, int64_t kv_rank, int64_t rot_dim, float scale, int64_t splits, void* scratch, int dt,
                    void* stream);

/* The same for one token per sequence (token b belongs to sequence b; qa [B, H, kv_rank + rot_dim]): each CTA reads a span of one
 * sequence's rows once for all heads.  H <= 32, kv_rank <= 512; scratch fp32 [B * H, splits, 2 + kv_rank], splits >= 1. */
int mbh_attn_latent_decode(const void* qa, const void* ring, const void* positions, const void* slots, void* o_lat, int64_t B, int64_t W, int64_t H,
                           int64_t kv_rank, int64_t rot_dim, float scale, int64_t splits, void* scratch, int dt, void* stream);

/* out [T, H * dv] = (W_uv[h] o_lat[t, h]) * sigmoid(gate[t * g_pitch + g_off + h]); w_uv [H * dv, kv_rank]; gate null: no gate. */
int mbh_latent_vup(const void* o_lat, const void* w_uv, const void* gate, int64_t g_pitch, int64_t g_off, void* out, int64_t T, int64_t H,
                   int64_t dv, int64_t kv_rank, int dt, void* stream);

/* Router of a mixture of experts, fp32: s = softmax(W_r h) over n outputs (score 0) or sigmoid of each output (score 1), choice = s + correction (null: none); the outputs form
 * `groups` equal groups of neighbours and only those of the `keep` groups with the largest choice stay eligible; the `top` largest
 * eligible choices are taken, weighted by s * scale.  dense: fp32 [T, n] (0 where not chosen); idx int32 / wsel fp32 [T, top]. */
int mbh_moe_route(const void* h, const void* w_router, const void* correction, void* dense, void* idx, void* wsel, int64_t T, int64_t width,
                  int64_t n, int64_t groups, int64_t keep, int64_t top, int score, float scale, int dt, void* stream);

/* The chosen experts of few tokens: y32 [T, width] = sum_k wsel[t, k] * expert(idx[t, k])(h[t]); an index >= E is an identity
 * expert (output = h[t]).  w13 [E * 2 * ff, width] (gate and up rows interleaved), w2 [width, E * ff]; act: scratch [T * top, ff].
 * glu 0: experts silu(gate) * up.  glu 1: the weight multiplies the expert's INPUT and the unit is the clamped one of mbh_linear's
 * epilogue 2: y32 = sum_k expert(wsel[t, k] * h[t]), g = min(w gate, limit), u = clamp(w up, -limit, limit).
 * glu 2: experts without a gate, W_down max(W_up h, 0)^2, with w13 [E * ff, width] plain rows; the weight multiplies the OUTPUT.
 * accumulate 1: the sum is ADDED to y32 (the fp32 residual stream) instead of stored. */
int mbh_moe_sparse(const void* h, const void* w13, const void* w2, const void* idx, const void* wsel, void* act, void* y32, int64_t T, int64_t width,
                   int64_t ff, int64_t E, int64_t top, int glu, float limit, float alpha, int accumulate, int dt, void* stream);

/* y32[t, :] += (dense[t, first] + ... + dense[t, n - 1]) * h[t, :]. */
int mbh_rows_axpy(void* y32, const void* h, const void* dense, int64_t T, int64_t n, int64_t first, int64_t D, int dt, void* stream);

/* mbh_attn_bias with a sliding window and a ring that may be shorter than the sequence.  window > 0: the token at position p sees keys
 * p - window + 1 .. p only.  own_k [T, G*d] / own_v [T, G*e] (token-major, with seqpos [B] = tokens cached before this call): keys and
 * values of THIS call's tokens, read from there instead of the ring, so that a prompt longer than the ring finds all its keys; the ring
 * is written after attention (mbh_kv_scatter).  Without them every visible key must be in the ring (W >= min(window, sequence length)).
 * chunk: keys per warp and step of the exact kernel, 1 .. 128 (0: 128); with `splits` CTAs of 4 warps per (token, head) a CTA takes
 * 4 * chunk keys per round, so a short ring read by few tokens is spread over splits = ceil(W / (4 * chunk)) CTAs.
 * weights 0: softmax over the visible keys.  weights 1: every visible key weighs sigmoid(score) and nothing is normalised (bias_tab with
 * n_tab = 1 is then a number per head inside the sigmoid). */
int mbh_attn_window(const void* q, const void* cache_k, const void* cache_v, const void* bias_tab, int64_t n_tab, const void* positions,
                    const void* q_start, const void* slots, void* out, int64_t T, int64_t B, int64_t W, int64_t H, int64_t G, int64_t d, int64_t e,
                    float scale, int64_t n_tiles, int64_t splits, void* scratch, int64_t window, const void* own_k, const void* own_v,
                    const void* seqpos, int64_t chunk, int weights, int dt, void* stream);

/* Linear with interleaved gate/up rows and the clamped gated unit of mbh_linear's epilogue 2; gate and up of column c are multiplied by
 * rowscale[m, c / rs_group] (fp32 [M, rs_pitch]; null: 1) BEFORE the clamps.  mbh_glu_epilogue applies the same to y[M, N] of another GEMM. */
int mbh_linear_glu(const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K, float limit, float alpha, const void* rowscale,
                   int64_t rs_pitch, int64_t rs_group, int dt, void* stream);
int mbh_glu_epilogue(const void* y, void* out, int64_t M, int64_t N, float limit, float alpha, const void* rowscale, int64_t rs_pitch, int64_t rs_group,
                     int dt, void* stream);

/* x32[t, :] = table[tokens[t], :] * scale + pos_table[positions[t], :] (learned positions; positions int32 [T]). */
int mbh_embed_pos(const void* tokens, const void* positions, const void* table, const void* pos_table, float scale, void* x32, int64_t T, int64_t D,
                  int dt, void* stream);

/* Splits qkv[T, H*d + G*d + G*e]; rotates the first rot_dims entries of every q and k head as interleaved pairs (2i, 2i + 1) by the angle
 * positions[t] * freq[i] (freq: float64 [rot_dims / 2]); with unit_norm divides every rotated head by sqrt(mean(x^2) + eps).  Writes
 * q_out [T, H*d]; k_out [T, G*d] and v_out [T, G*e] (both or neither); and, when cache_rows is given, k and v of token t into ring row
 * cache_rows[t] (-1: not cached). */
int mbh_rot_prep(const void* qkv, const void* freq, const void* positions, const void* cache_rows, void* q_out, void* k_out, void* v_out, void* ring_k,
                 void* ring_v, int64_t T, int64_t H, int64_t G, int64_t d, int64_t e, int64_t rot_dims, int unit_norm, float eps, int dt, void* stream);

/* ring_k[cache_rows[t]] = k[t] (Nk entries), ring_v[cache_rows[t]] = v[t] (Nv entries) for every t with cache_rows[t] >= 0. */
int mbh_kv_scatter(const void* k, const void* v, const void* cache_rows, void* ring_k, void* ring_v, int64_t T, int64_t Nk, int64_t Nv, int dt,
                   void* stream);

/* Gated linear recurrence per head: S <- diag(a_t) S + b_t v_t^T, o_t = S^T q_t.  qab fp32 [T, 3, H*d] = q | a | b; value (t, h, c) at
 * v[t * v_pitch + v_off + h*e + c] (storage type); state fp32 [slots, state_stride], head h's matrix [d, e + ones] at h * d * (e + ones),
 * read (unless seqpos[b] == 0: zero) and written back; o32 fp32 [T, H * e].  ones = 1: one more state column whose value is 1 for every
 * token (a normaliser n <- a n + b); nq fp32 [T, H * d] gets n_t[i] * q_t[i] (summed over d by mbh_scan_post); ones = 0: nq null.
 * chunks > 1 (long prompts): the same recurrence chunk-parallel, `chunks` = ceil(longest sequence / chunk_len) chunks of chunk_len
 * tokens per sequence; scratch: fp32 [B*H*chunks*d*(e + ones + 1)].  chunks <= 1: one CTA column walks each sequence; no scratch.
 * Key sizes above 128 are split into blocks of 128 keys over CTAs that add their partial outputs into o32 (T tokens, zeroed first). */
int mbh_gated_scan(const void* qab, const void* v, int64_t v_pitch, int64_t v_off, void* state, int64_t state_stride, const void* q_start,
                   const void* seqpos, const void* slots, void* o32, void* nq, int64_t T, int64_t B, int64_t H, int64_t d, int64_t e,
                   int ones, int64_t chunk_len, int64_t chunks, void* scratch, int dt, void* stream);

/* HGRN2 gates from qfv [T, pitch] = silu(q) | f_pre | v: f = lower + (1 - lower) * sigmoid(f_pre); qab [T, 3, Hd] = q | f | 1 - f. */
int mbh_hgrn2_gates(const void* qfv, const void* lower, void* qab, int64_t T, int64_t Hd, int64_t pitch, int dt, void* stream);

/* mLSTM gates.  gif fp32 [T, 2H] = i_pre | f_pre; i = cap tanh(i_pre / cap), f = logsigmoid(cap tanh(f_pre / cap)); the running maximum
 * m_t = max(f + m_(t-1), i) starts at 0 (seqpos[b] == 0) or at state[slot * state_stride + m_off + h] and is written back there.
 * gates fp32 [T, H, 3] = exp(f + m_(t-1) - m_t), exp(i - m_t), exp(-m_t); qab [T, 3, H*d] = q * qscale | decay | exp(i - m_t) k, with
 * q and k the first two blocks of qkvg [T, pitch]. */
int mbh_mlstm_gates(const void* qkvg, const void* gif, void* gates, void* qab, void* state, int64_t state_stride, int64_t m_off, const void* q_start,
                    const void* seqpos, const void* slots, int64_t T, int64_t B, int64_t H, int64_t d, int64_t pitch, float cap, float qscale, int dt,
                    void* stream);

/* After a scan: o = o32[t, h, :e] (divided by max(|sum_i nq[t, h, i]|, gates[t, h, 2]) + 1e-6 with ones = 1; nq [T, H * d]); y = o / sqrt(mean(o^2) + eps) * w
 * (w [H*e] with w_per_head, else [e] shared by the heads; null: no weight) * act(gate[t * g_pitch + g_off + h*e + c]) (gate null: none;
 * gate_act 0: sigmoid, 1: SiLU).  y [T, H*e]. */
int mbh_scan_post(const void* o32, const void* nq, int64_t d, const void* gates, const void* w, int w_per_head, const void* gate, int64_t g_pitch,
                  int64_t g_off, int gate_act, void* y, int64_t T, int64_t H, int64_t e, int ones, float eps, int dt, void* stream);

/* h[t] = x32[t] + sum_j w[:, j] * x32[t - taps + 1 + j] over the tokens of t's sequence: a causal convolution over time on every channel
 * (w [D, taps], storage type), added to its input; inputs before the sequence's start are zero.  The last taps - 1 inputs of the
 * sequence in slot s are kept, fp32 [taps - 1, D], at state + s * state_stride + state_off: read when seqpos[b] > 0, written back by
 * this call.  h [T, D] storage type.  one_each = 1: one token per sequence (T == B), one launch. */
int mbh_canon_conv(const void* x32, const void* w, void* state, int64_t state_stride, int64_t state_off, const void* q_start, const void* seqpos,
                   const void* slots, void* h, int64_t T, int64_t B, int64_t D, int64_t taps, int one_each, int dt, void* stream);

/* acc32[t] += y32[t] / sqrt(mean(y32[t]^2) + eps) * w (fp32 rows [T, D]; w storage type): the norm of a sublayer's output on its way into
 * the residual stream.  With stack: afterwards out32[t] = sum_(j < n - 1) coef[j] * stack[j * stack_stride + t * D ..] + coef[n - 1] *
 * acc32[t], the weighted average over the results of the layers so far (coef [n] storage type; stack_stride in floats). */
int mbh_rmsnorm_add(const void* y32, const void* w, void* acc32, int64_t T, int64_t D, float eps, const void* stack, int64_t stack_stride,
                    const void* coef, int64_t n, void* out32, int dt, void* stream);

/* out32[i] = sum_(j < n) coef[j] * stack[j * stack_stride + i], i < count. */
int mbh_depth_mix(const void* stack, int64_t stack_stride, const void* coef, int64_t n, void* out32, int64_t count, int dt, void* stream);

/* Retention gates from qk [T, pitch] = q (H*d) | k (H*d) | ...: the first rot_dims entries of each head turn by positions[t] * freq[i]
 * (freq float64 [rot_dims / 2]), entry i paired with entry i + rot_dims / 2; qab fp32 [T, 3, H*d] = rot(q) | decay[h] | rot(k) * kscale. */
int mbh_retention_qab(const void* qk, int64_t pitch, const void* freq, const void* decay, const void* positions, void* qab, int64_t T, int64_t H,
                      int64_t d, int64_t rot_dims, float kscale, int dt, void* stream);

/* Gated-linear-attention gates: qab fp32 [T, 3, Hd] = q * qscale | exp(logsigmoid(z32) * inv_tau) | k, z32 fp32 [T, Hd]. */
int mbh_gla_qab(const void* qk, int64_t pitch, const void* z32, void* qab, int64_t T, int64_t Hd, float qscale, float inv_tau, int dt, void* stream);

/* Splits qkv [T, Nq + Nk + Nv]; q <- rms_norm(q) * qnorm over all Nq entries, k <- rms_norm(k) * knorm over all Nk entries.  Outputs as
 * mbh_rot_prep: q_out [T, Nq]; k_out / v_out token-major or null; ring rows cache_rows[t] (null: no ring write; -1: not cached). */
int mbh_whole_norm_prep(const void* qkv, const void* qnorm, const void* knorm, const void* cache_rows, void* q_out, void* k_out, void* v_out,
                        void* ring_k, void* ring_v, int64_t T, int64_t Nq, int64_t Nk, int64_t Nv, float eps, int dt, void* stream);

/* out[M, N] = max(x W^T, 0)^2 * rowscale[m, n / rs_group] (rowscale fp32 [M, rs_pitch] or null); mbh_relu2_epilogue applies the same to
 * y[M, N] (N even) of another GEMM. */
int mbh_linear_relu2(const void* x, const void* w, void* out, int64_t M, int64_t N, int64_t K, const void* rowscale, int64_t rs_pitch,
                     int64_t rs_group, int dt, void* stream);
int mbh_relu2_epilogue(const void* y, void* out, int64_t M, int64_t N, const void* rowscale, int64_t rs_pitch, int64_t rs_group, int dt,
                       void* stream);

#ifdef __cplusplus
}
#endif
#endif
