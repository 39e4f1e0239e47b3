"""Attention / FeedForward / RMSNorm / TransformerBlock (API mirror of mistral_inference/transformer_layers.py).

The classes keep the reference's names and wiring, but every FLOP goes through libmb200 (C ABI in
include/mistral_b200.h); weights are stored pre-packed for the fused kernels:
  Attention.wqkv  [(H + 2*KV) * hd, dim] = wq ++ wk ++ wv        (one GEMM / one weight stream)
  FeedForward.w13 [2 * hidden, dim], row 2i = w1[i], row 2i+1 = w3[i]  (SiLU*mul in the epilogue)
`wq/wk/wv/w1/w3` are exposed as zero-copy views for state-dict compatibility.
"""
from typing import List, Optional, Tuple

import torch
from torch import nn

from . import _abi
from .args import LoraArgs, MoeArgs
from .cache import CacheView
from .moe import MoeLayer


class _WeightView:
    """Stands in for an nn.Linear whose weight is a view into a packed parameter."""

    def __init__(self, getter):
        self._getter = getter

    @property
    def weight(self) -> torch.Tensor:
        return self._getter()


class RMSNorm(nn.Module):
    """transformer_layers.py:109-120."""

    def __init__(self, dim: int, eps: float = 1e-6):
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim), requires_grad=False)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return _abi.rmsnorm(x, self.weight, self.eps)


class Attention(nn.Module):
    """transformer_layers.py:31-93."""

    def __init__(self, dim: int, n_heads: int, head_dim: int, n_kv_heads: int, lora: Optional[LoraArgs] = None):
        super().__init__()
        assert lora is None, "LoRA adapters must be merged into the weights (lora.py:118-139); unmerged LoRA is out of scope"
        self.dim = dim
        self.n_heads = n_heads
        self.head_dim = head_dim
        self.n_kv_heads = n_kv_heads
        self.repeats = n_heads // n_kv_heads
        self.scale = head_dim ** -0.5
        self.q_dim = n_heads * head_dim
        self.kv_dim = n_kv_heads * head_dim
        self.wqkv = nn.Parameter(torch.empty(self.q_dim + 2 * self.kv_dim, dim), requires_grad=False)
        self.wo_weight = nn.Parameter(torch.empty(dim, self.q_dim), requires_grad=False)

    # state-dict compatible views
    @property
    def wq(self) -> _WeightView:
        return _WeightView(lambda: self.wqkv[: self.q_dim])

    @property
    def wk(self) -> _WeightView:
        return _WeightView(lambda: self.wqkv[self.q_dim: self.q_dim + self.kv_dim])

    @property
    def wv(self) -> _WeightView:
        return _WeightView(lambda: self.wqkv[self.q_dim + self.kv_dim:])

    @property
    def wo(self) -> _WeightView:
        return _WeightView(lambda: self.wo_weight)

    def attend(self, x: torch.Tensor, norm_w: torch.Tensor, eps: float, rope: torch.Tensor, positions: torch.Tensor,
               cache: Optional[CacheView], ws: "_abi.Workspace") -> torch.Tensor:
        """RMSNorm + QKV + RoPE + cache phase + attention core.  Returns the pre-`wo` output [T, H*hd]."""
        T = x.shape[0]
        q = torch.empty(T, self.q_dim, dtype=x.dtype, device=x.device)
        k = torch.empty(T, self.kv_dim, dtype=x.dtype, device=x.device)
        v = torch.empty(T, self.kv_dim, dtype=x.dtype, device=x.device)
        out = torch.empty(T, self.q_dim, dtype=x.dtype, device=x.device)
        H, KV, hd = self.n_heads, self.n_kv_heads, self.head_dim
        if cache is None:
            # cache-less forward: unmasked over the whole flattened batch
            _abi.attn_qkv(x, norm_w, self.wqkv, rope, positions, q, k, v, None, None, None, H, KV, hd, eps, ws)
            _abi.attn_prefill(q, k, v, None, None, None, None, out, 1, T, 0, H, KV, hd, causal=False)
            return out
        md = cache.metadata
        if md.prefill:
            # read the old ring, THEN write (transformer_layers.py:75-76)
            _abi.attn_qkv(x, norm_w, self.wqkv, rope, positions, q, k, v, None, None, None, H, KV, hd, eps, ws)
            _abi.attn_prefill(q, k, v, cache.cache_k, cache.cache_v, md.q_start, md.seqpos, out, len(md.seqlens), md.max_seqlen,
                              md.window, H, KV, hd, causal=True, first_prefill=md.first_prefill)
            _abi.kv_ring_write(k, v, cache.cache_k, cache.cache_v, md.cache_rows, KV, hd)
        else:
            # write, THEN read the ring (transformer_layers.py:78-81); the scatter is the QKV kernel's epilogue
            _abi.attn_qkv(x, norm_w, self.wqkv, rope, positions, q, k, v, cache.cache_k, cache.cache_v, md.cache_rows, H, KV, hd, eps, ws)
            B = len(md.seqlens)
            _abi.attn_decode(q, cache.cache_k, cache.cache_v, md.kv_len, out, H, KV, hd, decode_splits(B, KV, md.window), ws)
        return out


def decode_splits(B: int, KV: int, W: int, n_sm: int = 148) -> int:
    """KV splits per (sequence, kv head): as many as fit ONE wave of two CTAs per SM (a second, partial wave costs more than the
    idle SMs of an incomplete first one; with B * KV >= 2 * n_sm / 2 there is no split and no combine step at all), at least 64
    keys per split."""
    s = max(1, (2 * n_sm) // (B * KV))
    return int(max(1, min(s, 64, (W + 63) // 64)))


class FeedForward(nn.Module):
    """transformer_layers.py:96-106."""

    def __init__(self, dim: int, hidden_dim: int, lora: Optional[LoraArgs] = None):
        super().__init__()
        assert lora is None
        self.dim = dim
        self.hidden_dim = hidden_dim
        self.w13 = nn.Parameter(torch.empty(2 * hidden_dim, dim), requires_grad=False)
        self.w2_weight = nn.Parameter(torch.empty(dim, hidden_dim), requires_grad=False)

    @property
    def w1(self) -> _WeightView:
        return _WeightView(lambda: self.w13.view(self.hidden_dim, 2, self.dim)[:, 0])

    @property
    def w3(self) -> _WeightView:
        return _WeightView(lambda: self.w13.view(self.hidden_dim, 2, self.dim)[:, 1])

    @property
    def w2(self) -> _WeightView:
        return _WeightView(lambda: self.w2_weight)

    def run(self, x: torch.Tensor, norm_w: Optional[torch.Tensor], eps: float, residual: Optional[torch.Tensor],
            ws: "_abi.Workspace") -> torch.Tensor:
        """[norm] -> gate/up -> silu*mul -> down [+ residual]."""
        T = x.shape[0]
        g = torch.empty(T, self.hidden_dim, dtype=x.dtype, device=x.device)
        _abi.ffn_gateup(x, norm_w, self.w13, g, eps, ws)
        out = torch.empty(T, self.dim, dtype=x.dtype, device=x.device)
        _abi.linear_residual(g, self.w2_weight, residual, out, ws)
        return out

    def forward(self, x: torch.Tensor, ws: Optional["_abi.Workspace"] = None) -> torch.Tensor:
        ws = ws or _abi.Workspace(_abi.workspace_bytes(x.shape[0], self.dim, 1, 1, 128, self.hidden_dim, 0, 1), x.device)
        return self.run(x, None, 0.0, None, ws)


class TransformerBlock(nn.Module):
    """transformer_layers.py:123-169: pre-norm residual wiring; FeedForward or MoeLayer."""

    def __init__(self, dim: int, hidden_dim: int, n_heads: int, n_kv_heads: int, head_dim: int, norm_eps: float,
                 lora: Optional[LoraArgs] = None, moe: Optional[MoeArgs] = None, expert_shard: Tuple[int, int] = (0, 1), expert_group=None):
        super().__init__()
        self.n_heads = n_heads
        self.dim = dim
        self.norm_eps = norm_eps
        self.attention = Attention(dim=dim, n_heads=n_heads, head_dim=head_dim, n_kv_heads=n_kv_heads, lora=lora)
        self.attention_norm = RMSNorm(dim, eps=norm_eps)
        self.ffn_norm = RMSNorm(dim, eps=norm_eps)
        self.feed_forward: nn.Module
        if moe is not None:
            g, G = expert_shard  # this rank allocates only the experts it owns (e % G == g): SURVEY.md 8(e)
            self.feed_forward = MoeLayer(experts={e: FeedForward(dim=dim, hidden_dim=hidden_dim, lora=lora) for e in range(moe.num_experts) if e % G == g},
                                         gate_weight=nn.Parameter(torch.empty(moe.num_experts, dim), requires_grad=False), moe_args=moe,
                                         expert_shard=expert_shard, expert_group=expert_group)
        else:
            self.feed_forward = FeedForward(dim=dim, hidden_dim=hidden_dim, lora=lora)

    def forward(self, x: torch.Tensor, rope: torch.Tensor, positions: torch.Tensor, cache: Optional[CacheView],
                ws: "_abi.Workspace") -> torch.Tensor:
        # r = attention(attention_norm(x)); h = x + r        (transformer_layers.py:165-166)
        a = self.attention.attend(x, self.attention_norm.weight, self.norm_eps, rope, positions, cache, ws)
        h = torch.empty_like(x)
        _abi.linear_residual(a, self.attention.wo_weight, x, h, ws)
        # r = feed_forward(ffn_norm(h)); out = h + r          (transformer_layers.py:167-168)
        if isinstance(self.feed_forward, MoeLayer):
            hn = _abi.rmsnorm(h, self.ffn_norm.weight, self.norm_eps)
            return self.feed_forward.run(hn, h, ws)  # router + grouped experts + ordered combine + residual, no host sync
        return self.feed_forward.run(h, self.ffn_norm.weight, self.norm_eps, h, ws)


# ============================================================================= layered decoders
# Mixers and feed-forward of models described layer by layer (args.LayeredArgs).  They run on libmb200_hybrid
# (include/mistral_b200_hybrid.h): the residual stream `x32` is fp32 and updated in place by the epilogue of each
# sublayer's last Linear; activations and weights are stored in the model dtype (bf16 or fp32).
import math  # noqa: E402
from typing import Dict  # noqa: E402

from . import _abi_hybrid as _h  # noqa: E402
from .args import (BiasedAttentionArgs, ClampedGluArgs, GlaArgs, Hgrn2Args, LatentAttentionArgs, LightningArgs, MlstmArgs, MoeFfArgs,  # noqa: E402
                   Relu2FfArgs, Relu2MoeArgs, RetentionArgs, RotaryAttentionArgs, ScaledInputMoeArgs, SideBySideArgs, SigmoidAttentionArgs)
from .rope import scaled_frequencies  # noqa: E402
from .cache import LayerCacheSpec  # noqa: E402


FLASH_MIN_QUERIES = 16  # prompts (portions) at least this long take the tensor-core attention kernel in bf16
MOE_SPARSE_MAX_TOKENS = 16  # up to this many tokens a mixture of experts streams only the chosen experts' weights


class Norm(nn.Module):
    """The norm of a layered decoder: "rms" (weight), "rms_scalar" (ONE number as weight; kept as a vector of equal entries, so the
    same kernel serves it) or "layer" (mean removed; weight and bias).  Reads the fp32 residual stream (or an fp32 sublayer output)
    and either returns the normed rows in the model dtype or adds them, in fp32, to `add_to`.  `mix` = (stack, n, coef, out), with an
    rms norm that adds: the depth average out = sum_j coef[j] * stack[j] over the n layer results so far follows in the same kernel
    (stack[n - 1] is `add_to`)."""

    def __init__(self, width: int, eps: float, kind: str):
        super().__init__()
        assert kind in ("rms", "rms_scalar", "layer"), kind
        self.kind, self.eps = kind, eps
        self.weight = nn.Parameter(torch.empty(width), requires_grad=False)
        self.bias = nn.Parameter(torch.empty(width), requires_grad=False) if kind == "layer" else None

    def forward(self, x32: torch.Tensor, add_to: Optional[torch.Tensor] = None, mix: Optional[tuple] = None) -> torch.Tensor:
        if self.kind == "layer":
            assert mix is None, "a depth average after a layer norm is not built"
            return _h.layernorm(x32, self.weight, self.bias, self.eps, add_to=add_to)
        if add_to is not None:
            stack, n, coef, out = mix if mix is not None else (None, 0, None, None)
            return _h.rmsnorm_add(x32, self.weight, add_to, self.eps, stack, n, coef, out)
        return _h.rmsnorm(x32, self.weight, self.eps)

    def load_weight(self, v: torch.Tensor) -> None:
        """Takes the checkpoint's weight: a vector, or the single number of an "rms_scalar" norm."""
        if self.kind == "rms_scalar":
            assert v.numel() == 1, f"a norm with one number got {tuple(v.shape)}"
            self.weight.copy_(v.reshape(1).expand_as(self.weight))
        else:
            assert v.shape == self.weight.shape, f"norm weight {tuple(v.shape)} != {tuple(self.weight.shape)}"
            self.weight.copy_(v)


def project_out(y: torch.Tensor, w: torch.Tensor, x32: torch.Tensor, post, scale: float = 1.0, bias: Optional[torch.Tensor] = None) -> None:
    """The last Linear of a sublayer: added to the fp32 residual stream by its epilogue (times `scale`, for a sublayer that enters a
    weighted sum), or, when the block norms the sublayer's output first (`post`, called as post(fp32 rows, add_to=stream)), written in
    fp32 and added by the norm kernel."""
    if post is None and scale != 1.0:
        _h.linear(y, w, bias, epi=_h.EPI_RESIDUAL_SCALED, residual=x32, alpha=scale)
    elif post is None:
        _h.linear(y, w, bias, epi=_h.EPI_RESIDUAL, residual=x32)
    else:
        assert scale == 1.0, "a scaled sublayer with a norm after it is not built"
        post(_h.linear(y, w, bias, epi=_h.EPI_F32), add_to=x32)


def distance_buckets(rows: int, far: float) -> List[int]:
    """bucket(n) for n = 0 .. n_sat, where n_sat is the first distance in the last bucket: one row per distance below rows/2,
    then (rows - rows/2) logarithmic steps up to `far`.  Evaluated in double precision on the host, once per layer."""
    half = rows // 2
    assert far > half > 0, "the logarithmic part of the distance bias needs bias_max > rows / 2"
    out: List[int] = []
    n = 0
    while True:
        b = n if n < half else min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))
        out.append(b)
        if b == rows - 1:
            return out
        n += 1


class BiasedAttention(nn.Module):
    """Causal softmax attention with per-head q/k RMS norm, position-dependent query temperature, learned distance bias and
    optional value mixing.  Packed weights: wqkv = q ++ k ++ v rows (+ bqkv), like `Attention.wqkv`."""

    def __init__(self, width: int, a: BiasedAttentionArgs, eps: float, first_vmix: bool, rel_rows: int = 0):
        super().__init__()
        self.a, self.eps, self.first_vmix = a, eps, first_vmix
        self.nq, self.nk, self.nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
        n = self.nq + self.nk + self.nv
        self.wqkv = nn.Parameter(torch.empty(n, width), requires_grad=False)
        self.bqkv = nn.Parameter(torch.empty(n), requires_grad=False)
        self.q_norm = nn.Parameter(torch.empty(a.dim), requires_grad=False)
        self.k_norm = nn.Parameter(torch.empty(a.dim), requires_grad=False)
        self.rel = nn.Parameter(torch.empty(max(rel_rows, 2), a.heads), requires_grad=False)  # resized by the loader to the checkpoint's rows
        self.vmix = nn.Parameter(torch.empty(()), requires_grad=False)
        self.wo = nn.Parameter(torch.empty(width, a.heads * a.vdim), requires_grad=False)
        self._bias_tab: Optional[torch.Tensor] = None

    def cache_spec(self) -> LayerCacheSpec:
        return LayerCacheSpec(kind="ring", n_kv_heads=self.a.kv_heads, k_dim=self.a.dim, v_dim=self.a.vdim, window=None)

    def bias_table(self) -> torch.Tensor:
        """fp32 [n_sat + 1, heads]: the bias of every distance up to the first one of the last bucket (larger ones share it)."""
        if self._bias_tab is None or self._bias_tab.device != self.rel.device:
            idx = torch.tensor(distance_buckets(self.rel.shape[0], self.a.bias_max), device=self.rel.device)
            self._bias_tab = self.rel.float().index_select(0, idx).contiguous()
        return self._bias_tab

    def run(self, hn: torch.Tensor, x32: torch.Tensor, view: CacheView, ctx: Dict[str, torch.Tensor], post: Optional[Norm] = None) -> None:
        a, md = self.a, view.metadata
        T = hn.shape[0]
        qkv = _h.linear(hn, self.wqkv, self.bqkv)
        q = torch.empty(T, self.nq, dtype=hn.dtype, device=hn.device)
        mode = 0
        if a.v_mix:
            if self.first_vmix:
                ctx["v_first"] = torch.empty(T, self.nv, dtype=hn.dtype, device=hn.device)
                mode = 1
            else:
                assert ctx["v_first"].shape[1] == self.nv, "value mixing needs equal value sizes in the mixed layers"
                mode = 2
        _h.attn_prep(qkv, self.q_norm, self.k_norm, md.positions, md.cache_rows, q, view.cache_k, view.cache_v, ctx.get("v_first"), self.vmix, mode,
                     a.heads, a.kv_heads, a.dim, a.vdim, self.eps, a.temp_coef, a.temp_every)
        out = torch.empty(T, a.heads * a.vdim, dtype=hn.dtype, device=hn.device)
        _h.attn_bias(q, view.cache_k, view.cache_v, self.bias_table(), md.positions, md.q_start, md.slots, out, len(md.seqlens), md.window,
                     a.heads, a.kv_heads, a.dim, a.vdim, a.scale,
                     n_tiles=sum((n + 63) // 64 for n in md.seqlens) if md.max_seqlen >= FLASH_MIN_QUERIES else 0,
                     splits=_h.attn_splits(T, a.heads, md.window))
        project_out(out, self.wo, x32, post)


class LightningMixer(nn.Module):
    """Linear attention with a fixed per-head decay: S <- decay S + k v^T, o = S^T q (fp32 state in the cache), all heads RMS-normed
    together, gated by sigmoid(W_g h).  Packed weights: wqkvg = q ++ k ++ v ++ g rows; SiLU on q, k, v in the Linear's epilogue."""

    def __init__(self, width: int, a: LightningArgs, eps: float):
        super().__init__()
        self.a, self.eps = a, eps
        self.nqk, self.nv = a.heads * a.dim, a.heads * a.vdim
        self.wqkvg = nn.Parameter(torch.empty(2 * self.nqk + 2 * self.nv, width), requires_grad=False)
        self.norm = nn.Parameter(torch.empty(self.nv), requires_grad=False)
        self.wo = nn.Parameter(torch.empty(width, self.nv), requires_grad=False)
        self.register_buffer("decay", torch.tensor(a.decay, dtype=torch.float32), persistent=False)

    def cache_spec(self) -> LayerCacheSpec:
        return LayerCacheSpec(kind="state", state_shape=(self.a.heads, self.a.dim, self.a.vdim))

    def run(self, hn: torch.Tensor, x32: torch.Tensor, view: CacheView, ctx: Dict[str, torch.Tensor], post: Optional[Norm] = None) -> None:
        a, md = self.a, view.metadata
        T = hn.shape[0]
        qkvg = _h.linear(hn, self.wqkvg, n_act=2 * self.nqk + self.nv)
        o32 = torch.empty(T, self.nv, dtype=torch.float32, device=hn.device)
        _h.lightning_scan(qkvg, view.state, self.decay, md.q_start, md.seqpos, md.slots, o32, len(md.seqlens), a.heads, a.dim, a.vdim)
        y = _h.gated_headnorm(o32, self.norm, qkvg, qkvg.shape[1], 2 * self.nqk + self.nv, self.eps)
        project_out(y, self.wo, x32, post)


class ClampedGLU(nn.Module):
    """Feed-forward with clamped gate and up projections (args.ClampedGluArgs).  w13 interleaves gate and up rows like
    `FeedForward.w13`, so the activation is the epilogue of one Linear."""

    def __init__(self, width: int, a: ClampedGluArgs):
        super().__init__()
        self.a, self.width = a, width
        self.w13 = nn.Parameter(torch.empty(2 * a.ff, width), requires_grad=False)
        self.w2 = nn.Parameter(torch.empty(width, a.ff), requires_grad=False)

    def run(self, hn: torch.Tensor, x32: torch.Tensor, post: Optional[Norm] = None) -> None:
        y = _h.linear(hn, self.w13, epi=_h.EPI_GLU, limit=self.a.limit, alpha=self.a.alpha)
        project_out(y, self.w2, x32, post)

    def checkpoint_names(self) -> List[str]:
        return ["gate", "up", "down"]

    def assign(self, name: str, put) -> bool:
        if name == "gate":
            put(self.w13.view(self.a.ff, 2, self.width)[:, 0])
        elif name == "up":
            put(self.w13.view(self.a.ff, 2, self.width)[:, 1])
        elif name == "down":
            put(self.w2)
        else:
            return False
        return True


class LatentAttention(nn.Module):
    """Causal softmax attention through latents (args.LatentAttentionArgs).  With h the normed input:
        c_q = rms(W_dq h) * n_q,  q = W_uq c_q  (per head [dim plain | rot_dim rotated]);
        [c' | k_r] = W_dkv h,  c = rms(c') * n_c;   k_h = [W_uk,h c | rot(k_r)],  v_h = W_uv,h c;
        out = W_o concat_h( sigmoid(W_g h)_h * softmax(q_h . k_h * scale) v_h ).
    The ring holds one row [c | rot(k_r)] per token.  Attention runs on the rows themselves: W_uk is folded into the query
    (q_h . W_uk,h c = (W_uk,h^T q_h) . c) and W_uv is applied to the attention-weighted sum of latents, so a decode step reads
    kv_rank + rot_dim numbers per cached token, whatever the number of heads.  Packed weights: w_in = dq ++ dkv ++ g rows."""

    def __init__(self, width: int, a: LatentAttentionArgs, eps: float):
        super().__init__()
        self.a, self.eps = a, eps
        self.n_in = a.q_rank + a.kv_rank + a.rot_dim + a.heads
        self.w_in = nn.Parameter(torch.empty(self.n_in, width), requires_grad=False)
        self.q_norm = nn.Parameter(torch.empty(a.q_rank), requires_grad=False)
        self.c_norm = nn.Parameter(torch.empty(a.kv_rank), requires_grad=False)
        self.w_uq = nn.Parameter(torch.empty(a.heads * (a.dim + a.rot_dim), a.q_rank), requires_grad=False)
        self.w_uk = nn.Parameter(torch.empty(a.heads * a.dim, a.kv_rank), requires_grad=False)
        self.w_uv = nn.Parameter(torch.empty(a.heads * a.vdim, a.kv_rank), requires_grad=False)
        self.wo = nn.Parameter(torch.empty(width, a.heads * a.vdim), requires_grad=False)
        self._freq: Optional[torch.Tensor] = None
        self._mag = 1.0
        self.shared_decode = True   # decode steps read each latent row once for all heads (else: the per-head kernel)
        self.expand_prompts = True  # whole bf16 prompts of suitable head sizes run multi-head attention on the tensor cores

    def cache_spec(self) -> LayerCacheSpec:
        # one shared "head" whose key row is the latent row; the values are its first kv_rank entries, so no value ring
        return LayerCacheSpec(kind="ring", n_kv_heads=1, k_dim=self.a.kv_rank + self.a.rot_dim, v_dim=0, window=None)

    def frequencies(self) -> torch.Tensor:
        if self._freq is None or self._freq.device != self.wo.device:
            f, self._mag = scaled_frequencies(self.a.rot_dims, self.a.rot_base, self.a.rot_scaling)
            self._freq = f.to(self.wo.device)
        return self._freq

    def run(self, hn: torch.Tensor, x32: torch.Tensor, view: CacheView, ctx: Dict[str, torch.Tensor], post: Optional[Norm] = None) -> None:
        a, md = self.a, view.metadata
        T = hn.shape[0]
        freq = self.frequencies()
        y = _h.linear(hn, self.w_in)
        cq = _h.latent_prep(y, self.q_norm, self.c_norm, freq, md.positions, md.cache_rows, view.cache_k, a.q_rank, a.kv_rank, a.rot_dim,
                            a.rot_dims, self.eps, self._mag)
        q = _h.linear(cq, self.w_uq)
        if (md.first_prefill and hn.dtype == torch.bfloat16 and md.max_seqlen >= FLASH_MIN_QUERIES and (a.dim + a.rot_dim, a.vdim) in _h.FLASH_SIZES
                and self.expand_prompts):
            # whole prompts: ordinary multi-head attention on the tensor cores over keys and values written out per head
            B = len(md.seqlens)
            # the latents of this call's tokens, gathered from their ring rows (every token of a whole prompt has one)
            lat = view.cache_k.view(-1, a.kv_rank + a.rot_dim).index_select(0, md.cache_rows.long())[:, : a.kv_rank].contiguous()
            kfull, vfull = _h.latent_expand(_h.linear(lat, self.w_uk), _h.linear(lat, self.w_uv), view.cache_k, md.positions, md.cache_rows, md.q_start,
                                            B, md.max_seqlen, a.heads, a.dim, a.rot_dim, a.vdim, a.kv_rank)
            qr = _h.latent_absorb(q, None, freq, md.positions, a.heads, a.dim, a.rot_dim, a.rot_dims, a.kv_rank, self._mag)
            out = torch.empty(T, a.heads * a.vdim, dtype=hn.dtype, device=hn.device)
            _h.attn_bias(qr, kfull, vfull, None, md.positions, md.q_start, _h.iota(B, hn.device), out, B, md.max_seqlen, a.heads, a.heads,
                         a.dim + a.rot_dim, a.vdim, a.scale, n_tiles=sum((n + 63) // 64 for n in md.seqlens))
            _h.head_gate(out, y, self.n_in, a.q_rank + a.kv_rank + a.rot_dim, a.heads, a.vdim)
            return project_out(out, self.wo, x32, post)
        qa = _h.latent_absorb(q, self.w_uk, freq, md.positions, a.heads, a.dim, a.rot_dim, a.rot_dims, a.kv_rank, self._mag)
        if not md.prefill and self.shared_decode and a.heads <= _h.LATENT_DECODE_MAX_HEADS and a.kv_rank <= _h.LATENT_DECODE_MAX_RANK:
            # one token per sequence: every latent row is read once for all heads
            o_lat = _h.attn_latent_decode(qa, view.cache_k, md.positions, md.slots, T, md.window, a.heads, a.kv_rank, a.rot_dim, a.scale)
        else:
            o_lat = _h.attn_latent(qa, view.cache_k, md.positions, md.q_start, md.slots, len(md.seqlens), md.window, a.heads, a.kv_rank, a.rot_dim,
                                   a.scale, splits=_h.attn_splits(T, a.heads, md.window))
        out = _h.latent_vup(o_lat, self.w_uv, y, self.n_in, a.q_rank + a.kv_rank + a.rot_dim, a.heads, a.vdim, a.kv_rank)
        project_out(out, self.wo, x32, post)

    def checkpoint_names(self) -> List[str]:
        return ["dq", "dq.norm", "uq", "dkv", "dkv.norm", "uk", "uv", "g", "o"]

    def assign(self, name: str, put) -> bool:
        a = self.a
        o1, o2 = a.q_rank, a.q_rank + a.kv_rank + a.rot_dim
        targets = {"dq": lambda: self.w_in[:o1], "dkv": lambda: self.w_in[o1:o2], "g": lambda: self.w_in[o2:], "dq.norm": lambda: self.q_norm,
                   "dkv.norm": lambda: self.c_norm, "uq": lambda: self.w_uq, "uk": lambda: self.w_uk, "uv": lambda: self.w_uv, "o": lambda: self.wo}
        if name not in targets:
            return False
        put(targets[name]())
        return True


class MoeFeedForward(nn.Module):
    """Mixture of gated experts with an fp32 softmax router (args.MoeFfArgs).  Packed weights: w13 [E * 2 * ff, width], expert after
    expert with gate and up rows interleaved; w2 [width, E * ff], expert e's down projection in columns e*ff ..; identity experts have
    no weights.  Few tokens (decode) stream the chosen experts only; prompts run all experts as two Linears, the first one's
    epilogue scaling every expert's hidden units by the token's routing weight (0 when not chosen)."""

    def __init__(self, width: int, a: MoeFfArgs):
        super().__init__()
        self.a, self.width = a, width
        self.router = nn.Parameter(torch.empty(a.routed, width), requires_grad=False)
        self.correction = nn.Parameter(torch.empty(a.routed), requires_grad=False)
        self.w13 = nn.Parameter(torch.empty(a.experts * 2 * a.ff, width), requires_grad=False)
        self.w2 = nn.Parameter(torch.empty(width, a.experts * a.ff), requires_grad=False)
        self.sparse_max_tokens = MOE_SPARSE_MAX_TOKENS

    def run(self, hn: torch.Tensor, x32: torch.Tensor, post: Optional[Norm] = None) -> None:
        a = self.a
        dense, idx, wsel = _h.moe_route(hn, self.router, self.correction, a.groups, a.keep, a.top)
        if hn.shape[0] <= self.sparse_max_tokens:
            y32 = _h.moe_sparse(hn, self.w13, self.w2, idx, wsel, a.experts, a.ff)
        else:
            act = _h.linear_swiglu(hn, self.w13, rowscale=dense, group=a.ff)
            y32 = _h.linear(act, self.w2, epi=_h.EPI_F32)
            if a.identity:
                _h.rows_axpy(y32, hn, dense, a.experts)
        if post is None:
            x32.add_(y32)
        else:
            post(y32, add_to=x32)

    def checkpoint_names(self) -> List[str]:
        return ["router", "correction"] + [f"e{e}.{n}" for e in range(self.a.experts) for n in ("gate", "up", "down")]

    def assign(self, name: str, put) -> bool:
        a = self.a
        if name == "router":
            put(self.router)
        elif name == "correction":
            put(self.correction)
        elif name[0] == "e" and "." in name and name[1:name.index(".")].isdigit() and int(name[1:name.index(".")]) < a.experts:
            e, part = int(name[1:name.index(".")]), name[name.index(".") + 1:]
            if part == "gate":
                put(self.w13.view(a.experts, a.ff, 2, self.width)[e, :, 0])
            elif part == "up":
                put(self.w13.view(a.experts, a.ff, 2, self.width)[e, :, 1])
            elif part == "down":
                put(self.w2.view(self.width, a.experts, a.ff)[:, e])
            else:
                return False
        else:
            return False
        return True




class RotaryWindowAttention(nn.Module):
    """Causal softmax attention with rotary positions, a unit RMS norm of the rotated q and k heads, grouped key/value heads and an
    optional sliding window (args.RotaryAttentionArgs).  The ring holds min(window, longest sequence) rows per sequence.  A decode
    step writes its key and value into the ring, then attends over it; a prompt (portion) attends over the OLD ring plus its own
    keys and values, and writes the ring afterwards, so a prompt longer than the ring still finds every key inside each token's
    window.  Packed weights: wqkv = q ++ k ++ v rows."""

    def __init__(self, width: int, a: RotaryAttentionArgs, eps: float):
        super().__init__()
        self.a, self.eps = a, eps
        self.nq, self.nk, self.nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
        self.wqkv = nn.Parameter(torch.empty(self.nq + self.nk + self.nv, width), requires_grad=False)
        self.wo = nn.Parameter(torch.empty(width, a.heads * a.vdim), requires_grad=False)
        self._freq: Optional[torch.Tensor] = None

    def cache_spec(self) -> LayerCacheSpec:
        return LayerCacheSpec(kind="ring", n_kv_heads=self.a.kv_heads, k_dim=self.a.dim, v_dim=self.a.vdim, window=self.a.window)

    def frequencies(self) -> torch.Tensor:
        """float64 [rot_dims / 2]: rot_base^(-2i / rot_dims) / rot_factor, evaluated on the host in double precision."""
        if self._freq is None or self._freq.device != self.wo.device:
            f, _ = scaled_frequencies(self.a.rot_dims, self.a.rot_base, None) if self.a.rot_dims else (torch.zeros(0, dtype=torch.float64), 1.0)
            self._freq = (f / self.a.rot_factor).to(self.wo.device)
        return self._freq

    def run(self, hn: torch.Tensor, x32: torch.Tensor, view: CacheView, ctx: Dict[str, torch.Tensor], post: Optional[Norm] = None,
            scale: float = 1.0) -> None:
        a, md = self.a, view.metadata
        T, B, W = hn.shape[0], len(md.seqlens), md.window
        qkv = _h.linear(hn, self.wqkv)
        out = torch.empty(T, a.heads * a.vdim, dtype=hn.dtype, device=hn.device)
        window = a.window or 0
        if md.prefill:
            q, k, v = _h.rot_prep(qkv, self.frequencies(), md.positions, None, None, None, a.heads, a.kv_heads, a.dim, a.vdim, a.rot_dims, a.unit_norm,
                                  self.eps, own=True)
            _h.attn_window(q, view.cache_k, view.cache_v, md.positions, md.q_start, md.slots, out, B, W, a.heads, a.kv_heads, a.dim, a.vdim, a.scale,
                           window, own_k=k, own_v=v, seqpos=md.seqpos,
                           n_tiles=sum((n + 63) // 64 for n in md.seqlens) if md.max_seqlen >= FLASH_MIN_QUERIES else 0)
            _h.kv_scatter(k, v, md.cache_rows, view.cache_k, view.cache_v)
        else:
            q, _, _ = _h.rot_prep(qkv, self.frequencies(), md.positions, md.cache_rows, view.cache_k, view.cache_v, a.heads, a.kv_heads, a.dim, a.vdim,
                                  a.rot_dims, a.unit_norm, self.eps, own=False)
            splits, chunk = _h.window_decode_plan(T, a.heads, W)
            _h.attn_window(q, view.cache_k, view.cache_v, md.positions, md.q_start, md.slots, out, B, W, a.heads, a.kv_heads, a.dim, a.vdim, a.scale,
                           window, splits=splits, chunk=chunk)
        project_out(out, self.wo, x32, post, scale)

    def checkpoint_names(self) -> List[str]:
        return ["q", "k", "v", "o"]

    def assign(self, name: str, put) -> bool:
        spans = {"q": (0, self.nq), "k": (self.nq, self.nq + self.nk), "v": (self.nq + self.nk, self.nq + self.nk + self.nv)}
        if name in spans:
            put(self.wqkv[spans[name][0]: spans[name][1]])
        elif name == "o":
            put(self.wo)
        else:
            return False
        return True


class Hgrn2Mixer(nn.Module):
    """Gated linear recurrence (args.Hgrn2Args): q = silu(W_q h), f = lower + (1 - lower) sigmoid(W_f h + b_f), v = W_v h; per head
    S <- diag(f) S + (1 - f) v^T, o = S^T q in fp32 (state in the cache); every head RMS-normed with one weight [vdim] shared by the
    heads.  Packed weights: wqfv = q ++ f ++ v rows, bqfv zero outside the f rows; SiLU on q in the Linear's epilogue."""

    def __init__(self, width: int, a: Hgrn2Args, eps: float):
        super().__init__()
        self.a, self.eps = a, eps
        self.nqk, self.nv = a.heads * a.dim, a.heads * a.vdim
        self.wqfv = nn.Parameter(torch.empty(2 * self.nqk + self.nv, width), requires_grad=False)
        self.bqfv = nn.Parameter(torch.empty(2 * self.nqk + self.nv), requires_grad=False)
        self.lower = nn.Parameter(torch.empty(self.nqk), requires_grad=False)
        self.norm = nn.Parameter(torch.empty(a.vdim), requires_grad=False)
        self.wo = nn.Parameter(torch.empty(width, self.nv), requires_grad=False)

    def cache_spec(self) -> LayerCacheSpec:
        return LayerCacheSpec(kind="state", state_shape=(self.a.heads, self.a.dim, self.a.vdim))

    def run(self, hn: torch.Tensor, x32: torch.Tensor, view: CacheView, ctx: Dict[str, torch.Tensor], post: Optional[Norm] = None,
            scale: float = 1.0) -> None:
        a, md = self.a, view.metadata
        qfv = _h.linear(hn, self.wqfv, self.bqfv, n_act=self.nqk)
        qab = _h.hgrn2_gates(qfv, self.lower, self.nqk)
        o32 = _h.gated_scan(qab, qfv, qfv.shape[1], 2 * self.nqk, view.state, md.q_start, md.seqpos, md.slots, len(md.seqlens), a.heads, a.dim, a.vdim,
                            ones=False, max_seqlen=md.max_seqlen)
        y = _h.scan_post(o32, None, self.norm, False, None, 0, 0, a.heads, a.vdim, False, self.eps)
        project_out(y, self.wo, x32, post, scale)

    def checkpoint_names(self) -> List[str]:
        return ["q", "f", "f.b", "lower", "v", "norm", "o"]

    def assign(self, name: str, put) -> bool:
        n = self.nqk
        if name == "q":
            put(self.wqfv[:n])
        elif name == "f":
            put(self.wqfv[n: 2 * n])
        elif name == "v":
            put(self.wqfv[2 * n:])
        elif name == "f.b":
            self.bqfv.zero_()  # q and v have no bias
            put(self.bqfv[n: 2 * n])
        elif name in ("lower", "norm"):
            put(getattr(self, name))
        elif name == "o":
            put(self.wo)
        else:
            return False
        return True


class SideBySideMixer(nn.Module):
    """Two mixers on the same input, summed with fixed weights (args.SideBySideArgs): left_scale * rotary window attention +
    right_scale * gated linear recurrence.  The layer's cache entry holds the attention's ring AND the recurrence's state; each
    mixer's output Linear adds its weighted result to the residual stream in its epilogue.  Checkpoint names: left.*, right.*."""

    def __init__(self, width: int, a: SideBySideArgs, eps: float):
        super().__init__()
        self.a = a
        self.left = RotaryWindowAttention(width, a.left, eps)
        self.right = Hgrn2Mixer(width, a.right, eps)

    def cache_spec(self) -> LayerCacheSpec:
        sp = self.left.cache_spec()
        sp.state_shape = self.right.cache_spec().state_shape
        return sp

    def run(self, hn: torch.Tensor, x32: torch.Tensor, view: CacheView, ctx: Dict[str, torch.Tensor], post: Optional[Norm] = None) -> None:
        assert post is None, "a norm after a weighted sum of mixers is not built"
        self.left.run(hn, x32, view, ctx, None, self.a.left_scale)
        self.right.run(hn, x32, view, ctx, None, self.a.right_scale)

    def checkpoint_names(self) -> List[str]:
        return ["left." + n for n in self.left.checkpoint_names()] + ["right." + n for n in self.right.checkpoint_names()]

    def assign(self, name: str, put) -> bool:
        side, _, rest = name.partition(".")
        if side == "left":
            return self.left.assign(rest, put)
        if side == "right":
            return self.right.assign(rest, put)
        return False


class MlstmMixer(nn.Module):
    """Matrix memory with exponential gates (args.MlstmArgs).  q = W_q h / sqrt(dim), k, v; per head log gates i = cap tanh(. / cap),
    f = logsigmoid(cap tanh(. / cap)); m_t = max(f + m_(t-1), i) (m_0 = 0); S <- exp(f + m_(t-1) - m_t) S + exp(i - m_t) k v^T, n
    likewise with k alone; o = S^T q / (max(|n . q|, exp(-m_t)) + 1e-6); every head divided by its root mean square, times a weight over
    all heads and sigmoid(W_g h).  The state row of a sequence is [heads, dim, vdim + 1] (the normaliser is the last column: a value
    that is 1 for every token; the scan carries it beside the value columns) followed by the heads' m, all fp32.  Packed weights: wqkvg = q ++ k ++ v ++ g rows; wif = i ++ f rows
    (+ bif), whose outputs stay fp32."""

    def __init__(self, width: int, a: MlstmArgs, eps: float):
        super().__init__()
        self.a, self.eps = a, eps
        self.nqk, self.nv = a.heads * a.dim, a.heads * a.vdim
        self.wqkvg = nn.Parameter(torch.empty(2 * self.nqk + 2 * self.nv, width), requires_grad=False)
        self.wif = nn.Parameter(torch.empty(2 * a.heads, width), requires_grad=False)
        self.bif = nn.Parameter(torch.empty(2 * a.heads), requires_grad=False)
        self.norm = nn.Parameter(torch.empty(self.nv), requires_grad=False)
        self.wo = nn.Parameter(torch.empty(width, self.nv), requires_grad=False)
        self.m_off = a.heads * a.dim * (a.vdim + 1)

    def cache_spec(self) -> LayerCacheSpec:
        return LayerCacheSpec(kind="state", state_shape=(self.m_off + self.a.heads,))

    def run(self, hn: torch.Tensor, x32: torch.Tensor, view: CacheView, ctx: Dict[str, torch.Tensor], post: Optional[Norm] = None,
            scale: float = 1.0) -> None:
        a, md = self.a, view.metadata
        B = len(md.seqlens)
        qkvg = _h.linear(hn, self.wqkvg)
        gif = _h.linear(hn, self.wif, self.bif, epi=_h.EPI_F32)
        gates, qab = _h.mlstm_gates(qkvg, gif, view.state, self.m_off, md.q_start, md.seqpos, md.slots, B, a.heads, a.dim, a.gate_cap, a.dim ** -0.5)
        o32, nq = _h.gated_scan(qab, qkvg, qkvg.shape[1], 2 * self.nqk, view.state, md.q_start, md.seqpos, md.slots, B, a.heads, a.dim, a.vdim,
                                ones=True, max_seqlen=md.max_seqlen)
        y = _h.scan_post(o32, gates, self.norm, True, qkvg, qkvg.shape[1], 2 * self.nqk + self.nv, a.heads, a.vdim, True, self.eps, nq=nq)
        project_out(y, self.wo, x32, post, scale)

    def checkpoint_names(self) -> List[str]:
        return ["q", "k", "v", "g", "i", "i.b", "f", "f.b", "norm", "o"]

    def assign(self, name: str, put) -> bool:
        H = self.a.heads
        o = [0, self.nqk, 2 * self.nqk, 2 * self.nqk + self.nv, 2 * self.nqk + 2 * self.nv]
        idx = {"q": 0, "k": 1, "v": 2, "g": 3}
        if name in idx:
            put(self.wqkvg[o[idx[name]]: o[idx[name] + 1]])
        elif name in ("i", "f"):
            put(self.wif[:H] if name == "i" else self.wif[H:])
        elif name in ("i.b", "f.b"):
            put(self.bif[:H] if name == "i.b" else self.bif[H:])
        elif name == "norm":
            put(self.norm)
        elif name == "o":
            put(self.wo)
        else:
            return False
        return True


class ScaledInputMoe(nn.Module):
    """Mixture of clamped gated experts whose INPUT is scaled by the routing weight (args.ScaledInputMoeArgs): fp32 sigmoid router,
    the `top` largest scores chosen, output = sum over the chosen of expert(score * h) + shared(h).  Packed like MoeFeedForward (w13
    [E * 2 * ff, width] interleaved gate/up rows, w2 [width, E * ff]).  W (s h) = s (W h), so the score multiplies gate and up of the
    expert's hidden units before the clamps: few tokens stream only the chosen experts, prompts run all experts as two Linears with the
    score (0 when not chosen, which gives exactly 0) applied in the first one's epilogue."""

    def __init__(self, width: int, a: ScaledInputMoeArgs):
        super().__init__()
        self.a, self.width = a, width
        self.router = nn.Parameter(torch.empty(a.experts, width), requires_grad=False)
        self.w13 = nn.Parameter(torch.empty(a.experts * 2 * a.ff, width), requires_grad=False)
        self.w2 = nn.Parameter(torch.empty(width, a.experts * a.ff), requires_grad=False)
        self.shared = ClampedGLU(width, a.shared) if a.shared is not None else None
        self.sparse_max_tokens = MOE_SPARSE_MAX_TOKENS

    def run(self, hn: torch.Tensor, x32: torch.Tensor, post: Optional[Norm] = None) -> None:
        assert post is None, "a norm after this feed-forward is not built"
        a = self.a
        dense, idx, wsel = _h.moe_route(hn, self.router, None, 1, 1, a.top, score=1)
        if hn.shape[0] <= self.sparse_max_tokens:
            _h.moe_sparse(hn, self.w13, self.w2, idx, wsel, a.experts, a.ff, glu=True, limit=a.limit, alpha=a.alpha, add_to=x32)
        else:
            act = _h.linear_glu(hn, self.w13, a.limit, a.alpha, rowscale=dense, group=a.ff)
            _h.linear(act, self.w2, epi=_h.EPI_RESIDUAL, residual=x32)
        if self.shared is not None:
            self.shared.run(hn, x32)

    def checkpoint_names(self) -> List[str]:
        names = ["router"] + [f"e{e}.{n}" for e in range(self.a.experts) for n in ("gate", "up", "down")]
        return names + (["shared." + n for n in self.shared.checkpoint_names()] if self.shared is not None else [])

    def assign(self, name: str, put) -> bool:
        a = self.a
        head, _, part = name.partition(".")
        if name == "router":
            put(self.router)
        elif head == "shared" and self.shared is not None:
            return self.shared.assign(part, put)
        elif head[:1] == "e" and head[1:].isdigit() and int(head[1:]) < a.experts:
            e = int(head[1:])
            if part == "gate":
                put(self.w13.view(a.experts, a.ff, 2, self.width)[e, :, 0])
            elif part == "up":
                put(self.w13.view(a.experts, a.ff, 2, self.width)[e, :, 1])
            elif part == "down":
                put(self.w2.view(self.width, a.experts, a.ff)[:, e])
            else:
                return False
        else:
            return False
        return True


class RetentionMixer(nn.Module):
    """Linear attention with a fixed decay per head, rotated queries and keys and no normaliser (args.RetentionArgs): per head
    S <- decay_h S + (rot(k) dim^(-1/2)) v^T, o = S^T rot(q) in fp32 (state in the cache), every head divided by its root mean square
    (no weight), times silu(W_g h).  The rotation and the key scale are fp32 steps between the projections and the scan; the scan is
    the gated one with a_t = decay_h.  Packed weights: wqkvg = q ++ k ++ v ++ g rows."""

    def __init__(self, width: int, a: RetentionArgs, eps: float):
        super().__init__()
        self.a, self.eps = a, eps
        self.nqk, self.nv = a.heads * a.dim, a.heads * a.vdim
        self.wqkvg = nn.Parameter(torch.empty(2 * self.nqk + 2 * self.nv, width), requires_grad=False)
        self.wo = nn.Parameter(torch.empty(width, self.nv), requires_grad=False)
        self._freq: Optional[torch.Tensor] = None
        self._decay: Optional[torch.Tensor] = None

    def cache_spec(self) -> LayerCacheSpec:
        return LayerCacheSpec(kind="state", state_shape=(self.a.heads, self.a.dim, self.a.vdim))

    def constants(self) -> Tuple[torch.Tensor, torch.Tensor]:
        """(float64 [rot_dims / 2] frequencies rot_base^(-2i / rot_dims), fp32 [heads] decays), made on the host once per device."""
        if self._freq is None or self._freq.device != self.wo.device:
            f = scaled_frequencies(self.a.rot_dims, self.a.rot_base, None)[0] if self.a.rot_dims else torch.zeros(0, dtype=torch.float64)
            self._freq = f.to(self.wo.device)
            self._decay = torch.tensor(self.a.decay, dtype=torch.float32, device=self.wo.device)
        return self._freq, self._decay

    def run(self, hn: torch.Tensor, x32: torch.Tensor, view: CacheView, ctx: Dict[str, torch.Tensor], post=None, scale: float = 1.0) -> None:
        a, md = self.a, view.metadata
        freq, decay = self.constants()
        qkvg = _h.linear(hn, self.wqkvg)
        qab = _h.retention_qab(qkvg, freq, decay, md.positions, a.heads, a.dim, a.rot_dims, a.dim ** -0.5)
        o32 = _h.gated_scan(qab, qkvg, qkvg.shape[1], 2 * self.nqk, view.state, md.q_start, md.seqpos, md.slots, len(md.seqlens), a.heads, a.dim, a.vdim,
                            ones=False, max_seqlen=md.max_seqlen)
        y = _h.scan_post(o32, None, None, False, qkvg, qkvg.shape[1], 2 * self.nqk + self.nv, a.heads, a.vdim, False, self.eps, silu_gate=True)
        project_out(y, self.wo, x32, post, scale)

    def checkpoint_names(self) -> List[str]:
        return ["q", "k", "v", "g", "o"]

    def assign(self, name: str, put) -> bool:
        o = [0, self.nqk, 2 * self.nqk, 2 * self.nqk + self.nv, 2 * self.nqk + 2 * self.nv]
        idx = {"q": 0, "k": 1, "v": 2, "g": 3}
        if name in idx:
            put(self.wqkvg[o[idx[name]]: o[idx[name] + 1]])
        elif name == "o":
            put(self.wo)
        else:
            return False
        return True


class GlaMixer(nn.Module):
    """Gated linear attention (args.GlaArgs): a decay per key channel alpha = sigmoid(z)^(1 / tau), z = W_a2 (W_a1 h) + b (fp32 out of
    the second Linear); per head S <- diag(alpha) S + k v^T, o = S^T (q dim^(-1/2)) in fp32 (state in the cache); every head RMS-normed
    with one weight [vdim] shared by the heads, times silu(W_g h).  Packed weights: wqkvg = q ++ k ++ v ++ g rows; the rank of the
    decay projection comes with the checkpoint."""

    def __init__(self, width: int, a: GlaArgs, eps: float):
        super().__init__()
        self.a, self.eps, self.width = a, eps, width
        self.nqk, self.nv = a.heads * a.dim, a.heads * a.vdim
        self.wqkvg = nn.Parameter(torch.empty(2 * self.nqk + 2 * self.nv, width), requires_grad=False)
        self.wa1 = nn.Parameter(torch.empty(1, width), requires_grad=False)       # resized by the loader to the checkpoint's rank
        self.wa2 = nn.Parameter(torch.empty(self.nqk, 1), requires_grad=False)
        self.ba2 = nn.Parameter(torch.empty(self.nqk), requires_grad=False)
        self.norm = nn.Parameter(torch.empty(a.vdim), requires_grad=False)
        self.wo = nn.Parameter(torch.empty(width, self.nv), requires_grad=False)

    def cache_spec(self) -> LayerCacheSpec:
        return LayerCacheSpec(kind="state", state_shape=(self.a.heads, self.a.dim, self.a.vdim))

    def run(self, hn: torch.Tensor, x32: torch.Tensor, view: CacheView, ctx: Dict[str, torch.Tensor], post=None, scale: float = 1.0) -> None:
        a, md = self.a, view.metadata
        qkvg = _h.linear(hn, self.wqkvg)
        z32 = _h.linear(_h.linear(hn, self.wa1), self.wa2, self.ba2, epi=_h.EPI_F32)
        qab = _h.gla_qab(qkvg, z32, self.nqk, a.dim ** -0.5, 1.0 / a.tau)
        o32 = _h.gated_scan(qab, qkvg, qkvg.shape[1], 2 * self.nqk, view.state, md.q_start, md.seqpos, md.slots, len(md.seqlens), a.heads, a.dim, a.vdim,
                            ones=False, max_seqlen=md.max_seqlen)
        y = _h.scan_post(o32, None, self.norm, False, qkvg, qkvg.shape[1], 2 * self.nqk + self.nv, a.heads, a.vdim, False, self.eps, silu_gate=True)
        project_out(y, self.wo, x32, post, scale)

    def checkpoint_names(self) -> List[str]:
        return ["q", "k", "v", "g", "a1", "a2", "a2.b", "norm", "o"]

    def prepare(self, name: str, shape: Tuple[int, ...]) -> None:
        """Called by the loader before `assign`: the decay projection takes the rank of the checkpoint's tensors."""
        if name == "a1" and len(shape) == 2 and shape[1] == self.width and tuple(shape) != tuple(self.wa1.shape):
            self.wa1 = nn.Parameter(torch.empty(tuple(shape), dtype=self.wa1.dtype, device=self.wa1.device), requires_grad=False)
        if name == "a2" and len(shape) == 2 and shape[0] == self.nqk and tuple(shape) != tuple(self.wa2.shape):
            self.wa2 = nn.Parameter(torch.empty(tuple(shape), dtype=self.wa2.dtype, device=self.wa2.device), requires_grad=False)

    def assign(self, name: str, put) -> bool:
        o = [0, self.nqk, 2 * self.nqk, 2 * self.nqk + self.nv, 2 * self.nqk + 2 * self.nv]
        idx = {"q": 0, "k": 1, "v": 2, "g": 3}
        if name in idx:
            put(self.wqkvg[o[idx[name]]: o[idx[name] + 1]])
        elif name == "a1":
            put(self.wa1)
        elif name == "a2":
            put(self.wa2)
        elif name == "a2.b":
            put(self.ba2)
        elif name == "norm":
            put(self.norm)
        elif name == "o":
            put(self.wo)
        else:
            return False
        return True


class SigmoidWindowAttention(nn.Module):
    """Attention with sigmoid weights (args.SigmoidAttentionArgs): q and k RMS-normed over their whole projections (weights of that
    size), no rotation, a visible key weighs sigmoid(q.k * scale + pb[h]) with nothing normalised over the keys, grouped key/value
    heads, an optional sliding window, head h's output times sigmoid(W_g h)_h; q, k, v and o have biases.  The ring and the order of
    attention and ring writes are those of RotaryWindowAttention.  Packed weights: wqkvg = q ++ k ++ v ++ g rows (the gate's bias 0)."""

    def __init__(self, width: int, a: SigmoidAttentionArgs, eps: float):
        super().__init__()
        self.a, self.eps = a, eps
        self.nq, self.nk, self.nv = a.heads * a.dim, a.kv_heads * a.dim, a.kv_heads * a.vdim
        self.wqkv = nn.Parameter(torch.empty(self.nq + self.nk + self.nv, width), requires_grad=False)
        self.bqkv = nn.Parameter(torch.empty(self.nq + self.nk + self.nv), requires_grad=False)
        self.wg = nn.Parameter(torch.empty(a.heads, width), requires_grad=False)
        self.q_norm = nn.Parameter(torch.empty(self.nq), requires_grad=False)
        self.k_norm = nn.Parameter(torch.empty(self.nk), requires_grad=False)
        self.pb = nn.Parameter(torch.empty(a.heads), requires_grad=False)
        self.wo = nn.Parameter(torch.empty(width, a.heads * a.vdim), requires_grad=False)
        self.bo = nn.Parameter(torch.empty(width), requires_grad=False)
        self._pb32: Optional[torch.Tensor] = None

    def cache_spec(self) -> LayerCacheSpec:
        return LayerCacheSpec(kind="ring", n_kv_heads=self.a.kv_heads, k_dim=self.a.dim, v_dim=self.a.vdim, window=self.a.window)

    def head_bias(self) -> torch.Tensor:
        if self._pb32 is None or self._pb32.device != self.pb.device:
            self._pb32 = self.pb.detach().float().contiguous()
        return self._pb32

    def run(self, hn: torch.Tensor, x32: torch.Tensor, view: CacheView, ctx: Dict[str, torch.Tensor], post=None, scale: float = 1.0) -> None:
        a, md = self.a, view.metadata
        T, B, W = hn.shape[0], len(md.seqlens), md.window
        qkv = _h.linear(hn, self.wqkv, self.bqkv)
        gate = _h.linear(hn, self.wg)
        out = torch.empty(T, a.heads * a.vdim, dtype=hn.dtype, device=hn.device)
        window = a.window or 0
        if md.prefill:
            q, k, v = _h.whole_norm_prep(qkv, self.q_norm, self.k_norm, None, None, None, self.nq, self.nk, self.nv, self.eps, own=True)
            _h.attn_window(q, view.cache_k, view.cache_v, md.positions, md.q_start, md.slots, out, B, W, a.heads, a.kv_heads, a.dim, a.vdim, a.scale,
                           window, own_k=k, own_v=v, seqpos=md.seqpos, head_bias=self.head_bias(),
                           n_tiles=sum((n + 63) // 64 for n in md.seqlens) if md.max_seqlen >= FLASH_MIN_QUERIES else 0)
            _h.kv_scatter(k, v, md.cache_rows, view.cache_k, view.cache_v)
        else:
            q, _, _ = _h.whole_norm_prep(qkv, self.q_norm, self.k_norm, md.cache_rows, view.cache_k, view.cache_v, self.nq, self.nk, self.nv, self.eps,
                                         own=False)
            splits, chunk = _h.window_decode_plan(T, a.heads, W)
            _h.attn_window(q, view.cache_k, view.cache_v, md.positions, md.q_start, md.slots, out, B, W, a.heads, a.kv_heads, a.dim, a.vdim, a.scale,
                           window, splits=splits, chunk=chunk, head_bias=self.head_bias())
        _h.head_gate(out, gate, a.heads, 0, a.heads, a.vdim)
        project_out(out, self.wo, x32, post, scale, bias=self.bo)

    def checkpoint_names(self) -> List[str]:
        return ["q", "q.b", "k", "k.b", "v", "v.b", "q.norm", "k.norm", "pb", "g", "o", "o.b"]

    def assign(self, name: str, put) -> bool:
        spans = {"q": (0, self.nq), "k": (self.nq, self.nq + self.nk), "v": (self.nq + self.nk, self.nq + self.nk + self.nv)}
        direct = {"q.norm": "q_norm", "k.norm": "k_norm", "g": "wg", "o": "wo", "o.b": "bo"}
        if name in spans:
            put(self.wqkv[spans[name][0]: spans[name][1]])
        elif name.endswith(".b") and name[:-2] in spans:
            put(self.bqkv[spans[name[:-2]][0]: spans[name[:-2]][1]])
        elif name == "pb":
            put(self.pb)
            self._pb32 = None
        elif name in direct:
            put(getattr(self, direct[name]))
        else:
            return False
        return True


class Relu2FeedForward(nn.Module):
    """Feed-forward without a gate, W_down max(W_up h, 0)^2 (args.Relu2FfArgs); the square of the rectifier is the epilogue of the
    first Linear.  `run` adds into `y32` (an fp32 sum of sublayer parts) or, with `post`, norms its own output into the stream."""

    def __init__(self, width: int, a: Relu2FfArgs):
        super().__init__()
        self.a, self.width = a, width
        self.w_up = nn.Parameter(torch.empty(a.ff, width), requires_grad=False)
        self.w_down = nn.Parameter(torch.empty(width, a.ff), requires_grad=False)

    def run(self, hn: torch.Tensor, x32: torch.Tensor, post=None) -> None:
        project_out(_h.linear_relu2(hn, self.w_up), self.w_down, x32, post)

    def checkpoint_names(self) -> List[str]:
        return ["up", "down"]

    def assign(self, name: str, put) -> bool:
        if name == "up":
            put(self.w_up)
        elif name == "down":
            put(self.w_down)
        else:
            return False
        return True


class Relu2Moe(nn.Module):
    """Mixture of ungated experts W_down max(W_up h, 0)^2 (args.Relu2MoeArgs): fp32 softmax router over all experts, the `top` largest
    scores chosen, weights score * router_scale (not renormalised), plus a shared expert for every token.  Packed weights: w_up
    [E * ff, width], expert after expert; w2 [width, E * ff], expert e's down projection in columns e*ff ..  Few tokens (decode) stream
    only the chosen experts; prompts run all experts as two Linears, the first one's epilogue scaling every expert's hidden units by
    the token's routing weight (0 when not chosen).  The parts are summed in fp32 before the norm that follows."""

    def __init__(self, width: int, a: Relu2MoeArgs):
        super().__init__()
        self.a, self.width = a, width
        self.router = nn.Parameter(torch.empty(a.experts, width), requires_grad=False)
        self.w_up = nn.Parameter(torch.empty(a.experts * a.ff, width), requires_grad=False)
        self.w2 = nn.Parameter(torch.empty(width, a.experts * a.ff), requires_grad=False)
        self.shared = Relu2FeedForward(width, a.shared) if a.shared is not None else None
        self.sparse_max_tokens = MOE_SPARSE_MAX_TOKENS

    def run(self, hn: torch.Tensor, x32: torch.Tensor, post=None) -> None:
        a = self.a
        dense, idx, wsel = _h.moe_route(hn, self.router, None, 1, 1, a.top, score=0, scale=a.router_scale)
        if hn.shape[0] <= self.sparse_max_tokens:
            y32 = _h.moe_sparse(hn, self.w_up, self.w2, idx, wsel, a.experts, a.ff, glu=2)
        else:
            y32 = _h.linear(_h.linear_relu2(hn, self.w_up, rowscale=dense, group=a.ff), self.w2, epi=_h.EPI_F32)
        if self.shared is not None:
            self.shared.run(hn, y32)
        if post is None:
            x32.add_(y32)
        else:
            post(y32, add_to=x32)

    def checkpoint_names(self) -> List[str]:
        names = ["router"] + [f"e{e}.{n}" for e in range(self.a.experts) for n in ("up", "down")]
        return names + (["shared." + n for n in self.shared.checkpoint_names()] if self.shared is not None else [])

    def assign(self, name: str, put) -> bool:
        a = self.a
        head, _, part = name.partition(".")
        if name == "router":
            put(self.router)
        elif head == "shared" and self.shared is not None:
            return self.shared.assign(part, put)
        elif head[:1] == "e" and head[1:].isdigit() and int(head[1:]) < a.experts:
            e = int(head[1:])
            if part == "up":
                put(self.w_up[e * a.ff: (e + 1) * a.ff])
            elif part == "down":
                put(self.w2.view(self.width, a.experts, a.ff)[:, e])
            else:
                return False
        else:
            return False
        return True


class CanonConv(nn.Module):
    """What a sublayer reads, replaced by itself plus a causal convolution over time on every channel: h_t = x_t + sum_j w[:, j]
    x_(t - taps + 1 + j), zeros before the sequence's start.  Reads the fp32 stream, writes the model dtype.  The last taps - 1 inputs
    of every sequence are part `index` of the layer's convolution state in the cache."""

    def __init__(self, width: int, taps: int, index: int):
        super().__init__()
        self.width, self.taps, self.index = width, taps, index
        self.weight = nn.Parameter(torch.empty(width, taps), requires_grad=False)

    def forward(self, x32: torch.Tensor, view: CacheView) -> torch.Tensor:
        md = view.metadata
        return _h.canon_conv(x32, self.weight, view.conv, self.index * (self.taps - 1) * self.width, md.q_start, md.seqpos, md.slots, len(md.seqlens),
                             one_each=not md.prefill)


MIXERS = {"attention": BiasedAttention, "lightning": LightningMixer, "latent_attention": LatentAttention, "parallel": SideBySideMixer,
          "mlstm": MlstmMixer, "mlstm_2": MlstmMixer}
# mixers that a design names with a type another design uses differently are found by their argument class first
MIXERS_BY_ARGS = {RetentionArgs: RetentionMixer, GlaArgs: GlaMixer, SigmoidAttentionArgs: SigmoidWindowAttention}
FEED_FORWARDS = {ClampedGluArgs: ClampedGLU, MoeFfArgs: MoeFeedForward, ScaledInputMoeArgs: ScaledInputMoe, Relu2MoeArgs: Relu2Moe}


class _PostNorm:
    """The norm after a sublayer as the sublayers call it, post(fp32 rows, add_to=stream), with the depth average that follows the
    layer's last sublayer."""

    def __init__(self, norm: Norm, mix: Optional[tuple]):
        self.norm, self.mix = norm, mix

    def __call__(self, y32: torch.Tensor, add_to: torch.Tensor) -> torch.Tensor:
        return self.norm(y32, add_to=add_to, mix=self.mix)


class LayeredBlock(nn.Module):
    """x <- x + mixer(norm1(x)); x <- x + ff(norm2(x)) when the layer has a feed-forward; with `post_norm` each sublayer's output
    goes through a norm of its own (norm1b, norm2b) before it is added.  `parallel`: one norm, h = norm1(x), and both sublayers read
    it: x <- x + mixer(h) + ff(h).  Without `pre_norm` (and with `post_norm`) the sublayers read the stream itself and norm1 / norm2
    act on their outputs: x <- x + norm1(mixer(x)), x <- x + norm2(ff(x)).  `canon_taps` > 0: what a sublayer reads (normed or not) is
    first replaced by itself plus a causal convolution over time (canon1 for the mixer, canon2 for the feed-forward; their last inputs
    are the layer's convolution state in the cache).  `depth_results` = n > 0: the block holds n weights `dwa` and, given
    `mix` = (stack, out), leaves in `out` the weighted average of stack[0 .. n-1], whose last entry is this layer's result.
    `x32` is updated in place."""

    def __init__(self, width: int, eps: float, mixer: nn.Module, mlp: Optional[nn.Module], norm: str = "rms", post_norm: bool = False,
                 parallel: bool = False, pre_norm: bool = True, canon_taps: int = 0, depth_results: int = 0):
        super().__init__()
        assert not (parallel and post_norm), "a parallel block with norms after the sublayers is not built"
        assert pre_norm or (post_norm and not parallel and canon_taps > 0), "sublayers that read the stream itself: norms after them, through a convolution"
        self.eps, self.parallel, self.pre_norm, self.width = eps, parallel, pre_norm, width
        self.norm1 = Norm(width, eps, norm)  # before the mixer; without pre_norm: after it
        self.norm1b = Norm(width, eps, norm) if post_norm and pre_norm else None
        self.mix = mixer
        self.mlp = mlp
        self.norm2 = Norm(width, eps, norm) if mlp is not None and not parallel else None
        self.norm2b = Norm(width, eps, norm) if mlp is not None and post_norm and pre_norm else None
        assert canon_taps == 0 or not pre_norm, "a convolution after a norm is not built"
        self.canon1 = CanonConv(width, canon_taps, 0) if canon_taps > 0 else None
        self.canon2 = CanonConv(width, canon_taps, 1) if canon_taps > 0 and mlp is not None else None
        self.depth_results = depth_results
        self.dwa = nn.Parameter(torch.empty(depth_results), requires_grad=False) if depth_results > 0 else None

    def conv_shape(self) -> Tuple[int, ...]:
        """fp32 numbers per sequence that the block's convolutions carry: [convolutions, taps - 1, width]."""
        if self.canon1 is None or self.canon1.taps < 2:
            return ()
        return (1 + int(self.canon2 is not None), self.canon1.taps - 1, self.width)

    def forward(self, x32: torch.Tensor, view: CacheView, ctx: Dict[str, torch.Tensor], mix: Optional[tuple] = None) -> torch.Tensor:
        if not self.pre_norm:
            m = (mix[0], self.depth_results, self.dwa, mix[1]) if mix is not None else None
            last_is_mixer = self.mlp is None
            self.mix.run(self.canon1(x32, view), x32, view, ctx, _PostNorm(self.norm1, m if last_is_mixer else None))
            if self.mlp is not None:
                self.mlp.run(self.canon2(x32, view), x32, _PostNorm(self.norm2, m))
            return x32
        assert mix is None, "the depth average follows a norm that adds to the stream"
        if self.parallel:  # the sublayers read hn only, so each may add its output to the stream as it finishes
            hn = self.norm1(x32)
            self.mix.run(hn, x32, view, ctx, None)
            if self.mlp is not None:
                self.mlp.run(hn, x32, None)
            return x32
        self.mix.run(self.norm1(x32), x32, view, ctx, self.norm1b)
        if self.mlp is not None:
            self.mlp.run(self.norm2(x32), x32, self.norm2b)
        return x32
