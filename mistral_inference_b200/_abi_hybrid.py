"""ctypes binding of libmb200_hybrid.so (C ABI: include/mistral_b200_hybrid.h): the kernels of layered decoders.

Same rules as `_abi`: the only place Python touches this library, and no fallback -- a missing library is built once
in-tree by `build.build_hybrid()` (a fresh checkout has no binaries), a failing call raises.
"""
import ctypes
import os
from ctypes import c_char_p, c_float, c_int, c_int64, c_void_p
from typing import Optional

import torch

from . import _abi, build
from ._abi import Mb200Error

ABI_VERSION = 4
EPI_STORE, EPI_RESIDUAL, EPI_GLU, EPI_F32, EPI_RESIDUAL_SCALED = 0, 1, 2, 3, 5
_DT = {torch.bfloat16: 0, torch.float32: 1}
_lib: Optional[ctypes.CDLL] = None

P, I, F = c_void_p, c_int64, c_float
_SIGNATURES = {
    "mbh_abi_version": (c_int, []),
    "mbh_last_error": (c_char_p, []),
    "mbh_embed_scale": (c_int, [P, P, F, P, I, I, c_int, P]),
    "mbh_rmsnorm": (c_int, [P, P, P, I, I, F, c_int, P]),
    "mbh_linear": (c_int, [P, P, P, P, P, I, I, I, c_int, I, F, F, c_int, P]),
    "mbh_linear_epilogue": (c_int, [P, P, P, P, I, I, c_int, I, F, F, c_int, P]),
    "mbh_attn_prep": (c_int, [P, P, P, P, P, P, P, P, P, P, c_int, I, I, I, I, I, F, F, I, c_int, P]),
    "mbh_attn_bias": (c_int, [P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, F, I, I, P, c_int, P]),
    "mbh_lightning_scan": (c_int, [P, P, P, P, P, P, P, I, I, I, I, c_int, P]),
    "mbh_gated_headnorm": (c_int, [P, P, P, I, I, P, I, I, F, c_int, P]),
    "mbh_embed_add": (c_int, [P, P, F, P, I, I, c_int, P]),
    "mbh_layernorm": (c_int, [P, P, P, P, P, I, I, F, c_int, P]),
    "mbh_linear_swiglu": (c_int, [P, P, P, I, I, I, P, I, I, c_int, P]),
    "mbh_swiglu_epilogue": (c_int, [P, P, I, I, P, I, I, c_int, P]),
    "mbh_latent_prep": (c_int, [P, P, P, P, P, P, P, P, I, I, I, I, I, I, F, F, c_int, P]),
    "mbh_latent_absorb": (c_int, [P, P, P, P, P, I, I, I, I, I, I, F, c_int, P]),
    "mbh_latent_expand": (c_int, [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, c_int, P]),
    "mbh_head_gate": (c_int, [P, P, I, I, I, I, I, c_int, P]),
    "mbh_attn_latent": (c_int, [P, P, P, P, P, P, I, I, I, I, I, I, F, I, P, c_int, P]),
    "mbh_attn_latent_decode": (c_int, [P, P, P, P, P, I, I, I, I, I, F, I, P, c_int, P]),
    "mbh_latent_vup": (c_int, [P, P, P, I, I, P, I, I, I, I, c_int, P]),
    "mbh_moe_route": (c_int, [P, P, P, P, P, P, I, I, I, I, I, I, c_int, F, c_int, P]),
    "mbh_moe_sparse": (c_int, [P, P, P, P, P, P, P, I, I, I, I, I, c_int, F, F, c_int, c_int, P]),
    "mbh_attn_window": (c_int, [P, P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, F, I, I, P, I, P, P, P, I, c_int, c_int, P]),
    "mbh_linear_glu": (c_int, [P, P, P, I, I, I, F, F, P, I, I, c_int, P]),
    "mbh_glu_epilogue": (c_int, [P, P, I, I, F, F, P, I, I, c_int, P]),
    "mbh_embed_pos": (c_int, [P, P, P, P, F, P, I, I, c_int, P]),
    "mbh_rot_prep": (c_int, [P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, c_int, F, c_int, P]),
    "mbh_kv_scatter": (c_int, [P, P, P, P, P, I, I, I, c_int, P]),
    "mbh_gated_scan": (c_int, [P, P, I, I, P, I, P, P, P, P, P, I, I, I, I, I, c_int, I, I, P, c_int, P]),
    "mbh_hgrn2_gates": (c_int, [P, P, P, I, I, I, c_int, P]),
    "mbh_mlstm_gates": (c_int, [P, P, P, P, P, I, I, P, P, P, I, I, I, I, I, F, F, c_int, P]),
    "mbh_scan_post": (c_int, [P, P, I, P, P, c_int, P, I, I, c_int, P, I, I, I, c_int, F, c_int, P]),
    "mbh_canon_conv": (c_int, [P, P, P, I, I, P, P, P, P, I, I, I, I, c_int, c_int, P]),
    "mbh_rmsnorm_add": (c_int, [P, P, P, I, I, F, P, I, P, I, P, c_int, P]),
    "mbh_depth_mix": (c_int, [P, I, P, I, P, I, c_int, P]),
    "mbh_retention_qab": (c_int, [P, I, P, P, P, P, I, I, I, I, F, c_int, P]),
    "mbh_gla_qab": (c_int, [P, I, P, P, I, I, F, F, c_int, P]),
    "mbh_whole_norm_prep": (c_int, [P, P, P, P, P, P, P, P, P, I, I, I, I, F, c_int, P]),
    "mbh_linear_relu2": (c_int, [P, P, P, I, I, I, P, I, I, c_int, P]),
    "mbh_relu2_epilogue": (c_int, [P, P, I, I, P, I, I, c_int, P]),
    "mbh_rows_axpy": (c_int, [P, P, P, I, I, I, I, c_int, P]),
}


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        path = build.build_hybrid()
        handle = ctypes.CDLL(str(path))
        for name, (restype, argtypes) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype, fn.argtypes = restype, argtypes
        if handle.mbh_abi_version() != ABI_VERSION:
            raise Mb200Error(f"libmb200_hybrid ABI {handle.mbh_abi_version()} != expected {ABI_VERSION}")
        _lib = handle
    return _lib


def _check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().mbh_last_error()
        raise Mb200Error(f"{what} failed ({rc}): {msg.decode() if msg else '?'}")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "libmb200_hybrid takes contiguous CUDA tensors"
    return t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def dt_of(dtype: torch.dtype) -> int:
    if dtype not in _DT:
        raise Mb200Error(f"layered decoders store activations and weights as bfloat16 or float32, not {dtype}")
    return _DT[dtype]


def embed_scale(tokens: torch.Tensor, table: torch.Tensor, scale: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    T, D = tokens.shape[0], table.shape[1]
    assert tokens.dtype == torch.long
    out = torch.empty(T, D, dtype=torch.float32, device=table.device) if out is None else out
    _check(lib().mbh_embed_scale(_ptr(tokens), _ptr(table), scale, _ptr(out), T, D, dt_of(table.dtype), _stream()), "mbh_embed_scale")
    return out


def rmsnorm(x32: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    T, D = x32.shape
    assert x32.dtype == torch.float32
    y = torch.empty(T, D, dtype=w.dtype, device=x32.device)
    _check(lib().mbh_rmsnorm(_ptr(x32), _ptr(w), _ptr(y), T, D, eps, dt_of(w.dtype), _stream()), "mbh_rmsnorm")
    return y


_ws: dict = {}


def _workspace(device: torch.device) -> "_abi.Workspace":
    if device not in _ws:
        _ws[device] = _abi.Workspace(_abi.workspace_bytes(1, 64, 1, 1, 128, 64, 0, 1), device)
    return _ws[device]


def _prompt_gemm_ok(x: torch.Tensor, M: int, N: int, K: int) -> bool:
    """Large bf16 Linears of prompts go to the main library's persistent tcgen05 GEMM when it is built and the shape fits its
    tiles (K % 64 == 0, N % 128 == 0, at least one 128-row tile); everything else runs on this library's own kernels.  A checkout
    that has only libmb200_hybrid.so never builds the main library for this."""
    return (x.dtype == torch.bfloat16 and M >= 128 and K % 64 == 0 and N % 128 == 0 and os.environ.get("MB200_HYBRID_GEMM", "1") != "0"
            and _abi.library_path().exists())


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None, *, epi: int = EPI_STORE, n_act: int = 0,
           residual: Optional[torch.Tensor] = None, limit: float = 0.0, alpha: float = 0.0) -> torch.Tensor:
    """x [M, K] @ w [N, K]^T with the epilogues of include/mistral_b200_hybrid.h.  EPI_RESIDUAL adds into `residual` (fp32, in
    place; EPI_RESIDUAL_SCALED: times `alpha`) and returns it; EPI_F32 returns fp32 [M, N] (soft-capped at `limit` when positive);
    EPI_GLU returns [M, N/2]."""
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and x.dtype == w.dtype
    out = out32 = None
    if epi in (EPI_RESIDUAL, EPI_RESIDUAL_SCALED):
        assert residual is not None and residual.dtype == torch.float32 and residual.shape == (M, N)
        out32 = residual
    elif epi == EPI_F32:
        out32 = torch.empty(M, N, dtype=torch.float32, device=x.device)
    else:
        out = torch.empty(M, N // 2 if epi == EPI_GLU else N, dtype=x.dtype, device=x.device)
    if _prompt_gemm_ok(x, M, N, K):
        # the framework's tcgen05 GEMM (bf16 out), then this library's epilogue over its result
        y = torch.empty(M, N, dtype=x.dtype, device=x.device)
        _abi.linear_residual(x, w, None, y, _workspace(x.device))
        _check(lib().mbh_linear_epilogue(_ptr(y), _ptr(bias), _ptr(out), _ptr(out32), M, N, epi, n_act, limit, alpha, dt_of(x.dtype), _stream()),
               "mbh_linear_epilogue")
        return out if out is not None else out32
    _check(lib().mbh_linear(_ptr(x), _ptr(w), _ptr(bias), _ptr(out), _ptr(out32), M, N, K, epi, n_act, limit, alpha, dt_of(x.dtype), _stream()),
           "mbh_linear")
    return out if out is not None else out32


def attn_prep(qkv, qnorm, knorm, positions, cache_rows, q_out, cache_k, cache_v, v_first, vmix, vmix_mode: int, H: int, G: int, d: int, e: int,
              eps: float, temp_coef: float, temp_every: int) -> None:
    _check(lib().mbh_attn_prep(_ptr(qkv), _ptr(qnorm), _ptr(knorm), _ptr(positions), _ptr(cache_rows), _ptr(q_out), _ptr(cache_k), _ptr(cache_v),
                               _ptr(v_first), _ptr(vmix), vmix_mode, qkv.shape[0], H, G, d, e, eps, temp_coef, temp_every, dt_of(qkv.dtype),
                               _stream()), "mbh_attn_prep")


def attn_bias(q, cache_k, cache_v, bias_tab, positions, q_start, slots, out, B: int, W: int, H: int, G: int, d: int, e: int, scale: float,
              n_tiles: int = 0, splits: int = 1) -> None:
    """n_tiles = sum over sequences of ceil(len / 64) selects the tensor-core prompt kernel (bf16); 0 the exact fp32 one."""
    assert bias_tab is None or (bias_tab.dtype == torch.float32 and bias_tab.shape[1] == H)
    scratch = torch.empty(q.shape[0] * H * splits * (2 + e), dtype=torch.float32, device=q.device) if splits > 1 and n_tiles == 0 else None
    _check(lib().mbh_attn_bias(_ptr(q), _ptr(cache_k), _ptr(cache_v), _ptr(bias_tab), bias_tab.shape[0] if bias_tab is not None else 0, _ptr(positions), _ptr(q_start), _ptr(slots),
                               _ptr(out), q.shape[0], B, W, H, G, d, e, scale, n_tiles, splits, _ptr(scratch), dt_of(q.dtype), _stream()), "mbh_attn_bias")


def attn_splits(T: int, H: int, W: int, n_sm: int = 148) -> int:
    """CTAs per (token, head) along the keys: enough to fill two CTAs per SM, at most one per 512 ring rows (a function of the
    batch and the ring only, so that a captured decode graph stays valid as the context grows)."""
    return int(max(1, min((2 * n_sm + T * H - 1) // (T * H), (W + 511) // 512, 32)))


def lightning_scan(qkvg, state, decay, q_start, seqpos, slots, o32, B: int, H: int, d: int, e: int) -> None:
    assert state.dtype == torch.float32 and decay.dtype == torch.float32 and o32.dtype == torch.float32
    _check(lib().mbh_lightning_scan(_ptr(qkvg), _ptr(state), _ptr(decay), _ptr(q_start), _ptr(seqpos), _ptr(slots), _ptr(o32), B, H, d, e,
                                    dt_of(qkvg.dtype), _stream()), "mbh_lightning_scan")


def gated_headnorm(o32, w, g, g_pitch: int, g_off: int, eps: float) -> torch.Tensor:
    T, N = o32.shape
    y = torch.empty(T, N, dtype=w.dtype, device=o32.device)
    _check(lib().mbh_gated_headnorm(_ptr(o32), _ptr(w), _ptr(g), g_pitch, g_off, _ptr(y), T, N, eps, dt_of(w.dtype), _stream()), "mbh_gated_headnorm")
    return y


# ------------------------------------------------------------------------------------------------ layer norm, re-added embedding
def embed_add(tokens: torch.Tensor, table: torch.Tensor, scale: float, x32: torch.Tensor) -> torch.Tensor:
    """x32 += table[tokens] * scale."""
    T, D = tokens.shape[0], table.shape[1]
    assert tokens.dtype == torch.long and x32.dtype == torch.float32 and x32.shape == (T, D)
    _check(lib().mbh_embed_add(_ptr(tokens), _ptr(table), scale, _ptr(x32), T, D, dt_of(table.dtype), _stream()), "mbh_embed_add")
    return x32


def layernorm(x32: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], eps: float, add_to: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Layer norm of fp32 rows.  Returns the normed rows in the weights' dtype, or, with `add_to` (fp32), adds them to it in fp32."""
    T, D = x32.shape
    assert x32.dtype == torch.float32
    if add_to is not None:
        assert add_to.dtype == torch.float32 and add_to.shape == x32.shape
        y = None
    else:
        y = torch.empty(T, D, dtype=w.dtype, device=x32.device)
    _check(lib().mbh_layernorm(_ptr(x32), _ptr(w), _ptr(b), _ptr(y), _ptr(add_to), T, D, eps, dt_of(w.dtype), _stream()), "mbh_layernorm")
    return y if add_to is None else add_to


# ------------------------------------------------------------------------------------------------ gated feed-forward, experts
def linear_swiglu(x: torch.Tensor, w: torch.Tensor, rowscale: Optional[torch.Tensor] = None, group: int = 0) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) with gate/up rows interleaved in w [2F, K]; column c is multiplied by rowscale[m, c // group]."""
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and x.dtype == w.dtype and N % 2 == 0
    pitch = 0
    if rowscale is not None:
        assert rowscale.dtype == torch.float32 and rowscale.shape[0] == M and group > 0 and (N // 2 + group - 1) // group <= rowscale.shape[1]
        pitch = rowscale.shape[1]
    out = torch.empty(M, N // 2, dtype=x.dtype, device=x.device)
    if _prompt_gemm_ok(x, M, N, K):
        y = torch.empty(M, N, dtype=x.dtype, device=x.device)
        _abi.linear_residual(x, w, None, y, _workspace(x.device))
        _check(lib().mbh_swiglu_epilogue(_ptr(y), _ptr(out), M, N, _ptr(rowscale), pitch, group, dt_of(x.dtype), _stream()), "mbh_swiglu_epilogue")
        return out
    _check(lib().mbh_linear_swiglu(_ptr(x), _ptr(w), _ptr(out), M, N, K, _ptr(rowscale), pitch, group, dt_of(x.dtype), _stream()), "mbh_linear_swiglu")
    return out


def moe_route(h: torch.Tensor, w_router: torch.Tensor, correction: Optional[torch.Tensor], groups: int, keep: int, top: int, score: int = 0,
              scale: float = 1.0):
    """(dense fp32 [T, n], idx int32 [T, top], wsel fp32 [T, top]) of the fp32 router; score 0: softmax, 1: sigmoid; the weights are the
    chosen scores times `scale`."""
    T, D = h.shape
    n = w_router.shape[0]
    dense = torch.empty(T, n, dtype=torch.float32, device=h.device)
    idx = torch.empty(T, top, dtype=torch.int32, device=h.device)
    wsel = torch.empty(T, top, dtype=torch.float32, device=h.device)
    _check(lib().mbh_moe_route(_ptr(h), _ptr(w_router), _ptr(correction), _ptr(dense), _ptr(idx), _ptr(wsel), T, D, n, groups, keep, top, score,
                               scale, dt_of(h.dtype), _stream()), "mbh_moe_route")
    return dense, idx, wsel


def moe_sparse(h: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, idx: torch.Tensor, wsel: torch.Tensor, E: int, ff: int,
               glu: int = 0, limit: float = 0.0, alpha: float = 0.0, add_to: Optional[torch.Tensor] = None) -> torch.Tensor:
    """fp32 [T, width]: the weighted sum of each token's chosen experts (indices >= E: identity), streaming only their weights.
    glu 1 (True): clamped gated experts whose INPUT is multiplied by the routing weight; glu 2: experts without a gate,
    W_down max(W_up h, 0)^2, with w13 [E * ff, width] plain rows.  add_to (fp32 [T, width], the residual stream): the
    sum is added to it in place instead of returned in a new tensor."""
    T, D = h.shape
    top = idx.shape[1]
    act = torch.empty(T * top, ff, dtype=h.dtype, device=h.device)
    if add_to is not None:
        assert add_to.dtype == torch.float32 and add_to.shape == (T, D)
    y32 = torch.empty(T, D, dtype=torch.float32, device=h.device) if add_to is None else add_to
    _check(lib().mbh_moe_sparse(_ptr(h), _ptr(w13), _ptr(w2), _ptr(idx), _ptr(wsel), _ptr(act), _ptr(y32), T, D, ff, E, top, int(glu), limit, alpha,
                                int(add_to is not None), dt_of(h.dtype), _stream()), "mbh_moe_sparse")
    return y32


def rows_axpy(y32: torch.Tensor, h: torch.Tensor, dense: torch.Tensor, first: int) -> None:
    """y32[t] += (dense[t, first:].sum()) * h[t]."""
    T, D = h.shape
    _check(lib().mbh_rows_axpy(_ptr(y32), _ptr(h), _ptr(dense), T, dense.shape[1], first, D, dt_of(h.dtype), _stream()), "mbh_rows_axpy")


# ------------------------------------------------------------------------------------------------ latent attention
def latent_prep(y, qnorm, cnorm, freq, positions, cache_rows, ring, q_rank: int, kv_rank: int, rot_dim: int, rot_dims: int, eps: float,
                mag: float) -> torch.Tensor:
    assert freq.dtype == torch.float64 and freq.numel() == rot_dims // 2
    T = y.shape[0]
    cq = torch.empty(T, q_rank, dtype=y.dtype, device=y.device)
    _check(lib().mbh_latent_prep(_ptr(y), _ptr(qnorm), _ptr(cnorm), _ptr(freq), _ptr(positions), _ptr(cache_rows), _ptr(cq), _ptr(ring), T,
                                 y.shape[1], q_rank, kv_rank, rot_dim, rot_dims, eps, mag, dt_of(y.dtype), _stream()), "mbh_latent_prep")
    return cq


FLASH_SIZES = {(32, 32), (64, 32), (64, 64), (128, 64), (64, 128), (128, 128), (96, 64), (192, 128)}  # (key, value) sizes of the tensor-core prompt kernel
_iota: dict = {}


def iota(n: int, device: torch.device) -> torch.Tensor:
    """int32 [n] = 0 .. n-1 (row blocks of a temporary ring), made once per device and length."""
    if (device, n) not in _iota:
        _iota[(device, n)] = torch.arange(n, dtype=torch.int32, device=device)
    return _iota[(device, n)]


def latent_expand(kn, v, ring, positions, cache_rows, q_start, B: int, Wt: int, H: int, dn: int, rot_dim: int, dv: int, kv_rank: int):
    kfull = torch.empty(B * Wt, H, dn + rot_dim, dtype=kn.dtype, device=kn.device)
    vfull = torch.empty(B * Wt, H, dv, dtype=kn.dtype, device=kn.device)
    _check(lib().mbh_latent_expand(_ptr(kn), _ptr(v), _ptr(ring), _ptr(positions), _ptr(cache_rows), _ptr(q_start), _ptr(kfull), _ptr(vfull), kn.shape[0],
                                   B, Wt, H, dn, rot_dim, dv, kv_rank, dt_of(kn.dtype), _stream()), "mbh_latent_expand")
    return kfull, vfull


def head_gate(out, gate, g_pitch: int, g_off: int, H: int, dv: int) -> None:
    _check(lib().mbh_head_gate(_ptr(out), _ptr(gate), g_pitch, g_off, out.shape[0], H, dv, dt_of(out.dtype), _stream()), "mbh_head_gate")


def latent_absorb(q, w_uk, freq, positions, H: int, dn: int, rot_dim: int, rot_dims: int, kv_rank: int, mag: float) -> torch.Tensor:
    """w_uk None: the queries are only rotated ([T, H * (dn + rot_dim)])."""
    T = q.shape[0]
    qa = torch.empty(T, H * ((kv_rank if w_uk is not None else dn) + rot_dim), dtype=q.dtype, device=q.device)
    _check(lib().mbh_latent_absorb(_ptr(q), _ptr(w_uk), _ptr(freq), _ptr(positions), _ptr(qa), T, H, dn, rot_dim, rot_dims, kv_rank, mag,
                                   dt_of(q.dtype), _stream()), "mbh_latent_absorb")
    return qa


def attn_latent(qa, ring, positions, q_start, slots, B: int, W: int, H: int, kv_rank: int, rot_dim: int, scale: float, splits: int = 1) -> torch.Tensor:
    T = qa.shape[0]
    o = torch.empty(T, H * kv_rank, dtype=qa.dtype, device=qa.device)
    scratch = torch.empty(T * H * splits * (2 + kv_rank), dtype=torch.float32, device=qa.device) if splits > 1 else None
    _check(lib().mbh_attn_latent(_ptr(qa), _ptr(ring), _ptr(positions), _ptr(q_start), _ptr(slots), _ptr(o), T, B, W, H, kv_rank, rot_dim, scale,
                                 splits, _ptr(scratch), dt_of(qa.dtype), _stream()), "mbh_attn_latent")
    return o


LATENT_DECODE_MAX_HEADS, LATENT_DECODE_MAX_RANK = 32, 512


def latent_decode_splits(B: int, W: int, n_sm: int = 148) -> int:
    """CTAs per sequence along the keys: two CTAs per SM over the batch, at least 64 ring rows each (batch and ring size only, so a
    captured decode graph stays valid as the context grows)."""
    return int(max(1, min((2 * n_sm) // B, (W + 63) // 64, 64)))


def attn_latent_decode(qa, ring, positions, slots, B: int, W: int, H: int, kv_rank: int, rot_dim: int, scale: float) -> torch.Tensor:
    splits = latent_decode_splits(B, W)
    o = torch.empty(B, H * kv_rank, dtype=qa.dtype, device=qa.device)
    scratch = torch.empty(B * H * splits * (2 + kv_rank), dtype=torch.float32, device=qa.device)
    _check(lib().mbh_attn_latent_decode(_ptr(qa), _ptr(ring), _ptr(positions), _ptr(slots), _ptr(o), B, W, H, kv_rank, rot_dim, scale, splits,
                                        _ptr(scratch), dt_of(qa.dtype), _stream()), "mbh_attn_latent_decode")
    return o


def latent_vup(o_lat, w_uv, gate, g_pitch: int, g_off: int, H: int, dv: int, kv_rank: int) -> torch.Tensor:
    T = o_lat.shape[0]
    out = torch.empty(T, H * dv, dtype=o_lat.dtype, device=o_lat.device)
    _check(lib().mbh_latent_vup(_ptr(o_lat), _ptr(w_uv), _ptr(gate), g_pitch, g_off, _ptr(out), T, H, dv, kv_rank, dt_of(o_lat.dtype), _stream()),
           "mbh_latent_vup")
    return out


# ------------------------------------------------------------------------------------------------ learned positions, rotary window attention
def embed_pos(tokens: torch.Tensor, positions: torch.Tensor, table: torch.Tensor, pos_table: torch.Tensor, scale: float) -> torch.Tensor:
    """fp32 [T, D] = table[tokens] * scale + pos_table[positions]."""
    T, D = tokens.shape[0], table.shape[1]
    assert tokens.dtype == torch.long and positions.dtype == torch.int32 and pos_table.shape[1] == D and pos_table.dtype == table.dtype
    out = torch.empty(T, D, dtype=torch.float32, device=table.device)
    _check(lib().mbh_embed_pos(_ptr(tokens), _ptr(positions), _ptr(table), _ptr(pos_table), scale, _ptr(out), T, D, dt_of(table.dtype), _stream()),
           "mbh_embed_pos")
    return out


def rot_prep(qkv, freq, positions, cache_rows, ring_k, ring_v, H: int, G: int, d: int, e: int, rot_dims: int, unit_norm: bool, eps: float, own: bool):
    """(q [T, H*d], k [T, G*d] or None, v [T, G*e] or None): rotated (and unit-normed) queries and keys.  `own`: k and v are
    returned token-major; `cache_rows` given: they are written into the ring rows as well."""
    assert freq.dtype == torch.float64 and freq.numel() == rot_dims // 2
    T = qkv.shape[0]
    q = torch.empty(T, H * d, dtype=qkv.dtype, device=qkv.device)
    k = torch.empty(T, G * d, dtype=qkv.dtype, device=qkv.device) if own else None
    v = torch.empty(T, G * e, dtype=qkv.dtype, device=qkv.device) if own else None
    _check(lib().mbh_rot_prep(_ptr(qkv), _ptr(freq), _ptr(positions), _ptr(cache_rows), _ptr(q), _ptr(k), _ptr(v), _ptr(ring_k), _ptr(ring_v), T, H, G,
                              d, e, rot_dims, int(unit_norm), eps, dt_of(qkv.dtype), _stream()), "mbh_rot_prep")
    return q, k, v


def kv_scatter(k, v, cache_rows, ring_k, ring_v) -> None:
    _check(lib().mbh_kv_scatter(_ptr(k), _ptr(v), _ptr(cache_rows), _ptr(ring_k), _ptr(ring_v), k.shape[0], k.shape[1], v.shape[1], dt_of(k.dtype),
                                _stream()), "mbh_kv_scatter")


def attn_window(q, cache_k, cache_v, positions, q_start, slots, out, B: int, W: int, H: int, G: int, d: int, e: int, scale: float, window: int,
                own_k=None, own_v=None, seqpos=None, n_tiles: int = 0, splits: int = 1, chunk: int = 0, head_bias=None) -> None:
    """`attn_bias` without a bias, with a sliding window (0: none) and, for prompts, this call's own keys and values beside the ring.
    chunk: keys per warp and step of the exact kernel (0: 128), see `window_decode_plan`.  head_bias (fp32 [H]): sigmoid weights instead
    of the softmax, every visible key weighing sigmoid(score + head_bias[h]), not normalised."""
    scratch = torch.empty(q.shape[0] * H * splits * (2 + e), dtype=torch.float32, device=q.device) if splits > 1 and n_tiles == 0 else None
    assert head_bias is None or (head_bias.dtype == torch.float32 and head_bias.numel() == H)
    _check(lib().mbh_attn_window(_ptr(q), _ptr(cache_k), _ptr(cache_v), _ptr(head_bias), int(head_bias is not None), _ptr(positions), _ptr(q_start),
                                 _ptr(slots), _ptr(out), q.shape[0], B, W, H, G, d, e, scale, n_tiles, splits, _ptr(scratch), window, _ptr(own_k),
                                 _ptr(own_v), _ptr(seqpos), chunk, int(head_bias is not None), dt_of(q.dtype), _stream()), "mbh_attn_window")


def window_decode_plan(T: int, H: int, W: int):
    """(splits, chunk) of a decode step over a ring of W rows: a CTA of 4 warps takes 4 * chunk keys per round.  32-key chunks (a
    key per lane) and one round per CTA measured fastest from 1 to 32 sequences over rings of 72 to 4096 rows: a decode step's
    attention is latency, not bandwidth, and the ring is spread over ceil(W / 128) CTAs per (token, head) -- fewer when the batch
    alone gives thousands of CTAs.  A function of the batch and the ring only (CUDA-graph decode)."""
    chunk = 32
    splits = max(1, min((W + 4 * chunk - 1) // (4 * chunk), 8192 // max(T * H, 1), 64))
    return int(splits), chunk


# ------------------------------------------------------------------------------------------------ gated linear recurrences
SCAN_CHUNK = 256       # tokens per chunk of the chunk-parallel scan
SCAN_CHUNK_FROM = 512  # sequences (portions) at least this long run chunk-parallel


def gated_scan(qab, v, v_pitch: int, v_off: int, state, q_start, seqpos, slots, B: int, H: int, d: int, e: int, ones: bool,
               max_seqlen: int = 0):
    """fp32 o [T, H * e] of S <- diag(a) S + b v^T, o = S^T q; the state rows of `slots` are read and written.  With `ones` the state
    has a normaliser column and the result is (o, nq [T, H * d]) for `scan_post`.  With the longest sequence of the call given and at
    least SCAN_CHUNK_FROM, the scan runs chunk-parallel (same recurrence, fp32)."""
    assert qab.dtype == torch.float32 and state.dtype == torch.float32
    T = qab.shape[0]
    ec = e + int(ones)
    o = torch.empty(T, H * e, dtype=torch.float32, device=qab.device)
    nq = torch.empty(T, H * d, dtype=torch.float32, device=qab.device) if ones else None
    chunks, scratch = 1, None
    if max_seqlen >= SCAN_CHUNK_FROM and max_seqlen > SCAN_CHUNK:
        chunks = (max_seqlen + SCAN_CHUNK - 1) // SCAN_CHUNK
        scratch = torch.empty(B * H * chunks * d * (ec + 1), dtype=torch.float32, device=qab.device)
    _check(lib().mbh_gated_scan(_ptr(qab), _ptr(v), v_pitch, v_off, _ptr(state), state[0].numel(), _ptr(q_start), _ptr(seqpos), _ptr(slots), _ptr(o), _ptr(nq), T, B, H,
                                d, e, int(ones), SCAN_CHUNK, chunks, _ptr(scratch), dt_of(v.dtype), _stream()), "mbh_gated_scan")
    return (o, nq) if ones else o


def hgrn2_gates(qfv, lower, Hd: int) -> torch.Tensor:
    T = qfv.shape[0]
    qab = torch.empty(T, 3, Hd, dtype=torch.float32, device=qfv.device)
    _check(lib().mbh_hgrn2_gates(_ptr(qfv), _ptr(lower), _ptr(qab), T, Hd, qfv.shape[1], dt_of(qfv.dtype), _stream()), "mbh_hgrn2_gates")
    return qab


def mlstm_gates(qkvg, gif, state, m_off: int, q_start, seqpos, slots, B: int, H: int, d: int, cap: float, qscale: float):
    """(gates fp32 [T, H, 3], qab fp32 [T, 3, H*d]); advances the running maxima kept in `state`."""
    T = qkvg.shape[0]
    gates = torch.empty(T, H, 3, dtype=torch.float32, device=qkvg.device)
    qab = torch.empty(T, 3, H * d, dtype=torch.float32, device=qkvg.device)
    _check(lib().mbh_mlstm_gates(_ptr(qkvg), _ptr(gif), _ptr(gates), _ptr(qab), _ptr(state), state[0].numel(), m_off, _ptr(q_start), _ptr(seqpos),
                                 _ptr(slots), T, B, H, d, qkvg.shape[1], cap, qscale, dt_of(qkvg.dtype), _stream()), "mbh_mlstm_gates")
    return gates, qab


def scan_post(o32, gates, w, w_per_head: bool, gate, g_pitch: int, g_off: int, H: int, e: int, ones: bool, eps: float, nq=None, silu_gate: bool = False,
              dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """Every head of o32 divided by its root mean square, times w (None: no weight; then `dtype` names the storage type) and the gate's
    sigmoid (silu_gate: its SiLU)."""
    T = o32.shape[0]
    dtype = w.dtype if w is not None else (gate.dtype if gate is not None else dtype)
    y = torch.empty(T, H * e, dtype=dtype, device=o32.device)
    _check(lib().mbh_scan_post(_ptr(o32), _ptr(nq), nq.shape[1] // H if nq is not None else 0, _ptr(gates), _ptr(w), int(w_per_head), _ptr(gate), g_pitch, g_off,
                               int(silu_gate), _ptr(y), T, H, e, int(ones), eps, dt_of(dtype), _stream()), "mbh_scan_post")
    return y


def linear_glu(x: torch.Tensor, w: torch.Tensor, limit: float, alpha: float, rowscale: Optional[torch.Tensor] = None, group: int = 0) -> torch.Tensor:
    """The clamped gated unit over interleaved gate/up rows of w [2F, K]; gate and up of column c are multiplied by
    rowscale[m, c // group] before the clamps (experts whose input is scaled by the routing weight, run densely)."""
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and x.dtype == w.dtype and N % 2 == 0
    pitch = 0
    if rowscale is not None:
        assert rowscale.dtype == torch.float32 and rowscale.shape[0] == M and group > 0 and (N // 2 + group - 1) // group <= rowscale.shape[1]
        pitch = rowscale.shape[1]
    out = torch.empty(M, N // 2, dtype=x.dtype, device=x.device)
    if _prompt_gemm_ok(x, M, N, K):
        y = torch.empty(M, N, dtype=x.dtype, device=x.device)
        _abi.linear_residual(x, w, None, y, _workspace(x.device))
        _check(lib().mbh_glu_epilogue(_ptr(y), _ptr(out), M, N, limit, alpha, _ptr(rowscale), pitch, group, dt_of(x.dtype), _stream()), "mbh_glu_epilogue")
        return out
    _check(lib().mbh_linear_glu(_ptr(x), _ptr(w), _ptr(out), M, N, K, limit, alpha, _ptr(rowscale), pitch, group, dt_of(x.dtype), _stream()), "mbh_linear_glu")
    return out


# ------------------------------------------------------------------------------------------------ sublayers that read the stream itself
def canon_conv(x32: torch.Tensor, w: torch.Tensor, state: Optional[torch.Tensor], state_off: int, q_start, seqpos, slots, B: int, one_each: bool) -> torch.Tensor:
    """h = x32 + causal convolution over time of x32 on every channel (w [D, taps]), in the weights' dtype; the sequences' last taps - 1
    inputs live in `state` (fp32 [rows, ...], this convolution's part at `state_off` floats into a row) and are advanced."""
    T, D = x32.shape
    assert x32.dtype == torch.float32 and w.shape[0] == D
    assert (state is None and w.shape[1] == 1) or state.dtype == torch.float32, "more than one tap needs the state of the last inputs"
    h = torch.empty(T, D, dtype=w.dtype, device=x32.device)
    _check(lib().mbh_canon_conv(_ptr(x32), _ptr(w), _ptr(state), state[0].numel() if state is not None else 0, state_off, _ptr(q_start), _ptr(seqpos), _ptr(slots), _ptr(h), T, B, D,
                                w.shape[1], int(one_each), dt_of(w.dtype), _stream()), "mbh_canon_conv")
    return h


def rmsnorm_add(y32: torch.Tensor, w: torch.Tensor, acc32: torch.Tensor, eps: float, stack: Optional[torch.Tensor] = None, n: int = 0,
                coef: Optional[torch.Tensor] = None, out32: Optional[torch.Tensor] = None) -> torch.Tensor:
    """acc32 += rms_norm(y32) * w.  With stack (fp32 [>= n, T, D], whose row n - 1 is acc32): out32 = sum_j coef[j] * stack[j]."""
    T, D = y32.shape
    assert y32.dtype == torch.float32 and acc32.dtype == torch.float32 and acc32.shape == y32.shape
    if stack is not None:
        assert stack.dtype == torch.float32 and coef.numel() == n and coef.dtype == w.dtype and out32.shape == y32.shape
        assert stack[n - 1].data_ptr() == acc32.data_ptr(), "the last averaged result is the stream that was just updated"
    _check(lib().mbh_rmsnorm_add(_ptr(y32), _ptr(w), _ptr(acc32), T, D, eps, _ptr(stack), T * D, _ptr(coef), n, _ptr(out32), dt_of(w.dtype), _stream()),
           "mbh_rmsnorm_add")
    return acc32


def depth_mix(stack: torch.Tensor, n: int, coef: torch.Tensor, out32: torch.Tensor) -> torch.Tensor:
    """out32 = sum_(j < n) coef[j] * stack[j]; stack fp32 [>= n, T, D]."""
    assert stack.dtype == torch.float32 and out32.dtype == torch.float32 and coef.numel() == n
    _check(lib().mbh_depth_mix(_ptr(stack), stack[0].numel(), _ptr(coef), n, _ptr(out32), out32.numel(), dt_of(coef.dtype), _stream()), "mbh_depth_mix")
    return out32


def retention_qab(qk: torch.Tensor, freq: torch.Tensor, decay: torch.Tensor, positions, H: int, d: int, rot_dims: int, kscale: float) -> torch.Tensor:
    assert freq.dtype == torch.float64 and freq.numel() == rot_dims // 2 and decay.dtype == torch.float32 and decay.numel() == H
    T = qk.shape[0]
    qab = torch.empty(T, 3, H * d, dtype=torch.float32, device=qk.device)
    _check(lib().mbh_retention_qab(_ptr(qk), qk.shape[1], _ptr(freq), _ptr(decay), _ptr(positions), _ptr(qab), T, H, d, rot_dims, kscale, dt_of(qk.dtype),
                                   _stream()), "mbh_retention_qab")
    return qab


def gla_qab(qk: torch.Tensor, z32: torch.Tensor, Hd: int, qscale: float, inv_tau: float) -> torch.Tensor:
    T = qk.shape[0]
    assert z32.dtype == torch.float32 and z32.shape == (T, Hd)
    qab = torch.empty(T, 3, Hd, dtype=torch.float32, device=qk.device)
    _check(lib().mbh_gla_qab(_ptr(qk), qk.shape[1], _ptr(z32), _ptr(qab), T, Hd, qscale, inv_tau, dt_of(qk.dtype), _stream()), "mbh_gla_qab")
    return qab


def whole_norm_prep(qkv, qnorm, knorm, cache_rows, ring_k, ring_v, Nq: int, Nk: int, Nv: int, eps: float, own: bool):
    """(q, k or None, v or None) with q and k RMS-normed over their whole projections; `own`: k and v returned token-major;
    `cache_rows` given: written into the ring rows."""
    T = qkv.shape[0]
    q = torch.empty(T, Nq, dtype=qkv.dtype, device=qkv.device)
    k = torch.empty(T, Nk, dtype=qkv.dtype, device=qkv.device) if own else None
    v = torch.empty(T, Nv, dtype=qkv.dtype, device=qkv.device) if own else None
    _check(lib().mbh_whole_norm_prep(_ptr(qkv), _ptr(qnorm), _ptr(knorm), _ptr(cache_rows), _ptr(q), _ptr(k), _ptr(v), _ptr(ring_k), _ptr(ring_v), T, Nq,
                                     Nk, Nv, eps, dt_of(qkv.dtype), _stream()), "mbh_whole_norm_prep")
    return q, k, v


def linear_relu2(x: torch.Tensor, w: torch.Tensor, rowscale: Optional[torch.Tensor] = None, group: int = 0) -> torch.Tensor:
    """max(x W^T, 0)^2, column c multiplied by rowscale[m, c // group] (experts without a gate, run densely)."""
    M, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and x.dtype == w.dtype
    pitch = 0
    if rowscale is not None:
        assert rowscale.dtype == torch.float32 and rowscale.shape[0] == M and group > 0 and (N + group - 1) // group <= rowscale.shape[1]
        pitch = rowscale.shape[1]
    out = torch.empty(M, N, dtype=x.dtype, device=x.device)
    if _prompt_gemm_ok(x, M, N, K):
        y = torch.empty(M, N, dtype=x.dtype, device=x.device)
        _abi.linear_residual(x, w, None, y, _workspace(x.device))
        _check(lib().mbh_relu2_epilogue(_ptr(y), _ptr(out), M, N, _ptr(rowscale), pitch, group, dt_of(x.dtype), _stream()), "mbh_relu2_epilogue")
        return out
    _check(lib().mbh_linear_relu2(_ptr(x), _ptr(w), _ptr(out), M, N, K, _ptr(rowscale), pitch, group, dt_of(x.dtype), _stream()), "mbh_linear_relu2")
    return out
