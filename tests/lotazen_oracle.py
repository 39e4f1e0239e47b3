"""Plain, slow statement of the Lotazen design: one function per mechanism, whole sequences, loops over tokens and heads.

Shares no code with the package.  `w` maps checkpoint names to tensors (any float dtype; everything is computed in the dtype
of `embed`, so a float64 copy of the weights gives a float64 oracle); `cfg` is the parsed config.json.
"""
import math
from typing import Dict, List, Optional

import torch


def clamped_glu(h, gate, up, down, limit: float):
    """Clamped gated unit: g = min(W_g h, limit), u = clamp(W_u h, +-limit), y = g sigmoid(1.702 g) (u + 1), out = W_d y."""
    g = (gate @ h).clamp(max=limit)
    u = (up @ h).clamp(min=-limit, max=limit)
    return down @ (g * torch.sigmoid(1.702 * g) * (u + 1))


def scalar_rms_norm(x, g, eps: float):
    """x / sqrt(mean(x^2) + eps) * g with ONE number g."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * g


def unit_rms(x, eps: float):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rotate_pairs(x, pos: int, base: float, dims: int, factor: float):
    """x [heads, dim]: entries (2i, 2i + 1), i < dims / 2, turn by pos * base^(-2i / dims) / factor; the rest pass."""
    out = x.clone()
    for i in range(dims // 2):
        a = pos * (base ** (-2.0 * i / dims)) / factor
        c, s = math.cos(a), math.sin(a)
        u, v = x[:, 2 * i], x[:, 2 * i + 1]
        out[:, 2 * i] = u * c - v * s
        out[:, 2 * i + 1] = v * c + u * s
    return out


def window_attention(hs, w: Dict[str, torch.Tensor], p: str, a: dict, eps: float):
    """Softmax attention of one sequence hs [T, width] (positions 0 .. T-1): rotated, unit-normed q and k, grouped key/value
    heads, a sliding window of mask.size positions (the token itself included)."""
    T = hs.shape[0]
    H, G, d, e = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
    rot = a.get("rot")
    win = (a.get("mask") or {}).get("size")
    qs, ks, vs = [], [], []
    for t in range(T):
        q = (w[p + "q"] @ hs[t]).view(H, d)
        k = (w[p + "k"] @ hs[t]).view(G, d)
        v = (w[p + "v"] @ hs[t]).view(G, e)
        if rot:
            f = float((rot.get("scaling") or {}).get("factor", 1.0))
            q = rotate_pairs(q, t, float(rot["base"]), int(rot["dims"]), f)
            k = rotate_pairs(k, t, float(rot["base"]), int(rot["dims"]), f)
        qs.append(unit_rms(q, eps)); ks.append(unit_rms(k, eps)); vs.append(v)
    K, V = torch.stack(ks), torch.stack(vs)  # [T, G, d], [T, G, e]
    out = []
    for t in range(T):
        lo = 0 if win is None else max(0, t - win + 1)  # the token sees itself and the win - 1 tokens before it
        heads = []
        for h in range(H):
            g = h // (H // G)
            pr = torch.softmax(K[lo:t + 1, g] @ qs[t][h] * a["scale"], 0)
            heads.append(pr @ V[lo:t + 1, g])
        out.append(w[p + "o"] @ torch.cat(heads))
    return torch.stack(out)


def hgrn2(hs, w: Dict[str, torch.Tensor], p: str, a: dict, eps: float):
    """Gated linear recurrence per head: S <- diag(f) S + (1 - f) v^T, o = S^T q, with f = l + (1 - l) sigmoid(W_f h + b)."""
    H, d, e = a["heads"], a["dim"], a["vdim"]
    S = [torch.zeros(d, e, dtype=hs.dtype) for _ in range(H)]
    low = w[p + "lower"].view(H, d)
    out = []
    for t in range(hs.shape[0]):
        q = torch.nn.functional.silu(w[p + "q"] @ hs[t]).view(H, d)
        v = (w[p + "v"] @ hs[t]).view(H, e)
        f = low + (1 - low) * torch.sigmoid((w[p + "f"] @ hs[t] + w[p + "f.b"]).view(H, d))
        heads = []
        for h in range(H):
            S[h] = f[h][:, None] * S[h] + (1 - f[h])[:, None] * v[h][None, :]
            o = S[h].t() @ q[h]
            heads.append(o / torch.sqrt((o * o).mean() + eps) * w[p + "norm"])
        out.append(w[p + "o"] @ torch.cat(heads))
    return torch.stack(out)


def mlstm(hs, w: Dict[str, torch.Tensor], p: str, a: dict, eps: float):
    """Matrix memory with exponential gates kept in range by a running maximum m (m starts at 0)."""
    H, d, e, cap = a["heads"], a["dim"], a["vdim"], float(a["gate_cap"])
    S = [torch.zeros(d, e, dtype=hs.dtype) for _ in range(H)]
    n = [torch.zeros(d, dtype=hs.dtype) for _ in range(H)]
    m = [torch.zeros((), dtype=hs.dtype) for _ in range(H)]
    out = []
    for t in range(hs.shape[0]):
        q = (w[p + "q"] @ hs[t]).view(H, d) * d ** -0.5
        k = (w[p + "k"] @ hs[t]).view(H, d)
        v = (w[p + "v"] @ hs[t]).view(H, e)
        ig = cap * torch.tanh((w[p + "i"] @ hs[t] + w[p + "i.b"]) / cap)
        fg = torch.nn.functional.logsigmoid(cap * torch.tanh((w[p + "f"] @ hs[t] + w[p + "f.b"]) / cap))
        heads = []
        for h in range(H):
            m_new = torch.maximum(fg[h] + m[h], ig[h])
            S[h] = torch.exp(fg[h] + m[h] - m_new) * S[h] + torch.exp(ig[h] - m_new) * k[h][:, None] * v[h][None, :]
            n[h] = torch.exp(fg[h] + m[h] - m_new) * n[h] + torch.exp(ig[h] - m_new) * k[h]
            m[h] = m_new
            o = S[h].t() @ q[h] / (torch.maximum((n[h] * q[h]).sum().abs(), torch.exp(-m_new)) + 1e-6)
            heads.append(o / torch.sqrt((o * o).mean() + eps))
        y = torch.cat(heads) * w[p + "norm"] * torch.sigmoid(w[p + "g"] @ hs[t])
        out.append(w[p + "o"] @ y)
    return torch.stack(out)


def route(h, router, top: int):
    """(indices, weights): the `top` largest sigmoid scores of the fp32 router, weights not renormalised."""
    s = torch.sigmoid(router @ h)
    idx = torch.topk(s, top).indices
    return idx.tolist(), [s[i] for i in idx.tolist()]


def moe(hs, w: Dict[str, torch.Tensor], p: str, a: dict):
    out = []
    for t in range(hs.shape[0]):
        idx, wt = route(hs[t], w[p + "router"], int(a["router"]["top"]))
        y = torch.zeros_like(hs[t])
        for e, s in zip(idx, wt):
            y = y + clamped_glu(s * hs[t], w[f"{p}e{e}.gate"], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"], float(a["expert"]["limit"]))
        if a.get("shared"):
            y = y + clamped_glu(hs[t], w[p + "shared.gate"], w[p + "shared.up"], w[p + "shared.down"], float(a["shared"]["limit"]))
        out.append(y)
    return torch.stack(out)


def mixer(hs, w, p: str, L: dict, eps: float):
    a = L["mixer"]
    if L["type"] == "parallel":
        return a["left_scale"] * window_attention(hs, w, p + "left.", a["left"], eps) + a["right_scale"] * hgrn2(hs, w, p + "right.", a["right"], eps)
    if L["type"] in ("mlstm", "mlstm_2"):
        return mlstm(hs, w, p, a, eps)
    raise ValueError(L["type"])


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], taps: Optional[list] = None):
    """Logits [T, vocab] of one whole sequence; `taps` collects the residual stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = torch.stack([w["embed"][t] + w["pos"][i] for i, t in enumerate(tokens)])
    for i, L in enumerate(cfg["layers"]):
        hs = scalar_rms_norm(x, w[f"l{i}.norm1"], eps)
        y = mixer(hs, w, f"l{i}.mix.", L, eps)
        if L.get("mlp") is not None:
            y = y + moe(hs, w, f"l{i}.mlp.", L["mlp"])
        x = x + y
        if taps is not None:
            taps.append(x.clone())
    z = scalar_rms_norm(x, w["final.norm"], eps) @ w["head"].t()
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * torch.tanh(z / cap) if cap > 0 else z
