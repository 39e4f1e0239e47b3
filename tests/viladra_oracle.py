"""Plain, slow statement of the Viladra design: one function per mechanism, whole sequences, loops over tokens and heads.

Shares no code with the package.  `w` maps checkpoint names to tensors (any float dtype; everything is computed in the dtype
of `embed`, so a float64 copy of the weights gives a float64 oracle); `cfg` is the parsed config.json.

The design in short.  Sublayers read the residual stream x itself, through a short causal convolution over time, and their OUTPUT is
RMS-normed before it is added: x <- x + norm1(mixer(x + conv1(x))), x <- x + norm2(ff(x + conv2(x))).  With X_0 the embedding
output and X_(i+1) the result of layer i, layer i + 1 (and after the last layer the final norm) reads sum_(j <= i+1) dwa_i[j] X_j.
Mixers: retention (fixed decay per head, rotated q and k), gated linear attention (decay per key channel), attention with sigmoid
weights inside a sliding window.  Feed-forward: a mixture of ungated experts with the squared rectifier, plus a shared expert.
The logits use the embedding table and are soft-capped.
"""
import math
from typing import Dict, List, Optional

import torch


def unit_rms(x, eps: float):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def causal_conv_added(xs, taps_w):
    """xs [T, width], taps_w [width, taps]: out_t = x_t + sum_j taps_w[:, j] * x_(t - taps + 1 + j), nothing before the first token."""
    T, taps = xs.shape[0], taps_w.shape[1]
    out = []
    for t in range(T):
        acc = xs[t].clone()
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                acc = acc + taps_w[:, j] * xs[s]
        out.append(acc)
    return torch.stack(out)


def rotate_halves(x, pos: int, base: float, dims: int):
    """x [heads, dim]: entry i < dims / 2 and entry i + dims / 2 turn together by pos * base^(-2i / dims); entries >= dims pass."""
    out = x.clone()
    half = dims // 2
    for i in range(half):
        a = pos * (base ** (-2.0 * i / dims))
        c, s = math.cos(a), math.sin(a)
        u, v = x[:, i], x[:, i + half]
        out[:, i] = u * c - v * s
        out[:, i + half] = v * c + u * s
    return out


def retention(hs, w: Dict[str, torch.Tensor], p: str, a: dict, eps: float):
    """Per head S <- decay_h S + (rot(k) / sqrt(dim)) v^T, o = S^T rot(q); every head divided by its root mean square; times
    silu(W_g h); W_o."""
    H, d, e = a["heads"], a["dim"], a["vdim"]
    rot = a.get("rot")
    S = [torch.zeros(d, e, dtype=hs.dtype) for _ in range(H)]
    out = []
    for t in range(hs.shape[0]):
        q = (w[p + "q"] @ hs[t]).view(H, d)
        k = (w[p + "k"] @ hs[t]).view(H, d)
        v = (w[p + "v"] @ hs[t]).view(H, e)
        if rot:
            q = rotate_halves(q, t, float(rot["base"]), int(rot["dims"]))
            k = rotate_halves(k, t, float(rot["base"]), int(rot["dims"]))
        k = k * d ** -0.5
        heads = []
        for h in range(H):
            S[h] = float(a["decay"][h]) * S[h] + torch.outer(k[h], v[h])
            heads.append(unit_rms(S[h].T @ q[h], eps))
        g = w[p + "g"] @ hs[t]
        out.append(w[p + "o"] @ (torch.cat(heads) * g * torch.sigmoid(g)))
    return torch.stack(out)


def gla(hs, w: Dict[str, torch.Tensor], p: str, a: dict, eps: float):
    """Per head S <- diag(alpha_t) S + k v^T with alpha = sigmoid(W_a2 W_a1 h + b)^(1 / tau) per key channel, o = S^T (q / sqrt(dim));
    every head RMS-normed with one weight [vdim]; times silu(W_g h); W_o."""
    H, d, e = a["heads"], a["dim"], a["vdim"]
    S = [torch.zeros(d, e, dtype=hs.dtype) for _ in range(H)]
    out = []
    for t in range(hs.shape[0]):
        q = (w[p + "q"] @ hs[t]).view(H, d) * d ** -0.5
        k = (w[p + "k"] @ hs[t]).view(H, d)
        v = (w[p + "v"] @ hs[t]).view(H, e)
        z = w[p + "a2"] @ (w[p + "a1"] @ hs[t]) + w[p + "a2.b"]
        alpha = torch.sigmoid(z).pow(1.0 / float(a["tau"])).view(H, d)
        heads = []
        for h in range(H):
            S[h] = alpha[h][:, None] * S[h] + torch.outer(k[h], v[h])
            heads.append(unit_rms(S[h].T @ q[h], eps) * w[p + "norm"])
        g = w[p + "g"] @ hs[t]
        out.append(w[p + "o"] @ (torch.cat(heads) * g * torch.sigmoid(g)))
    return torch.stack(out)


def sigmoid_attention(hs, w: Dict[str, torch.Tensor], p: str, a: dict, eps: float):
    """q, k, v with biases; q and k RMS-normed over the WHOLE projection with weights of that size; token t sees keys j with
    0 <= t - j < mask.size; a visible key weighs sigmoid(q.k * scale + pb[head]), not normalised; head h times sigmoid(W_g h)_h;
    W_o with bias."""
    T = hs.shape[0]
    H, G, d, e = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
    win = (a.get("mask") or {}).get("size")
    qs, ks, vs = [], [], []
    for t in range(T):
        q = w[p + "q"] @ hs[t] + w[p + "q.b"]
        k = w[p + "k"] @ hs[t] + w[p + "k.b"]
        qs.append((unit_rms(q, eps) * w[p + "q.norm"]).view(H, d))
        ks.append((unit_rms(k, eps) * w[p + "k.norm"]).view(G, d))
        vs.append((w[p + "v"] @ hs[t] + w[p + "v.b"]).view(G, e))
    out = []
    for t in range(T):
        lo = 0 if win is None else max(0, t - win + 1)
        gate = torch.sigmoid(w[p + "g"] @ hs[t])
        heads = []
        for h in range(H):
            g = h // (H // G)
            acc = torch.zeros(e, dtype=hs.dtype)
            for j in range(lo, t + 1):
                acc = acc + torch.sigmoid(torch.dot(qs[t][h], ks[j][g]) * a["scale"] + w[p + "pb"][h]) * vs[j][g]
            heads.append(acc * gate[h])
        out.append(w[p + "o"] @ torch.cat(heads) + w[p + "o.b"])
    return torch.stack(out)


def relu2_expert(h, up, down):
    return down @ torch.relu(up @ h).pow(2)


def router(h, w_router, top: int, scale: float):
    """(indices, weights): softmax over all experts, the `top` largest scores, weights score * scale, not renormalised."""
    s = torch.softmax(w_router @ h, 0)
    val, idx = torch.topk(s, top)
    return idx.tolist(), (val * scale).tolist()


def moe(hs, w: Dict[str, torch.Tensor], p: str, f: dict):
    r = f["router"]
    out = []
    for t in range(hs.shape[0]):
        idx, wts = router(hs[t], w[p + "router"], int(r["top"]), float(r.get("scale", 1.0)))
        y = torch.zeros_like(hs[t])
        for e, wt in zip(idx, wts):
            y = y + wt * relu2_expert(hs[t], w[f"{p}e{e}.up"], w[f"{p}e{e}.down"])
        if f.get("shared"):
            y = y + relu2_expert(hs[t], w[p + "shared.up"], w[p + "shared.down"])
        out.append(y)
    return torch.stack(out)


MIXERS = {"retention": retention, "gla": gla, "attention": sigmoid_attention}


def depth_average(results: List[torch.Tensor], coef):
    return sum(coef[j] * results[j] for j in range(len(results)))


def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], taps: Optional[list] = None, mixer_taps: Optional[list] = None):
    """Logits [T, vocab] of one sequence.  taps: gets the stream after every layer (after its depth average); mixer_taps: the raw
    mixer outputs."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens)] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    results = [x]
    for i, L in enumerate(cfg["layers"]):
        p = f"l{i}."
        y = MIXERS[L["type"]](causal_conv_added(x, w[p + "canon1"]), w, p + "mix.", L["mixer"], eps)
        if mixer_taps is not None:
            mixer_taps.append(y)
        x = x + unit_rms(y, eps) * w[p + "norm1"]
        if L.get("mlp"):
            x = x + unit_rms(moe(causal_conv_added(x, w[p + "canon2"]), w, p + "mlp.", L["mlp"]), eps) * w[p + "norm2"]
        results.append(x)
        x = depth_average(results, w[p + "dwa"])
        if taps is not None:
            taps.append(x)
    z = (unit_rms(x, eps) * w["final.norm"]) @ w["embed"].T
    cap = float(cfg.get("logit_softcap") or 0.0)
    return cap * torch.tanh(z / cap) if cap > 0 else z
