"""Small random Viladra models for the tests: configurations, weights with the checkpoint's names, folders on disk."""
import json
import math
from pathlib import Path
from typing import Dict, Optional

import torch


def retention_cfg(heads=3, dim=10, vdim=6, decay=(0.9, 0.97, 0.5), rot=(100.0, 6)) -> dict:
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return {"type": "retention", "mixer": m}


def gla_cfg(heads=2, dim=12, vdim=10, tau=8.0, rank=5) -> dict:
    # `rank` is not part of config.json (the checkpoint's tensors give it); make_weights reads it and make_config drops it
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "_rank": rank}


def attn_cfg(heads=4, kv_heads=2, dim=12, vdim=10, scale=0.5, window: Optional[int] = 5) -> dict:
    a = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        a["mask"] = {"size": window}
    return {"type": "attention", "mixer": a}


def moe_cfg(ff=12, experts=5, top=2, scale=1.3, shared: Optional[int] = 20) -> dict:
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "scale": scale}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def make_config(width=40, vocab=50, layers=None, eps=1e-4, taps=4, softcap=9.0, embed_scale=2.0) -> dict:
    """layers: list of (mixer entry from retention_cfg / gla_cfg / attn_cfg, mlp dict or None)."""
    cfg = {"architecture": "Viladra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "canon": {"taps": taps}, "embedding": {"scale": embed_scale},
           "logit_softcap": softcap, "layers": [{"type": m["type"], "mixer": m["mixer"], "mlp": f} for m, f in layers]}
    cfg["_ranks"] = [m.get("_rank", 0) for m, _ in layers]
    return cfg


def on_disk(cfg: dict) -> dict:
    return {k: v for k, v in cfg.items() if not k.startswith("_")}


def make_weights(cfg: dict, seed: int = 0, dtype=torch.float32, router_gain: float = 4.0, long_memory: bool = False) -> Dict[str, torch.Tensor]:
    """long_memory: decays close to 1 (the fixed ones are the configuration's; the gated ones get a large bias), so that what a state
    took in hundreds of tokens ago still shows in the output."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    taps = cfg["canon"]["taps"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * s / math.sqrt(i)).to(dtype)

    def vec(n, mean=0.0, s=0.3):
        return (mean + s * torch.randn(n, generator=g)).to(dtype)

    w = {"embed": torch.randn(cfg["vocab"], W, generator=g).to(dtype), "final.norm": vec(W, 1.0)}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", L["mixer"]
        w[f"l{i}.norm1"] = vec(W, 1.0)
        w[f"l{i}.canon1"] = (0.4 * torch.randn(W, taps, generator=g)).to(dtype)
        w[f"l{i}.dwa"] = (torch.cat([0.3 * torch.randn(i + 1, generator=g), torch.ones(1)]) / math.sqrt(i + 2.0)).to(dtype)
        if L["type"] == "attention":
            H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[p + "q"], w[p + "k"], w[p + "v"] = mat(H * d, W, 2.0), mat(G * d, W, 2.0), mat(G * e, W)
            w[p + "q.b"], w[p + "k.b"], w[p + "v.b"] = vec(H * d), vec(G * d), vec(G * e)
            w[p + "q.norm"], w[p + "k.norm"] = vec(H * d, 1.0), vec(G * d, 1.0)
            w[p + "pb"], w[p + "g"] = vec(H, -0.5, 0.7), mat(H, W, 2.0)
            w[p + "o"], w[p + "o.b"] = mat(W, H * e), vec(W)
        else:
            H, d, e = m["heads"], m["dim"], m["vdim"]
            w[p + "q"], w[p + "k"], w[p + "v"], w[p + "g"] = mat(H * d, W, 2.0), mat(H * d, W, 2.0), mat(H * e, W), mat(H * e, W, 2.0)
            w[p + "o"] = mat(W, H * e)
            if L["type"] == "gla":
                r = cfg["_ranks"][i]
                w[p + "a1"], w[p + "a2"] = mat(r, W, 2.0), mat(H * d, r, 2.0)
                w[p + "a2.b"] = vec(H * d, 7.0 if long_memory else 1.0, 1.0)
                w[p + "norm"] = vec(e, 1.0)
        if L["mlp"]:
            q, f = f"l{i}.mlp.", L["mlp"]
            w[f"l{i}.norm2"] = vec(W, 1.0)
            w[f"l{i}.canon2"] = (0.4 * torch.randn(W, taps, generator=g)).to(dtype)
            w[q + "router"] = mat(f["router"]["experts"], W, router_gain)
            for e in range(f["router"]["experts"]):
                ff = f["expert"]["ff"]
                w[f"{q}e{e}.up"], w[f"{q}e{e}.down"] = mat(ff, W, 2.0), mat(W, ff, 2.0)
            if f.get("shared"):
                w[q + "shared.up"], w[q + "shared.down"] = mat(f["shared"]["ff"], W, 2.0), mat(W, f["shared"]["ff"], 2.0)
    return w


def write_folder(path: Path, cfg: dict, weights: Dict[str, torch.Tensor]) -> Path:
    from safetensors.torch import save_file

    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(on_disk(cfg)))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(path / "model.safetensors"))
    return path


def f32(weights: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return {k: v.float() for k, v in weights.items()}
