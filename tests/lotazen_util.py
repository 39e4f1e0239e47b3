"""Small random Lotazen models for the tests: configurations, weights with the checkpoint's names, folders on disk."""
import json
import math
from pathlib import Path
from typing import Dict, Optional

import torch


def attn_cfg(heads=4, kv_heads=2, dim=12, vdim=10, scale=0.6, window: Optional[int] = 5, rot=(100.0, 8, 3.0)) -> dict:
    a = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        a["mask"] = {"size": window}
    if rot is not None:
        a["rot"] = {"base": rot[0], "dims": rot[1]}
        if rot[2] is not None:
            a["rot"]["scaling"] = {"factor": rot[2]}
    return a


def side_cfg(left=None, right=None, left_scale=0.7, right_scale=1.3) -> dict:
    return {"type": "parallel", "mixer": {"left": left or attn_cfg(), "right": right or {"heads": 3, "dim": 10, "vdim": 7},
                                          "left_scale": left_scale, "right_scale": right_scale}}


def mlstm_cfg(heads=3, dim=10, vdim=14, cap=8.0, kind="mlstm") -> dict:
    return {"type": kind, "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def moe_cfg(ff=12, limit=0.8, experts=5, top=2, shared=(20, 1.5)) -> dict:
    m = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


def make_config(width=40, vocab=50, layers=None, eps=1e-4, max_positions=1024, softcap=9.0) -> dict:
    """layers: list of (mixer entry from side_cfg / mlstm_cfg, mlp dict or None)."""
    return {"architecture": "Lotazen", "vocab": vocab, "width": width, "norm": {"eps": eps}, "max_positions": max_positions,
            "logit_softcap": softcap, "layers": [{**m, "mlp": f} for m, f in layers]}


def make_weights(cfg: dict, seed: int = 0, dtype=torch.float32, router_gain: float = 4.0, long_memory: bool = False) -> Dict[str, torch.Tensor]:
    """long_memory: forget gates close to 1 (lower bounds up to 0.9995, large forget biases), so that what a recurrent state took
    in hundreds of tokens ago still shows in the output."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def mat(o, i, s=1.0):
        return (torch.randn(o, i, generator=g) * s / math.sqrt(i)).to(dtype)

    def vec(n, mean=0.0, s=0.3):
        return (mean + s * torch.randn(n, generator=g)).to(dtype)

    def one(mean=1.0, s=0.2):
        return (mean + s * torch.randn((), generator=g)).to(dtype)

    w = {"embed": torch.randn(cfg["vocab"], W, generator=g).to(dtype), "pos": (0.5 * torch.randn(cfg["max_positions"], W, generator=g)).to(dtype),
         "head": mat(cfg["vocab"], W, 3.0), "final.norm": one()}
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", L["mixer"]
        w[f"l{i}.norm1"] = one()
        if L["type"] == "parallel":
            a, r = m["left"], m["right"]
            w[p + "left.q"], w[p + "left.k"] = mat(a["heads"] * a["dim"], W, 2.0), mat(a["kv_heads"] * a["dim"], W, 2.0)
            w[p + "left.v"], w[p + "left.o"] = mat(a["kv_heads"] * a["vdim"], W), mat(W, a["heads"] * a["vdim"])
            n = r["heads"] * r["dim"]
            w[p + "right.q"], w[p + "right.f"], w[p + "right.f.b"] = mat(n, W), mat(n, W, 2.0), vec(n, 0.0, 1.0)
            lo = torch.rand(n, generator=g)
            w[p + "right.lower"] = (1 - 0.5 * 10 ** (-3 * lo) if long_memory else lo * 0.9).to(dtype)
            w[p + "right.v"], w[p + "right.norm"], w[p + "right.o"] = mat(r["heads"] * r["vdim"], W), vec(r["vdim"], 1.0), mat(W, r["heads"] * r["vdim"])
        else:
            H, d, e = m["heads"], m["dim"], m["vdim"]
            w[p + "q"], w[p + "k"], w[p + "v"], w[p + "g"] = mat(H * d, W, 2.0), mat(H * d, W, 2.0), mat(H * e, W), mat(H * e, W, 2.0)
            w[p + "i"], w[p + "i.b"] = mat(H, W, 3.0), vec(H, 0.0, 2.0)
            w[p + "f"], w[p + "f.b"] = mat(H, W, 3.0), vec(H, 6.0 if long_memory else 1.0, 2.0)
            w[p + "norm"], w[p + "o"] = vec(H * e, 1.0), mat(W, H * e)
        if L["mlp"]:
            q, f = f"l{i}.mlp.", L["mlp"]
            w[q + "router"] = mat(f["router"]["experts"], W, router_gain)
            for e in range(f["router"]["experts"]):
                ff = f["expert"]["ff"]
                w[f"{q}e{e}.gate"], w[f"{q}e{e}.up"], w[f"{q}e{e}.down"] = mat(ff, W, 3.0), mat(ff, W, 3.0), mat(W, ff, 2.0)
            if f.get("shared"):
                ff = f["shared"]["ff"]
                w[q + "shared.gate"], w[q + "shared.up"], w[q + "shared.down"] = mat(ff, W, 3.0), mat(ff, W, 3.0), mat(W, ff, 2.0)
    return w


def write_folder(path: Path, cfg: dict, weights: Dict[str, torch.Tensor]) -> Path:
    from safetensors.torch import save_file

    path.mkdir(parents=True, exist_ok=True)
    (path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in weights.items()}, str(path / "model.safetensors"))
    return path


def f32(weights: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    return {k: v.float() for k, v in weights.items()}
