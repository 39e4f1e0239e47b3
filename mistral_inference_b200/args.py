"""`params.json` schema (mirror of mistral_inference/args.py:29-59 and moe.py:10-13).

`simple_parsing` is not a dependency here: `from_dict` is a few lines (the reference only uses
`Serializable.from_dict`, transformer.py:306-307).
"""
from dataclasses import dataclass, fields
from typing import List, Optional, Union


@dataclass
class MoeArgs:
    num_experts: int
    num_experts_per_tok: int

    @classmethod
    def from_dict(cls, d: dict) -> "MoeArgs":
        return cls(**{f.name: d[f.name] for f in fields(cls) if f.name in d})


@dataclass
class LoraArgs:
    rank: int
    scaling: float

    @classmethod
    def from_dict(cls, d: dict) -> "LoraArgs":
        return cls(**{f.name: d[f.name] for f in fields(cls) if f.name in d})


@dataclass
class TransformerArgs:
    dim: int
    n_layers: int
    head_dim: int
    hidden_dim: int
    n_heads: int
    n_kv_heads: int
    norm_eps: float
    vocab_size: int

    max_batch_size: int = 0

    # For rotary embeddings. If not set, 1e6 is used (transformer.py:115).
    rope_theta: Optional[float] = None
    # If this is set, MoE layers replace the dense FeedForward.
    moe: Optional[MoeArgs] = None
    lora: Optional[LoraArgs] = None
    sliding_window: Union[None, int, List[Optional[int]]] = None
    _sliding_window: Union[None, int, List[Optional[int]]] = None
    model_type: str = "transformer"

    vision_encoder: Optional[dict] = None

    def __post_init__(self) -> None:
        assert self.model_type == "transformer", self.model_type
        assert self.sliding_window is None or self._sliding_window is None
        # same aliasing as args.py:58-59
        self.sliding_window = self.sliding_window if self.sliding_window is not None else self._sliding_window
        if self.vision_encoder is not None:
            raise NotImplementedError("vision_encoder (Pixtral) is outside the accelerated hot path (SURVEY.md 2, row 10)")
        if isinstance(self.moe, dict):
            self.moe = MoeArgs.from_dict(self.moe)
        if isinstance(self.lora, dict):
            self.lora = LoraArgs.from_dict(self.lora)

    @classmethod
    def from_dict(cls, d: dict) -> "TransformerArgs":
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in known})


# ----------------------------------------------------------------------------- layered decoders (config.json)
@dataclass
class BiasedAttentionArgs:
    """Softmax attention without rotation: per-head RMS norm of q and k, a query temperature that grows with the position,
    a learned additive bias by (bucketed) distance, optional mixing of the values with an earlier layer's."""
    heads: int
    kv_heads: int
    dim: int            # per-head query/key size
    vdim: int           # per-head value size
    scale: float        # multiplies q.k (not the bias)
    bias_max: float     # distance at which the logarithmic part of the bias buckets ends
    temp_coef: float = 0.0
    temp_every: int = 0  # 0: no temperature
    v_mix: bool = False

    @classmethod
    def from_dict(cls, d: dict) -> "BiasedAttentionArgs":
        qt = d.get("q_temp") or {}
        return cls(heads=int(d["heads"]), kv_heads=int(d["kv_heads"]), dim=int(d["dim"]), vdim=int(d["vdim"]), scale=float(d["scale"]),
                   bias_max=float(d["bias_max"]), temp_coef=float(qt.get("coef", 0.0)), temp_every=int(qt.get("every", 0)),
                   v_mix=bool(d.get("v_mix", False)))


@dataclass
class LightningArgs:
    """Linear attention with one fixed decay per head and an fp32 state [heads, dim, vdim] per sequence."""
    heads: int
    dim: int
    vdim: int
    decay: List[float]

    @classmethod
    def from_dict(cls, d: dict) -> "LightningArgs":
        a = cls(heads=int(d["heads"]), dim=int(d["dim"]), vdim=int(d["vdim"]), decay=[float(x) for x in d["decay"]])
        assert len(a.decay) == a.heads, "one decay per head"
        return a


@dataclass
class ClampedGluArgs:
    """Dense feed-forward y = g * sigmoid(alpha * g) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit)."""
    ff: int
    limit: float
    alpha: float = 1.702

    @classmethod
    def from_dict(cls, d: dict) -> "ClampedGluArgs":
        assert d.get("kind", "dense") == "dense", f"unknown feed-forward kind {d.get('kind')}"
        return cls(ff=int(d["ff"]), limit=float(d["limit"]))


@dataclass
class RotScalingArgs:
    """YaRN-style frequency scaling of a rotation (rope.scaled_frequencies)."""
    factor: float
    original: float
    fast: float
    slow: float


@dataclass
class LatentAttentionArgs:
    """Softmax attention whose queries, keys and values come from per-token latents: the cache keeps the key/value latent
    (kv_rank) and one rotated key part (rot_dim) shared by the heads.  Each head has `dim` unrotated and `rot_dim` rotated query/key
    entries and `vdim` value entries; a sigmoid gate per head on the output."""
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_base: float
    rot_dims: int
    rot_scaling: Optional[RotScalingArgs] = None

    @classmethod
    def from_dict(cls, d: dict) -> "LatentAttentionArgs":
        rot = d["rot"]
        sc = rot.get("scaling")
        a = cls(heads=int(d["heads"]), dim=int(d["dim"]), rot_dim=int(d["rot_dim"]), vdim=int(d["vdim"]), q_rank=int(d["q_rank"]),
                kv_rank=int(d["kv_rank"]), scale=float(d["scale"]), rot_base=float(rot["base"]), rot_dims=int(rot.get("dims", d["rot_dim"])),
                rot_scaling=RotScalingArgs(float(sc["factor"]), float(sc["original"]), float(sc["fast"]), float(sc["slow"])) if sc else None)
        assert a.rot_dims <= a.rot_dim and a.rot_dims % 2 == 0, "the rotation covers an even number of the rotated entries"
        return a


@dataclass
class MoeFfArgs:
    """Mixture of gated (SiLU) experts of size `ff`.  The router has experts + identity outputs; the last `identity` of them stand
    for experts whose output is their input.  Softmax scores; the choice adds a per-output correction and is limited to the best
    `keep` of `groups` groups of neighbouring outputs; the weights are the chosen outputs' plain scores."""
    ff: int
    experts: int
    top: int
    identity: int = 0
    groups: int = 1
    keep: int = 1

    @property
    def routed(self) -> int:
        return self.experts + self.identity

    @classmethod
    def from_dict(cls, d: dict) -> "MoeFfArgs":
        r = d["router"]
        g = r.get("groups") or {}
        a = cls(ff=int(d["expert"]["ff"]), experts=int(r["experts"]), top=int(r["top"]), identity=int(r.get("identity", 0)),
                groups=int(g.get("count", 1)), keep=int(g.get("keep", g.get("count", 1))))
        assert a.routed % a.groups == 0 and 1 <= a.keep <= a.groups, "router groups must be equal and keep <= count"
        assert a.top <= a.routed // a.groups * a.keep, "more experts per token than the kept groups hold"
        return a


@dataclass
class RotaryAttentionArgs:
    """Softmax attention with rotary positions on the first `rot_dims` entries of every query and key head (interleaved pairs
    (2i, 2i + 1), angle position * rot_base^(-2i / rot_dims) / rot_factor), optionally a unit RMS norm of every rotated head, grouped
    key/value heads with separate key and value sizes, and optionally a sliding window of `window` positions (the token itself
    included; None: the whole sequence)."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int] = None
    rot_base: float = 10000.0
    rot_dims: int = 0          # 0: no rotation
    rot_factor: float = 1.0    # linear scaling: every frequency divided by it
    unit_norm: bool = True

    @classmethod
    def from_dict(cls, d: dict) -> "RotaryAttentionArgs":
        rot = d.get("rot") or {}
        a = cls(heads=int(d["heads"]), kv_heads=int(d["kv_heads"]), dim=int(d["dim"]), vdim=int(d["vdim"]), scale=float(d["scale"]),
                window=int(d["mask"]["size"]) if d.get("mask") else None, rot_base=float(rot.get("base", 10000.0)),
                rot_dims=int(rot.get("dims", d["dim"])) if rot else 0, rot_factor=float((rot.get("scaling") or {}).get("factor", 1.0)))
        assert a.heads % a.kv_heads == 0, "query heads must be a multiple of key/value heads"
        assert a.rot_dims <= a.dim and a.rot_dims % 2 == 0, "the rotation covers an even number of a head's entries"
        assert a.window is None or a.window >= 1
        return a


@dataclass
class Hgrn2Args:
    """Linear attention whose per-channel forget gate f = lower + (1 - lower) sigmoid(.) also decides what is written:
    S <- diag(f) S + (1 - f) v^T, o = S^T q; fp32 state [heads, dim, vdim] per sequence."""
    heads: int
    dim: int
    vdim: int

    @classmethod
    def from_dict(cls, d: dict) -> "Hgrn2Args":
        return cls(heads=int(d["heads"]), dim=int(d["dim"]), vdim=int(d["vdim"]))


@dataclass
class SideBySideArgs:
    """Two mixers reading the same input, summed with fixed weights: left_scale * attention + right_scale * recurrence."""
    left: RotaryAttentionArgs
    right: Hgrn2Args
    left_scale: float
    right_scale: float

    @classmethod
    def from_dict(cls, d: dict) -> "SideBySideArgs":
        return cls(left=RotaryAttentionArgs.from_dict(d["left"]), right=Hgrn2Args.from_dict(d["right"]), left_scale=float(d["left_scale"]),
                   right_scale=float(d["right_scale"]))


@dataclass
class MlstmArgs:
    """Matrix memory with exponential input and forget gates (capped by gate_cap * tanh(. / gate_cap)) and a running maximum that
    keeps them in range; fp32 state per sequence: [heads, dim, vdim] memory, [heads, dim] normaliser, [heads] maximum."""
    heads: int
    dim: int
    vdim: int
    gate_cap: float

    @classmethod
    def from_dict(cls, d: dict) -> "MlstmArgs":
        return cls(heads=int(d["heads"]), dim=int(d["dim"]), vdim=int(d["vdim"]), gate_cap=float(d["gate_cap"]))


@dataclass
class ScaledInputMoeArgs:
    """Mixture of clamped gated experts (ClampedGluArgs form) with an fp32 sigmoid router: the `top` largest scores are chosen and
    each chosen expert runs on score * input (scores not renormalised); an optional shared expert runs for every token."""
    ff: int
    limit: float
    experts: int
    top: int
    shared: Optional[ClampedGluArgs] = None
    alpha: float = 1.702

    @classmethod
    def from_dict(cls, d: dict) -> "ScaledInputMoeArgs":
        r, sh = d["router"], d.get("shared")
        a = cls(ff=int(d["expert"]["ff"]), limit=float(d["expert"]["limit"]), experts=int(r["experts"]), top=int(r["top"]),
                shared=ClampedGluArgs(ff=int(sh["ff"]), limit=float(sh["limit"])) if sh else None)
        assert 1 <= a.top <= a.experts, "top must be between 1 and the number of experts"
        return a


@dataclass
class RetentionArgs:
    """Linear attention with one fixed decay per head and no normaliser: S <- decay_h S + k v^T, o = S^T q.  Queries and keys are
    rotated on the first `rot_dims` entries of each head, entry i paired with entry i + rot_dims / 2 (angle position *
    rot_base^(-2i / rot_dims)); the rotated key is scaled by dim^(-1/2).  fp32 state [heads, dim, vdim] per sequence."""
    heads: int
    dim: int
    vdim: int
    decay: List[float]
    rot_base: float = 10000.0
    rot_dims: int = 0

    @classmethod
    def from_dict(cls, d: dict) -> "RetentionArgs":
        rot = d.get("rot") or {}
        a = cls(heads=int(d["heads"]), dim=int(d["dim"]), vdim=int(d["vdim"]), decay=[float(x) for x in d["decay"]],
                rot_base=float(rot.get("base", 10000.0)), rot_dims=int(rot.get("dims", d["dim"])) if rot else 0)
        assert len(a.decay) == a.heads, "one decay per head"
        assert a.rot_dims <= a.dim and a.rot_dims % 2 == 0, "the rotation covers an even number of a head's entries"
        return a


@dataclass
class GlaArgs:
    """Gated linear attention: a decay per key channel, alpha = sigmoid(z)^(1 / tau) with z from a low-rank projection (its rank is
    the checkpoint's), S <- diag(alpha) S + k v^T, o = S^T (q dim^(-1/2)).  fp32 state [heads, dim, vdim] per sequence."""
    heads: int
    dim: int
    vdim: int
    tau: float

    @classmethod
    def from_dict(cls, d: dict) -> "GlaArgs":
        return cls(heads=int(d["heads"]), dim=int(d["dim"]), vdim=int(d["vdim"]), tau=float(d["tau"]))


@dataclass
class SigmoidAttentionArgs:
    """Attention without a softmax and without rotation: q and k are RMS-normed over their whole projections, a visible key weighs
    sigmoid(q.k * scale + a number per head), weights are not normalised; grouped key/value heads, optional sliding window of
    `window` positions (the token itself included), a sigmoid gate per head on the output; q, k, v and output projections have biases."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int] = None

    @classmethod
    def from_dict(cls, d: dict) -> "SigmoidAttentionArgs":
        a = cls(heads=int(d["heads"]), kv_heads=int(d["kv_heads"]), dim=int(d["dim"]), vdim=int(d["vdim"]), scale=float(d["scale"]),
                window=int(d["mask"]["size"]) if d.get("mask") else None)
        assert a.heads % a.kv_heads == 0, "query heads must be a multiple of key/value heads"
        assert a.window is None or a.window >= 1
        return a


@dataclass
class Relu2FfArgs:
    """Feed-forward without a gate: W_down max(W_up h, 0)^2."""
    ff: int


@dataclass
class Relu2MoeArgs:
    """Mixture of experts of the Relu2FfArgs form with an fp32 softmax router over all experts: the `top` largest scores are chosen,
    weighted by score * router_scale (not renormalised); an optional shared expert runs for every token."""
    ff: int
    experts: int
    top: int
    router_scale: float = 1.0
    shared: Optional[Relu2FfArgs] = None

    @classmethod
    def from_dict(cls, d: dict) -> "Relu2MoeArgs":
        r, sh = d["router"], d.get("shared")
        a = cls(ff=int(d["expert"]["ff"]), experts=int(r["experts"]), top=int(r["top"]), router_scale=float(r.get("scale", 1.0)),
                shared=Relu2FfArgs(ff=int(sh["ff"])) if sh else None)
        assert 1 <= a.top <= a.experts, "top must be between 1 and the number of experts"
        return a


MLP_ARGS = {"dense": ClampedGluArgs, "moe": MoeFfArgs}


@dataclass
class LayerArgs:
    type: str                                             # a key of MIXER_ARGS
    mixer: Union[BiasedAttentionArgs, LightningArgs, LatentAttentionArgs, SideBySideArgs, MlstmArgs, RetentionArgs, GlaArgs, SigmoidAttentionArgs]
    mlp: Union[None, ClampedGluArgs, MoeFfArgs, ScaledInputMoeArgs, Relu2MoeArgs]


MIXER_ARGS = {"attention": BiasedAttentionArgs, "lightning": LightningArgs, "latent_attention": LatentAttentionArgs,
              "parallel": SideBySideArgs, "mlstm": MlstmArgs, "mlstm_2": MlstmArgs}


@dataclass
class LoopArgs:
    """Layers start .. stop-1 run `times` times in a row with the same weights (each pass with a cache of its own); before every
    pass but the first the embedding output is added to the residual stream."""
    start: int
    stop: int
    times: int


# What a design fixes (not in config.json): the kind of norm, whether each sublayer's output is normed again before it is added
# to the residual stream, whether mixer and feed-forward of a layer read the same normed input (one norm per layer) and are added
# together, whether a learned position vector is added to the embedding, and which feed-forward a kind names (default: MLP_ARGS).
# "pre_norm": False -- the sublayers read the stream itself and norm1 / norm2 act on their OUTPUTS; "canon" -- what a sublayer reads
# is first replaced by itself plus a causal convolution over time (taps from config "canon"); "depth_average" -- what goes on to the
# next layer is a learned weighted average of the embedding output and every layer result so far; "tied_head" -- the logits use the
# embedding table.  DESIGN_MIXER_ARGS: which mixer a type names in a design (default: MIXER_ARGS).
DESIGNS = {
    "Fesenex": {"norm": "rms", "post_norm": False},
    "Taruvik": {"norm": "layer", "post_norm": True},
    "Lotazen": {"norm": "rms_scalar", "post_norm": False, "parallel_block": True, "learned_positions": True},
    "Viladra": {"norm": "rms", "post_norm": True, "pre_norm": False, "canon": True, "depth_average": True, "tied_head": True},
}
DESIGN_MLP_ARGS = {"Lotazen": {"moe": ScaledInputMoeArgs}, "Viladra": {"moe": Relu2MoeArgs}}
DESIGN_MIXER_ARGS = {"Viladra": {"attention": SigmoidAttentionArgs, "retention": RetentionArgs, "gla": GlaArgs}}


@dataclass
class LayeredArgs:
    """config.json of a layered decoder (an architecture of DESIGNS): a list of layers, each naming its mixer kind."""
    architecture: str
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: List[LayerArgs]
    max_batch_size: int = 0
    norm: str = "rms"            # "rms": weight only; "rms_scalar": one number as weight; "layer": mean removed, weight and bias
    post_norm: bool = False      # x <- x + norm_b(sublayer(norm(x))) instead of x <- x + sublayer(norm(x))
    loop: Optional[LoopArgs] = None
    parallel_block: bool = False     # h = norm1(x); x <- x + mixer(h) + ff(h): one norm per layer, both sublayers read it
    learned_positions: bool = False  # x = embed[token] + pos[position]; max_positions rows
    max_positions: int = 0
    logit_softcap: float = 0.0       # > 0: logits <- cap * tanh(logits / cap)
    pre_norm: bool = True            # False (with post_norm): x <- x + norm(sublayer(x)), norm1 / norm2 on the outputs only
    canon: bool = False              # sublayers read x + causal_conv(x); canon_taps taps
    canon_taps: int = 0
    depth_average: bool = False      # the next layer reads sum_j dwa[j] X_j over the embedding output and the layer results so far
    tied_head: bool = False          # logits = embed x (the table without its scale)

    def layer_runs(self) -> List[int]:
        """The layer index of every layer run, in order (a looped layer appears once per pass)."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        lp = self.loop
        return list(range(lp.start)) + list(range(lp.start, lp.stop)) * lp.times + list(range(lp.stop, n))

    @property
    def vocab_size(self) -> int:
        return self.vocab

    @classmethod
    def from_dict(cls, d: dict) -> "LayeredArgs":
        layers = []
        if d["architecture"] not in DESIGNS:
            raise ValueError(f"unknown architecture {d['architecture']!r} (known: {sorted(DESIGNS)})")
        mlp_args = {**MLP_ARGS, **DESIGN_MLP_ARGS.get(d["architecture"], {})}
        mixer_args = {**MIXER_ARGS, **DESIGN_MIXER_ARGS.get(d["architecture"], {})}
        design = dict(DESIGNS[d["architecture"]])
        if design.get("canon"):
            design["canon_taps"] = int(d["canon"]["taps"])
            assert design["canon_taps"] >= 1, "canon.taps >= 1"
        for L in d["layers"]:
            if L["type"] not in mixer_args:
                raise ValueError(f"unknown mixer type {L['type']!r}")
            mlp = None
            if L.get("mlp") is not None:
                # without "kind": the design's own feed-forward when it has exactly one, else the dense one
                own = DESIGN_MLP_ARGS.get(d["architecture"], {})
                kind = L["mlp"].get("kind", next(iter(own)) if len(own) == 1 else "dense")
                if kind not in mlp_args:
                    raise ValueError(f"unknown feed-forward kind {kind!r}")
                mlp = mlp_args[kind].from_dict(L["mlp"])
            layers.append(LayerArgs(type=L["type"], mixer=mixer_args[L["type"]].from_dict(L["mixer"]), mlp=mlp))
        loop = None
        if d.get("loop"):
            lp = d["loop"]
            loop = LoopArgs(int(lp["start"]), int(lp["stop"]), int(lp["times"]))
            assert 0 <= loop.start < loop.stop <= len(layers) and loop.times >= 1, "loop: 0 <= start < stop <= layers, times >= 1"
        return cls(architecture=d["architecture"], vocab=int(d["vocab"]), width=int(d["width"]),
                   embedding_scale=float((d.get("embedding") or {}).get("scale", 1.0)), norm_eps=float(d["norm"]["eps"]), layers=layers,
                   loop=loop, max_positions=int(d.get("max_positions", 0)), logit_softcap=float(d.get("logit_softcap") or 0.0),
                   **design)
