"""Layered decoder: a model given as a list of layers, each with its own kind of token mixer (softmax attention with a
distance bias, lightning attention with a recurrent state, latent attention, ...) and an optional feed-forward (gated, or a
mixture of experts), optionally with a span of layers that runs several times (args.LayeredArgs; architectures "Fesenex",
"Taruvik", "Lotazen", "Viladra").  It plugs into the same places as `Transformer`: `from_folder`, `forward(input_ids, seqlens, cache)` over ragged
batches, `BufferCache` (per-layer rings and states, `make_cache`), `forward_logprobs` / `next_token_logits` for `generate()`.

On disk: config.json + model.safetensors with tensors `embed`, `l<i>.norm1|norm2` (and `norm1b|norm2b` with norms after the
sublayers; a layer norm's bias is the weight's name + `.b`), `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`, `head` (none when the head is
the embedding table), and for designs that have them `l<i>.canon1|canon2` (convolution taps) and `l<i>.dwa` (depth-average weights).
The residual stream is fp32; weights and activations are bf16 or fp32 (`dtype`), the latter in true
fp32 arithmetic.  All compute runs in libmb200_hybrid.so (include/mistral_b200_hybrid.h); CUDA only, no fallback.
"""
import json
import os
from pathlib import Path
from typing import Any, Dict, List, Optional, Tuple, Union

import torch
from torch import nn

from . import _abi, _abi_hybrid as _h
from .args import LayeredArgs
from .cache import BufferCache, CacheInputMetadata
from .transformer_layers import FEED_FORWARDS, MIXERS, MIXERS_BY_ARGS, BiasedAttention, LayeredBlock, LightningMixer, Norm


class LayeredTransformer(nn.Module):
    def __init__(self, args: LayeredArgs, softmax_fp32: bool = True):
        super().__init__()
        self.args = args
        self.vocab_size = args.vocab
        self.n_layers = self.n_local_layers = len(args.layers)
        self.runs = args.layer_runs()  # layer index of every layer run; each run has its own cache entry
        self.embed = nn.Parameter(torch.empty(args.vocab, args.width), requires_grad=False)
        blocks = []
        seen_vmix = False
        assert not (args.depth_average and args.loop is not None), "a depth average over looped layers is not built"
        for li, L in enumerate(args.layers):
            if type(L.mixer) in MIXERS_BY_ARGS:
                mixer = MIXERS_BY_ARGS[type(L.mixer)](args.width, L.mixer, args.norm_eps)
            elif L.type == "attention":
                mixer: nn.Module = BiasedAttention(args.width, L.mixer, args.norm_eps, first_vmix=L.mixer.v_mix and not seen_vmix)
                seen_vmix = seen_vmix or L.mixer.v_mix
            else:
                mixer = MIXERS[L.type](args.width, L.mixer, args.norm_eps)
            mlp = FEED_FORWARDS[type(L.mlp)](args.width, L.mlp) if L.mlp is not None else None
            blocks.append(LayeredBlock(args.width, args.norm_eps, mixer, mlp, norm=args.norm, post_norm=args.post_norm, parallel=args.parallel_block,
                                       pre_norm=args.pre_norm, canon_taps=args.canon_taps if args.canon else 0,
                                       depth_results=li + 2 if args.depth_average else 0))
        self.layers = nn.ModuleList(blocks)
        self.pos = nn.Parameter(torch.empty(args.max_positions, args.width), requires_grad=False) if args.learned_positions else None
        self.final_norm = Norm(args.width, args.norm_eps, args.norm)
        # a tied head is the embedding table itself (without the embedding's scale): no parameter of its own
        self.head = nn.Parameter(torch.empty(args.vocab, args.width), requires_grad=False) if not args.tied_head else None
        self.last_argmax: Optional[torch.Tensor] = None

    # ------------------------------------------------------------------ properties
    @property
    def dtype(self) -> torch.dtype:
        return self.embed.dtype

    @property
    def device(self) -> torch.device:
        return self.embed.device

    def make_cache(self, max_batch_size: int, max_seq_len: int) -> BufferCache:
        """The cache of this model, one entry per layer RUN (a layer that runs in several passes keeps each pass's keys apart): a
        whole-sequence ring per attention layer, an fp32 state per lightning layer."""
        specs = [self.layers[i].mix.cache_spec() for i in self.runs]
        for sp, i in zip(specs, self.runs):
            sp.conv_shape = self.layers[i].conv_shape()
        cache = BufferCache(len(specs), max_batch_size, max_seq_len, 0, 0, None, layer_specs=specs)
        cache.to(device=self.device, dtype=self.dtype)
        cache.reset()
        return cache

    # ------------------------------------------------------------------ forward
    def _check_runnable(self) -> None:
        if self.device.type != "cuda":
            raise _abi.Mb200Error(f"layered decoders run on CUDA only (got {self.device}); no fallback exists")
        _h.dt_of(self.dtype)

    @torch.inference_mode()
    def hidden(self, input_ids: torch.Tensor, seqlens: List[int], cache: Optional[BufferCache]) -> torch.Tensor:
        """The fp32 residual stream [T, width] after the last layer.  Advances the cache.  Without a cache every sequence
        is taken as whole, from position 0."""
        self._check_runnable()
        (num_toks,) = input_ids.shape
        assert sum(seqlens) == num_toks, (sum(seqlens), num_toks)
        if cache is None:
            cache = self.make_cache(len(seqlens), max(seqlens))
        self._check_room(cache, seqlens)
        x = self._run_layers(input_ids, cache.get_input_metadata(seqlens), cache)
        cache.update_seqlens(seqlens)
        return x

    def _check_room(self, cache: BufferCache, seqlens: List[int]) -> None:
        past = cache._kv_seqlens_host or [0] * len(seqlens)
        longest = max(p + s for p, s in zip(past, seqlens))
        assert longest <= cache.max_seq_len, "sequence longer than the cache"
        assert self.pos is None or longest <= self.pos.shape[0], f"sequence of {longest} tokens, {self.pos.shape[0]} learned positions"

    def _run_layers(self, input_ids: torch.Tensor, md: List[CacheInputMetadata], cache: BufferCache) -> torch.Tensor:
        if self.pos is not None:
            x = _h.embed_pos(input_ids, md[0].positions, self.embed, self.pos, self.args.embedding_scale)
        else:
            x = _h.embed_scale(input_ids, self.embed, self.args.embedding_scale)
        ctx: Dict[str, torch.Tensor] = {}
        if self.args.depth_average:
            return self._run_layers_averaged(x, md, cache, ctx)
        lp = self.args.loop
        first_pass = True
        for r, i in enumerate(self.runs):
            if lp is not None and i == lp.start:
                if not first_pass:  # every pass but the first starts from the stream plus the embedding output
                    _h.embed_add(input_ids, self.embed, self.args.embedding_scale, x)
                first_pass = False
            self.layers[i](x, cache.get_view(r, md[r]), ctx)
            if self._tap is not None:
                self._tap(r, x)
        return x

    def _run_layers_averaged(self, x0: torch.Tensor, md: List[CacheInputMetadata], cache: BufferCache, ctx: Dict[str, torch.Tensor]) -> torch.Tensor:
        """Layers whose input is a weighted average over depth: stack[0] is the embedding output, stack[i + 1] the result of layer i.
        Layer i works in place on stack[i + 1], which the layer before left holding ITS average (layer 0: a copy of the embedding
        output); the kernel of the layer's last norm then writes the average over stack[0 .. i + 1] into stack[i + 2], the next layer's
        stream.  The last slot is what the final norm reads."""
        n = len(self.runs)
        stack = torch.empty(n + 2, *x0.shape, dtype=torch.float32, device=x0.device)
        stack[0].copy_(x0)
        stack[1].copy_(x0)
        for r, i in enumerate(self.runs):
            self.layers[i](stack[r + 1], cache.get_view(r, md[r]), ctx, mix=(stack, stack[r + 2]))
            if self._tap is not None:
                self._tap(r, stack[r + 2])
        return stack[n + 1]

    _tap = None  # debugging hook: called with (layer run, residual stream) after every layer run

    def logits_of(self, x32: torch.Tensor) -> torch.Tensor:
        """Final norm + head, fp32 [rows, vocab]."""
        return _h.linear(self.final_norm(x32), self.head if self.head is not None else self.embed, epi=_h.EPI_F32, limit=self.args.logit_softcap)

    def _graph_decode_ok(self, seqlens: List[int], cache: Optional[BufferCache]) -> bool:
        if cache is None or self._tap is not None or os.environ.get("MB200_DECODE_GRAPH", "1") == "0":
            return False
        host = cache._kv_seqlens_host
        return host is not None and len(host) == len(seqlens) and min(host) > 0 and all(s == 1 for s in seqlens)

    @torch.inference_mode()
    def decode_static(self, tokens: torch.Tensor, cache: BufferCache) -> torch.Tensor:
        """One decode step for every live sequence of `cache`, replayed from a CUDA graph (the launch-bound inner loop of
        generation; same scheme as `Transformer.decode_static` for batches).  The step's metadata block is built on the host and
        copied into a static device buffer before the replay; the kernels' grids depend on the batch size only.  Returns the
        STATIC fp32 logits [B, vocab] (overwritten by the next step).  The first call per (cache, batch) runs eagerly, the second
        captures; `BufferCache.retire` drops the graphs of the old batch."""
        self._check_runnable()
        B = tokens.shape[0]
        seqlens = [1] * B
        self._check_room(cache, seqlens)
        st = cache.__dict__.setdefault("_mb200_decode_states", {}).setdefault((id(self), "layered", B), {})
        host, layout = cache.build_metadata_host(seqlens)
        if "meta" not in st:
            st.update({"meta": torch.zeros(len(host), dtype=torch.int32, device=self.device), "graph": None, "warmed": False, "logits": None,
                       "tokens": torch.zeros(B, dtype=torch.long, device=self.device)})
        st["meta"].copy_(torch.from_numpy(host))      # pageable source: staged by the runtime before the call returns
        st["tokens"].copy_(tokens, non_blocking=True)
        md = cache.metadata_from_block(st["meta"], layout, seqlens)

        def run() -> None:
            st["logits"] = self.logits_of(self._run_layers(st["tokens"], md, cache))

        if st["graph"] is None and not st["warmed"]:
            run()
            st["warmed"] = True
        elif st["graph"] is None:
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                run()
            st["graph"] = g
            g.replay()
        else:
            st["graph"].replay()
        cache.update_seqlens(seqlens)
        return st["logits"]

    @torch.inference_mode()
    def forward(self, input_ids: torch.Tensor, seqlens: List[int], cache: Optional[BufferCache] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        """fp32 logits [T, vocab] of a ragged batch (or of the flattened token places `rows` only)."""
        self.last_argmax = None
        if self._graph_decode_ok(seqlens, cache):
            out = self.decode_static(input_ids, cache)
            return out.clone() if rows is None else out.index_select(0, rows)
        x = self.hidden(input_ids, seqlens, cache)
        return self.logits_of(x if rows is None else x.index_select(0, rows))

    # ------------------------------------------------------------------ generate() support
    def last_argmax_valid_for(self, logits: torch.Tensor) -> bool:
        return False

    @torch.inference_mode()
    def next_token_logits(self, tokens: torch.Tensor, cache: BufferCache) -> torch.Tensor:
        """fp32 logits [B, vocab] of one decode step; on the graph path the step's static buffer (valid until the next step)."""
        tokens = tokens.reshape(-1)
        if self._graph_decode_ok([1] * tokens.numel(), cache):
            return self.decode_static(tokens, cache)
        return self.forward(tokens, [1] * tokens.numel(), cache)

    @torch.inference_mode()
    def forward_logprobs(self, input_ids: torch.Tensor, seqlens: List[int], cache: Optional[BufferCache],
                         targets: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
        """One prompt chunk for generate(): (log-probability of targets[t] at every place with targets[t] >= 0, logits of each
        sequence's last token)."""
        logits = self.forward(input_ids, seqlens, cache)
        lp = _abi.logprob_gather(logits, targets)
        last_idx = torch.tensor(seqlens, device=input_ids.device).cumsum(0) - 1
        return lp, logits.index_select(0, last_idx)

    # ------------------------------------------------------------------ weights
    def _assign(self, k: str, v: torch.Tensor) -> None:
        def put(dst: torch.Tensor) -> None:
            assert dst.shape == v.shape, f"{k}: shape {tuple(v.shape)} != expected {tuple(dst.shape)}"
            dst.copy_(v)

        if k == "embed":
            return put(self.embed)
        if k == "final.norm":
            return self.final_norm.load_weight(v)
        if k == "pos" and self.pos is not None:
            return put(self.pos)
        if k == "final.norm.b" and self.final_norm.bias is not None:
            return put(self.final_norm.bias)
        if k == "head" and self.head is not None:
            return put(self.head)
        lid, rest = k.split(".", 1)
        assert lid[0] == "l" and lid[1:].isdigit() and int(lid[1:]) < self.n_layers, f"Unexpected key {k}"
        blk: LayeredBlock = self.layers[int(lid[1:])]  # type: ignore[assignment]
        base = rest[:-2] if rest.endswith(".b") else rest
        if base in ("norm1", "norm2", "norm1b", "norm2b") and getattr(blk, base) is not None:
            nrm: Norm = getattr(blk, base)
            if base == rest:
                return nrm.load_weight(v)
            if nrm.bias is not None:
                return put(nrm.bias)
        if rest in ("canon1", "canon2") and getattr(blk, rest) is not None:
            return put(getattr(blk, rest).weight)
        if rest == "dwa" and blk.dwa is not None:
            return put(blk.dwa)
        part, name = rest.split(".", 1) if "." in rest else (rest, "")
        if part == "mix" and hasattr(blk.mix, "prepare"):
            blk.mix.prepare(name, tuple(v.shape))
        if part == "mlp" and blk.mlp is not None and blk.mlp.assign(name, put):
            return None
        m = blk.mix
        if part == "mix" and hasattr(m, "assign") and m.assign(name, put):
            return None
        if part == "mix" and isinstance(m, BiasedAttention):
            spans = {"q": (0, m.nq), "k": (m.nq, m.nq + m.nk), "v": (m.nq + m.nk, m.nq + m.nk + m.nv)}
            if name in spans:
                return put(m.wqkv[spans[name][0]: spans[name][1]])
            if name.endswith(".b") and name[:-2] in spans:
                return put(m.bqkv[spans[name[:-2]][0]: spans[name[:-2]][1]])
            if name == "rel":  # the table's row count comes with the checkpoint
                m.rel = nn.Parameter(torch.empty(v.shape, dtype=m.rel.dtype, device=m.rel.device), requires_grad=False)
                m._bias_tab = None
            direct = {"q.norm": "q_norm", "k.norm": "k_norm", "rel": "rel", "vmix": "vmix", "o": "wo"}
            if name in direct:
                return put(getattr(m, direct[name]))
        if part == "mix" and isinstance(m, LightningMixer):
            o = [0, m.nqk, 2 * m.nqk, 2 * m.nqk + m.nv, 2 * m.nqk + 2 * m.nv]
            idx = {"q": 0, "k": 1, "v": 2, "g": 3}
            if name in idx:
                return put(m.wqkvg[o[idx[name]]: o[idx[name] + 1]])
            if name == "norm":
                return put(m.norm)
            if name == "o":
                return put(m.wo)
        raise ValueError(f"Unexpected key {k}")

    def checkpoint_keys(self) -> List[str]:
        def norm_keys(name: str, nrm: Optional[Norm]) -> List[str]:
            return [] if nrm is None else [name] + ([name + ".b"] if nrm.bias is not None else [])

        keys = ["embed"] + (["head"] if self.head is not None else []) + norm_keys("final.norm", self.final_norm) + (["pos"] if self.pos is not None else [])
        for i, blk in enumerate(self.layers):
            p = f"l{i}."
            for n in ("norm1", "norm1b", "norm2", "norm2b"):
                keys += norm_keys(p + n, getattr(blk, n))
            if isinstance(blk.mix, BiasedAttention):
                keys += [p + "mix." + n for n in ("q", "q.b", "k", "k.b", "v", "v.b", "q.norm", "k.norm", "rel", "vmix", "o")]
            elif isinstance(blk.mix, LightningMixer):
                keys += [p + "mix." + n for n in ("q", "k", "v", "g", "norm", "o")]
            else:
                keys += [p + "mix." + n for n in blk.mix.checkpoint_names()]
            if blk.mlp is not None:
                keys += [p + "mlp." + n for n in blk.mlp.checkpoint_names()]
            keys += [p + n for n in ("canon1", "canon2") if getattr(blk, n) is not None] + ([p + "dwa"] if blk.dwa is not None else [])
        return keys

    def load_state_dict(self, state_dict: Any, strict: bool = True, assign: bool = False) -> None:  # type: ignore[override]
        """Takes checkpoint-keyed tensors and packs them."""
        del assign
        with torch.no_grad():
            for k, v in state_dict.items():
                self._assign(k, v)
        if strict:
            missing = set(self.checkpoint_keys()) - set(state_dict.keys())
            assert not missing, f"missing keys: {sorted(missing)[:8]}"

    @staticmethod
    def empty(args: LayeredArgs, device: Union[torch.device, str] = "cuda", dtype: torch.dtype = torch.bfloat16, **kwargs: Any) -> "LayeredTransformer":
        dev = torch.device(device)
        if dev.type == "cuda" and dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        with torch.device("meta"):
            m = LayeredTransformer(args, **kwargs)
        m = m.to(dtype=dtype).to_empty(device=dev)
        for blk, L in zip(m.layers, args.layers):  # non-persistent buffers do not survive to_empty
            if isinstance(blk.mix, LightningMixer):
                blk.mix.decay = torch.tensor(L.mixer.decay, dtype=torch.float32, device=dev)
        return m

    @staticmethod
    def from_folder(folder: Union[Path, str], max_batch_size: int = 1, num_pipeline_ranks: int = 1, device: Union[torch.device, str] = "cuda",
                    dtype: Optional[torch.dtype] = None, softmax_fp32: bool = True, **kwargs: Any) -> "LayeredTransformer":
        assert num_pipeline_ranks == 1 and not kwargs, "layered decoders run on one GPU"
        import safetensors

        with open(Path(folder) / "config.json", "r") as f:
            args = LayeredArgs.from_dict(json.load(f))
        args.max_batch_size = max_batch_size
        with safetensors.safe_open(str(Path(folder) / "model.safetensors"), framework="pt", device="cpu") as f:
            keys = list(f.keys())
            model = LayeredTransformer.empty(args, device, dtype or f.get_tensor("final.norm").dtype, softmax_fp32=softmax_fp32)
            with torch.no_grad():
                for k in keys:
                    model._assign(k, f.get_tensor(k))
            missing = set(model.checkpoint_keys()) - set(keys)
            assert not missing, f"missing keys: {sorted(missing)[:8]}"
        return model.eval()
