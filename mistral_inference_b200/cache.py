"""Rotating KV cache (API mirror of mistral_inference/cache.py:140-263).

Same storage contract as the reference -- per layer `cache_k[i]`, `cache_v[i]` of shape
[max_batch, W_i, n_kv_heads, head_dim], token at absolute position p of sequence b in slot p % W_i
(cache.py:235), `kv_seqlens[b]` = tokens seen -- but the per-forward metadata is different in kind:
the reference builds xformers mask objects and bool/index tensors per LAYER with Python list
comprehensions and `.tolist()` syncs (cache.py:197-263); here one small int32 block is built on the host
with numpy (sequence lengths are host-known), uploaded with ONE copy per forward and shared by all
layers with the same window.  The kernels derive masks from (positions, seqpos, W) arithmetically.

Beyond the reference: a layer may be described by a `LayerCacheSpec` -- a ring with its own number of key/value heads and
separate key and value sizes, or a fixed-size fp32 recurrent STATE per sequence (linear-attention layers) -- and the sequences
of a batch are addressed through physical row blocks (`slots`), so that a sequence that ends can be retired from a running
batch while the others keep their rows, and rows are handed out again by the next batch.  A state is never cleared on the
host: the kernels start from zero when a sequence has no tokens yet, so a reused row cannot leak.
"""
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple, Union

import numpy as np
import torch

SlidingWindow = Union[None, int, List[Optional[int]]]


def get_cache_sizes(n_layers: int, max_seq_len: int, sliding_window: SlidingWindow) -> List[int]:
    """cache.py:13-24."""
    if sliding_window is None:
        return n_layers * [max_seq_len]
    elif isinstance(sliding_window, int):
        return n_layers * [sliding_window]
    else:
        assert isinstance(sliding_window, list), f"Expected list, got {type(sliding_window)}"
        assert n_layers % len(sliding_window) == 0, f"Expected n_layers % len(sliding_window) == 0, got {n_layers} % {len(sliding_window)}"
        num_repeats = n_layers // len(sliding_window)
        return num_repeats * [w if w is not None else max_seq_len for w in sliding_window]


@dataclass
class LayerCacheSpec:
    """What one layer keeps per sequence.  kind "ring": keys [W, n_kv_heads, k_dim] and values [W, n_kv_heads, v_dim] in the model
    dtype (window None = the whole sequence).  kind "state": one fp32 tensor of `state_shape`, carried from token to token.  A ring
    layer with a non-empty `state_shape` keeps both (a layer whose mixer is an attention beside a recurrence).  `conv_shape`: beside
    either, an fp32 tensor with the last inputs of the layer's short convolutions over time (a layer whose sublayers read their
    input through a causal convolution)."""
    kind: str = "ring"
    n_kv_heads: int = 0
    k_dim: int = 0
    v_dim: int = 0
    window: Optional[int] = None
    state_shape: Tuple[int, ...] = ()
    conv_shape: Tuple[int, ...] = ()


@dataclass
class CacheInputMetadata:
    """What one layer's kernels need for this forward (device int32 tensors are views into one upload)."""
    positions: torch.Tensor   # [T] absolute positions (rope + masks)
    cache_rows: torch.Tensor  # [T] flat ring row slot + b*W, or -1 when the token is not cached (cache.py:226,235)
    kv_len: torch.Tensor      # [B] decode only: valid ring slots once this token is written = min(seqpos+1, W)
    q_start: torch.Tensor     # [B+1] prefix sums of seqlens
    seqpos: torch.Tensor      # [B] tokens already cached before this forward
    prefill: bool             # first or subsequent prefill (cache.py:236-237); False = one-token decode
    first_prefill: bool       # nothing cached yet for any sequence (cache.py:236,239)
    seqlens: List[int]
    max_seqlen: int
    window: int               # W of this layer
    slots: Optional[torch.Tensor] = None  # [B] physical row block of each sequence (kernels that take it; else slot b = b)


class CacheView:
    """cache.py:70-137: one layer's ring plus the metadata of this forward."""

    def __init__(self, cache_k: Optional[torch.Tensor], cache_v: Optional[torch.Tensor], metadata: CacheInputMetadata, kv_seqlens_host: List[int],
                 state: Optional[torch.Tensor] = None, conv: Optional[torch.Tensor] = None):
        self.conv = conv    # fp32 [rows, *conv_shape]: the last inputs of the layer's convolutions over time
        self.cache_k = cache_k
        self.cache_v = cache_v
        self.state = state  # fp32 [rows, *state_shape] of a recurrent layer
        self.metadata = metadata
        self.kv_seqlens_host = kv_seqlens_host

    @property
    def max_seq_len(self) -> int:
        return self.cache_k.shape[1]

    @property
    def key(self) -> torch.Tensor:
        return self.cache_k[: len(self.kv_seqlens_host)]

    @property
    def value(self) -> torch.Tensor:
        return self.cache_v[: len(self.kv_seqlens_host)]

    @property
    def prefill(self) -> bool:
        return self.metadata.prefill


class BufferCache:
    """Rectangular rotating cache; constructor and methods as cache.py:140-195."""

    def __init__(self, n_layers: int, max_batch_size: int, max_seq_len: int, n_kv_heads: int, head_dim: int,
                 sliding_window: SlidingWindow = None, layer_specs: Optional[List[LayerCacheSpec]] = None):
        self.max_seq_len = max_seq_len
        self.layer_specs = layer_specs
        self.cache_state: Dict[int, torch.Tensor] = {}
        self.cache_conv: Dict[int, torch.Tensor] = {}
        self._rows: Optional[List[int]] = None  # physical row block of each live sequence, in batch order
        self.n_kv_heads = n_kv_heads
        self.head_dim = head_dim
        self.n_layers = n_layers
        self.max_batch_size = max_batch_size
        if layer_specs is None:
            self.cache_sizes: List[int] = get_cache_sizes(n_layers, max_seq_len, sliding_window)
        else:  # a state layer has no ring; it shares the metadata of a whole-sequence ring
            assert len(layer_specs) == n_layers
            self.cache_sizes = [min(sp.window, max_seq_len) if (sp.kind == "ring" and sp.window) else max_seq_len for sp in layer_specs]
        assert len(self.cache_sizes) == n_layers, f"Expected {n_layers} cache sizes, got {len(self.cache_sizes)}"
        self.cache_k: Dict[int, torch.Tensor] = {}
        self.cache_v: Dict[int, torch.Tensor] = {}
        for i, cache_size in enumerate(self.cache_sizes):
            sp = layer_specs[i] if layer_specs is not None else None
            if sp is None:
                self.cache_k[i] = torch.empty((max_batch_size, cache_size, n_kv_heads, head_dim))
                self.cache_v[i] = torch.empty((max_batch_size, cache_size, n_kv_heads, head_dim))
            elif sp.kind == "ring":
                self.cache_k[i] = torch.empty((max_batch_size, cache_size, sp.n_kv_heads, sp.k_dim))
                self.cache_v[i] = torch.empty((max_batch_size, cache_size, sp.n_kv_heads, sp.v_dim))
                if sp.state_shape:
                    self.cache_state[i] = torch.empty((max_batch_size, *sp.state_shape), dtype=torch.float32)
            else:
                assert sp.kind == "state", sp.kind
                self.cache_state[i] = torch.empty((max_batch_size, *sp.state_shape), dtype=torch.float32)
            if sp is not None and sp.conv_shape:
                self.cache_conv[i] = torch.empty((max_batch_size, *sp.conv_shape), dtype=torch.float32)
        # host copy of the valid length per batch element (the reference keeps it on the device and syncs, cache.py:217)
        self._kv_seqlens_host: Optional[List[int]] = None

    # -- reference API --------------------------------------------------------------------------
    def get_view(self, layer_id: int, metadata: CacheInputMetadata) -> CacheView:
        assert self._kv_seqlens_host is not None
        return CacheView(self.cache_k.get(layer_id), self.cache_v.get(layer_id), metadata, self._kv_seqlens_host,
                         state=self.cache_state.get(layer_id), conv=self.cache_conv.get(layer_id))

    def reset(self) -> None:
        self._kv_seqlens_host = None
        self._rows = None

    def init_kvseqlens(self, batch_size: int) -> None:
        assert batch_size <= self.max_batch_size, f"batch of {batch_size} in a cache of {self.max_batch_size} rows"
        self._kv_seqlens_host = [0] * batch_size
        self._rows = list(range(batch_size))

    @property
    def rows(self) -> List[int]:
        """Physical row block of each live sequence, in batch order."""
        if self._rows is None:
            self._rows = list(range(len(self._kv_seqlens_host or [])))
        return self._rows

    def retire(self, indices: List[int]) -> None:
        """Sequences `indices` (places in the current batch order) have ended: what they hold is given back, the others keep
        their rows and their order.  The next `reset()` + batch hands every row out again."""
        assert self._kv_seqlens_host is not None
        assert self.layer_specs is not None, "retiring from a running batch needs kernels that address rows by slot (layered models)"
        gone = set(indices)
        assert all(0 <= i < len(self._kv_seqlens_host) for i in gone), indices
        rows = self.rows
        self._rows = [r for i, r in enumerate(rows) if i not in gone]
        self._kv_seqlens_host = [n for i, n in enumerate(self._kv_seqlens_host) if i not in gone]
        self.__dict__.pop("_mb200_decode_states", None)  # captured decode graphs are per batch size and row set

    @property
    def kv_seqlens(self) -> Optional[torch.Tensor]:
        if self._kv_seqlens_host is None:
            return None
        return torch.tensor(self._kv_seqlens_host, device=self.device, dtype=torch.long)

    @property
    def device(self) -> torch.device:
        return next(iter(self.cache_k.values() if self.cache_k else self.cache_state.values())).device

    def to(self, device: torch.device, dtype: torch.dtype) -> "BufferCache":
        for i in self.cache_k:
            self.cache_k[i] = self.cache_k[i].to(device=device, dtype=dtype)
            self.cache_v[i] = self.cache_v[i].to(device=device, dtype=dtype)
        for i in self.cache_state:  # recurrent state stays fp32
            self.cache_state[i] = self.cache_state[i].to(device=device)
        for i in self.cache_conv:
            self.cache_conv[i] = self.cache_conv[i].to(device=device)
        return self

    def update_seqlens(self, seqlens: List[int]) -> None:
        assert self._kv_seqlens_host is not None
        self._kv_seqlens_host = [a + b for a, b in zip(self._kv_seqlens_host, seqlens)]

    # -- metadata ---------------------------------------------------------------------------------
    def get_input_metadata(self, seqlens: List[int]) -> List[CacheInputMetadata]:
        """One CacheInputMetadata per layer (shared objects for layers with equal W)."""
        host, layout = self.build_metadata_host(seqlens)
        dev = torch.from_numpy(host).to(self.device, non_blocking=False)
        return self.metadata_from_block(dev, layout, seqlens)

    def build_metadata_host(self, seqlens: List[int]) -> Tuple[np.ndarray, dict]:
        """Packs [positions | q_start | seqpos | (cache_rows, kv_len) per distinct W | slots] into one int32 array."""
        if self._kv_seqlens_host is None:
            self.init_kvseqlens(len(seqlens))
        assert self._kv_seqlens_host is not None
        assert len(seqlens) == len(self._kv_seqlens_host), (
            f"Batch size is {len(self._kv_seqlens_host)}, got {len(seqlens)}, did you forget to reset cache?")
        assert len(seqlens) > 0, seqlens
        seqpos = np.asarray(self._kv_seqlens_host, dtype=np.int64)
        sl = np.asarray(seqlens, dtype=np.int64)
        B, T = len(seqlens), int(sl.sum())
        first_prefill = bool(seqpos[0] == 0)
        subsequent_prefill = bool((sl > 1).any())
        if first_prefill:
            assert (seqpos == 0).all(), seqpos.tolist()  # cache.py:239
        q_start = np.zeros(B + 1, dtype=np.int64)
        np.cumsum(sl, out=q_start[1:])
        batch_idx = np.repeat(np.arange(B, dtype=np.int64), sl)
        local = np.arange(T, dtype=np.int64) - q_start[batch_idx]
        positions = seqpos[batch_idx] + local
        distinct = sorted(set(self.cache_sizes))
        slot = np.asarray(self.rows, dtype=np.int64)
        with_slots = self.layer_specs is not None  # kernels of layered models take the row block of each sequence
        assert with_slots or self.rows == list(range(B)), "this model's kernels address sequence b at row block b"
        total = T + (B + 1) + B + len(distinct) * (T + B) + (B if with_slots else 0)
        host = np.empty(total, dtype=np.int32)
        layout = {"T": T, "B": B, "prefill": first_prefill or subsequent_prefill, "first_prefill": first_prefill, "max_seqlen": int(sl.max()), "windows": distinct}
        o = 0
        host[o:o + T] = positions; o += T
        host[o:o + B + 1] = q_start; o += B + 1
        host[o:o + B] = seqpos; o += B
        for W in distinct:
            cached = local >= (sl[batch_idx] - W)  # only the last W tokens of each chunk (cache.py:226)
            rows = np.where(cached, positions % W + slot[batch_idx] * W, -1)
            host[o:o + T] = rows; o += T
            host[o:o + B] = np.minimum(seqpos + np.minimum(sl, W), W); o += B
        if with_slots:
            host[o:o + B] = slot; o += B
        layout["slots"] = with_slots
        return host, layout

    def metadata_from_block(self, dev: torch.Tensor, layout: dict, seqlens: List[int]) -> List[CacheInputMetadata]:
        T, B = layout["T"], layout["B"]
        o = 0
        positions = dev[o:o + T]; o += T
        q_start = dev[o:o + B + 1]; o += B + 1
        seqpos = dev[o:o + B]; o += B
        per_w: Dict[int, CacheInputMetadata] = {}
        so = o + len(layout["windows"]) * (T + B)
        slots = dev[so:so + B] if layout.get("slots") else None
        for W in layout["windows"]:
            rows = dev[o:o + T]; o += T
            kv_len = dev[o:o + B]; o += B
            per_w[W] = CacheInputMetadata(slots=slots, positions=positions, cache_rows=rows, kv_len=kv_len, q_start=q_start, seqpos=seqpos,
                                          prefill=layout["prefill"], first_prefill=layout["first_prefill"], seqlens=list(seqlens), max_seqlen=layout["max_seqlen"], window=W)
        return [per_w[W] for W in self.cache_sizes]
