"""The Lotazen design on the GPU against the plain statement in tests/lotazen_oracle.py: every mechanism alone (learned positions,
one-number norm, soft cap, rotary window attention, gated linear recurrence, matrix memory, sigmoid router, experts with scaled
input dense and sparse), then whole models of several shapes through the cache: prompts against token-by-token decoding,
portions, ragged batches, reused rows, window edges, long memories, long decoding, and greedy generation through `generate()`.
fp32 runs are compared tightly, bf16 runs by an error norm per token."""
import math

import pytest
import torch

from tests import lotazen_oracle as O
from tests.lotazen_util import attn_cfg, f32, make_config, make_weights, mlstm_cfg, moe_cfg, side_cfg, write_folder

pytestmark = pytest.mark.gpu
DEV = "cuda"

SHAPES = {
    # sizes that are no multiple of 8 or 32, 4 query heads on 2 key/value heads, a window of 5, rotation over part of a head with
    # scaled frequencies, a layer without feed-forward, one without shared expert, full attention without frequency scaling
    "odd": dict(width=40, vocab=50, layers=[
        (side_cfg(), moe_cfg()),
        (mlstm_cfg(), None),
        (mlstm_cfg(1, 20, 6, 15.0, "mlstm_2"), moe_cfg(ff=9, experts=3, top=1, shared=None)),
        (side_cfg(left=attn_cfg(2, 2, 16, 24, 0.4, None, (50.0, 16, None)), right={"heads": 1, "dim": 40, "vdim": 36}, left_scale=1.0, right_scale=0.25),
         moe_cfg(ff=14, limit=0.5, experts=4, top=4, shared=(6, 0.3)))]),
    # head sizes of the tensor-core prompt kernel, a window that crosses its 64-key tiles, a matrix memory first, heads wider
    # than 64 keys and more value columns than one CTA holds
    "tc": dict(width=64, vocab=70, layers=[
        (mlstm_cfg(2, 72, 136, 10.0), moe_cfg(ff=32, experts=6, top=2, shared=(16, 2.0))),
        (side_cfg(left=attn_cfg(4, 2, 32, 32, 0.35, 70, (10000.0, 16, 2.0)), right={"heads": 2, "dim": 16, "vdim": 16}), moe_cfg(ff=32, experts=4, top=1)),
        (side_cfg(left=attn_cfg(2, 1, 64, 64, 0.2, 33, (500.0, 64, 4.0)), right={"heads": 1, "dim": 64, "vdim": 130}), None)]),
    # nothing is a multiple of 2, 4 or 8 where it need not be: width 30, odd head sizes (the last entry of a head has no partner to
    # rotate with), 3 query heads on 1 key/value head, 17 words
    "awkward": dict(width=30, vocab=17, layers=[
        (side_cfg(left=attn_cfg(3, 1, 7, 5, 0.5, 9, (10000.0, 6, 1.5)), right={"heads": 2, "dim": 5, "vdim": 9}), moe_cfg(ff=7, experts=3, top=2, shared=(5, 1.0))),
        (mlstm_cfg(2, 7, 3, 4.0), moe_cfg(ff=6, experts=2, top=1, shared=None))]),
    # everything 1: one head, one expert of which one is used, a window that shows only the token itself, rotation of one pair
    "one": dict(width=24, vocab=20, softcap=3.0, layers=[
        (side_cfg(left=attn_cfg(1, 1, 8, 8, 1.0, 1, (10.0, 2, 1.0)), right={"heads": 1, "dim": 4, "vdim": 4}, left_scale=1.0, right_scale=1.0),
         moe_cfg(ff=8, experts=1, top=1, shared=(8, 1.0))),
        (mlstm_cfg(1, 4, 4, 1.0), moe_cfg(ff=8, experts=2, top=2, shared=None))]),
}


def _model(tmp_path, name, dtype, seed=0, weights=None, **over):
    from mistral_inference_b200.registry import load_model

    long_memory = over.pop("long_memory", False)
    cfg = make_config(**{**SHAPES[name], **over}) if isinstance(name, str) else name
    w = weights if weights is not None else make_weights(cfg, seed, long_memory=long_memory)
    m = load_model(write_folder(tmp_path / "m", cfg, w), device=DEV, dtype=dtype)
    if dtype == torch.bfloat16:  # the oracle sees the rounded weights
        w = {k: v.to(torch.bfloat16) for k, v in w.items()}
    return m, cfg, f32(w)


def _tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def _close(got, ref, dtype, what="", tol=3e-4):
    got, ref = got.float().cpu(), ref.float().cpu()
    if dtype == torch.float32:
        torch.testing.assert_close(got, ref, rtol=tol, atol=tol, msg=lambda m: f"{what}: {m}")
    else:
        # per token: most are within bf16 rounding; a near tie of a router turns the other way for a few tokens in a hundred
        got, ref = got.reshape(-1, got.shape[-1]), ref.reshape(-1, ref.shape[-1])
        err = (got - ref).pow(2).mean(-1).sqrt() / ref.pow(2).mean(-1).sqrt().clamp_min(1e-6)
        assert err.median() < 0.04, f"{what}: median relative rms error {err.median():.4f}"
        assert int((err > 0.25).sum()) <= max(1, len(err) // 10), f"{what}: {int((err > 0.25).sum())} of {len(err)} tokens are far off ({err.max():.3f})"


def _run(m, pieces, cache=None, taps=None):
    """Feeds one sequence in `pieces` (lists of tokens) through one cache row; returns the logits of all tokens."""
    cache = cache or m.make_cache(1, sum(len(p) for p in pieces))
    m._tap = (lambda r, x: taps.setdefault(r, []).append(x.clone())) if taps is not None else None
    try:
        out = [m.forward(torch.tensor(p, device=DEV), [len(p)], cache) for p in pieces]
    finally:
        m._tap = None
    return torch.cat(out)


# ----------------------------------------------------------------------------- mechanisms alone
def test_positions_norm_and_soft_cap():
    from mistral_inference_b200 import _abi_hybrid as h
    from mistral_inference_b200.transformer_layers import Norm

    tab, pos = torch.randn(9, 44, device=DEV), torch.randn(30, 44, device=DEV)
    tok, p = torch.tensor([3, 8, 0, 3, 1], device=DEV), torch.tensor([0, 1, 29, 7, 7], dtype=torch.int32, device=DEV)
    _close(h.embed_pos(tok, p, tab, pos, 1.0), tab.cpu()[tok.cpu()] + pos.cpu()[p.cpu().long()], torch.float32, tol=1e-6)
    n = Norm(44, 1e-3, "rms_scalar").to(DEV)
    n.load_weight(torch.tensor(1.7))
    x = torch.randn(6, 44, device=DEV) * 5
    _close(n(x), O.scalar_rms_norm(x.cpu(), torch.tensor(1.7), 1e-3), torch.float32, tol=1e-5)
    with pytest.raises(AssertionError):
        n.load_weight(torch.ones(44))
    a, w = torch.randn(5, 32, device=DEV), torch.randn(21, 32, device=DEV) * 2
    z = a.cpu() @ w.cpu().T
    _close(h.linear(a, w, epi=h.EPI_F32, limit=2.5), 2.5 * torch.tanh(z / 2.5), torch.float32, tol=1e-4)
    _close(h.linear(a, w, epi=h.EPI_F32), z, torch.float32, tol=1e-4)
    r = torch.randn(5, 21, device=DEV)
    want = r.cpu() + 0.3 * z
    h.linear(a, w, epi=h.EPI_RESIDUAL_SCALED, residual=r, alpha=0.3)
    _close(r, want, torch.float32, tol=1e-4)


@pytest.mark.parametrize("E,top", [(5, 2), (12, 1), (3, 3), (40, 6)])
def test_sigmoid_router(E, top):
    from mistral_inference_b200 import _abi_hybrid as h

    g = torch.Generator().manual_seed(E)
    x, wr = torch.randn(40, 24, generator=g), torch.randn(E, 24, generator=g)
    dense, idx, wsel = h.moe_route(x.to(DEV), wr.to(DEV), None, 1, 1, top, score=1)
    for t in range(40):
        ri, rw = O.route(x[t], wr, top)
        assert sorted(idx[t].tolist()) == sorted(ri), (t, idx[t].tolist(), ri)
        got = dict(zip(idx[t].tolist(), wsel[t].tolist()))
        for i, s in zip(ri, rw):
            assert abs(got[i] - float(s)) < 1e-5 and abs(float(dense[t, i]) - float(s)) < 1e-5
        assert int((dense[t] != 0).sum()) == top


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 5, 16, 17, 150])
@pytest.mark.parametrize("f", [moe_cfg(), moe_cfg(ff=32, limit=0.3, experts=4, top=1, shared=None), moe_cfg(ff=16, experts=3, top=3, shared=(64, 5.0))])
def test_experts_with_scaled_input(dtype, T, f):
    """The feed-forward alone (router, chosen experts on score * input, shared expert), in the sparse form (few tokens) and the
    dense one; limits small enough that the clamps act, where scaling the input and scaling the output differ."""
    from mistral_inference_b200.args import ScaledInputMoeArgs
    from mistral_inference_b200.transformer_layers import ScaledInputMoe

    W = 64
    cfg = make_config(width=W, layers=[(mlstm_cfg(), f)])
    w = {k: v.to(dtype) for k, v in make_weights(cfg, 3).items()}
    mod = ScaledInputMoe(W, ScaledInputMoeArgs.from_dict(f)).to(device=DEV, dtype=dtype)
    for k, v in w.items():
        if k.startswith("l0.mlp."):
            assert mod.assign(k[len("l0.mlp."):], lambda dst, v=v: dst.copy_(v)), k
    hn = torch.randn(T, W, generator=torch.Generator().manual_seed(T)).to(dtype)
    x32 = torch.zeros(T, W, device=DEV)
    mod.run(hn.to(DEV), x32)
    _close(x32, O.moe(hn.float(), f32(w), "l0.mlp.", f), dtype, f"T={T}")


MIXER_LAYERS = {
    "attention": side_cfg(right_scale=0.0),
    "attention_full": side_cfg(left=attn_cfg(3, 3, 20, 12, 0.5, None, None), right_scale=0.0),
    "attention_tc": side_cfg(left=attn_cfg(4, 2, 64, 64, 0.15, 40, (1000.0, 32, 1.5)), right_scale=0.0),
    "recurrence": side_cfg(left_scale=0.0),
    "recurrence_wide": side_cfg(right={"heads": 2, "dim": 70, "vdim": 150}, left_scale=0.0),
    "both": side_cfg(),
    "matrix_memory": mlstm_cfg(),
    "matrix_memory_2": mlstm_cfg(2, 36, 130, 3.0, "mlstm_2"),
    "matrix_memory_keys": mlstm_cfg(2, 200, 24, 6.0),          # more keys than one CTA's registers hold: split over CTAs
    "recurrence_keys": side_cfg(right={"heads": 1, "dim": 260, "vdim": 20}, left_scale=0.0),
}


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", sorted(MIXER_LAYERS))
def test_mixer_alone(tmp_path, dtype, kind):
    """One layer without feed-forward (and with one side switched off): a prompt of 90 tokens, whole and cut into portions and single
    tokens, against the oracle's residual stream after the layer."""
    cfg = make_config(width=48, layers=[(MIXER_LAYERS[kind], None)])
    m, cfg, w = _model(tmp_path, cfg, dtype, seed=7)
    toks = _tokens(cfg, 90, 1)
    ref = []
    O.forward(cfg, w, toks, ref)
    for cuts in ([90], [64, 26], [17, 2, 40, 1, 1, 29], [1] * 90 if dtype == torch.float32 else [3] * 30):
        taps, o = {}, 0
        pieces = []
        for c in cuts:
            pieces.append(toks[o:o + c]); o += c
        _run(m, pieces, taps=taps)
        _close(torch.cat(taps[0]), ref[0], dtype, f"{kind} cut {cuts[:6]}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["recurrence", "recurrence_wide", "matrix_memory", "matrix_memory_2", "both", "matrix_memory_keys"])
@pytest.mark.parametrize("chunk", [4, 16, 37])
def test_chunk_parallel_scan(tmp_path, monkeypatch, dtype, kind, chunk):
    """The chunk-parallel form of the scan (long prompts) with small chunks: whole prompts whose length is no multiple of the chunk,
    a second portion that starts from a carried state, a ragged batch in which one sequence is shorter than a chunk."""
    from mistral_inference_b200 import _abi_hybrid as h

    monkeypatch.setattr(h, "SCAN_CHUNK", chunk)
    monkeypatch.setattr(h, "SCAN_CHUNK_FROM", chunk + 1)
    cfg = make_config(width=48, layers=[(MIXER_LAYERS[kind], None)])
    m, cfg, w = _model(tmp_path, cfg, dtype, seed=11)
    toks = _tokens(cfg, 90, 1)
    ref = []
    O.forward(cfg, w, toks, ref)
    for cuts in ([90], [41, 49], [3, 86, 1]):
        taps, o, pieces = {}, 0, []
        for c in cuts:
            pieces.append(toks[o:o + c]); o += c
        _run(m, pieces, taps=taps)
        _close(torch.cat(taps[0]), ref[0], dtype, f"{kind} chunk {chunk} cut {cuts}")
    reqs = [_tokens(cfg, n, 20 + n) for n in (70, 3, 55)]
    cache = m.make_cache(3, 80)
    lg = m.forward(torch.tensor([t for r in reqs for t in r], device=DEV), [len(r) for r in reqs], cache)
    o = 0
    for r in reqs:
        _close(lg[o:o + len(r)], O.forward(cfg, w, r), dtype, f"{kind} chunk {chunk} in a batch")
        o += len(r)
    nxt = m.forward(torch.tensor([1, 2, 3], device=DEV), [1, 1, 1], cache)  # the states the chunked prompt left
    for i, r in enumerate(reqs):
        _close(nxt[i], O.forward(cfg, w, r + [i + 1])[-1], dtype, f"{kind} chunk {chunk}: next token of {i}")


# ----------------------------------------------------------------------------- whole models
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", sorted(SHAPES))
def test_prompt_decode_portions(tmp_path, dtype, name):
    m, cfg, w = _model(tmp_path, name, dtype)
    toks = _tokens(cfg, 150, 2)
    ref_taps = []
    ref = O.forward(cfg, w, toks, ref_taps)
    taps = {}
    whole = _run(m, [toks], taps=taps)
    for r in range(len(cfg["layers"])):
        _close(taps[r][0], ref_taps[r], dtype, f"{name} layer {r}")
    _close(whole, ref, dtype, f"{name} whole")
    by_token = _run(m, [toks[:100]] + [[t] for t in toks[100:]])
    _close(by_token, ref, dtype, f"{name} prompt + 50 decoded")
    tol = dict(tol=2e-4) if dtype == torch.float32 else {}
    _close(by_token, whole, dtype, f"{name} decoded against whole", **tol)
    for cuts in ([2] * 75, [7, 64, 3, 65, 11], [149, 1], [1, 149]):
        o, pieces = 0, []
        for c in cuts:
            pieces.append(toks[o:o + c]); o += c
        _close(_run(m, pieces), whole, dtype, f"{name} portions {cuts[:5]}", **tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("name", ["odd", "tc"])
def test_ragged_batch_retire_and_reuse(tmp_path, dtype, name):
    """Three unequal requests as one batch: prompts together, then token by token; the shorter ones end first.  Then other requests
    in the same rows (states and rings of the first batch must not show).  Each against the request alone."""
    m, cfg, w = _model(tmp_path, name, dtype)
    cache = m.make_cache(3, 140)
    tol = dict(tol=2e-4) if dtype == torch.float32 else {}
    for round_, (lens, dec) in enumerate([((70, 3, 100), (20, 5, 30)), ((1, 90, 33), (40, 3, 8))]):
        reqs = [_tokens(cfg, n + d, 10 * round_ + i) for i, (n, d) in enumerate(zip(lens, dec))]
        alone = [_run(m, [r]) for r in reqs]
        if round_ == 0:
            _close(alone[0], O.forward(cfg, w, reqs[0]), dtype, "alone against the oracle")
        cache.reset()
        cache.init_kvseqlens(3)
        got = [[] for _ in reqs]
        live = [0, 1, 2]
        flat = [t for r, n in zip(reqs, lens) for t in r[:n]]
        lg = m.forward(torch.tensor(flat, device=DEV), list(lens), cache)
        o = 0
        for i, n in enumerate(lens):
            got[i].append(lg[o:o + n]); o += n
        step = 0
        while live:
            ended = [k for k, i in enumerate(live) if step >= dec[i]]
            if ended:
                cache.retire(ended)
                live = [i for k, i in enumerate(live) if k not in ended]
                if not live:
                    break
            lg = m.forward(torch.tensor([reqs[i][lens[i] + step] for i in live], device=DEV), [1] * len(live), cache)
            for k, i in enumerate(live):
                got[i].append(lg[k:k + 1])
            step += 1
        for i in range(3):
            _close(torch.cat(got[i]), alone[i], dtype, f"{name} round {round_} request {i}", **tol)


@pytest.mark.parametrize("phase", ["prompt", "decoded"])
def test_window_edges(tmp_path, phase):
    """A token whose value stands out (its embedding lies along a direction that only W_v sees strongly): the positions at which it
    is the last key inside the window and the first one outside differ visibly, in a prompt and in decoding, with windows of 1, 2,
    the tile size of the prompt kernel and beyond it."""
    for win, d in [(1, 16), (2, 16), (7, 16), (64, 32), (65, 32), (100, 64)]:
        cfg = make_config(width=48, vocab=12, layers=[(side_cfg(left=attn_cfg(2, 1, d, d, 0.2, win, (100.0, 8, 2.0)), right_scale=0.0), None)])
        w = make_weights(cfg, 3)
        z = torch.zeros(48); z[5] = 1.0
        w["embed"][:, 5] = 0; w["pos"][:, 5] = 0
        w["embed"][11] = 0.05 * w["embed"][11] + 30 * z          # the marker token
        w["l0.mix.left.v"][:, 5] = 40.0                            # every value column sees the marked direction
        for dtype in (torch.float32, torch.bfloat16):
            m, _, wf = _model(tmp_path / f"{win}{dtype}", cfg, dtype, weights={k: v.clone() for k, v in w.items()})
            n, at = win + 80, 30
            toks = [t % 11 for t in _tokens(cfg, n, win)]
            toks[at] = 11
            ref_taps = []
            O.forward(cfg, wf, toks, ref_taps)
            cut = n if phase == "prompt" else at + 3
            taps = {}
            _run(m, [toks[:cut]] + [[t] for t in toks[cut:]], taps=taps)
            got = torch.cat(taps[0])
            _close(got, ref_taps[0], dtype, f"window {win}")
            inside, outside = at + win - 1, at + win
            delta = (ref_taps[0][inside] - ref_taps[0][outside]).abs().max()
            assert delta > 0.5, "the marker must show"
            assert (got[inside].cpu() - ref_taps[0][inside]).abs().max() < 0.1 * delta and (got[outside].cpu() - ref_taps[0][outside]).abs().max() < 0.1 * delta


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_memory_and_long_decoding(tmp_path, dtype):
    """600 tokens with forget gates close to 1: what the states took in at the start still shows at the end (the oracle's logits
    change when the first tokens do).  A prompt of 200 and 400 decoded tokens, the ring of the windowed layer going round many times."""
    m, cfg, w = _model(tmp_path, "odd", dtype, long_memory=True)
    toks = _tokens(cfg, 600, 4)
    ref = O.forward(cfg, w, toks)
    other = O.forward(cfg, w, [(t + 1) % cfg["vocab"] for t in toks[:20]] + toks[20:])
    assert (ref[-1] - other[-1]).abs().max() > 1e-2, "the first tokens must still show at the end"
    got = _run(m, [toks[:200]] + [[t] for t in toks[200:]])
    _close(got, ref, dtype, "long", tol=1e-3)
    _close(_run(m, [toks]), ref, dtype, "long prompt (chunk-parallel scan)", tol=1e-3)


def test_first_tokens_and_rows_far_apart(tmp_path):
    """Sequences of 1 and 2 tokens, and a sequence in the last row of a large cache."""
    m, cfg, w = _model(tmp_path, "odd", torch.float32)
    for n in (1, 2, 3):
        toks = _tokens(cfg, n, n)
        _close(_run(m, [toks]), O.forward(cfg, w, toks), torch.float32, f"{n} tokens")
        _close(_run(m, [[t] for t in toks]), O.forward(cfg, w, toks), torch.float32, f"{n} tokens, one by one")
    cache = m.make_cache(6, 64)
    cache.init_kvseqlens(1)
    cache._rows = [5]
    toks = _tokens(cfg, 40, 9)
    _close(_run(m, [toks[:30]] + [[t] for t in toks[30:]], cache=cache), O.forward(cfg, w, toks), torch.float32, "row 5")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_generate_greedy(tmp_path, dtype):
    """Greedy generation through generate() (chunked prompts, the CUDA-graph decode step) repeats the oracle's choices wherever the
    oracle's best two logits are not close."""
    from mistral_inference_b200.generate import generate

    m, cfg, w = _model(tmp_path, "tc", dtype)
    m.args.max_batch_size = 2
    prompts = [_tokens(cfg, 70, 1), _tokens(cfg, 80, 2)]
    for chunk in (None, 16):
        out, lps = generate(prompts, m, max_tokens=12, temperature=0.0, chunk_size=chunk)
        for p, o in zip(prompts, out):
            seq = list(p)
            for tok in o:
                lg = O.forward(cfg, w, seq)[-1]
                top2 = torch.topk(lg, 2).values
                if top2[0] - top2[1] > (0.02 if dtype == torch.float32 else 0.5):
                    assert tok == int(lg.argmax()), (chunk, len(seq))
                seq.append(tok)
        assert len(lps[0]) == len(prompts[0]) - 1 + 12


def test_command_line_and_trace_runner(tmp_path):
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    cfg = make_config(**SHAPES["odd"])
    w = make_weights(cfg, 0)
    folder = write_folder(tmp_path / "m", cfg, {k: v.to(torch.bfloat16) for k, v in w.items()})
    repo = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    r = subprocess.run([sys.executable, "-m", "mistral_inference_b200.main", "generate", str(folder), "--prompt", "1 2 3 4", "--max-tokens", "5", "--dtype", "float32"],
                       cwd=repo, capture_output=True, text=True)
    assert r.returncode == 0 and len(r.stdout.split()) == 5, r.stderr[-2000:]
    a, b = _tokens(cfg, 30, 1), _tokens(cfg, 9, 2)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:25], "want": [0, 24]}, {"id": "b", "tokens": b[:8], "want": [7]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[25:26], "want": []}, {"id": "b", "tokens": b[8:9], "want": [0]}], "end": ["b"]}]
    steps += [{"step": 2 + i, "entries": [{"id": "a", "tokens": [a[26 + i]], "want": [0]}], "end": ["a"] if i == 3 else []} for i in range(4)]
    steps += [{"step": 6, "entries": [{"id": "c", "tokens": b, "want": [8]}], "end": ["c"]}]
    r = subprocess.run([os.path.join(repo, "bin", "trace_run"), "--model", str(folder), "--dtype", "float32", "--out", str(tmp_path / "o"), "--max-tokens", "64"],
                       input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.split("\n") if ln.startswith("done")] == [f"done {i}" for i in range(7)]
    wf = f32({k: v.to(torch.bfloat16) for k, v in w.items()})
    ra, rb = O.forward(cfg, wf, a), O.forward(cfg, wf, b)

    def out(i):
        return torch.from_numpy(np.fromfile(tmp_path / "o" / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))

    _close(out(0), torch.stack([ra[0], ra[24], rb[7]]), torch.float32)
    _close(out(1), rb[8:9], torch.float32)
    assert (tmp_path / "o" / "1.f32").stat().st_size == 4 * cfg["vocab"]
    for i in range(4):
        _close(out(2 + i), ra[26 + i: 27 + i], torch.float32)
    _close(out(6), rb[8:9], torch.float32)
