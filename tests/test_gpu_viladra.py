"""The Viladra design on the GPU against the plain statement in tests/viladra_oracle.py: every mechanism alone (convolution on the
stream with its carried inputs, norm after the sublayer with the depth average, softmax router with scaled weights, ungated experts
dense and sparse, retention, gated linear attention, sigmoid-weight window attention), then whole models of several shapes through
the cache: prompts against token-by-token decoding, portions, ragged batches, reused rows, window edges, long memories, long
decoding, and greedy generation through `generate()`.  fp32 runs are compared tightly, bf16 runs by an error norm per token."""
import math

import pytest
import torch

from tests import viladra_oracle as O
from tests.viladra_util import attn_cfg, f32, gla_cfg, make_config, make_weights, moe_cfg, retention_cfg, write_folder

pytestmark = pytest.mark.gpu
DEV = "cuda"

SHAPES = {
    # sizes that are no multiple of 8 or 32, 4 query heads on 2 key/value heads, a window of 5, rotation over part of a head, a layer
    # without feed-forward, one without shared expert, attention over the whole sequence, a retention layer without rotation
    "odd": dict(width=40, vocab=50, taps=4, layers=[
        (gla_cfg(), moe_cfg()),
        (retention_cfg(), None),
        (attn_cfg(), moe_cfg(ff=9, experts=3, top=1, shared=None)),
        (attn_cfg(2, 2, 16, 24, 0.4, None), moe_cfg(ff=14, experts=4, top=4, scale=0.7, shared=6)),
        (retention_cfg(1, 20, 36, (0.8,), None), moe_cfg())]),
    # head sizes of the tensor-core prompt kernel, windows that cross its 64-key tiles, keys wider than 64 and more value columns
    # than one CTA of the scan holds, two taps
    "tc": dict(width=64, vocab=70, taps=2, layers=[
        (attn_cfg(4, 2, 32, 32, 0.35, 70), moe_cfg(ff=32, experts=6, top=2, shared=16)),
        (gla_cfg(2, 72, 136, 16.0, 8), moe_cfg(ff=32, experts=4, top=1)),
        (attn_cfg(2, 1, 64, 64, 0.2, 33), None),
        (retention_cfg(2, 64, 32, (0.96875, 0.99), (10000.0, 64)), moe_cfg(ff=16, experts=2, top=2, scale=2.0, shared=None)),
        (attn_cfg(3, 3, 128, 64, 0.1, 200), None)]),
    # nothing is a multiple of 2, 4 or 8 where it need not be: width 30, odd head sizes, 3 query heads on 1 key/value head, 17 words,
    # five taps, a decay projection of rank 1
    "awkward": dict(width=30, vocab=17, taps=5, layers=[
        (attn_cfg(3, 1, 7, 5, 0.5, 9), moe_cfg(ff=7, experts=3, top=2, shared=5)),
        (gla_cfg(2, 7, 3, 3.0, 1), moe_cfg(ff=6, experts=2, top=1, shared=None)),
        (retention_cfg(2, 5, 9, (0.6, 0.95), (33.0, 2)), None)]),
    # everything 1: one head, one expert of which one is used, a window that shows only the token itself, one tap (no carried
    # inputs), no embedding scale, tau 1
    "one": dict(width=24, vocab=20, taps=1, softcap=3.0, embed_scale=1.0, layers=[
        (attn_cfg(1, 1, 8, 8, 1.0, 1), moe_cfg(ff=8, experts=1, top=1, scale=1.0, shared=8)),
        (gla_cfg(1, 4, 4, 1.0, 2), moe_cfg(ff=8, experts=2, top=2, shared=None)),
        (retention_cfg(1, 4, 4, (1.0,), (10.0, 2)), None)]),
}
MIXER_LAYERS = {
    "retention": retention_cfg(), "retention_plain": retention_cfg(2, 16, 8, (0.9, 0.5), None), "retention_wide": retention_cfg(1, 136, 40, (0.99,), (1e4, 100)),
    "gla": gla_cfg(), "gla_wide": gla_cfg(1, 130, 140, 16.0, 3),
    "attention": attn_cfg(), "attention_full": attn_cfg(2, 2, 16, 24, 0.4, None), "attention_tc": attn_cfg(4, 1, 64, 32, 0.2, 40),
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


def _i32(xs):
    return torch.tensor(xs, dtype=torch.int32, device=DEV)


# ----------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps", [1, 2, 3, 6, 9, 20])
@pytest.mark.parametrize("D", [37, 40, 520])
def test_convolution_on_the_stream(dtype, taps, D):
    """Two sequences in rows 4 and 1 of the state, fed whole, in portions (shorter and longer than the taps reach back) and token
    by token; a row that held another sequence before is started afresh.  Channel counts that the four-at-a-time prompt kernel takes
    (40; 520: more than one CTA of channels) and one it does not; tap counts on both sides of its limit."""
    from mistral_inference_b200 import _abi_hybrid as h

    lens = (23, 9)
    g = torch.Generator().manual_seed(taps)
    xs = [torch.randn(n, D, generator=g) for n in lens]
    w = (0.5 * torch.randn(D, taps, generator=g)).to(dtype)
    ref = [O.causal_conv_added(x, w.float()) for x in xs]
    state = torch.full((6, 2, max(taps - 1, 1), D), 777.0, device=DEV) if taps > 1 else None  # stale numbers must not show
    slots = _i32([4, 1])
    for cuts in ([lens], [(1, 1)] * 9 + [(14, 0)], [(2, 3), (1, 1), (7, 5), (13, 0)], [(20, 8), (1, 1), (2, 0)]):
        done = [0, 0]
        got = [[], []]
        for step in cuts:
            live = [i for i in (0, 1) if step[i] > 0]
            x = torch.cat([xs[i][done[i]:done[i] + step[i]] for i in live]).to(DEV)
            qs = [0]
            for i in live:
                qs.append(qs[-1] + step[i])
            one_each = all(step[i] == 1 for i in live) and all(done[i] > 0 for i in live)
            out = h.canon_conv(x, w.to(DEV), state, (taps - 1) * D, _i32(qs), _i32([done[i] for i in live]), slots[live], len(live), one_each)
            for k, i in enumerate(live):
                got[i].append(out[qs[k]:qs[k + 1]])
                done[i] += step[i]
        for i in (0, 1):
            _close(torch.cat(got[i]), ref[i].to(dtype), torch.float32, f"taps {taps} cuts {cuts[:3]}", tol=1e-5 if dtype == torch.float32 else 2e-2)
        if state is not None:
            assert bool((state[:, 0] == 777.0).all()) and bool((state[0] == 777.0).all()), "only this convolution's part of its own rows is written"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_after_the_sublayer_and_depth_average(dtype):
    from mistral_inference_b200 import _abi_hybrid as h
    from mistral_inference_b200.transformer_layers import Norm

    T, D, n = 11, 44, 4
    nrm = Norm(D, 1e-3, "rms").to(DEV).to(dtype)
    nrm.load_weight((1 + 0.3 * torch.randn(D)).to(dtype))
    y = torch.randn(T, D, device=DEV) * 5
    stack = torch.randn(n + 1, T, D, device=DEV)
    coef = torch.randn(n).to(dtype).to(DEV)
    before = stack.clone().cpu()
    want_acc = before[n - 1] + O.unit_rms(y.cpu(), 1e-3) * nrm.weight.float().cpu()
    nrm(y, add_to=stack[n - 1], mix=(stack, n, coef, stack[n]))
    _close(stack[n - 1], want_acc, torch.float32, tol=1e-5)
    _close(stack[n], O.depth_average([*before[:n - 1], want_acc], coef.float().cpu()), torch.float32, tol=1e-5)
    assert torch.equal(stack[:n - 1].cpu(), before[:n - 1])
    acc = torch.randn(T, D, device=DEV)
    want = acc.cpu() + O.unit_rms(y.cpu(), 1e-3) * nrm.weight.float().cpu()
    nrm(y, add_to=acc)
    _close(acc, want, torch.float32, tol=1e-5)
    out = torch.empty(T, D, device=DEV)
    h.depth_mix(stack, 3, coef[:3].contiguous(), out)
    _close(out, O.depth_average(list(stack[:3].cpu()), coef.float().cpu()), torch.float32, tol=1e-5)


@pytest.mark.parametrize("E,top,scale", [(5, 2, 1.3), (12, 1, 0.5), (3, 3, 2.0), (40, 6, 1.0)])
def test_softmax_router_with_scaled_weights(E, top, scale):
    from mistral_inference_b200 import _abi_hybrid as h

    x, wr = torch.randn(9, 24, device=DEV), torch.randn(E, 24, device=DEV)
    dense, idx, wsel = h.moe_route(x, wr, None, 1, 1, top, score=0, scale=scale)
    for t in range(9):
        ref_idx, ref_w = O.router(x[t].cpu(), wr.cpu(), top, scale)
        assert idx[t].tolist() == ref_idx
        _close(wsel[t], torch.tensor(ref_w), torch.float32, tol=1e-5)
        row = torch.zeros(E)
        row[ref_idx] = torch.tensor(ref_w)
        _close(dense[t], row, torch.float32, tol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T", [1, 5, 16, 17, 150])
@pytest.mark.parametrize("f", [moe_cfg(), moe_cfg(ff=32, experts=4, top=1, scale=0.5, shared=None), moe_cfg(ff=16, experts=3, top=3, shared=64)])
def test_ungated_experts(dtype, T, f):
    """The feed-forward alone, dense (prompts) and sparse (few tokens), against the oracle on the same inputs."""
    from mistral_inference_b200.args import Relu2MoeArgs
    from mistral_inference_b200.transformer_layers import Relu2Moe

    width = 40
    cfg = make_config(width=width, layers=[(retention_cfg(), f)])
    w = {k: v.to(dtype) for k, v in make_weights(cfg, 5).items()}
    ff = Relu2Moe(width, Relu2MoeArgs.from_dict(f)).to(DEV).to(dtype)
    for k, v in w.items():
        if k.startswith("l0.mlp."):
            assert ff.assign(k[len("l0.mlp."):], lambda dst: dst.copy_(v))
    hs = torch.randn(T, width).to(dtype)
    x32 = torch.zeros(T, width, device=DEV)
    ff.run(hs.to(DEV), x32)
    _close(x32, O.moe(hs.float(), f32(w), "l0.mlp.", f), dtype, f"T={T}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", sorted(MIXER_LAYERS))
def test_mixer_alone(tmp_path, dtype, kind):
    """A model of one layer without feed-forward: the stream after the layer, for a prompt, a prompt with decoded tokens and
    portions."""
    cfg = make_config(width=48, vocab=30, taps=3, layers=[(MIXER_LAYERS[kind], None)])
    m, _, w = _model(tmp_path, cfg, dtype, seed=7)
    toks = _tokens(cfg, 90, 1)
    ref = []
    O.forward(cfg, w, toks, ref)
    for pieces in ([toks], [toks[:60]] + [[t] for t in toks[60:]], [toks[:2], toks[2:19], toks[19:83], toks[83:]]):
        taps = {}
        _run(m, pieces, taps=taps)
        _close(torch.cat(taps[0]), ref[0], dtype, f"{kind} in {len(pieces)} pieces")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("kind", ["retention", "retention_wide", "gla", "gla_wide"])
@pytest.mark.parametrize("chunk", [4, 16, 37])
def test_chunk_parallel_scan(tmp_path, monkeypatch, dtype, kind, chunk):
    """Long prompts run the scan chunk-parallel; the same recurrence, so the same numbers as the walk over the whole sequence."""
    from mistral_inference_b200 import _abi_hybrid as h

    cfg = make_config(width=48, vocab=30, taps=3, layers=[(MIXER_LAYERS[kind], None)])
    m, _, w = _model(tmp_path, cfg, dtype, seed=3)
    toks = _tokens(cfg, 120, 2)
    ref = []
    O.forward(cfg, w, toks, ref)
    monkeypatch.setattr(h, "SCAN_CHUNK", chunk)
    monkeypatch.setattr(h, "SCAN_CHUNK_FROM", 2 * chunk)
    for pieces in ([toks], [toks[:50], toks[50:]], [toks[:100]] + [[t] for t in toks[100:]]):
        taps = {}
        _run(m, pieces, taps=taps)
        _close(torch.cat(taps[0]), ref[0], dtype, f"{kind} chunk {chunk}")


# ----------------------------------------------------------------------------- whole models through the cache
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
    in the same rows (states, rings and carried convolution inputs of the first batch must not show).  Each against the request alone."""
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
    """A token whose value stands out (its embedding lies along a direction that only W_v sees strongly, and every key is made to
    weigh about one half): the positions at which it is the last key inside the window and the first one outside differ visibly, in
    a prompt and in decoding, with windows of 1, 2, the tile size of the prompt kernel and beyond it."""
    for win, d in [(1, 16), (2, 16), (7, 16), (64, 32), (65, 32), (100, 64)]:
        cfg = make_config(width=48, vocab=12, taps=1, layers=[(attn_cfg(2, 1, d, d, 0.05, win), None)])
        w = make_weights(cfg, 3)
        z = torch.zeros(48); z[5] = 1.0
        w["embed"][:, 5] = 0
        w["l0.canon1"].zero_()                                     # the marker stays at its own position
        w["embed"][11] = 0.05 * w["embed"][11] + 30 * z            # the marker token
        w["l0.mix.v"][:, 5] = 40.0                                 # every value column sees the marked direction
        w["l0.mix.q"][:, 5] = 0; w["l0.mix.k"][:, 5] = 0; w["l0.mix.g"][:, 5] = 0
        w["l0.mix.pb"].zero_()
        for dtype in (torch.float32, torch.bfloat16):
            m, _, wf = _model(tmp_path / f"{win}{dtype}", cfg, dtype, weights={k: v.clone() for k, v in w.items()})
            n, at = win + 80, 30
            toks = [t % 11 for t in _tokens(cfg, n, win)]
            toks[at] = 11
            mix_ref, ref_taps = [], []
            O.forward(cfg, wf, toks, ref_taps, mix_ref)
            ref = mix_ref[0]  # the mixer's raw output shows the marker directly; the stream after the layer is what can be compared
            cut = n if phase == "prompt" else at + 3
            taps = {}
            _run(m, [toks[:cut]] + [[t] for t in toks[cut:]], taps=taps)
            got = torch.cat(taps[0])
            _close(got, ref_taps[0], dtype, f"window {win}")
            inside, outside = at + win - 1, at + win
            assert (ref[inside] - ref[outside]).abs().max() > 50, "the marker must dominate the mixer's output while it is visible"
            delta = (ref_taps[0][inside] - ref_taps[0][outside]).abs().max()
            assert delta > 0.3, "the marker must show in the stream"
            assert (got[inside].cpu() - ref_taps[0][inside]).abs().max() < 0.1 * delta and (got[outside].cpu() - ref_taps[0][outside]).abs().max() < 0.1 * delta


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_long_memory_and_long_decoding(tmp_path, dtype):
    """600 tokens with decays close to 1: what the states took in at the start still shows at the end (the oracle's logits change
    when the first tokens do).  A prompt of 200 and 400 decoded tokens, the ring of the windowed layer going round many times."""
    layers = [(gla_cfg(tau=16.0), moe_cfg()), (retention_cfg(2, 10, 6, (0.9990234375, 0.998046875), (1e4, 10)), None), (attn_cfg(), moe_cfg(shared=None))]
    cfg = make_config(width=40, vocab=50, taps=3, layers=layers)
    m, _, w = _model(tmp_path, cfg, dtype, weights=make_weights(cfg, 4, long_memory=True))
    toks = _tokens(cfg, 600, 4)
    ref = O.forward(cfg, w, toks)
    other = O.forward(cfg, w, [(t + 1) % cfg["vocab"] for t in toks[:20]] + toks[20:])
    assert (ref[-1] - other[-1]).abs().max() > 1e-2, "the first tokens must still show at the end"
    got = _run(m, [toks[:200]] + [[t] for t in toks[200:]])
    _close(got, ref, dtype, "long", tol=1e-3)
    _close(_run(m, [toks]), ref, dtype, "long prompt (chunk-parallel scan)", tol=1e-3)


def test_first_tokens_and_rows_far_apart(tmp_path):
    """Sequences of 1, 2 and 3 tokens (shorter than the convolution reaches back), and a sequence in the last row of a large cache."""
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

    def rows(i):
        return torch.from_numpy(np.fromfile(tmp_path / "o" / f"{i}.f32", dtype="<f4").reshape(-1, cfg["vocab"]))

    _close(rows(0), torch.stack([ra[0], ra[24], rb[7]]), torch.float32, "step 0")
    _close(rows(1), rb[8:9], torch.float32, "step 1")
    for i in range(4):
        _close(rows(2 + i), ra[26 + i:27 + i], torch.float32, f"step {2 + i}")
    _close(rows(6), rb[8:9], torch.float32, "a new batch in used rows")
    assert not math.isnan(float(rows(6).sum()))
