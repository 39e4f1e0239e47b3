"""`bench.py --design fesenex|taruvik|lotazen|viladra`: prefill and decode throughput of the layered decoder at layer sizes of real models (random
weights), beside the dense `Transformer` of equal width / heads / feed-forward size / depth / vocabulary, plus the time of each
hybrid kernel at those shapes against its roofline (bf16 tensor peak or HBM copy bandwidth from MEASURED_PEAKS.json).
For `taruvik` (latent attention, mixture of experts) the neighbour is the `Transformer` with a mixture of experts of equal
width / heads / experts / depth; for `lotazen` (rotary window attention beside a gated recurrence, matrix memories, experts with scaled
input) it is the Fesenex design at equal width / heads / depth, and every new kernel is timed next to the like kernel at the same shape;
for `viladra` (convolution on the stream, norms after the sublayers with a depth average, retention, gated linear attention,
sigmoid-weight window attention, ungated experts) the neighbour is the Lotazen design at equal width / heads / experts / depth.  Timed with CUDA events after warm-up; the prompt batch and the weights exceed L2 at the larger size, and L2 is flushed between
timed kernel launches.  Prints one JSON line."""
import json
import math
import time

import torch

SIZES = {
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, ff=8192, vocab=32768, layers=8, lin_heads=16),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, ff=14336, vocab=32768, layers=4, lin_heads=32),
}


def layered_config(s: dict) -> dict:
    att = {"type": "attention", "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["dim"], "vdim": s["dim"], "scale": s["dim"] ** -0.5,
                                          "bias_max": 4096, "q_temp": {"coef": 0.1, "every": 1024}, "v_mix": True},
           "mlp": {"kind": "dense", "ff": s["ff"], "limit": 7.0}}
    lin = {"type": "lightning", "mixer": {"heads": s["lin_heads"], "dim": s["dim"], "vdim": s["dim"],
                                          "decay": [math.exp(-1.0 / (4 + 8 * h)) for h in range(s["lin_heads"])]},
           "mlp": {"kind": "dense", "ff": s["ff"], "limit": 7.0}}
    return {"architecture": "Fesenex", "vocab": s["vocab"], "width": s["width"], "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5},
            "layers": [lin if (i in s["lightning_at"] if "lightning_at" in s else i % 4 == 3) else att for i in range(s["layers"])]}


def build_layered(s: dict, dev):
    from mistral_inference_b200.args import LayeredArgs
    from mistral_inference_b200.layered import LayeredTransformer
    from mistral_inference_b200.transformer_layers import BiasedAttention

    m = LayeredTransformer.empty(LayeredArgs.from_dict(layered_config(s)), dev, torch.bfloat16)
    g = torch.Generator(device=dev).manual_seed(0)
    with torch.no_grad():
        for blk in m.layers:
            if isinstance(blk.mix, BiasedAttention):
                blk.mix.rel = torch.nn.Parameter(torch.empty(32, blk.mix.a.heads, dtype=torch.bfloat16, device=dev), requires_grad=False)
        for n, p in m.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g, device=dev, dtype=torch.float32) / math.sqrt(p.shape[-1]))
            elif "norm" in n:
                p.fill_(1.0)
            else:
                p.copy_(torch.randn(p.shape, generator=g, device=dev, dtype=torch.float32) * 0.1)
    return m.eval()


def build_dense(s: dict, dev):
    import mistral_inference_b200 as mi
    from mistral_inference_b200.transformer import Transformer

    args = mi.TransformerArgs(dim=s["width"], n_layers=s["layers"], head_dim=s["dim"], hidden_dim=s["ff"], n_heads=s["heads"], n_kv_heads=s["kv_heads"],
                              norm_eps=1e-5, vocab_size=s["vocab"], max_batch_size=8)
    m = Transformer.empty(args, dev, torch.bfloat16)
    g = torch.Generator(device=dev).manual_seed(0)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g, device=dev, dtype=torch.float32) / math.sqrt(p.shape[-1]))
            else:
                p.fill_(1.0)
    return m.eval()


def _time(fn, warmup: int, steps: int, flush=None) -> float:
    """Median milliseconds of fn() over `steps` runs."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(steps):
        if flush is not None:
            flush.add_(1.0)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    ts.sort()
    return ts[len(ts) // 2]


def end_to_end(model, vocab: int, T: int, ctx: int, batches, warmup: int, steps: int, dev) -> dict:
    out = {}
    ids = torch.randint(0, vocab, (T,), device=dev)
    cache = model.make_cache(max(batches), ctx + 64 + warmup + steps)

    def prefill():
        cache.reset()
        model.forward(ids, [T], cache)

    ms = _time(prefill, max(3, warmup // 4), max(3, steps // 8))
    out["prefill"] = {"tokens": T, "ms": round(ms, 3), "tok_s": round(T / ms * 1e3, 1)}
    for B in batches:
        cache.reset()
        n = ctx // 2 if B > 1 else ctx
        model.forward(ids[:n].repeat(B), [n] * B, cache)
        tok = torch.randint(0, vocab, (B,), device=dev)
        ms = _time(lambda: model.next_token_logits(tok, cache), warmup, steps)
        out[f"decode_b{B}"] = {"context": n, "ms": round(ms, 4), "tok_s": round(B / ms * 1e3, 1)}
    return out


def kernel_table(s: dict, T: int, ctx: int, peaks: dict, dev) -> dict:
    """Every hybrid kernel alone at this size: time, achieved rate, fraction of the measured roofline."""
    from mistral_inference_b200 import _abi_hybrid as h

    bf = torch.bfloat16
    W, H, G, d, ff = s["width"], s["heads"], s["kv_heads"], s["dim"], s["ff"]
    flush = torch.zeros(160 << 20, dtype=torch.float32, device=dev)  # 640 MB > L2
    rows = {}

    def rec(name, ms, flops=0.0, bytes_=0.0):
        r = {"ms": round(ms, 4)}
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
            r["of_bf16_peak"] = round(flops / ms / 1e9 / peaks["bf16_tflops"], 3)
        if bytes_:
            r["gb_s"] = round(bytes_ / ms / 1e6, 1)
            r["of_hbm_peak"] = round(bytes_ / ms / 1e6 / peaks["hbm_gbs"], 3)
        rows[name] = r

    x = torch.randn(T, W, device=dev).to(bf)
    w13 = torch.randn(2 * ff, W, device=dev).to(bf) * 0.02
    rec("prompt linear gate/up+glu (tcgen05 GEMM + epilogue pass)", _time(lambda: h.linear(x, w13, epi=h.EPI_GLU, limit=7.0, alpha=1.702), 3, 8, flush), flops=2.0 * T * 2 * ff * W)
    for M in (1, 8):
        xs = x[:M].contiguous()
        rec(f"linear_skinny gate/up+glu M={M}", _time(lambda: h.linear(xs, w13, epi=h.EPI_GLU, limit=7.0, alpha=1.702), 3, 8, flush), bytes_=w13.numel() * 2.0)
    # attention: a prompt of T tokens, then one token per sequence at context ctx
    from mistral_inference_b200.cache import BufferCache, LayerCacheSpec
    B = 8
    cache = BufferCache(1, B, ctx + 8, 0, 0, None, layer_specs=[LayerCacheSpec(kind="ring", n_kv_heads=G, k_dim=d, v_dim=d)]).to(dev, bf)
    cache.cache_k[0].normal_(); cache.cache_v[0].normal_()
    tab = torch.zeros(64, H, device=dev)
    md = cache.get_input_metadata([T])[0]
    q = torch.randn(T, H * d, device=dev).to(bf)
    o = torch.empty_like(q)
    att = lambda: h.attn_bias(q, cache.cache_k[0], cache.cache_v[0], tab, md.positions, md.q_start, md.slots, o, 1, ctx + 8, H, G, d, d, d ** -0.5,
                              n_tiles=(T + 63) // 64)  # noqa: E731
    rec("attn_bias_flash prompt", _time(att, 2, 5, flush), flops=4.0 * d * H * T * (T + 1) / 2)
    cache.reset(); cache.init_kvseqlens(B); cache.update_seqlens([ctx] * B)
    md2 = cache.get_input_metadata([1] * B)[0]
    q2, o2 = q[:B].contiguous(), torch.empty(B, H * d, device=dev, dtype=bf)
    dec = lambda: h.attn_bias(q2, cache.cache_k[0], cache.cache_v[0], tab, md2.positions, md2.q_start, md2.slots, o2, B, ctx + 8, H, G, d, d, d ** -0.5,
                              splits=h.attn_splits(B, H, ctx + 8))  # noqa: E731
    rec(f"attn_bias decode B={B} ctx={ctx}", _time(dec, 3, 8, flush), bytes_=2.0 * B * (ctx + 1) * G * d * 2)
    # lightning: prompt and decode
    LH = s["lin_heads"]
    qkvg = torch.randn(T, 4 * LH * d, device=dev).to(bf) * 0.1
    state = torch.zeros(B, LH, d, d, device=dev)
    dec_ = torch.full((LH,), 0.97, device=dev)
    o32 = torch.empty(T, LH * d, device=dev)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    rec("lightning_scan prompt", _time(lambda: h.lightning_scan(qkvg, state, dec_, md.q_start, zero, md.slots, o32, 1, LH, d, d), 2, 5, flush),
        flops=4.0 * T * LH * d * d)
    one = torch.ones(B, dtype=torch.int32, device=dev)
    rec(f"lightning_scan decode B={B}", _time(lambda: h.lightning_scan(qkvg, state, dec_, md2.q_start, one, md2.slots, o32, B, LH, d, d), 3, 8, flush),
        bytes_=2.0 * state.numel() * 4)
    return rows


# ----------------------------------------------------------------------------------------------- Taruvik
TARUVIK_SIZES = {
    "w2048": dict(width=2048, heads=16, dim=128, rot_dim=64, vdim=128, q_rank=768, kv_rank=512, experts=16, identity=4, top=4, groups=4, keep=2,
                  ff=1408, vocab=32768, layers=4),
    "w4096": dict(width=4096, heads=32, dim=128, rot_dim=64, vdim=128, q_rank=1536, kv_rank=512, experts=8, identity=0, top=2, groups=1, keep=1,
                  ff=14336, vocab=32768, layers=2),
}


def taruvik_config(s: dict) -> dict:
    mix = {"heads": s["heads"], "dim": s["dim"], "rot_dim": s["rot_dim"], "vdim": s["vdim"], "q_rank": s["q_rank"], "kv_rank": s["kv_rank"],
           "scale": (s["dim"] + s["rot_dim"]) ** -0.5,
           "rot": {"base": 10000.0, "dims": s["rot_dim"], "scaling": {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}}}
    mlp = {"kind": "moe", "expert": {"ff": s["ff"]},
           "router": {"experts": s["experts"], "identity": s["identity"], "top": s["top"], "groups": {"count": s["groups"], "keep": s["keep"]}}}
    return {"architecture": "Taruvik", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5},
            "layers": [{"type": "latent_attention", "mixer": mix, "mlp": mlp} for _ in range(s["layers"])]}


def build_taruvik(s: dict, dev):
    from mistral_inference_b200.args import LayeredArgs
    from mistral_inference_b200.layered import LayeredTransformer

    m = LayeredTransformer.empty(LayeredArgs.from_dict(taruvik_config(s)), dev, torch.bfloat16)
    g = torch.Generator(device=dev).manual_seed(0)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g, device=dev, dtype=torch.float32) / math.sqrt(p.shape[-1]))
            elif n.endswith("weight") or "norm" in n.rsplit(".", 1)[-1]:
                p.fill_(1.0)
            else:
                p.copy_(torch.randn(p.shape, generator=g, device=dev, dtype=torch.float32) * 0.01)
    return m.eval()


def build_moe_transformer(s: dict, dev):
    import mistral_inference_b200 as mi
    from mistral_inference_b200.args import MoeArgs
    from mistral_inference_b200.transformer import Transformer

    args = mi.TransformerArgs(dim=s["width"], n_layers=s["layers"], head_dim=s["dim"], hidden_dim=s["ff"], n_heads=s["heads"], n_kv_heads=s["heads"],
                              norm_eps=1e-5, vocab_size=s["vocab"], max_batch_size=8, moe=MoeArgs(num_experts=s["experts"], num_experts_per_tok=s["top"]))
    m = Transformer.empty(args, dev, torch.bfloat16)
    g = torch.Generator(device=dev).manual_seed(0)
    with torch.no_grad():
        for n, p in m.named_parameters():
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g, device=dev, dtype=torch.float32) / math.sqrt(p.shape[-1]))
            else:
                p.fill_(1.0)
    return m.eval()


def taruvik_kernel_table(s: dict, T: int, ctx: int, peaks: dict, dev) -> dict:
    """Every kernel that the design added, alone at this size: time, achieved rate, fraction of the measured roofline (bytes and
    FLOPs are the algorithm's: what a perfect kernel would have to move or compute)."""
    from mistral_inference_b200 import _abi_hybrid as h
    from mistral_inference_b200.cache import BufferCache, LayerCacheSpec
    from mistral_inference_b200.rope import scaled_frequencies

    bf = torch.bfloat16
    W, H, dn, dr, dv, rq, rk, E, ff, top = (s[k] for k in ("width", "heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "experts", "ff", "top"))
    n_routed = E + s["identity"]
    flush = torch.zeros(160 << 20, dtype=torch.float32, device=dev)
    rows = {}

    def rec(name, ms, flops=0.0, bytes_=0.0, note=None):
        r = {"ms": round(ms, 4)}
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 1)
            r["of_bf16_peak"] = round(flops / ms / 1e9 / peaks["bf16_tflops"], 3)
        if bytes_:
            r["gb_s"] = round(bytes_ / ms / 1e6, 1)
            r["of_hbm_peak"] = round(bytes_ / ms / 1e6 / peaks["hbm_gbs"], 3)
        if note:
            r["note"] = note
        rows[name] = r

    B = 8
    x32 = torch.randn(T, W, device=dev)
    wv, bv = torch.ones(W, device=dev).to(bf), torch.zeros(W, device=dev).to(bf)
    rec("layernorm prompt", _time(lambda: h.layernorm(x32, wv, bv, 1e-5), 3, 8, flush), bytes_=T * W * 6.0)
    acc = torch.zeros(T, W, device=dev)
    rec("layernorm + residual add prompt", _time(lambda: h.layernorm(x32, wv, bv, 1e-5, add_to=acc), 3, 8, flush), bytes_=T * W * 12.0)
    # latent attention
    freq, mag = scaled_frequencies(dr, 10000.0, None)
    freq = freq.to(dev)
    n_in = rq + rk + dr + H
    cache = BufferCache(1, B, ctx + 8, 0, 0, None, layer_specs=[LayerCacheSpec(kind="ring", n_kv_heads=1, k_dim=rk + dr, v_dim=0)]).to(dev, bf)
    cache.cache_k[0].normal_()
    md = cache.get_input_metadata([T])[0]
    y = torch.randn(T, n_in, device=dev).to(bf)
    qn, cn = torch.ones(rq, device=dev).to(bf), torch.ones(rk, device=dev).to(bf)
    rec("latent_prep prompt", _time(lambda: h.latent_prep(y, qn, cn, freq, md.positions, md.cache_rows, cache.cache_k[0], rq, rk, dr, dr, 1e-5, mag), 3, 8, flush),
        bytes_=T * (n_in + rq + rk + dr) * 2.0)
    q = torch.randn(T, H * (dn + dr), device=dev).to(bf)
    w_uk = (torch.randn(H * dn, rk, device=dev) / math.sqrt(rk)).to(bf)
    rec("latent_absorb prompt", _time(lambda: h.latent_absorb(q, w_uk, freq, md.positions, H, dn, dr, dr, rk, mag), 2, 5, flush), flops=2.0 * T * H * dn * rk)
    qa = torch.randn(T, H * (rk + dr), device=dev).to(bf)
    Tp = min(T, 1024)  # the exact kernel on a prompt: a shorter one keeps the run short
    mdp = cache.get_input_metadata([Tp])[0]
    qp = qa[:Tp].contiguous()
    rec(f"attn_latent (latent form, portions of prompts and fp32) T={Tp}", _time(lambda: h.attn_latent(qp, cache.cache_k[0], mdp.positions, mdp.q_start, mdp.slots, 1, ctx + 8, H, rk, dr, 0.07,
                                                                 splits=h.attn_splits(Tp, H, ctx + 8)), 1, 3, flush),
        flops=2.0 * H * (2 * rk + dr) * Tp * (Tp + 1) / 2, note="exact fp32 FMA kernel, no tensor cores")
    cache.reset(); cache.init_kvseqlens(B); cache.update_seqlens([ctx] * B)
    md2 = cache.get_input_metadata([1] * B)[0]
    q2 = qa[:B].contiguous()
    rec(f"attn_latent (a CTA per head) decode B={B} ctx={ctx}", _time(lambda: h.attn_latent(q2, cache.cache_k[0], md2.positions, md2.q_start, md2.slots, B, ctx + 8, H, rk, dr, 0.07,
                                                                            splits=h.attn_splits(B, H, ctx + 8)), 3, 8, flush),
        bytes_=B * (ctx + 1) * (rk + dr) * 2.0, note="bytes: every latent row once; each head's CTAs re-read them through L2")
    rec(f"attn_latent_decode (rows shared by the heads) B={B} ctx={ctx}",
        _time(lambda: h.attn_latent_decode(q2, cache.cache_k[0], md2.positions, md2.slots, B, ctx + 8, H, rk, dr, 0.07), 3, 8, flush),
        bytes_=B * (ctx + 1) * (rk + dr) * 2.0)
    if (dn + dr, dv) in h.FLASH_SIZES:  # whole prompts: multi-head attention over written-out keys and values
        kf = torch.randn(T, H, dn + dr, device=dev).to(bf)
        vf = torch.randn(T, H, dv, device=dev).to(bf)
        qr = torch.randn(T, H * (dn + dr), device=dev).to(bf)
        of = torch.empty(T, H * dv, device=dev, dtype=bf)
        rec(f"prompt attention over written-out keys (attn_bias_flash, {dn + dr}/{dv}) T={T}",
            _time(lambda: h.attn_bias(qr, kf, vf, None, md.positions, md.q_start, h.iota(1, dev), of, 1, T, H, H, dn + dr, dv, 0.07, n_tiles=(T + 63) // 64), 2, 5, flush),
            flops=2.0 * H * (dn + dr + dv) * T * (T + 1) / 2)
    o_lat = torch.randn(T, H * rk, device=dev).to(bf)
    w_uv = (torch.randn(H * dv, rk, device=dev) / math.sqrt(rk)).to(bf)
    rec("latent_vup prompt", _time(lambda: h.latent_vup(o_lat, w_uv, y, n_in, rq + rk + dr, H, dv, rk), 2, 5, flush), flops=2.0 * T * H * dv * rk)
    ob = o_lat[:B].contiguous()
    rec(f"latent_vup decode B={B}", _time(lambda: h.latent_vup(ob, w_uv, y, n_in, rq + rk + dr, H, dv, rk), 3, 8, flush), bytes_=w_uv.numel() * 2.0)
    qb = q[:B].contiguous()
    rec(f"latent_absorb decode B={B}", _time(lambda: h.latent_absorb(qb, w_uk, freq, md2.positions, H, dn, dr, dr, rk, mag), 3, 8, flush), bytes_=w_uk.numel() * 2.0)
    # mixture of experts
    x = torch.randn(T, W, device=dev).to(bf)
    wr = (torch.randn(n_routed, W, device=dev) / math.sqrt(W) * 4).to(bf)
    corr = torch.zeros(n_routed, device=dev).to(bf)
    rec("moe_route prompt", _time(lambda: h.moe_route(x, wr, corr, s["groups"], s["keep"], top), 3, 8, flush), bytes_=T * W * 2.0)
    dense, idx, wsel = h.moe_route(x, wr, corr, s["groups"], s["keep"], top)
    w13 = (torch.randn(E * 2 * ff, W, device=dev) * 0.02).to(bf)
    w2 = (torch.randn(W, E * ff, device=dev) * 0.02).to(bf)

    def dense_form():
        act = h.linear_swiglu(x, w13, rowscale=dense, group=ff)
        return h.linear(act, w2, epi=h.EPI_F32)

    rec("experts prompt (all experts, masked)", _time(dense_form, 2, 5, flush), flops=6.0 * T * top * ff * W,
        note=f"useful FLOPs (top {top} of {E}); the kernels compute all {E} experts")
    for M in (1, B):
        xs, ii, ww = x[:M].contiguous(), idx[:M].contiguous(), wsel[:M].contiguous()
        live = int((ii < E).sum())
        rec(f"experts decode (chosen only) M={M}", _time(lambda: h.moe_sparse(xs, w13, w2, ii, ww, E, ff), 3, 8, flush), bytes_=live * 3.0 * ff * W * 2)
    return rows


def run_taruvik(a, peaks: dict) -> dict:
    dev = torch.device("cuda", torch.cuda.current_device())
    T, ctx = a.prefill, a.prefill
    res = {"design": "Taruvik", "dtype": "bf16", "data": "synthetic", "prompt_tokens": T, "peaks": {k: peaks.get(k) for k in ("hbm_gbs", "bf16_tflops")}, "sizes": {}}
    for name, s in TARUVIK_SIZES.items():
        t0 = time.time()
        m = build_taruvik(s, dev)
        new = end_to_end(m, s["vocab"], T, ctx, (1, 8), a.warmup, a.steps, dev)
        del m
        torch.cuda.empty_cache()
        try:
            d = build_moe_transformer(s, dev)
            old = end_to_end(d, s["vocab"], T, ctx, (1, 8), a.warmup, a.steps, dev)
            del d
        except Exception as e:  # the neighbour's kernels may not take this size
            old = {"unavailable": f"{type(e).__name__}: {e}"[:300]}
        torch.cuda.empty_cache()
        res["sizes"][name] = {"config": s, "layered": new, "moe_transformer": old, "kernels": taruvik_kernel_table(s, T, ctx, peaks, dev),
                              "seconds": round(time.time() - t0, 1)}
    return res


# ----------------------------------------------------------------------------------------------- Lotazen
LOTAZEN_SIZES = {
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, window=1024, rec_heads=16, experts=16, top=2, ff=1408, shared_ff=2816, vocab=32768,
                  order="ppmp", lin_heads=16),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, window=2048, rec_heads=32, experts=8, top=2, ff=3584, shared_ff=7168, vocab=32768,
                  order="pm", lin_heads=32),
}


def lotazen_config(s: dict) -> dict:
    d = s["dim"]
    side = {"type": "parallel", "mixer": {
        "left": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": d, "vdim": d, "scale": d ** -0.5, "mask": {"size": s["window"]},
                 "rot": {"base": 500000.0, "dims": d, "scaling": {"factor": 2.0}}},
        "right": {"heads": s["rec_heads"], "dim": d, "vdim": d}, "left_scale": 0.6, "right_scale": 0.5}}
    mem = {"type": "mlstm", "mixer": {"heads": s["rec_heads"], "dim": d, "vdim": d, "gate_cap": 12.0}}
    mlp = {"kind": "moe", "expert": {"ff": s["ff"], "limit": 7.0}, "router": {"experts": s["experts"], "top": s["top"]},
           "shared": {"ff": s["shared_ff"], "limit": 7.0}}
    return {"architecture": "Lotazen", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5}, "max_positions": 8192, "logit_softcap": 30.0,
            "layers": [{**(side if c == "p" else mem), "mlp": mlp} for c in s["order"]]}


def build_lotazen(s: dict, dev):
    from mistral_inference_b200.args import LayeredArgs
    from mistral_inference_b200.layered import LayeredTransformer

    m = LayeredTransformer.empty(LayeredArgs.from_dict(lotazen_config(s)), dev, torch.bfloat16)
    g = torch.Generator(device=dev).manual_seed(0)
    with torch.no_grad():
        for n, p in m.named_parameters():
            last = n.rsplit(".", 1)[-1]
            if p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g, device=dev, dtype=torch.float32) / math.sqrt(p.shape[-1]))
            elif last in ("weight", "norm"):
                p.fill_(1.0)
            elif last == "lower":
                p.copy_(torch.rand(p.shape, generator=g, device=dev) * 0.9)
            else:
                p.copy_(torch.randn(p.shape, generator=g, device=dev, dtype=torch.float32) * 0.1)
    return m.eval()


def fesenex_like(s: dict) -> dict:
    """The closest existing design at equal size: attention layers of the same heads where Lotazen has attention beside a recurrence,
    a lightning layer where it has a matrix memory, a dense feed-forward of the size of the experts one token uses."""
    return dict(width=s["width"], heads=s["heads"], kv_heads=s["kv_heads"], dim=s["dim"], ff=s["top"] * s["ff"] + s["shared_ff"], vocab=s["vocab"],
                layers=len(s["order"]), lin_heads=s["lin_heads"], lightning_at=[i for i, c in enumerate(s["order"]) if c == "m"])


def lotazen_kernel_table(s: dict, T: int, ctx: int, peaks: dict, dev) -> dict:
    """Every kernel the design added, alone at this size, each next to the like kernel of the closest design at the same shape."""
    from mistral_inference_b200 import _abi_hybrid as h
    from mistral_inference_b200.cache import BufferCache, LayerCacheSpec

    bf = torch.bfloat16
    W, H, G, d, win, RH, E, ff, top = (s[k] for k in ("width", "heads", "kv_heads", "dim", "window", "rec_heads", "experts", "ff", "top"))
    flush = torch.zeros(160 << 20, dtype=torch.float32, device=dev)
    rows = {}

    def rec(name, ms, flops=0.0, bytes_=0.0, note=None):
        r = {"ms": round(ms, 4)}
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 2)
            r["of_bf16_peak"] = round(flops / ms / 1e9 / peaks["bf16_tflops"], 4)
        if bytes_:
            r["gb_s"] = round(bytes_ / ms / 1e6, 1)
            r["of_hbm_peak"] = round(bytes_ / ms / 1e6 / peaks["hbm_gbs"], 3)
        if note:
            r["note"] = note
        rows[name] = r

    B = 8
    # ---- attention: a prompt through the window, then one token per sequence
    ring = BufferCache(1, B, ctx + 8, 0, 0, None, layer_specs=[LayerCacheSpec(kind="ring", n_kv_heads=G, k_dim=d, v_dim=d, window=win)]).to(dev, bf)
    full = BufferCache(1, B, ctx + 8, 0, 0, None, layer_specs=[LayerCacheSpec(kind="ring", n_kv_heads=G, k_dim=d, v_dim=d)]).to(dev, bf)
    for c in (ring, full):
        c.cache_k[0].normal_(); c.cache_v[0].normal_()
    md = ring.get_input_metadata([T])[0]
    mdf = full.get_input_metadata([T])[0]
    qkv = torch.randn(T, (H + 2 * G) * d, device=dev).to(bf)
    freq = (torch.tensor(500000.0, dtype=torch.float64) ** (-torch.arange(0, d, 2, dtype=torch.float64) / d) / 2.0).to(dev)
    rec("rot_prep prompt", _time(lambda: h.rot_prep(qkv, freq, md.positions, None, None, None, H, G, d, d, d, True, 1e-5, own=True), 3, 8, flush),
        bytes_=2.0 * qkv.numel() * 2)
    q, k, v = h.rot_prep(qkv, freq, md.positions, None, None, None, H, G, d, d, d, True, 1e-5, own=True)
    o = torch.empty(T, H * d, device=dev, dtype=bf)
    nt = (T + 63) // 64
    pairs = sum(min(p + 1, win) for p in range(T))  # (query, key) pairs inside the window
    rec(f"attn_window prompt (tensor-core kernel, window {win})",
        _time(lambda: h.attn_window(q, ring.cache_k[0], ring.cache_v[0], md.positions, md.q_start, md.slots, o, 1, md.window, H, G, d, d, 0.09, win, own_k=k, own_v=v,
                                    seqpos=md.seqpos, n_tiles=nt), 2, 5, flush), flops=4.0 * d * H * pairs)
    tab = torch.zeros(64, H, device=dev)
    rec("like: attn_bias_flash prompt (all keys)",
        _time(lambda: h.attn_bias(q, full.cache_k[0], full.cache_v[0], tab, mdf.positions, mdf.q_start, mdf.slots, o, 1, ctx + 8, H, G, d, d, 0.09, n_tiles=nt), 2, 5, flush),
        flops=4.0 * d * H * T * (T + 1) / 2)
    rec("kv_scatter prompt", _time(lambda: h.kv_scatter(k, v, md.cache_rows, ring.cache_k[0], ring.cache_v[0]), 3, 8, flush), bytes_=2.0 * min(T, win) * 2 * G * d * 2)
    for c in (ring, full):
        c.reset(); c.init_kvseqlens(B); c.update_seqlens([ctx] * B)
    md2, md2f = ring.get_input_metadata([1] * B)[0], full.get_input_metadata([1] * B)[0]
    q2, o2 = q[:B].contiguous(), torch.empty(B, H * d, device=dev, dtype=bf)
    rec(f"attn_window decode B={B} (ring of {md2.window})",
        _time(lambda: h.attn_window(q2, ring.cache_k[0], ring.cache_v[0], md2.positions, md2.q_start, md2.slots, o2, B, md2.window, H, G, d, d, 0.09, win,
                                    splits=h.window_decode_plan(B, H, md2.window)[0], chunk=h.window_decode_plan(B, H, md2.window)[1]), 3, 8, flush),
        bytes_=2.0 * B * min(ctx + 1, win) * G * d * 2)
    q1, o1 = q[:1].contiguous(), torch.empty(1, H * d, device=dev, dtype=bf)
    ring.reset(); ring.init_kvseqlens(1); ring.update_seqlens([ctx])
    md1 = ring.get_input_metadata([1])[0]
    for label, (sp, ch) in (("128-key chunks", (h.attn_splits(1, H, md1.window), 0)), ("planned chunks", h.window_decode_plan(1, H, md1.window))):
        rec(f"attn_window decode B=1 (ring of {md1.window}), {label}: {sp} splits",
            _time(lambda: h.attn_window(q1, ring.cache_k[0], ring.cache_v[0], md1.positions, md1.q_start, md1.slots, o1, 1, md1.window, H, G, d, d, 0.09, win,
                                        splits=sp, chunk=ch), 3, 8, flush), bytes_=2.0 * min(ctx + 1, win) * G * d * 2)
    rec(f"like: attn_bias decode B={B} ctx={ctx}",
        _time(lambda: h.attn_bias(q2, full.cache_k[0], full.cache_v[0], tab, md2f.positions, md2f.q_start, md2f.slots, o2, B, ctx + 8, H, G, d, d, 0.09,
                                  splits=h.attn_splits(B, H, ctx + 8)), 3, 8, flush), bytes_=2.0 * B * (ctx + 1) * G * d * 2)
    # ---- recurrences
    Hd = RH * d
    qfv = (torch.randn(T, 3 * Hd, device=dev) * 0.3).to(bf)
    lower = (torch.rand(Hd, device=dev) * 0.9).to(bf)
    rec("hgrn2_gates prompt", _time(lambda: h.hgrn2_gates(qfv, lower, Hd), 3, 8, flush), bytes_=T * Hd * (2 * 2 + 3 * 4.0))
    qab = h.hgrn2_gates(qfv, lower, Hd)
    state = torch.zeros(B, RH, d, d, device=dev)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    rec("gated_scan prompt (HGRN2)", _time(lambda: h.gated_scan(qab, qfv, 3 * Hd, 2 * Hd, state, md.q_start, zero, md.slots, 1, RH, d, d, ones=False), 2, 5, flush),
        flops=4.0 * T * RH * d * d, note="one CTA column walks the sequence, fp32 FMA")
    rec("gated_scan prompt (HGRN2), chunk-parallel",
        _time(lambda: h.gated_scan(qab, qfv, 3 * Hd, 2 * Hd, state, md.q_start, zero, md.slots, 1, RH, d, d, ones=False, max_seqlen=T), 2, 5, flush),
        flops=4.0 * T * RH * d * d, note="useful FLOPs; the chunks run twice (local state, then outputs), fp32 FMA")
    qkvg = torch.randn(T, 4 * Hd, device=dev).to(bf) * 0.1
    lstate = torch.zeros(B, RH, d, d, device=dev)
    decay = torch.full((RH,), 0.97, device=dev)
    o32 = torch.empty(T, Hd, device=dev)
    rec("like: lightning_scan prompt", _time(lambda: h.lightning_scan(qkvg, lstate, decay, md.q_start, zero, md.slots, o32, 1, RH, d, d), 2, 5, flush),
        flops=4.0 * T * RH * d * d, note="sequential in the tokens, fp32 FMA")
    mstate = torch.zeros(B, RH * d * (d + 1) + RH, device=dev)
    gif = torch.randn(T, 2 * RH, device=dev)
    rec("mlstm_gates prompt", _time(lambda: h.mlstm_gates(qkvg, gif, mstate, RH * d * (d + 1), md.q_start, zero, md.slots, 1, RH, d, 12.0, d ** -0.5), 3, 8, flush),
        bytes_=T * Hd * (2 * 2 + 3 * 4.0), note="includes the running maximum, one warp per head over all tokens")
    gates, qab2 = h.mlstm_gates(qkvg, gif, mstate, RH * d * (d + 1), md.q_start, zero, md.slots, 1, RH, d, 12.0, d ** -0.5)
    rec("gated_scan prompt (mLSTM, normaliser column)",
        _time(lambda: h.gated_scan(qab2, qkvg, 4 * Hd, 2 * Hd, mstate, md.q_start, zero, md.slots, 1, RH, d, d, ones=True), 2, 5, flush), flops=4.0 * T * RH * d * (d + 1))
    rec("gated_scan prompt (mLSTM, normaliser column), chunk-parallel",
        _time(lambda: h.gated_scan(qab2, qkvg, 4 * Hd, 2 * Hd, mstate, md.q_start, zero, md.slots, 1, RH, d, d, ones=True, max_seqlen=T), 2, 5, flush),
        flops=4.0 * T * RH * d * (d + 1))
    om, nq = h.gated_scan(qab2, qkvg, 4 * Hd, 2 * Hd, mstate, md.q_start, zero, md.slots, 1, RH, d, d, ones=True)
    nw = torch.ones(Hd, device=dev).to(bf)
    rec("scan_post prompt (mLSTM)", _time(lambda: h.scan_post(om, gates, nw, True, qkvg, 4 * Hd, 3 * Hd, RH, d, True, 1e-5, nq=nq), 3, 8, flush), bytes_=T * Hd * (4 + 4 + 2 + 2.0))
    rec("like: gated_headnorm prompt", _time(lambda: h.gated_headnorm(o32, nw, qkvg, 4 * Hd, 3 * Hd, 1e-5), 3, 8, flush), bytes_=T * Hd * (4 + 2 + 2.0))
    one = torch.ones(B, dtype=torch.int32, device=dev)
    qabB = qab[:B].contiguous()
    rec(f"gated_scan decode B={B} (HGRN2)", _time(lambda: h.gated_scan(qabB, qfv, 3 * Hd, 2 * Hd, state, md2.q_start, one, md2.slots, B, RH, d, d, ones=False), 3, 8, flush),
        bytes_=2.0 * state.numel() * 4)
    rec(f"like: lightning_scan decode B={B}", _time(lambda: h.lightning_scan(qkvg, lstate, decay, md2.q_start, one, md2.slots, o32, B, RH, d, d), 3, 8, flush),
        bytes_=2.0 * lstate.numel() * 4)
    # ---- experts
    x = torch.randn(T, W, device=dev).to(bf)
    wr = (torch.randn(E, W, device=dev) / math.sqrt(W) * 4).to(bf)
    rec("moe_route prompt (sigmoid)", _time(lambda: h.moe_route(x, wr, None, 1, 1, top, score=1), 3, 8, flush), bytes_=T * W * 2.0)
    dense, idx, wsel = h.moe_route(x, wr, None, 1, 1, top, score=1)
    w13 = (torch.randn(E * 2 * ff, W, device=dev) * 0.02).to(bf)
    w2 = (torch.randn(W, E * ff, device=dev) * 0.02).to(bf)
    x32 = torch.zeros(T, W, device=dev)

    def dense_form():
        act = h.linear_glu(x, w13, 7.0, 1.702, rowscale=dense, group=ff)
        return h.linear(act, w2, epi=h.EPI_RESIDUAL, residual=x32)

    def dense_like():
        act = h.linear_swiglu(x, w13, rowscale=dense, group=ff)
        return h.linear(act, w2, epi=h.EPI_F32)

    rec("experts prompt (all experts, scaled input, masked)", _time(dense_form, 2, 5, flush), flops=6.0 * T * top * ff * W,
        note=f"useful FLOPs (top {top} of {E}); the kernels compute all {E} experts")
    rec("like: experts prompt of the softmax-routed mixture", _time(dense_like, 2, 5, flush), flops=6.0 * T * top * ff * W)
    for M in (1, B):
        xs, ii, ww = x[:M].contiguous(), idx[:M].contiguous(), wsel[:M].contiguous()
        rec(f"experts decode (chosen only, scaled input) M={M}", _time(lambda: h.moe_sparse(xs, w13, w2, ii, ww, E, ff, glu=True, limit=7.0, alpha=1.702), 3, 8, flush),
            bytes_=M * top * 3.0 * ff * W * 2)
        rec(f"like: experts decode of the softmax-routed mixture M={M}", _time(lambda: h.moe_sparse(xs, w13, w2, ii, ww, E, ff), 3, 8, flush),
            bytes_=M * top * 3.0 * ff * W * 2)
    return rows


def run_lotazen(a, peaks: dict) -> dict:
    dev = torch.device("cuda", torch.cuda.current_device())
    T, ctx = a.prefill, a.prefill
    res = {"design": "Lotazen", "dtype": "bf16", "data": "synthetic", "prompt_tokens": T, "peaks": {k: peaks.get(k) for k in ("hbm_gbs", "bf16_tflops")}, "sizes": {}}
    for name, s in LOTAZEN_SIZES.items():
        t0 = time.time()
        m = build_lotazen(s, dev)
        new = end_to_end(m, s["vocab"], T, ctx, (1, 8), a.warmup, a.steps, dev)
        del m
        torch.cuda.empty_cache()
        f = fesenex_like(s)
        d = build_layered(f, dev)
        old = end_to_end(d, s["vocab"], T, ctx, (1, 8), a.warmup, a.steps, dev)
        del d
        torch.cuda.empty_cache()
        res["sizes"][name] = {"config": s, "layered": new, "fesenex_equal_size": old, "kernels": lotazen_kernel_table(s, T, ctx, peaks, dev),
                              "seconds": round(time.time() - t0, 1)}
    return res

# ----------------------------------------------------------------------------------------------- Viladra
VILADRA_SIZES = {
    "w2048": dict(width=2048, heads=16, kv_heads=4, dim=128, window=1024, rec_heads=16, experts=16, top=2, ff=1408, shared_ff=2816, vocab=32768,
                  order="grag", rank=64, taps=4),
    "w4096": dict(width=4096, heads=32, kv_heads=8, dim=128, window=2048, rec_heads=32, experts=8, top=2, ff=3584, shared_ff=7168, vocab=32768,
                  order="ar", rank=128, taps=4),
}


def viladra_config(s: dict) -> dict:
    d, RH = s["dim"], s["rec_heads"]
    mixers = {
        "a": {"type": "attention", "mixer": {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": d, "vdim": d, "scale": d ** -0.5, "mask": {"size": s["window"]}}},
        "r": {"type": "retention", "mixer": {"heads": RH, "dim": d, "vdim": d, "decay": [1.0 - 2.0 ** (-5 - 5 * i / max(RH - 1, 1)) for i in range(RH)],
                                             "rot": {"base": 500000.0, "dims": d}}},
        "g": {"type": "gla", "mixer": {"heads": RH, "dim": d, "vdim": d, "tau": 16.0}},
    }
    mlp = {"kind": "moe", "expert": {"ff": s["ff"]}, "router": {"experts": s["experts"], "top": s["top"], "scale": 1.5}, "shared": {"ff": s["shared_ff"]}}
    return {"architecture": "Viladra", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5}, "canon": {"taps": s["taps"]},
            "embedding": {"scale": 1.0}, "logit_softcap": 30.0, "layers": [{**mixers[c], "mlp": mlp} for c in s["order"]]}


def build_viladra(s: dict, dev):
    from mistral_inference_b200.args import LayeredArgs
    from mistral_inference_b200.layered import LayeredTransformer
    from mistral_inference_b200.transformer_layers import GlaMixer

    m = LayeredTransformer.empty(LayeredArgs.from_dict(viladra_config(s)), dev, torch.bfloat16)
    for blk in m.layers:  # the rank of the decay projection comes with a checkpoint; here it is the size table's
        if isinstance(blk.mix, GlaMixer):
            blk.mix.prepare("a1", (s["rank"], s["width"]))
            blk.mix.prepare("a2", (blk.mix.nqk, s["rank"]))
    g = torch.Generator(device=dev).manual_seed(0)
    with torch.no_grad():
        for n, p in m.named_parameters():
            last = n.rsplit(".", 1)[-1]
            if last == "dwa":
                p.fill_(1.0 / p.numel())
            elif last == "weight" and p.dim() == 2:  # convolution taps
                p.copy_(torch.randn(p.shape, generator=g, device=dev, dtype=torch.float32) * 0.2)
            elif p.dim() >= 2:
                p.copy_(torch.randn(p.shape, generator=g, device=dev, dtype=torch.float32) / math.sqrt(p.shape[-1]))
            elif last in ("weight", "norm", "q_norm", "k_norm"):
                p.fill_(1.0)
            elif last == "ba2":
                p.fill_(3.0)
            else:
                p.copy_(torch.randn(p.shape, generator=g, device=dev, dtype=torch.float32) * 0.1)
    return m.eval()


def lotazen_like(s: dict) -> dict:
    """The closest existing design at equal size: rotary window attention beside a gated recurrence where Viladra has sigmoid-weight
    window attention, a matrix memory where it has retention or gated linear attention, the same experts (gated there)."""
    return dict(width=s["width"], heads=s["heads"], kv_heads=s["kv_heads"], dim=s["dim"], window=s["window"], rec_heads=s["rec_heads"], experts=s["experts"],
                top=s["top"], ff=s["ff"], shared_ff=s["shared_ff"], vocab=s["vocab"], order="".join("p" if c == "a" else "m" for c in s["order"]),
                lin_heads=s["rec_heads"])


def viladra_kernel_table(s: dict, T: int, ctx: int, peaks: dict, dev) -> dict:
    """Every kernel the design added or extended, alone at this size, each next to the like kernel of the closest design at the same shape."""
    from mistral_inference_b200 import _abi_hybrid as h
    from mistral_inference_b200.cache import BufferCache, LayerCacheSpec

    bf = torch.bfloat16
    W, H, G, d, win, RH, E, ff, top, taps, rank = (s[k] for k in ("width", "heads", "kv_heads", "dim", "window", "rec_heads", "experts", "ff", "top", "taps", "rank"))
    flush = torch.zeros(160 << 20, dtype=torch.float32, device=dev)
    rows = {}

    def rec(name, ms, flops=0.0, bytes_=0.0, note=None):
        r = {"ms": round(ms, 4)}
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 2)
            r["of_bf16_peak"] = round(flops / ms / 1e9 / peaks["bf16_tflops"], 4)
        if bytes_:
            r["gb_s"] = round(bytes_ / ms / 1e6, 1)
            r["of_hbm_peak"] = round(bytes_ / ms / 1e6 / peaks["hbm_gbs"], 3)
        if note:
            r["note"] = note
        rows[name] = r

    B = 8
    ring = BufferCache(1, B, ctx + 8, 0, 0, None, layer_specs=[LayerCacheSpec(kind="ring", n_kv_heads=G, k_dim=d, v_dim=d, window=win)]).to(dev, bf)
    ring.cache_k[0].normal_(); ring.cache_v[0].normal_()
    md = ring.get_input_metadata([T])[0]
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    # ---- the stream: convolution in, norm and depth average out
    x32 = torch.randn(T, W, device=dev)
    cw = (torch.randn(W, taps, device=dev) * 0.2).to(bf)
    cstate = torch.zeros(B, 2, taps - 1, W, device=dev)
    nw = torch.ones(W, device=dev).to(bf)
    rec("canon_conv prompt", _time(lambda: h.canon_conv(x32, cw, cstate, 0, md.q_start, zero, md.slots, 1, False), 3, 8, flush), bytes_=T * W * (4 + 2.0),
        note="reads the fp32 stream, writes bf16; includes the state write-back launch")
    rec("like: rmsnorm prompt", _time(lambda: h.rmsnorm(x32, nw, 1e-5), 3, 8, flush), bytes_=T * W * (4 + 2.0))
    n_mix = 5
    stack = torch.randn(n_mix + 1, T, W, device=dev)
    y32 = torch.randn(T, W, device=dev)
    coef = torch.full((n_mix,), 1.0 / n_mix, device=dev).to(bf)
    rec("rmsnorm_add prompt", _time(lambda: h.rmsnorm_add(y32, nw, stack[n_mix - 1], 1e-5), 3, 8, flush), bytes_=T * W * 12.0)
    rec(f"rmsnorm_add + depth average over {n_mix} prompt", _time(lambda: h.rmsnorm_add(y32, nw, stack[n_mix - 1], 1e-5, stack, n_mix, coef, stack[n_mix]), 3, 8, flush),
        bytes_=T * W * 4.0 * (3 + n_mix))
    rec("like: layernorm add prompt", _time(lambda: h.layernorm(y32, nw, nw, 1e-5, add_to=stack[0]), 3, 8, flush), bytes_=T * W * 12.0)
    # ---- attention
    qkv = torch.randn(T, (H + 2 * G) * d, device=dev).to(bf)
    qn, kn = torch.ones(H * d, device=dev).to(bf), torch.ones(G * d, device=dev).to(bf)
    rec("whole_norm_prep prompt", _time(lambda: h.whole_norm_prep(qkv, qn, kn, None, None, None, H * d, G * d, G * d, 1e-5, own=True), 3, 8, flush),
        bytes_=2.0 * qkv.numel() * 2)
    freq = (torch.tensor(500000.0, dtype=torch.float64) ** (-torch.arange(0, d, 2, dtype=torch.float64) / d)).to(dev)
    rec("like: rot_prep prompt", _time(lambda: h.rot_prep(qkv, freq, md.positions, None, None, None, H, G, d, d, d, True, 1e-5, own=True), 3, 8, flush),
        bytes_=2.0 * qkv.numel() * 2)
    q, k, v = h.whole_norm_prep(qkv, qn, kn, None, None, None, H * d, G * d, G * d, 1e-5, own=True)
    o = torch.empty(T, H * d, device=dev, dtype=bf)
    nt = (T + 63) // 64
    pairs = sum(min(p + 1, win) for p in range(T))
    pb = torch.zeros(H, device=dev)
    for label, hb in (("attn_window prompt, sigmoid weights", pb), ("like: attn_window prompt, softmax", None)):
        rec(f"{label} (tensor-core kernel, window {win})",
            _time(lambda: h.attn_window(q, ring.cache_k[0], ring.cache_v[0], md.positions, md.q_start, md.slots, o, 1, md.window, H, G, d, d, 0.09, win, own_k=k,
                                        own_v=v, seqpos=md.seqpos, n_tiles=nt, head_bias=hb), 2, 5, flush), flops=4.0 * d * H * pairs)
    ring.reset(); ring.init_kvseqlens(B); ring.update_seqlens([ctx] * B)
    md2 = ring.get_input_metadata([1] * B)[0]
    q2, o2 = q[:B].contiguous(), torch.empty(B, H * d, device=dev, dtype=bf)
    sp, ch = h.window_decode_plan(B, H, md2.window)
    for label, hb in (("attn_window decode, sigmoid weights", pb), ("like: attn_window decode, softmax", None)):
        rec(f"{label} B={B} (ring of {md2.window})",
            _time(lambda: h.attn_window(q2, ring.cache_k[0], ring.cache_v[0], md2.positions, md2.q_start, md2.slots, o2, B, md2.window, H, G, d, d, 0.09, win,
                                        splits=sp, chunk=ch, head_bias=hb), 3, 8, flush), bytes_=2.0 * B * min(ctx + 1, win) * G * d * 2)
    # ---- recurrences
    Hd = RH * d
    qkvg = (torch.randn(T, 4 * Hd, device=dev) * 0.1).to(bf)
    decay = torch.full((RH,), 0.97, device=dev)
    rec("retention_qab prompt", _time(lambda: h.retention_qab(qkvg, freq, decay, md.positions, RH, d, d, d ** -0.5), 3, 8, flush), bytes_=T * Hd * (2 * 2 + 3 * 4.0))
    z32 = torch.randn(T, Hd, device=dev)
    rec("gla_qab prompt", _time(lambda: h.gla_qab(qkvg, z32, Hd, d ** -0.5, 1 / 16.0), 3, 8, flush), bytes_=T * Hd * (2 * 2 + 4 + 3 * 4.0))
    lower = (torch.rand(Hd, device=dev) * 0.9).to(bf)
    rec("like: hgrn2_gates prompt", _time(lambda: h.hgrn2_gates(qkvg, lower, Hd), 3, 8, flush), bytes_=T * Hd * (2 * 2 + 3 * 4.0))
    qab = h.gla_qab(qkvg, z32, Hd, d ** -0.5, 1 / 16.0)
    state = torch.zeros(B, RH, d, d, device=dev)
    rec("gated_scan prompt (gated linear attention), chunk-parallel",
        _time(lambda: h.gated_scan(qab, qkvg, 4 * Hd, 2 * Hd, state, md.q_start, zero, md.slots, 1, RH, d, d, ones=False, max_seqlen=T), 2, 5, flush),
        flops=4.0 * T * RH * d * d, note="the kernel of the closest design's recurrences, same launch; useful FLOPs, the chunks run twice, fp32 FMA")
    o32 = h.gated_scan(qab, qkvg, 4 * Hd, 2 * Hd, state, md.q_start, zero, md.slots, 1, RH, d, d, ones=False, max_seqlen=T)
    hw = torch.ones(d, device=dev).to(bf)
    rec("scan_post prompt (shared weight, SiLU gate)", _time(lambda: h.scan_post(o32, None, hw, False, qkvg, 4 * Hd, 3 * Hd, RH, d, False, 1e-5, silu_gate=True), 3, 8, flush),
        bytes_=T * Hd * (4 + 2 + 2.0))
    rec("scan_post prompt (no weight, SiLU gate)", _time(lambda: h.scan_post(o32, None, None, False, qkvg, 4 * Hd, 3 * Hd, RH, d, False, 1e-5, silu_gate=True), 3, 8, flush),
        bytes_=T * Hd * (4 + 2 + 2.0))
    rec("like: scan_post prompt (shared weight, no gate)", _time(lambda: h.scan_post(o32, None, hw, False, None, 0, 0, RH, d, False, 1e-5), 3, 8, flush), bytes_=T * Hd * (4 + 2.0))
    one = torch.ones(B, dtype=torch.int32, device=dev)
    qabB = qab[:B].contiguous()
    rec(f"gated_scan decode B={B}", _time(lambda: h.gated_scan(qabB, qkvg, 4 * Hd, 2 * Hd, state, md2.q_start, one, md2.slots, B, RH, d, d, ones=False), 3, 8, flush),
        bytes_=2.0 * state.numel() * 4, note="the closest design's kernel")
    # ---- experts
    x = torch.randn(T, W, device=dev).to(bf)
    wr = (torch.randn(E, W, device=dev) / math.sqrt(W) * 4).to(bf)
    rec("moe_route prompt (softmax, scaled weights)", _time(lambda: h.moe_route(x, wr, None, 1, 1, top, score=0, scale=1.5), 3, 8, flush), bytes_=T * W * 2.0)
    rec("like: moe_route prompt (sigmoid)", _time(lambda: h.moe_route(x, wr, None, 1, 1, top, score=1), 3, 8, flush), bytes_=T * W * 2.0)
    dense, idx, wsel = h.moe_route(x, wr, None, 1, 1, top, score=0, scale=1.5)
    w_up = (torch.randn(E * ff, W, device=dev) * 0.02).to(bf)
    w13 = (torch.randn(E * 2 * ff, W, device=dev) * 0.02).to(bf)
    w2 = (torch.randn(W, E * ff, device=dev) * 0.02).to(bf)
    xr = torch.zeros(T, W, device=dev)

    def dense_form():
        return h.linear(h.linear_relu2(x, w_up, rowscale=dense, group=ff), w2, epi=h.EPI_F32)

    def dense_like():
        return h.linear(h.linear_glu(x, w13, 7.0, 1.702, rowscale=dense, group=ff), w2, epi=h.EPI_RESIDUAL, residual=xr)

    rec("experts prompt (all experts, ungated, masked)", _time(dense_form, 2, 5, flush), flops=4.0 * T * top * ff * W,
        note=f"useful FLOPs (top {top} of {E}); the kernels compute all {E} experts")
    rec("like: experts prompt of the scaled-input gated mixture", _time(dense_like, 2, 5, flush), flops=6.0 * T * top * ff * W)
    for M in (1, B):
        xs, ii, ww = x[:M].contiguous(), idx[:M].contiguous(), wsel[:M].contiguous()
        rec(f"experts decode (chosen only, ungated) M={M}", _time(lambda: h.moe_sparse(xs, w_up, w2, ii, ww, E, ff, glu=2), 3, 8, flush),
            bytes_=M * top * 2.0 * ff * W * 2)
        rec(f"like: experts decode of the scaled-input gated mixture M={M}", _time(lambda: h.moe_sparse(xs, w13, w2, ii, ww, E, ff, glu=1, limit=7.0, alpha=1.702), 3, 8, flush),
            bytes_=M * top * 3.0 * ff * W * 2)
    # ---- one decode step's convolution and norms
    xB = x32[:B].contiguous()
    rec(f"canon_conv decode B={B}", _time(lambda: h.canon_conv(xB, cw, cstate, 0, md2.q_start, one, md2.slots, B, True), 3, 8, flush),
        bytes_=B * W * (4 + 2 + 2 * (taps - 1) * 4.0), note="latency: a few KB")
    rec(f"like: rmsnorm decode B={B}", _time(lambda: h.rmsnorm(xB, nw, 1e-5), 3, 8, flush), bytes_=B * W * (4 + 2.0))
    return rows


def run_viladra(a, peaks: dict) -> dict:
    dev = torch.device("cuda", torch.cuda.current_device())
    T, ctx = a.prefill, a.prefill
    res = {"design": "Viladra", "dtype": "bf16", "data": "synthetic", "prompt_tokens": T, "peaks": {k: peaks.get(k) for k in ("hbm_gbs", "bf16_tflops")}, "sizes": {}}
    for name, s in VILADRA_SIZES.items():
        t0 = time.time()
        m = build_viladra(s, dev)
        new = end_to_end(m, s["vocab"], T, ctx, (1, 8), a.warmup, a.steps, dev)
        del m
        torch.cuda.empty_cache()
        d = build_lotazen(lotazen_like(s), dev)
        old = end_to_end(d, s["vocab"], T, ctx, (1, 8), a.warmup, a.steps, dev)
        del d
        torch.cuda.empty_cache()
        res["sizes"][name] = {"config": s, "layered": new, "lotazen_equal_size": old, "kernels": viladra_kernel_table(s, T, ctx, peaks, dev),
                              "seconds": round(time.time() - t0, 1)}
    return res


def run(a, peaks: dict) -> dict:
    if a.design == "viladra":
        return run_viladra(a, peaks)
    if a.design == "taruvik":
        return run_taruvik(a, peaks)
    if a.design == "lotazen":
        return run_lotazen(a, peaks)
    dev = torch.device("cuda", torch.cuda.current_device())
    T, ctx = a.prefill, a.prefill
    res = {"design": "Fesenex", "dtype": "bf16", "data": "synthetic", "prompt_tokens": T, "peaks": {k: peaks.get(k) for k in ("hbm_gbs", "bf16_tflops")}, "sizes": {}}
    for name, s in SIZES.items():
        t0 = time.time()
        m = build_layered(s, dev)
        new = end_to_end(m, s["vocab"], T, ctx, (1, 8), a.warmup, a.steps, dev)
        del m
        torch.cuda.empty_cache()
        d = build_dense(s, dev)
        old = end_to_end(d, s["vocab"], T, ctx, (1, 8), a.warmup, a.steps, dev)
        del d
        torch.cuda.empty_cache()
        res["sizes"][name] = {"config": s, "layered": new, "dense_transformer": old, "kernels": kernel_table(s, T, ctx, peaks, dev),
                              "seconds": round(time.time() - t0, 1)}
    return res
