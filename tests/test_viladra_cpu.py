"""Host-side logic of the Viladra design: configuration, registry, checkpoint packing, cache layout."""
import pytest
import torch

from tests.viladra_util import attn_cfg, gla_cfg, make_config, make_weights, moe_cfg, on_disk, retention_cfg


def _cfg():
    return make_config(width=40, vocab=50, taps=4, layers=[(gla_cfg(), moe_cfg()), (retention_cfg(), None), (attn_cfg(), moe_cfg(shared=None)),
                                                            (attn_cfg(2, 2, 16, 24, 0.4, None), moe_cfg(top=1)), (retention_cfg(1, 8, 8, (0.75,), None), moe_cfg())])


def test_config():
    from mistral_inference_b200.args import (DESIGN_MIXER_ARGS, DESIGN_MLP_ARGS, MIXER_ARGS, BiasedAttentionArgs, GlaArgs, LayeredArgs, Relu2MoeArgs,
                                             RetentionArgs, SigmoidAttentionArgs)

    a = LayeredArgs.from_dict(on_disk(_cfg()))
    assert a.norm == "rms" and a.post_norm and not a.pre_norm and a.canon and a.canon_taps == 4 and a.depth_average and a.tied_head
    assert a.logit_softcap == 9.0 and a.embedding_scale == 2.0
    L0, L1, L2, L3, L4 = a.layers
    assert isinstance(L0.mixer, GlaArgs) and L0.mixer.tau == 8.0 and isinstance(L0.mlp, Relu2MoeArgs) and L0.mlp.router_scale == 1.3 and L0.mlp.shared.ff == 20
    assert isinstance(L1.mixer, RetentionArgs) and L1.mixer.decay == [0.9, 0.97, 0.5] and L1.mixer.rot_dims == 6 and L1.mixer.rot_base == 100.0 and L1.mlp is None
    assert isinstance(L2.mixer, SigmoidAttentionArgs) and L2.mixer.window == 5 and L2.mlp.shared is None and L3.mixer.window is None and L3.mlp.top == 1
    assert L4.mixer.rot_dims == 0
    # the same type name means another mixer in another design
    assert MIXER_ARGS["attention"] is BiasedAttentionArgs and DESIGN_MIXER_ARGS["Viladra"]["attention"] is SigmoidAttentionArgs
    assert DESIGN_MLP_ARGS["Viladra"]["moe"] is Relu2MoeArgs
    for path, value in ((("layers", 1, "mixer", "rot", "dims"), 14), (("layers", 1, "mixer", "rot", "dims"), 5), (("layers", 0, "mlp", "router", "top"), 6),
                        (("layers", 1, "mixer", "decay"), [0.5]), (("layers", 2, "mixer", "kv_heads"), 3), (("canon", "taps"), 0)):
        bad = on_disk(_cfg())
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(AssertionError):
            LayeredArgs.from_dict(bad)


def test_registry_and_packing(tmp_path):
    from mistral_inference_b200.args import LayeredArgs
    from mistral_inference_b200.layered import LayeredTransformer
    from mistral_inference_b200.registry import ARCHITECTURES, architecture_of
    from tests.viladra_util import write_folder

    cfg = _cfg()
    w = make_weights(cfg, 1)
    assert architecture_of(write_folder(tmp_path / "m", cfg, w)) == "Viladra" and "Viladra" in ARCHITECTURES
    m = LayeredTransformer(LayeredArgs.from_dict(on_disk(cfg)))
    assert sorted(m.checkpoint_keys()) == sorted(w.keys())
    assert m.head is None  # the logits use the embedding table
    m.load_state_dict(w)
    b0, b1, b2 = m.layers[0], m.layers[1], m.layers[2]
    assert not b0.pre_norm and b0.norm1b is None and b1.norm2 is None and b1.canon2 is None and b0.canon2 is not None
    assert torch.equal(b0.canon1.weight, w["l0.canon1"]) and torch.equal(b0.canon2.weight, w["l0.canon2"]) and torch.equal(b2.dwa, w["l2.dwa"])
    assert b0.dwa.shape == (2,) and m.layers[4].dwa.shape == (6,)
    g = b0.mix  # q | k | v | g rows; the decay projection takes the checkpoint's rank
    assert torch.equal(g.wqkvg[24:48], w["l0.mix.k"]) and torch.equal(g.wqkvg[68:], w["l0.mix.g"]) and g.wa1.shape == (5, 40) and g.wa2.shape == (24, 5)
    assert torch.equal(g.wa2, w["l0.mix.a2"]) and torch.equal(g.ba2, w["l0.mix.a2.b"]) and torch.equal(g.norm, w["l0.mix.norm"])
    r = b1.mix
    assert torch.equal(r.wqkvg[30:60], w["l1.mix.k"]) and torch.equal(r.wqkvg[60:78], w["l1.mix.v"]) and torch.equal(r.wo, w["l1.mix.o"])
    at = b2.mix
    assert torch.equal(at.wqkv[48:72], w["l2.mix.k"]) and torch.equal(at.bqkv[72:], w["l2.mix.v.b"]) and torch.equal(at.q_norm, w["l2.mix.q.norm"])
    assert torch.equal(at.pb, w["l2.mix.pb"]) and torch.equal(at.wg, w["l2.mix.g"]) and torch.equal(at.bo, w["l2.mix.o.b"])
    ff = b0.mlp
    assert torch.equal(ff.w_up[36:48], w["l0.mlp.e3.up"]) and torch.equal(ff.w2.view(40, 5, 12)[:, 4], w["l0.mlp.e4.down"])
    assert torch.equal(ff.shared.w_up, w["l0.mlp.shared.up"]) and b2.mlp.shared is None
    missing = dict(w)
    del missing["l3.canon2"]
    with pytest.raises(AssertionError):
        LayeredTransformer(LayeredArgs.from_dict(on_disk(cfg))).load_state_dict(missing)
    with pytest.raises(ValueError):
        m.load_state_dict({"l1.canon2": w["l0.canon2"]}, strict=False)  # a layer without feed-forward has no second convolution


def test_cache_layout():
    from mistral_inference_b200.args import LayeredArgs
    from mistral_inference_b200.cache import BufferCache
    from mistral_inference_b200.layered import LayeredTransformer

    m = LayeredTransformer(LayeredArgs.from_dict(on_disk(_cfg())))
    specs = [blk.mix.cache_spec() for blk in m.layers]
    for sp, blk in zip(specs, m.layers):
        sp.conv_shape = blk.conv_shape()
    assert [sp.kind for sp in specs] == ["state", "state", "ring", "ring", "state"]
    assert specs[0].state_shape == (2, 12, 10) and specs[1].state_shape == (3, 10, 6) and specs[2].window == 5 and specs[3].window is None
    assert specs[0].conv_shape == (2, 3, 40) and specs[1].conv_shape == (1, 3, 40)  # last taps - 1 inputs of each convolution
    c = BufferCache(5, 3, 64, 0, 0, None, layer_specs=specs)
    assert c.cache_conv[0].shape == (3, 2, 3, 40) and c.cache_conv[0].dtype == torch.float32 and c.cache_conv[1].shape == (3, 1, 3, 40)
    assert c.cache_k[2].shape == (3, 5, 2, 12) and c.cache_v[3].shape == (3, 64, 2, 24) and c.cache_state[4].shape == (3, 1, 8, 8)
    c.init_kvseqlens(2)
    md = c.get_input_metadata([7, 2])
    v = c.get_view(0, md[0])
    assert v.conv is c.cache_conv[0] and v.state is c.cache_state[0] and c.get_view(2, md[2]).conv is c.cache_conv[2]
    one_tap = LayeredTransformer(LayeredArgs.from_dict({**on_disk(_cfg()), "canon": {"taps": 1}}))
    assert one_tap.layers[0].conv_shape() == ()
