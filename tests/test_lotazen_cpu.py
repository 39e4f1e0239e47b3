"""Host-side logic of the Lotazen design: configuration, registry, checkpoint packing, cache layout."""
import pytest
import torch

from tests.lotazen_util import attn_cfg, make_config, make_weights, mlstm_cfg, moe_cfg, side_cfg


def _cfg():
    return make_config(width=40, vocab=50, layers=[(side_cfg(), moe_cfg()), (mlstm_cfg(), None), (mlstm_cfg(1, 20, 6, 15.0, "mlstm_2"), moe_cfg(shared=None)),
                                                   (side_cfg(left=attn_cfg(2, 2, 16, 24, 0.4, None, None)), moe_cfg(top=1))])


def test_config():
    from mistral_inference_b200.args import LayeredArgs, MlstmArgs, ScaledInputMoeArgs, SideBySideArgs

    a = LayeredArgs.from_dict(_cfg())
    assert a.norm == "rms_scalar" and a.parallel_block and a.learned_positions and a.max_positions == 1024 and a.logit_softcap == 9.0
    L0, L1, L2, L3 = a.layers
    assert isinstance(L0.mixer, SideBySideArgs) and L0.mixer.left.window == 5 and L0.mixer.left.rot_dims == 8 and L0.mixer.left.rot_factor == 3.0
    assert L0.mixer.left_scale == 0.7 and L0.mixer.right.vdim == 7
    assert isinstance(L0.mlp, ScaledInputMoeArgs) and L0.mlp.top == 2 and L0.mlp.shared.ff == 20 and L0.mlp.shared.limit == 1.5 and L0.mlp.limit == 0.8
    assert isinstance(L1.mixer, MlstmArgs) and L1.mlp is None and isinstance(L2.mixer, MlstmArgs) and L2.mixer.gate_cap == 15.0 and L2.mlp.shared is None
    assert L3.mixer.left.window is None and L3.mixer.left.rot_dims == 0 and L3.mixer.left.rot_factor == 1.0
    bad = _cfg()
    bad["layers"][0]["mixer"]["left"]["rot"]["dims"] = 14
    with pytest.raises(AssertionError):
        LayeredArgs.from_dict(bad)
    bad = _cfg()
    bad["layers"][0]["mlp"]["router"]["top"] = 6
    with pytest.raises(AssertionError):
        LayeredArgs.from_dict(bad)
    # the same kind name means another feed-forward in another design
    from mistral_inference_b200.args import DESIGN_MLP_ARGS, MLP_ARGS, MoeFfArgs
    assert MLP_ARGS["moe"] is MoeFfArgs and DESIGN_MLP_ARGS["Lotazen"]["moe"] is ScaledInputMoeArgs


def test_registry_and_packing(tmp_path):
    from mistral_inference_b200.args import LayeredArgs
    from mistral_inference_b200.layered import LayeredTransformer
    from mistral_inference_b200.registry import ARCHITECTURES, architecture_of
    from tests.lotazen_util import write_folder

    cfg = _cfg()
    w = make_weights(cfg, 1)
    assert architecture_of(write_folder(tmp_path / "m", cfg, w)) == "Lotazen" and "Lotazen" in ARCHITECTURES
    m = LayeredTransformer(LayeredArgs.from_dict(cfg))
    assert sorted(m.checkpoint_keys()) == sorted(w.keys())
    m.load_state_dict(w)
    blk = m.layers[0]
    assert blk.norm2 is None and blk.parallel
    assert torch.equal(blk.norm1.weight, w["l0.norm1"].expand(40)) and torch.equal(m.final_norm.weight, w["final.norm"].expand(40))
    left, right = blk.mix.left, blk.mix.right
    assert torch.equal(left.wqkv[48:72], w["l0.mix.left.k"]) and torch.equal(left.wo, w["l0.mix.left.o"])
    assert torch.equal(right.wqfv[30:60], w["l0.mix.right.f"]) and torch.equal(right.bqfv[30:60], w["l0.mix.right.f.b"])
    assert right.bqfv[:30].abs().sum() == 0 and right.bqfv[60:].abs().sum() == 0
    mm = m.layers[1].mix
    assert torch.equal(mm.wif[3:], w["l1.mix.f"]) and torch.equal(mm.bif[:3], w["l1.mix.i.b"]) and torch.equal(mm.wqkvg[60:102], w["l1.mix.v"])
    ff = blk.mlp
    assert torch.equal(ff.w13.view(5, 12, 2, 40)[3, :, 1], w["l0.mlp.e3.up"]) and torch.equal(ff.w2.view(40, 5, 12)[:, 4], w["l0.mlp.e4.down"])
    assert torch.equal(ff.shared.w13.view(20, 2, 40)[:, 0], w["l0.mlp.shared.gate"]) and m.layers[2].mlp.shared is None
    with pytest.raises(ValueError):
        m._assign("l0.mix.left.bogus", torch.zeros(1))
    missing = dict(w)
    del missing["l1.mix.i.b"]
    with pytest.raises(AssertionError):
        m.load_state_dict(missing)


def test_cache_layout():
    from mistral_inference_b200.args import LayeredArgs
    from mistral_inference_b200.layered import LayeredTransformer

    m = LayeredTransformer(LayeredArgs.from_dict(_cfg()))
    specs = [m.layers[i].mix.cache_spec() for i in m.runs]
    assert specs[0].kind == "ring" and specs[0].window == 5 and specs[0].state_shape == (3, 10, 7) and (specs[0].n_kv_heads, specs[0].k_dim, specs[0].v_dim) == (2, 12, 10)
    assert specs[1].kind == "state" and specs[1].state_shape == (3 * 10 * 15 + 3,)
    assert specs[3].window is None
    from mistral_inference_b200.cache import BufferCache

    c = BufferCache(4, 3, 64, 0, 0, None, layer_specs=specs)
    assert c.cache_sizes == [5, 64, 64, 64]
    assert c.cache_k[0].shape == (3, 5, 2, 12) and c.cache_state[0].shape == (3, 3, 10, 7) and c.cache_state[0].dtype == torch.float32
    assert 1 not in c.cache_k and c.cache_state[1].shape == (3, 453)
    # a prompt longer than the ring: only its last 5 tokens get a ring row, in ring order
    c.init_kvseqlens(2)
    host, layout = c.build_metadata_host([8, 3])
    md = c.metadata_from_block(torch.from_numpy(host), layout, [8, 3])
    assert md[0].window == 5 and md[0].cache_rows.tolist() == [-1, -1, -1, 3, 4, 0, 1, 2, 5, 6, 7]
    assert md[1].window == 64 and md[0].positions.tolist() == list(range(8)) + list(range(3))
