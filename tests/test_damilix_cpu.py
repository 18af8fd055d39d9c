"""CPU-side checks of the Damilix family: registry, configuration, tensor inventory, checkpoint round trip, the rotation's
frequency table, and the oracle's own invariants (the GPU tests compare the engine with this oracle)."""
import json
import math
import os

import pytest
import torch

import damilix_oracle as O


def _save(tmp_path, cfg, W, name="m"):
    from safetensors.torch import save_file
    d = os.path.join(str(tmp_path), name)
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in W.items()}, os.path.join(d, "model.safetensors"))
    return d


def test_registry_resolves_by_architecture():
    from nanorlhf_b200.models.damilix import DamilixForCausalLM
    from nanorlhf_b200.models.registry import resolve
    cls, kind = resolve({"architecture": "Damilix"})
    assert cls is DamilixForCausalLM and kind == "hybrid"
    assert resolve({"model_type": "damilix"})[0] is DamilixForCausalLM


def test_config_reads_every_size_and_constant():
    from nanorlhf_b200.models.damilix import DamilixConfig
    d = O.make_config(vocab=211, width=56, eps=3e-4, side=10, layers=("latent2", "gla", "latent", "gla"), ffs=("moe", None, "dense", "moe"),
                      gla=dict(heads=3, dim=6, vdim=14, tau=5.5), dense_ff=72,
                      latent=dict(heads=5, dim=12, rot_dim=6, vdim=14, kv_rank=20, scale=0.77, base=777.0,
                                  scaling=dict(factor=3.0, original=64, fast=16.0, slow=2.0)),
                      latent2=dict(heads=4, dim=10, rot_dim=12, vdim=8, kv_rank=24, scale=0.11, base=123.0),
                      moe=dict(ff=24, experts=9, identity=3, top=4, scale=2.5, shared=40))
    d.pop("_rank")
    c = DamilixConfig.from_dict(d)
    st, specs = c.stream_spec(), c.layer_specs()
    assert st.kind == "post_norm" and c.norm_eps == 3e-4 and c.side_dim == 10 and (c.vocab_size, c.hidden_size, c.num_hidden_layers) == (211, 56, 4)
    b, g, a = specs[0].mixers[0], specs[1].mixers[0], specs[2].mixers[0]
    assert (a.kind, a.heads, a.kv_heads, a.dim, a.rot_dim, a.rot_dims, a.vdim, a.kv_rank, a.scale, a.rot_base, a.rot_layout) == \
        ("latent_attention", 5, 1, 12, 6, 6, 14, 20, 0.77, 777.0, "interleaved")
    assert a.rot_scaling == dict(factor=3.0, original=64, fast=16.0, slow=2.0) and a.head_sink and a.head_gate
    assert (b.kind, b.heads, b.dim, b.rot_dim, b.vdim, b.kv_rank, b.scale, b.rot_base, b.rot_layout, b.rot_scaling) == \
        ("latent_attention", 4, 10, 12, 8, 24, 0.11, 123.0, "half", None)
    assert (g.kind, g.heads, g.kv_heads, g.dim, g.vdim, g.tau) == ("gla", 3, 3, 6, 14, 5.5)
    m = specs[0]
    assert (m.ff, m.ff_kind, m.ff_act, m.experts, m.identity_experts, m.top, m.route, m.route_scale, m.shared_ff, m.shared_gate, m.side_dim) == \
        (24, "moe", "swiglu", 9, 3, 4, "softmax_all", 2.5, 40, True, 10)
    assert specs[1].ff == 0 and (specs[2].ff, specs[2].ff_kind, specs[2].ff_act) == (72, "dense", "swiglu")
    assert DamilixConfig.from_dict(c.to_dict()).to_dict() == c.to_dict()
    shapes = c.tensor_shapes()
    assert "l1.norm2" not in shapes and shapes["side.embed"] == (211, 40) and shapes["l0.mlp.router"] == (12, 56)
    d2 = O.make_config(side=0, moe=dict(shared=0, identity=0))
    d2.pop("_rank")
    c2 = DamilixConfig.from_dict(d2)
    assert not any("side" in n or "shared" in n for n in c2.tensor_shapes()) and c2.layer_specs()[1].identity_experts == 0


def test_unknown_layer_or_feed_forward_is_refused():
    from nanorlhf_b200.models.damilix import DamilixConfig
    d = O.make_config()
    d["layers"][0]["type"] = "ssm"
    with pytest.raises(ValueError):
        DamilixConfig.from_dict(d)
    d = O.make_config()
    d["layers"][0]["mlp"]["kind"] = "glu"
    with pytest.raises(ValueError):
        DamilixConfig.from_dict(d)
    d = O.make_config(latent=dict(rot_dim=4, dims=6))
    with pytest.raises(ValueError):
        DamilixConfig.from_dict(d)


def test_tensor_inventory_matches_the_oracle_weights_and_round_trips(tmp_path):
    from nanorlhf_b200.models.damilix import DamilixConfig
    from nanorlhf_b200.models.registry import load_model
    d = O.make_config(layers=("gla", "latent", "latent2", "gla"), ffs=("dense", "moe", None, "moe"), rank=7)
    W = O.random_weights(d, seed=1)
    shapes = DamilixConfig.from_dict(d).tensor_shapes(gla_rank=7)
    assert set(shapes) == set(W) and all(tuple(W[n].shape) == tuple(s) for n, s in shapes.items())
    path = _save(tmp_path, d, W)
    m = load_model(path, torch_dtype=torch.bfloat16)                 # the decay projection's inner width comes from the tensors
    assert tuple(m.tensor("l0.mix.a1").shape) == (7, 48) and torch.equal(m.tensor("l1.mix.sink"), W["l1.mix.sink"])
    m.save_pretrained(os.path.join(str(tmp_path), "again"))
    m2 = load_model(os.path.join(str(tmp_path), "again"))
    assert all(torch.equal(m.tensor(n), m2.tensor(n)) for n in m.names)
    extra = dict(W)
    extra["l2.norm2"] = torch.ones(48)                              # a norm of a feed-forward the layer does not have: not read
    del extra["l1.mlp.correction"]                                  # no correction: the scores alone choose
    m3 = load_model(_save(tmp_path, d, extra, "extra"))
    assert not m3.has_tensor("l2.norm2") and not m3.has_tensor("l1.mlp.correction")
    bad = dict(W)
    bad["l1.mix.uk"] = bad["l1.mix.uk"][:-1]
    with pytest.raises(ValueError):
        load_model(_save(tmp_path, d, bad, "bad"))
    bad = dict(W)
    bad["l0.mix.a2"] = bad["l0.mix.a2"][:, :-1]
    with pytest.raises(ValueError):
        load_model(_save(tmp_path, d, bad, "bad2"))
    bad = dict(W)
    del bad["l1.mix.sink"]
    with pytest.raises(ValueError):
        load_model(_save(tmp_path, d, bad, "bad3"))


def test_random_init_from_config():
    from nanorlhf_b200.models.damilix import DamilixConfig, DamilixForCausalLM
    d = O.make_config()
    d.pop("_rank")
    m = DamilixForCausalLM.from_config(DamilixConfig.from_dict(d), seed=3)
    assert all(torch.isfinite(m.tensor(n).float()).all() for n in m.names)


def test_frequency_table_of_the_engine_matches_the_oracle():
    """The engine's frequency table (float64 on the host) against the oracle's angles; with and without the stretch."""
    from nanorlhf_b200.ops.hybrid import rotary_frequencies
    for rot in (dict(base=10000.0, dims=8), dict(base=5e5, dims=12, scaling=dict(factor=2.5, original=512, fast=16.0, slow=2.0)),
                dict(base=500.0, dims=6, scaling=dict(factor=8.0, original=40, fast=4.0, slow=0.5))):
        f, mult = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        cos, sin = O.rotary_tables(rot, torch.tensor([0, 1, 37]))
        want_mult = 0.1 * math.log(rot["scaling"]["factor"]) + 1.0 if rot.get("scaling") else 1.0
        assert abs(mult - want_mult) < 1e-15
        a = torch.tensor([0.0, 1.0, 37.0], dtype=torch.float64)[:, None] * torch.tensor(f, dtype=torch.float64)[None]
        assert (torch.cos(a) * mult - cos).abs().max() < 1e-12 and (torch.sin(a) * mult - sin).abs().max() < 1e-12
    f, _ = rotary_frequencies(12, 5e5, dict(factor=2.5, original=512, fast=16.0, slow=2.0))
    plain = [5e5 ** (-2.0 * i / 12) for i in range(6)]
    assert f[0] == plain[0] and abs(f[-1] - plain[-1] / 2.5) < 1e-18       # fast pairs keep their frequency, slow ones are divided


# ---- the oracle's own invariants -------------------------------------------------------------------------------------
def test_oracle_is_causal_and_rotation_depends_on_distance_only():
    d = O.make_config(layers=("latent", "gla", "latent2"))
    W = O.random_weights(d, seed=5)
    toks = [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11]
    full = O.forward(W, d, toks)
    assert (O.forward(W, d, toks[:6]) - full[:6]).abs().max() < 1e-9
    # scores of rotated parts depend on the distance of the two positions only
    x = torch.randn(1, 8, dtype=torch.float64)
    y = torch.randn(1, 8, dtype=torch.float64)
    for layout in ("interleaved", "half"):
        rot = dict(base=100.0, dims=8)
        def score(pq, pk):
            cq, sq = O.rotary_tables(rot, torch.tensor([pq]))
            ck, sk = O.rotary_tables(rot, torch.tensor([pk]))
            return float((O.rotate(x, cq, sq, layout) * O.rotate(y, ck, sk, layout)).sum())
        assert abs(score(9, 4) - score(105, 100)) < 1e-9 and abs(score(9, 4) - score(9, 5)) > 1e-6


def test_oracle_sink_takes_mass_and_identity_experts_pass_the_input():
    d = O.make_config(layers=("latent",), ffs=("moe",), moe=dict(experts=2, identity=2, top=4, shared=0, scale=1.0))
    W = {k: v.double() for k, v in O.random_weights(d, seed=6).items()}
    h = torch.randn(5, d["width"], dtype=torch.float64)
    # every expert chosen: the identity experts' share of the input is their softmax mass
    s = torch.softmax(h @ W["l0.mlp.router"].T, -1)
    want = sum(s[:, e:e + 1] * O.swiglu(W, f"l0.mlp.e{e}.", h) for e in range(2)) + s[:, 2:].sum(-1, keepdim=True) * h
    assert (O.moe(W, "l0.mlp.", d["layers"][0]["mlp"], h) - want).abs().max() < 1e-9
    # a huge sink silences the head; a very negative one is ordinary softmax attention
    m = d["layers"][0]["mixer"]
    W["l0.mix.sink"] = torch.full_like(W["l0.mix.sink"], 60.0)
    assert O.latent_attention(W, "l0.mix.", m, h, 1e-5, "interleaved").abs().max() < 1e-12
    W["l0.mix.sink"] = torch.full_like(W["l0.mix.sink"], -60.0)
    a = O.latent_attention(W, "l0.mix.", m, h[:1], 1e-5, "interleaved")      # one token: the whole weight on itself
    c = O.rms((h[:1] @ W["l0.mix.dkv"].T)[:, :m["kv_rank"]], 1e-5) * W["l0.mix.dkv.norm"]
    v = (c @ W["l0.mix.uv"].T).reshape(1, m["heads"], m["vdim"]) * torch.sigmoid(h[:1] @ W["l0.mix.g"].T)[:, :, None]
    assert (a - v.reshape(1, -1) @ W["l0.mix.o"].T).abs().max() < 1e-9


def test_oracle_gla_state_decays_per_channel():
    d = O.make_config(layers=("gla",), ffs=(None,))
    W = {k: v.double() for k, v in O.random_weights(d, seed=7).items()}
    m = d["layers"][0]["mixer"]
    h = torch.randn(6, d["width"], dtype=torch.float64)
    W["l0.mix.a2.b"] = torch.full_like(W["l0.mix.a2.b"], -200.0)           # decay 0: every token sees only itself
    W["l0.mix.a2"] = torch.zeros_like(W["l0.mix.a2"])
    got = O.gla(W, "l0.mix.", m, h, 1e-5)
    assert all((got[t] - O.gla(W, "l0.mix.", m, h[t:t + 1], 1e-5)[0]).abs().max() < 1e-9 for t in range(6))
