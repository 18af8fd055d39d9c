"""Lukarax without a GPU: configuration, tensor shapes, registry, checkpoint round trip, the host-side tables of the serving
path against the oracle's formulas, and the oracle's own consistency."""
import json
import math
import os

import pytest
import torch

import lukarax_oracle as O
from nanorlhf_b200.models.lukarax import LukaraxConfig, LukaraxForCausalLM
from nanorlhf_b200.models.registry import load_model, resolve, sampler_kind


def test_config_shapes_and_specs():
    cfg = O.make_config()
    c = LukaraxConfig.from_dict(cfg)
    assert {n: tuple(s) for n, s in c.tensor_shapes(rel_buckets=10).items()} == O.tensor_shapes(cfg, 10)
    specs = c.layer_specs()
    assert [len(s.mixers) for s in specs] == [2, 1, 1, 1, 2]
    assert specs[3].mixers[0].kv_from == 2 and specs[2].mixers[0].kv_from == -1
    assert specs[1].mixers[0].values_from_keys and specs[1].mixers[0].head_sink and specs[1].mixers[0].rot_layout == "half"
    assert specs[2].mixers[0].maps == 2 and specs[2].mixers[0].rot_layout == "interleaved"
    assert specs[0].mixers[0].rot_dims == 0 and specs[0].mixers[0].keep_first == 5 and specs[0].mixers[1].kind == "mlstm"
    assert specs[1].route_groups == 4 and specs[1].route_keep == 2 and specs[1].identity_experts == 3 and specs[4].ff == 0
    st = c.stream_spec()
    assert st.kind == "hyper" and st.streams == 3 and st.tied_head and st.hyper_weights
    assert LukaraxConfig.from_dict(c.to_dict()).to_dict() == c.to_dict()
    plain = LukaraxConfig.from_dict(O.make_config(streams=None))
    assert plain.stream_spec().streams == 1 and not plain.stream_spec().hyper_weights
    assert not any(".hc" in n for n in plain.tensor_shapes())


@pytest.mark.parametrize("edit,msg", [(lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
                                      (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
                                      (lambda c: c["layers"][3]["mixer"].update(vdim=8), "kv_from"),
                                      (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
                                      (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
                                      (lambda c: c["layers"][1]["mlp"]["router"]["groups"].update(count=3), "groups"),
                                      (lambda c: c["layers"][2]["mixer"].update(heads=3), "multiple")])
def test_config_errors(edit, msg):
    cfg = O.make_config()
    edit(cfg)
    with pytest.raises(ValueError, match=msg):
        LukaraxConfig.from_dict(cfg)


def test_registry_and_checkpoint_round_trip(tmp_path):
    cfg = O.make_config(layers=("parallel", "attention_2", "attention", "shared"), ffs=("moe", None, "dense", "moe"))
    assert resolve(cfg)[0] is LukaraxForCausalLM
    model = LukaraxForCausalLM.from_config(LukaraxConfig.from_dict(cfg), torch.float32, "cpu", seed=3, rel_buckets=12)
    path = os.path.join(str(tmp_path), "m")
    model.save_pretrained(path)
    again = load_model(path, torch_dtype=torch.float32)
    assert sampler_kind(again) == "hybrid" and again.names == model.names
    assert again.tensor("l0.mix.left.rel").shape == (12, cfg["layers"][0]["mixer"]["left"]["heads"])
    for n in model.names:
        assert torch.equal(again.tensor(n), model.tensor(n))
    with open(os.path.join(path, "config.json")) as f:
        assert json.load(f)["layers"] == cfg["layers"]
    logits = O.forward({n: model.tensor(n).detach() for n in model.names}, cfg, [1, 2, 3, 4, 5])      # random weights of the product run
    assert torch.isfinite(logits).all()


@pytest.mark.parametrize("B,D", [(10, 40), (24, 200), (4, 6), (7, 17), (2, 5), (16, 1000)])
def test_distance_table_matches_buckets(B, D):
    from nanorlhf_b200.ops.hybrid import distance_bias_table
    rel = torch.randn(B, 3)
    table = distance_bias_table(rel, D)
    assert table.shape == (D + 1, 3)
    for n in list(range(D + 1)):
        assert torch.equal(table[n], rel[O.distance_bucket(n, B, D)])
    for n in (D + 1, 5 * D, 10 ** 6):                     # from bias_max on the last bucket holds
        assert O.distance_bucket(n, B, D) == B - 1 and torch.equal(table[D], rel[B - 1])


@pytest.mark.parametrize("scaling", [None, dict(factor=6.0, original=512, fast=16.0, slow=2.0), dict(factor=1.5, original=20, fast=3.0, slow=1.0)])
def test_rotary_frequencies_match_oracle(scaling):
    from nanorlhf_b200.ops.hybrid import rotary_frequencies
    rot = {"dims": 24, "base": 3e4, **({"scaling": scaling} if scaling else {})}
    f, mult = rotary_frequencies(24, 3e4, scaling)
    pos = torch.tensor([0, 1, 17, 4000])
    cos, sin = O.rotary_tables(rot, pos)
    a = pos.double()[:, None] * torch.tensor(f, dtype=torch.float64)[None, :]
    assert torch.allclose(torch.cos(a) * mult, cos, atol=1e-12) and torch.allclose(torch.sin(a) * mult, sin, atol=1e-12)


def test_oracle_matrix_memory_carries_its_state():
    g = torch.Generator().manual_seed(0)
    T, H, d, dv = 23, 2, 6, 5
    q, k, v = (torch.randn(T, H, n, generator=g, dtype=torch.float64) for n in (d, d, dv))
    ig, fg = torch.randn(T, H, generator=g, dtype=torch.float64) * 3, -torch.rand(T, H, generator=g, dtype=torch.float64)
    whole, _ = O.matrix_memory_core(q, k, v, ig, fg)
    a, st = O.matrix_memory_core(q[:9], k[:9], v[:9], ig[:9], fg[:9])
    b, _ = O.matrix_memory_core(q[9:], k[9:], v[9:], ig[9:], fg[9:], st)
    assert torch.allclose(torch.cat([a, b]), whole, atol=1e-12)


def test_oracle_router_groups():
    """A group that is not among the best stays closed even when its experts' scores beat chosen ones inside kept groups."""
    w = {"r.router": torch.eye(6, dtype=torch.float64) * 4.0, "r.correction": torch.tensor([0.0, 0.0, 0.0, 0.0, -0.5, -0.5], dtype=torch.float64)}
    mlp = {"router": {"experts": 4, "identity": 2, "top": 2, "scale": 1.0, "groups": {"count": 3, "keep": 1}}}
    h = torch.zeros(1, 6, dtype=torch.float64)
    h[0, 0], h[0, 2] = 1.0, 0.9                                   # best group {0, 1}; expert 2 scores above expert 1 but is closed
    ids, wt = O.route(w, "r.", mlp, h)
    assert sorted(ids[0].tolist()) == [0, 1] and abs(float(wt.sum()) - 1.0) < 1e-9
