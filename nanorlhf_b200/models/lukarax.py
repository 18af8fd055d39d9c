"""Lukarax: a decoder over several residual streams (hyper-connections) whose layers mix rotated attention in three forms
with a matrix memory, and feed dense or grouped mixture-of-experts feed-forwards.

* Embedding: every one of ``streams`` copies starts as ``embed[token] * embedding.scale``.
* Sublayer q of a layer (1: mixer, 2: feed-forward): ``u = sum_s hc<q>.in[s] x_s``, ``y = sublayer(layernorm(u))`` (weight ``norm<q>``, bias
  ``norm<q>.b``), then all streams at once ``x_t <- sum_s hc<q>.mix[s, t] x_s + hc<q>.out[t] y``.  A config without ``streams`` has one
  stream and the plain residual sum.
* ``attention`` mixer: differential attention.  q and k hold two score maps per head ([map 1, map 2] head by head), rotated on
  interleaved pairs; both maps are causal softmax attentions over the same values; ``o = a_1 - lambda a_2`` with
  ``lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff``, RMS-normed per head, times ``1 - diff``; the concatenated heads times
  ``sigmoid(g h)``; output projection.  With ``kv_from: j`` the layer has no key / value projections and reads layer j's pages.
* ``attention_2`` mixer: biased q / k projections, values = the keys as projected; rotation on (i, i + dims / 2) pairs with a
  frequency-dependent stretch; q and k divided by their root mean square after the rotation; capped scores
  ``softcap * tanh(s / softcap)``; a sliding window; a sink per head in the softmax denominator; biased output projection.
* ``parallel`` mixer: ``left_scale * left + right_scale * right`` of two mixers reading the same input.  Left: unrotated attention
  over a sliding window that also keeps the first positions, with a learned bias per (distance bucket, head).  Right: a matrix
  memory with exponential gates and a running maximum (mLSTM), per-head RMS norm, weight, sigmoid gate.
* Feed-forward: SwiGLU; or routed SwiGLU experts plus identity experts, chosen by softmax score + ``correction`` among the
  experts of the best ``groups.keep`` of ``groups.count`` groups, weights = chosen scores / their sum * ``scale``.
* Output: layer norm (``final.norm``) of the streams' sum; ``logits = embed x``.

This module holds the configuration (every size and constant is read from ``config.json`` or a tensor's shape) and the
checkpoint tensors under their own names; it describes the layers as generic specs (models/hybrid_spec.py) that the step
engine (sampler/hybrid_sampler.py) executes.  There is no forward loop here.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from .hybrid_spec import LayerSpec, MixerSpec, StreamSpec, TensorModel
from .registry import register_model

LAYER_TYPES = ("attention", "attention_2", "parallel")


def _rot_fields(rot: Optional[dict], layout: str) -> dict:
    if not rot or not int(rot.get("dims", 0)):
        return dict(rot_dims=0)
    return dict(rot_dims=int(rot["dims"]), rot_base=float(rot["base"]), rot_layout=layout,
                rot_scaling=dict(rot["scaling"]) if rot.get("scaling") else None)


@dataclass
class LukaraxConfig:
    vocab: int = 256
    width: int = 128
    norm_eps: float = 1e-6
    embed_scale: float = 1.0
    streams: Optional[int] = None                            # None: one stream, plain residual sum, no hc tensors
    layers: List[dict] = field(default_factory=list)         # the checkpoint's own layer descriptions
    model_type: str = "lukarax"
    architecture: str = "Lukarax"
    pad_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    max_positions: int = 1 << 30                             # positions are rotations and distances: nothing bounds a sequence's length

    @classmethod
    def from_dict(cls, d: dict) -> "LukaraxConfig":
        layers = list(d["layers"])
        for i, layer in enumerate(layers):
            if layer["type"] not in LAYER_TYPES:
                raise ValueError(f"layer {i}: unknown layer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") not in ("dense", "moe"):
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            m = layer["mixer"]
            att = m["left"] if layer["type"] == "parallel" else m
            if int(att["heads"]) % int(att["kv_heads"]):
                raise ValueError(f"layer {i}: heads must be a multiple of kv_heads")
            rot = att.get("rot")
            if rot and (int(rot["dims"]) % 2 or int(rot["dims"]) > int(att["dim"])):
                raise ValueError(f"layer {i}: rot.dims must be even and at most dim")
            src = m.get("kv_from")
            if src is not None:
                if layer["type"] != "attention" or not 0 <= int(src) < i or layers[int(src)]["type"] != "attention" or \
                        layers[int(src)]["mixer"].get("kv_from") is not None:
                    raise ValueError(f"layer {i}: kv_from must name an earlier attention layer with projections of its own")
                o = layers[int(src)]["mixer"]
                if any(o[k] != m[k] for k in ("kv_heads", "dim", "vdim")) or o.get("rot") != m.get("rot"):
                    raise ValueError(f"layer {i}: kv_from layer {src} has other key / value sizes or another rotation")
            if mlp is not None and mlp["kind"] == "moe":
                r = mlp["router"]
                n_out, g = int(r["experts"]) + int(r.get("identity", 0)), r.get("groups")
                if g and (n_out % int(g["count"]) or int(g["keep"]) * (n_out // int(g["count"])) < int(r["top"])):
                    raise ValueError(f"layer {i}: the router's groups do not fit its outputs")
        emb = d.get("embedding") or {}
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(d["norm"]["eps"]), embed_scale=float(emb.get("scale", 1.0)),
                   streams=int(d["streams"]) if d.get("streams") is not None else None, layers=layers,
                   pad_token_id=d.get("pad_token_id"), eos_token_id=d.get("eos_token_id"))

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "embedding": {"scale": self.embed_scale}, "layers": self.layers,
               "norm": {"eps": self.norm_eps}, "vocab": self.vocab, "width": self.width}
        if self.streams is not None:
            out["streams"] = self.streams
        for k in ("pad_token_id", "eos_token_id"):
            if getattr(self, k) is not None:
                out[k] = getattr(self, k)
        return out

    @classmethod
    def from_pretrained(cls, path: str) -> "LukaraxConfig":
        with open(os.path.join(path, "config.json")) as f:
            return cls.from_dict(json.load(f))

    # ---- names the engines share with the other model families ----
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    def stream_spec(self) -> StreamSpec:
        return StreamSpec(kind="hyper", positions=False, embed_scale=self.embed_scale, streams=self.streams or 1,
                          hyper_weights=self.streams is not None, tied_head=True)

    def layer_specs(self) -> List[LayerSpec]:
        specs = []
        for i, layer in enumerate(self.layers):
            m, p = layer["mixer"], f"l{i}.mix."
            if layer["type"] == "attention":
                src = m.get("kv_from")
                mixers = [MixerSpec("rot_attention", p, heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]),
                                    vdim=int(m["vdim"]), scale=float(m["scale"]), maps=2, diff=float(m["diff"]), out_gate=True,
                                    kv_from=-1 if src is None else int(src), **_rot_fields(m.get("rot"), "interleaved"))]
            elif layer["type"] == "attention_2":
                mixers = [MixerSpec("rot_attention", p, heads=int(m["heads"]), kv_heads=int(m["kv_heads"]), dim=int(m["dim"]),
                                    vdim=int(m["dim"]), scale=float(m["scale"]), window=int(m["mask"]["size"]), qk_bias=True, out_bias=True,
                                    unit_qk_norm=True, values_from_keys=True, softcap=float(m.get("softcap", 0.0)), head_sink=True,
                                    **_rot_fields(m.get("rot"), "half"))]
            else:
                a, r = m["left"], m["right"]
                mixers = [MixerSpec("rot_attention", p + "left.", out_scale=float(m["left_scale"]), heads=int(a["heads"]),
                                    kv_heads=int(a["kv_heads"]), dim=int(a["dim"]), vdim=int(a["vdim"]), scale=float(a["scale"]),
                                    window=int(a["mask"]["size"]), keep_first=int(a["mask"].get("keep_first", 0)),
                                    bias_max=int(a["bias_max"]), rot_dims=0),
                          MixerSpec("mlstm", p + "right.", out_scale=float(m["right_scale"]), heads=int(r["heads"]), kv_heads=int(r["heads"]),
                                    dim=int(r["dim"]), vdim=int(r["vdim"]), gate_cap=float(r["gate_cap"]))]
            spec = LayerSpec(i, mixers)
            mlp = layer.get("mlp")
            if mlp is not None and mlp["kind"] == "dense":
                spec.ff, spec.ff_act = int(mlp["ff"]), "swiglu"
            elif mlp is not None:
                r, g = mlp["router"], mlp["router"].get("groups")
                spec.ff, spec.ff_act, spec.ff_kind = int(mlp["expert"]["ff"]), "swiglu", "moe"
                spec.experts, spec.top = int(r["experts"]), int(r["top"])
                spec.route, spec.route_scale = "softmax_all", float(r.get("scale", 1.0))
                spec.identity_experts = int(r.get("identity", 0))
                if g:
                    spec.route_groups, spec.route_keep = int(g["count"]), int(g["keep"])
            specs.append(spec)
        return specs

    def tensor_shapes(self, rel_buckets: int = 32) -> Dict[str, tuple]:
        """Name -> shape of every checkpoint tensor.  ``rel_buckets``: rows of the distance-bias tables, which the config does not
        name: a checkpoint's own tensors give them."""
        W, S = self.width, self.streams
        out: Dict[str, tuple] = {"embed": (self.vocab, W)}
        for spec in self.layer_specs():
            p = f"l{spec.index}."
            for q in ("1", "2") if spec.ff else ("1",):
                out[p + "norm" + q], out[p + "norm" + q + ".b"] = (W,), (W,)
            for m in spec.mixers:
                x = m.prefix
                if m.kind == "mlstm":
                    nk, nv = m.heads * m.dim, m.heads * m.vdim
                    out.update({x + "q": (nk, W), x + "k": (nk, W), x + "v": (nv, W), x + "g": (nv, W), x + "o": (W, nv), x + "norm": (nv,),
                                x + "i": (m.heads, W), x + "i.b": (m.heads,), x + "f": (m.heads, W), x + "f.b": (m.heads,)})
                    continue
                nq, nk = m.maps * m.heads * m.dim, m.maps * m.kv_heads * m.dim
                out[x + "q"] = (nq, W)
                if m.qk_bias:
                    out[x + "q.b"] = (nq,)
                if m.kv_from < 0:
                    out[x + "k"] = (nk, W)
                    if m.qk_bias:
                        out[x + "k.b"] = (nk,)
                    if not m.values_from_keys:
                        out[x + "v"] = (m.kv_heads * m.vdim, W)
                if m.bias_max:
                    out[x + "rel"] = (rel_buckets, m.heads)
                if m.head_sink:
                    out[x + "sink"] = (m.heads,)
                if m.maps == 2:
                    for n in ("lq1", "lk1", "lq2", "lk2"):
                        out[x + n] = (m.dim,)
                if m.out_gate:
                    out[x + "g"] = (m.heads * m.vdim, W)
                out[x + "o"] = (W, m.heads * m.vdim)
                if m.out_bias:
                    out[x + "o.b"] = (W,)
            f = p + "mlp."
            if spec.ff and spec.ff_kind == "dense":
                out.update({f + "gate": (spec.ff, W), f + "up": (spec.ff, W), f + "down": (W, spec.ff)})
            elif spec.ff:
                for e in range(spec.experts):
                    out.update({f"{f}e{e}.gate": (spec.ff, W), f"{f}e{e}.up": (spec.ff, W), f"{f}e{e}.down": (W, spec.ff)})
                n_out = spec.experts + spec.identity_experts
                out[f + "router"], out[f + "correction"] = (n_out, W), (n_out,)
            if S is not None:
                for q in ("1", "2") if spec.ff else ("1",):
                    out.update({f"{p}hc{q}.in": (S,), f"{p}hc{q}.out": (S,), f"{p}hc{q}.mix": (S, S)})
        out["final.norm"], out["final.norm.b"] = (W,), (W,)
        return out


@register_model("Lukarax", "lukarax", sampler="hybrid")
class LukaraxForCausalLM(TensorModel):
    """Lukarax checkpoint tensors under their own names; executed by ``sampler.hybrid_sampler.HybridSampler``."""
    config_class = LukaraxConfig

    @staticmethod
    def free_shape(name: str) -> bool:
        return name.endswith(".rel")                       # the number of distance buckets is the checkpoint's choice

    @classmethod
    def from_pretrained(cls, path: str, torch_dtype=torch.bfloat16, device="cpu", **kw):
        cfg = LukaraxConfig.from_pretrained(path)
        from .hf_io import load_state_dict
        sd = load_state_dict(os.path.join(path, "model.safetensors"))
        want = cfg.tensor_shapes()
        # a router without a score correction is a router whose correction is zero
        want = {n: s for n, s in want.items() if n in sd or not n.endswith("mlp.correction")}
        missing = [n for n in want if n not in sd]
        if missing:
            raise ValueError(f"checkpoint does not fit its config: missing {missing[:4]}")
        shapes = {}
        for n, shp in want.items():
            shapes[n] = tuple(sd[n].shape)
            if cls.free_shape(n):
                if len(shapes[n]) != 2 or shapes[n][1] != shp[1] or shapes[n][0] < 2:
                    raise ValueError(f"tensor {n}: shape {shapes[n]} does not fit the config")
            elif shapes[n] != tuple(shp):
                raise ValueError(f"tensor {n}: shape {shapes[n]} does not fit the config ({tuple(shp)})")
        model = cls(cfg, shapes, dtype=torch_dtype, device=device)
        with torch.no_grad():
            for n in model.names:
                model.tensor(n).copy_(sd[n].to(torch_dtype))
        return model

    @staticmethod
    def init_value(n: str, t: torch.Tensor, g: torch.Generator) -> torch.Tensor:
        """Random weights (benchmarks, smoke tests): projections ~ N(0, 1/fan_in), gains around 1, stream weights near a plain residual."""
        leaf = n.rsplit(".", 1)[-1]
        if ".hc" in n:
            if leaf == "mix":
                return torch.eye(t.shape[0]) + torch.randn(t.shape, generator=g) * 0.05
            if leaf == "in":
                return torch.full(t.shape, 1.0 / t.shape[0]) + torch.randn(t.shape, generator=g) * 0.05
            return torch.ones(t.shape) + torch.randn(t.shape, generator=g) * 0.05
        if leaf == "rel":
            return torch.randn(t.shape, generator=g) * 0.5
        if t.dim() == 2:
            if leaf == "embed":
                return torch.randn(t.shape, generator=g) * 0.5
            return torch.randn(t.shape, generator=g) / (t.shape[1] ** 0.5)
        if leaf == "b":
            if n.endswith("f.b"):
                return torch.rand(t.shape, generator=g) * 3.0 + 1.0          # forget gates that keep most of the state
            return torch.randn(t.shape, generator=g) * 0.1
        if leaf in ("sink", "lq1", "lk1", "lq2", "lk2"):
            return torch.randn(t.shape, generator=g) * (1.0 if leaf == "sink" else 0.1)
        if leaf == "correction":
            return torch.randn(t.shape, generator=g) * 0.02
        return torch.rand(t.shape, generator=g) * 0.5 + 0.75                # norm weights
