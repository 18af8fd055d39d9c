"""Damilix: a decoder whose layers mix latent attention and gated linear attention, with dense or mixture-of-experts
feed-forwards and a per-layer token input, on a stream that norms only what a sublayer returns.

* Embedding: ``x = rmsnorm(embed[token]) * embed.norm``.
* Layer: ``x += rmsnorm(mixer(x)) * norm1``, then ``x += rmsnorm(ff(x)) * norm2`` (if the layer has a feed-forward), then the token
  input ``y = side.proj (gelu_tanh(side.gate x) * side.embed[token][slice of the layer])``, ``x += rmsnorm(y) * side.norm``.
  Sublayers read ``x`` itself.
* ``latent_attention`` / ``latent_attention_2`` mixers: per head ``dim`` unrotated and ``rot_dim`` rotated query columns; one
  projection ``dkv`` gives a latent of ``kv_rank`` columns (RMS-normed, ``dkv.norm``) and one rotated key part shared by all heads;
  unrotated keys ``uk latent`` and values ``uv latent`` per head; causal softmax of ``(q.k) * scale`` whose denominator also holds
  ``exp(sink_h)``; a sigmoid gate per head (``g``); output projection ``o``.  The first rotates interleaved pairs and may stretch
  its frequencies (``rot.scaling``), the second rotates (i, i + dims / 2) pairs.  Only the latent and the shared key part are cached.
* ``gla`` mixer: ``S = diag(alpha) S + k v^T``, ``o = S^T q dim^-1/2`` per head with ``alpha = sigmoid(a2 (a1 h) + a2.b)^(1 / tau)`` per
  key channel; per-head RMS norm with a shared weight, times ``silu(g h)``, output projection.
* Feed-forward: SwiGLU; or ``experts`` SwiGLU experts plus ``identity`` experts that return their input, routed by a softmax over
  all router outputs (choice by score + ``correction``, weights = chosen scores / their sum * ``scale``), plus a shared expert
  times ``sigmoid(shared.sg h)``.
* Output: ``logits = head (rmsnorm(x) * final.norm)``.

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

LAYER_TYPES = {"latent_attention": "interleaved", "latent_attention_2": "half", "gla": None}


@dataclass
class DamilixConfig:
    vocab: int = 256
    width: int = 128
    norm_eps: float = 1e-6
    side_dim: int = 0                                        # 0: no per-layer token input
    layers: List[dict] = field(default_factory=list)         # the checkpoint's own layer descriptions
    model_type: str = "damilix"
    architecture: str = "Damilix"
    pad_token_id: Optional[int] = None
    eos_token_id: Optional[int] = None
    max_positions: int = 1 << 30                             # positions are rotations: nothing bounds a sequence's length

    @classmethod
    def from_dict(cls, d: dict) -> "DamilixConfig":
        for i, layer in enumerate(d["layers"]):
            if layer["type"] not in LAYER_TYPES:
                raise ValueError(f"layer {i}: unknown layer type {layer['type']!r}")
            mlp = layer.get("mlp")
            if mlp is not None and mlp.get("kind") not in ("dense", "moe"):
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp.get('kind')!r}")
            m = layer["mixer"]
            if layer["type"] != "gla":
                rot = m["rot"]
                if int(rot["dims"]) % 2 or int(rot["dims"]) > int(m["rot_dim"]):
                    raise ValueError(f"layer {i}: rot.dims must be even and at most rot_dim")
        side = d.get("token_side") or {}
        return cls(vocab=int(d["vocab"]), width=int(d["width"]), norm_eps=float(d["norm"]["eps"]), side_dim=int(side.get("dim", 0)),
                   layers=list(d["layers"]), pad_token_id=d.get("pad_token_id"), eos_token_id=d.get("eos_token_id"))

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "layers": self.layers, "norm": {"eps": self.norm_eps}, "vocab": self.vocab,
               "width": self.width}
        if self.side_dim:
            out["token_side"] = {"dim": self.side_dim}
        for k in ("pad_token_id", "eos_token_id"):
            if getattr(self, k) is not None:
                out[k] = getattr(self, k)
        return out

    @classmethod
    def from_pretrained(cls, path: str) -> "DamilixConfig":
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
        return StreamSpec(kind="post_norm", positions=False)

    def layer_specs(self) -> List[LayerSpec]:
        specs = []
        for i, layer in enumerate(self.layers):
            m, p = layer["mixer"], f"l{i}.mix."
            if layer["type"] == "gla":
                mixer = MixerSpec("gla", p, heads=int(m["heads"]), kv_heads=int(m["heads"]), dim=int(m["dim"]), vdim=int(m["vdim"]),
                                  tau=float(m["tau"]))
            else:
                rot = m["rot"]
                mixer = MixerSpec("latent_attention", p, heads=int(m["heads"]), kv_heads=1, dim=int(m["dim"]), vdim=int(m["vdim"]),
                                  scale=float(m["scale"]), kv_rank=int(m["kv_rank"]), rot_dim=int(m["rot_dim"]), rot_dims=int(rot["dims"]),
                                  rot_base=float(rot["base"]), rot_layout=LAYER_TYPES[layer["type"]],
                                  rot_scaling=dict(rot["scaling"]) if rot.get("scaling") else None, head_gate=True, head_sink=True)
            spec = LayerSpec(i, [mixer], side_dim=self.side_dim)
            mlp = layer.get("mlp")
            if mlp is not None and mlp["kind"] == "dense":
                spec.ff, spec.ff_act = int(mlp["ff"]), "swiglu"
            elif mlp is not None:
                r, sh = mlp["router"], mlp.get("shared")
                spec.ff, spec.ff_act, spec.ff_kind = int(mlp["expert"]["ff"]), "swiglu", "moe"
                spec.experts, spec.top = int(r["experts"]), int(r["top"])
                spec.route, spec.route_scale = "softmax_all", float(r.get("scale", 1.0))
                spec.identity_experts = int(r.get("identity", 0))
                if sh:
                    spec.shared_ff, spec.shared_gate = int(sh["ff"]), True
            specs.append(spec)
        return specs

    def tensor_shapes(self, gla_rank: int = 16) -> Dict[str, tuple]:
        """Name -> shape of every checkpoint tensor.  ``gla_rank``: inner width of the decay projection (a1 / a2), which the
        config does not name: a checkpoint's own tensors give it."""
        W = self.width
        out: Dict[str, tuple] = {"embed": (self.vocab, W), "embed.norm": (W,)}
        if self.side_dim:
            out["side.embed"] = (self.vocab, len(self.layers) * self.side_dim)
        for spec in self.layer_specs():
            p = f"l{spec.index}."
            out[p + "norm1"] = (W,)
            if spec.ff:
                out[p + "norm2"] = (W,)
            m = spec.mixers[0]
            q = m.prefix
            if m.kind == "gla":
                nk, nv = m.heads * m.dim, m.heads * m.vdim
                out.update({q + "q": (nk, W), q + "k": (nk, W), q + "v": (nv, W), q + "g": (nv, W), q + "o": (W, nv), q + "norm": (m.vdim,),
                            q + "a1": (gla_rank, W), q + "a2": (nk, gla_rank), q + "a2.b": (nk,)})
            else:
                out.update({q + "q": (m.heads * (m.dim + m.rot_dim), W), q + "dkv": (m.kv_rank + m.rot_dim, W), q + "dkv.norm": (m.kv_rank,),
                            q + "uk": (m.heads * m.dim, m.kv_rank), q + "uv": (m.heads * m.vdim, m.kv_rank), q + "sink": (m.heads,),
                            q + "g": (m.heads, W), q + "o": (W, m.heads * m.vdim)})
            f = p + "mlp."
            if spec.ff and spec.ff_kind == "dense":
                out.update({f + "gate": (spec.ff, W), f + "up": (spec.ff, W), f + "down": (W, spec.ff)})
            elif spec.ff:
                for e in range(spec.experts):
                    out.update({f"{f}e{e}.gate": (spec.ff, W), f"{f}e{e}.up": (spec.ff, W), f"{f}e{e}.down": (W, spec.ff)})
                n_out = spec.experts + spec.identity_experts
                out[f + "router"], out[f + "correction"] = (n_out, W), (n_out,)
                if spec.shared_ff:
                    out.update({f + "shared.gate": (spec.shared_ff, W), f + "shared.up": (spec.shared_ff, W),
                                f + "shared.down": (W, spec.shared_ff), f + "shared.sg": (1, W)})
            if self.side_dim:
                out.update({p + "side.gate": (self.side_dim, W), p + "side.proj": (W, self.side_dim), p + "side.norm": (W,)})
        out["final.norm"] = (W,)
        out["head"] = (self.vocab, W)
        return out


@register_model("Damilix", "damilix", sampler="hybrid")
class DamilixForCausalLM(TensorModel):
    """Damilix checkpoint tensors under their own names; executed by ``sampler.hybrid_sampler.HybridSampler``."""
    config_class = DamilixConfig

    @staticmethod
    def free_shape(name: str) -> bool:
        return name.endswith(".mix.a1") or name.endswith(".mix.a2")     # their inner width is the checkpoint's choice

    @classmethod
    def from_pretrained(cls, path: str, torch_dtype=torch.bfloat16, device="cpu", **kw):
        cfg = DamilixConfig.from_pretrained(path)
        from .hf_io import load_state_dict
        sd = load_state_dict(os.path.join(path, "model.safetensors"))
        want = cfg.tensor_shapes()
        # a router without a score correction is a router whose correction is zero; tensors the config gives no use for
        # (the second norm of a layer without a feed-forward) are not read
        want = {n: s for n, s in want.items() if n in sd or not n.endswith("mlp.correction")}
        missing = [n for n in want if n not in sd]
        if missing:
            raise ValueError(f"checkpoint does not fit its config: missing {missing[:4]}")
        shapes = {}
        for n, shp in want.items():
            shapes[n] = tuple(sd[n].shape)
            if shapes[n] != tuple(shp) and not cls.free_shape(n):
                raise ValueError(f"tensor {n}: shape {shapes[n]} does not fit the config ({tuple(shp)})")
        for spec in cfg.layer_specs():
            m, q = spec.mixers[0], spec.mixers[0].prefix
            if m.kind == "gla":
                a1, a2 = shapes[q + "a1"], shapes[q + "a2"]
                if len(a1) != 2 or len(a2) != 2 or a1[1] != cfg.width or a2[0] != m.heads * m.dim or a2[1] != a1[0]:
                    raise ValueError(f"tensors {q}a1 / {q}a2: shapes {a1} / {a2} do not fit the config")
        model = cls(cfg, shapes, dtype=torch_dtype, device=device)
        with torch.no_grad():
            for n in model.names:
                model.tensor(n).copy_(sd[n].to(torch_dtype))
        return model

    @staticmethod
    def init_value(n: str, t: torch.Tensor, g: torch.Generator) -> torch.Tensor:
        """Random weights (benchmarks, smoke tests): projections ~ N(0, 1/fan_in), gains around 1, decays in a useful range."""
        leaf = n.rsplit(".", 1)[-1]
        if t.dim() == 2:
            if leaf == "embed":
                return torch.randn(t.shape, generator=g)
            return torch.randn(t.shape, generator=g) / (t.shape[1] ** 0.5)
        if n.endswith("a2.b"):
            return torch.rand(t.shape, generator=g) * 4.0 + 1.0          # sigmoid(1..5)^(1/tau): slow decays
        if leaf == "sink":
            return torch.randn(t.shape, generator=g)
        if leaf == "correction":
            return torch.randn(t.shape, generator=g) * 0.02
        return torch.rand(t.shape, generator=g) * 0.5 + 0.75            # norm weights
