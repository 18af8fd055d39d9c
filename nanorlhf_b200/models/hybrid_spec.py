"""What the step engine (sampler/hybrid_sampler.py) needs to know about a hybrid decoder: generic descriptions of its token
mixers, feed-forwards and residual stream, and a module that holds checkpoint tensors under their own names.

A model family (models/nezavik.py, models/vilosun.py) turns its ``config.json`` into these specs; the engine executes them
with the kernels of ``ops/hybrid.py``.  Model files contain no forward loop.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch
import torch.nn as nn

from .hf_io import load_state_dict, save_state_dict


@dataclass
class MixerSpec:
    """One token mixer of a layer.  ``kind``: window_attention | conv_attention | ssd | gated_delta | latent_attention | gla |
    rot_attention | mlstm.  ``prefix``: tensor-name prefix."""
    kind: str
    prefix: str
    out_scale: float = 1.0
    heads: int = 0
    kv_heads: int = 0            # key/value heads (attention), q/k heads (delta rule), groups (ssd)
    dim: int = 0                 # query/key size per head; state size N (ssd)
    vdim: int = 0                # value size per head
    window: int = 0              # attention: keys seen, the token itself included (mask "window"); chunk length (mask "chunk")
    scale: float = 1.0           # attention: score multiplier
    conv: int = 0                # taps of the short causal convolution
    norm_groups: int = 1         # ssd: equal parts of the gated RMS norm
    per_channel: bool = False    # delta rule: decay per head and key channel + low-rank sigmoid gate
    # conv_attention (biased projections, short convolution on q / k / v, no q / k norm, no rotation):
    mask: str = "window"         # "window": the last `window` keys; "chunk": the keys of the query's own chunk of `window` positions
    slope_exp: float = 0.0       # > 0: head h's score loses 2^(-slope_exp (h + 1) / heads) per position of distance
    head_temp: bool = False      # learned score multiplier per head (tensor "temp")
    head_gate: bool = False      # head output times sigmoid of a per-head projection of the mixer's input (tensor "g")
    v_blend: int = -1            # -1: none; else the layer whose values this layer's values are blended with (tensor "vmix"),
                                 # its own index for the layer that only provides them
    # latent_attention (keys and values of all heads are projections "uk" / "uv" of one RMS-normed latent of `kv_rank` columns per
    # token, plus one rotated key part of `rot_dim` columns shared by the heads; only the latent and that part are cached;
    # `dim` is the unrotated query/key size per head; causal; `head_gate` and `head_sink` as below):
    kv_rank: int = 0
    rot_dim: int = 0             # rotated query/key columns per head, behind the `dim` unrotated ones
    rot_dims: int = 0            # how many of the rot_dim columns turn (the rest pass unchanged)
    rot_base: float = 10000.0    # frequency i of rot_dims / 2 is rot_base^(-2 i / rot_dims)
    rot_layout: str = "interleaved"   # "interleaved": column 2i turns with 2i + 1;  "half": i with i + rot_dims / 2
    rot_scaling: Optional[dict] = None  # frequency-dependent stretch {"factor", "original", "fast", "slow"} with its cos / sin multiplier
    head_sink: bool = False      # the softmax denominator also holds exp(sink_h) (tensor "sink"): a score with no key and no value
    # gla (gated linear attention, S = diag(decay) S + k v^T, o = S^T q D^-1/2; decay = sigmoid(a2 (a1 h) + a2.b)^(1 / tau) per key channel):
    tau: float = 1.0
    # rot_attention (projections q / k / v with grouped heads; the first `rot_dims` columns of every head rotated (`rot_base`, `rot_layout`,
    # `rot_scaling`; 0: no rotation); `window` keys seen (0: all earlier ones); `head_sink` as above; and the optional terms below):
    qk_bias: bool = False        # biases on the q and k projections (tensors "q.b", "k.b")
    out_bias: bool = False       # bias on the output projection (tensor "o.b")
    unit_qk_norm: bool = False   # q and k divided by their root mean square per head after the rotation (no weight)
    values_from_keys: bool = False   # no v projection: the values are the keys as projected (bias included), before rotation and norm
    softcap: float = 0.0         # > 0: score <- softcap * tanh(score / softcap)
    keep_first: int = 0          # > 0: the first positions of a sequence stay visible behind the window
    bias_max: int = 0            # > 0: a learned bias per (distance bucket, head) is added to the score (tensor "rel" [buckets, heads]);
                                 # the first half of the buckets hold one distance each, the others grow logarithmically up to bias_max
    maps: int = 1                # 2: differential attention, q and k hold two score maps per head over the same values (tensors lq1, lk1,
                                 # lq2, lk2 [dim]): o = a_1 - lambda a_2 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff, RMS-normed per
                                 # head, times (1 - diff)
    diff: float = 0.0
    out_gate: bool = False       # the concatenated heads times sigmoid(g h), element by element (tensor "g" [heads * vdim, W])
    kv_from: int = -1            # >= 0: no k / v projections; the layer reads the pages of that earlier layer
    # mlstm (matrix memory with exponential gates: log gates i = cap tanh((i h + i.b) / cap), f = logsigmoid(cap tanh((f h + f.b) / cap));
    # m' = max(f + m, i); S = exp(f + m - m') S + exp(i - m') k v^T, n likewise with k; o = S^T q / (max(|n . q|, exp(-m')) + 1e-6) with
    # q scaled by dim^-1/2; per-head RMS norm, weight "norm", sigmoid gate "g"):
    gate_cap: float = 0.0


@dataclass
class LayerSpec:
    index: int
    mixers: List[MixerSpec]
    ff: int = 0                  # 0: no feed-forward; else its inner width (of one expert for "moe")
    ff_act: str = "relu2"        # "relu2": W_down relu(W_up h)^2;  "swiglu": W_down (silu(W_gate h) * W_up h)
    ff_kind: str = "dense"       # "dense" | "moe" (experts e0.., top-k router)
    experts: int = 0
    top: int = 0
    route: str = "softmax_top"   # "softmax_top": the largest logits (+ bias "router.b"), weights = softmax over the chosen logits
                                 # "softmax_all": scores = softmax over all router outputs, chosen by score + "correction",
                                 #                weights = the chosen scores / their sum * route_scale
    route_scale: float = 1.0
    route_groups: int = 1        # "softmax_all": > 1: the router outputs form that many equal groups of neighbours and only experts of the
    route_keep: int = 1          # `route_keep` groups with the largest choice score can be chosen
    identity_experts: int = 0    # router outputs behind the `experts` real ones whose expert returns its input
    shared_ff: int = 0           # > 0: a SwiGLU expert of this width for every token (tensors "shared.*")
    shared_gate: bool = False    # its result times sigmoid(shared.sg h), one number per token
    side_dim: int = 0            # > 0: per-layer token input after the feed-forward (stream kind "post_norm"): columns
                                 # [index * side_dim, (index + 1) * side_dim) of the table "side.embed", gated by gelu_tanh(side.gate x),
                                 # projected by side.proj, RMS-normed with side.norm and added


@dataclass
class StreamSpec:
    """How layers read and write the residual stream, and what surrounds them.

    ``kind`` "depth_weighted": every layer reads one single-gain RMS norm of a learned weighted sum of all earlier results and
    adds ``mixer + ff`` of it (tensors norm1, dwa).  ``kind`` "sandwich": ``x += norm1b(g1 * mixer(norm1 x))`` then
    ``x += norm2b(g2 * ff(norm2 x))`` with group RMS norms (a weight per column) and, when ``gated_residual``, sigmoid gates
    ``g = sigmoid(rg h + rg.b)`` of the sublayer's input.  ``kind`` "post_norm": sublayers read the stream itself and only their
    result is normed, ``x += norm1(mixer(x))`` then ``x += norm2(ff(x))`` (single-group RMS norms with a weight per column); the
    embedding is normed too (tensor "embed.norm").  ``kind`` "hyper": ``streams`` copies of the stream (all equal to the embedding at
    the start); sublayer q of a layer reads ``layernorm(sum_s hc<q>.in[s] x_s)`` (weight norm<q>, bias norm<q>.b) and every stream becomes
    ``x_t <- sum_s hc<q>.mix[s, t] x_s + hc<q>.out[t] y``; the output reads the layer norm of the streams' sum (``hyper_weights`` False:
    one stream with the plain residual sum, no hc tensors)."""
    kind: str = "depth_weighted"
    norm_groups: int = 1
    gated_residual: bool = False
    embed_scale: float = 1.0
    positions: bool = True                      # learned position vectors added to the embedding (tensor "pos")
    pair_buckets: int = 0                       # > 0: hashed (previous token, token) embedding rows (tensor "bigram")
    pair_mul_prev: int = 0
    pair_mul_cur: int = 0
    logit_scale: float = 1.0
    streams: int = 1                            # "hyper": copies of the residual stream
    hyper_weights: bool = True                  # "hyper": the layers carry hc1 / hc2 tensors
    tied_head: bool = False                     # logits = embed x (the table itself, without embed_scale); no "head" tensor


def _mangle(name: str) -> str:
    return name.replace(".", "__")


class TensorModel(nn.Module):
    """Holds the checkpoint tensors (``tensor(name)``) of a hybrid decoder; executed by ``sampler.hybrid_sampler.HybridSampler``.

    Subclasses set ``config_class`` (with ``from_pretrained`` / ``to_dict`` / ``layer_specs`` / ``stream_spec`` /
    ``tensor_shapes``) and may override ``free_shape`` (tensors whose shape the config does not fix) and ``init_value``."""
    config_class = None
    int_tensors = ()                            # names stored as int32

    def __init__(self, cfg, shapes: Optional[Dict[str, tuple]] = None, dtype=torch.bfloat16, device="cpu"):
        super().__init__()
        self.config = cfg
        shapes = shapes or cfg.tensor_shapes()
        self.names = list(shapes)
        self.weights = nn.ParameterDict({_mangle(n): nn.Parameter(torch.empty(shapes[n], dtype=dtype, device=device),
                                                                  requires_grad=False) for n in self.names})

    def tensor(self, name: str) -> torch.Tensor:
        return self.weights[_mangle(name)]

    def has_tensor(self, name: str) -> bool:
        return _mangle(name) in self.weights

    def layer_specs(self) -> List[LayerSpec]:
        return self.config.layer_specs()

    def stream_spec(self) -> StreamSpec:
        return self.config.stream_spec()

    @property
    def device(self):
        return next(self.parameters()).device

    @property
    def dtype(self):
        return next(self.parameters()).dtype

    @staticmethod
    def free_shape(name: str) -> bool:
        return False

    # ---- checkpoint I/O (config.json + model.safetensors, tensors under their own names) ----
    @classmethod
    def from_pretrained(cls, path: str, torch_dtype=torch.bfloat16, device="cpu", **_):
        cfg = cls.config_class.from_pretrained(path)
        sd = load_state_dict(os.path.join(path, "model.safetensors"))
        want = cfg.tensor_shapes()
        missing = [n for n in want if n not in sd]
        extra = [n for n in sd if n not in want]
        if missing or extra:
            raise ValueError(f"checkpoint does not fit its config: missing {missing[:4]}, unexpected {extra[:4]}")
        shapes = {n: tuple(sd[n].shape) for n in want}
        for n, shp in want.items():
            if shapes[n] != tuple(shp) and not cls.free_shape(n):
                raise ValueError(f"tensor {n}: shape {shapes[n]} does not fit the config ({tuple(shp)})")
        model = cls(cfg, shapes, dtype=torch_dtype, device=device)
        with torch.no_grad():
            for n in model.names:
                model.tensor(n).copy_(sd[n].to(torch_dtype))
        return model

    def save_pretrained(self, path: str):
        os.makedirs(path, exist_ok=True)
        with open(os.path.join(path, "config.json"), "w") as f:
            json.dump(self.config.to_dict(), f, indent=1)
        save_state_dict({n: self.tensor(n) for n in self.names}, os.path.join(path, "model.safetensors"))

    @staticmethod
    def init_value(name: str, t: torch.Tensor, g: torch.Generator) -> torch.Tensor:
        raise NotImplementedError

    @classmethod
    def from_config(cls, cfg, torch_dtype=torch.bfloat16, device="cpu", seed: Optional[int] = None, **shape_kw):
        """Random weights (benchmarks, smoke tests)."""
        model = cls(cfg, cfg.tensor_shapes(**shape_kw), dtype=torch_dtype, device=device)
        g = torch.Generator(device="cpu")
        g.manual_seed(0 if seed is None else seed)
        with torch.no_grad():
            for n in model.names:
                t = model.tensor(n)
                t.copy_(cls.init_value(n, t, g).to(torch_dtype))
        return model
