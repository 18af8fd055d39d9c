"""Step engine for hybrid decoders: layers that mix paged-KV attention with recurrent state (state-space scans, delta rules).

Where ``NativeSampler`` prefills whole prompts and then decodes one token per row, this engine runs STEPS: a step is a
batch of entries, each a run of consecutive tokens of one sequence -- a prompt portion of any length or a single decoded
token -- executed together by the same kernels.  That is what recurrent layers need (their state is carried from step to
step in a per-sequence slot) and it gives chunked prefill and continuous batching for free:

* sequences, KV pages (16 tokens) and state slots are owned by the C++ ``StepScheduler`` (csrc/runtime.cpp), which also
  builds each step's packed plan (token offsets, positions, KV slots, block tables, state slots) and runs the admission /
  token-budget policy of ``generate``;
* per layer the weights are fused into TWO matrices: every projection that reads the normed stream (q, k, v, state-space
  input, gates, decays, feed-forward up) is one GEMM, and every projection that writes the stream (attention out,
  state-space out, feed-forward down) is one GEMM over the concatenated activations, mixer scales folded into the
  activations;
* two kinds of residual stream (``StreamSpec.kind``): "depth_weighted" (one norm per layer, mixers and feed-forward side by
  side, the stream a learned weighted sum of all earlier results) and "sandwich" (a norm before and after each sublayer, a
  sigmoid gate on the sublayer's result; the mixer and the feed-forward are two stages, each with its own pair of fused
  matrices); a mixture-of-experts feed-forward runs only the chosen experts, rows sorted by expert through a grouped
  tcgen05 GEMM (float32 serving: dense form on cuBLAS);
* a third kind of stream, "post_norm", has sublayers that read the stream itself and norms only what they return; its
  layers may end with a gated per-layer token input (a third stage); its mixers are latent attention (one cached latent row
  per token serves all heads: queries are absorbed into the latent space before the paged attention kernel and the result
  is expanded per head after it) and gated linear attention (the delta-rule scan without the delta);
* a fourth kind, "hyper", keeps several copies of the stream that learned weights mix at every sublayer (hyper-connections) with a
  layer norm (weight and bias) in front of each sublayer; its mixers are rotated attention with optional terms (biases, unit norm of
  q / k, capped scores, a sink, kept first positions, a bias by distance bucket, values that are the keys, two differential score
  maps, pages borrowed from an earlier layer) and a matrix memory with exponential gates (mLSTM); its router may limit the choice to
  the best groups of experts;
* the residual stream, its depth-weighted average, norms, scores, softmax, decays and recurrent state are float32 in both
  serving modes; ``dtype="bf16"`` keeps GEMM operands and KV pages in bf16 (fp32 accumulation, fp32 GEMM results),
  ``dtype="fp32"`` keeps everything in float32 with TF32 off;
* ``generate`` has the call shape and sampling semantics of ``NativeSampler.generate`` (temperature, top-p, n samples per
  prompt, seeded per-row streams, EOS kept, right-padded).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..models.hybrid_spec import StreamSpec
from ..ops import gemm as _gemm, hybrid as hy, native


def _unwrap(model):
    m = getattr(model, "policy", model)
    return getattr(m, "base_model", m) if hasattr(m, "peft_config") else m


class StepPlan:
    """Device views of one step's packed plan (layout fixed by ``StepScheduler.plan``)."""
    __slots__ = ("E", "T", "max_blocks", "tokens", "cu", "tok_entry", "pos", "kv_slot", "start", "state_slot", "block_table")

    def __init__(self, buf: torch.Tensor, E: int, T: int, MB: int):
        self.E, self.T, self.max_blocks = E, T, MB
        o = 0

        def take(n):
            nonlocal o
            v = buf[o:o + n]
            o += n
            return v
        self.tokens, self.cu, self.tok_entry, self.pos, self.kv_slot = take(T), take(E + 1), take(T), take(T), take(T)
        self.start, self.state_slot = take(E), take(E)
        self.block_table = take(E * MB).view(E, MB)


class _Mixer:
    __slots__ = ("spec", "cols", "out_col", "out_size", "vec", "k_cache", "v_cache", "conv_state", "state", "w_lr2", "lr_cols", "rank",
                 "w_uk", "w_uv", "rot_mult", "aux_state", "lam", "owns_kv")


class _Layer:
    """One pair of fused matrices with what runs between them: a whole layer of a depth-weighted stream (mixers and the
    feed-forward side by side), or one sublayer of a sandwich stream (the mixer, or the feed-forward)."""
    __slots__ = ("spec", "gain", "dw", "w_in", "w_out", "mixers", "ff_col", "ff_out_col", "n_in", "k_out", "out_pad",
                 "w_pre", "w_post", "gate_col", "gate_bias", "router_col", "router_bias", "w_gate_up", "w_down",
                 "shared_col", "shared_out_col", "sg_col", "side_col", "side_out_col", "side_col0", "hc_in", "hc_out", "hc_mix", "w_pre_b",
                 "out_bias")


def _pad8(n: int) -> int:
    return (n + 7) // 8 * 8


class HybridSampler:
    PAGE = 16

    def __init__(self, model, dtype: str = "bf16", kv_block_size: int = 16, max_num_seqs: int = 64, pool_tokens: Optional[int] = None,
                 prefill_token_budget: int = 8192, gemm: str = "tc", rollout_dtype: Optional[str] = None,
                 use_cuda_graph: bool = True, moe: str = "auto", **_unused):
        if kv_block_size != self.PAGE:
            raise ValueError("KV pages hold 16 tokens")
        native.load()
        dtype = {"bfloat16": "bf16", "float32": "fp32"}.get(rollout_dtype or dtype, rollout_dtype or dtype)
        if dtype not in ("bf16", "fp32"):
            raise ValueError(f"unknown serving dtype {dtype!r}")
        self.model = model
        self.lm = _unwrap(model)
        self.cfg = self.lm.config
        self.device = next(self.lm.parameters()).device
        if self.device.type != "cuda":
            raise RuntimeError("the step engine runs on CUDA only")
        self.rollout_dtype = dtype
        self.fp32 = dtype == "fp32"
        self.wdtype = torch.float32 if self.fp32 else torch.bfloat16
        if self.fp32:                                     # true float32 products
            torch.backends.cuda.matmul.allow_tf32 = False
            torch.backends.cudnn.allow_tf32 = False
        self.gemm_backend = gemm
        if moe not in ("auto", "grouped", "dense"):
            raise ValueError(f"unknown mixture-of-experts form {moe!r}")
        self.moe_form = moe                                # "auto": grouped tcgen05 GEMM in bf16 when the sizes fit, else dense
        self.max_num_seqs = max_num_seqs
        self.pool_tokens = pool_tokens
        self.prefill_token_budget = prefill_token_budget
        self.sharded_sync = None
        self._weights_version = None
        self.layers: List[_Layer] = []
        self.sched = None
        self.num_blocks = 0
        self.stats = {"steps": 0, "tokens": 0, "decode_tokens": 0, "prefill_tokens": 0, "graph_replays": 0}
        self.use_cuda_graph = use_cuda_graph
        self._graphs: Dict[tuple, tuple] = {}             # (entries, block-table width) -> (graph, plan buffer, logits, launches)
        self._graph_seen: set = set()
        self._bt_width = 0                                # generate() fixes the block-table width so decode steps can be replayed
        self._build_arena()

    # ------------------------------------------------------------------------------------------
    # weights: two fused matrices per layer + float vectors
    # ------------------------------------------------------------------------------------------
    def _t(self, name):
        return self.lm.tensor(name).detach()

    def _f(self, name):
        return self._t(name).to(device=self.device, dtype=torch.float32).contiguous()

    @torch.no_grad()
    def _build_arena(self):
        lm, dev, wd = self.lm, self.device, self.wdtype
        W = self.cfg.width
        self.stream = lm.stream_spec() if hasattr(lm, "stream_spec") else StreamSpec()
        st = self.stream
        self.layers = []
        for spec in lm.layer_specs():
            p = f"l{spec.index}."
            if st.kind == "depth_weighted":               # one stage: mixers and feed-forward read the same norm
                L = self._build_stage(spec, spec.mixers, True)
                L.gain = self._f(p + "norm1").reshape(1)
                L.dw = self._f(p + "dwa")
                self.layers.append(L)
            elif st.kind == "sandwich":                   # two stages: the mixer, then the feed-forward, each between its norms
                for k, (mixers, ff) in enumerate(((spec.mixers, False), ([], True))):
                    if ff and not spec.ff:
                        continue
                    n = str(k + 1)
                    L = self._build_stage(spec, mixers, ff, gate=p + "rg" + n if st.gated_residual else None)
                    L.w_pre, L.w_post = self._f(p + "norm" + n), self._f(p + "norm" + n + "b")
                    self.layers.append(L)
            elif st.kind == "post_norm":                  # up to three stages: mixer, feed-forward, token input; only results are normed
                L = self._build_stage(spec, spec.mixers, False)
                L.w_post = self._f(p + "norm1")
                self.layers.append(L)
                if spec.ff:
                    L = self._build_stage(spec, [], True)
                    L.w_post = self._f(p + "norm2")
                    self.layers.append(L)
                if spec.side_dim:
                    L = self._build_stage(spec, [], False, side=True)
                    L.w_post = self._f(p + "side.norm")
                    self.layers.append(L)
            elif st.kind == "hyper":                      # two stages per layer, each behind its own layer norm and stream weights
                for k, (mixers, ff) in enumerate(((spec.mixers, False), ([], True))):
                    if ff and not spec.ff:
                        continue
                    n = str(k + 1)
                    L = self._build_stage(spec, mixers, ff)
                    L.w_pre = self._f(p + "norm" + n)
                    L.w_pre_b = self._f(p + "norm" + n + ".b") if lm.has_tensor(p + "norm" + n + ".b") else None
                    if st.hyper_weights:
                        L.hc_in, L.hc_out, L.hc_mix = (self._f(f"{p}hc{n}.{x}") for x in ("in", "out", "mix"))
                    self.layers.append(L)
            else:
                raise ValueError(f"unknown stream kind {st.kind!r}")
        self.embed_gain = self._f("embed.norm") if st.kind == "post_norm" else None
        self.side_table = (self._t("side.embed").to(device=dev, dtype=wd).contiguous()
                           if st.kind == "post_norm" and lm.has_tensor("side.embed") else None)
        self.embed = self._t("embed").to(device=dev, dtype=wd).contiguous()
        self.pos_table = self._t("pos").to(device=dev, dtype=wd).contiguous() if st.positions else None
        self.pair_table = self._t("bigram").to(device=dev, dtype=wd).contiguous() if st.pair_buckets else None
        self.final_gain = self._f("final.norm").reshape(1) if st.kind == "depth_weighted" else self._f("final.norm")
        self.final_bias = self._f("final.norm.b") if st.kind == "hyper" and lm.has_tensor("final.norm.b") else None
        V = self.cfg.vocab
        self.head = torch.zeros(_pad8(V), W, dtype=wd, device=dev)
        self.head[:V] = self._t("embed" if st.tied_head else "head").to(device=dev, dtype=wd)
        self._weights_version = self.weights_fingerprint()

    def _build_stage(self, spec, mixer_specs, with_ff: bool, gate: Optional[str] = None, side: bool = False) -> _Layer:
        """Fuse every projection that reads the stage's normed input into ``w_in`` and every projection that writes the stream
        into ``w_out``; keep the small vectors as float32."""
        dev, wd, W = self.device, self.wdtype, self.cfg.width
        p = f"l{spec.index}."
        L = _Layer()
        L.spec = spec
        L.gain = L.dw = L.w_pre = L.w_post = L.gate_col = L.gate_bias = L.router_col = L.router_bias = None
        L.w_gate_up = L.w_down = None
        L.shared_col = L.shared_out_col = L.sg_col = L.side_col = L.side_out_col = None
        L.hc_in = L.hc_out = L.hc_mix = L.w_pre_b = L.out_bias = None
        L.side_col0 = 0
        rows_in: List[torch.Tensor] = []
        cols_out: List[torch.Tensor] = []
        n_in = k_out = 0
        L.mixers = []

        def add_in(name):
            nonlocal n_in
            t = self._t(name) if isinstance(name, str) else name
            rows_in.append(t)
            c = (n_in, t.shape[0])
            n_in += t.shape[0]
            return c

        def pad_in():
            """Zero rows up to the next multiple of 8: what follows starts on a 32-byte boundary of the GEMM's float result."""
            nonlocal n_in
            if n_in % 8:
                rows_in.append(torch.zeros(8 - n_in % 8, W, dtype=self._t("embed").dtype, device=self._t("embed").device))
                n_in += rows_in[-1].shape[0]

        def add_out(name):
            nonlocal k_out
            t = self._t(name)
            cols_out.append(t)
            c = k_out
            k_out += t.shape[1]
            return c, t.shape[1]

        for ms in mixer_specs:
            M = _Mixer()
            M.spec, M.cols, M.vec = ms, {}, {}
            M.k_cache = M.v_cache = M.conv_state = M.state = M.w_lr2 = M.w_uk = M.w_uv = M.aux_state = None
            M.lam, M.owns_kv = 0.0, True
            q = ms.prefix
            if ms.kind == "window_attention":
                for n in ("q", "k", "v"):
                    M.cols[n] = add_in(q + n)
                M.vec["qw"], M.vec["kw"] = self._f(q + "q.norm"), self._f(q + "k.norm")
            elif ms.kind == "conv_attention":
                for n in ("q", "k", "v"):
                    M.cols[n] = add_in(q + n)
                if ms.head_gate:
                    M.cols["g"] = add_in(q + "g")
                M.vec["conv"] = torch.cat([self._f(q + n + ".conv") for n in ("q", "k", "v")], 0).contiguous()
                M.vec["in_bias"] = torch.cat([self._f(q + n + ".b") for n in ("q", "k", "v")], 0).contiguous()
                if ms.head_temp:
                    M.vec["temp"] = self._f(q + "temp")
                if ms.slope_exp > 0:
                    hs = torch.arange(1, ms.heads + 1, dtype=torch.float64)
                    M.vec["slope"] = torch.exp2(-ms.slope_exp * hs / ms.heads).to(device=dev, dtype=torch.float32)
                if ms.v_blend >= 0 and ms.v_blend != spec.index:
                    M.vec["vmix"] = self._f(q + "vmix").reshape(1)
            elif ms.kind == "ssd":
                M.cols["in"] = add_in(q + "in")
                for n in ("conv", "conv.b", "dt_bias", "A_log", "D", "norm"):
                    M.vec[n] = self._f(q + n)
            elif ms.kind == "gated_delta":
                for n in ("q", "k", "v", "b"):
                    M.cols[n] = add_in(q + n)
                if ms.per_channel:
                    M.cols["a1"], M.cols["g1"] = add_in(q + "a1"), add_in(q + "g1")
                    a2, g2 = self._t(q + "a2"), self._t(q + "g2")
                    r = a2.shape[1]
                    M.rank = r
                    na, ng = a2.shape[0], g2.shape[0]
                    w2 = torch.zeros(_pad8(na + ng), _pad8(2 * r), dtype=wd, device=dev)     # block diagonal: [a2 0; 0 g2]
                    w2[:na, :r] = a2.to(wd)
                    w2[na:na + ng, r:2 * r] = g2.to(wd)
                    M.w_lr2, M.lr_cols = w2, (na, ng)
                else:
                    M.cols["a"], M.cols["g"] = add_in(q + "a"), add_in(q + "g")
                M.vec["conv"] = torch.cat([self._f(q + n + ".conv") for n in ("q", "k", "v")], 0).contiguous()
                for n in ("dt_bias", "A_log", "norm"):
                    M.vec[n] = self._f(q + n)
            elif ms.kind == "latent_attention":
                for n in ("q", "dkv"):
                    M.cols[n] = add_in(q + n)
                if ms.head_gate:
                    M.cols["g"] = add_in(q + "g")
                M.vec["dkv.norm"] = self._f(q + "dkv.norm")
                if ms.head_sink:
                    M.vec["sink"] = self._f(q + "sink")
                freq, M.rot_mult = hy.rotary_frequencies(ms.rot_dims, ms.rot_base, ms.rot_scaling)
                M.vec["freq"] = torch.tensor(freq, dtype=torch.float64, device=dev)
                # per head: uk [dim, rank] takes a query into the latent space, uv^T [rank, vdim] expands the latent result
                M.w_uk = self._t(q + "uk").to(device=dev, dtype=wd).reshape(ms.heads, ms.dim, ms.kv_rank).contiguous()
                M.w_uv = self._t(q + "uv").to(device=dev, dtype=wd).reshape(ms.heads, ms.vdim, ms.kv_rank).transpose(1, 2).contiguous()
            elif ms.kind == "gla":
                for n in ("q", "k", "v", "g"):
                    M.cols[n] = add_in(q + n)
                M.cols["a1"] = add_in(q + "a1")
                a2 = self._t(q + "a2")
                M.rank = a2.shape[1]
                w2 = torch.zeros(_pad8(a2.shape[0]), _pad8(M.rank), dtype=wd, device=dev)
                w2[:a2.shape[0], :M.rank] = a2.to(wd)
                M.w_lr2 = w2
                M.vec["a2.b"], M.vec["norm"] = self._f(q + "a2.b"), self._f(q + "norm")
            elif ms.kind == "rot_attention":
                wq = self._t(q + "q")
                if ms.maps == 2:
                    # the two score maps become heads of their own: query rows [H, map, dim] are reordered to (key/value head, map,
                    # query head of the group), so that the kernels' grouping (consecutive query heads share a key head) pairs map m of
                    # a head with key head 2 g + m; the read side undoes the order
                    R = ms.heads // ms.kv_heads
                    wq = wq.reshape(ms.kv_heads, R, 2, ms.dim, W).permute(0, 2, 1, 3, 4).reshape(2 * ms.heads * ms.dim, W)
                M.cols["q"] = add_in(wq)
                M.owns_kv = ms.kv_from < 0
                if M.owns_kv:
                    M.cols["k"] = add_in(q + "k")
                    if not ms.values_from_keys:
                        M.cols["v"] = add_in(q + "v")
                if ms.out_gate:
                    M.cols["g"] = add_in(q + "g")
                if ms.qk_bias:
                    qb = self._f(q + "q.b")
                    if ms.maps == 2:
                        qb = qb.reshape(ms.kv_heads, ms.heads // ms.kv_heads, 2, ms.dim).permute(0, 2, 1, 3).reshape(-1).contiguous()
                    M.vec["q.b"] = qb
                    if M.owns_kv:
                        M.vec["k.b"] = self._f(q + "k.b")
                if ms.head_sink:
                    M.vec["sink"] = self._f(q + "sink")
                if ms.bias_max:                            # one row per distance 0 .. bias_max (the last one holds from there on)
                    M.vec["rel"] = hy.distance_bias_table(self._f(q + "rel"), ms.bias_max)
                if ms.rot_dims:
                    freq, M.rot_mult = hy.rotary_frequencies(ms.rot_dims, ms.rot_base, ms.rot_scaling)
                    M.vec["freq"] = torch.tensor(freq, dtype=torch.float64, device=dev)
                else:
                    M.rot_mult = 1.0
                if ms.maps == 2:
                    l1 = (self._t(q + "lq1").double() * self._t(q + "lk1").double()).sum().item()
                    l2 = (self._t(q + "lq2").double() * self._t(q + "lk2").double()).sum().item()
                    M.lam = math.exp(l1) - math.exp(l2) + ms.diff
                if ms.out_bias:
                    b = self._f(q + "o.b") * ms.out_scale
                    L.out_bias = b if L.out_bias is None else L.out_bias + b
            elif ms.kind == "mlstm":
                for n in ("q", "k", "v", "g", "i", "f"):
                    M.cols[n] = add_in(q + n)
                pad_in()
                for n in ("i.b", "f.b", "norm"):
                    M.vec[n] = self._f(q + n)
            else:
                raise ValueError(f"unknown mixer kind {ms.kind!r}")
            M.out_col, M.out_size = add_out(q + "o")
            L.mixers.append(M)
        L.ff_col = L.ff_out_col = None
        if with_ff and spec.ff:
            if spec.ff_kind == "dense" and spec.ff_act == "swiglu":      # [gate rows | up rows]
                c0 = add_in(p + "mlp.gate")[0]
                add_in(p + "mlp.up")
                L.ff_col = (c0, 2 * spec.ff)
                L.ff_out_col = add_out(p + "mlp.down")
            elif spec.ff_kind == "dense":
                L.ff_col = add_in(p + "mlp.up")
                L.ff_out_col = add_out(p + "mlp.down")
            elif spec.ff_kind == "moe" and self._moe_grouped(spec):
                # sorted-by-expert form: only the router rides in the fused matrix; the experts' matrices are stacked for the
                # grouped GEMM, [experts * 2 ff, W] (gate rows, then up rows) and [experts * W, ff]
                L.router_col = add_in(p + "mlp.router")
                L.router_bias = self._router_vector(spec, p)
                if spec.ff % 32 == 0:                      # gate / up rows interleaved: the SwiGLU is formed in the GEMM's epilogue
                    L.w_gate_up = torch.cat([hy.interleave_gate_up(self._t(f"{p}mlp.e{e}.gate").to(device=dev, dtype=wd),
                                                                   self._t(f"{p}mlp.e{e}.up").to(device=dev, dtype=wd))
                                             for e in range(spec.experts)], 0).contiguous()
                else:
                    L.w_gate_up = torch.cat([self._t(f"{p}mlp.e{e}.{n}").to(device=dev, dtype=wd) for e in range(spec.experts)
                                             for n in ("gate", "up")], 0).contiguous()
                L.w_down = torch.cat([self._t(f"{p}mlp.e{e}.down").to(device=dev, dtype=wd) for e in range(spec.experts)], 0).contiguous()
            elif spec.ff_kind == "moe":                   # dense form: router, then per expert its gate rows and its up rows
                L.router_col = add_in(p + "mlp.router")
                L.router_bias = self._router_vector(spec, p)
                c0 = n_in
                for e in range(spec.experts):
                    add_in(f"{p}mlp.e{e}.gate")
                    add_in(f"{p}mlp.e{e}.up")
                L.ff_col = (c0, n_in - c0)
                c0 = k_out
                for e in range(spec.experts):
                    add_out(f"{p}mlp.e{e}.down")
                L.ff_out_col = (c0, k_out - c0)
            else:
                raise ValueError(f"unknown feed-forward kind {spec.ff_kind!r}")
            if spec.ff_kind == "moe" and spec.shared_ff:     # an expert for every token: rides in the fused matrices like a dense one
                pad_in()
                c0 = add_in(p + "mlp.shared.gate")[0]
                add_in(p + "mlp.shared.up")
                L.shared_col = (c0, 2 * spec.shared_ff)
                if spec.shared_gate:
                    L.sg_col = add_in(p + "mlp.shared.sg")
                L.shared_out_col = add_out(p + "mlp.shared.down")
        if side:                                          # per-layer token input: gate projection in, projection to the stream out
            L.side_col = add_in(p + "side.gate")
            L.side_out_col = add_out(p + "side.proj")
            L.side_col0 = spec.index * spec.side_dim
        if gate is not None:
            L.gate_col = add_in(gate)
            L.gate_bias = self._f(gate + ".b") if self.lm.has_tensor(gate + ".b") else None
        L.n_in, L.k_out = _pad8(n_in), _pad8(k_out)
        L.out_pad = L.k_out != k_out
        L.w_in = torch.zeros(L.n_in, W, dtype=wd, device=dev)
        L.w_in[:n_in] = torch.cat([t.to(device=dev, dtype=wd) for t in rows_in], 0)
        L.w_out = torch.zeros(W, L.k_out, dtype=wd, device=dev)
        if cols_out:
            L.w_out[:, :k_out] = torch.cat([t.to(device=dev, dtype=wd) for t in cols_out], 1)
        return L

    def _router_vector(self, spec, p):
        """The vector added to the router's outputs before the choice: a bias on the logits, or a correction of the scores."""
        name = p + ("mlp.correction" if spec.route == "softmax_all" else "mlp.router.b")
        return self._f(name) if self.lm.has_tensor(name) else None

    def _moe_grouped(self, spec) -> bool:
        fits = not self.fp32 and self.cfg.width % 8 == 0 and spec.ff % 8 == 0
        if self.moe_form == "grouped" and not fits:
            raise ValueError("the grouped mixture-of-experts form needs bf16 serving and width / expert width that are multiples of 8")
        return fits and self.moe_form != "dense"

    def weights_fingerprint(self):
        return getattr(self.lm, "_nrl_version", 0)

    def sync_weights(self, force: bool = False):
        """Re-fuse the arena when the model's weights changed (the optimizer bumps ``_nrl_version``)."""
        if force or self._weights_version != self.weights_fingerprint():
            pools = [(M.k_cache, M.v_cache, M.conv_state, M.state, M.aux_state) for L in self.layers for M in L.mixers]
            self._graphs.clear()                          # captured graphs hold the old arena's addresses
            self._graph_seen.clear()
            self._build_arena()
            for M, pl in zip([M for L in self.layers for M in L.mixers], pools):
                M.k_cache, M.v_cache, M.conv_state, M.state, M.aux_state = pl

    def release(self):
        self._graphs.clear()
        self._graph_seen.clear()
        self.layers, self.sched, self.num_blocks = [], None, 0

    # ------------------------------------------------------------------------------------------
    # cache pages and state slots
    # ------------------------------------------------------------------------------------------
    def reset_pool(self, pool_tokens: int, num_slots: int):
        """(Re)build the page pool for ``pool_tokens`` tokens and ``num_slots`` state slots; all sequences are dropped."""
        from .. import _C
        dev, wd = self.device, self.wdtype
        n = max(1, (pool_tokens + self.PAGE - 1) // self.PAGE)
        f32 = dict(dtype=torch.float32, device=dev)
        for L in self.layers:
            for M in L.mixers:
                ms = M.spec
                if ms.kind == "window_attention":
                    M.k_cache = torch.zeros(n, ms.kv_heads, self.PAGE, ms.dim, dtype=wd, device=dev)
                    M.v_cache = torch.zeros(n, ms.kv_heads, self.PAGE, ms.vdim, dtype=wd, device=dev)
                elif ms.kind == "conv_attention":
                    M.k_cache = torch.zeros(n, ms.kv_heads, self.PAGE, ms.dim, dtype=wd, device=dev)
                    M.v_cache = torch.zeros(n, ms.kv_heads, self.PAGE, ms.vdim, dtype=wd, device=dev)
                    ch = ms.heads * ms.dim + ms.kv_heads * (ms.dim + ms.vdim)
                    M.conv_state = torch.zeros(num_slots, ms.conv - 1, ch, **f32)
                elif ms.kind == "latent_attention":       # one row per token: [normed latent | rotated shared key part]
                    M.k_cache = torch.zeros(n, 1, self.PAGE, ms.kv_rank + ms.rot_dim, dtype=wd, device=dev)
                elif ms.kind == "gla":
                    M.state = torch.zeros(num_slots, ms.heads, ms.dim, ms.vdim, **f32)
                elif ms.kind == "rot_attention":
                    if M.owns_kv:                          # every score map has key heads of its own; the values are shared by the maps
                        M.k_cache = torch.zeros(n, ms.maps * ms.kv_heads, self.PAGE, ms.dim, dtype=wd, device=dev)
                        M.v_cache = torch.zeros(n, ms.kv_heads, self.PAGE, ms.vdim, dtype=wd, device=dev)
                elif ms.kind == "mlstm":                   # S with the normaliser n as column vdim (rows padded to 32 bytes); the running maximum
                    M.state = torch.zeros(num_slots, ms.heads, ms.dim, _pad8(ms.vdim + 1), **f32)
                    M.aux_state = torch.zeros(num_slots, ms.heads, **f32)
                elif ms.kind == "ssd":
                    ch = ms.heads * ms.vdim + 2 * ms.kv_heads * ms.dim
                    M.conv_state = torch.zeros(num_slots, ms.conv - 1, ch, **f32)
                    M.state = torch.zeros(num_slots, ms.heads, ms.dim, ms.vdim, **f32)
                else:
                    ch = 2 * ms.kv_heads * ms.dim + ms.heads * ms.vdim
                    M.conv_state = torch.zeros(num_slots, ms.conv - 1, ch, **f32)
                    M.state = torch.zeros(num_slots, ms.heads, ms.dim, ms.vdim, **f32)
        for L in self.layers:                             # layers that read an earlier layer's pages
            for M in L.mixers:
                if M.spec.kind == "rot_attention" and not M.owns_kv:
                    src = next(m for l in self.layers if l.spec.index == M.spec.kv_from for m in l.mixers if m.spec.kind == "rot_attention")
                    M.k_cache, M.v_cache = src.k_cache, src.v_cache
        # the last token of every sequence (hashed pair embedding): part of a sequence's state like the convolution taps
        self.prev_token = torch.zeros(num_slots, dtype=torch.int32, device=dev) if self.stream.pair_buckets else None
        self.num_blocks, self.num_slots = n, num_slots
        self._graphs.clear()                              # captured graphs hold the old pool's addresses
        self._graph_seen.clear()
        self.sched = _C.StepScheduler(n, self.PAGE, num_slots)

    def open(self, reserve_tokens: int = 0) -> int:
        """Admit a sequence: it gets a state slot now and KV pages as its tokens arrive."""
        return self.sched.open(reserve_tokens)

    def close(self, sid: int):
        """Give the sequence's pages and state slot back."""
        self.sched.close(sid)

    # ------------------------------------------------------------------------------------------
    # the step
    # ------------------------------------------------------------------------------------------
    def _mm(self, x, w):
        """x [T, K] . w [N, K]^T -> float32 [T, N]."""
        if self.fp32:
            return torch.mm(x, w.t())
        if (self.gemm_backend == "tc" and x.shape[1] % 64 == 0 and w.shape[0] % 8 == 0 and x.is_contiguous() and w.is_contiguous()
                and x.data_ptr() % 16 == 0):
            out = torch.empty(x.shape[0], w.shape[0], dtype=torch.float32, device=x.device)
            _gemm.gemm(x, w, out_f32=out)                 # tcgen05 GEMM with the float32 epilogue (csrc/gemm_tc.cu)
            return out
        return torch.mm(x, w.t(), out_dtype=torch.float32)

    @torch.no_grad()
    def step(self, entries: Sequence[Tuple[int, Sequence[int], Sequence[int]]]) -> torch.Tensor:
        """Run one batch.  ``entries``: (sequence id, its next tokens, indices among them whose logits are wanted).
        Returns float32 logits [wanted, vocab] in entry order."""
        sids = [int(e[0]) for e in entries]
        counts = [len(e[1]) for e in entries]
        data, E, T, MB = self.sched.plan(sids, counts, self._bt_width)
        o, rows = 0, []
        for (_sid, toks, want), c in zip(entries, counts):
            data[o:o + c] = np.asarray(toks, dtype=np.int32)
            rows += [o + int(j) for j in want]
            o += c
        self.stats["steps"] += 1
        self.stats["tokens"] += T
        if self.use_cuda_graph and self._bt_width and T == E and len(rows) == T:
            return self._decode_step_graphed(data, E, MB)
        plan = StepPlan(torch.from_numpy(data).to(self.device), E, T, MB)
        return self._forward(plan, rows)

    def _decode_step_graphed(self, data, E: int, MB: int) -> torch.Tensor:
        """A step of single tokens (one per sequence, all logits wanted) has the same launches whatever the sequences hold:
        the second time a batch size shows up its launches are captured into a CUDA graph, from then on a step is one copy
        of the plan and one replay.  (The first time runs eagerly: it is a real step, and it warms up lazy kernel setup.)"""
        key = (E, MB)
        entry = self._graphs.get(key)
        if entry is None:
            if key not in self._graph_seen:
                self._graph_seen.add(key)
                return self._forward(StepPlan(torch.from_numpy(data).to(self.device), E, E, MB), list(range(E)))
            buf = torch.from_numpy(data).to(self.device)
            torch.cuda.synchronize(self.device)
            g = torch.cuda.CUDAGraph()
            n0 = native.launches()
            with torch.cuda.graph(g, capture_error_mode="thread_local"):
                logits = self._forward(StepPlan(buf, E, E, MB), list(range(E)))
            if len(self._graphs) >= 16:
                self._graphs.pop(next(iter(self._graphs)))
            entry = self._graphs[key] = (g, buf, logits, native.launches() - n0)
        else:
            entry[1].copy_(torch.from_numpy(data))
        entry[0].replay()
        native._count(entry[3])
        self.stats["graph_replays"] += 1
        return entry[2]

    def _forward(self, plan: StepPlan, rows: List[int]) -> torch.Tensor:
        if self.stream.kind == "sandwich":
            return self._forward_sandwich(plan, rows)
        if self.stream.kind == "post_norm":
            return self._forward_post_norm(plan, rows)
        if self.stream.kind == "hyper":
            return self._forward_hyper(plan, rows)
        return self._forward_depth_weighted(plan, rows)

    def _run_mixers(self, L, U, A, plan, eps, ctx=None):
        for M in L.mixers:
            out = A[:, M.out_col:M.out_col + M.out_size]
            kind = M.spec.kind
            if kind == "latent_attention":
                self._latent_attention(M, U, plan, eps, out)
            elif kind == "gla":
                self._gla(M, U, plan, eps, out)
            elif kind == "rot_attention":
                self._rot_attention(M, U, plan, eps, out)
            elif kind == "mlstm":
                self._mlstm(M, U, plan, eps, out)
            elif kind == "conv_attention":
                self._conv_attention(M, U, plan, out, ctx, L.spec.index)
            elif kind == "gated_delta":
                self._gated_delta(M, U, plan, eps, out)
            elif kind == "window_attention":
                self._window_attention(M, U, plan, eps, out)
            else:
                self._ssd(M, U, plan, eps, out)

    def _forward_post_norm(self, plan: StepPlan, rows: List[int], keep: Optional[list] = None) -> torch.Tensor:
        """Stream whose sublayers read x itself: ``x += rmsnorm(sublayer(x)) * w``.  One fused kernel per stage boundary norms the
        stage's result, adds it and hands the new x to the next stage as GEMM operand (the last one applies the final norm).
        ``keep``: a list that receives a copy of the stream after every layer."""
        cfg, dev, wd = self.cfg, self.device, self.wdtype
        T, W, eps = plan.T, cfg.width, cfg.norm_eps
        f32 = dict(dtype=torch.float32, device=dev)
        x = torch.empty(T, W, **f32)
        h = torch.empty(T, W, dtype=wd, device=dev)
        hy.embed_norm(self.embed, plan.tokens, self.embed_gain, eps, x, h)
        ctx: Dict[int, torch.Tensor] = {}
        for i, L in enumerate(self.layers):
            U = self._mm(h, L.w_in)                                                   # [T, n_in] float
            A = (torch.zeros if L.out_pad else torch.empty)(T, L.k_out, dtype=wd, device=dev)
            self._run_mixers(L, U, A, plan, eps, ctx)
            self_w = None
            if L.side_col is not None:
                (c, n), (oc, on) = L.side_col, L.side_out_col
                hy.side_gate(U[:, c:c + n], self.side_table, L.side_col0, plan.tokens, A[:, oc:oc + on], n)
            if L.shared_col is not None:
                (c, n), (oc, on) = L.shared_col, L.shared_out_col
                hy.swiglu_cols(U[:, c:c + n], U[:, L.sg_col[0]:L.sg_col[0] + 1] if L.sg_col is not None else None, A[:, oc:oc + on])
            if L.ff_col is not None:
                self_w = self._feed_forward(L, U, A)
            o = self._mm(A, L.w_out) if L.k_out else None                             # [T, W] float
            if L.w_gate_up is not None:
                o, self_w = self._experts_grouped(L, U, h, o, want_self=True)
            last = i + 1 == len(self.layers)
            hy.post_norm_residual(x, o, self_w, L.w_post, self.final_gain if last else None, eps, h)
            if keep is not None and (last or self.layers[i + 1].spec.index != L.spec.index):
                keep.append(x.clone())
        if not rows:
            return torch.empty(0, cfg.vocab, **f32)
        hw = h if rows == list(range(T)) else h[torch.tensor(rows, device=dev)]
        return self._mm(hw.contiguous(), self.head)[:, :cfg.vocab]

    def _forward_hyper(self, plan: StepPlan, rows: List[int], keep: Optional[list] = None) -> torch.Tensor:
        """Several copies of the stream mixed by learned weights.  One fused kernel per sublayer boundary closes the sublayer (all
        streams from the old ones plus its result, output bias and identity experts' share included) and forms the next sublayer's
        layer-normed input (the last one: the final norm of the streams' sum).  ``keep``: a list that receives the sum of the streams
        after every layer."""
        cfg, dev, wd, st = self.cfg, self.device, self.wdtype, self.stream
        T, W, eps = plan.T, cfg.width, cfg.norm_eps
        f32 = dict(dtype=torch.float32, device=dev)
        xs = torch.empty(T, st.streams, W, **f32)
        hy.embed_streams(self.embed, plan.tokens, st.embed_scale, xs)
        h = torch.empty(T, W, dtype=wd, device=dev)
        first = self.layers[0]
        hy.hyper_boundary(xs, None, None, None, None, None, first.hc_in, first.w_pre, first.w_pre_b, eps, h)
        for i, L in enumerate(self.layers):
            U = self._mm(h, L.w_in)                                                   # [T, n_in] float
            A = (torch.zeros if L.out_pad else torch.empty)(T, L.k_out, dtype=wd, device=dev)
            self._run_mixers(L, U, A, plan, eps)
            self_w = None
            if L.ff_col is not None:
                self_w = self._feed_forward(L, U, A)
            o = self._mm(A, L.w_out) if L.k_out else None                             # [T, W] float
            if L.w_gate_up is not None:
                o, self_w = self._experts_grouped(L, U, h, o, want_self=True)
            last = i + 1 == len(self.layers)
            nxt = None if last else self.layers[i + 1]
            hy.hyper_boundary(xs, o, L.out_bias, self_w, L.hc_mix, L.hc_out, None if last else nxt.hc_in,
                              self.final_gain if last else nxt.w_pre, self.final_bias if last else nxt.w_pre_b, eps, h)
            if keep is not None and (last or nxt.spec.index != L.spec.index):
                keep.append(xs.sum(1))
        if not rows:
            return torch.empty(0, cfg.vocab, **f32)
        hw = h if rows == list(range(T)) else h[torch.tensor(rows, device=dev)]
        return self._mm(hw.contiguous(), self.head)[:, :cfg.vocab]

    def _rot_attention(self, M, U, plan, eps, out):
        """Attention with rotated (or plain) grouped heads and the optional terms of its spec.  One launch finishes the queries in
        place (bias, rotation, unit norm) and writes keys and values to their pages; the paged kernel applies cap, distance bias,
        window with kept first positions and sink; two differential maps run as heads of their own over shared values and are
        combined, normed and gated by one more launch."""
        ms = M.spec
        T, dev = plan.T, U.device
        cq, nq = M.cols["q"]
        q = U[:, cq:cq + nq]
        k = v = None
        if M.owns_kv:
            ck, nk = M.cols["k"]
            k = U[:, ck:ck + nk]
            if not ms.values_from_keys:
                cv, nv = M.cols["v"]
                v = U[:, cv:cv + nv]
        hy.rot_kv_write(q, M.vec.get("q.b"), k, M.vec.get("k.b"), v, M.vec.get("freq"), ms.rot_dims, M.rot_mult,
                        ms.rot_layout == "interleaved", ms.unit_qk_norm, None, None, eps, plan, M.k_cache, M.v_cache)
        window = ms.window if ms.window > 0 else 1 << 30
        gate = None
        if ms.out_gate:
            cg, ng = M.cols["g"]
            gate = U[:, cg:cg + ng]
        if ms.maps == 2:
            a = torch.empty(T, 2 * ms.heads * ms.vdim, dtype=torch.float32, device=dev)    # the maps are subtracted before they are rounded
            hy.window_attention(q, M.k_cache, M.v_cache, plan, window, ms.scale, 1.0, a, head_sink=M.vec.get("sink"), softcap=ms.softcap,
                                keep_first=ms.keep_first, dist_bias=M.vec.get("rel"), v_div=2)
            hy.diff_combine(a, M.lam, 1.0 - ms.diff, eps, gate, ms.out_scale, out, ms.heads, ms.kv_heads)
            return
        if gate is not None:
            raise NotImplementedError("an element-wise output gate goes with two score maps")
        hy.window_attention(q, M.k_cache, M.v_cache, plan, window, ms.scale, ms.out_scale, out, head_sink=M.vec.get("sink"),
                            softcap=ms.softcap, keep_first=ms.keep_first, dist_bias=M.vec.get("rel"))

    def _mlstm(self, M, U, plan, eps, out):
        """Matrix memory with exponential gates: the scan carries S, the normaliser and the running maximum per slot and reads the
        projections where the fused GEMM left them; a second launch divides, norms per head, weights and gates."""
        ms = M.spec
        T, dev = plan.T, U.device
        o = torch.empty(T, ms.heads * (ms.vdim + 1), dtype=torch.float32, device=dev)
        m = torch.empty(T, ms.heads, dtype=torch.float32, device=dev)
        hy.mlstm_scan(U, M.cols["q"][0], M.cols["k"][0], M.cols["v"][0], M.cols["i"][0], M.cols["f"][0], M.vec["i.b"], M.vec["f.b"],
                      ms.gate_cap, ms.dim ** -0.5, M.state, M.aux_state, o, m, plan)
        cg, ng = M.cols["g"]
        hy.mlstm_out(o, m, U[:, cg:cg + ng], M.vec["norm"], eps, ms.out_scale, out, ms.heads)

    def _latent_attention(self, M, U, plan, eps, out):
        """Latent attention in its absorbed form.  The cache holds one row [latent | rotated shared key part] per token; a head's
        query is taken into that space (``uk_h^T q_unrotated | q_rotated``), the paged kernel treats the row as the one key head
        whose first ``kv_rank`` columns are also the value, and the latent result is expanded by ``uv_h`` afterwards; the gate and the
        sink are per head, so they commute with the expansion."""
        ms = M.spec
        T, dev, wd = plan.T, U.device, self.wdtype
        H, dn, dr, r, dv = ms.heads, ms.dim, ms.rot_dim, ms.kv_rank, ms.vdim
        (cq, nq), (cd, nd) = M.cols["q"], M.cols["dkv"]
        D = r + dr
        q = U[:, cq:cq + nq]
        # queries head-major [H, T, D]: the batched GEMM writes a head's absorbed columns in place, the kernel its rotated ones
        qa = torch.empty(H, T, D, dtype=torch.float32, device=dev)
        if self.fp32:
            qn = q.unflatten(1, (H, dn + dr))[:, :, :dn].transpose(0, 1)                  # a strided view is a valid operand
            hy.latent_kv_write(q, H, dn, dr, U[:, cd:cd + nd], M.vec["dkv.norm"], eps, M.vec["freq"], ms.rot_dims, M.rot_mult,
                               ms.rot_layout == "interleaved", plan, M.k_cache, qa)
            native._count()
            torch.bmm(qn, M.w_uk, out=qa[:, :, :r])
        else:
            qn = torch.empty(H, T, dn, dtype=wd, device=dev)
            hy.latent_kv_write(q, H, dn, dr, U[:, cd:cd + nd], M.vec["dkv.norm"], eps, M.vec["freq"], ms.rot_dims, M.rot_mult,
                               ms.rot_layout == "interleaved", plan, M.k_cache, qa, qn)
            native._count()
            torch.bmm(qn, M.w_uk, out_dtype=torch.float32, out=qa[:, :, :r])
        gate = None
        if ms.head_gate:
            cg, ng = M.cols["g"]
            gate = U[:, cg:cg + ng]
        lat = torch.empty(T, H * r, dtype=wd, device=dev)
        hy.window_attention(qa, M.k_cache, M.k_cache, plan, 1 << 30, ms.scale, ms.out_scale, lat, gate=gate, head_sink=M.vec.get("sink"),
                            value_size=r)
        # expansion per head straight into the out-projection's operand (float32 accumulation, rounded once)
        native._count()
        torch.bmm(lat.unflatten(1, (H, r)).transpose(0, 1), M.w_uv, out=out.unflatten(1, (H, dv)).transpose(0, 1))

    def _gla(self, M, U, plan, eps, out):
        """Gated linear attention: the scan of the delta rule without the delta, decays per key channel from a low-rank projection."""
        ms = M.spec
        T, dev = plan.T, U.device
        nk, nv = ms.heads * ms.dim, ms.heads * ms.vdim
        cq, _ = M.cols["q"]
        qkv = U[:, cq:cq + 2 * nk + nv]
        c1, r = M.cols["a1"]
        t1 = (torch.zeros if M.w_lr2.shape[1] != r else torch.empty)(T, M.w_lr2.shape[1], dtype=self.wdtype, device=dev)
        hy.act_cols(U[:, c1:c1 + r], t1[:, :r], "copy")
        z = self._mm(t1, M.w_lr2)
        decay = torch.empty(T, nk, dtype=torch.float32, device=dev)
        hy.gla_prep(qkv, z[:, :nk], M.vec["a2.b"], ms.tau, decay, ms.heads, ms.dim)
        o = torch.empty(T, nv, dtype=torch.float32, device=dev)
        hy.delta_scan(qkv, nk, 2 * nk, None, decay, M.state, o, plan, ms.heads, True)
        cg, ng = M.cols["g"]
        hy.gated_part_rmsnorm(o, U[:, cg:cg + ng], M.vec["norm"], ms.vdim, "silu", False, eps, ms.out_scale, out)

    def _forward_sandwich(self, plan: StepPlan, rows: List[int], keep: Optional[list] = None) -> torch.Tensor:
        """Stream with a norm before and after every sublayer: ``x += norm_b(gate * sublayer(norm(x)))``.  One fused kernel per
        sublayer boundary closes the sublayer (gate, post-norm, residual add) and forms the next sublayer's normed input.
        ``keep``: a list that receives a copy of the stream after every layer."""
        cfg, dev, wd, st = self.cfg, self.device, self.wdtype, self.stream
        T, W, eps = plan.T, cfg.width, cfg.norm_eps
        f32 = dict(dtype=torch.float32, device=dev)
        x = torch.empty(T, W, **f32)
        hy.embed_hashed(self.embed, self.pair_table, plan, self.prev_token, st.embed_scale, st.pair_mul_prev, st.pair_mul_cur,
                        st.pair_buckets, x)
        h = torch.empty(T, W, dtype=wd, device=dev)
        ctx: Dict[int, torch.Tensor] = {}                 # values that later layers blend with, by providing layer
        hy.group_norm_residual(x, None, None, None, None, self.layers[0].w_pre, st.norm_groups, eps, h)
        for i, L in enumerate(self.layers):
            U = self._mm(h, L.w_in)                                                   # [T, n_in] float
            A = (torch.zeros if L.out_pad else torch.empty)(T, L.k_out, dtype=wd, device=dev)
            for M in L.mixers:
                out = A[:, M.out_col:M.out_col + M.out_size]
                if M.spec.kind == "conv_attention":
                    self._conv_attention(M, U, plan, out, ctx, L.spec.index)
                elif M.spec.kind == "gated_delta":
                    self._gated_delta(M, U, plan, eps, out)
                elif M.spec.kind == "window_attention":
                    self._window_attention(M, U, plan, eps, out)
                else:
                    self._ssd(M, U, plan, eps, out)
            if L.ff_col is not None:
                self._feed_forward(L, U, A)
            o = self._mm(A, L.w_out) if L.k_out else None                             # [T, W] float
            if L.w_gate_up is not None:
                o = self._experts_grouped(L, U, h, o)
            gate = None
            if L.gate_col is not None:
                c, n = L.gate_col
                gate = U[:, c:c + n]
            last = i + 1 == len(self.layers)
            w_next = self.final_gain if last else self.layers[i + 1].w_pre
            hy.group_norm_residual(x, o, gate, L.gate_bias, L.w_post, w_next, st.norm_groups, eps, h)
            if keep is not None and (last or self.layers[i + 1].spec.index != L.spec.index):
                keep.append(x.clone())
        if not rows:
            return torch.empty(0, cfg.vocab, **f32)
        hw = h if rows == list(range(T)) else h[torch.tensor(rows, device=dev)]
        logits = self._mm(hw.contiguous(), self.head)
        if st.logit_scale != 1.0:
            native._count()
            logits.mul_(st.logit_scale)
        return logits[:, :cfg.vocab]                      # rows keep their padded (16-byte aligned) stride

    def _experts_grouped(self, L, U, h, o, want_self: bool = False):
        """Route, then run only the chosen experts: rows sorted by expert through two grouped GEMMs.  ``want_self``: also return the
        per-token weight of the chosen identity experts (None without such experts)."""
        spec = L.spec
        T, dev = h.shape[0], h.device
        rc, E = L.router_col
        ids = torch.empty(T, spec.top, dtype=torch.int32, device=dev)
        wts = torch.empty(T, spec.top, dtype=torch.float32, device=dev)
        self_w = None
        if spec.route == "softmax_all":
            if spec.identity_experts:
                self_w = torch.empty(T, dtype=torch.float32, device=dev)
            hy.moe_route_all(U[:, rc:rc + E], L.router_bias, spec.experts, spec.top, spec.route_scale, ids=ids, wts=wts, self_w=self_w,
                             groups=spec.route_groups, keep=spec.route_keep)
        else:
            hy.moe_route(U[:, rc:rc + E], L.router_bias, spec.top, ids=ids, wts=wts)
        y = torch.empty(T, self.cfg.width, dtype=torch.float32, device=dev)
        hy.moe_grouped_ffn(h, ids, wts, L.w_gate_up, L.w_down, spec.experts, spec.ff, y, fused_act=spec.ff % 32 == 0,
                           identity=spec.identity_experts)
        if o is not None:
            native._count()
            y = o.add_(y)
        return (y, self_w) if want_self else y

    def _feed_forward(self, L, U, A):
        spec = L.spec
        c, n = L.ff_col
        oc, on = L.ff_out_col
        if spec.ff_kind == "moe" and spec.route == "softmax_all":
            rc, E = L.router_col
            self_w = torch.empty(U.shape[0], dtype=torch.float32, device=U.device) if spec.identity_experts else None
            hy.moe_route_all(U[:, rc:rc + E], L.router_bias, spec.experts, spec.top, spec.route_scale, gu=U[:, c:c + n], ff=spec.ff,
                             act=A[:, oc:oc + on], self_w=self_w, groups=spec.route_groups, keep=spec.route_keep)
            return self_w
        if spec.ff_kind == "moe":
            rc, E = L.router_col
            hy.moe_route(U[:, rc:rc + E], L.router_bias, spec.top, gu=U[:, c:c + n], ff=spec.ff, act=A[:, oc:oc + on])
        elif spec.ff_act == "swiglu":
            hy.swiglu_cols(U[:, c:c + n], None, A[:, oc:oc + on])
        else:
            hy.act_cols(U[:, c:c + n], A[:, oc:oc + on], spec.ff_act)
        return None

    def _conv_attention(self, M, U, plan, out, ctx, layer_index):
        """Biased q / k / v through one short causal convolution (taps carried per slot), values blended with an earlier
        layer's, keys and values into their pages, then attention with the per-head score terms and output gate."""
        ms = M.spec
        T, dev = plan.T, U.device
        nq, nk, nv = ms.heads * ms.dim, ms.kv_heads * ms.dim, ms.kv_heads * ms.vdim
        cq, _ = M.cols["q"]
        qkv = torch.empty(T, nq + nk + nv, dtype=torch.float32, device=dev)
        hy.causal_conv(U[:, cq:cq + nq + nk + nv], M.vec["conv"], None, M.conv_state, qkv, plan, in_bias=M.vec["in_bias"], act="none")
        q, k, v = qkv[:, :nq], qkv[:, nq:nq + nk], qkv[:, nq + nk:]
        other = lam = None
        if ms.v_blend >= 0 and ms.v_blend != layer_index:
            other, lam = ctx[ms.v_blend], M.vec["vmix"]
        hy.kv_write_blend(k, v, other, lam, M.k_cache, M.v_cache, plan)
        if ms.v_blend == layer_index:
            ctx[layer_index] = v
        gate = None
        if ms.head_gate:
            cg, ng = M.cols["g"]
            gate = U[:, cg:cg + ng]
        hy.window_attention(q, M.k_cache, M.v_cache, plan, ms.window, ms.scale, ms.out_scale, out, chunked=ms.mask == "chunk",
                            head_scale=M.vec.get("temp"), head_slope=M.vec.get("slope"), gate=gate)

    def _forward_depth_weighted(self, plan: StepPlan, rows: List[int]) -> torch.Tensor:
        cfg, dev, wd = self.cfg, self.device, self.wdtype
        T, W, eps = plan.T, cfg.width, cfg.norm_eps
        f32 = dict(dtype=torch.float32, device=dev)
        nl = len(self.layers)
        results = torch.empty(nl + 1, T, W, **f32)
        hy.embed_pos(self.embed, self.pos_table, plan.tokens, plan.pos, results[0])
        xbuf = [torch.empty(T, W, **f32), torch.empty(T, W, **f32)]
        h = torch.empty(T, W, dtype=wd, device=dev)
        o = xprev = None
        for i, L in enumerate(self.layers):
            xcur = xbuf[i & 1]
            hy.stream_norm(results, i, o, xprev, self.layers[i - 1].dw if i else None, L.gain, eps, xcur, h, T)
            U = self._mm(h, L.w_in)                                                   # [T, n_in] float
            A = (torch.zeros if L.out_pad else torch.empty)(T, L.k_out, dtype=wd, device=dev)
            for M in L.mixers:
                out = A[:, M.out_col:M.out_col + M.out_size]
                if M.spec.kind == "window_attention":
                    self._window_attention(M, U, plan, eps, out)
                elif M.spec.kind == "ssd":
                    self._ssd(M, U, plan, eps, out)
                else:
                    self._gated_delta(M, U, plan, eps, out)
            if L.ff_col is not None:
                self._feed_forward(L, U, A)
            o = self._mm(A, L.w_out)                                                  # [T, W] float
            if L.w_gate_up is not None:
                o = self._experts_grouped(L, U, h, o)
            xprev = xcur
        hy.stream_norm(results, nl, o, xprev, self.layers[-1].dw, self.final_gain, eps, xbuf[nl & 1], h, T)
        if not rows:
            return torch.empty(0, cfg.vocab, **f32)
        hw = h if rows == list(range(T)) else h[torch.tensor(rows, device=dev)]
        return self._mm(hw.contiguous(), self.head)[:, :cfg.vocab]

    def _window_attention(self, M, U, plan, eps, out):
        ms = M.spec
        (cq, nq), (ck, nk), (cv, nv) = M.cols["q"], M.cols["k"], M.cols["v"]
        q = U[:, cq:cq + nq]
        hy.qknorm_kv_write(q, U[:, ck:ck + nk], U[:, cv:cv + nv], M.vec["qw"], M.vec["kw"], eps, M.k_cache, M.v_cache, plan)
        hy.window_attention(q, M.k_cache, M.v_cache, plan, ms.window, ms.scale, ms.out_scale, out)

    def _ssd(self, M, U, plan, eps, out):
        ms = M.spec
        T = plan.T
        inner, gn = ms.heads * ms.vdim, ms.kv_heads * ms.dim
        ch = inner + 2 * gn
        c0, _ = M.cols["in"]
        z, raw, dt_raw = U[:, c0:c0 + inner], U[:, c0 + inner:c0 + inner + ch], U[:, c0 + inner + ch:c0 + inner + ch + ms.heads]
        xbc = torch.empty(T, ch, dtype=torch.float32, device=U.device)
        hy.causal_conv(raw, M.vec["conv"], M.vec["conv.b"], M.conv_state, xbc, plan)
        y = torch.empty(T, inner, dtype=torch.float32, device=U.device)
        hy.ssd_scan(xbc, inner, inner + gn, dt_raw, M.vec["dt_bias"], M.vec["A_log"], M.vec["D"], M.state, y, plan, ms.kv_heads)
        hy.gated_part_rmsnorm(y, z, M.vec["norm"], inner // ms.norm_groups, "silu", True, eps, ms.out_scale, out)

    def _gated_delta(self, M, U, plan, eps, out):
        ms = M.spec
        T, dev = plan.T, U.device
        nk, nv = ms.kv_heads * ms.dim, ms.heads * ms.vdim
        cq, _ = M.cols["q"]
        qkv = torch.empty(T, 2 * nk + nv, dtype=torch.float32, device=dev)
        hy.causal_conv(U[:, cq:cq + 2 * nk + nv], M.vec["conv"], None, M.conv_state, qkv, plan)
        cb, nb = M.cols["b"]
        if ms.per_channel:
            c1, r = M.cols["a1"]
            t1 = (torch.zeros if M.w_lr2.shape[1] != 2 * r else torch.empty)(T, M.w_lr2.shape[1], dtype=self.wdtype, device=dev)
            hy.act_cols(U[:, c1:c1 + 2 * r], t1[:, :2 * r], "copy")
            ag = self._mm(t1, M.w_lr2)
            na, ng = M.lr_cols
            a_raw, gate = ag[:, :na], ag[:, na:na + ng]
        else:
            (ca, na), (cg, ng) = M.cols["a"], M.cols["g"]
            a_raw, gate = U[:, ca:ca + na], U[:, cg:cg + ng]
        beta = torch.empty(T, ms.heads, dtype=torch.float32, device=dev)
        decay = torch.empty(T, na, dtype=torch.float32, device=dev)
        hy.delta_prep(qkv, nk, U[:, cb:cb + nb], a_raw, M.vec["dt_bias"], M.vec["A_log"], beta, decay, ms.kv_heads, ms.dim, ms.per_channel)
        o = torch.empty(T, nv, dtype=torch.float32, device=dev)
        hy.delta_scan(qkv, nk, 2 * nk, beta, decay, M.state, o, plan, ms.kv_heads, ms.per_channel)
        hy.gated_part_rmsnorm(o, gate, M.vec["norm"], ms.vdim, "sigmoid" if ms.per_channel else "silu", False, eps, ms.out_scale, out)

    # ------------------------------------------------------------------------------------------
    # generation: continuous batching with chunked prefill on top of step()
    # ------------------------------------------------------------------------------------------
    @torch.no_grad()
    def generate(self, prompts: Sequence[Sequence[int]], n: int, temperature: float, top_p: float, max_tokens: int,
                 eos_id: Optional[int], pad_id: int, seed: int) -> torch.Tensor:
        dev = self.device
        total = len(prompts) * n
        out = torch.full((total, max_tokens), pad_id, dtype=torch.long)
        if any(len(p) + max_tokens > self.cfg.max_positions for p in prompts):
            raise ValueError("prompt + max_tokens exceeds the model's learned positions")
        slots = min(total, self.max_num_seqs)
        per_seq = [(len(p) + max_tokens + self.PAGE - 1) // self.PAGE * self.PAGE for p in prompts for _ in range(n)]
        need = self.pool_tokens or sum(sorted(per_seq, reverse=True)[:slots])
        if self.sched is None or self.sched.num_open() or self.num_blocks * self.PAGE < need or self.num_slots < slots:
            self.reset_pool(need, slots)
        sched = self.sched
        self._bt_width = max(per_seq) // self.PAGE        # fixed width: decode steps of one batch size share a CUDA graph
        toks: Dict[int, List[int]] = {}
        gen: Dict[int, int] = {}
        for p in prompts:
            for _ in range(n):
                rid = sched.submit(len(p), max_tokens)
                toks[rid], gen[rid] = list(p), 0
        rid0 = min(toks)
        while sched.num_running() or sched.num_waiting():
            ids, offs, cnts = sched.schedule(self.prefill_token_budget)
            if not ids:
                raise RuntimeError("page pool too small: no waiting request can be admitted")
            entries, sampled = [], []
            for rid, off, cnt in zip(ids, offs, cnts):
                last = off + cnt == len(toks[rid])
                entries.append((sched.seq_of(rid), toks[rid][off:off + cnt], [cnt - 1] if last else []))
                if last:
                    sampled.append(rid)
                self.stats["decode_tokens" if gen[rid] else "prefill_tokens"] += cnt
            logits = self.step(entries)
            for rid, cnt in zip(ids, cnts):
                sched.fed(rid, cnt)
            if not sampled:
                continue
            row_ids = torch.tensor([r - rid0 for r in sampled], dtype=torch.int32, device=dev)
            row_steps = torch.tensor([gen[r] for r in sampled], dtype=torch.int32, device=dev)
            new = native.sample(logits, temperature, top_p, seed, 0, row_ids, row_steps).tolist()   # rows keep their padded stride
            for rid, t in zip(sampled, new):
                out[rid - rid0, gen[rid]] = t
                gen[rid] += 1
                if (eos_id is not None and t == eos_id) or gen[rid] >= max_tokens:
                    sched.finish(rid)
                else:
                    toks[rid].append(int(t))
                    sched.push_token(rid)
        self._bt_width = 0
        return out.to(dev)
