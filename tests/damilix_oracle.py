"""Plain float64 implementation of the Damilix decoder, one function per mechanism, written from the design's equations.

It shares no code with the serving path: whole sequences only, no cache, no pages, no batching; every recurrence is a Python
loop over tokens and every attention builds its full score matrix.  ``weights`` maps checkpoint tensor names to tensors,
``cfg`` is the parsed ``config.json``.
"""
import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def rotary_tables(rot, positions):
    """cos, sin [tokens, dims / 2] for the rotation described by ``rot`` (base, dims, optional scaling)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    mult = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def corr(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(corr(float(sc["fast"]))), 0)
        hi = min(math.ceil(corr(float(sc["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mult = 0.1 * math.log(factor) + 1.0
    a = positions.to(F64)[:, None] * f[None, :]
    return torch.cos(a) * mult, torch.sin(a) * mult


def rotate(x, cos, sin, layout):
    """x [tokens, ..., dims]: the whole last axis is rotated.  ``layout``: "interleaved" pairs (2i, 2i+1), "half" pairs (i, i + dims/2)."""
    d = x.shape[-1]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [d // 2]
    c, s = cos.reshape(shape), sin.reshape(shape)
    out = torch.empty_like(x)
    if layout == "interleaved":
        u, v = x[..., 0::2], x[..., 1::2]
        out[..., 0::2] = u * c - v * s
        out[..., 1::2] = v * c + u * s
    else:
        u, v = x[..., :d // 2], x[..., d // 2:]
        out[..., :d // 2] = u * c - v * s
        out[..., d // 2:] = v * c + u * s
    return out


def latent_core(q, dkv, gate_raw, w, p, m, eps, layout, positions=None):
    """The attention itself, from the projections: q [T, H * (dim + rot_dim)], dkv [T, kv_rank + rot_dim], gate_raw [T, H].
    Returns the gated head results [T, H * vdim] (before the output projection)."""
    T = q.shape[0]
    H, dn, dr, dv, r = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    q = q.reshape(T, H, dn + dr)
    qn, qr = q[..., :dn], q[..., dn:]
    c = rms(dkv[:, :r], eps) * w[p + "dkv.norm"]
    kr = dkv[:, r:]
    cos, sin = rotary_tables(m["rot"], torch.arange(T) if positions is None else positions)
    nd = int(m["rot"]["dims"])
    qr = torch.cat([rotate(qr[..., :nd], cos, sin, layout), qr[..., nd:]], -1)
    kr = torch.cat([rotate(kr[:, :nd], cos, sin, layout), kr[:, nd:]], -1)
    kn = (c @ w[p + "uk"].T).reshape(T, H, dn)
    v = (c @ w[p + "uv"].T).reshape(T, H, dv)
    gate = torch.sigmoid(gate_raw)                               # [T, H]
    out = torch.zeros(T, H, dv, dtype=F64)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for hd in range(H):
        s = (qn[:, hd] @ kn[:, hd].T + qr[:, hd] @ kr.T) * float(m["scale"])
        s = s.masked_fill(~mask, -math.inf)
        sink = w[p + "sink"][hd]
        mx = torch.maximum(s.max(-1, keepdim=True).values, sink)
        e = torch.exp(s - mx)
        pr = e / (e.sum(-1, keepdim=True) + torch.exp(sink - mx))
        out[:, hd] = (pr @ v[:, hd]) * gate[:, hd:hd + 1]
    return out.reshape(T, H * dv)


def latent_attention(w, p, m, h, eps, layout):
    """Attention over a low-rank latent: keys and values of every head are projections of one normed latent per token, plus one
    rotated key part shared by the heads; causal softmax whose denominator also holds exp(sink) per head; sigmoid gate per head."""
    return latent_core(h @ w[p + "q"].T, h @ w[p + "dkv"].T, h @ w[p + "g"].T, w, p, m, eps, layout) @ w[p + "o"].T


def gla_core(q, k, v, z, m, state=None):
    """The recurrence: q, k [T, H, dim] (q already scaled), v [T, H, vdim], decay logits z [T, H, dim].  Returns (o, final state)."""
    T, H, dk = q.shape
    dv, tau = v.shape[-1], float(m["tau"])
    alpha = torch.sigmoid(z) ** (1.0 / tau)
    S = torch.zeros(H, dk, dv, dtype=F64) if state is None else state.clone()
    o = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


def gla(w, p, m, h, eps):
    """Gated linear attention: a matrix state per head decays per key channel and accumulates k v^T; read out with q."""
    T = h.shape[0]
    H, dk, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "q"].T).reshape(T, H, dk) * dk ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, dk)
    v = (h @ w[p + "v"].T).reshape(T, H, dv)
    z = ((h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]).reshape(T, H, dk)
    o, _ = gla_core(q, k, v, z, m)
    o = rms(o, eps) * w[p + "norm"]
    return (o.reshape(T, H * dv) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def swiglu(w, p, h):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(w, p, mlp, h):
    """Chosen experts [T, top] and their weights: softmax over all router outputs, the choice by score + correction, the
    weights the plain scores of the chosen, normalised and scaled."""
    r = mlp["router"]
    s = torch.softmax(h @ w[p + "router"].T, -1)
    choice = s + w[p + "correction"] if (p + "correction") in w else s
    ids = torch.topk(choice, int(r["top"]), dim=-1).indices
    ws = torch.gather(s, 1, ids)
    ws = ws / (ws.sum(-1, keepdim=True) + 1e-20) * float(r.get("scale", 1.0))
    return ids, ws


def moe(w, p, mlp, h):
    r = mlp["router"]
    n_exp = int(r["experts"])
    ids, ws = route(w, p, mlp, h)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), ws[t]):
            if e >= n_exp:                                     # identity expert: the input itself
                out[t] += a * h[t]
            else:
                out[t] += a * swiglu(w, f"{p}e{e}.", h[t:t + 1])[0]
    if mlp.get("shared"):
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * swiglu(w, p + "shared.", h)
    return out


def feed_forward(w, p, mlp, h):
    if mlp["kind"] == "dense":
        return swiglu(w, p, h)
    return moe(w, p, mlp, h)


def token_side(w, cfg, i, tokens, x, eps):
    """Per-layer token input: a slice of a second embedding of the token, gated by a projection of the stream."""
    d = int(cfg["token_side"]["dim"])
    p = f"l{i}.side."
    e = w["side.embed"][tokens][:, i * d:(i + 1) * d]
    g = gelu_tanh(x @ w[p + "gate"].T) * e
    y = g @ w[p + "proj"].T
    return rms(y, eps) * w[p + "norm"]


def model_norm(x, weight, eps):
    return rms(x, eps) * weight


def mixer(w, cfg, i, x, eps):
    layer = cfg["layers"][i]
    p = f"l{i}.mix."
    if layer["type"] == "gla":
        return gla(w, p, layer["mixer"], x, eps)
    layout = {"latent_attention": "interleaved", "latent_attention_2": "half"}[layer["type"]]
    return latent_attention(w, p, layer["mixer"], x, eps, layout)


def forward(weights, cfg, tokens, keep=None):
    """Logits [tokens, vocab] of one whole sequence; ``keep`` receives the stream after every layer."""
    w = {k: v.to(F64) if v.is_floating_point() else v for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = model_norm(w["embed"][tokens], w["embed.norm"], eps)
    for i, layer in enumerate(cfg["layers"]):
        x = x + model_norm(mixer(w, cfg, i, x, eps), w[f"l{i}.norm1"], eps)
        if layer.get("mlp"):
            x = x + model_norm(feed_forward(w, f"l{i}.mlp.", layer["mlp"], x), w[f"l{i}.norm2"], eps)
        if cfg.get("token_side"):
            x = x + token_side(w, cfg, i, tokens, x, eps)
        if keep is not None:
            keep.append(x.clone())
    return model_norm(x, w["final.norm"], eps) @ w["head"].T


# ---- small configurations and random weights for the tests ------------------------------------------------------------
def make_config(vocab=97, width=48, eps=1e-5, side=6, layers=("gla", "latent", "latent2"), gla=None, latent=None, latent2=None,
                dense_ff=40, moe=None, ffs=None, rank=5):
    """A ``config.json`` dictionary.  ``layers``: "gla" | "latent" (interleaved rotation) | "latent2" (half rotation); ``ffs``: per
    layer "dense" | "moe" | None (default: dense, moe, dense, ...); the dictionaries override sizes.  ``rank`` (inner width of the
    decay projection) is not part of the config: it is returned under "_rank" for ``random_weights`` and removed by it."""
    g = dict(heads=2, dim=8, vdim=12, tau=8.0)
    g.update(gla or {})
    a = dict(heads=3, dim=8, rot_dim=4, vdim=10, kv_rank=16, scale=0.3, base=10000.0,
             scaling=dict(factor=4.0, original=32, fast=8.0, slow=1.0))
    a.update(latent or {})
    b = dict(heads=2, dim=4, rot_dim=8, vdim=6, kv_rank=12, scale=0.25, base=500.0, scaling=None)
    b.update(latent2 or {})
    m = dict(ff=16, experts=5, identity=2, top=3, scale=1.5, shared=16)
    m.update(moe or {})
    out = []
    for i, t in enumerate(layers):
        if t == "gla":
            mixer = dict(heads=g["heads"], dim=g["dim"], vdim=g["vdim"], tau=g["tau"])
            typ = "gla"
        else:
            s = a if t == "latent" else b
            rot = dict(base=s["base"], dims=s.get("dims", s["rot_dim"]))
            if s.get("scaling"):
                rot["scaling"] = dict(s["scaling"])
            mixer = dict(heads=s["heads"], dim=s["dim"], rot_dim=s["rot_dim"], vdim=s["vdim"], kv_rank=s["kv_rank"], scale=s["scale"], rot=rot)
            typ = "latent_attention" if t == "latent" else "latent_attention_2"
        kind = ffs[i] if ffs is not None else ("moe" if i % 2 else "dense")
        if kind == "dense":
            mlp = dict(kind="dense", ff=dense_ff)
        elif kind == "moe":
            mlp = dict(kind="moe", expert=dict(ff=m["ff"]), router=dict(experts=m["experts"], identity=m["identity"], top=m["top"], scale=m["scale"]))
            if m.get("shared"):
                mlp["shared"] = dict(ff=m["shared"])
        else:
            mlp = None
        out.append(dict(type=typ, mixer=mixer, mlp=mlp))
    cfg = dict(architecture="Damilix", vocab=vocab, width=width, norm=dict(eps=eps), layers=out, _rank=rank)
    if side:
        cfg["token_side"] = dict(dim=side)
    return cfg


def random_weights(cfg, seed=0, dtype=torch.bfloat16):
    """Random checkpoint tensors for ``cfg`` (rounded to ``dtype``, so that the oracle and the engine read the same numbers)."""
    gen = torch.Generator().manual_seed(seed)
    rank = cfg.pop("_rank", 5)
    W, V = cfg["width"], cfg["vocab"]
    w = {}

    def lin(name, o, i, s=1.0):
        w[name] = torch.randn(o, i, generator=gen) * s / i ** 0.5

    def gain(name, n):
        w[name] = torch.rand(n, generator=gen) * 0.5 + 0.75
    w["embed"] = torch.randn(V, W, generator=gen)
    gain("embed.norm", W)
    side = (cfg.get("token_side") or {}).get("dim", 0)
    if side:
        w["side.embed"] = torch.randn(V, side * len(cfg["layers"]), generator=gen)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        gain(p + "norm1", W)
        q = p + "mix."
        if layer["type"] == "gla":
            nk, nv = m["heads"] * m["dim"], m["heads"] * m["vdim"]
            lin(q + "q", nk, W), lin(q + "k", nk, W), lin(q + "v", nv, W), lin(q + "g", nv, W), lin(q + "o", W, nv)
            gain(q + "norm", m["vdim"])
            lin(q + "a1", rank, W), lin(q + "a2", nk, rank, 2.0)
            w[q + "a2.b"] = torch.rand(nk, generator=gen) * 4.0
        else:
            H, r = m["heads"], m["kv_rank"]
            lin(q + "q", H * (m["dim"] + m["rot_dim"]), W), lin(q + "dkv", r + m["rot_dim"], W)
            gain(q + "dkv.norm", r)
            lin(q + "uk", H * m["dim"], r), lin(q + "uv", H * m["vdim"], r)
            w[q + "sink"] = torch.randn(H, generator=gen)
            lin(q + "g", H, W), lin(q + "o", W, H * m["vdim"])
        mlp = layer.get("mlp")
        f = p + "mlp."
        if mlp is not None:
            gain(p + "norm2", W)
        if mlp is not None and mlp["kind"] == "dense":
            lin(f + "gate", mlp["ff"], W), lin(f + "up", mlp["ff"], W), lin(f + "down", W, mlp["ff"])
        elif mlp is not None:
            r, ff = mlp["router"], mlp["expert"]["ff"]
            for e in range(r["experts"]):
                lin(f"{f}e{e}.gate", ff, W), lin(f"{f}e{e}.up", ff, W), lin(f"{f}e{e}.down", W, ff)
            n_out = r["experts"] + r.get("identity", 0)
            lin(f + "router", n_out, W, 2.0)
            w[f + "correction"] = torch.randn(n_out, generator=gen) * 0.05
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                lin(f + "shared.gate", sf, W), lin(f + "shared.up", sf, W), lin(f + "shared.down", W, sf), lin(f + "shared.sg", 1, W)
        if side:
            lin(p + "side.gate", side, W), lin(p + "side.proj", W, side)
            gain(p + "side.norm", W)
    gain("final.norm", W)
    lin("head", V, W)
    return {k: v.to(dtype) for k, v in w.items()}
