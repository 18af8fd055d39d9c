"""Plain float64 implementation of the Lukarax decoder, one function per mechanism, written from the design's equations.

It shares no code with the serving path: whole sequences only, no cache, no pages, no batching; every recurrence is a Python
loop over tokens and every attention builds its full score matrix.  ``weights`` maps checkpoint tensor names to tensors,
``cfg`` is the parsed ``config.json``.
"""
import math

import torch

F64 = torch.float64


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def rotary_tables(rot, positions):
    """cos, sin [tokens, dims / 2] of the rotation ``rot`` (base, dims, optional frequency stretch)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=F64)
    f = base ** (-2.0 * i / dims)
    mult = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def pair_of(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(pair_of(float(sc["fast"]))), 0)
        hi = min(math.ceil(pair_of(float(sc["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mult = 0.1 * math.log(factor) + 1.0
    a = positions.to(F64)[:, None] * f[None, :]
    return torch.cos(a) * mult, torch.sin(a) * mult


def rotate_front(x, cos, sin, dims, layout):
    """x [tokens, heads, D]: the first ``dims`` columns of every head turn, the rest pass.  "interleaved" pairs (2i, 2i+1),
    "half" pairs (i, i + dims / 2)."""
    out = x.clone()
    c, s = cos[:, None, :], sin[:, None, :]
    if layout == "interleaved":
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    else:
        u, v = x[..., :dims // 2], x[..., dims // 2:dims]
        out[..., :dims // 2] = u * c - v * s
        out[..., dims // 2:dims] = v * c + u * s
    return out


def softmax_rows(score, visible, sink=None):
    """Softmax of every row over its visible columns; ``sink`` [rows]: one more term exp(sink) in the denominator only."""
    score = score.masked_fill(~visible, -math.inf)
    m = score.max(-1, keepdim=True).values
    if sink is not None:
        m = torch.maximum(m, sink[:, None])
    e = torch.exp(score - m)
    den = e.sum(-1, keepdim=True)
    if sink is not None:
        den = den + torch.exp(sink[:, None] - m)
    return e / den


def causal(n):
    i = torch.arange(n)
    return i[None, :] <= i[:, None]


# ---- differential attention ------------------------------------------------------------------------------------------
def diff_keys_values(w, p, m, h):
    """Rotated keys [T, G, 2, dim] and values [T, G, vdim] of a differential-attention layer (what later layers may borrow)."""
    T = h.shape[0]
    G, d, dv = int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    cos, sin = rotary_tables(m["rot"], torch.arange(T))
    k = (h @ w[p + "k"].T).view(T, G * 2, d)
    k = rotate_front(k, cos, sin, int(m["rot"]["dims"]), "interleaved").view(T, G, 2, d)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    return k, v


def diff_attention(w, p, m, h, eps, kv):
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    diff = float(m["diff"])
    k, v = kv
    cos, sin = rotary_tables(m["rot"], torch.arange(T))
    q = (h @ w[p + "q"].T).view(T, H * 2, d)
    q = rotate_front(q, cos, sin, int(m["rot"]["dims"]), "interleaved").view(T, H, 2, d)
    lam = math.exp(float((w[p + "lq1"] * w[p + "lk1"]).sum())) - math.exp(float((w[p + "lq2"] * w[p + "lk2"]).sum())) + diff
    vis = causal(T)
    heads = []
    for hq in range(H):
        g = hq // (H // G)
        a = []
        for mp in range(2):
            pr = softmax_rows((q[:, hq, mp] @ k[:, g, mp].T) * float(m["scale"]), vis)
            a.append(pr @ v[:, g])
        o = a[0] - lam * a[1]
        heads.append(unit_rms(o, eps) * (1.0 - diff))
    o = torch.cat(heads, -1) * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


# ---- sliding-window attention whose values are its keys ------------------------------------------------------------------
def window_attention_2(w, p, m, h, eps):
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    rot = m["rot"]
    cos, sin = rotary_tables(rot, torch.arange(T))
    q = (h @ w[p + "q"].T + w[p + "q.b"]).view(T, H, d)
    k = (h @ w[p + "k"].T + w[p + "k.b"]).view(T, G, d)
    v = k                                                        # as projected
    q = unit_rms(rotate_front(q, cos, sin, int(rot["dims"]), "half"), eps)
    kr = unit_rms(rotate_front(k, cos, sin, int(rot["dims"]), "half"), eps)
    i = torch.arange(T)
    dist = i[:, None] - i[None, :]
    vis = (dist >= 0) & (dist < int(m["mask"]["size"]))
    cap = float(m["softcap"])
    heads = []
    for hq in range(H):
        g = hq // (H // G)
        s = (q[:, hq] @ kr[:, g].T) * float(m["scale"])
        s = cap * torch.tanh(s / cap)
        pr = softmax_rows(s, vis, sink=w[p + "sink"][hq].expand(T))
        heads.append(pr @ v[:, g])
    return torch.cat(heads, -1) @ w[p + "o"].T + w[p + "o.b"]


# ---- windowed attention with kept first tokens and a bias by distance ---------------------------------------------------------
def distance_bucket(n, B, D):
    half = B // 2
    if n < half:
        return n
    return min(B - 1, half + int(math.floor(math.log(n / half) / math.log(D / half) * (B - half))))


def biased_window_attention(w, p, m, h):
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (h @ w[p + "q"].T).view(T, H, d)
    k = (h @ w[p + "k"].T).view(T, G, d)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    rel = w[p + "rel"]
    B, D = rel.shape[0], int(m["bias_max"])
    i = torch.arange(T)
    dist = i[:, None] - i[None, :]
    vis = (dist >= 0) & ((dist < int(m["mask"]["size"])) | (i[None, :] < int(m["mask"].get("keep_first", 0))))
    bk = torch.tensor([[distance_bucket(a - b, B, D) if a >= b else 0 for b in range(T)] for a in range(T)])
    heads = []
    for hq in range(H):
        g = hq // (H // G)
        s = (q[:, hq] @ k[:, g].T) * float(m["scale"]) + rel[:, hq][bk]
        heads.append(softmax_rows(s, vis) @ v[:, g])
    return torch.cat(heads, -1) @ w[p + "o"].T


# ---- matrix memory with exponential gates and a running maximum -----------------------------------------------------------
def matrix_memory_core(q, k, v, ig, fg, state=None):
    """q, k [T, H, d], v [T, H, dv], log gates ig, fg [T, H].  ``state`` (S [H, d, dv], n [H, d], m [H]) is carried."""
    T, H, d = q.shape
    dv = v.shape[-1]
    if state is None:
        state = (torch.zeros(H, d, dv, dtype=F64), torch.zeros(H, d, dtype=F64), torch.zeros(H, dtype=F64))
    S, n, m = state
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        m_new = torch.maximum(fg[t] + m, ig[t])
        a = torch.exp(fg[t] + m - m_new)
        b = torch.exp(ig[t] - m_new)
        S = a[:, None, None] * S + b[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = a[:, None] * n + b[:, None] * k[t]
        m = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
        out[t] = num / den[:, None]
    return out, (S, n, m)


def matrix_memory(w, p, m, h, eps):
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    cap = float(m["gate_cap"])
    q = (h @ w[p + "q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[p + "k"].T).view(T, H, d)
    v = (h @ w[p + "v"].T).view(T, H, dv)
    ig = cap * torch.tanh((h @ w[p + "i"].T + w[p + "i.b"]) / cap)
    fg = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w[p + "f"].T + w[p + "f.b"]) / cap))
    o, _ = matrix_memory_core(q, k, v, ig, fg)
    o = unit_rms(o, eps).reshape(T, H * dv) * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def parallel_mixer(w, p, m, h, eps):
    left = biased_window_attention(w, p + "left.", m["left"], h)
    right = matrix_memory(w, p + "right.", m["right"], h, eps)
    return float(m["left_scale"]) * left + float(m["right_scale"]) * right


# ---- feed-forwards ---------------------------------------------------------------------------------------------------
def swiglu(w, p, h):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(w, p, mlp, h):
    """(chosen outputs [T, top], weights [T, top]) of the grouped router; outputs >= experts are identity experts."""
    r = mlp["router"]
    s = torch.softmax(h @ w[p + "router"].T, -1)
    choice = s + w[p + "correction"] if (p + "correction") in w else s.clone()
    E = s.shape[-1]
    groups = r.get("groups")
    if groups and int(groups["count"]) > 1:
        cnt, keep = int(groups["count"]), int(groups["keep"])
        gs = choice.view(-1, cnt, E // cnt).max(-1).values
        order = torch.sort(gs, dim=-1, descending=True, stable=True).indices[:, :keep]
        ok = torch.zeros_like(gs, dtype=torch.bool)
        ok.scatter_(1, order, True)
        choice = choice.masked_fill(~ok.repeat_interleave(E // cnt, 1), -math.inf)
    ids = torch.sort(choice, dim=-1, descending=True, stable=True).indices[:, :int(r["top"])]
    wt = s.gather(1, ids)
    wt = wt / (wt.sum(-1, keepdim=True) + 1e-20) * float(r.get("scale", 1.0))
    return ids, wt


def moe(w, p, mlp, h):
    r = mlp["router"]
    n_real = int(r["experts"])
    ids, wt = route(w, p, mlp, h)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), wt[t]):
            out[t] += a * (swiglu(w, f"{p}e{e}.", h[t:t + 1])[0] if e < n_real else h[t])
    return out


def feed_forward(w, p, mlp, h):
    return swiglu(w, p, h) if mlp["kind"] == "dense" else moe(w, p, mlp, h)


# ---- the model -------------------------------------------------------------------------------------------------------
def mixer(w, cfg, i, h, eps, shared):
    layer = cfg["layers"][i]
    m, p = layer["mixer"], f"l{i}.mix."
    if layer["type"] == "parallel":
        return parallel_mixer(w, p, m, h, eps)
    if layer["type"] == "attention_2":
        return window_attention_2(w, p, m, h, eps)
    src = m.get("kv_from")
    if src is None:
        shared[i] = diff_keys_values(w, p, m, h)
        src = i
    return diff_attention(w, p, m, h, eps, shared[src])


def forward(weights, cfg, tokens, keep=None):
    """Logits [T, vocab] of one whole sequence; ``keep`` receives the sum of the streams after every layer."""
    w = {k: v.to(F64) for k, v in weights.items()}
    eps = float(cfg["norm"]["eps"])
    ns = int(cfg.get("streams") or 1)
    x0 = w["embed"][torch.tensor(tokens)] * float(cfg["embedding"]["scale"])
    xs = [x0.clone() for _ in range(ns)]
    shared = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        for q in (1, 2):
            if q == 2 and layer.get("mlp") is None:
                continue
            hc = p + f"hc{q}."
            plain = cfg.get("streams") is None              # one stream and the plain residual sum
            u = xs[0] if plain else sum(w[hc + "in"][s] * xs[s] for s in range(ns))
            h = layer_norm(u, w[p + f"norm{q}"], w[p + f"norm{q}.b"], eps)
            y = mixer(w, cfg, i, h, eps, shared) if q == 1 else feed_forward(w, p + "mlp.", layer["mlp"], h)
            if plain:
                xs = [xs[0] + y]
            else:
                xs = [sum(w[hc + "mix"][s, t] * xs[s] for s in range(ns)) + w[hc + "out"][t] * y for t in range(ns)]
        if keep is not None:
            keep.append(sum(xs))
    x = layer_norm(sum(xs), w["final.norm"], w["final.norm.b"], eps)
    return x @ w["embed"].T


# ---- small random models for the tests -----------------------------------------------------------------------------------
def make_config(vocab=96, width=48, streams=3, eps=1e-5, embed_scale=2.0, layers=("parallel", "attention_2", "attention", "shared", "parallel"),
                ffs=("dense", "moe", "moe", "dense", None), dense_ff=80, left=None, right=None, att2=None, att=None, moe=None,
                left_scale=0.7, right_scale=1.2):
    """A config dict of the checkpoint format.  Layer kinds: "parallel", "attention_2", "attention" and "shared" (an attention layer that
    reads the pages of the nearest earlier attention layer with projections)."""
    left = dict(dict(heads=4, kv_heads=2, dim=16, vdim=8, scale=0.3, bias_max=40, size=12, keep_first=5), **(left or {}))
    right = dict(dict(heads=2, dim=16, vdim=24, gate_cap=10.0), **(right or {}))
    att2 = dict(dict(heads=4, kv_heads=2, dim=24, scale=0.5, softcap=8.0, size=20, dims=16, base=1e4,
                     scaling=dict(factor=4.0, original=32, fast=8.0, slow=1.0)), **(att2 or {}))
    att = dict(dict(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.25, diff=0.25, dims=8, base=500.0), **(att or {}))
    moe = dict(dict(ff=24, experts=5, identity=3, top=3, scale=1.5, groups=4, keep=2), **(moe or {}))
    out, last_own = [], None
    for i, (kind, ff) in enumerate(zip(layers, ffs)):
        if kind == "parallel":
            lm = {k: left[k] for k in ("heads", "kv_heads", "dim", "vdim", "scale", "bias_max")}
            lm["mask"] = {"size": left["size"], "keep_first": left["keep_first"]}
            mixer = {"left": lm, "right": dict(right), "left_scale": left_scale, "right_scale": right_scale}
        elif kind == "attention_2":
            mixer = {k: att2[k] for k in ("heads", "kv_heads", "dim", "scale", "softcap")}
            mixer["vdim"] = att2["dim"]
            mixer["mask"] = {"size": att2["size"]}
            mixer["rot"] = {"base": att2["base"], "dims": att2["dims"]}
            if att2.get("scaling"):
                mixer["rot"]["scaling"] = dict(att2["scaling"])
        else:
            mixer = {k: att[k] for k in ("heads", "kv_heads", "dim", "vdim", "scale", "diff")}
            mixer["rot"] = {"base": att["base"], "dims": att["dims"]}
            if kind == "shared":
                mixer["kv_from"] = last_own
            else:
                last_own = i
        if ff == "dense":
            mlp = {"kind": "dense", "ff": dense_ff}
        elif ff == "moe":
            router = {"experts": moe["experts"], "identity": moe["identity"], "top": moe["top"], "scale": moe["scale"]}
            if moe.get("groups"):
                router["groups"] = {"count": moe["groups"], "keep": moe["keep"]}
            mlp = {"kind": "moe", "expert": {"ff": moe["ff"]}, "router": router}
        else:
            mlp = None
        out.append({"type": "attention" if kind == "shared" else kind, "mixer": mixer, "mlp": mlp})
    cfg = {"architecture": "Lukarax", "vocab": vocab, "width": width, "norm": {"eps": eps}, "embedding": {"scale": embed_scale},
           "layers": out}
    if streams is not None:
        cfg["streams"] = streams
    return cfg


def tensor_shapes(cfg, rel_buckets=10):
    W, S = cfg["width"], cfg.get("streams")
    out = {"embed": (cfg["vocab"], W), "final.norm": (W,), "final.norm.b": (W,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        subs = ("1", "2") if layer.get("mlp") else ("1",)
        for q in subs:
            out[p + "norm" + q], out[p + "norm" + q + ".b"] = (W,), (W,)
            if S is not None:
                out[f"{p}hc{q}.in"], out[f"{p}hc{q}.out"], out[f"{p}hc{q}.mix"] = (S,), (S,), (S, S)
        x = p + "mix."
        if layer["type"] == "parallel":
            a, r = m["left"], m["right"]
            out.update({x + "left.q": (a["heads"] * a["dim"], W), x + "left.k": (a["kv_heads"] * a["dim"], W),
                        x + "left.v": (a["kv_heads"] * a["vdim"], W), x + "left.rel": (rel_buckets, a["heads"]),
                        x + "left.o": (W, a["heads"] * a["vdim"])})
            nk, nv = r["heads"] * r["dim"], r["heads"] * r["vdim"]
            out.update({x + "right.q": (nk, W), x + "right.k": (nk, W), x + "right.v": (nv, W), x + "right.g": (nv, W), x + "right.o": (W, nv),
                        x + "right.norm": (nv,), x + "right.i": (r["heads"], W), x + "right.i.b": (r["heads"],),
                        x + "right.f": (r["heads"], W), x + "right.f.b": (r["heads"],)})
        elif layer["type"] == "attention_2":
            nq, nk = m["heads"] * m["dim"], m["kv_heads"] * m["dim"]
            out.update({x + "q": (nq, W), x + "q.b": (nq,), x + "k": (nk, W), x + "k.b": (nk,), x + "sink": (m["heads"],), x + "o": (W, nq),
                        x + "o.b": (W,)})
        else:
            nq, nv = m["heads"] * 2 * m["dim"], m["heads"] * m["vdim"]
            out.update({x + "q": (nq, W), x + "g": (nv, W), x + "o": (W, nv)})
            for n in ("lq1", "lk1", "lq2", "lk2"):
                out[x + n] = (m["dim"],)
            if m.get("kv_from") is None:
                out.update({x + "k": (m["kv_heads"] * 2 * m["dim"], W), x + "v": (m["kv_heads"] * m["vdim"], W)})
        mlp, f = layer.get("mlp"), p + "mlp."
        if mlp and mlp["kind"] == "dense":
            out.update({f + "gate": (mlp["ff"], W), f + "up": (mlp["ff"], W), f + "down": (W, mlp["ff"])})
        elif mlp:
            r, ff = mlp["router"], mlp["expert"]["ff"]
            for e in range(r["experts"]):
                out.update({f"{f}e{e}.gate": (ff, W), f"{f}e{e}.up": (ff, W), f"{f}e{e}.down": (W, ff)})
            out[f + "router"], out[f + "correction"] = (r["experts"] + r.get("identity", 0), W), (r["experts"] + r.get("identity", 0),)
    return out


def random_weights(cfg, seed=0, rel_buckets=10, dtype=torch.float32):
    """Random tensors of a size that keeps every mechanism alive: scores of order one, gates that neither close nor saturate, sinks
    and distance biases that matter, stream weights away from a plain residual."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for n, shp in tensor_shapes(cfg, rel_buckets).items():
        leaf = n.rsplit(".", 1)[-1]
        if ".hc" in n:
            t = torch.randn(shp, generator=g) * 0.3 + (torch.eye(shp[0]) if leaf == "mix" else 0.6)
        elif leaf in ("rel", "sink"):
            t = torch.randn(shp, generator=g)
        elif len(shp) == 2:
            t = torch.randn(shp, generator=g) * (0.5 if leaf == "embed" else 1.3 / shp[1] ** 0.5)
        elif n.endswith(".b") and "norm" not in n:
            t = torch.randn(shp, generator=g) * 0.3 + (1.5 if n.endswith("f.b") else 0.0)
        elif leaf == "b":
            t = torch.randn(shp, generator=g) * 0.1
        elif leaf in ("lq1", "lk1", "lq2", "lk2"):
            t = torch.randn(shp, generator=g) * 0.3
        elif leaf == "correction":
            t = torch.randn(shp, generator=g) * 0.05
        else:
            t = torch.rand(shp, generator=g) * 0.5 + 0.75
        out[n] = t.to(dtype)
    return out
