"""Lukarax on the step engine against the plain float64 oracle (tests/lukarax_oracle.py): small random models of several
shapes, written to disk as a checkpoint, loaded through the model registry and run through ``HybridSampler.step`` /
``generate`` under different schedules (whole prompts, token by token, portions, mixed batches, reused pages and slots),
and every new mechanism alone against the oracle's function for it."""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import lukarax_oracle as O

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32_TOL = 2e-4
BF16_TOL = 6e-2


# ---- helpers -----------------------------------------------------------------------------------------------------
def _save(tmp_path, cfg, W, name="m"):
    from safetensors.torch import save_file
    d = os.path.join(str(tmp_path), name)
    os.makedirs(d, exist_ok=True)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.contiguous() for k, v in W.items()}, os.path.join(d, "model.safetensors"))
    return d


def _engine(tmp_path, cfg, W, dtype="fp32", pool_tokens=1024, slots=4, name="m", **kw):
    from nanorlhf_b200.models.registry import load_model
    from nanorlhf_b200.sampler.hybrid_sampler import HybridSampler
    path = _save(tmp_path, cfg, W, name)
    model = load_model(path, torch_dtype=torch.float32 if dtype == "fp32" else torch.bfloat16, device="cuda")
    eng = HybridSampler(model, dtype=dtype, max_num_seqs=slots, **kw)
    eng.reset_pool(pool_tokens, slots)
    return eng


def _tokens(cfg, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()


def _run_alone(eng, toks, cuts):
    """Feed one sequence in portions ``cuts``; logits of every position."""
    sid = eng.open()
    out, lo = [], 0
    for n in cuts:
        out.append(eng.step([(sid, toks[lo:lo + n], list(range(n)))]).double().cpu())
        lo += n
    eng.close(sid)
    assert lo == len(toks)
    return torch.cat(out)


def _rows(got, want):
    return (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()


def _close(got, want, dtype):
    rows = _rows(got, want)
    if dtype == "fp32":
        return bool(rows.max() < F32_TOL)
    return bool((rows > BF16_TOL).double().mean() <= 0.1 and rows.max() < 3 * BF16_TOL and rows.mean() < 0.5 * BF16_TOL)


def _cuts(total, sizes):
    out, i, k = [], 0, 0
    while i < total:
        n = min(sizes[k % len(sizes)], total - i)
        out.append(n)
        i += n
        k += 1
    return out


SHAPES = {
    # every layer type and feed-forward kind; a layer that borrows pages; sizes that differ from their neighbours
    "mixed": dict(),
    # values that usual defaults make equal or 1: one stream, one head everywhere, top 1, one group, window 1, one kept key,
    # scales 1, rotation over the whole head, no stretch, bias_max barely past the single-distance buckets
    "ones": dict(streams=1, layers=("attention", "parallel", "attention_2", "shared"), ffs=("moe", "moe", "dense", None),
                 left=dict(heads=1, kv_heads=1, dim=8, vdim=8, scale=1.0, bias_max=6, size=1, keep_first=1),
                 right=dict(heads=1, dim=8, vdim=8, gate_cap=1.0),
                 att2=dict(heads=1, kv_heads=1, dim=8, scale=1.0, softcap=1.0, size=1, dims=8, scaling=None),
                 att=dict(heads=1, kv_heads=1, dim=8, vdim=8, scale=1.0, diff=0.5, dims=8),
                 moe=dict(ff=8, experts=1, identity=1, top=1, scale=1.0, groups=1, keep=1), left_scale=1.0, right_scale=1.0, embed_scale=1.0),
    # no stream weights at all (plain residual), no identity experts, no groups, every expert chosen, a width off the vector paths,
    # head sizes that are no multiples of 8 (scalar attention kernels in both serving types), kept keys beyond the window's size
    "plain": dict(streams=None, width=44, vocab=61, layers=("attention_2", "attention", "parallel"), ffs=("moe", "dense", "moe"),
                  left=dict(heads=3, kv_heads=3, dim=6, vdim=10, scale=0.4, bias_max=17, size=3, keep_first=9),
                  right=dict(heads=3, dim=6, vdim=5, gate_cap=30.0),
                  att2=dict(heads=2, kv_heads=1, dim=12, scale=0.3, softcap=50.0, size=7, dims=4, base=100.0, scaling=None),
                  att=dict(heads=3, kv_heads=1, dim=10, vdim=6, scale=0.3, diff=0.8, dims=6, base=50.0),
                  moe=dict(ff=12, experts=3, identity=0, top=3, scale=0.7, groups=None)),
    # sizes of a small real model: sizes on the tensor-core tiles, many heads and experts, eight streams, long windows
    "medium": dict(vocab=1000, width=256, streams=8, dense_ff=512, layers=("attention", "parallel", "shared", "attention_2"),
                   ffs=("moe", "dense", "moe", "moe"),
                   left=dict(heads=8, kv_heads=2, dim=64, vdim=64, scale=0.125, bias_max=128, size=48, keep_first=33),
                   right=dict(heads=4, dim=64, vdim=128, gate_cap=15.0),
                   att2=dict(heads=8, kv_heads=4, dim=128, scale=0.09, softcap=20.0, size=100, dims=64, base=2e5,
                             scaling=dict(factor=6.0, original=64, fast=16.0, slow=1.0)),
                   att=dict(heads=8, kv_heads=2, dim=64, vdim=128, scale=0.125, diff=0.2, dims=64, base=1e4),
                   moe=dict(ff=64, experts=13, identity=3, top=4, scale=2.5, groups=8, keep=3)),
    # odd counts everywhere: a width that is odd, five streams, odd heads, value sizes off every tile
    "odd": dict(vocab=333, width=51, streams=5, dense_ff=30, layers=("parallel", "attention", "attention_2", "shared", "attention"),
                ffs=("moe", None, "dense", "moe", "dense"),
                left=dict(heads=6, kv_heads=3, dim=10, vdim=14, scale=0.2, bias_max=50, size=9, keep_first=4),
                right=dict(heads=5, dim=10, vdim=7, gate_cap=5.0),
                att2=dict(heads=5, kv_heads=5, dim=14, scale=0.35, softcap=3.0, size=16, dims=10, base=300.0,
                          scaling=dict(factor=1.5, original=20, fast=3.0, slow=1.0)),
                att=dict(heads=6, kv_heads=2, dim=14, vdim=10, scale=0.3, diff=0.1, dims=2, base=7.0),
                moe=dict(ff=20, experts=4, identity=5, top=3, scale=1.2, groups=3, keep=2)),
}
REL = {"mixed": 10, "ones": 4, "plain": 7, "medium": 32, "odd": 9}


def _decisive_routers(cfg, W):
    """For bf16 runs: a choice of experts that rounding cannot flip (well separated corrections decide alone; the weights, which
    the corrections do not enter, stay token dependent).  Token-dependent choices are checked in float32."""
    out = dict(W)
    g = torch.Generator().manual_seed(11)
    for k in W:
        if k.endswith("mlp.router"):
            out[k[:-6] + "correction"] = (torch.randperm(W[k].shape[0], generator=g).float() * 2.0).to(W[k].dtype)
    return out


def _model(name, seed=0, dtype="fp32"):
    cfg = O.make_config(**SHAPES[name])
    W = O.random_weights(cfg, seed=seed, rel_buckets=REL[name])
    return cfg, (_decisive_routers(cfg, W) if dtype == "bf16" else W)


def _plan(entries, slots, start=None, pages=None, page=16):
    """A hand-made step plan: entries = token counts of sequences that already hold ``start`` tokens; pages given or consecutive."""
    from nanorlhf_b200.sampler.hybrid_sampler import StepPlan
    E, T = len(entries), sum(entries)
    start = start or [0] * E
    MB = max((s + n + page - 1) // page for s, n in zip(start, entries))
    cu, te, pos, kv, bt, nxt = [0], [], [], [], [], 0
    for e, (s, n) in enumerate(zip(start, entries)):
        need = (s + n + page - 1) // page
        pg = pages[e] if pages else list(range(nxt, nxt + need))
        nxt += need
        bt.append(pg + [0] * (MB - len(pg)))
        for j in range(n):
            te.append(e)
            pos.append(s + j)
            kv.append(pg[(s + j) // page] * page + (s + j) % page)
        cu.append(cu[-1] + n)
    flat = [0] * T + cu + te + pos + kv + start + slots + [x for r in bt for x in r]
    return StepPlan(torch.tensor(flat, dtype=torch.int32, device="cuda"), E, T, MB)


# ---- mechanisms alone ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("W,S,T", [(48, 3, 5), (51, 1, 3), (256, 8, 4), (1030, 4, 2)])
def test_stream_boundary(W, S, T):
    """Embedding into every stream; the boundary that mixes the streams, adds a sublayer's result (with bias and the identity
    experts' share of its input) and layer-norms the next sublayer's input; the final sum."""
    from nanorlhf_b200.ops import hybrid as hy
    g = torch.Generator().manual_seed(W + S)
    emb = torch.randn(20, W, generator=g)
    tok = torch.randint(0, 20, (T,), generator=g)
    xs = torch.empty(T, S, W, device="cuda")
    hy.embed_streams(emb.cuda(), tok.int().cuda(), 1.7, xs)
    assert torch.allclose(xs.cpu(), (emb[tok] * 1.7)[:, None, :].expand(T, S, W), atol=1e-6)
    x = torch.randn(T, S, W, generator=g).double()
    o, ob, sw = torch.randn(T, W, generator=g).double(), torch.randn(W, generator=g).double(), torch.rand(T, generator=g).double()
    mix, outw, inw = torch.randn(S, S, generator=g).double(), torch.randn(S, generator=g).double(), torch.randn(S, generator=g).double()
    lw, lb = torch.randn(W, generator=g).double(), torch.randn(W, generator=g).double()
    hprev = torch.randn(T, W, generator=g).double()
    for use_sw, use_b, use_in in ((True, True, True), (False, False, False)):
        y = o + (ob if use_b else 0) + (sw[:, None] * hprev if use_sw else 0)
        xn = torch.einsum("sr,tsw->trw", mix, x) + outw[None, :, None] * y[:, None, :]      # mix is indexed [from, to]
        u = (xn * inw[None, :, None]).sum(1) if use_in else xn.sum(1)
        want_h = O.layer_norm(u, lw, lb, 1e-5)
        xs = x.float().cuda()
        h = hprev.float().cuda()
        f = lambda t: t.float().cuda()
        hy.hyper_boundary(xs, f(o), f(ob) if use_b else None, f(sw) if use_sw else None, f(mix), f(outw), f(inw) if use_in else None,
                          f(lw), f(lb), 1e-5, h)
        assert (xs.double().cpu() - xn).abs().max() < 1e-4
        assert (h.double().cpu() - want_h).abs().max() < 2e-4
    # opening boundary: nothing closes, the streams stay as they are
    xs = x.float().cuda()
    h = torch.empty(T, W, device="cuda")
    hy.hyper_boundary(xs, None, None, None, None, None, inw.float().cuda(), lw.float().cuda(), None, 1e-5, h)
    assert torch.equal(xs.cpu(), x.float())
    assert (h.double().cpu() - O.layer_norm((x * inw[None, :, None]).sum(1), lw, 0.0, 1e-5)).abs().max() < 2e-4


@pytest.mark.parametrize("E,n_real,top,groups,keep", [(8, 5, 3, 4, 2), (16, 12, 4, 4, 3), (6, 6, 2, 3, 1), (9, 4, 3, 3, 2), (4, 2, 1, 1, 1),
                                                      (64, 60, 8, 16, 5)])
def test_router_groups(E, n_real, top, groups, keep):
    """Choice among the experts of the best groups only (negative choice scores included), weights from the uncorrected scores."""
    from nanorlhf_b200.ops import hybrid as hy
    g = torch.Generator().manual_seed(E * top)
    T, Wd = 200, 12
    h = torch.randn(T, Wd, generator=g).double()
    w = {"r.router": torch.randn(E, Wd, generator=g).double(), "r.correction": torch.randn(E, generator=g).double() * 0.3 - 0.4}
    mlp = {"router": {"experts": n_real, "identity": E - n_real, "top": top, "scale": 1.3, "groups": {"count": groups, "keep": keep}}}
    ids_w, wt_w = O.route(w, "r.", mlp, h)
    z = (h @ w["r.router"].T).float().cuda()
    ids = torch.empty(T, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(T, top, device="cuda")
    self_w = torch.empty(T, device="cuda")
    hy.moe_route_all(z, w["r.correction"].float().cuda(), n_real, top, 1.3, ids=ids, wts=wts, self_w=self_w, groups=groups, keep=keep)
    ids, wts = ids.cpu().long(), wts.cpu().double()
    same = (ids == ids_w).all(-1)
    assert same.double().mean() > 0.97                      # a float tie may flip a choice; the others must agree exactly
    real = ids_w < n_real
    assert ((wts - torch.where(real, wt_w, torch.zeros_like(wt_w)))[same].abs().max()) < 1e-5
    assert ((self_w.cpu().double() - (wt_w * ~real).sum(-1))[same].abs().max()) < 1e-5
    grp = E // groups                                       # every choice lies in one of the `keep` best groups
    s = torch.softmax(h @ w["r.router"].T, -1) + w["r.correction"]
    best = s.view(T, groups, grp).max(-1).values.topk(keep, dim=-1).indices
    assert bool(((ids // grp)[:, :, None] == best[:, None, :]).any(-1)[same].all())


@pytest.mark.parametrize("H,D,Dv,impl", [(2, 16, 24, "auto"), (1, 8, 8, "column"), (3, 6, 5, "global"), (4, 64, 128, "auto"),
                                         (2, 40, 72, "column"), (2, 128, 200, "auto"), (1, 130, 9, "auto"), (5, 10, 7, "column")])
def test_matrix_memory_scan(H, D, Dv, impl):
    """The scan with its carried state (S, normaliser, running maximum) against the token loop: a batch of entries of unequal
    length, continued in a second step in other slots' company, gates that swing far both ways."""
    from nanorlhf_b200.ops import hybrid as hy
    g = torch.Generator().manual_seed(H * D + Dv)
    lens, cap = [7, 1, 33], 9.0
    slots = [2, 0, 3]
    state = torch.full((4, H, D, Dv + 1), 7.0, device="cuda")        # stale content that a new sequence must not see
    mstate = torch.full((4, H), -3.0, device="cuda")
    cols = 2 * H * D + H * Dv + 2 * H
    carried = [None] * 3
    held = [0, 0, 0]
    for step in range(2):
        data = [torch.randn(n, cols, generator=g) for n in lens]
        for d in data:
            d[:, -2 * H:] *= 6.0                                       # raw gates well past the cap's linear range
        ib, fb = torch.randn(H, generator=g), torch.randn(H, generator=g) + 1.0
        plan = _plan(lens, slots, start=list(held))
        U = torch.cat(data).cuda()
        o = torch.empty(sum(lens), H * (Dv + 1), device="cuda")
        m = torch.empty(sum(lens), H, device="cuda")
        cq, ck, cv, ci = 0, H * D, 2 * H * D, 2 * H * D + H * Dv
        hy.mlstm_scan(U, cq, ck, cv, ci, ci + H, ib.cuda(), fb.cuda(), cap, D ** -0.5, state, mstate, o, m, plan, impl=impl)
        gate, w = torch.randn(sum(lens), H * Dv, generator=g), torch.rand(H * Dv, generator=g) + 0.5
        out = torch.empty(sum(lens), H * Dv, device="cuda")
        hy.mlstm_out(o, m, gate.cuda(), w.cuda(), 1e-5, 1.1, out, H)
        lo = 0
        for e, n in enumerate(lens):
            d = data[e].double()
            q = d[:, cq:ck].view(n, H, D) * D ** -0.5
            k, v = d[:, ck:cv].view(n, H, D), d[:, cv:ci].view(n, H, Dv)
            ig = cap * torch.tanh((d[:, ci:ci + H] + ib) / cap)
            fg = torch.nn.functional.logsigmoid(cap * torch.tanh((d[:, ci + H:] + fb) / cap))
            y, carried[e] = O.matrix_memory_core(q, k, v, ig, fg, carried[e])
            want = 1.1 * O.unit_rms(y, 1e-5).reshape(n, H * Dv) * w * torch.sigmoid(gate[lo:lo + n].double())
            assert (out[lo:lo + n].double().cpu() - want).abs().max() < 2e-4 * max(1.0, want.abs().max().item())
            S, nrm, mm = carried[e]
            assert (state[slots[e], :, :, :Dv].double().cpu() - S).abs().max() < 1e-4 * max(1.0, S.abs().max().item())
            assert (state[slots[e], :, :, Dv].double().cpu() - nrm).abs().max() < 1e-4 * max(1.0, nrm.abs().max().item())
            assert (mstate[slots[e]].double().cpu() - mm).abs().max() < 1e-4
            held[e] += n
            lo += n
        lens = [1, 12, 2]


def _plain_attention(q, k, v, pos_q, window, scale, softcap=0.0, keep_first=0, rel=None, bias_max=0, sink=None, v_div=1):
    """q [Tq, Hq, D] at positions pos_q over keys k [Tk, Hk, D] / values v [Tk, Hk / v_div, Dv] at positions 0 .. Tk-1, float64."""
    Tq, Hq, _ = q.shape
    Tk, Hk, _ = k.shape
    j = torch.arange(Tk)
    dist = pos_q[:, None] - j[None, :]
    vis = (dist >= 0) & ((dist < window) | (j[None, :] < keep_first))
    out = []
    for h in range(Hq):
        g = h // (Hq // Hk)
        sc = (q[:, h] @ k[:, g].T) * scale
        if softcap > 0:
            sc = softcap * torch.tanh(sc / softcap)
        if rel is not None:
            B = rel.shape[0]
            bk = torch.tensor([[O.distance_bucket(int(d), B, bias_max) if d >= 0 else 0 for d in row] for row in dist.tolist()])
            sc = sc + rel[:, h][bk]
        pr = O.softmax_rows(sc, vis, sink=None if sink is None else sink[h].expand(Tq))
        out.append(pr @ v[:, g // v_div])
    return torch.stack(out, 1)


ATT_CASES = {
    # name: (Hq, Hk, D, Dv, window, terms)
    "cap_sink": (4, 2, 24, 24, 20, dict(softcap=4.0, sink=True)),
    "kept_bias": (4, 2, 16, 8, 12, dict(keep_first=5, rel=10, bias_max=40)),
    "kept_far": (6, 3, 40, 56, 44, dict(keep_first=19, rel=24, bias_max=200)),
    "kept_wide": (2, 1, 8, 8, 3, dict(keep_first=70)),                # more kept keys than a key block holds, a tiny window
    "two_maps": (8, 4, 16, 24, 1 << 30, dict(v_div=2)),
    "two_maps_wide": (12, 4, 40, 72, 1 << 30, dict(v_div=2)),
    "all": (6, 6, 64, 32, 33, dict(softcap=2.5, sink=True, keep_first=17, rel=8, bias_max=100, v_div=3)),
    "odd": (3, 3, 6, 10, 5, dict(softcap=7.0, sink=True, keep_first=2, rel=7, bias_max=17)),
    "window_one": (2, 2, 8, 8, 1, dict(sink=True)),
}


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("case", sorted(ATT_CASES))
def test_attention_terms(case, dtype):
    """Every optional term of the paged attention kernels, alone and together, on every kernel that takes the shape: a prompt cut
    into portions (the second one starting inside a page), then single tokens, against a plain softmax over the whole sequence.
    Keys at the window's edges and among the kept first ones are made to stand out, so that a mask one token off shows."""
    from nanorlhf_b200.ops import hybrid as hy
    Hq, Hk, D, Dv, window, terms = ATT_CASES[case]
    v_div = terms.get("v_div", 1)
    Hv = Hk // v_div
    g = torch.Generator().manual_seed(len(case) + D)
    n = 150
    q, k, v = torch.randn(n, Hq, D, generator=g), torch.randn(n, Hk, D, generator=g), torch.randn(n, Hv, Dv, generator=g)
    keep = terms.get("keep_first", 0)
    for t in (60, 100, 149):                                  # the query at t looks hard at the keys around its mask's edges
        for j in {t - window, t - window + 1, keep - 1, keep}:
            if 0 <= j < n:
                k[j] = q[t, ::Hq // Hk] * 1.5 + 0.1 * k[j]
    rel = torch.randn(terms["rel"], Hq, generator=g) if "rel" in terms else None
    sink = torch.randn(Hq, generator=g) if terms.get("sink") else None
    wd = torch.float32 if dtype == "fp32" else torch.bfloat16
    kq, vq = (k.to(wd).double(), v.to(wd).double())           # the pages hold rounded keys and values
    scale = 0.7 / D ** 0.5
    want = _plain_attention(q.double(), kq, vq, torch.arange(n), window, scale, terms.get("softcap", 0.0), keep, None if rel is None else rel.double(),
                            terms.get("bias_max", 0), None if sink is None else sink.double(), v_div).reshape(n, Hq * Dv)
    table = hy.distance_bias_table(rel.cuda(), terms["bias_max"]) if rel is not None else None
    impls = ["tile", "simple", "auto"] + (["mma"] if dtype == "bf16" and D % 8 == 0 and Dv % 8 == 0 else [])
    order = torch.randperm(16, generator=g).tolist()          # pages in no order
    # over bf16 pages the result may also be asked for as float32 (maps that are subtracted before they are rounded)
    for impl, od in [(i, wd) for i in impls] + ([(i, torch.float32) for i in impls] if dtype == "bf16" else []):
        kc = torch.zeros(16, Hk, 16, D, dtype=wd, device="cuda")
        vc = torch.zeros(16, Hv, 16, Dv, dtype=wd, device="cuda")
        got, lo = [], 0
        for cnt in [70, 41, 2] + [1] * 37:
            plan = _plan([cnt], [0], start=[lo], pages=[order[:(lo + cnt + 15) // 16]])
            qs = q[lo:lo + cnt].reshape(cnt, Hq * D).cuda().contiguous()
            hy.rot_kv_write(qs, None, k[lo:lo + cnt].reshape(cnt, -1).cuda(), None, v[lo:lo + cnt].reshape(cnt, -1).cuda(), None, 0, 1.0, True,
                            False, None, None, 1e-6, plan, kc, vc)
            out = torch.empty(cnt, Hq * Dv, dtype=od, device="cuda")
            hy.window_attention(qs, kc, vc, plan, window, scale, 1.0, out, impl=impl, head_sink=None if sink is None else sink.cuda(),
                                softcap=terms.get("softcap", 0.0), keep_first=keep, dist_bias=table, v_div=v_div)
            got.append(out.double().cpu())
            lo += cnt
        got = torch.cat(got)
        tol = 2e-5 if dtype == "fp32" else 2.5e-2
        err = (got - want).abs().max().item()
        assert err < tol * max(1.0, want.abs().max().item()), (impl, od, err)


@pytest.mark.parametrize("layout,dims,D,scaling,norm,bias,own_v", [("interleaved", 8, 16, None, False, False, True),
                                                                   ("half", 16, 24, dict(factor=4.0, original=32, fast=8.0, slow=1.0), True, True, False),
                                                                   ("half", 2, 6, None, True, False, True), ("interleaved", 0, 8, None, False, True, False),
                                                                   ("interleaved", 40, 40, dict(factor=6.0, original=512, fast=16.0, slow=2.0), True, True, True)])
def test_rotation_and_cache_write(layout, dims, D, scaling, norm, bias, own_v):
    """Queries in place and keys / values in their pages: bias, rotation of the first columns in either pairing with the stretch,
    unit norm after the rotation, values that are the keys as projected; far positions (angles are reduced in double)."""
    from nanorlhf_b200.ops import hybrid as hy
    Hq, Hk, Dv = 4, 2, (12 if own_v else D)
    g = torch.Generator().manual_seed(D + dims)
    starts, cnts = [0, 100000, 37], [5, 3, 20]
    plan = _plan(cnts, [0, 1, 2], start=starts, pages=[[3], list(range(10, 10 + (100003 + 15) // 16)), [4, 5, 6, 7]])
    T = sum(cnts)
    q, k, v = torch.randn(T, Hq * D, generator=g), torch.randn(T, Hk * D, generator=g), torch.randn(T, Hk * Dv, generator=g)
    qb, kb = (torch.randn(Hq * D, generator=g), torch.randn(Hk * D, generator=g)) if bias else (None, None)
    pos = torch.tensor([s + j for s, c in zip(starts, cnts) for j in range(c)])
    rot = {"dims": dims, "base": 1e4, **({"scaling": scaling} if scaling else {})}
    qd = (q.double() + (qb.double() if bias else 0)).view(T, Hq, D)
    kd = (k.double() + (kb.double() if bias else 0)).view(T, Hk, D)
    if dims:
        cos, sin = O.rotary_tables(rot, pos)
        qr, kr = O.rotate_front(qd, cos, sin, dims, layout), O.rotate_front(kd, cos, sin, dims, layout)
    else:
        qr, kr = qd, kd
    if norm:
        qr, kr = O.unit_rms(qr, 1e-5), O.unit_rms(kr, 1e-5)
    freq = mult = None
    if dims:
        f, mult = hy.rotary_frequencies(dims, 1e4, scaling)
        freq = torch.tensor(f, dtype=torch.float64, device="cuda")
    pages = 10 + (100003 + 15) // 16 + 1
    kc, vc = torch.zeros(pages, Hk, 16, D, device="cuda"), torch.zeros(pages, Hk, 16, Dv, device="cuda")
    qs = q.cuda()
    hy.rot_kv_write(qs, qb.cuda() if bias else None, k.cuda(), kb.cuda() if bias else None, v.cuda() if own_v else None, freq, dims, mult or 1.0,
                    layout == "interleaved", norm, None, None, 1e-5, plan, kc, vc)
    assert (qs.double().cpu().view(T, Hq, D) - qr).abs().max() < 3e-5
    slot = plan.kv_slot.cpu().long()
    kgot = kc.permute(0, 2, 1, 3).reshape(-1, Hk, D)[slot].double().cpu()
    vgot = vc.permute(0, 2, 1, 3).reshape(-1, Hk, Dv)[slot].double().cpu()
    assert (kgot - kr).abs().max() < 3e-5
    assert (vgot - (v.double().view(T, Hk, Dv) if own_v else kd)).abs().max() < 1e-6
    # queries only (a layer that reads another layer's pages): the pages stay as they are
    kc2, vc2 = kc.clone(), vc.clone()
    qs2 = q.cuda()
    hy.rot_kv_write(qs2, qb.cuda() if bias else None, None, None, None, freq, dims, mult or 1.0, layout == "interleaved", norm, None, None, 1e-5,
                    plan, kc2, vc2)
    assert torch.equal(qs2, qs) and torch.equal(kc2, kc) and torch.equal(vc2, vc)


@pytest.mark.parametrize("H,G,Dv", [(4, 2, 24), (1, 1, 8), (6, 2, 10), (8, 8, 96)])
def test_differential_combine(H, G, Dv):
    from nanorlhf_b200.ops import hybrid as hy
    g = torch.Generator().manual_seed(H + Dv)
    T, R = 9, H // G
    a = torch.randn(T, H, 2, Dv, generator=g)                 # [token, head, map, value]
    gate = torch.randn(T, H * Dv, generator=g)
    lam, diff = 0.37, 0.3
    o = a[:, :, 0].double() - lam * a[:, :, 1].double()
    want = (O.unit_rms(o, 1e-5) * (1.0 - diff)).reshape(T, H * Dv) * torch.sigmoid(gate.double()) * 0.6
    packed = a.view(T, G, R, 2, Dv).permute(0, 1, 3, 2, 4).reshape(T, 2 * H * Dv).contiguous().cuda()      # (kv head, map, head of the group)
    out = torch.empty(T, H * Dv, device="cuda")
    hy.diff_combine(packed, lam, 1.0 - diff, 1e-5, gate.cuda(), 0.6, out, H, G)
    assert (out.double().cpu() - want).abs().max() < 1e-5


# ---- whole models under schedules ----------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("name", sorted(SHAPES))
def test_whole_prompt_matches_oracle(tmp_path, name, dtype):
    cfg, W = _model(name, dtype=dtype)
    eng = _engine(tmp_path, cfg, W, dtype)
    toks = _tokens(cfg, 150, 1)
    got = _run_alone(eng, toks, [len(toks)])
    Wq = {k: v.to(torch.bfloat16) for k, v in W.items()} if dtype == "bf16" else W
    want = O.forward(Wq, cfg, toks)
    assert _close(got, want, dtype), _rows(got, want).max().item()


@pytest.mark.parametrize("name", ["mixed", "odd", "plain"])
def test_layers_match_oracle(tmp_path, name):
    """The sum of the streams after every layer (float32)."""
    import numpy as np
    from nanorlhf_b200.sampler.hybrid_sampler import StepPlan
    cfg, W = _model(name, seed=3)
    eng = _engine(tmp_path, cfg, W, "fp32")
    toks = _tokens(cfg, 40, 2)
    keep_o, keep_e = [], []
    O.forward(W, cfg, toks, keep_o)
    sid = eng.open()
    data, E, T, MB = eng.sched.plan([sid], [len(toks)], 0)
    data[:T] = np.asarray(toks, dtype=np.int32)
    eng._forward_hyper(StepPlan(torch.from_numpy(data).cuda(), E, T, MB), [], keep_e)
    assert len(keep_e) == len(keep_o) == len(cfg["layers"])
    for i, (a, b) in enumerate(zip(keep_e, keep_o)):
        assert (a.double().cpu() - b).abs().max() < 2e-4 * max(1.0, b.abs().max().item()), i


@pytest.mark.parametrize("name", ["mixed", "ones", "odd", "medium"])
def test_prefill_against_token_by_token_and_portions(tmp_path, name):
    """The logits do not depend on how a sequence is cut: all at once, one token at a time (long decoding through windows,
    kept keys and the matrix memory), and portions of several sizes down to two tokens, starting anywhere in a page."""
    cfg, W = _model(name, seed=4)
    eng = _engine(tmp_path, cfg, W, "fp32")
    toks = _tokens(cfg, 140, 5)
    whole = _run_alone(eng, toks, [len(toks)])
    want = O.forward(W, cfg, toks)
    assert _close(whole, want, "fp32")
    for cuts in ([1] * len(toks), _cuts(len(toks), [2, 3, 17, 2, 31, 5, 16, 1, 64]), _cuts(len(toks), [50, 2]), [3] + [1] * 137):
        got = _run_alone(eng, toks, cuts)
        assert _rows(got, whole).max() < F32_TOL, cuts[:4]


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("name", ["mixed", "odd"])
def test_mixed_batches_and_reuse(tmp_path, name, dtype):
    """Up to four live sequences, prompt portions beside single tokens; pages and slots are given back and used again by later
    sequences; every sequence must see what it sees alone."""
    cfg, W = _model(name, seed=6, dtype=dtype)
    eng = _engine(tmp_path, cfg, W, dtype, pool_tokens=4 * 96, slots=4)
    lens = [90, 33, 2, 61, 77, 1, 48, 95, 18]
    seqs = [_tokens(cfg, n, 20 + i) for i, n in enumerate(lens)]
    Wq = {k: v.to(torch.bfloat16) for k, v in W.items()} if dtype == "bf16" else W
    want = [O.forward(Wq, cfg, s) for s in seqs]
    got = [[] for _ in seqs]
    fed = [0] * len(seqs)
    live, nxt, step = {}, 0, 0
    sizes = [13, 2, 40, 1, 1, 7, 1, 29]
    while nxt < len(seqs) or live:
        while len(live) < 4 and nxt < len(seqs):
            live[nxt] = eng.open()
            nxt += 1
        entries, who = [], []
        for i, sid in live.items():
            if (step + i) % 5 == 4:                          # a request may sit a step out
                continue
            n = min(sizes[(step + 3 * i) % len(sizes)], lens[i] - fed[i])
            entries.append((sid, seqs[i][fed[i]:fed[i] + n], list(range(n))))
            who.append((i, n))
        step += 1
        if not entries:
            continue
        out = eng.step(entries).double().cpu()
        o = 0
        for i, n in who:
            got[i].append(out[o:o + n])
            o += n
            fed[i] += n
            if fed[i] == lens[i]:
                eng.close(live.pop(i))
    for i in range(len(seqs)):
        assert _close(torch.cat(got[i]), want[i], dtype), (i, _rows(torch.cat(got[i]), want[i]).max().item())


def test_far_keys_and_window_edges_in_a_model(tmp_path):
    """A long sequence through a model whose embedding makes one early token and the tokens at the masks' edges matter: the
    differential layers must reach the far token, the windowed ones must not, in prompts and in decoding."""
    cfg, W = _model("mixed", seed=8)
    W = dict(W)
    W["embed"] = W["embed"].clone()
    W["embed"][7] *= 6.0                                      # token 7 stands out wherever it is visible
    eng = _engine(tmp_path, cfg, W, "fp32", pool_tokens=2048)
    toks = [t if t != 7 else 8 for t in _tokens(cfg, 700, 9)]
    for at in (0, 3, 5, 650, 680, 688, 699 - 12, 699 - 20):
        toks[at] = 7
    want = O.forward(W, cfg, toks)
    got = _run_alone(eng, toks, [300, 333, 2, 33] + [1] * 32)
    assert _close(got, want, "fp32"), _rows(got, want).max().item()


def test_greedy_generation_through_the_entry_point(tmp_path):
    """Greedy generation through ``sampler.engine.generate`` (scheduler, chunked prefill, graph-replayed single-token steps)
    against the oracle's argmax continuation."""
    from nanorlhf_b200.models.registry import load_model
    from nanorlhf_b200.sampler.engine import generate, get_native_engine, release_native_engine

    class _Tok:
        pad_token_id = 0
        eos_token_id = None

    cfg, W = _model("mixed", seed=10)
    path = _save(tmp_path, cfg, W)
    model = load_model(path, torch_dtype=torch.float32, device="cuda")
    prompts = [_tokens(cfg, n, 40 + n) for n in (5, 37, 1, 70, 9)]
    new = 24
    out = generate(1, model, _Tok(), prompts, 0.0, new, top_p=1.0, seed=1, rollout_dtype="fp32", max_num_seqs=3,
                   prefill_token_budget=32).cpu()
    for p, row in zip(prompts, out.tolist()):
        seq = list(p)
        for j, t in enumerate(row):
            lg = O.forward(W, cfg, seq)[-1]
            top2 = lg.topk(2).values
            if top2[0] - top2[1] < 1e-3:                      # a near tie: either token is right, and the texts part from here
                break
            assert t == int(lg.argmax()), (len(p), j)
            seq.append(t)
    assert get_native_engine(model, rollout_dtype="fp32").stats["graph_replays"] > 0      # decode steps replay a CUDA graph
    release_native_engine(model)


def test_trace_runner_command_line(tmp_path):
    """bin/trace_run replays a trace of steps (portions, single tokens, a request that ends and whose slot is used again)."""
    import numpy as np
    cfg, W = _model("odd", seed=12)
    path = _save(tmp_path, cfg, W)
    a, b, c = _tokens(cfg, 40, 1), _tokens(cfg, 21, 2), _tokens(cfg, 9, 3)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:30], "want": [0, 29]}, {"id": "b", "tokens": b[:2], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[30:31], "want": [0]}, {"id": "b", "tokens": b[2:], "want": [18]}], "end": ["b"]},
             {"step": 2, "entries": [{"id": "c", "tokens": c, "want": [8]}, {"id": "a", "tokens": a[31:], "want": [8]}], "end": ["a", "c"]}]
    out = os.path.join(str(tmp_path), "out")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", path, "--dtype", "float32", "--out", out,
                        "--max-tokens", "192", "--slots", "2"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True,
                       text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb, wc = O.forward(W, cfg, a), O.forward(W, cfg, b), O.forward(W, cfg, c)
    want = {0: torch.stack([wa[0], wa[29]]), 1: torch.stack([wa[30], wb[20]]), 2: torch.stack([wc[8], wa[39]])}
    for st, w in want.items():
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{st}.f32"), dtype="<f4").reshape(w.shape[0], -1).copy()).double()
        assert _close(got, w, "fp32"), st


def test_sampler_command_line(tmp_path):
    """``python -m nanorlhf_b200.sampler`` on a Lukarax checkpoint: greedy tokens follow the oracle; sampled tokens repeat under a seed."""
    cfg, W = _model("plain", seed=14)
    path = _save(tmp_path, cfg, W)
    prompt = _tokens(cfg, 11, 3)
    base = [sys.executable, "-m", "nanorlhf_b200.sampler", "--model", path, "--prompt-ids", ",".join(map(str, prompt)), "--dtype", "float32"]

    def run(extra):
        r = subprocess.run(base + extra, capture_output=True, text=True, timeout=900, cwd=ROOT)
        assert r.returncode == 0, r.stderr[-2000:]
        return [json.loads(l)["tokens"] for l in r.stdout.splitlines() if l.startswith("{")]
    greedy = run(["--max-tokens", "6"])[0]
    seq = list(prompt)
    for t in greedy:
        lg = O.forward(W, cfg, seq)[-1]
        top2 = lg.topk(2).values
        if top2[0] - top2[1] < 1e-3:
            break
        assert t == int(lg.argmax())
        seq.append(t)
    a = run(["--max-tokens", "8", "--temperature", "0.9", "--top-p", "0.9", "--seed", "5", "--n", "2"])
    b = run(["--max-tokens", "8", "--temperature", "0.9", "--top-p", "0.9", "--seed", "5", "--n", "2"])
    assert a == b and len(a) == 2 and all(0 <= t < cfg["vocab"] for row in a for t in row)
