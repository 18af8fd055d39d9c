"""Damilix on the step engine against the plain float64 oracle (tests/damilix_oracle.py): small random models of several
shapes, written to disk as a checkpoint, loaded through the model registry and run through ``HybridSampler.step`` /
``generate`` under different schedules (whole prompts, token by token, portions, mixed batches, reused pages and slots),
and every new mechanism alone against the oracle's function for it."""
import json
import os
import subprocess
import sys

import pytest
import torch

import damilix_oracle as O

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
F32_TOL = 2e-4
BF16_TOL = 8e-2        # five post-normed layers of width 48 in bf16: mean row error 1 - 3 %, a tail up to 15 %


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


def _rel(got, want):
    """Worst row error relative to the RMS of the oracle's logits."""
    return ((got - want).pow(2).mean(-1).sqrt().max() / want.pow(2).mean().sqrt()).item()


def _close(got, want, dtype):
    rows = (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()
    if dtype == "fp32":
        return bool(rows.max() < F32_TOL)
    return bool((rows > BF16_TOL).double().mean() <= 0.12 and rows.max() < 3 * BF16_TOL and rows.mean() < 0.5 * BF16_TOL)


def _cuts(total, sizes):
    out, i, k = [], 0, 0
    while i < total:
        n = min(sizes[k % len(sizes)], total - i)
        out.append(n)
        i += n
        k += 1
    return out


SHAPES = {
    # every layer type and feed-forward kind, sizes that differ from their neighbours
    "mixed": dict(layers=("gla", "latent", "latent2", "gla", "latent"), ffs=("dense", "moe", "dense", "moe", None)),
    # values that usual defaults make equal or 1: one head, top 1, one expert + one identity, no shared expert, scale 1, tau 1,
    # rot_dim == dim, kv_rank == vdim, side input of one column, rank 1 decay projection
    "ones": dict(layers=("latent2", "gla", "latent"), ffs=("moe", "moe", "dense"), side=1, rank=1, gla=dict(heads=1, dim=8, vdim=8, tau=1.0),
                 latent=dict(heads=1, dim=8, rot_dim=8, vdim=16, kv_rank=16, scale=1.0, scaling=None),
                 latent2=dict(heads=1, dim=4, rot_dim=4, vdim=4, kv_rank=4, scale=1.0),
                 moe=dict(ff=8, experts=1, identity=1, top=1, scale=1.0, shared=0)),
    # no token input, no identity experts, every expert chosen, a rotation that turns only part of the rotated columns,
    # a stretch on the half-layout rotation, a width that is no multiple of 8
    "plain": dict(width=44, layers=("latent", "latent2", "gla"), ffs=("moe", "dense", "moe"), side=0,
                  latent=dict(heads=2, dim=6, rot_dim=8, dims=4, vdim=6, kv_rank=10, scaling=None),
                  latent2=dict(heads=3, dim=8, rot_dim=6, vdim=12, kv_rank=20, scaling=dict(factor=3.0, original=16, fast=4.0, slow=0.5)),
                  gla=dict(heads=3, dim=12, vdim=4, tau=3.0), moe=dict(ff=12, experts=3, identity=0, top=3, scale=0.7, shared=20)),
    # sizes of a small real model: wide latent (key rows past 128 columns), many heads, many experts, sizes on the GEMM tiles
    "medium": dict(vocab=1000, width=256, layers=("gla", "latent", "gla", "latent2"), ffs=("dense", "moe", "moe", "dense"), side=16, rank=16,
                   dense_ff=512, gla=dict(heads=4, dim=64, vdim=128, tau=16.0),
                   latent=dict(heads=8, dim=32, rot_dim=16, vdim=48, kv_rank=160, scale=0.12, base=5e5,
                               scaling=dict(factor=2.5, original=128, fast=24.0, slow=1.5)),
                   latent2=dict(heads=4, dim=64, rot_dim=32, vdim=64, kv_rank=96, scale=0.1, base=1e4),
                   moe=dict(ff=64, experts=8, identity=2, top=2, scale=2.0, shared=128)),
    # a width that is odd (no vector path anywhere, every GEMM off the tensor-core tiles), tiny feed-forwards
    "narrow": dict(width=51, vocab=101, side=3, layers=("latent", "gla", "latent2"), ffs=("moe", "dense", "moe"), dense_ff=30,
                   moe=dict(ff=10, experts=3, identity=1, top=2, scale=1.1, shared=6)),
    # sizes off every tile: odd counts of heads and experts, head sizes that are no multiples of 8 (key rows of 4 k + 2 columns
    # run on the one-query kernel), more identity than real experts
    "odd": dict(vocab=333, width=72, layers=("latent", "gla", "latent2"), ffs=("moe", "dense", "moe"), side=5, rank=3, dense_ff=100,
                gla=dict(heads=5, dim=10, vdim=6, tau=2.5),
                latent=dict(heads=5, dim=10, rot_dim=6, vdim=14, kv_rank=20, scale=0.2, base=300.0, scaling=dict(factor=1.5, original=20, fast=3.0, slow=1.0)),
                latent2=dict(heads=7, dim=6, rot_dim=10, vdim=10, kv_rank=28, scale=0.4),
                moe=dict(ff=20, experts=2, identity=3, top=3, scale=1.2, shared=12)),
}


def _decisive_routers(cfg, W):
    """For bf16 runs: a choice of experts that rounding cannot flip.  With random routers some token always has two choice
    scores nearly tied, bf16 rounding of the router's input picks the other one and that token's logits move by far more than
    rounding.  Here the corrections are well separated and decide alone, while the weights (the softmax scores, which the
    corrections do not enter) stay token dependent.  Token-dependent choices are checked in float32."""
    out = dict(W)
    g = torch.Generator().manual_seed(11)
    for k in W:
        if k.endswith("mlp.router"):
            out[k[:-6] + "correction"] = (torch.randperm(W[k].shape[0], generator=g).float() * 2.0).to(W[k].dtype)
    return out


def _model(name, seed=0, dtype="fp32"):
    cfg = O.make_config(**SHAPES[name])
    W = O.random_weights(cfg, seed=seed)
    return cfg, (_decisive_routers(cfg, W) if dtype == "bf16" else W)


# ---- mechanisms alone ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("W,T", [(48, 5), (44, 3), (333, 7), (1024, 2)])
def test_stream_boundaries(W, T):
    """Embedding norm and the boundary that norms only a sublayer's result, with and without the identity share and the final
    norm, for widths on and off the vector path."""
    from nanorlhf_b200.ops import hybrid as hy
    g = torch.Generator().manual_seed(W)
    eps = 1e-5
    table = torch.randn(20, W, generator=g)
    tok = torch.randint(0, 20, (T,), generator=g).int()
    w0, w1, w2 = (torch.rand(W, generator=g) + 0.5 for _ in range(3))
    x = torch.empty(T, W, device="cuda")
    for hd in (torch.float32, torch.bfloat16):
        h = torch.empty(T, W, device="cuda", dtype=hd)
        hy.embed_norm(table.cuda(), tok.cuda(), w0.cuda(), eps, x, h)
        want = O.model_norm(table.double()[tok.long()], w0.double(), eps)
        assert (x.double().cpu() - want).abs().max() < 1e-5
        assert (h.double().cpu() - want).abs().max() < (1e-5 if hd == torch.float32 else 3e-2)
    o = torch.randn(T, W, generator=g) * 3.0
    sw = torch.rand(T, generator=g)
    for self_w, w_pre in ((None, None), (sw, None), (None, w2), (sw, w2)):
        x = want.float().cuda()
        h = torch.empty(T, W, device="cuda")
        hy.post_norm_residual(x, o.cuda(), None if self_w is None else self_w.cuda(), w1.cuda(), None if w_pre is None else w_pre.cuda(), eps, h)
        x0 = want.float().double()
        y = o.double() + (0 if self_w is None else self_w.double()[:, None] * x0)
        x1 = x0 + O.model_norm(y, w1.double(), eps)
        assert (x.double().cpu() - x1).abs().max() < 2e-5
        hw = x1 if w_pre is None else O.model_norm(x1, w_pre.double(), eps)
        assert (h.double().cpu() - hw).abs().max() < 2e-5


def test_side_gate_and_gated_swiglu():
    from nanorlhf_b200.ops import hybrid as hy
    g = torch.Generator().manual_seed(3)
    T, dim, L = 9, 5, 3
    u = torch.randn(T, 16, generator=g) * 2
    table = torch.randn(30, dim * L, generator=g)
    tok = torch.randint(0, 30, (T,), generator=g).int()
    for i in range(L):
        out = torch.full((T, 8), 7.0, device="cuda")
        hy.side_gate(u.cuda()[:, 2:2 + dim], table.cuda(), i * dim, tok.cuda(), out, dim)
        want = O.gelu_tanh(u.double()[:, 2:2 + dim]) * table.double()[tok.long()][:, i * dim:(i + 1) * dim]
        assert (out.double().cpu()[:, :dim] - want).abs().max() < 1e-5 and float(out[:, dim:].abs().max()) == 0.0
    gu = torch.randn(T, 2 * 12 + 1, generator=g) * 2
    for gated in (False, True):
        out = torch.empty(T, 12, device="cuda")
        hy.swiglu_cols(gu.cuda()[:, :24], gu.cuda()[:, 24:25] if gated else None, out)
        want = O.silu(gu.double()[:, :12]) * gu.double()[:, 12:24] * (torch.sigmoid(gu.double()[:, 24:25]) if gated else 1.0)
        assert (out.double().cpu() - want).abs().max() < 1e-5


@pytest.mark.parametrize("E,ident,top", [(1, 1, 1), (5, 2, 3), (4, 0, 4), (2, 3, 5), (40, 2, 6), (12, 3, 5)])
def test_routing_by_a_softmax_over_all_outputs(E, ident, top):
    from nanorlhf_b200.ops import hybrid as hy
    g = torch.Generator().manual_seed(E * 7 + ident)
    T, n = 50, E + ident
    z = torch.randn(T, n, generator=g) * 2
    corr = torch.randn(n, generator=g) * 0.3
    ids = torch.empty(T, top, dtype=torch.int32, device="cuda")
    wts = torch.empty(T, top, device="cuda")
    self_w = torch.empty(T, device="cuda")
    hy.moe_route_all(z.cuda(), corr.cuda(), E, top, 1.7, ids=ids, wts=wts, self_w=self_w)
    mlp = dict(router=dict(experts=E, identity=ident, top=top, scale=1.7))
    w = {"r.router": torch.eye(n, dtype=torch.float64), "r.correction": corr.double()}
    want_ids, want_w = O.route(w, "r.", mlp, z.double())
    assert torch.equal(ids.cpu().long(), want_ids)
    real = want_ids < E
    assert (wts.double().cpu() - want_w * real).abs().max() < 1e-5
    assert (self_w.double().cpu() - (want_w * ~real).sum(-1)).abs().max() < 1e-5
    # the correction decides the choice only: the weights are the plain scores
    ids2 = torch.empty_like(ids)
    hy.moe_route_all(z.cuda(), None, E, top, 1.0, ids=ids2, wts=wts, self_w=self_w)
    s = torch.softmax(z.double(), -1)
    assert torch.equal(ids2.cpu().long(), torch.topk(s, top, dim=-1).indices)


def _mixer_engine(tmp_path, cfg, W, dtype="fp32", pool=1024):
    eng = _engine(tmp_path, cfg, W, dtype=dtype, pool_tokens=pool)
    return eng, eng.layers[0].mixers[0]


def _feed(eng, sid, n):
    """A plan for the next ``n`` tokens of sequence ``sid`` (token ids do not matter to a mixer)."""
    import numpy as np
    from nanorlhf_b200.sampler.hybrid_sampler import StepPlan
    data, E, T, MB = eng.sched.plan([sid], [n], 0)
    data[:T] = np.zeros(T, dtype=np.int32)
    return StepPlan(torch.from_numpy(data).cuda(), E, T, MB)


def _latent_case(tmp_path, layout, dtype, T, needles, seed=0, **sizes):
    """One latent-attention mixer driven with hand-made projections.  ``needles``: (query position, key position) pairs; the
    query of head 0 is turned to the key's unrotated part so that this one score stands far above all others (when the key is
    visible), and the key's latent is made distinctive.  Returns (engine result fed in ``cuts``, oracle) makers."""
    kind = "latent" if layout == "interleaved" else "latent2"
    cfg = O.make_config(layers=(kind,), ffs=(None,), side=0, **{kind: sizes})
    W = O.random_weights(cfg, seed=seed)
    m = cfg["layers"][0]["mixer"]
    H, dn, dr, r, dv = m["heads"], m["dim"], m["rot_dim"], m["kv_rank"], m["vdim"]
    g = torch.Generator().manual_seed(seed + 1)
    q = torch.randn(T, H * (dn + dr), generator=g, dtype=torch.float64)
    dkv = torch.randn(T, r + dr, generator=g, dtype=torch.float64)
    gate = torch.randn(T, H, generator=g, dtype=torch.float64)
    Wd = {k: v.double() for k, v in W.items()}
    for qi, kj in needles:
        dkv[kj, :r] = torch.randn(r, generator=g, dtype=torch.float64) * 3.0
        c = O.rms(dkv[kj:kj + 1, :r], cfg["norm"]["eps"]) * Wd["l0.mix.dkv.norm"]
        kn = (c @ Wd["l0.mix.uk"].T)[0, :dn]
        q[qi, :dn] = 25.0 / m["scale"] * kn / kn.pow(2).sum()
        q[qi, dn:dn + dr] = 0.0
    want = O.latent_core(q, dkv, gate, Wd, "l0.mix.", m, cfg["norm"]["eps"], layout)

    def run(cuts, pool=1024):
        eng, M = _mixer_engine(tmp_path, cfg, W, dtype=dtype, pool=pool)
        (cq, nq), (cd, nd), (cg, ng) = M.cols["q"], M.cols["dkv"], M.cols["g"]
        sid = eng.open()
        outs, lo = [], 0
        for n in cuts:
            U = torch.zeros(n, eng.layers[0].n_in, device="cuda")
            U[:, cq:cq + nq], U[:, cd:cd + nd], U[:, cg:cg + ng] = q[lo:lo + n].float().cuda(), dkv[lo:lo + n].float().cuda(), gate[lo:lo + n].float().cuda()
            out = torch.empty(n, H * dv, device="cuda", dtype=eng.wdtype)
            eng._latent_attention(M, U, _feed(eng, sid, n), cfg["norm"]["eps"], out)
            outs.append(out.double().cpu())
            lo += n
        eng.close(sid)
        return torch.cat(outs)
    return run, want


@pytest.mark.parametrize("layout", ["interleaved", "half"])
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_latent_attention_sees_exactly_the_causal_keys(tmp_path, layout, dtype):
    """Loud keys planted far away, at page borders, at the query's own position (the last key it sees) and one position later (the
    first it does not), in whole prompts, in portions and in single-token steps."""
    T = 330
    needles = [(300, 2), (47, 47), (15, 16), (17, 17), (31, 32), (200, 15), (255, 256), (320, 319), (329, 1), (100, 101)]
    run, want = _latent_case(tmp_path, layout, dtype, T, needles, heads=3, dim=8, rot_dim=8, vdim=12, kv_rank=24, scale=0.3,
                             base=100.0, scaling=None)
    tol = 1e-4 if dtype == "fp32" else 4e-2
    scale = want.abs().max()
    for cuts in ([T], _cuts(T, [16, 1, 31, 2, 17]), [290] + [1] * 40):
        got = run(cuts)
        assert (got - want).abs().max() < tol * scale, cuts[:4]
    # the planted keys matter: a result that missed one (or saw one it must not see) would be far off
    _, plain = _latent_case(tmp_path, layout, dtype, T, [], heads=3, dim=8, rot_dim=8, vdim=12, kv_rank=24, scale=0.3, base=100.0, scaling=None)
    assert all((want[qi, :12] - plain[qi, :12]).abs().max() > 0.05 * scale for qi, kj in needles if kj <= qi)


@pytest.mark.parametrize("sizes", [dict(heads=1, dim=4, rot_dim=4, vdim=4, kv_rank=4), dict(heads=7, dim=24, rot_dim=16, vdim=72, kv_rank=168),
                                   dict(heads=5, dim=10, rot_dim=6, vdim=14, kv_rank=20), dict(heads=2, dim=6, rot_dim=8, dims=4, vdim=6, kv_rank=10),
                                   dict(heads=20, dim=16, rot_dim=8, vdim=16, kv_rank=264), dict(heads=3, dim=8, rot_dim=2, vdim=8, kv_rank=300)])
def test_latent_attention_sizes(tmp_path, sizes):
    """Head counts and sizes on and off every kernel's tile; the stretch of the rotation's frequencies; positions in the hundreds."""
    scaling = dict(factor=4.0, original=64, fast=8.0, slow=1.0)
    for layout in ("interleaved", "half"):
        run, want = _latent_case(tmp_path, layout, "fp32", 150, [(140, 3), (17, 18)], scale=0.2, base=1000.0, scaling=scaling, **sizes)
        for cuts in ([150], [120] + [1] * 30, _cuts(150, [2, 29, 1])):
            assert (run(cuts) - want).abs().max() < 1e-4 * want.abs().max()


@pytest.mark.parametrize("sizes", [dict(heads=7, dim=24, rot_dim=16, vdim=72, kv_rank=136), dict(heads=20, dim=16, rot_dim=8, vdim=16, kv_rank=264),
                                   dict(heads=3, dim=16, rot_dim=64, vdim=24, kv_rank=512), dict(heads=70, dim=8, rot_dim=16, vdim=8, kv_rank=64),
                                   dict(heads=5, dim=8, rot_dim=8, vdim=8, kv_rank=24), dict(heads=17, dim=8, rot_dim=32, vdim=8, kv_rank=352)])
def test_latent_attention_on_the_tensor_cores(tmp_path, sizes):
    """bf16 pages: the tensor-core kernels for portions and for single-token steps, for every tile width (rows of up to 128, 256,
    384 and 576 columns), one and several value slices (the last one partial), more than 16 and more than 64 heads, loud keys at
    the causal edge and far away, several sequences in one query tile."""
    T = 200
    needles = [(190, 2), (47, 47), (63, 64), (64, 64), (127, 128), (150, 15), (199, 198)]
    run, want = _latent_case(tmp_path, "interleaved", "bf16", T, needles, scale=0.2, base=1000.0, scaling=None, **sizes)
    scale = want.abs().max()
    for cuts in ([T], _cuts(T, [16, 1, 31, 2, 70]), [150] + [1] * 50):
        got = run(cuts)
        assert (got - want).abs().max() < 4e-2 * scale, cuts[:4]
        assert (got - want).pow(2).mean().sqrt() < 6e-3 * scale, cuts[:4]


def test_latent_attention_long_context_on_the_tensor_cores(tmp_path):
    """Hundreds of keys per query: many key blocks per tile, portions that start and end inside pages and key blocks, single-token
    steps whose page walk is cut into parts."""
    T = 700
    needles = [(690, 5), (650, 330), (331, 332), (420, 419), (699, 699)]
    run, want = _latent_case(tmp_path, "half", "bf16", T, needles, heads=4, dim=16, rot_dim=24, vdim=16, kv_rank=280, scale=0.2, base=1000.0,
                             scaling=None)
    scale = want.abs().max()
    for cuts in ([T], [100, 1, 250, 3, 346], [650] + [1] * 50):
        got = run(cuts)
        assert (got - want).abs().max() < 4e-2 * scale, cuts[:4]
        assert (got - want).pow(2).mean().sqrt() < 6e-3 * scale, cuts[:4]


@pytest.mark.parametrize("sizes", [dict(heads=7, dim=24, rot_dim=24, vdim=40, kv_rank=112), dict(heads=5, dim=16, rot_dim=24, vdim=16, kv_rank=232),
                                   dict(heads=18, dim=8, rot_dim=16, vdim=8, kv_rank=320)])
def test_latent_attention_batches_on_the_tensor_cores(tmp_path, sizes):
    """Several sequences of unequal lengths in one step (tiles that span sequences) and single-token steps of a batch, bf16; for
    the 64-key and the 32-key prompt kernels, 128 and 256 value columns per block, more than 16 heads."""
    cfg = O.make_config(layers=("latent",), ffs=(None,), side=0, latent=dict(scale=0.2, scaling=None, **sizes))
    W = O.random_weights(cfg, seed=3)
    m = cfg["layers"][0]["mixer"]
    Wd = {k: v.double() for k, v in W.items()}
    eng, M = _mixer_engine(tmp_path, cfg, W, dtype="bf16", pool=2048)
    (cq, nq), (cd, nd), (cg, ng) = M.cols["q"], M.cols["dkv"], M.cols["g"]
    g = torch.Generator().manual_seed(8)
    lens = [5, 70, 1, 150]
    data = [(torch.randn(n, nq, generator=g), torch.randn(n, nd, generator=g), torch.randn(n, ng, generator=g)) for n in lens]
    want = [O.latent_core(q.double(), d.double(), gt.double(), Wd, "l0.mix.", m, 1e-5, "interleaved") for q, d, gt in data]
    import numpy as np
    from nanorlhf_b200.sampler.hybrid_sampler import StepPlan
    sids = [eng.open() for _ in lens]
    got = [[] for _ in lens]
    for lo, hi in ((0, 0.6), (0.6, 1.0)):                   # two mixed steps, then the last tokens one by one as a batch
        cnt = [int(n * hi) - int(n * lo) if hi < 1.0 else max(n - 3, int(n * lo)) - int(n * lo) for n in lens]
        use = [i for i, c in enumerate(cnt) if c > 0]
        buf, E, T, MB = eng.sched.plan([sids[i] for i in use], [cnt[i] for i in use], 0)
        buf[:T] = np.zeros(T, dtype=np.int32)
        plan = StepPlan(torch.from_numpy(buf).cuda(), E, T, MB)
        U = torch.zeros(T, eng.layers[0].n_in, device="cuda")
        o = 0
        for i in use:
            a = int(lens[i] * lo)
            for col, n_, src in ((cq, nq, 0), (cd, nd, 1), (cg, ng, 2)):
                U[o:o + cnt[i], col:col + n_] = data[i][src][a:a + cnt[i]].cuda()
            o += cnt[i]
        out = torch.empty(T, sizes["heads"] * sizes["vdim"], device="cuda", dtype=torch.bfloat16)
        eng._latent_attention(M, U, plan, 1e-5, out)
        o = 0
        for i in use:
            got[i].append(out[o:o + cnt[i]].double().cpu())
            o += cnt[i]
    done = [sum(len(x) for x in gi) for gi in got]
    while any(d < n for d, n in zip(done, lens)):
        use = [i for i in range(len(lens)) if done[i] < lens[i]]
        buf, E, T, MB = eng.sched.plan([sids[i] for i in use], [1] * len(use), 0)
        buf[:T] = np.zeros(T, dtype=np.int32)
        plan = StepPlan(torch.from_numpy(buf).cuda(), E, T, MB)
        U = torch.zeros(T, eng.layers[0].n_in, device="cuda")
        for r, i in enumerate(use):
            for col, n_, src in ((cq, nq, 0), (cd, nd, 1), (cg, ng, 2)):
                U[r, col:col + n_] = data[i][src][done[i]].cuda()
        out = torch.empty(T, sizes["heads"] * sizes["vdim"], device="cuda", dtype=torch.bfloat16)
        eng._latent_attention(M, U, plan, 1e-5, out)
        for r, i in enumerate(use):
            got[i].append(out[r:r + 1].double().cpu())
            done[i] += 1
    for i, n in enumerate(lens):
        assert (torch.cat(got[i]) - want[i]).abs().max() < 4e-2 * want[i].abs().max(), i


def test_latent_cache_rows_hold_the_normed_latent_and_the_rotated_key_part(tmp_path):
    """What the page holds after a step: [rmsnorm(latent) * w | rotation(position) of the shared key part], at the token's slot."""
    cfg = O.make_config(layers=("latent2",), ffs=(None,), side=0, latent2=dict(heads=2, dim=4, rot_dim=6, vdim=4, kv_rank=10, scale=1.0, base=50.0))
    W = O.random_weights(cfg, seed=0)
    eng, M = _mixer_engine(tmp_path, cfg, W)
    sid = eng.open()
    (cq, nq), (cd, nd) = M.cols["q"], M.cols["dkv"]
    g = torch.Generator().manual_seed(5)
    dkv = torch.randn(40, 16, generator=g)
    lo = 0
    for n in (17, 1, 22):
        U = torch.zeros(n, eng.layers[0].n_in, device="cuda")
        U[:, cd:cd + nd] = dkv[lo:lo + n].cuda()
        plan = _feed(eng, sid, n)
        eng._latent_attention(M, U, plan, 1e-5, torch.empty(n, 8, device="cuda"))
        rows = M.k_cache.view(-1, 16)[plan.kv_slot.long()].double().cpu()
        c = O.rms(dkv[lo:lo + n, :10].double(), 1e-5) * W["l0.mix.dkv.norm"].double()
        cos, sin = O.rotary_tables(dict(base=50.0, dims=6), torch.arange(lo, lo + n))
        assert (rows[:, :10] - c).abs().max() < 1e-5
        assert (rows[:, 10:] - O.rotate(dkv[lo:lo + n, 10:].double(), cos, sin, "half")).abs().max() < 1e-5
        lo += n


@pytest.mark.parametrize("sizes", [dict(heads=2, dim=8, vdim=12, tau=8.0), dict(heads=1, dim=128, vdim=128, tau=16.0),
                                   dict(heads=3, dim=10, vdim=6, tau=1.0), dict(heads=2, dim=160, vdim=40, tau=4.0),
                                   dict(heads=1, dim=24, vdim=300, tau=2.0)])
def test_gated_linear_attention_scan(tmp_path, sizes):
    """The recurrence alone (every scan kernel the sizes select) in portions and single tokens, the state carried per slot."""
    from nanorlhf_b200.ops import hybrid as hy
    H, dk, dv, tau = sizes["heads"], sizes["dim"], sizes["vdim"], sizes["tau"]
    T = 70
    g = torch.Generator().manual_seed(dk)
    qkv = torch.randn(T, 2 * H * dk + H * dv, generator=g)
    z = torch.randn(T, H * dk, generator=g) * 2 + 2
    bias = torch.randn(H * dk, generator=g)
    m = dict(tau=tau)
    q = qkv[:, :H * dk].double().reshape(T, H, dk) * dk ** -0.5
    k = qkv[:, H * dk:2 * H * dk].double().reshape(T, H, dk)
    v = qkv[:, 2 * H * dk:].double().reshape(T, H, dv)
    want, _ = O.gla_core(q, k, v, (z.double() + bias.double()).reshape(T, H, dk), m)
    cfg = O.make_config(layers=("gla",), ffs=(None,), side=0, gla=sizes)
    eng, M = _mixer_engine(tmp_path, cfg, O.random_weights(cfg, seed=1))
    for cuts in ([T], [40] + [1] * 30, _cuts(T, [2, 17, 1, 5])):
        sid = eng.open()
        outs, lo = [], 0
        for n in cuts:
            plan = _feed(eng, sid, n)
            x = qkv[lo:lo + n].cuda().contiguous()
            decay = torch.empty(n, H * dk, device="cuda")
            hy.gla_prep(x, z[lo:lo + n].cuda(), bias.cuda(), tau, decay, H, dk)
            o = torch.empty(n, H * dv, device="cuda")
            hy.delta_scan(x, H * dk, 2 * H * dk, None, decay, M.state, o, plan, H, True)
            outs.append(o.double().cpu())
            lo += n
        eng.close(sid)
        assert (torch.cat(outs).reshape(T, H, dv) - want).abs().max() < 2e-4 * want.abs().max(), cuts[:3]


def test_each_layer_type_alone_and_the_stream_after_every_layer(tmp_path):
    import numpy as np
    from nanorlhf_b200.sampler.hybrid_sampler import StepPlan
    for kind in ("gla", "latent", "latent2"):
        for ff in ("dense", "moe", None):
            cfg = O.make_config(layers=(kind,), ffs=(ff,))
            W = O.random_weights(cfg, seed=2)
            toks = _tokens(cfg, 40, 1)
            eng = _engine(tmp_path, cfg, W, name=f"{kind}{ff}")
            assert _rel(_run_alone(eng, toks, [33, 2, 1, 4]), O.forward(W, cfg, toks)) < F32_TOL, (kind, ff)
    cfg, W = _model("mixed")
    toks = _tokens(cfg, 20, 2)
    want = []
    O.forward(W, cfg, toks, keep=want)
    eng = _engine(tmp_path, cfg, W)
    sid = eng.open()
    data, E, T, MB = eng.sched.plan([sid], [len(toks)], 0)
    data[:T] = np.asarray(toks, dtype=np.int32)
    keep = []
    eng._forward_post_norm(StepPlan(torch.from_numpy(data).cuda(), E, T, MB), [], keep)
    assert len(keep) == len(want) == len(cfg["layers"])
    for got, ref in zip(keep, want):
        assert (got.double().cpu() - ref).abs().max().item() < 1e-4 * ref.abs().max().item()


# ---- schedules -----------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
@pytest.mark.parametrize("shape", list(SHAPES))
def test_prefill_decode_and_portions_agree_with_oracle(tmp_path, shape, dtype):
    cfg, W = _model(shape, dtype=dtype)
    n = 90
    toks = _tokens(cfg, n, 5)
    want = O.forward(W, cfg, toks)
    eng = _engine(tmp_path, cfg, W, dtype=dtype)
    whole = _run_alone(eng, toks, [n])
    assert _close(whole, want, dtype)
    schedules = {"prefill_then_decode": [n - 40] + [1] * 40, "ragged": _cuts(n, [3, 37, 2, 16, 1, 17, 5]), "pairs": [2] * (n // 2)}
    if dtype == "fp32":
        schedules["by_token"] = [1] * n
    for name, cuts in schedules.items():
        got = _run_alone(eng, toks, cuts)
        assert _close(got, want, dtype), name
        assert _close(got, whole, dtype), name


def test_first_tokens_of_a_sequence(tmp_path):
    """One- and two-token sequences: position 0 (no rotation), a sink beside a single key, an empty recurrent state."""
    cfg, W = _model("mixed")
    eng = _engine(tmp_path, cfg, W)
    for toks in ([5], [5, 5], [0, 96, 3]):
        want = O.forward(W, cfg, toks)
        assert _rel(_run_alone(eng, toks, [len(toks)]), want) < F32_TOL
        assert _rel(_run_alone(eng, toks, [1] * len(toks)), want) < F32_TOL


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_mixed_batches_match_each_request_alone(tmp_path, dtype):
    """Unequal requests share steps (portions beside single tokens, requests that pause); pages and slots are freed and reused."""
    cfg, W = _model("mixed", dtype=dtype)
    eng = _engine(tmp_path, cfg, W, dtype=dtype, pool_tokens=16 * 12, slots=3)
    reqs = {name: _tokens(cfg, n, 10 + i) for i, (name, n) in enumerate([("a", 70), ("b", 23), ("c", 1), ("d", 41), ("e", 64), ("f", 9)])}
    want = {k: O.forward(W, cfg, v) for k, v in reqs.items()}
    got = {k: [] for k in reqs}
    fed = {k: 0 for k in reqs}
    live = {}
    waiting = list(reqs)
    portion = {"a": [16, 3, 1, 1, 30, 2, 1, 16], "b": [2, 1, 20], "c": [1], "d": [40, 1], "e": [5, 1, 1, 57], "f": [3, 3, 3]}
    step = 0
    while waiting or live:
        while waiting and len(live) < 3 and eng.sched.num_free_blocks() * 16 >= len(reqs[waiting[0]]) + 16 * len(live):
            live[waiting.pop(0)] = eng.open()
        entries, names = [], []
        for name in list(live):
            if name == "a" and step % 3 == 2:
                continue                                   # a request may sit out a step
            k = portion[name]
            n = min(k[len(got[name]) % len(k)], len(reqs[name]) - fed[name])
            entries.append((live[name], reqs[name][fed[name]:fed[name] + n], list(range(n))))
            names.append((name, n))
        out = eng.step(entries).double().cpu()
        o = 0
        for name, n in names:
            got[name].append(out[o:o + n])
            o += n
            fed[name] += n
            if fed[name] == len(reqs[name]):
                eng.close(live.pop(name))
        step += 1
    assert eng.sched.num_open() == 0
    for k in reqs:
        assert _close(torch.cat(got[k]), want[k], dtype), k


def test_long_decoding(tmp_path):
    """Hundreds of single-token steps: the recurrent state is carried without drift and the attention keeps every key."""
    cfg, W = _model("odd")
    toks = _tokens(cfg, 260, 8)
    eng = _engine(tmp_path, cfg, W)
    assert _rel(_run_alone(eng, toks, [4] + [1] * 256), O.forward(W, cfg, toks)) < F32_TOL


def test_distant_tokens_reach_through_state_and_cache(tmp_path):
    """Changing an early token must change late logits, in the engine as in the oracle, through the recurrent state alone
    (slow decays) and through the latent cache alone, in portions and in decoding."""
    for layers in (("gla", "gla"), ("latent", "latent2")):
        cfg = O.make_config(layers=layers, ffs=("dense", None), side=0)
        W = O.random_weights(cfg, seed=4)
        for k in W:
            if k.endswith("a2.b"):
                W[k] = torch.full_like(W[k], 6.0)          # decays close to 1: a long memory
        a = _tokens(cfg, 150, 3)
        b = list(a)
        b[1] = (b[1] + 1) % cfg["vocab"]
        wa, wb = O.forward(W, cfg, a), O.forward(W, cfg, b)
        assert _rel(wa[-8:], wb[-8:]) > 20 * F32_TOL, layers
        eng = _engine(tmp_path, cfg, W, name=layers[0])
        for toks, want in ((a, wa), (b, wb)):
            assert _rel(_run_alone(eng, toks, [130] + [1] * 20)[-8:], want[-8:]) < F32_TOL


def test_grouped_and_dense_expert_forms_agree(tmp_path):
    """bf16 serving runs only the chosen experts (rows sorted by expert, identity experts without rows of their own); the dense
    form runs every expert.  Both against the oracle."""
    cfg = O.make_config(layers=("gla", "latent"), ffs=("moe", "moe"), width=64, moe=dict(ff=24, experts=6, identity=2, top=3, shared=24))
    W = _decisive_routers(cfg, O.random_weights(cfg, seed=9))
    toks = _tokens(cfg, 150, 4)
    want = O.forward(W, cfg, toks)
    for form in ("grouped", "dense"):
        eng = _engine(tmp_path, cfg, W, dtype="bf16", name=form, moe=form)
        assert any(L.w_gate_up is not None for L in eng.layers) == (form == "grouped")
        assert _close(_run_alone(eng, toks, [100, 2, 47, 1]), want, "bf16"), form


# ---- generation through the framework's entry point ------------------------------------------------------------------
class _Tok:
    pad_token_id = 0
    eos_token_id = None


@pytest.mark.parametrize("dtype", ["fp32", "bf16"])
def test_greedy_generation_through_the_engine_entry_point(tmp_path, dtype):
    from nanorlhf_b200.models.registry import load_model
    from nanorlhf_b200.sampler.engine import generate, get_native_engine, release_native_engine
    cfg, W = _model("mixed", dtype=dtype)
    path = _save(tmp_path, cfg, W)
    model = load_model(path, torch_dtype=torch.float32 if dtype == "fp32" else torch.bfloat16, device="cuda")
    prompts = [_tokens(cfg, n, 20 + n) for n in (3, 17, 1, 40, 9)]
    new = 24
    out = generate(1, model, _Tok(), prompts, 0.0, new, top_p=1.0, seed=1, rollout_dtype=dtype, max_num_seqs=3,
                   prefill_token_budget=32).cpu()
    far = 0
    for p, row in zip(prompts, out.tolist()):
        seq = list(p)
        for t in row:
            logits = O.forward(W, cfg, seq)[-1]
            best = int(logits.argmax())
            if dtype == "fp32":
                assert t == best
            elif t != best and float(logits[best] - logits[t]) > 0.05 * float(logits.std()):
                far += 1                                   # bf16: a near tie of two logits may go the other way
            seq.append(t)
    assert far <= 0.05 * len(prompts) * new
    assert get_native_engine(model, rollout_dtype=dtype).stats["graph_replays"] > 0      # decode steps replay a CUDA graph
    release_native_engine(model)


def test_trace_runner_replays_a_mixed_trace(tmp_path):
    """bin/trace_run as a subprocess: portions beside single tokens, a pool that forces pages and slots to be reused."""
    import numpy as np
    cfg, W = _model("mixed")
    path = _save(tmp_path, cfg, W)
    reqs = {k: _tokens(cfg, n, 30 + n) for k, n in (("x", 50), ("y", 33), ("z", 2), ("w", 40))}
    steps = [
        {"step": 0, "entries": [{"id": "x", "tokens": reqs["x"][:30], "want": [0, 29]}, {"id": "z", "tokens": reqs["z"], "want": [1]}], "end": ["z"]},
        {"step": 1, "entries": [{"id": "x", "tokens": reqs["x"][30:31], "want": [0]}, {"id": "y", "tokens": reqs["y"][:31], "want": []}], "end": []},
        {"step": 2, "entries": [{"id": "y", "tokens": reqs["y"][31:], "want": [0, 1]}, {"id": "x", "tokens": reqs["x"][31:], "want": [18]}], "end": ["x", "y"]},
        {"step": 3, "entries": [{"id": "w", "tokens": reqs["w"], "want": [39]}], "end": ["w"]},
    ]
    outdir = os.path.join(str(tmp_path), "out")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", path, "--dtype", "float32", "--out", outdir,
                        "--max-tokens", "128"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                       timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == [f"done {i}" for i in range(4)]
    full = {k: O.forward(W, cfg, v) for k, v in reqs.items()}
    want = {0: [full["x"][0], full["x"][29], full["z"][1]], 1: [full["x"][30]], 2: [full["y"][31], full["y"][32], full["x"][49]], 3: [full["w"][39]]}
    for i, rows in want.items():
        got = torch.from_numpy(np.fromfile(os.path.join(outdir, f"{i}.f32"), dtype="<f4").reshape(len(rows), cfg["vocab"])).double()
        assert _rel(got, torch.stack(rows)) < F32_TOL


def test_sampler_command_line_generates_greedily(tmp_path):
    """``python -m nanorlhf_b200.sampler`` on a Damilix checkpoint: the class and the engine come from config.json."""
    cfg, W = _model("plain")
    path = _save(tmp_path, cfg, W)
    prompts = [_tokens(cfg, 7, 1), _tokens(cfg, 19, 2)]
    cmd = [sys.executable, "-m", "nanorlhf_b200.sampler", "--model", path, "--dtype", "float32", "--max-tokens", "6"]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(map(str, p))]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    rows = [json.loads(ln) for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert [(x["prompt"], x["sample"]) for x in rows] == [(0, 0), (1, 0)]
    for p, x in zip(prompts, rows):
        seq = list(p)
        for t in x["tokens"]:
            assert t == int(O.forward(W, cfg, seq)[-1].argmax())
            seq.append(t)
