"""Zelinex on the GPU against the plain restatement of tests/zelinex_oracle.py: the new operators called directly, every
mixer and feed-forward alone, looped stacks, prompts against token-by-token decoding, portions down to two tokens, mixed
batches, re-used pages and slots, keys just inside and just outside the window (at page borders too), tokens far back that
only the recurrent states remember, the convolution's history, the first tokens of a sequence, long decoding, sizes where
counts collapse to 1 or are not multiples of 4, the tensor-core paths, greedy generation through the engine's scheduler,
the command line and the trace replay program."""
import copy
import ctypes as C
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import zelinex_oracle as O

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL32, TOL16 = 2e-4, 5e-2
F = torch.float64


def make(cfg=None, seed=0, dtype="float32", edit=None, **kw):
    from proxy_inference_engine_b200.zelinex import ZelinexArgs, ZelinexModel, random_weights
    cfg = copy.deepcopy(cfg) if cfg else O.random_config(**kw)
    args = ZelinexArgs.from_dict(cfg)
    w = random_weights(args, seed=seed)
    if edit:
        edit(w)
    return cfg, w, ZelinexModel(args, w, "cuda", dtype)


def engine(model, max_tokens=1024, max_seqs=4, graph=True):
    from proxy_inference_engine_b200.engine import HybridEngine
    return HybridEngine(model, max_tokens, max_seqs, use_graph=graph)


def toks(n, vocab=96, seed=1, avoid=()):
    g = torch.Generator().manual_seed(seed)
    out = torch.randint(0, vocab, (n,), generator=g).tolist()
    return [t if t not in avoid else (t + 1) % vocab for t in out]


def rows_err(got, want):
    got, want = got.double().cpu(), want.double()
    return (got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean(-1).sqrt().clamp_min(1e-9)


def err(got, want):
    return float(rows_err(got, want).max())


def whole(eng, ids, sid="s"):
    out = eng.forward([(sid, ids, list(range(len(ids))))])
    eng.finish(sid)
    return out


def in_portions(eng, ids, sizes, sid="s"):
    """Feeds ids in portions of the given sizes (the last size repeats), every row wanted."""
    outs, at, k = [], 0, 0
    while at < len(ids):
        n = min(sizes[min(k, len(sizes) - 1)], len(ids) - at)
        outs.append(eng.forward([(sid, ids[at:at + n], list(range(n)))]))
        at, k = at + n, k + 1
    eng.finish(sid)
    return torch.cat(outs)


# ---- the operators, called directly ------------------------------------------------------------------------------------------
def _lib():
    from proxy_inference_engine_b200 import _lib as lib
    return lib, lib.load_hybrid(build_if_missing=True)


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _st():
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _rand(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.rand(shape, generator=g, dtype=F) * 2 - 1) * scale


def _batch(seqs):
    """seqs: [(rows, context, slot)] -> (BatchDetails, descriptor, keepalive); pages are not used by the recurrences."""
    from proxy_inference_engine_b200.ragged import BatchDetails
    b = BatchDetails.build([(i, [0] * n, ctx, list(range((ctx + n + 63) // 64)), slot) for i, (n, ctx, slot) in enumerate(seqs)])
    desc, keep = b.hybrid_descriptor()
    return b, desc, keep


@pytest.mark.parametrize("M,N,K", [(5, 40, 24), (70, 96, 64), (33, 17, 128)])
def test_linear_with_xielu_and_tanh(M, N, K):
    lib, L = _lib()
    x, w, b = _rand(M, K, seed=1, scale=2.0), _rand(N, K, seed=2, scale=0.5), _rand(N, seed=3)
    for dt, code, tol in ((torch.float32, lib.DTYPE_F32, 1e-5), (torch.bfloat16, lib.DTYPE_BF16, 2e-2)):
        xd, wd, bd = x.to(dt).cuda(), w.to(dt).cuda(), b.float().cuda()
        z = xd.double().cpu() @ wd.double().cpu().T + b
        for act, a0, a1, want in ((lib.EPI_XIELU, 0.8, 1.3, O.xielu(z, torch.tensor(math.log(math.e ** 0.8 - 1), dtype=F),
                                                                   torch.tensor(math.log(math.e ** 0.8 - 1), dtype=F))),
                                  (lib.EPI_TANH, 0.0, 0.0, torch.tanh(z))):
            out = torch.empty((M, N), dtype=torch.float32, device="cuda")
            lib.check_hybrid(L.pieh_linear_act(_ptr(out), lib.DTYPE_F32, N, _ptr(xd), code, K, _ptr(wd), code, _ptr(bd), M, N, K,
                                               act, a0, a1, _st()), "linear_act")
            assert float((out.double().cpu() - want).abs().max()) < tol * float(want.abs().max())


def test_xielu_is_continuous_and_has_both_branches():
    z = torch.tensor([-3.0, -1e-3, 0.0, 1e-3, 2.0], dtype=F)
    p, q = torch.tensor(0.3, dtype=F), torch.tensor(-0.4, dtype=F)
    y = O.xielu(z, p, q)
    ap, aq = math.log1p(math.exp(0.3)), 0.5 + math.log1p(math.exp(-0.4))
    assert abs(float(y[4]) - (ap * 4 + 1)) < 1e-12 and abs(float(y[0]) - (aq * (math.exp(-3) + 2) - 1.5)) < 1e-12
    assert float(y[2]) == 0 and abs(float(y[1]) + float(y[3])) < 1e-5          # slope 1/2 on both sides of zero


@pytest.mark.parametrize("groups,gs,fn,first", [(4, 16, 1, 0), (2, 24, 2, 1), (1, 50, 2, 1), (3, 7, 0, 0), (6, 130, 1, 1)])
def test_gated_group_norm(groups, gs, fn, first):
    lib, L = _lib()
    T, n, eps = 9, groups * gs, 1e-5
    x, g, w = _rand(T, n + 5, seed=4, scale=3.0), _rand(T, 2 * n, seed=5, scale=2.0), 1 + _rand(n, seed=6, scale=0.3)
    xs, gate = x[:, :n], g[:, n // 2:n // 2 + n]                 # both read through a row stride
    f = torch.sigmoid(gate) if fn == 1 else O.silu(gate) if fn == 2 else torch.ones_like(gate)
    if first:
        want = O.unit_rms((xs * f).view(T, groups, gs), eps).reshape(T, n) * w
    else:
        want = O.unit_rms(xs.view(T, groups, gs), eps).reshape(T, n) * w * f
    xd, gd, wd = x.float().cuda(), g.float().cuda(), w.float().cuda()
    out = torch.empty((T, n), dtype=torch.float32, device="cuda")
    lib.check_hybrid(L.pieh_gated_group_norm(_ptr(out), lib.DTYPE_F32, _ptr(xd), n + 5, C.c_void_p(gd.data_ptr() + 4 * (n // 2)),
                                             2 * n, _ptr(wd), groups, gs, eps, fn, first, T, _st()), "gated_group_norm")
    assert float((out.double().cpu() - want).abs().max()) < 1e-5 * float(want.abs().max())


def test_sandwich_add_with_and_without_its_parts():
    lib, L = _lib()
    T, W, eps, mult = 7, 100, 1e-5, 0.6
    x, y, rows, vec = _rand(T, W, seed=7, scale=2.0), _rand(T, W, seed=8, scale=5.0), _rand(T, W, seed=9), _rand(W, seed=10)
    pw, nw = 1 + _rand(W, seed=11, scale=0.3), 1 + _rand(W, seed=12, scale=0.3)
    yd, rd, vd, pwd, nwd = (t.float().cuda() for t in (y, rows, vec, pw, nw))
    for use_y, use_rows, use_vec, use_h in ((1, 1, 1, 1), (1, 0, 0, 1), (0, 1, 1, 1), (1, 0, 1, 0), (0, 0, 0, 1)):
        want = x.clone()
        if use_y:
            want = want + mult * O.unit_rms(y, eps) * pw
        if use_rows:
            want = want + rows
        if use_vec:
            want = want + vec
        xd, h = x.float().cuda(), torch.zeros((T, W), dtype=torch.float32, device="cuda")
        lib.check_hybrid(L.pieh_sandwich_add(_ptr(xd), _ptr(yd) if use_y else None, None, _ptr(pwd) if use_y else None, mult,
                                             _ptr(rd) if use_rows else None, _ptr(vd) if use_vec else None,
                                             _ptr(h) if use_h else None, lib.DTYPE_F32, _ptr(nwd) if use_h else None, eps, T, W,
                                             _st()), "sandwich_add")
        assert float((xd.double().cpu() - want).abs().max()) < 1e-5
        if use_h:
            assert float((h.double().cpu() - O.unit_rms(want, eps) * nw).abs().max()) < 1e-5


@pytest.mark.parametrize("H,dk,dv", [(2, 16, 16), (3, 12, 20), (1, 40, 6), (2, 64, 64), (1, 130, 9), (2, 32, 40), (1, 128, 24), (2, 64, 7)])
def test_generalized_delta_scan_with_states_in_slots(H, dk, dv):
    """Two sequences of unequal length in one step, then both continue from their slots (one of them a slot that held
    another sequence's state before)."""
    lib, L = _lib()
    lens = [23, 5]
    full = {}
    for s, n in enumerate(lens):
        r, k, v = (_rand(n, H, d, seed=20 + 3 * s + j) for j, d in enumerate((dk, dk, dv)))
        decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(_rand(n, H, dk, seed=40 + s, scale=3.0)))
        a = torch.sigmoid(_rand(n, H, dk, seed=50 + s, scale=2.0))
        o = torch.zeros((n, H, dv), dtype=F)
        for h in range(H):
            S = torch.zeros((dk, dv), dtype=F)
            for t in range(n):
                u = k[t, h] / torch.sqrt((k[t, h] ** 2).sum() + 1e-6)
                S = decay[t, h][:, None] * S - torch.outer(a[t, h] * u, u @ S) + torch.outer(k[t, h], v[t, h])
                o[t, h] = S.T @ r[t, h]
        full[s] = (r, k, v, decay, a, o)
    state = torch.full((3, H, dk, dv), 7.0, dtype=torch.float32, device="cuda")       # dirty slots
    cuts = [[(0, 17), (17, 23)], [(0, 2), (2, 5)]]
    for part in range(2):
        spans = [cuts[s][part] for s in range(2)]
        _, desc, keep = _batch([(hi - lo, lo, 2 - s) for s, (lo, hi) in enumerate(spans)])
        cat = lambda j: torch.cat([full[s][j][lo:hi] for s, (lo, hi) in enumerate(spans)]).float()
        r, k, v, decay, a = (cat(j) for j in range(5))
        T = r.shape[0]
        proj = torch.cat([r.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1).contiguous().cuda()
        u = k / torch.sqrt((k.double() ** 2).sum(-1, keepdim=True) + 1e-6).float()
        gd = lib.HybGdelta(H, dk, dv, 0, H * dk, 2 * H * dk, 0, None, math.exp(-0.5), 1e-6, _ptr(state))
        o = torch.empty((T, H, dv), dtype=torch.float32, device="cuda")
        dc, uc, auc = decay.contiguous().cuda(), u.contiguous().cuda(), (a * u).contiguous().cuda()
        lib.check_hybrid(L.pieh_gdelta_scan(_ptr(o), _ptr(proj), proj.stride(0), _ptr(dc), _ptr(uc), _ptr(auc), C.byref(gd),
                                            C.byref(desc), _st()), "gdelta_scan")
        want = torch.cat([full[s][5][lo:hi] for s, (lo, hi) in enumerate(spans)])
        assert float((o.double().cpu() - want).abs().max()) < 2e-5 * max(1.0, float(want.abs().max())), part
        del keep


def test_generalized_delta_prepare():
    lib, L = _lib()
    T, H, dk = 6, 3, 20
    k, al, dl, ab = _rand(T, H * dk, seed=60), _rand(T, H * dk, seed=61, scale=2.0), _rand(T, H * dk + 3, seed=62, scale=3.0), \
        _rand(H * dk, seed=63)
    proj, abd, dld = torch.cat([k, al], 1).float().cuda(), ab.float().cuda(), dl.float().cuda()
    gd = lib.HybGdelta(H, dk, dk, 0, 0, 0, H * dk, _ptr(abd), math.exp(-0.5), 1e-6, _ptr(proj))   # the state is not touched
    out = [torch.empty((T, H, dk), dtype=torch.float32, device="cuda") for _ in range(3)]
    lib.check_hybrid(L.pieh_gdelta_prepare(_ptr(out[0]), _ptr(out[1]), _ptr(out[2]), _ptr(proj), proj.stride(0), _ptr(dld),
                                           dld.stride(0), C.byref(gd), T, _st()), "gdelta_prepare")
    kk = k.view(T, H, dk)
    u = kk / torch.sqrt((kk ** 2).sum(-1, keepdim=True) + 1e-6)
    want = (torch.exp(-math.exp(-0.5) * torch.sigmoid(dl[:, :H * dk])).view(T, H, dk), u,
            torch.sigmoid(al + ab).view(T, H, dk) * u)
    for got, w_ in zip(out, want):
        assert float((got.double().cpu() - w_).abs().max()) < 1e-5


@pytest.mark.parametrize("H,P,N,G,taps", [(4, 8, 12, 2, 3), (2, 6, 10, 1, 1), (3, 20, 33, 3, 4), (2, 64, 128, 1, 2), (6, 5, 7, 2, 8),
                                          (4, 8, 32, 2, 3), (2, 10, 16, 1, 2), (4, 3, 64, 4, 4), (3, 5, 64, 1, 2)])
def test_state_space_prepare_and_scan_with_states_in_slots(H, P, N, G, taps):
    lib, L = _lib()
    inner, Cn = H * P, H * P + 2 * G * N
    lens = [21, 4]
    cw, cb = _rand(Cn, taps, seed=70) + torch.eye(taps, dtype=F)[-1], _rand(Cn, seed=71, scale=0.3)
    dtb, alog, D = _rand(H, seed=72) - 0.5, torch.log(0.5 + 2 * torch.rand(H, dtype=F)), 1 + _rand(H, seed=74, scale=0.5)
    full = {}
    for s, n in enumerate(lens):
        raw, dtl = _rand(n, Cn, seed=80 + s, scale=2.0), _rand(n, H, seed=90 + s, scale=2.0)
        xbc = O.causal_conv_silu(raw, cw, cb)
        dt = O.softplus(dtl + dtb)
        y = O.ssd_scan(xbc[:, :inner].reshape(n, H, P), xbc[:, inner:inner + G * N].reshape(n, G, N),
                       xbc[:, inner + G * N:].reshape(n, G, N), dt, alog, D)
        full[s] = (raw, dtl, y.reshape(n, inner))
    state = torch.full((3, H, N, P), -3.0, dtype=torch.float32, device="cuda")        # dirty slots
    hist = torch.full((3, max(taps - 1, 1), Cn), 5.0, dtype=torch.float32, device="cuda")
    cu = lambda t: t.float().contiguous().cuda()
    cwd, cbd, dtbd, alogd, Dd = cu(cw), cu(cb), cu(dtb), cu(alog), cu(D)
    cuts = [[(0, 2), (2, 3), (3, 21)], [(0, 1), (1, 2), (2, 4)]]
    for part in range(3):
        spans = [cuts[s][part] for s in range(2)]
        _, desc, keep = _batch([(hi - lo, lo, 2 * s) for s, (lo, hi) in enumerate(spans)])
        raw = torch.cat([full[s][0][lo:hi] for s, (lo, hi) in enumerate(spans)])
        dtl = torch.cat([full[s][1][lo:hi] for s, (lo, hi) in enumerate(spans)])
        T = raw.shape[0]
        proj = cu(torch.cat([torch.zeros((T, 3), dtype=F), raw, dtl], 1))
        ss = lib.HybSsd(H, P, N, G, taps, 3, 3 + Cn, _ptr(cwd), _ptr(cbd), _ptr(dtbd), _ptr(alogd), _ptr(Dd),
                        _ptr(hist) if taps > 1 else None, _ptr(state))
        xbc = torch.empty((T, Cn), dtype=torch.float32, device="cuda")
        dtd = torch.empty((T, H, 2), dtype=torch.float32, device="cuda")
        lib.check_hybrid(L.pieh_ssd_prepare(_ptr(xbc), _ptr(dtd), _ptr(proj), proj.stride(0), C.byref(ss), C.byref(desc), _st()),
                         "ssd_prepare")
        y = torch.empty((T, inner), dtype=torch.float32, device="cuda")
        lib.check_hybrid(L.pieh_ssd_scan(_ptr(y), _ptr(xbc), _ptr(dtd), C.byref(ss), C.byref(desc), _st()), "ssd_scan")
        want = torch.cat([full[s][2][lo:hi] for s, (lo, hi) in enumerate(spans)])
        assert float((y.double().cpu() - want).abs().max()) < 2e-5 * max(1.0, float(want.abs().max())), part
        del keep


# ---- every mechanism alone, through the model ----------------------------------------------------------------------------------
@pytest.mark.parametrize("pattern,ffs,loop", [("g", "-", None), ("p", "-", None), ("g", "d", None), ("g", "m", None),
                                               ("p", "m", (0, 1, 2)), ("gp", "dm", (0, 1, 2))])
def test_each_mixer_and_feed_forward_alone(pattern, ffs, loop):
    cfg, w, model = make(pattern=pattern, ffs=ffs, loop=loop)
    ids = toks(40)
    trace, otrace = [], []
    eng = engine(model, graph=False)
    got = eng.forward([("s", ids, list(range(40)))], trace=trace)
    want = O.forward(cfg, w, ids, otrace)
    assert len(trace) == len(otrace)
    for a, b in zip(trace, otrace):
        assert err(a, b) < TOL32
    assert err(got, want) < TOL32


@pytest.mark.parametrize("pattern,loop", [("gpg", (0, 3, 2)), ("gpg", (1, 2, 3)), ("pgp", (1, 3, 2)), ("pg", (0, 2, 1)),
                                          ("gp", (1, 2, 1)), ("pgg", (2, 3, 4)), ("gp", None)])
def test_looped_stacks(pattern, loop):
    """The loop anywhere in the stack, once or several times: each pass has its own cache entries, the embedding comes back
    before every pass but the first and the pass vector before every pass."""
    cfg, w, model = make(pattern=pattern, ffs="dm-", loop=loop, seed=3)
    ids = toks(50, seed=2)
    trace, otrace = [], []
    eng = engine(model, graph=False)
    got = eng.forward([("s", ids[:31], list(range(31)))], trace=trace)
    want = O.forward(cfg, w, ids, otrace)
    runs = len(pattern) + ((loop[1] - loop[0]) * (loop[2] - 1) if loop else 0)
    assert len(trace) == len(otrace) == runs == len(eng.cache.layers)
    for a, b in zip(trace, otrace):
        assert err(a, b[:31]) < TOL32
    rest = torch.cat([eng.forward([("s", ids[31:33], [0, 1])])] + [eng.forward([("s", [t], [0])]) for t in ids[33:]])
    assert err(torch.cat([got, rest]), want) < TOL32
    if loop and loop[2] > 1:                       # the pass vector and the returning embedding do matter
        other = dict(w)
        other["loop.step"] = torch.zeros_like(w["loop.step"])
        assert err(O.forward(cfg, other, ids), want) > 50 * TOL32


def test_bf16_tracks_the_restatement():
    """In bf16 a token whose routing margin is within rounding may take another expert than the restatement, and nudges
    the tokens after it (attention, recurrent state): rows up to the first close call must be within the tolerance, nine
    rows in ten of all, and none far off."""
    cfg, w, model = make(pattern="gpg", ffs="dmd", dtype="bfloat16", seed=5)
    ids = toks(150)
    margins = []
    e = rows_err(in_portions(engine(model), ids, [70, 33, 1]), O.forward(cfg, w, ids, None, margins))
    per_token = torch.tensor(margins).view(-1, len(ids)).min(0).values
    clear = torch.cummin(per_token, 0).values > 0.02
    assert int(clear.sum()) >= 5 and float(e[clear].max()) < TOL16
    assert float(e.quantile(0.9)) < TOL16 and float(e.max()) < 6 * TOL16


def test_bf16_without_routing_is_within_tolerance_everywhere():
    cfg, w, model = make(pattern="gpg", ffs="d-d", dtype="bfloat16")
    ids = toks(150)
    assert err(in_portions(engine(model), ids, [70, 33, 1]), O.forward(cfg, w, ids)) < TOL16


@pytest.mark.parametrize("dtype,dim", [("float32", 64), ("bfloat16", 64), ("bfloat16", 128)])
def test_tensor_core_paths(dtype, dim):
    """Sizes at which prompt portions take the tiled attention kernel (equal head sizes of 64 / 128 over bf16 pages) and the
    tcgen05 products (K a multiple of 64, more than 32 rows), with a window that ends inside a page."""
    cfg = O.random_config(width=128, pattern="pg", ffs="d-", heads=2, kv_heads=1, dim=dim, vdim=dim, window=90, rot_dims=32,
                          s_heads=2, s_vdim=32, state=64, groups=1, d_heads=2, d_dim=64, ff=128, loop=(0, 2, 2))
    cfg, w, model = make(cfg, dtype=dtype)
    ids = toks(300)
    e = rows_err(in_portions(engine(model), ids, [170, 80, 1]), O.forward(cfg, w, ids))
    assert float(e.max()) < (TOL32 if dtype == "float32" else TOL16)
    assert model.L.pieh_pipeline_error() == 0


# ---- prompts, decoding, portions, batches ---------------------------------------------------------------------------------------
def test_prefill_against_token_by_token_decoding():
    cfg, w, model = make(pattern="gpg", ffs="dmd")
    ids = toks(70)
    want = O.forward(cfg, w, ids)
    eng = engine(model)
    assert err(whole(eng, ids), want) < TOL32
    assert err(in_portions(eng, ids, [1]), want) < TOL32            # one token at a time from the first one (graph replay)
    assert err(in_portions(engine(model, graph=False), ids, [1]), want) < TOL32


@pytest.mark.parametrize("sizes", [[2], [3, 2, 5, 2, 64, 7, 2], [63, 2, 1], [64, 64, 2], [65, 1], [17, 16, 15, 2]])
def test_portions_of_several_sizes(sizes):
    cfg, w, model = make(pattern="gpg", ffs="dmd")
    ids = toks(140, seed=3)
    assert err(in_portions(engine(model), ids, sizes), O.forward(cfg, w, ids)) < TOL32


def test_unequal_requests_in_one_batch_match_each_alone():
    cfg, w, model = make(pattern="pgp", ffs="mdm", loop=(1, 3, 2))
    seqs = {"a": toks(90, seed=5), "b": toks(31, seed=6), "c": toks(7, seed=7), "d": toks(130, seed=8)}
    want = {k: O.forward(cfg, w, v) for k, v in seqs.items()}
    eng = engine(model, max_tokens=512)
    plan = {"a": [40, 1, 1, 30, 2, 16], "b": [1, 1, 2, 20, 7], "c": [2, 5], "d": [64, 64, 1, 1]}
    at = {k: 0 for k in seqs}
    got = {k: [] for k in seqs}
    step = 0
    while any(at[k] < len(seqs[k]) for k in seqs):
        entries = []
        for k in seqs:
            if at[k] >= len(seqs[k]) or (k == "c" and step < 2):          # c is admitted later, into a used batch
                continue
            sizes = plan[k]
            n = min(sizes[step % len(sizes)], len(seqs[k]) - at[k])
            entries.append((k, seqs[k][at[k]:at[k] + n], list(range(n))))
            at[k] += n
        out = eng.forward(entries)
        r = 0
        for k, part, _ in entries:
            got[k].append(out[r:r + len(part)])
            r += len(part)
            if at[k] == len(seqs[k]):
                eng.finish(k)
        step += 1
    for k in seqs:
        assert err(torch.cat(got[k]), want[k]) < TOL32, k


def test_pages_and_slots_are_used_again():
    cfg, w, model = make(pattern="gpg", ffs="dmd")
    eng = engine(model, max_tokens=128, max_seqs=1)                  # two pages, one slot: everything is re-used
    for seed, n, sizes in ((11, 120, [50, 1]), (12, 100, [3, 64, 1]), (13, 128, [128]), (14, 9, [1]), (15, 2, [2])):
        ids = toks(n, seed=seed)
        assert err(in_portions(eng, ids, sizes, sid=seed), O.forward(cfg, w, ids)) < TOL32, seed
    assert eng.cache.allocator.get_num_free_pages() == 2 and len(eng.cache.free_slots) == 1


def test_long_decoding():
    cfg, w, model = make(pattern="gp", ffs="dm", window=50)
    ids = toks(260, seed=9)
    assert err(in_portions(engine(model), ids, [20, 1]), O.forward(cfg, w, ids)) < TOL32


# ---- inputs made so that one token stands out -----------------------------------------------------------------------------------
def _point_a_key_at_a_query(w, cfg, q_tok, k_tok, gain, bias=-3.0):
    """Rewrites the embedding of k_tok so that its key (layer 0, as many key heads as query heads) is a positive multiple of
    the query of q_tok, and lowers the score bias: wherever both tokens are visible that key weighs almost 1 while ordinary
    keys weigh little, so one key more or less in the window shows."""
    f = lambda n: w[n].double()
    h_q = O.unit_rms(f("embed")[q_tok], cfg["norm"]["eps"]) * f("l0.norm1")
    h_k = torch.linalg.pinv(f("l0.mix.left.k")) @ (f("l0.mix.left.q") @ h_q)     # k(h_k) = q(h_q)
    e = h_k / f("l0.norm1")
    w["embed"][k_tok] = (e / e.abs().max()).to(torch.bfloat16)                    # the norm takes the length out again
    w["l0.mix.left.k"] = (gain * f("l0.mix.left.k")).to(torch.bfloat16)
    w["l0.mix.left.pb"] = torch.full_like(w["l0.mix.left.pb"], bias)


@pytest.mark.parametrize("window,probe", [(6, 20), (64, 64), (64, 100), (65, 130), (90, 200), (1, 9), (128, 191)])
def test_keys_just_inside_and_just_outside_the_window(window, probe):
    """One earlier token's key points at the probe's query, just inside the window or just outside it, so a window that is
    one token off changes the logits by far more than the tolerance."""
    cfg = O.random_config(pattern="p", ffs="-", heads=2, kv_heads=2, window=window, rot_dims=4, loop=None)
    cfg, w, model = make(cfg, edit=lambda w: _point_a_key_at_a_query(w, cfg, 95, 94, 2.0))
    for dist in (window - 1, window):
        ids = toks(probe + 6, seed=20 + dist, avoid=(94, 95))
        ids[probe], ids[probe - dist] = 95, 94
        want = O.forward(cfg, w, ids)
        other = copy.deepcopy(cfg)
        other["layers"][0]["mixer"]["left"]["mask"]["size"] = window + (1 if dist == window else -1)
        if other["layers"][0]["mixer"]["left"]["mask"]["size"] > 0:
            assert float(rows_err(O.forward(other, w, ids), want)[probe]) > 50 * TOL32   # the case does show the edge
        assert err(whole(engine(model), ids), want) < TOL32                              # inside a prompt
        assert err(in_portions(engine(model), ids, [probe - 3, 1]), want) < TOL32        # decoded alone
        assert err(in_portions(engine(model), ids, [probe - dist + 1, 2]), want) < TOL32  # portions that start at the edge


def test_window_edges_on_the_tiled_attention_kernel():
    """The same planted key in bf16 at head size 64, where prompt portions run on 64-row tiles over whole pages: the edge
    falls inside a tile and inside a page."""
    cfg = O.random_config(width=160, pattern="p", ffs="-", heads=2, kv_heads=2, dim=64, vdim=64, window=70, rot_dims=8, loop=None)
    cfg, w, model = make(cfg, dtype="bfloat16", edit=lambda w: _point_a_key_at_a_query(w, cfg, 95, 94, 3.0, -8.0))
    probe = 150
    for dist in (69, 70):
        ids = toks(probe + 40, seed=30 + dist, avoid=(94, 95))
        ids[probe], ids[probe - dist] = 95, 94
        want = O.forward(cfg, w, ids)
        other = copy.deepcopy(cfg)
        other["layers"][0]["mixer"]["left"]["mask"]["size"] = 70 + (1 if dist == 70 else -1)
        assert float(rows_err(O.forward(other, w, ids), want)[probe]) > 3 * TOL16      # the norm on the mixer's output bounds it
        assert float(rows_err(whole(engine(model), ids), want)[probe]) < TOL16
        assert float(rows_err(in_portions(engine(model), ids, [100, 90]), want)[probe]) < TOL16


def _slow_forgetting(w):
    """Decays next to 1 and almost no removal: what a token writes into a state stays for hundreds of tokens."""
    for k in list(w):
        if k.endswith("mix.w0"):
            w[k] = torch.full_like(w[k], -9.0)
        if k.endswith("mix.w2"):
            w[k] = torch.zeros_like(w[k])
        if k.endswith("mix.a.b"):
            w[k] = torch.full_like(w[k], -9.0)
        if k.endswith("mix.a"):
            w[k] = torch.zeros_like(w[k])
        if k.endswith("right.A_log"):
            w[k] = torch.full_like(w[k], -9.0)


@pytest.mark.parametrize("pattern,far,probe", [("g", 0, 63), ("g", 3, 300), ("p", 0, 64), ("p", 65, 447), ("p", 2, 129)])
def test_tokens_far_back_live_on_in_the_states(pattern, far, probe):
    """With slow forgetting, a token hundreds of positions back (far outside the attention window) still moves the logits
    through the recurrent state; the state has to survive portions, page borders and decoding."""
    cfg, w, model = make(pattern=pattern, ffs="-", loop=None, window=5, edit=_slow_forgetting)
    ids = toks(probe + 3, seed=40 + far)
    want = O.forward(cfg, w, ids)
    moved = list(ids)
    moved[far] = (ids[far] + 1) % 96
    assert float(rows_err(O.forward(cfg, w, moved), want)[probe]) > 10 * TOL32           # the far token carries weight
    eng = engine(model)
    assert err(whole(eng, ids), want) < TOL32
    assert err(in_portions(eng, ids, [probe - 1, 1]), want) < TOL32
    assert err(in_portions(eng, ids, [far + 1, 37]), want) < TOL32


def test_convolution_history_crosses_portions_and_starts_empty():
    def taps(w):
        w["l0.mix.right.conv"] = (1.5 * w["l0.mix.right.conv"].float()).to(torch.bfloat16)
    cfg, w, model = make(pattern="p", ffs="-", conv=4, loop=None, edit=taps)
    ids = toks(40, seed=70)
    want = O.forward(cfg, w, ids)
    flat = dict(w)
    flat["l0.mix.right.conv"] = w["l0.mix.right.conv"].clone()
    flat["l0.mix.right.conv"][:, :-1] = 0                       # only the current token's tap
    assert err(O.forward(cfg, flat, ids), want) > 100 * TOL32
    eng = engine(model, max_tokens=64, max_seqs=1)                # one slot: every run starts on the last one's history
    for sizes in ([1], [2], [3, 1, 2, 5], [40]):
        assert err(in_portions(eng, ids, sizes), want) < TOL32, sizes


def test_the_score_bias_and_the_mixer_weights_count():
    cfg, w, model = make(pattern="p", ffs="-", loop=None)
    ids = toks(30, seed=50)
    want = O.forward(cfg, w, ids)
    none = dict(w)
    none["l0.mix.left.pb"] = torch.zeros_like(w["l0.mix.left.pb"])
    assert err(O.forward(cfg, none, ids), want) > 50 * TOL32
    swapped = copy.deepcopy(cfg)
    m = swapped["layers"][0]["mixer"]
    m["left_scale"], m["right_scale"] = m["right_scale"], m["left_scale"]
    assert err(O.forward(swapped, w, ids), want) > 50 * TOL32
    assert err(in_portions(engine(model), ids, [17, 1]), want) < TOL32


# ---- other sizes ---------------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kw", [
    dict(heads=2, kv_heads=2), dict(heads=1, kv_heads=1), dict(heads=4, kv_heads=1), dict(top=1), dict(experts=3, top=3),
    dict(experts=1, top=1), dict(conv=1), dict(conv=2), dict(conv=8), dict(rot_dims=16), dict(rot_dims=0), dict(window=1),
    dict(window=1000), dict(shared_ff=0), dict(scale=1.0), dict(groups=1), dict(groups=4), dict(norm_groups=1),
    dict(norm_groups=4), dict(s_heads=1, groups=1, norm_groups=1), dict(d_heads=1), dict(d_heads=3, d_dim=12),
    dict(mult=1.0, left_scale=1.0, right_scale=1.0, router_scale=1.0), dict(vdim=16), dict(eps=1e-3),
    dict(width=72, dim=12, vdim=20, rot_dims=6, s_vdim=6, state=10, d_dim=20, ff=28, expert_ff=10, shared_ff=12, experts=5, top=3),
    dict(width=40, dim=8, vdim=8, s_heads=2, s_vdim=4, state=4, groups=2, d_dim=8, ff=8, expert_ff=8, shared_ff=8, heads=2,
         kv_heads=2),
    dict(width=66, dim=10, vdim=34, rot_dims=10, s_heads=3, s_vdim=11, state=17, groups=3, norm_groups=3, d_heads=1, d_dim=34,
         ff=18, expert_ff=6, shared_ff=10),
    dict(vdim=136, heads=2, kv_heads=1, state=40, d_dim=72, d_heads=1)])
def test_other_sizes(kw):
    cfg, w, model = make(pattern="pgpg", ffs="mddm", seed=2, loop=(1, 3, 2), **kw)
    ids = toks(75, seed=4)
    assert err(in_portions(engine(model), ids, [37, 2, 1]), O.forward(cfg, w, ids)) < TOL32


# ---- the engine's own entry points ------------------------------------------------------------------------------------------------
def test_greedy_generation_through_the_scheduler():
    cfg, w, model = make(pattern="gpg", ffs="dmd")
    prompts = [toks(33, seed=80), toks(5, seed=81), toks(70, seed=82), toks(1, seed=83)]
    eng = engine(model, max_tokens=256, max_seqs=2)                  # four prompts over two slots and four pages
    outs = eng.generate(prompts, max_new_tokens=12, step_tokens=48)
    assert not eng.cache.seqs and len(eng.cache.free_slots) == 2
    for p, o in zip(prompts, outs):
        assert len(o) == 12
        logits = O.forward(cfg, w, p + o)
        for k, tok in enumerate(o):                                   # each new token is the restatement's choice, or ties it
            row = logits[len(p) + k - 1]
            assert float(row.max() - row[tok]) < 1e-3 * float(row.abs().max()), (k, tok)


def _save(tmp, cfg, w):
    from safetensors.torch import save_file
    tmp.mkdir(exist_ok=True)
    (tmp / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in w.items()}, str(tmp / "model.safetensors"))


def test_generate_command(tmp_path):
    cfg, w, model = make(pattern="pg", ffs="md")
    _save(tmp_path, cfg, w)
    prompts = [toks(9, seed=85), toks(40, seed=86)]
    cmd = [sys.executable, "-m", "proxy_inference_engine_b200", "generate", "--model", str(tmp_path), "--dtype", "float32",
           "--max-new-tokens", "6"] + [x for p in prompts for x in ("--prompt-ids", ",".join(map(str, p)))]
    r = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(ln) for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert [ln["prompt_ids"] for ln in lines] == prompts
    want = engine(model).generate(prompts, max_new_tokens=6)
    assert [ln["generated_ids"] for ln in lines] == want


def test_trace_replay_program(tmp_path):
    cfg, w, _ = make(pattern="gpg", ffs="dmd")
    mdir, odir = tmp_path / "model", tmp_path / "out"
    _save(mdir, cfg, w)
    a, b = toks(70, seed=90), toks(20, seed=91)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": a[66:68], "want": []}, {"id": "b", "tokens": b[:19], "want": [18]}], "end": []},
             {"step": 2, "entries": [{"id": "b", "tokens": b[19:], "want": [0]}, {"id": "a", "tokens": a[68:], "want": [1]}], "end": ["a", "b"]}]
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", str(mdir), "--dtype", "float32",
                        "--out", str(odir), "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n",
                       capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [ln for ln in r.stdout.splitlines() if ln.startswith("done")] == ["done 0", "done 1", "done 2"]
    wa, wb = O.forward(cfg, w, a), O.forward(cfg, w, b)
    read = lambda n: torch.frombuffer(bytearray((odir / f"{n}.f32").read_bytes()), dtype=torch.float32).view(-1, cfg["vocab"])
    assert err(read(0), wa[[0, 65]]) < TOL32
    assert err(read(1), wb[[18]]) < TOL32
    assert err(read(2), torch.stack([wb[19], wa[69]])) < TOL32
