"""Maginex on the GPU against the plain restatement of tests/maginex_oracle.py: every mixer and the feed-forward alone,
prompts against token-by-token decoding, portions down to two tokens, mixed batches, re-used pages and slots, keys just
inside and just outside the window, far keys and page borders, sinks, value blending, the first tokens of a sequence, long
decoding, sizes where counts collapse to 1 or are not multiples of 8, the tensor-core paths, greedy generation through the
engine's scheduler and the trace replay program."""
import copy
import json
import os
import subprocess
import sys

import pytest
import torch

import maginex_oracle as O

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TOL32, TOL16 = 2e-4, 5e-2


def make(cfg=None, seed=0, dtype="float32", edit=None, **kw):
    from proxy_inference_engine_b200.maginex import MaginexArgs, MaginexModel, random_weights
    cfg = copy.deepcopy(cfg) if cfg else O.random_config(**kw)
    args = MaginexArgs.from_dict(cfg)
    w = random_weights(args, seed=seed)
    if edit:
        edit(w)
    return cfg, w, MaginexModel(args, w, "cuda", dtype)


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


# ---- every mechanism alone --------------------------------------------------------------------------------------------
@pytest.mark.parametrize("pattern,mlp", [("a", False), ("l", False), ("m", False), ("m", True), ("alm", True)])
def test_each_mixer_and_the_experts_alone(pattern, mlp):
    cfg, w, model = make(pattern=pattern, mlp=mlp)
    ids = toks(40)
    trace, otrace = [], []
    eng = engine(model, graph=False)
    got = eng.forward([("s", ids, list(range(40)))], trace=trace)
    want = O.forward(cfg, w, ids, otrace)
    for a, b in zip(trace, otrace):
        assert err(a, b) < TOL32
    assert err(got, want) < TOL32


def test_bf16_tracks_the_restatement():
    """In bf16 a token whose routing margin is within rounding may take another expert than the restatement, and nudges
    the tokens after it (attention, recurrent state): rows up to the first close call must be within the tolerance, nine
    rows in ten of all, and none far off."""
    cfg, w, model = make(pattern="almal", dtype="bfloat16")
    ids = toks(150)
    margins = []
    e = rows_err(in_portions(engine(model), ids, [70, 33, 1]), O.forward(cfg, w, ids, None, margins))
    clear = torch.cummin(torch.stack(margins).min(0).values, 0).values > 0.02
    assert int(clear.sum()) >= 5 and float(e[clear].max()) < TOL16
    assert float(e.quantile(0.9)) < TOL16 and float(e.max()) < 6 * TOL16


def test_bf16_without_routing_is_within_tolerance_everywhere():
    cfg, w, model = make(pattern="almal", dtype="bfloat16", mlp=False)
    ids = toks(150)
    assert err(in_portions(engine(model), ids, [70, 33, 1]), O.forward(cfg, w, ids)) < TOL16


@pytest.mark.parametrize("dtype,tol", [("float32", TOL32), ("bfloat16", None)])
def test_tensor_core_paths(dtype, tol):
    """Sizes at which prompt portions take the tiled attention kernel (head sizes 64 / 128, latent rank 128) and the
    tcgen05 products, the per-head batched ones included (K a multiple of 64, more than 32 rows)."""
    cfg = O.random_config(width=128, pattern="al", heads=2, kv_heads=1, dim=64, vdim=64, window=40, rot_dims=32, q_rank=64,
                          kv_rank=128, experts=4, top=2, ff=64, shared_ff=64)
    cfg, w, model = make(cfg, dtype=dtype)
    ids = toks(200)
    e = rows_err(in_portions(engine(model), ids, [130, 50, 1]), O.forward(cfg, w, ids))
    if tol:
        assert float(e.max()) < tol
    else:
        assert float(e.quantile(0.9)) < TOL16 and float(e.max()) < 6 * TOL16
    assert model.L.pieh_pipeline_error() == 0


# ---- prompts, decoding, portions, batches -------------------------------------------------------------------------------
def test_prefill_against_token_by_token_decoding():
    cfg, w, model = make(pattern="alm")
    ids = toks(70)
    want = O.forward(cfg, w, ids)
    eng = engine(model)
    assert err(whole(eng, ids), want) < TOL32
    assert err(in_portions(eng, ids, [1]), want) < TOL32            # one token at a time from the first one (graph replay)
    assert err(in_portions(engine(model, graph=False), ids, [1]), want) < TOL32


@pytest.mark.parametrize("sizes", [[2], [3, 2, 5, 2, 64, 7, 2], [63, 2, 1], [64, 64, 2], [65, 1]])
def test_portions_of_several_sizes(sizes):
    cfg, w, model = make(pattern="alm")
    ids = toks(140, seed=3)
    assert err(in_portions(engine(model), ids, sizes), O.forward(cfg, w, ids)) < TOL32


def test_unequal_requests_in_one_batch_match_each_alone():
    cfg, w, model = make(pattern="alma")
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
    cfg, w, model = make(pattern="alm")
    eng = engine(model, max_tokens=128, max_seqs=1)                  # two pages, one slot: everything is re-used
    for seed, n, sizes in ((11, 120, [50, 1]), (12, 100, [3, 64, 1]), (13, 128, [128]), (14, 9, [1])):
        ids = toks(n, seed=seed)
        assert err(in_portions(eng, ids, sizes, sid=seed), O.forward(cfg, w, ids)) < TOL32, seed
    assert eng.cache.allocator.get_num_free_pages() == 2 and len(eng.cache.free_slots) == 1


def test_long_decoding():
    cfg, w, model = make(pattern="alm", window=50)
    ids = toks(260, seed=9)
    assert err(in_portions(engine(model), ids, [20, 1]), O.forward(cfg, w, ids)) < TOL32


# ---- inputs made so that one key stands out ----------------------------------------------------------------------------
def _tie_keys_to_queries(w, layer, kind, gain):
    """The key projection becomes the query projection (times a gain): a token's query finds the SAME token's key."""
    p = f"l{layer}.mix."
    if kind == "a":
        w[p + "k"] = (gain * w[p + "q"].float()).to(torch.bfloat16)
    else:
        w[p + "dkv"], w[p + "dkv.norm"] = w[p + "dq"].clone(), w[p + "dq.norm"].clone()
        w[p + "uk"] = (gain * w[p + "uq"].float()).to(torch.bfloat16)


def _point_a_key_at_a_query(w, cfg, q_tok, k_tok, gain):
    """Rewrites the embedding of k_tok so that its key (layer 0, as many key heads as query heads, one tap) is a multiple of
    the query of q_tok: wherever both are visible, that key takes most of the softmax."""
    f = lambda n: w[n].double()
    tap = 1 + f("l0.canon1")[:, -1]
    u_q = O.rms_norm(f("embed")[q_tok] * cfg["embedding"]["scale"], f("l0.norm1"), cfg["norm"]["eps"]) * tap
    u_k = torch.linalg.pinv(f("l0.mix.k")) @ (f("l0.mix.q") @ u_q)          # k(u_k) = q(u_q)
    e = u_k / tap / f("l0.norm1")
    w["embed"][k_tok] = (e / e.abs().max()).to(torch.bfloat16)                # the norm takes the length out again
    w["l0.mix.k"] = (gain * f("l0.mix.k")).to(torch.bfloat16)


@pytest.mark.parametrize("window,probe", [(6, 20), (64, 64), (64, 100), (65, 130), (90, 200)])
def test_keys_just_inside_and_just_outside_the_window(window, probe):
    """One earlier token's key points at the probe's query, just inside the window or just outside it, so a window that is
    one token off changes the logits by far more than the tolerance."""
    cfg = O.random_config(pattern="a", heads=2, kv_heads=2, window=window, rot_dims=4, mlp=False, taps=1)
    cfg, w, model = make(cfg, edit=lambda w: _point_a_key_at_a_query(w, cfg, 95, 94, 4.0))
    for dist in (window - 1, window):
        ids = toks(probe + 6, seed=20 + dist, avoid=(94, 95))
        ids[probe], ids[probe - dist] = 95, 94
        want = O.forward(cfg, w, ids)
        other = copy.deepcopy(cfg)
        other["layers"][0]["mixer"]["mask"]["size"] = window + (1 if dist == window else -1)
        assert float(rows_err(O.forward(other, w, ids), want)[probe]) > 50 * TOL32       # the case does show the edge
        assert err(whole(engine(model), ids), want) < TOL32                              # inside a prompt
        assert err(in_portions(engine(model), ids, [probe - 3, 1]), want) < TOL32        # decoded alone
        assert err(in_portions(engine(model), ids, [probe - dist + 1, 2]), want) < TOL32  # portions that start at the edge


@pytest.mark.parametrize("far,probe", [(0, 63), (2, 64), (1, 65), (63, 128), (64, 300), (5, 447)])
def test_far_keys_and_page_borders_in_latent_attention(far, probe):
    cfg = O.random_config(pattern="l", q_rank=32, kv_rank=32, mlp=False)
    cfg, w, model = make(cfg, edit=lambda w: _tie_keys_to_queries(w, 0, "l", 2.0))
    ids = toks(probe + 3, seed=40 + far, avoid=(95,))
    ids[probe], ids[far] = 95, 95
    want = O.forward(cfg, w, ids)
    moved = list(ids)
    moved[far] = 94
    assert float(rows_err(O.forward(cfg, w, moved), want)[probe]) > 50 * TOL32           # the far key carries weight
    eng = engine(model)
    assert err(whole(eng, ids), want) < TOL32
    assert err(in_portions(eng, ids, [probe - 1, 1]), want) < TOL32
    assert err(in_portions(eng, ids, [far + 1, 37]), want) < TOL32


@pytest.mark.parametrize("pattern", ["a", "l"])
def test_the_sink_takes_its_share(pattern):
    def big_sink(w):
        w["l0.mix.sink"] = torch.tensor([3.0, -2.0, 5.0, 0.5]).to(torch.bfloat16)
    cfg, w, model = make(pattern=pattern, mlp=False, edit=big_sink)
    ids = toks(30, seed=50)
    want = O.forward(cfg, w, ids)
    none = dict(w)
    none["l0.mix.sink"] = torch.full((4,), -60.0).to(torch.bfloat16)
    assert err(O.forward(cfg, none, ids), want) > 100 * TOL32
    assert err(in_portions(engine(model), ids, [17, 1]), want) < TOL32


def test_values_blend_with_the_first_blending_layer_only():
    cfg = O.random_config(pattern="aaaa", mlp=False)
    cfg["layers"][0]["mixer"]["v_mix"] = False          # not a blending layer: layer 1 is the first one, 2 does not blend
    cfg["layers"][2]["mixer"]["v_mix"] = False
    def strong(w):
        w["l3.mix.vmix"] = torch.tensor(0.75).to(torch.bfloat16)
        w["l1.mix.vmix"] = torch.tensor(0.9).to(torch.bfloat16)     # the first blending layer's own weight is not used
    cfg, w, model = make(cfg, edit=strong)
    ids = toks(50, seed=60)
    want = O.forward(cfg, w, ids)
    off = dict(w)
    off["l3.mix.vmix"] = torch.tensor(0.0).to(torch.bfloat16)
    assert err(O.forward(cfg, off, ids), want) > 100 * TOL32
    assert err(in_portions(engine(model), ids, [23, 2, 1]), want) < TOL32


def test_convolution_history_crosses_portions_and_starts_empty():
    def taps(w):
        for k in list(w):
            if "canon" in k:
                w[k] = (2.0 * w[k].float()).to(torch.bfloat16)
    cfg, w, model = make(pattern="m", taps=4, edit=taps)
    ids = toks(40, seed=70)
    want = O.forward(cfg, w, ids)
    flat = {k: (torch.zeros_like(v) if "canon" in k else v) for k, v in w.items()}
    assert err(O.forward(cfg, flat, ids), want) > 100 * TOL32
    eng = engine(model, max_tokens=64, max_seqs=1)
    for sizes in ([1], [2], [3, 1, 2, 5], [40]):
        assert err(in_portions(eng, ids, sizes), want) < TOL32, sizes


# ---- other sizes ---------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("kw", [
    dict(heads=2, kv_heads=2), dict(heads=1, kv_heads=1), dict(heads=4, kv_heads=1), dict(top=1), dict(experts=3, top=3),
    dict(experts=1, top=1), dict(taps=1), dict(taps=5), dict(rot_dims=16), dict(rot_dims=0), dict(window=0), dict(window=1),
    dict(shared_ff=0), dict(scale=1.0), dict(v_mix=False),
    dict(width=72, dim=12, vdim=20, rot_dims=6, q_rank=20, kv_rank=40, gru=36, ff=28, shared_ff=12, experts=5, top=3),
    dict(width=40, dim=8, vdim=8, kv_rank=8, q_rank=8, gru=8, ff=8, shared_ff=8, heads=2, kv_heads=2),
    dict(kv_rank=320, vdim=136, heads=2, kv_heads=1), dict(kv_rank=16), dict(kv_rank=8, q_rank=40), dict(width=66, gru=30, ff=18, shared_ff=10, q_rank=18, kv_rank=22, vdim=10)])
def test_other_sizes(kw):
    cfg, w, model = make(pattern="aalm", seed=2, **kw)
    ids = toks(75, seed=4)
    assert err(in_portions(engine(model), ids, [37, 2, 1]), O.forward(cfg, w, ids)) < TOL32


# ---- the engine's own entry points ----------------------------------------------------------------------------------------
def test_greedy_generation_through_the_scheduler():
    cfg, w, model = make(pattern="alm")
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


def test_generate_command(tmp_path):
    from safetensors.torch import save_file
    cfg, w, model = make(pattern="lma")
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in w.items()}, str(tmp_path / "model.safetensors"))
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
    from safetensors.torch import save_file
    cfg, w, _ = make(pattern="alm")
    mdir, odir = tmp_path / "model", tmp_path / "out"
    mdir.mkdir()
    (mdir / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in w.items()}, str(mdir / "model.safetensors"))
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
