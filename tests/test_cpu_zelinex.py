"""CPU: the host side of the Zelinex family -- config reader and registry, the order of layer runs under a loop, the
synthetic checkpoint's tensor names, one cache entry per run -- and checks of the plain restatement itself
(tests/zelinex_oracle.py) against closed forms, so that what the GPU tests compare with is pinned."""
import copy
import math

import pytest
import torch

import zelinex_oracle as O

F = torch.float64


def test_registry_and_config_reader():
    from proxy_inference_engine_b200.checkpoint import MODEL_REGISTRY, model_kind
    from proxy_inference_engine_b200.zelinex import ZelinexArgs
    cfg = O.random_config()
    a = ZelinexArgs.from_dict(cfg)
    assert (a.vocab, a.width, a.norm_eps, a.residual_mult) == (96, 64, 1e-5, 0.7)
    assert a.loop == {"start": 0, "stop": 1, "times": 2}
    assert ZelinexArgs.from_dict(a.to_dict()).layers == a.layers and ZelinexArgs.from_dict(a.to_dict()).loop == a.loop
    assert model_kind(cfg) == "Zelinex" and "Zelinex" in MODEL_REGISTRY
    plain = {k: v for k, v in cfg.items() if k not in ("loop", "residual_mult", "norm")}
    b = ZelinexArgs.from_dict(plain)
    assert b.loop is None and b.residual_mult == 1.0 and b.norm_eps == 1e-6
    for edit in (lambda c: c["layers"][0].update(type="attention"),
                 lambda c: c["layers"][0]["mixer"].pop("dim"),
                 lambda c: c["layers"][1]["mixer"].pop("right"),
                 lambda c: c["layers"][1]["mixer"]["left"].pop("scale"),
                 lambda c: c["layers"][1]["mixer"]["left"].update(kv_heads=3),
                 lambda c: c["layers"][1]["mixer"]["left"]["rot"].update(dims=7),
                 lambda c: c["layers"][1]["mixer"]["right"].update(groups=3),
                 lambda c: c["layers"][1]["mixer"]["right"].update(norm_groups=5),
                 lambda c: c["layers"][1]["mixer"]["right"].update(conv=12),
                 lambda c: c["layers"][0]["mlp"].update(kind="glu"),
                 lambda c: c["layers"][1]["mlp"]["router"].update(top=9),
                 lambda c: c["loop"].update(stop=5),
                 lambda c: c["loop"].update(start=1, stop=1),
                 lambda c: c["loop"].update(times=0)):
        bad = copy.deepcopy(cfg)
        edit(bad)
        with pytest.raises(ValueError):
            ZelinexArgs.from_dict(bad)


def test_order_of_layer_runs():
    from proxy_inference_engine_b200.zelinex import ZelinexArgs
    runs = lambda **kw: ZelinexArgs.from_dict(O.random_config(**kw)).runs()
    assert runs(pattern="gpg", loop=None) == [(0, None), (1, None), (2, None)]
    assert runs(pattern="gpg", loop=(0, 3, 1)) == [(0, 0), (1, None), (2, None)]
    assert runs(pattern="gpg", loop=(1, 2, 3)) == [(0, None), (1, 0), (1, 1), (1, 2), (2, None)]
    assert runs(pattern="gpgp", loop=(1, 3, 2)) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
    got, times = O.layer_runs(O.random_config(pattern="gpgp", loop=(1, 3, 2)))            # the restatement's own order agrees
    assert [i for i, _, _ in got] == [0, 1, 2, 1, 2, 3] and times == 2
    assert [(t, first) for _, t, first in got] == [(None, False), (0, True), (0, False), (1, True), (1, False), (None, False)]


def test_random_weights_cover_every_tensor_the_restatement_reads():
    from proxy_inference_engine_b200.zelinex import ZelinexArgs, random_weights
    cfg = O.random_config(pattern="gpgp", ffs="dm-d", loop=(1, 3, 2))
    w = random_weights(ZelinexArgs.from_dict(cfg), seed=3)
    for name in ("embed", "final.norm", "loop.step", "l0.norm1b", "l0.norm2b", "l0.mix.r", "l0.mix.a.b", "l0.mix.w0", "l0.mlp.act",
                 "l1.mix.left.pb", "l1.mix.right.in", "l1.mix.right.conv.b", "l1.mix.right.D", "l1.mlp.router", "l1.mlp.e5.down",
                 "l1.mlp.shared.gate"):
        assert name in w, name
    assert "head" not in w and "l2.norm2" not in w and "l2.mlp.up" not in w            # tied embeddings; layer 2 has no feed-forward
    assert w["loop.step"].shape == (2, 64) and w["l1.mix.right.in"].shape == (2 * 32 + 2 * 2 * 12 + 4, 64)
    assert w["l1.mix.right.conv"].shape == (32 + 48, 3) and w["l0.mix.w2"].shape[0] == 32
    trace = []
    logits = O.forward(cfg, w, [1, 2, 3, 4, 5, 6, 7, 8, 9], trace)
    assert logits.shape == (9, 96) and len(trace) == 6 and bool(torch.isfinite(logits).all())


def test_one_cache_entry_per_layer_run():
    from proxy_inference_engine_b200.cache import HybridCache

    class _Alloc:        # the allocator lives in the native library; this one hands out ids the same way
        def __init__(self, n, *_a, **_k): self.free = list(range(n - 1, -1, -1))
        def allocate_pages(self, n): return [self.free.pop() for _ in range(n)]
        def free_pages(self, ps): self.free += list(reversed(ps))
        def get_num_free_pages(self): return len(self.free)
    import proxy_inference_engine_b200.paging as paging
    par = {"pages": {"k": (2, 16), "v": (2, 24)}, "slots": {"state": (4, 12, 8), "conv": (2, 80)}}
    dl = {"slots": {"state": (2, 16, 16)}}
    orig, paging.PageAllocator = paging.PageAllocator, _Alloc
    try:
        c = HybridCache([dl, par, dl, par], 130, 2, "cpu", torch.bfloat16)     # a looped (delta, parallel) pair: four runs
    finally:
        paging.PageAllocator = orig
    assert c.n_pages == 3 and len(c.layers) == 4
    assert c.layers[1]["k"].shape == (3, 64, 2, 16) and c.layers[1]["v"].dtype == torch.bfloat16
    assert c.layers[1]["state"].shape == (2, 4, 12, 8) and c.layers[1]["conv"].shape == (2, 2, 80)
    assert c.layers[0]["state"].shape == (2, 2, 16, 16) and c.layers[0]["state"].dtype == torch.float32
    assert c.layers[1]["state"].data_ptr() != c.layers[3]["state"].data_ptr()           # each pass has its own
    assert {"state", "conv"} <= c.slot_keys


# ---- the restatement against closed forms --------------------------------------------------------------------------------------
def test_rotation_pairs_feature_i_with_i_plus_half():
    x = torch.zeros((3, 1, 6), dtype=F)
    x[:, 0, 0], x[:, 0, 5] = 1.0, 7.0
    y = O.rotate_half(x, torch.tensor([0, 1, 2]), 4, 100.0)
    assert torch.allclose(y[0], x[0]) and float(y[1, 0, 5]) == 7.0                    # position 0 and unrotated features
    assert torch.allclose(y[2, 0, :4], torch.tensor([math.cos(2.0), 0.0, math.sin(2.0), 0.0], dtype=F), atol=1e-12)
    q, k = torch.randn((1, 1, 4), dtype=F), torch.randn((1, 1, 4), dtype=F)           # scores depend on the distance only
    dot = lambda a, b: float((O.rotate_half(q, torch.tensor([a]), 4, 50.0) * O.rotate_half(k, torch.tensor([b]), 4, 50.0)).sum())
    assert abs(dot(9, 4) - dot(25, 20)) < 1e-9


def test_sigmoid_weights_are_not_normalised_and_the_window_counts_the_query_itself():
    q, k = torch.zeros((4, 1, 2), dtype=F), torch.zeros((4, 1, 2), dtype=F)
    v = torch.arange(4, dtype=F).view(4, 1, 1) + 1
    out = O.sigmoid_window_attention(q, k, v, 1.0, 10, torch.tensor([0.0]))
    assert torch.allclose(out[:, 0, 0], torch.tensor([0.5, 1.5, 3.0, 5.0], dtype=F))        # every key weighs 1/2: the sum grows
    out = O.sigmoid_window_attention(q, k, v, 1.0, 2, torch.tensor([math.log(3.0)]))
    assert torch.allclose(out[:, 0, 0], 0.75 * torch.tensor([1.0, 3.0, 5.0, 7.0], dtype=F))   # itself and ONE before it, 3/4 each
    q2 = torch.tensor([[[2.0, 0.0], [0.0, 2.0]], [[2.0, 0.0], [0.0, 2.0]]], dtype=F)       # two query heads share one key head
    k2 = torch.tensor([[[1.0, 4.0]], [[-1.0, 0.0]]], dtype=F)
    out = O.sigmoid_window_attention(q2, k2, torch.ones((2, 1, 1), dtype=F), 0.5, 5, torch.tensor([0.0, -1.0]))
    s = lambda z: 1 / (1 + math.exp(-z))
    assert abs(float(out[1, 0, 0]) - (s(1.0) + s(-1.0))) < 1e-12 and abs(float(out[1, 1, 0]) - (s(4.0 - 1.0) + s(-1.0))) < 1e-12


def test_convolution_is_causal_per_channel_with_bias_and_silu():
    g = torch.Generator().manual_seed(0)
    x, w, b = torch.randn((9, 5), generator=g, dtype=F), torch.randn((5, 3), generator=g, dtype=F), torch.randn(5, generator=g, dtype=F)
    lin = torch.nn.functional.conv1d(torch.nn.functional.pad(x.T[None], (2, 0)), w[:, None, :], bias=b, groups=5)[0].T
    assert torch.allclose(O.causal_conv_silu(x, w, b), lin * torch.sigmoid(lin), atol=1e-12)
    first = x[0] * w[:, 2] + b                                                         # the first row sees only itself
    assert torch.allclose(O.causal_conv_silu(x, w, b)[0], first * torch.sigmoid(first), atol=1e-12)


def test_state_space_scan_closed_form():
    L, dt, A = 5, 0.5, math.log(2.0)                   # decay exp(-2 * 0.5) = 1/e per token
    x, B, Cm = torch.ones((L, 1, 1), dtype=F), torch.ones((L, 1, 1), dtype=F), torch.full((L, 1, 1), 3.0, dtype=F)
    y = O.ssd_scan(x, B, Cm, torch.full((L, 1), dt, dtype=F), torch.tensor([A], dtype=F), torch.tensor([0.25], dtype=F))
    for t in range(L):                                 # S_t = dt (1 + e^-1 + ... + e^-t);  y = 3 S + D x
        s = dt * sum(math.exp(-j) for j in range(t + 1))
        assert abs(float(y[t, 0, 0]) - (3 * s + 0.25)) < 1e-12
    x2 = torch.ones((2, 4, 1), dtype=F)                # four heads, two groups: heads 0, 1 read group 0
    B2 = torch.tensor([[[1.0], [10.0]], [[1.0], [10.0]]], dtype=F)
    y2 = O.ssd_scan(x2, B2, torch.ones((2, 2, 1), dtype=F), torch.ones((2, 4), dtype=F), torch.full((4,), -50.0, dtype=F),
                    torch.zeros(4, dtype=F))
    assert torch.allclose(y2[1, :, 0], torch.tensor([2.0, 2.0, 20.0, 20.0], dtype=F), atol=1e-9)


def test_generalized_delta_rule_closed_form():
    n = 3
    e0 = torch.tensor([1.0, 0.0, 0.0], dtype=F)
    k = torch.stack([2 * e0, 2 * e0]).view(2, 1, n)
    v = torch.tensor([[1.0, 2.0, 3.0], [10.0, 20.0, 30.0]], dtype=F).view(2, 1, n)
    r = torch.stack([e0, e0]).view(2, 1, n)
    one = torch.ones((2, 1, n), dtype=F)
    # full removal along the key, no decay: the second write REPLACES what the first left in that direction (up to the 1e-6)
    o = O.delta_scan(r, k, v, one, one)
    assert torch.allclose(o[0, 0], 2 * v[0, 0], atol=1e-12)
    assert torch.allclose(o[1, 0], 2 * v[1, 0], atol=1e-4) and not torch.allclose(o[1, 0], 2 * v[1, 0], rtol=0, atol=1e-9)
    # no removal, decay 1/2 per token: the writes add up, the older one halved
    o = O.delta_scan(r, k, v, 0.5 * one, 0 * one)
    assert torch.allclose(o[1, 0], 2 * (0.5 * v[0, 0] + v[1, 0]), atol=1e-12)
    # the decay acts per KEY channel: a state row whose channel decays to zero is gone, the others stay
    k2 = torch.tensor([[1.0, 1.0, 0.0], [0.0, 0.0, 1.0]], dtype=F).view(2, 1, n)
    dec = torch.tensor([[1.0, 1.0, 1.0], [0.0, 1.0, 1.0]], dtype=F).view(2, 1, n)
    r2 = torch.tensor([[0.0, 0.0, 0.0], [1.0, 1.0, 0.0]], dtype=F).view(2, 1, n)
    o = O.delta_scan(r2, k2, v, dec, 0 * one)
    assert torch.allclose(o[1, 0], v[0, 0], atol=1e-12)          # row 0 forgotten, row 1 kept: one copy of v_0, not two


def test_decay_range_and_gates_of_the_delta_mixer():
    W, H, n = 4, 1, 2
    z = lambda *s: torch.zeros(s, dtype=F)
    w = {"r": z(2, W), "k": z(2, W), "v": z(2, W), "g": z(2, W), "a": z(2, W), "a.b": z(2), "w1": z(3, W), "w2": z(2, 3),
         "w0": torch.tensor([60.0, -60.0], dtype=F), "norm": torch.tensor([2.0, 3.0], dtype=F), "o": torch.eye(W, 2, dtype=F)}
    w["r"][:, 0] = w["k"][:, 0] = w["v"][:, 0] = 1.0
    h = torch.ones((1, W), dtype=F)
    out = O.delta_mixer(h, w, "", {"heads": H, "dim": n}, 0.0)
    # one token: S = k v^T, o = S^T r = |k.r| v = 2 (1, 1); unit rms -> (1, 1); weight (2, 3); gate sigmoid(0) = 1/2
    assert torch.allclose(out[0], torch.tensor([1.0, 1.5, 0.0, 0.0], dtype=F), atol=1e-12)
    lo, hi = math.exp(-math.exp(-0.5)), 1.0            # the decay lies between exp(-e^(-1/2)) = 0.545 and 1
    lora = torch.tanh(h @ w["w1"].T) @ w["w2"].T + w["w0"]
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(lora))
    assert abs(float(decay[0, 0]) - lo) < 1e-12 and abs(float(decay[0, 1]) - hi) < 1e-12


def test_xielu_branches():
    z = torch.tensor([-3.0, -1e-3, 0.0, 1e-3, 2.0], dtype=F)
    p, q = torch.tensor(0.3, dtype=F), torch.tensor(-0.4, dtype=F)
    y = O.xielu(z, p, q)
    ap, aq = math.log1p(math.exp(0.3)), 0.5 + math.log1p(math.exp(-0.4))
    assert abs(float(y[4]) - (ap * 4 + 1)) < 1e-12 and abs(float(y[0]) - (aq * (math.exp(-3) + 2) - 1.5)) < 1e-12
    assert float(y[2]) == 0 and abs(float(y[1]) + float(y[3])) < 1e-5          # slope 1/2 on both sides of zero


def test_router_renormalises_the_chosen_scores_and_adds_the_shared_expert():
    W = 4
    w = {"router": torch.eye(3, W, dtype=F)}
    for e, name in enumerate(("e0.", "e1.", "e2.", "shared.")):
        w[name + "gate"] = torch.full((1, W), 100.0, dtype=F)          # silu(large) = the value itself
        w[name + "up"] = torch.zeros((1, W), dtype=F)
        w[name + "up"][0, 3] = 1.0
        w[name + "down"] = torch.full((W, 1), float(10 ** e), dtype=F)
    mlp = {"router": {"experts": 3, "top": 2, "scale": 4.0}, "expert": {"ff": 1}, "shared": {"ff": 1}}
    h = torch.tensor([[2.0, 1.0, 5.0, 1.0]], dtype=F)                  # logits (2, 1, 5): experts 2 and 0
    out = O.moe(h, w, "", mlp)
    a = 1 / (1 + math.exp(-3.0))                                       # score_2 / (score_2 + score_0)
    gate = 100.0 * 9.0
    assert abs(float(out[0, 0]) - gate * (4.0 * (a * 100 + (1 - a) * 1) + 1000.0)) < 1e-6 * gate * 1400
    none = dict(mlp, shared=None)
    assert abs(float(O.moe(h, w, "", none)[0, 0]) - gate * 4.0 * (a * 100 + (1 - a) * 1)) < 1e-6 * gate * 400


def test_sandwich_residual_and_loop_injection():
    """One delta layer whose mixer output is made a constant direction: the residual gains mult * unit-rms * norm1b, and a
    second pass adds the embedding and its own pass vector first."""
    from proxy_inference_engine_b200.zelinex import ZelinexArgs, random_weights
    cfg = O.random_config(pattern="g", ffs="-", loop=(0, 1, 2), mult=0.25, width=16, d_heads=1, d_dim=8)
    w = random_weights(ZelinexArgs.from_dict(cfg), seed=1)
    trace = []
    O.forward(cfg, w, [3, 4], trace)
    f = lambda n: w[n].double()
    x0 = f("embed")[[3, 4]]
    x = x0 + f("loop.step")[0]
    y = O.delta_mixer(O.unit_rms(x, 1e-5) * f("l0.norm1"), {k[len("l0.mix."):]: f(k) for k in w if k.startswith("l0.mix.")}, "",
                      cfg["layers"][0]["mixer"], 1e-5)
    x1 = x + 0.25 * O.unit_rms(y, 1e-5) * f("l0.norm1b")
    assert torch.allclose(trace[0], x1, atol=1e-12)
    x = x1 + x0 + f("loop.step")[1]
    y = O.delta_mixer(O.unit_rms(x, 1e-5) * f("l0.norm1"), {k[len("l0.mix."):]: f(k) for k in w if k.startswith("l0.mix.")}, "",
                      cfg["layers"][0]["mixer"], 1e-5)
    assert torch.allclose(trace[1], x + 0.25 * O.unit_rms(y, 1e-5) * f("l0.norm1b"), atol=1e-12)
