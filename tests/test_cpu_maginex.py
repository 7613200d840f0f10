"""CPU: the host side of the Maginex family -- config reader and registry, the synthetic checkpoint's tensor names, the
cache spec that mixes page pools with slot tensors -- and checks of the plain restatement itself (tests/maginex_oracle.py)
against closed forms, so that what the GPU tests compare with is pinned."""
import copy
import math

import pytest
import torch

import maginex_oracle as O

F = torch.float64


def test_registry_and_config_reader():
    from proxy_inference_engine_b200.checkpoint import MODEL_REGISTRY, model_kind
    from proxy_inference_engine_b200.maginex import MaginexArgs
    cfg = O.random_config()
    a = MaginexArgs.from_dict(cfg)
    assert (a.vocab, a.width, a.norm_eps, a.embed_scale, a.taps) == (96, 64, 1e-5, 4.0, 3)
    assert MaginexArgs.from_dict(a.to_dict()).layers == a.layers
    assert model_kind(cfg) == "Maginex" and "Maginex" in MODEL_REGISTRY
    plain = {k: v for k, v in cfg.items() if k not in ("embedding", "canon")}
    b = MaginexArgs.from_dict(plain)
    assert b.embed_scale == 1.0 and b.taps == 1
    for edit in (lambda c: c["layers"][0].update(type="conv"),
                 lambda c: c["layers"][0]["mixer"].pop("scale"),
                 lambda c: c["layers"][0]["mixer"].update(kv_heads=3),
                 lambda c: c["layers"][0]["mixer"]["rot"].update(dims=7),
                 lambda c: c["layers"][1]["mixer"].pop("kv_rank"),
                 lambda c: c["layers"][2]["mlp"].update(kind="dense"),
                 lambda c: c["layers"][2]["mlp"]["router"].update(top=9),
                 lambda c: c["canon"].update(taps=12)):
        bad = copy.deepcopy(cfg)
        edit(bad)
        with pytest.raises(ValueError):
            MaginexArgs.from_dict(bad)
    two = O.random_config(pattern="aa")
    two["layers"][1]["mixer"]["vdim"] = 8       # value-mixing layers blend the SAME token's values: shapes must agree
    with pytest.raises(ValueError):
        MaginexArgs.from_dict(two)


def test_random_weights_cover_every_tensor_the_restatement_reads():
    from proxy_inference_engine_b200.maginex import MaginexArgs, random_weights
    cfg = O.random_config(pattern="alma")
    w = random_weights(MaginexArgs.from_dict(cfg), seed=3)
    for name in ("embed", "head", "final.norm", "l0.canon1", "l0.canon2", "l0.mix.sink", "l0.mix.vmix", "l0.mix.g",
                 "l1.mix.dq.norm", "l1.mix.uk", "l2.mix.z.b", "l2.mlp.router.b", "l2.mlp.e5.down", "l3.mlp.shared.up"):
        assert name in w, name
    assert w["l0.mix.g"].shape == (4, 64) and w["l1.mix.g"].shape == (4 * 24, 64) and w["l0.canon1"].shape == (64, 3)
    trace = []
    logits = O.forward(cfg, w, [1, 2, 3, 4, 5, 6, 7, 8, 9], trace)
    assert logits.shape == (9, 96) and len(trace) == 4 and bool(torch.isfinite(logits).all())


def test_cache_spec_with_pages_and_slots():
    from proxy_inference_engine_b200.cache import HybridCache

    class _Alloc:        # the allocator lives in the native library; this one hands out ids the same way
        def __init__(self, n, *_a, **_k): self.free = list(range(n - 1, -1, -1))
        def allocate_pages(self, n): return [self.free.pop() for _ in range(n)]
        def free_pages(self, ps): self.free += list(reversed(ps))
        def get_num_free_pages(self): return len(self.free)
    import proxy_inference_engine_b200.paging as paging
    orig, paging.PageAllocator = paging.PageAllocator, _Alloc
    try:
        c = HybridCache([{"pages": {"k": (2, 8), "v": (2, 12)}, "slots": {"canon": (2, 16)}}, {"slots": {"state": (10,)}},
                         {"kind": "attention", "G": 1, "d": 4, "dv": 4}], 200, 3, "cpu", torch.bfloat16)
    finally:
        paging.PageAllocator = orig
    assert c.n_pages == 4 and c.layers[0]["k"].shape == (4, 64, 2, 8) and c.layers[0]["v"].dtype == torch.bfloat16
    assert c.layers[0]["canon"].shape == (3, 2, 16) and c.layers[0]["canon"].dtype == torch.float32
    assert c.layers[1]["state"].shape == (3, 10) and c.layers[2]["k"].shape == (4, 64, 1, 8)
    assert {"canon", "state"} <= c.slot_keys
    s = c.admit("a")
    c.reserve("a", 70)
    assert len(s["pages"]) == 2
    c.release("a")
    assert c.admit("b")["slot"] == s["slot"] and c.reserve("b", 1)["pages"] == s["pages"][:1]   # both come back first


def test_canon_is_a_causal_depthwise_convolution():
    g = torch.Generator().manual_seed(0)
    h, w = torch.randn((9, 5), generator=g, dtype=F), torch.randn((5, 3), generator=g, dtype=F)
    want = h + torch.nn.functional.conv1d(torch.nn.functional.pad(h.T[None], (2, 0)), w[:, None, :], groups=5)[0].T
    assert torch.allclose(O.canon(h, w), want, atol=1e-12)
    assert torch.allclose(O.canon(h, w)[0], h[0] * (1 + w[:, 2]), atol=1e-12)        # the first row sees only itself


def test_rotation_pairs_feature_i_with_i_plus_half():
    x = torch.zeros((3, 1, 6), dtype=F)
    x[:, 0, 0], x[:, 0, 5] = 1.0, 7.0
    y = O.rotate_half(x, torch.tensor([0, 1, 2]), 4, 100.0)
    assert torch.allclose(y[0], x[0]) and float(y[1, 0, 5]) == 7.0                    # position 0 and unrotated features
    assert torch.allclose(y[2, 0, :4], torch.tensor([math.cos(2.0), 0.0, math.sin(2.0), 0.0], dtype=F), atol=1e-12)
    q, k = torch.randn((1, 1, 4), dtype=F), torch.randn((1, 1, 4), dtype=F)           # scores depend on the distance only
    dot = lambda a, b: float((O.rotate_half(q, torch.tensor([a]), 4, 50.0) * O.rotate_half(k, torch.tensor([b]), 4, 50.0)).sum())
    assert abs(dot(9, 4) - dot(25, 20)) < 1e-9


def test_sink_takes_its_share_and_window_counts_the_query_itself():
    q, k = torch.zeros((4, 1, 2), dtype=F), torch.zeros((4, 1, 2), dtype=F)
    v = torch.arange(4, dtype=F).view(4, 1, 1) + 1
    out = O.sink_attention(q, k, v, 1.0, 0, torch.tensor([math.log(2.0)]))
    assert torch.allclose(out[:, 0, 0], torch.tensor([1 / 3, 3 / 4, 6 / 5, 10 / 6], dtype=F))   # n keys of weight 1, sink 2
    out = O.sink_attention(q, k, v, 1.0, 2, torch.tensor([-1e9]))
    assert torch.allclose(out[:, 0, 0], torch.tensor([1.0, 1.5, 2.5, 3.5], dtype=F))            # itself and ONE before it


def test_mingru_closed_form():
    w = {"z": torch.zeros((2, 3), dtype=F), "z.b": torch.zeros(2, dtype=F), "x": torch.zeros((2, 3), dtype=F),
         "x.b": torch.tensor([1.0, -2.0], dtype=F), "g": torch.zeros((2, 3), dtype=F), "o": torch.eye(2, dtype=F)}
    w["g"][:, 0] = 1.0
    h = torch.ones((4, 3), dtype=F)
    out = O.mingru_mixer(h, w, "")
    cand = torch.tensor([1.5, 1 / (1 + math.exp(2.0))], dtype=F)       # u + 1/2 above zero, sigmoid(u) below
    silu1 = 1.0 / (1 + math.exp(-1.0))
    for t in range(4):                                                  # z = 1/2: S_t = cand (1 - 2^-(t+1))
        assert torch.allclose(out[t], cand * (1 - 0.5 ** (t + 1)) * silu1, atol=1e-12)


def test_router_takes_the_largest_logits_and_weighs_them_among_themselves():
    W = 4
    w = {"router": torch.eye(3, W, dtype=F), "router.b": torch.tensor([0.0, 0.0, 5.0], dtype=F)}
    for e in range(3):
        w[f"e{e}.up"] = torch.ones((1, W), dtype=F)
        w[f"e{e}.down"] = torch.full((W, 1), float(10 ** e), dtype=F)
    mlp = {"router": {"experts": 3, "top": 2}, "expert": {"ff": 1}, "shared": None}
    h = torch.tensor([[2.0, 1.0, 0.0, 0.0], [-3.0, -1.0, -9.0, 0.0]], dtype=F)      # logits (2, 1, 5) and (-3, -1, -4)
    out = O.moe(h, w, "", mlp)
    a = 1 / (1 + math.exp(-3.0))            # experts 2 and 0, weights softmax(5, 2)
    assert abs(float(out[0, 0]) - 9.0 * (a * 100 + (1 - a) * 1)) < 1e-9
    assert torch.allclose(out[1], torch.zeros(W, dtype=F))                            # relu^2 of a negative sum
