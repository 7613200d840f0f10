"""Throughput of the Golitar, Babodra, Maginex and Zelinex families at layer sizes of real models (random weights), with
every operator of the step timed in place and set against its roofline.  Golitar is shown beside the quantized Llama path
at equal width / feed-forward / depth; Babodra beside Golitar, Maginex beside Babodra, and Zelinex beside Golitar (the other
family built on a matrix-state recurrence and windowed attention), at equal width / depth / active feed-forward size.

``run(size, ...)`` is what ``bench.py --family golitar|babodra|maginex|zelinex`` prints.  Method: one prompt of ``prompt`` tokens goes through
``HybridEngine.forward`` in portions of ``portion`` rows (prefill tok/s, CUDA events around all portions), then ``batch``
sequences decode ``steps`` tokens each (decode tok/s).  The per-operator table wraps every library call of one prefill
portion and one decode step in a CUDA event pair; bytes and flops are the algorithmic ones of the call's shapes, the
roofline time is max(bytes / measured copy bandwidth, flops / measured bf16 tensor throughput), ``frac`` = roofline time /
measured time."""
from __future__ import annotations

import json
import os
import time

import torch

SIZES = {
    # width, feed-forward, heads x dims of the delta mixer and of the attention mixer, layers as a pattern string
    "1b": dict(width=2048, ff=8192, vocab=32000, pattern="dddadddadddadddA", dH=16, dG=16, dk=128, dv=128, aH=16, aG=4,
               ad=64, adv=128, window=1024, bab=dict(heads=16, kv_heads=4, dim=128, pattern="dmmmdmmmdmmmdmmm", experts=16, top=4,
                                                     groups=(4, 2), expert_ff=1536, shared_ff=2048),
               mag=dict(pattern="almalmalmalmalma", heads=16, kv_heads=4, dim=128, vdim=128, window=1024, rot_dims=64,
                        q_rank=768, kv_rank=128, gru=4096, experts=16, top=4, expert_ff=1536, shared_ff=2048, taps=4),
               zel=dict(pattern="gpgpgpgpgpgp", loop=(0, 4, 2), d_heads=16, d_dim=128, heads=16, kv_heads=4, dim=128, vdim=128,
                        window=1024, rot_dims=64, s_heads=32, s_vdim=64, state=128, groups=2, norm_groups=2, conv=4,
                        experts=16, top=4, expert_ff=1536, shared_ff=2048),
               llama=dict(hidden_size=2048, intermediate_size=8192, num_attention_heads=32,
                                                       num_key_value_heads=8, head_dim=64, vocab_size=32000)),
    "8b": dict(width=4096, ff=14336, vocab=32000, pattern="dddadddA", dH=32, dG=16, dk=128, dv=128, aH=32, aG=8, ad=64,
               adv=128, window=2048, bab=dict(heads=32, kv_heads=8, dim=128, pattern="dmmmdmmm", experts=16, top=4, groups=(4, 2),
                                              expert_ff=3072, shared_ff=2048),
               mag=dict(pattern="almalmal", heads=32, kv_heads=8, dim=128, vdim=128, window=2048, rot_dims=64, q_rank=1536,
                        kv_rank=128, gru=8192, experts=16, top=4, expert_ff=3072, shared_ff=2048, taps=4),
               zel=dict(pattern="gpgpgp", loop=(0, 2, 2), d_heads=32, d_dim=128, heads=32, kv_heads=8, dim=128, vdim=128,
                        window=2048, rot_dims=64, s_heads=64, s_vdim=64, state=128, groups=2, norm_groups=2, conv=4,
                        experts=16, top=4, expert_ff=3072, shared_ff=2048),
               llama=dict(hidden_size=4096, intermediate_size=14336, num_attention_heads=32,
                                                num_key_value_heads=8, head_dim=128, vocab_size=32000)),
}


def golitar_config(size: str) -> dict:
    s = SIZES[size]
    layers = []
    for ch in s["pattern"]:
        mlp = {"kind": "dense", "ff": s["ff"]}
        if ch == "d":
            layers.append({"type": "delta", "mlp": mlp,
                           "mixer": {"heads": s["dH"], "kv_heads": s["dG"], "dim": s["dk"], "vdim": s["dv"], "conv": 4}})
        else:
            layers.append({"type": "attention", "mlp": mlp,
                           "mixer": {"heads": s["aH"], "kv_heads": s["aG"], "dim": s["ad"], "vdim": s["adv"], "diff": 0.25,
                                     "scale": s["ad"] ** -0.5, "softcap": 40.0, "mask": {"size": s["window"]},
                                     "rot": {"base": 5e5, "dims": s["ad"],
                                             "scaling": {"factor": 4.0, "low": 1.0, "high": 2.0, "original": 4096}}}})
    return {"architecture": "Golitar", "vocab": s["vocab"], "width": s["width"], "streams": 2, "norm": {"eps": 1e-5},
            "logit_softcap": 30.0, "layers": layers}


def babodra_config(size: str, max_positions: int = 8192) -> dict:
    """Same width and depth as golitar_config(size); a dense layer has the same feed-forward size and a mixture layer the
    same ACTIVE size (top x expert ff + shared ff)."""
    s = SIZES[size]
    b = s["bab"]
    mixer = {"heads": b["heads"], "kv_heads": b["kv_heads"], "dim": b["dim"], "vdim": b["dim"], "scale": b["dim"] ** -0.5,
             "q_temp": {"coef": 0.1, "every": 1024}}
    moe = {"kind": "moe", "expert": {"ff": b["expert_ff"]}, "shared": {"ff": b["shared_ff"]},
           "router": {"experts": b["experts"], "top": b["top"], "scale": 2.5,
                      "groups": {"count": b["groups"][0], "keep": b["groups"][1]}}}
    dense = {"kind": "dense", "ff": s["ff"], "limit": 7.0}
    layers = [{"type": "attention", "mixer": dict(mixer), "mlp": dict(dense if ch == "d" else moe)} for ch in b["pattern"]]
    return {"architecture": "Babodra", "vocab": s["vocab"], "width": s["width"], "max_positions": max_positions,
            "norm": {"eps": 1e-5}, "layers": layers}


def maginex_config(size: str) -> dict:
    """Same width and depth as the other two; every layer carries a mixture with the ACTIVE size of babodra_config's
    (top x expert ff + shared ff); mixers alternate attention / latent attention / minGRU."""
    s = SIZES[size]
    m = s["mag"]
    moe = {"kind": "moe", "expert": {"ff": m["expert_ff"]}, "shared": {"ff": m["shared_ff"]},
           "router": {"experts": m["experts"], "top": m["top"]}}
    mixers = {"a": ("attention", {"heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
                                  "scale": m["dim"] ** -0.5, "mask": {"size": m["window"]}, "v_mix": True,
                                  "rot": {"base": 1e6, "dims": m["rot_dims"]}}),
              "l": ("latent_attention", {"heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "q_rank": m["q_rank"],
                                         "kv_rank": m["kv_rank"], "scale": m["dim"] ** -0.5}),
              "m": ("mingru", {"width": m["gru"]})}
    layers = [{"type": mixers[ch][0], "mixer": dict(mixers[ch][1]), "mlp": dict(moe)} for ch in m["pattern"]]
    return {"architecture": "Maginex", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5},
            "embedding": {"scale": 8.0}, "canon": {"taps": m["taps"]}, "layers": layers}


def zelinex_config(size: str) -> dict:
    """Same width as the others and the same number of layer RUNS (part of the stack is looped twice); generalized-delta
    layers carry the dense feed-forward of golitar_config, the parallel (windowed sigmoid attention + state-space) layers a
    mixture with the ACTIVE size of babodra_config's."""
    s = SIZES[size]
    z = s["zel"]
    moe = {"kind": "moe", "expert": {"ff": z["expert_ff"]}, "shared": {"ff": z["shared_ff"]},
           "router": {"experts": z["experts"], "top": z["top"], "scale": 2.0}}
    par = {"left": {"heads": z["heads"], "kv_heads": z["kv_heads"], "dim": z["dim"], "vdim": z["vdim"],
                    "scale": z["dim"] ** -0.5, "mask": {"size": z["window"]}, "rot": {"base": 1e6, "dims": z["rot_dims"]}},
           "right": {"heads": z["s_heads"], "vdim": z["s_vdim"], "state": z["state"], "groups": z["groups"], "conv": z["conv"],
                     "norm_groups": z["norm_groups"]}, "left_scale": 1.0, "right_scale": 1.0}
    layers = []
    for ch in z["pattern"]:
        if ch == "g":
            layers.append({"type": "general_delta", "mixer": {"heads": z["d_heads"], "dim": z["d_dim"]},
                           "mlp": {"kind": "dense", "ff": s["ff"]}})
        else:
            layers.append({"type": "parallel", "mixer": dict(par), "mlp": dict(moe)})
    a, b, t = z["loop"]
    return {"architecture": "Zelinex", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-5}, "residual_mult": 0.5,
            "loop": {"start": a, "stop": b, "times": t}, "layers": layers}


def _peaks(root):
    try:
        with open(os.path.join(root, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), float(p["bf16_tflops"]), "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


class _Timed:
    """Wraps the library so that every call is bracketed by CUDA events; cost(name, args) gives (bytes, flops)."""

    def __init__(self, lib):
        self._lib, self.log, self.on = lib, [], False

    def __getattr__(self, name):
        fn = getattr(self._lib, name)
        if not name.startswith("pieh_") or name in ("pieh_launch_count", "pieh_pipeline_error"):
            return fn

        def call(*args):
            if not self.on:
                return fn(*args)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            r = fn(*args)
            e1.record()
            self.log.append((name, args, e0, e1))
            return r
        return call


def _cost(name, a, model, batch_info):
    """Algorithmic (bytes, flops, label) of one call from its arguments."""
    act = 2 if model.act == 0 else 4
    T, n_seq, ctx = batch_info
    if name in ("pieh_linear", "pieh_linear_act"):
        M, N, K, epi = a[9], a[10], a[11], a[12] if name == "pieh_linear" else 0
        ob = 4 if a[1] == 1 else 2
        wb = 4 if a[7] == 1 else 2
        extra = 2 * model.S * M * N * 4 if epi == 3 else M * N * ob
        return N * K * wb + M * K * act + extra, 2.0 * M * N * K, f"linear M={M}"
    if name == "pieh_linear_glu":
        M, N, K = a[8], a[9], a[10]
        ob = 4 if a[1] == 1 else 2
        wb = 4 if a[7] == 1 else 2
        return N * K * wb + M * K * act + M * (N // 2) * ob, 2.0 * M * N * K, f"linear_glu M={M}"
    if name == "pieh_moe_linear":
        P, N, K, glu, E = a[9], a[10], a[11], a[13], a[17]._obj.E
        ob = 4 if a[1] == 1 else 2
        wb = 4 if a[7] == 1 else 2
        return min(E, P) * N * K * wb + P * K * act + P * (N // 2 if glu else N) * ob, 2.0 * P * N * K, f"moe_linear P={P}"
    if name == "pieh_linear_batched":
        nb, M, N, K = a[11], a[12], a[13], a[14]
        ob = 4 if a[1] == 1 else 2
        wb = 4 if a[9] == 1 else 2
        return nb * (N * K * wb + M * K * act + M * N * ob), 2.0 * nb * M * N * K, f"linear_batched M={M} N={N} K={K}"
    if name == "pieh_embed_scaled":
        return a[5] * a[6] * (act + 4), 0.0, "embed"
    if name == "pieh_residual_norm":
        Tn, W, mix = a[6], a[7], a[2]
        parts = mix._obj.top if mix is not None else 0
        return Tn * W * 4 * (parts + 2 + (1 if a[3] is not None else 0)), 0.0, "residual_norm" + ("(mixture)" if parts else "")
    if name == "pieh_sandwich_add":
        Tn, W, mix = a[11], a[12], a[2]
        parts = (mix._obj.top + 1) if mix is not None else (1 if a[1] is not None else 0)
        adds = (1 if a[5] is not None else 0)
        return (Tn * W * (4 * (parts + adds + 2) + (act if a[7] is not None else 0)), 0.0,
                "sandwich_add" + ("(mixture)" if mix is not None else ""))
    if name == "pieh_gated_group_norm":
        return a[12] * a[7] * a[8] * (8 + act), 0.0, "gated_group_norm"
    if name == "pieh_gdelta_prepare":
        d = a[7]._obj
        return a[8] * d.H * d.dk * 4 * 6, 0.0, "gdelta_prepare"
    if name == "pieh_gdelta_scan":
        d = a[6]._obj
        return (n_seq * 2 * d.H * d.dk * d.dv * 4 + T * d.H * (5 * d.dk + 2 * d.dv) * 4, 8.0 * T * d.H * d.dk * d.dv,
                "gdelta_scan")
    if name in ("pieh_ssd_prepare", "pieh_ssd_scan"):
        sd = a[4]._obj if name == "pieh_ssd_prepare" else a[3]._obj
        Cn = sd.H * sd.P + 2 * sd.G * sd.N
        if name == "pieh_ssd_prepare":
            return T * (2 * Cn + 3 * sd.H) * 4, 2.0 * T * Cn * sd.taps, "ssd_prepare"
        return (n_seq * 2 * sd.H * sd.N * sd.P * 4 + T * (Cn + sd.H * sd.P + 2 * sd.H) * 4, 5.0 * T * sd.H * sd.N * sd.P,
                "ssd_scan")
    if name == "pieh_canon_conv":
        cn = a[0]._obj
        return T * a[3] * (4 + cn.n_out * act), 2.0 * T * a[3] * cn.n_out * cn.taps, "canon_conv"
    if name == "pieh_mingru_scan":
        return T * a[4] * (12 + act), 0.0, "mingru_scan"      # the projection once, the output once
    if name == "pieh_latent_prepare":
        return T * (a[4] + a[6]) * (4 + act), 0.0, "latent_prepare"
    if name == "pieh_rot_table":
        return a[3] * a[4] * 8, 0.0, "rot_table"
    if name == "pieh_moe_route":
        pl = a[2]._obj
        return a[3] * (pl.E * 4 + pl.top * 16 * 2), 0.0, "moe_route"
    if name == "pieh_embed_positions":
        return a[8] * a[9] * (2 * act + 4 + act), 0.0, "embed"
    if name == "pieh_postnorm_add":
        Tn, W, mix = a[7], a[8], a[4]
        parts = (mix._obj.top + 1) if mix is not None else 1
        return Tn * W * (4 * parts + 8 + act), 0.0, "postnorm_add" + ("(mixture)" if mix is not None else "")
    if name.startswith("pieh_bias_attn"):
        at = a[-3]._obj
        H, G, d, dv = at.H, at.G, at.d, at.dv
        if name == "pieh_bias_attn_prepare":
            return T * ((H * d + G * d + G * dv + H * d) * 4 + G * (d + dv) * act), 0.0, "attn_prepare"
        own = T // max(n_seq, 1)
        keys = ctx + own
        per_q = ctx + (own + 1) / 2 if T > n_seq else keys
        if at.window:       # a query sees at most `window` keys; the step reads the pages its first row's window reaches
            per_q = min(per_q, at.window)
            keys = min(keys, at.window + own)
        shared_kv = 1 if at.k_pages == at.v_pages else 2      # latent attention: keys and values are one pool
        kvb = n_seq * keys * G * (d + dv) * act // (2 if shared_kv == 1 else 1)
        return (kvb + T * H * (d * 4 + dv * (act + 4)), 2.0 * T * H * per_q * (d + dv),
                "attn_run" + (f"(window {at.window})" if at.window else "") + ("(latent)" if shared_kv == 1 else ""))
    if name in ("pieh_stream_norm",):
        R, S, W = a[8], a[9], a[10]
        return R * S * W * 4 + R * W * act, 0.0, "stream_norm"
    if name == "pieh_embed_streams":
        return a[4] * a[5] * a[6] * 4, 0.0, "embed"
    if name.startswith("pieh_delta"):
        d = a[-3]._obj if name != "pieh_delta_gate" else a[6]._obj
        H, G, dk, dv = d.H, d.G, d.dk, d.dv
        C = 2 * G * dk + H * dv
        if name == "pieh_delta_prepare":
            return T * (C * 2 + 2 * H) * 4, 2.0 * T * C * d.taps, "delta_prepare"
        if name == "pieh_delta_scan":
            return n_seq * 2 * H * dk * dv * 4 + T * (2 * G * dk + 2 * H * dv + 2 * H) * 4, 6.0 * T * H * dk * dv, "delta_scan"
        return T * H * dv * (8 + act), 0.0, "delta_gate"
    at = a[-3]._obj
    H, G, d, dv = at.H, at.G, at.d, at.dv
    if name == "pieh_attn_prepare":
        return T * ((H + G) * 2 * d * 4 + G * dv * 4 + H * 2 * d * 4 + G * (2 * d + dv) * act), 0.0, "attn_prepare"
    keys = min(at.window or (ctx + T), ctx + T)
    per_q = min(keys, ctx + (T // max(n_seq, 1) + 1) / 2) if T > n_seq else keys
    kv_bytes = n_seq * min(ctx + T // max(n_seq, 1), keys + T // max(n_seq, 1)) * G * (2 * d + dv) * act
    return kv_bytes + T * H * (2 * d * 4 + dv * act), 2.0 * T * H * per_q * (2 * d + 2 * dv), "attn_run"


def _table(timed, model, batch_info, hbm, tfl):
    agg = {}
    for name, args, e0, e1 in timed.log:
        ms = e0.elapsed_time(e1)
        by, fl, label = _cost(name, args, model, batch_info)
        r = agg.setdefault(label, {"calls": 0, "us": 0.0, "bytes": 0.0, "flops": 0.0})
        r["calls"] += 1; r["us"] += ms * 1e3; r["bytes"] += by; r["flops"] += fl
    for r in agg.values():
        roof_us = max(r["bytes"] / (hbm * 1e3), r["flops"] / (tfl * 1e6))
        r["bound"] = "memory" if r["bytes"] / (hbm * 1e3) >= r["flops"] / (tfl * 1e6) else "tensor"
        r["frac"] = round(roof_us / r["us"], 4) if r["us"] else None
        r["us"] = round(r["us"], 1)
        r["gbytes"], r["gflops"] = round(r.pop("bytes") / 1e9, 4), round(r.pop("flops") / 1e9, 2)
    return agg


def run(size="1b", prompt=4096, portion=4096, batch=4, steps=32, warmup=3, root=".", with_llama=True,
        family="golitar") -> dict:
    """family "golitar": beside the quantized Llama path (with_llama); "babodra": beside Golitar at equal size."""
    from .engine import HybridEngine

    hbm, tfl, src = _peaks(root)
    t0 = time.time()
    if family == "zelinex":
        from .zelinex import ZelinexArgs, ZelinexModel, random_weights
        cfg = zelinex_config(size)
        args = ZelinexArgs.from_dict(cfg)
        weights = random_weights(args, seed=0, device="cuda")
        n_params = sum(v.numel() for v in weights.values())
        model = ZelinexModel(args, weights, "cuda", "bfloat16")
        del weights
        pattern = "".join(SIZES[size]["zel"]["pattern"][i] for i, _ in args.runs())
    elif family == "maginex":
        from .maginex import MaginexArgs, MaginexModel, random_weights
        cfg = maginex_config(size)
        args = MaginexArgs.from_dict(cfg)
        weights = random_weights(args, seed=0, device="cuda")
        n_params = sum(v.numel() for v in weights.values())
        model = MaginexModel(args, weights, "cuda", "bfloat16")
        del weights
        pattern = SIZES[size]["mag"]["pattern"]
    elif family == "babodra":
        from .babodra import BabodraArgs, BabodraModel, random_weights
        cfg = babodra_config(size, max_positions=prompt + steps + warmup + 64)
        args = BabodraArgs.from_dict(cfg)
        weights = random_weights(args, seed=0, device="cuda")
        n_params = sum(v.numel() for k, v in weights.items() if k != "pos")
        model = BabodraModel(args, weights, "cuda", "bfloat16")
        del weights
        pattern = SIZES[size]["bab"]["pattern"]
    else:
        from .golitar import GolitarArgs, GolitarModel, random_weights
        cfg = golitar_config(size)
        args = GolitarArgs.from_dict(cfg)
        model = GolitarModel(args, random_weights(args, seed=0, device="cuda"), "cuda", "bfloat16")
        n_params = sum(l.w.numel() for ly in model.layers for l in ly.values() if hasattr(l, "w")) + model.head.w.numel()
        pattern = SIZES[size]["pattern"]
    timed = _Timed(model.L)
    model.L = timed
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, args.vocab, (batch, prompt + steps + warmup + 1), generator=g).tolist()
    eng = HybridEngine(model, max_tokens=batch * (prompt + steps + warmup + 64), max_seqs=batch)
    ev = lambda: torch.cuda.Event(enable_timing=True)

    def prefill(sid, row):
        for at in range(0, prompt, portion):
            eng.forward([(sid, row[at:at + portion], None)])

    prefill("warm", ids[0]); eng.finish("warm")
    torch.cuda.synchronize()
    e0, e1 = ev(), ev()
    e0.record()
    for b in range(batch):
        prefill(b, ids[b])
    e1.record(); torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1) / batch
    pos = prompt
    for _ in range(warmup):
        eng.forward([(b, [ids[b][pos]], None) for b in range(batch)]); pos += 1
    torch.cuda.synchronize()
    e0, e1 = ev(), ev()
    e0.record()
    for _ in range(steps):
        eng.forward([(b, [ids[b][pos]], None) for b in range(batch)]); pos += 1
    e1.record(); torch.cuda.synchronize()
    decode_ms = e0.elapsed_time(e1) / steps
    # one decode step (launched directly, not replayed from the captured graph) and one prompt portion, every call timed
    eng.use_graph = False
    timed.on = True
    launches0 = int(timed._lib.pieh_launch_count())
    eng.forward([(b, [ids[b][pos]], None) for b in range(batch)])
    launches = int(timed._lib.pieh_launch_count()) - launches0      # kernels in the captured step
    torch.cuda.synchronize()
    dec_table = _table(timed, model, (batch, batch, pos), hbm, tfl)
    timed.log = []
    eng.finish(0)
    eng.forward([("p", ids[0][:portion], None)])
    torch.cuda.synchronize()
    pre_table = _table(timed, model, (portion, 1, 0), hbm, tfl)
    timed.on = False
    out = {"family": family, "size": size, "params": n_params, "layers": pattern, "dtype": "bf16",
           "data": "synthetic (random weights)", "peaks": {"hbm_gbs": hbm, "bf16_tflops": tfl, "source": src},
           "prefill": {"prompt": prompt, "portion": portion, "ms": round(prefill_ms, 2),
                       "tok_s": round(prompt / prefill_ms * 1e3, 1)},
           "decode": {"batch": batch, "context": prompt, "ms_per_step": round(decode_ms, 3),
                      "tok_s": round(batch / decode_ms * 1e3, 1), "launches_per_step": launches,
                      "cuda_graph": True},
           "kernels_prefill_portion": pre_table, "kernels_decode_step": dec_table,
           "pipeline_error": int(timed._lib.pieh_pipeline_error()), "setup_s": round(time.time() - t0, 1)}
    del eng, model
    torch.cuda.empty_cache()
    if family == "zelinex":
        if with_llama:      # the closest model of the framework (matrix-state recurrence + windowed attention) at the same sizes
            out["golitar_equal_size"] = run(size, prompt, portion, batch, steps, warmup, root, with_llama=False)
    elif family == "maginex":
        if with_llama:      # the closest model of the framework (sink attention + mixture of experts) at the same sizes
            out["babodra_equal_size"] = run(size, prompt, portion, batch, steps, warmup, root, with_llama=False,
                                            family="babodra")
    elif family == "babodra":
        if with_llama:      # the closest model of the framework at the same width, depth and active feed-forward size
            out["golitar_equal_size"] = run(size, prompt, portion, batch, steps, warmup, root, with_llama=False)
    elif with_llama:
        out["llama_equal_size"] = _llama(size, prompt, batch, steps, warmup)
    return out


def _llama(size, prompt, batch, steps, warmup) -> dict:
    """The quantized Llama path (q4, gs64) at the same width, feed-forward size and depth: whole-prompt prefill through
    Model.__call__ and graph-replayed decode through DecodeEngine."""
    from .checkpoint import build_model, random_weights
    from .decode import DecodeEngine
    from .llama import ModelArgs

    s = SIZES[size]
    margs = ModelArgs(num_hidden_layers=len(s["pattern"]), rms_norm_eps=1e-5, rope_theta=500000.0,
                      max_position_embeddings=131072, tie_word_embeddings=False,
                      rope_scaling={"factor": 8.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0},
                      quantization={"group_size": 64, "bits": 4}, **s["llama"])
    model = build_model(margs, random_weights(margs, seed=0, device="cuda"))
    eng = DecodeEngine(model, batch=batch, max_context=prompt + steps + warmup + 64)
    ids = torch.randint(0, margs.vocab_size, (batch, prompt), generator=torch.Generator().manual_seed(1))
    ev = lambda: torch.cuda.Event(enable_timing=True)
    eng.prefill(ids)
    torch.cuda.synchronize()
    e0, e1 = ev(), ev()
    e0.record(); eng.prefill(ids); e1.record(); torch.cuda.synchronize()
    prefill_ms = e0.elapsed_time(e1) / batch
    eng.step(max(warmup, 3))
    torch.cuda.synchronize()
    e0, e1 = ev(), ev()
    e0.record(); eng.step(steps); e1.record(); torch.cuda.synchronize()
    decode_ms = e0.elapsed_time(e1) / steps
    return {"model": "llama q4 gs64, same width / ff / depth", "prefill": {"prompt": prompt, "ms": round(prefill_ms, 2),
                                                                          "tok_s": round(prompt / prefill_ms * 1e3, 1)},
            "decode": {"batch": batch, "ms_per_step": round(decode_ms, 3), "tok_s": round(batch / decode_ms * 1e3, 1),
                       "launches_per_step": eng.launches_per_step}}
