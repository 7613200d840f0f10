"""Plain, slow restatement of the Maginex design, one function per mechanism, in float64 on the CPU.  It takes a whole
sequence at once (no cache, no batching) and shares no code with the package: the tests compare the engine's steps
(portions, decoding, mixed batches) against it."""
from __future__ import annotations

import math

import torch

F = torch.float64


def rms_norm(x, w, eps):
    """x [.., n] / sqrt(mean(x^2) + eps) * w"""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def canon(h, w):
    """h [L, W] -> h + causal per-channel convolution; w [W, taps], the last tap multiplies the current token."""
    L, taps = h.shape[0], w.shape[1]
    out = h.clone()
    for t in range(L):
        for j in range(taps):
            s = t - taps + 1 + j
            if s >= 0:
                out[t] += w[:, j] * h[s]
    return out


def rotate_half(x, positions, dims, base):
    """x [L, heads, d]: feature i < dims/2 pairs with i + dims/2; the features from `dims` on pass through."""
    half = dims // 2
    out = x.clone()
    for i in range(half):
        f = base ** (-2.0 * i / dims)
        ang = positions.to(F) * f
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        u, v = x[:, :, i], x[:, :, i + half]
        out[:, :, i] = u * c - v * s
        out[:, :, i + half] = v * c + u * s
    return out


def sink_attention(q, k, v, scale, window, sink):
    """q [L, H, d], k [L, G, d], v [L, G, dv], sink [H] (logits of a key-less, value-less term).  window 0: all earlier
    tokens.  -> [L, H, dv]"""
    L, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((L, H, v.shape[2]), dtype=F)
    for h in range(H):
        g = h // (H // G)
        for i in range(L):
            lo = max(0, i - window + 1) if window else 0
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = max(float(s.max()), float(sink[h]))
            e = torch.exp(s - m)
            den = e.sum() + math.exp(float(sink[h]) - m)
            out[i, h] = (e[:, None] * v[lo:i + 1, g]).sum(0) / den
    return out


def attention_mixer(h, w, p, m, v_first):
    """-> (output [L, W], this layer's (mixed) values [L, G, dv]).  v_first: the first value-mixing layer's values or None."""
    L = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(L, H, d)
    k = (h @ w[p + "k"].T).view(L, G, d)
    v = (h @ w[p + "v"].T).view(L, G, dv)
    rot = m.get("rot")
    if rot:
        pos = torch.arange(L)
        q, k = rotate_half(q, pos, rot["dims"], rot["base"]), rotate_half(k, pos, rot["dims"], rot["base"])
    if m.get("v_mix") and v_first is not None:
        lam = w[p + "vmix"]
        v = (1 - lam) * v + lam * v_first
    o = sink_attention(q, k, v, m["scale"], int((m.get("mask") or {}).get("size") or 0), w[p + "sink"])
    gate = torch.sigmoid(h @ w[p + "g"].T)                    # [L, H]
    o = o * gate[:, :, None]
    return o.reshape(L, H * dv) @ w[p + "o"].T, v


def latent_attention_mixer(h, w, p, m, eps):
    L = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(L, H, d)
    c = rms_norm(h @ w[p + "dkv"].T, w[p + "dkv.norm"], eps)
    k = (c @ w[p + "uk"].T).view(L, H, d)
    v = (c @ w[p + "uv"].T).view(L, H, dv)
    o = sink_attention(q, k, v, m["scale"], 0, w[p + "sink"]).reshape(L, H * dv)
    o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def mingru_mixer(h, w, p):
    z = torch.sigmoid(h @ w[p + "z"].T + w[p + "z.b"])
    u = h @ w[p + "x"].T + w[p + "x.b"]
    cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
    S = torch.zeros(z.shape[1], dtype=F)
    states = []
    for t in range(h.shape[0]):
        S = (1 - z[t]) * S + z[t] * cand[t]
        states.append(S)
    S = torch.stack(states)
    gate = h @ w[p + "g"].T
    return (S * gate * torch.sigmoid(gate)) @ w[p + "o"].T


def expert(h, w, p):
    a = torch.relu(h @ w[p + "up"].T)
    return (a * a) @ w[p + "down"].T


def moe(h, w, p, mlp, margins=None):
    """margins: list that receives, per token, the gap between the last chosen logit and the best one left out (how close
    the choice was; infinite when every expert is chosen)."""
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ w[p + "router"].T + w[p + "router.b"]
    out = torch.zeros_like(h)
    if margins is not None:
        zs = torch.sort(z, dim=-1, descending=True).values
        margins.append(zs[:, top - 1] - zs[:, top] if top < E else torch.full((h.shape[0],), float("inf"), dtype=F))
    for t in range(h.shape[0]):
        val, idx = torch.sort(z[t], descending=True, stable=True)
        wts = torch.softmax(val[:top], 0)
        for k in range(top):
            out[t] += wts[k] * expert(h[t], w, f"{p}e{int(idx[k])}.")
    if mlp.get("shared"):
        out = out + expert(h, w, p + "shared.")
    return out


def forward(cfg, weights, tokens, trace=None, margins=None):
    """tokens: list of ids -> logits [L, vocab] (float64).  trace: list that receives the residual after every layer;
    margins: list that receives every routed layer's per-token routing margin."""
    w = {k: v.to(F) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    v_first = None
    for i, ly in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = rms_norm(x, w[p + "norm1"], eps)
        hm = canon(h, w[p + "canon1"])
        m = ly["mixer"]
        if ly["type"] == "attention":
            y, v = attention_mixer(hm, w, p + "mix.", m, v_first)
            if m.get("v_mix") and v_first is None:
                v_first = v
        elif ly["type"] == "latent_attention":
            y = latent_attention_mixer(hm, w, p + "mix.", m, eps)
        elif ly["type"] == "mingru":
            y = mingru_mixer(hm, w, p + "mix.")
        else:
            raise ValueError(ly["type"])
        if ly.get("mlp"):
            y = y + moe(canon(h, w[p + "canon2"]), w, p + "mlp.", ly["mlp"], margins)
        x = x + y
        if trace is not None:
            trace.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def random_config(vocab=96, width=64, pattern="alm", heads=4, kv_heads=2, dim=16, vdim=24, window=6, rot_dims=8, q_rank=24,
                  kv_rank=32, gru=40, experts=6, top=2, ff=40, shared_ff=24, taps=3, scale=4.0, mlp=True, v_mix=True):
    """A small configuration; pattern: one letter per layer, a = attention, l = latent attention, m = minGRU."""
    layers = []
    for ch in pattern:
        if ch == "a":
            mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": dim ** -0.5, "v_mix": v_mix}
            if window:
                mixer["mask"] = {"size": window}
            if rot_dims:
                mixer["rot"] = {"base": 1e4, "dims": rot_dims}
            layers.append({"type": "attention", "mixer": mixer})
        elif ch == "l":
            layers.append({"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "q_rank": q_rank,
                                                                "kv_rank": kv_rank, "scale": dim ** -0.5}})
        else:
            layers.append({"type": "mingru", "mixer": {"width": gru}})
        layers[-1]["mlp"] = ({"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top},
                              "shared": {"ff": shared_ff} if shared_ff else None} if mlp else None)
    return {"architecture": "Maginex", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "embedding": {"scale": scale},
            "canon": {"taps": taps}, "layers": layers}
