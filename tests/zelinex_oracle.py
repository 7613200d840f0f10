"""Plain, slow restatement of the Zelinex design, one function per mechanism, in float64 on the CPU.  It takes a whole
sequence at once (no cache, no batching, token-by-token loops) and shares no code with the package: the tests compare the
engine's steps (portions, decoding, mixed batches) against it."""
from __future__ import annotations

import math

import torch

F = torch.float64


def unit_rms(x, eps):
    """x [.., n] / sqrt(mean(x^2) + eps)"""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def softplus(x):
    return torch.logaddexp(x, torch.zeros_like(x))


def silu(x):
    return x * torch.sigmoid(x)


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (e^z - 1 - z) + z/2"""
    ap, aq = softplus(p), 0.5 + softplus(q)
    return torch.where(z > 0, ap * z * z + 0.5 * z, aq * (torch.exp(torch.clamp(z, max=0.0)) - 1 - z) + 0.5 * z)


def rotate_half(x, positions, dims, base):
    """x [L, heads, d]: feature i < dims/2 pairs with i + dims/2 and turns by position * base^(-2i/dims); features from
    `dims` on pass through."""
    half = dims // 2
    out = x.clone()
    for i in range(half):
        ang = positions.to(F) * (base ** (-2.0 * i / dims))
        c, s = torch.cos(ang)[:, None], torch.sin(ang)[:, None]
        u, v = x[:, :, i], x[:, :, i + half]
        out[:, :, i] = u * c - v * s
        out[:, :, i + half] = v * c + u * s
    return out


def sigmoid_window_attention(q, k, v, scale, window, bias):
    """q [L, H, d], k [L, G, d], v [L, G, dv], bias [H].  Key j counts for query i when 0 <= i - j < window, with the
    weight sigmoid(q_i . k_j scale + bias_h); the weights are not normalised.  -> [L, H, dv]"""
    L, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((L, H, v.shape[2]), dtype=F)
    for h in range(H):
        g = h // (H // G)
        for i in range(L):
            lo = max(0, i - window + 1)
            p = torch.sigmoid((k[lo:i + 1, g] @ q[i, h]) * scale + bias[h])
            out[i, h] = (p[:, None] * v[lo:i + 1, g]).sum(0)
    return out


def attention_branch(h, w, p, m):
    L = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(L, H, d)
    k = (h @ w[p + "k"].T).view(L, G, d)
    v = (h @ w[p + "v"].T).view(L, G, dv)
    rot = m.get("rot")
    if rot and rot["dims"]:
        pos = torch.arange(L)
        q, k = rotate_half(q, pos, rot["dims"], rot["base"]), rotate_half(k, pos, rot["dims"], rot["base"])
    window = (m.get("mask") or {}).get("size") or L          # no mask: every earlier token
    o = sigmoid_window_attention(q, k, v, m["scale"], window, w[p + "pb"])
    return o.reshape(L, H * dv) @ w[p + "o"].T


def causal_conv_silu(x, w, b):
    """x [L, C], w [C, taps] (last column: the current token), b [C]; zeros before the start."""
    L, taps = x.shape[0], w.shape[1]
    out = torch.zeros_like(x)
    for t in range(L):
        acc = b.clone()
        for j in range(taps):
            s = t - (taps - 1) + j
            if s >= 0:
                acc = acc + w[:, j] * x[s]
        out[t] = silu(acc)
    return out


def ssd_scan(x, B, Cm, dt, A_log, D):
    """x [L, H, P], B / Cm [L, G, N], dt [L, H] (after softplus).  S_t = exp(-exp(A_log) dt) S + dt B x^T  (S [N, P]);
    y_t = S_t^T C + D x."""
    L, H, P = x.shape
    G, N = B.shape[1], B.shape[2]
    y = torch.zeros_like(x)
    for h in range(H):
        g = h // (H // G)
        S = torch.zeros((N, P), dtype=F)
        for t in range(L):
            S = torch.exp(-torch.exp(A_log[h]) * dt[t, h]) * S + dt[t, h] * torch.outer(B[t, g], x[t, h])
            y[t, h] = S.T @ Cm[t, g] + D[h] * x[t, h]
    return y


def ssd_branch(h, w, p, m, eps):
    L = h.shape[0]
    H, P, N, G, ng = m["heads"], m["vdim"], m["state"], m["groups"], m["norm_groups"]
    inner = H * P
    u = h @ w[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = causal_conv_silu(xbc, w[p + "conv"], w[p + "conv.b"])
    x = xbc[:, :inner].reshape(L, H, P)
    B = xbc[:, inner:inner + G * N].reshape(L, G, N)
    Cm = xbc[:, inner + G * N:].reshape(L, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    y = ssd_scan(x, B, Cm, dt, w[p + "A_log"], w[p + "D"]).reshape(L, inner)
    y = y * silu(z)
    y = unit_rms(y.view(L, ng, inner // ng), eps).reshape(L, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps):
    return (m["left_scale"] * attention_branch(h, w, p + "left.", m["left"])
            + m["right_scale"] * ssd_branch(h, w, p + "right.", m["right"], eps))


def delta_scan(r, k, v, decay, a):
    """r, k, v, decay, a [L, H, n].  u = k / sqrt(|k|^2 + 1e-6);
    S_t = diag(decay_t) S - (a_t u_t)(u_t^T S) + k_t v_t^T  (both corrections read the old S, S [n, n]);  o_t = S_t^T r_t."""
    L, H, n = r.shape
    o = torch.zeros_like(v)
    for h in range(H):
        S = torch.zeros((n, n), dtype=F)
        for t in range(L):
            u = k[t, h] / torch.sqrt((k[t, h] ** 2).sum() + 1e-6)
            S = decay[t, h][:, None] * S - torch.outer(a[t, h] * u, u @ S) + torch.outer(k[t, h], v[t, h])
            o[t, h] = S.T @ r[t, h]
    return o


def delta_mixer(h, w, p, m, eps):
    L = h.shape[0]
    H, n = m["heads"], m["dim"]
    r, k, v = [(h @ w[p + s].T).view(L, H, n) for s in ("r", "k", "v")]
    lora = torch.tanh(h @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(lora)).view(L, H, n)
    a = torch.sigmoid(h @ w[p + "a"].T + w[p + "a.b"]).view(L, H, n)
    o = unit_rms(delta_scan(r, k, v, decay, a), eps).reshape(L, H * n)
    o = o * w[p + "norm"] * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def glu_expert(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def moe(h, w, p, mlp, margins=None):
    """margins: if a list, the gap between the last chosen and the first rejected score of every token is appended."""
    E, top, scale = mlp["router"]["experts"], mlp["router"]["top"], mlp["router"]["scale"]
    s = torch.softmax(h @ w[p + "router"].T, -1)
    out = torch.zeros((h.shape[0], w[p + "e0.down"].shape[0]), dtype=F)
    for t in range(h.shape[0]):
        order = torch.argsort(s[t], descending=True, stable=True)
        pick = order[:top]
        if margins is not None and top < E:
            margins.append(float(s[t, order[top - 1]] - s[t, order[top]]))
        wt = s[t, pick] / (s[t, pick].sum() + 1e-20) * scale
        for e, c in zip(pick.tolist(), wt):
            out[t] += c * glu_expert(h[t], w, f"{p}e{e}.")
    if mlp.get("shared"):
        out = out + glu_expert(h, w, p + "shared.")
    return out


def dense_ff(h, w, p):
    return xielu(h @ w[p + "up"].T, w[p + "act"][0], w[p + "act"][1]) @ w[p + "down"].T


def layer_runs(cfg):
    """[(layer index, pass number or None, first of its pass)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or None
    if not loop:
        return [(i, None, False) for i in range(n)], 1
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    runs = [(i, None, False) for i in range(a)]
    for t in range(times):
        runs += [(i, t, i == a) for i in range(a, b)]
    runs += [(i, None, False) for i in range(b, n)]
    return runs, times


def forward(cfg, weights, tokens, trace=None, margins=None):
    """tokens: list of ids of ONE sequence from its start -> logits [L, vocab] (float64).  trace: if a list, the residual
    after every layer run is appended."""
    w = {k: v.to(F) for k, v in weights.items()}
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x0 = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    x = x0.clone()
    loop = cfg.get("loop") or None
    runs, _ = layer_runs(cfg)
    for i, t, first in runs:
        ly = cfg["layers"][i]
        p = f"l{i}."
        if loop and first:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t]
        h = unit_rms(x, eps) * w[p + "norm1"]
        if ly["type"] == "parallel":
            y = parallel_mixer(h, w, p + "mix.", ly["mixer"], eps)
        elif ly["type"] == "general_delta":
            y = delta_mixer(h, w, p + "mix.", ly["mixer"], eps)
        else:
            raise ValueError(ly["type"])
        x = x + mult * unit_rms(y, eps) * w[p + "norm1b"]
        mlp = ly.get("mlp")
        if mlp:
            h = unit_rms(x, eps) * w[p + "norm2"]
            y = dense_ff(h, w, p + "mlp.") if mlp["kind"] == "dense" else moe(h, w, p + "mlp.", mlp, margins)
            x = x + mult * unit_rms(y, eps) * w[p + "norm2b"]
        if trace is not None:
            trace.append(x.clone())
    return (unit_rms(x, eps) * w["final.norm"]) @ w["embed"].T


def random_config(vocab=96, width=64, pattern="gp", ffs="dm", heads=4, kv_heads=2, dim=16, vdim=24, window=6, rot_dims=8,
                  rot_base=10000.0, scale=None, s_heads=4, s_vdim=8, state=12, groups=2, conv=3, norm_groups=2, d_heads=2,
                  d_dim=16, ff=48, experts=6, top=2, expert_ff=24, shared_ff=16, router_scale=1.5, left_scale=1.1,
                  right_scale=0.8, mult=0.7, eps=1e-5, loop=(0, 1, 2)):
    """A small configuration: pattern 'g' = general_delta, 'p' = parallel; ffs per layer 'd' dense, 'm' experts, '-' none
    (the last letter repeats); loop (start, stop, times) or None."""
    layers = []
    for i, c in enumerate(pattern):
        if c == "g":
            mixer = {"heads": d_heads, "dim": d_dim}
        else:
            left = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
                    "scale": scale if scale is not None else dim ** -0.5, "mask": {"size": window}}
            if rot_dims:
                left["rot"] = {"base": rot_base, "dims": rot_dims}
            mixer = {"left": left, "left_scale": left_scale, "right_scale": right_scale,
                     "right": {"heads": s_heads, "vdim": s_vdim, "state": state, "groups": groups, "conv": conv,
                               "norm_groups": norm_groups}}
        f = ffs[min(i, len(ffs) - 1)]
        mlp = None
        if f == "d":
            mlp = {"kind": "dense", "ff": ff}
        elif f == "m":
            mlp = {"kind": "moe", "expert": {"ff": expert_ff}, "router": {"experts": experts, "top": top, "scale": router_scale},
                   "shared": {"ff": shared_ff} if shared_ff else None}
        layers.append({"type": "general_delta" if c == "g" else "parallel", "mixer": mixer, "mlp": mlp})
    cfg = {"architecture": "Zelinex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "residual_mult": mult,
           "layers": layers}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": min(loop[1], len(layers)), "times": loop[2]}
    return cfg
