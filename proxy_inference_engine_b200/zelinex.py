"""Zelinex: a decoder-only model of sandwich-norm blocks -- every sublayer has a norm before it and one on its output, and
the output joins the residual times a constant -- with tied input / output embeddings and an optional LOOP: a run of
layers is applied several times with the same weights (each pass with a cache and state of its own), the embedding being
added back and a learned per-pass vector added in front of every pass.  A layer's mixer is one of
    parallel        two mixers read the same input and their outputs are summed with fixed weights: sliding-window attention
                    whose weights are sigmoids (score + a bias per head; no softmax, no normalisation over the keys; grouped
                    heads, rotation of the leading features) beside a selective state-space layer in its scalar-decay form
                    (short causal convolution, matrix state per head, gate, grouped output norm)
    general_delta   the generalized delta rule: a matrix state per head with a decay per key channel (from a low-rank
                    tanh bottleneck) and a removal term along the unit key; per-head output norm, sigmoid gate
and its feed-forward is dense (xIELU activation: quadratic above zero, exponential below, two learned numbers) or a mixture
of silu-gated experts (softmax scores, the largest few renormalised and scaled) plus an always-on shared expert.
Served through the ragged step of libpie_b200_hybrid.so like the other hybrid families: same ``BatchDetails``, same
``cache.HybridCache`` (pages and state slots; one entry per layer RUN, so a looped layer holds one per pass), same
``engine.HybridEngine``.

config.json: ``architecture`` "Zelinex"; ``vocab``, ``width``, ``norm.eps``, ``residual_mult``, ``loop`` {start, stop,
times} | absent, and ``layers``, a list of ``{"type": "parallel" | "general_delta", "mixer": {...}, "mlp": {...} | null}``:
    parallel:       left {heads, kv_heads, dim, vdim, scale, mask.size, rot {base, dims}}, left_scale,
                    right {heads, vdim, state, groups, conv, norm_groups}, right_scale
    general_delta:  heads, dim
    mlp:            {"kind": "dense", "ff"}  or  {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "scale"},
                    "shared": {"ff"} | null}
Tensors: ``embed``, ``final.norm``, ``loop.step`` [times, width], per layer i ``l<i>.norm1|norm1b|norm2|norm2b``,
``l<i>.mix.left.q|k|v|pb|o``, ``l<i>.mix.right.in|conv|conv.b|dt_bias|A_log|D|norm|o`` (``in`` rows: gate z, x, B, C, dt),
``l<i>.mix.r|k|v|g|a|a.b|w1|w2|w0|norm|o``, ``l<i>.mlp.up|down|act`` or ``l<i>.mlp.router``, ``l<i>.mlp.e<j>.gate|up|down``,
``l<i>.mlp.shared.gate|up|down``.

One step over a ``ragged.BatchDetails`` (x: fp32 residual [T, W]; h: the next sublayer's normed input, act dtype):

    x      = embed(tokens)                                  (kept aside as x0 when a loop re-injects it)
    x, h   = sandwich_add(x; + pass vector; norm1 of the first run)
    per layer run:
      parallel:       p = linear(h; [q | k | v | z | x B C | dt] fused)
                      bias_attn_prepare (rotation, append to pages) -> bias_attn_run (window, sigmoid weights)
                      ssd_prepare (convolution + silu, dt, decay; history in the slot) -> ssd_scan (state in the slot)
                      -> gated_group_norm (silu(z) first, then the grouped norm)
                      y = left_scale * linear(attention; o_left) + right_scale * linear(state-space; o_right)
      general_delta:  p = linear(h; [r | k | v | g | a]);  decay logits = linear(linear(h; w1, tanh); w2, bias w0)
                      gdelta_prepare (decay, unit key, removal) -> gdelta_scan (state in the slot)
                      -> gated_group_norm (per-head norm, weight, sigmoid(g));  y = linear(.; o)
      x, h   = sandwich_add(x, y; norm1b, m; norm2)
      dense:  y = linear(linear_act(h; up, xIELU); down)
      moe:    z = linear(h; router) -> moe_route (softmax over the chosen = renormalised scores, times scale) -> two
              grouped products (silu pair between them) + the shared expert's two products; the sum is formed on the fly
      x, h   = sandwich_add(x, y | mixture; norm2b, m; + x0 + pass vector if the next run opens a pass; next run's norm1)
    logits = linear(stream_norm(x[wanted rows]; final norm); embed)                               fp32

dtype "bfloat16": matrix-product inputs and the key / value pages are bf16; accumulation, residual, norms, rotation angles,
attention scores and weights, routing, convolution, both recurrences and all their gates are fp32.  dtype "float32":
weights are widened once and every product is a plain fp32 multiply-add.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field

import torch

from . import _lib
from ._lib import (DTYPE_BF16, DTYPE_F32, EPI_NONE, EPI_STREAMS, EPI_TANH, EPI_XIELU, HybBiasAttn, HybGdelta, HybMixSum,
                   HybMoePlan, HybSsd)
from .babodra import interleave_pairs
from .cache import HybridCache
from .golitar import _Linear, _p, _stream
from .ragged import BatchDetails

MIXERS = ("parallel", "general_delta")
DECAY_SCALE = math.exp(-0.5)     # general_delta: decay = exp(-e^(-1/2) sigmoid(.)), so a channel keeps at least 54.5 % per token
KEY_EPS = 1e-6                   # general_delta: inside the root of the unit key's length


@dataclass
class ZelinexArgs:
    vocab: int
    width: int
    layers: list
    norm_eps: float = 1e-6
    residual_mult: float = 1.0
    loop: dict | None = None
    architecture: str = "Zelinex"
    raw: dict = field(default_factory=dict)

    @classmethod
    def from_dict(cls, cfg: dict) -> "ZelinexArgs":
        for key in ("vocab", "width", "layers"):
            if key not in cfg:
                raise ValueError(f"Zelinex config: '{key}' is missing")
        for i, ly in enumerate(cfg["layers"]):
            if ly.get("type") not in MIXERS:
                raise ValueError(f"Zelinex config: layer {i} has unknown type {ly.get('type')!r}")
            m = ly.get("mixer") or {}
            if ly["type"] == "general_delta":
                for key in ("heads", "dim"):
                    if key not in m:
                        raise ValueError(f"Zelinex config: layer {i} mixer lacks '{key}'")
            else:
                for side, keys in (("left", ("heads", "kv_heads", "dim", "vdim", "scale")),
                                   ("right", ("heads", "vdim", "state", "groups"))):
                    if side not in m:
                        raise ValueError(f"Zelinex config: layer {i} mixer lacks '{side}'")
                    for key in keys:
                        if key not in m[side]:
                            raise ValueError(f"Zelinex config: layer {i} mixer.{side} lacks '{key}'")
                le, ri = m["left"], m["right"]
                if int(le["heads"]) % int(le["kv_heads"]):
                    raise ValueError(f"Zelinex config: layer {i}: heads is not a multiple of kv_heads")
                rot = le.get("rot")
                if rot and (int(rot["dims"]) % 2 or int(rot["dims"]) > int(le["dim"])):
                    raise ValueError(f"Zelinex config: layer {i}: rot.dims must be even and at most dim")
                if int(ri["heads"]) % int(ri["groups"]):
                    raise ValueError(f"Zelinex config: layer {i}: right.heads is not a multiple of right.groups")
                if (int(ri["heads"]) * int(ri["vdim"])) % int(ri.get("norm_groups") or 1):
                    raise ValueError(f"Zelinex config: layer {i}: norm_groups does not divide heads * vdim")
                if not 1 <= int(ri.get("conv") or 1) <= 8:
                    raise ValueError(f"Zelinex config: layer {i}: right.conv must be between 1 and 8")
            mlp = ly.get("mlp")
            if mlp:
                if mlp.get("kind") not in ("dense", "moe"):
                    raise ValueError(f"Zelinex config: layer {i} has unknown feed-forward kind {mlp.get('kind')!r}")
                if mlp["kind"] == "moe" and int(mlp["router"]["top"]) > int(mlp["router"]["experts"]):
                    raise ValueError(f"Zelinex config: layer {i}: 'top' exceeds the number of experts")
        loop = cfg.get("loop") or None
        if loop:
            a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
            if not (0 <= a < b <= len(cfg["layers"])) or times < 1:
                raise ValueError("Zelinex config: loop needs 0 <= start < stop <= number of layers and times >= 1")
            loop = {"start": a, "stop": b, "times": times}
        return cls(vocab=int(cfg["vocab"]), width=int(cfg["width"]), layers=list(cfg["layers"]),
                   norm_eps=float((cfg.get("norm") or {}).get("eps", 1e-6)),
                   residual_mult=float(cfg.get("residual_mult", 1.0)), loop=loop,
                   architecture=cfg.get("architecture", "Zelinex"), raw=cfg)

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.norm_eps},
               "residual_mult": self.residual_mult, "layers": self.layers}
        if self.loop:
            out["loop"] = dict(self.loop)
        return out

    def runs(self) -> list:
        """The order the layers run in: [(layer index, number of the pass this run OPENS or None)]."""
        n = len(self.layers)
        if not self.loop:
            return [(i, None) for i in range(n)]
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        out = [(i, None) for i in range(a)]
        for t in range(times):
            out += [(i, t if i == a else None) for i in range(a, b)]
        return out + [(i, None) for i in range(b, n)]


def rotary_frequencies(rot: dict) -> list:
    """Angle per position of rotated pair i: base^(-2 i / dims)."""
    dims = int(rot["dims"])
    return [float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)]


def _softplus(v: float) -> float:
    return v if v > 30 else math.log1p(math.exp(v))


class ZelinexModel:
    def __init__(self, args: ZelinexArgs, weights: dict, device="cuda", dtype: str = "bfloat16"):
        if dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype must be 'bfloat16' or 'float32'")
        self.args, self.device, self.dtype = args, device, dtype
        self.exact = dtype == "float32"
        self.act_torch = torch.float32 if self.exact else torch.bfloat16
        self.act = DTYPE_F32 if self.exact else DTYPE_BF16
        self.L = _lib.load_hybrid(build_if_missing=True)
        self.W, W, self.S = args.width, args.width, 1        # one residual stream
        f32 = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        get = lambda name: weights[name]
        lin = lambda w, b=None: _Linear(w, b, self.exact, device)
        wdt = torch.float32 if self.exact else torch.bfloat16
        self.head = lin(get("embed"))            # tied: the table is both the embedding and the output matrix
        self.embed = self.head.w
        if tuple(self.embed.shape) != (args.vocab, W):
            raise ValueError(f"embed has shape {tuple(self.embed.shape)}, expected {(args.vocab, W)}")
        self.final_norm = f32(get("final.norm"))
        self.loop_step = None
        if args.loop:
            self.loop_step = f32(get("loop.step"))
            if tuple(self.loop_step.shape) != (args.loop["times"], W):
                raise ValueError(f"loop.step has shape {tuple(self.loop_step.shape)}, expected {(args.loop['times'], W)}")
        self.keep_x0 = bool(args.loop and args.loop["times"] > 1)
        self.layer_weights, self.rot_tables = [], {}
        for i, cfg in enumerate(args.layers):
            p, m, kind = f"l{i}.", cfg["mixer"], cfg["type"]
            mw = lambda n: get(p + "mix." + n)
            ly = {"type": kind, "norm1": f32(get(p + "norm1")), "norm1b": f32(get(p + "norm1b")), "mlp": None}
            if kind == "general_delta":
                H, n = int(m["heads"]), int(m["dim"])
                ly["dims"] = (H, n)
                ly["proj"] = lin(torch.cat([mw("r"), mw("k"), mw("v"), mw("g"), mw("a")], 0))
                ly["w1"], ly["w2"] = lin(mw("w1")), lin(mw("w2"), mw("w0"))
                ly["a_bias"], ly["out_norm"], ly["out"] = f32(mw("a.b")), f32(mw("norm")), lin(mw("o"))
                ly["cache"] = {"slots": {"state": (H, n, n)}}
            else:
                le, ri = m["left"], m["right"]
                H, G, d, dv = int(le["heads"]), int(le["kv_heads"]), int(le["dim"]), int(le["vdim"])
                Hs, P, N, Gs = int(ri["heads"]), int(ri["vdim"]), int(ri["state"]), int(ri["groups"])
                taps, ng = int(ri.get("conv") or 1), int(ri.get("norm_groups") or 1)
                inner, C_ = Hs * P, Hs * P + 2 * Gs * N
                lw, rw = (lambda n: mw("left." + n)), (lambda n: mw("right." + n))
                if tuple(rw("in").shape) != (2 * inner + 2 * Gs * N + Hs, W):
                    raise ValueError(f"{p}mix.right.in has shape {tuple(rw('in').shape)}, expected "
                                     f"{(2 * inner + 2 * Gs * N + Hs, W)}")
                conv = rw("conv") if taps > 1 or (p + "mix.right.conv") in weights else torch.ones((C_, 1))
                if tuple(conv.shape) != (C_, taps):
                    raise ValueError(f"{p}mix.right.conv has shape {tuple(conv.shape)}, expected {(C_, taps)}")
                ly["dims"] = (H, G, d, dv, Hs, P, N, Gs, taps, ng)
                ly["proj"] = lin(torch.cat([lw("q"), lw("k"), lw("v"), rw("in")], 0))     # one product for both mixers
                ly["pb"], ly["scale"] = f32(lw("pb")), float(le["scale"])
                ly["window"] = int((le.get("mask") or {}).get("size") or 0)
                rot = le.get("rot") or None
                ly["rot"] = None
                if rot and int(rot["dims"]) > 0:
                    key = (int(rot["dims"]), float(rot["base"]))
                    if key not in self.rot_tables:
                        self.rot_tables[key] = torch.tensor(rotary_frequencies(rot), dtype=torch.float64).to(device)
                    ly["rot"] = key
                ly["out_l"], ly["out_r"] = lin(lw("o")), lin(rw("o"))
                ly["conv_w"] = f32(conv)
                ly["conv_b"] = f32(rw("conv.b")) if (p + "mix.right.conv.b") in weights else None
                ly["dt_bias"], ly["A_log"], ly["D"] = f32(rw("dt_bias")), f32(rw("A_log")), f32(rw("D"))
                ly["out_norm"] = f32(rw("norm"))
                sc = lambda v: torch.tensor([float(v)], dtype=torch.float32, device=device)
                ly["sum"] = {"mix": sc(m.get("left_scale", 1.0)).view(1, 1), "out": sc(m.get("right_scale", 1.0))}
                slots = {"state": (Hs, N, P)}
                if taps > 1:
                    slots["conv"] = (taps - 1, C_)
                ly["cache"] = {"pages": {"k": (G, d), "v": (G, dv)}, "slots": slots}
            mlp = cfg.get("mlp")
            if mlp:
                q = p + "mlp."
                ly["norm2"], ly["norm2b"] = f32(get(p + "norm2")), f32(get(p + "norm2b"))
                if mlp["kind"] == "dense":
                    act = get(q + "act").double()
                    ly["mlp"] = {"kind": "dense", "up": lin(get(q + "up")), "down": lin(get(q + "down")),
                                 "coef": (_softplus(float(act[0])), 0.5 + _softplus(float(act[1])))}
                else:
                    r = mlp["router"]
                    E = int(r["experts"])
                    stack = lambda ts: torch.stack(ts, 0).to(device=device, dtype=wdt).contiguous()
                    ly["mlp"] = {"kind": "moe", "E": E, "top": int(r["top"]), "scale": float(r.get("scale", 1.0)),
                                 "router": lin(get(q + "router")),
                                 "gu": stack([interleave_pairs(get(f"{q}e{e}.gate"), get(f"{q}e{e}.up")) for e in range(E)]),
                                 "down": stack([get(f"{q}e{e}.down") for e in range(E)]),
                                 "counters": torch.zeros(2 * E + 2, dtype=torch.int32, device=device), "shared": None}
                    if mlp.get("shared"):
                        ly["mlp"]["shared"] = {"gu": lin(interleave_pairs(get(q + "shared.gate"), get(q + "shared.up"))),
                                               "down": lin(get(q + "shared.down"))}
            self.layer_weights.append(ly)
        # one entry per layer RUN: a looped layer appears once per pass, with the same weights and its own cache entry
        self.runs = args.runs()
        self.layers = [self.layer_weights[i] for i, _ in self.runs]
        self.cache_specs = [ly["cache"] for ly in self.layers]

    # ------------------------------------------------------------------------------------------------
    def make_cache(self, max_tokens: int, max_seqs: int = 4) -> HybridCache:
        return HybridCache(self.cache_specs, max_tokens, max_seqs, self.device, self.act_torch, lib=self.L)

    def _empty(self, shape, dtype=None):
        return torch.empty(shape, dtype=dtype or torch.float32, device=self.device)

    def _linear(self, lin: _Linear, x, M, out_dtype=None, act=EPI_NONE, coef=(0.0, 0.0), accumulate=None):
        """accumulate = (y, sum weights): y <- mix * y + out * product, in place (the STREAMS epilogue with one stream)."""
        if accumulate is not None:
            y, sw = accumulate
            _lib.check_hybrid(self.L.pieh_linear(_p(y), DTYPE_F32, 0, _p(x), self.act, x.stride(0), _p(lin.w), lin.w_dtype,
                                                 _p(lin.bias), M, lin.N, lin.K, EPI_STREAMS, 0.0, _p(sw["mix"]), _p(sw["out"]),
                                                 1, _stream()), "linear")
            return y
        out_dtype = DTYPE_F32 if out_dtype is None else out_dtype
        out = self._empty((M, lin.N), torch.float32 if out_dtype == DTYPE_F32 else torch.bfloat16)
        _lib.check_hybrid(self.L.pieh_linear_act(_p(out), out_dtype, out.stride(0), _p(x), self.act, x.stride(0), _p(lin.w),
                                                 lin.w_dtype, _p(lin.bias), M, lin.N, lin.K, act, float(coef[0]),
                                                 float(coef[1]), _stream()), "linear")
        return out

    def _sandwich(self, x, y, mix, post_w, h, next_w, T, add_rows=None, add_vec=None):
        _lib.check_hybrid(self.L.pieh_sandwich_add(_p(x), _p(y), C.byref(mix) if mix else None, _p(post_w),
                                                   float(self.args.residual_mult), _p(add_rows), _p(add_vec),
                                                   _p(h) if next_w is not None else None, self.act, _p(next_w),
                                                   float(self.args.norm_eps), T, self.W, _stream()), "sandwich_add")

    def _group_norm(self, x, gate_ptr, gate_ld, w, groups, gs, gate_fn, gate_first, T):
        out = self._empty((T, groups * gs), self.act_torch)
        _lib.check_hybrid(self.L.pieh_gated_group_norm(_p(out), self.act, _p(x), x.stride(0), gate_ptr, gate_ld, _p(w), groups,
                                                       gs, float(self.args.norm_eps), gate_fn, gate_first, T, _stream()),
                          "gated_group_norm")
        return out

    def _rot(self, key, batch, T, cache):
        """(cos, sin) table of this step for one (dims, base), formed once and shared by the layers that use it."""
        if key not in cache:
            cs = self._empty((T, key[0] // 2, 2))
            _lib.check_hybrid(self.L.pieh_rot_table(_p(cs), _p(batch.positions), _p(self.rot_tables[key]), T, key[0] // 2,
                                                    _stream()), "rot_table")
            cache[key] = cs
        return cache[key]

    def _parallel(self, ly, st, h, batch, bref, T, rot_cache):
        L, eps = self.L, float(self.args.norm_eps)
        H, G, d, dv, Hs, P, N, Gs, taps, ng = ly["dims"]
        inner = Hs * P
        proj = self._linear(ly["proj"], h, T)
        ld = proj.stride(0)
        col = lambda off: C.c_void_p(proj.data_ptr() + 4 * off)
        # left: windowed attention with sigmoid weights
        cs = self._rot(ly["rot"], batch, T, rot_cache) if ly["rot"] else None
        at = HybBiasAttn(H, G, d, dv, H * d, H * d + G * d, -1, None, None, eps, ly["scale"], 0.0, 0.0, None, 0, ly["window"],
                         _p(st["k"]), _p(st["v"]), self.act, None, 0, ly["rot"][0] if ly["rot"] else 0, _p(cs), None, None, 1,
                         _p(ly["pb"]))
        q = self._empty((T, H * d))
        _lib.check_hybrid(L.pieh_bias_attn_prepare(_p(q), _p(proj), ld, C.byref(at), bref, _stream()), "attn_prepare")
        left = self._empty((T, H * dv), self.act_torch)
        _lib.check_hybrid(L.pieh_bias_attn_run(_p(left), self.act, _p(q), None, 0, C.byref(at), bref, _stream()), "attn_run")
        # right: state-space layer; its projection columns are [z | x B C | dt] behind the attention's
        base = H * d + G * d + G * dv
        ss = HybSsd(Hs, P, N, Gs, taps, base + inner, base + 2 * inner + 2 * Gs * N, _p(ly["conv_w"]), _p(ly["conv_b"]),
                    _p(ly["dt_bias"]), _p(ly["A_log"]), _p(ly["D"]), _p(st["conv"]) if taps > 1 else None, _p(st["state"]))
        xbc, dtd = self._empty((T, inner + 2 * Gs * N)), self._empty((T, Hs, 2))
        _lib.check_hybrid(L.pieh_ssd_prepare(_p(xbc), _p(dtd), _p(proj), ld, C.byref(ss), bref, _stream()), "ssd_prepare")
        yr = self._empty((T, inner))
        _lib.check_hybrid(L.pieh_ssd_scan(_p(yr), _p(xbc), _p(dtd), C.byref(ss), bref, _stream()), "ssd_scan")
        right = self._group_norm(yr, col(base), ld, ly["out_norm"], ng, inner // ng, 2, 1, T)
        y = self._linear(ly["out_l"], left, T)
        return self._linear(ly["out_r"], right, T, accumulate=(y, ly["sum"]))

    def _general_delta(self, ly, st, h, bref, T):
        L = self.L
        H, n = ly["dims"]
        proj = self._linear(ly["proj"], h, T)          # [r | k | v | g | a]
        ld = proj.stride(0)
        low = self._linear(ly["w1"], h, T, out_dtype=self.act, act=EPI_TANH)
        dl = self._linear(ly["w2"], low, T)
        gd = HybGdelta(H, n, n, 0, H * n, 2 * H * n, 4 * H * n, _p(ly["a_bias"]), DECAY_SCALE, KEY_EPS, _p(st["state"]))
        decay, u, au = (self._empty((T, H, n)) for _ in range(3))
        _lib.check_hybrid(L.pieh_gdelta_prepare(_p(decay), _p(u), _p(au), _p(proj), ld, _p(dl), dl.stride(0), C.byref(gd), T,
                                                _stream()), "gdelta_prepare")
        o = self._empty((T, H * n))
        _lib.check_hybrid(L.pieh_gdelta_scan(_p(o), _p(proj), ld, _p(decay), _p(u), _p(au), C.byref(gd), bref, _stream()),
                          "gdelta_scan")
        mixed = self._group_norm(o, C.c_void_p(proj.data_ptr() + 4 * 3 * H * n), ld, ly["out_norm"], H, n, 1, 0, T)
        return self._linear(ly["out"], mixed, T)

    def _moe(self, ml, h, T):
        """-> (pieh_mix_sum describing the feed-forward's output, tensors to keep alive until it is consumed)."""
        L, E, top, W = self.L, ml["E"], ml["top"], self.W
        P = T * top
        z = self._linear(ml["router"], h, T)                       # [T, E] fp32 logits
        i32 = lambda n: self._empty((n,), torch.int32)
        bufs = [i32(P), i32(P), i32(P), self._empty((P,)), i32(1 + 3 * (P // 64 + E)), i32(1 + 3 * (P // 128 + E))]
        # the largest softmax scores are the largest logits, and score / (sum of the chosen scores) is the softmax over the
        # chosen logits alone: the routing mode that never forms the full softmax
        plan = HybMoePlan(E, top, 1, 1, ml["scale"], *[b.data_ptr() for b in bufs], ml["counters"].data_ptr(), 1)
        _lib.check_hybrid(L.pieh_moe_route(_p(z), z.stride(0), C.byref(plan), T, _stream()), "moe_route")
        wdt = DTYPE_F32 if self.exact else DTYPE_BF16
        ff2, ff = ml["gu"].shape[1], ml["gu"].shape[1] // 2
        hid = self._empty((P, ff), self.act_torch)
        _lib.check_hybrid(L.pieh_moe_linear(_p(hid), self.act, ff, _p(h), self.act, h.stride(0), _p(ml["gu"]), wdt, ff2 * W, P,
                                            ff2, W, 1, 1, 1.0, 0.0, 0.0, C.byref(plan), _stream()), "moe_gate_up")
        ys = self._empty((P, W))
        _lib.check_hybrid(L.pieh_moe_linear(_p(ys), DTYPE_F32, W, _p(hid), self.act, ff, _p(ml["down"]), wdt, W * ff, P, W, ff,
                                            0, 0, 1.0, 0.0, 0.0, C.byref(plan), _stream()), "moe_down")
        so = None
        if ml["shared"] is not None:
            g = ml["shared"]["gu"]
            sh = self._empty((T, g.N // 2), self.act_torch)
            _lib.check_hybrid(L.pieh_linear_glu(_p(sh), self.act, sh.stride(0), _p(h), self.act, h.stride(0), _p(g.w), g.w_dtype,
                                                T, g.N, g.K, 1.0, 0.0, 0.0, _stream()), "linear_glu")
            so = self._linear(ml["shared"]["down"], sh, T)
        mix = HybMixSum(ys.data_ptr(), bufs[2].data_ptr(), bufs[3].data_ptr(), top, so.data_ptr() if so is not None else None,
                        None, 0)
        return mix, (z, bufs, hid, ys, so)

    def _pass_adds(self, r):
        """What is added to x right before run r: (the saved embedding rows?, the pass vector or None)."""
        if r >= len(self.runs) or self.runs[r][1] is None:
            return False, None
        t = self.runs[r][1]
        return t > 0, self.loop_step[t]

    def step(self, batch: BatchDetails, cache: HybridCache, rows: torch.Tensor | None = None, trace: list | None = None):
        """One forward step over ``batch``; pages and state slots come from ``cache`` through the batch's block table and
        ``state_slots``.  rows: int32 device tensor of the token rows whose logits are wanted (None: each sequence's last
        row).  Returns fp32 logits [len(rows), vocab].  trace: if a list, the residual after every layer run is appended."""
        batch.validate()
        L, T, W, a = self.L, batch.total_tokens_in_step, self.W, self.args
        desc, keep = batch.hybrid_descriptor()
        bref = C.byref(desc)
        x, h = self._empty((T, W)), self._empty((T, W), self.act_torch)
        x0 = self._empty((T, W)) if self.keep_x0 else None
        for dst in (x, x0):
            if dst is not None:
                _lib.check_hybrid(L.pieh_embed_scaled(_p(dst), _p(self.embed), self.act, _p(batch.token_ids), 1.0, T, W, a.vocab,
                                                      _stream()), "embed")
        nruns = len(self.layers)
        use0, vec = self._pass_adds(0)
        self._sandwich(x, None, None, None, h, self.layers[0]["norm1"], T, x0 if use0 else None, vec)
        rot_cache = {}
        for r, (ly, st) in enumerate(zip(self.layers, cache.layers)):
            if ly["type"] == "parallel":
                y = self._parallel(ly, st, h, batch, bref, T, rot_cache)
            else:
                y = self._general_delta(ly, st, h, bref, T)
            ml, mix, alive, post = ly["mlp"], None, None, ly["norm1b"]
            if ml:
                self._sandwich(x, y, None, post, h, ly["norm2"], T)
                post = ly["norm2b"]
                if ml["kind"] == "dense":
                    hid = self._linear(ml["up"], h, T, out_dtype=self.act, act=EPI_XIELU, coef=ml["coef"])
                    y = self._linear(ml["down"], hid, T)
                else:
                    y = None
                    mix, alive = self._moe(ml, h, T)
            nxt = self.layers[r + 1]["norm1"] if r + 1 < nruns else None
            use0, vec = self._pass_adds(r + 1)
            if trace is None:       # the sublayer's output, what opens the next pass and the next run's norm: one pass over x
                self._sandwich(x, y, mix, post, h, nxt, T, x0 if use0 else None, vec)
            else:
                self._sandwich(x, y, mix, post, None, None, T)
                trace.append(x.clone())
                if nxt is not None:
                    self._sandwich(x, None, None, None, h, nxt, T, x0 if use0 else None, vec)
            del alive
        if rows is None:
            rows = batch.last_token_rows().to(torch.int32)
        R = int(rows.numel())
        xn = self._empty((R, W), self.act_torch)
        _lib.check_hybrid(L.pieh_stream_norm(_p(xn), self.act, _p(x), _p(rows), None, _p(self.final_norm), 0.0,
                                             float(a.norm_eps), R, 1, W, _stream()), "final_norm")
        logits = self._linear(self.head, xn, R)
        del keep
        return logits


def random_weights(args: ZelinexArgs, seed: int = 0, device="cpu") -> dict:
    """A synthetic checkpoint of this design (bf16 tensors): matrices U(-1, 1) scaled by 1 / sqrt(in), norm weights around
    1, biases of order one, decays spread over (0, 1), router rows large enough that choices are rarely near ties."""
    g = torch.Generator(device=device).manual_seed(seed)
    bf = torch.bfloat16
    rnd = lambda *s: torch.rand(s, generator=g, device=device) * 2 - 1
    lin = lambda o, i, gain=1.0: (gain * rnd(o, i) / math.sqrt(i)).to(bf)
    W = args.width
    w = {"embed": torch.randn((args.vocab, W), generator=g, device=device).to(bf), "final.norm": (1 + 0.1 * rnd(W)).to(bf)}
    if args.loop:
        w["loop.step"] = (0.5 * rnd(args.loop["times"], W)).to(bf)
    for i, cfg in enumerate(args.layers):
        p, m = f"l{i}.", cfg["mixer"]
        q = p + "mix."
        for nm in ("norm1", "norm1b") + (("norm2", "norm2b") if cfg.get("mlp") else ()):
            w[p + nm] = (1 + 0.2 * rnd(W)).to(bf)
        if cfg["type"] == "general_delta":
            H, n = m["heads"], m["dim"]
            low = max(4, min(64, W // 16))
            for nm in ("r", "k", "v", "g", "a"):
                w[q + nm] = lin(H * n, W, 2.0)
            w[q + "a.b"] = rnd(H * n).to(bf)
            w[q + "w1"], w[q + "w2"], w[q + "w0"] = lin(low, W, 2.0), lin(H * n, low, 3.0), (2 * rnd(H * n)).to(bf)
            w[q + "norm"], w[q + "o"] = (1 + 0.2 * rnd(H * n)).to(bf), lin(W, H * n)
        else:
            le, ri = m["left"], m["right"]
            H, G, d, dv = le["heads"], le["kv_heads"], le["dim"], le["vdim"]
            Hs, P, N, Gs, taps = ri["heads"], ri["vdim"], ri["state"], ri["groups"], ri.get("conv") or 1
            inner, C_ = Hs * P, Hs * P + 2 * Gs * N
            w[q + "left.q"], w[q + "left.k"], w[q + "left.v"] = lin(H * d, W, 2.0), lin(G * d, W, 2.0), lin(G * dv, W)
            w[q + "left.pb"], w[q + "left.o"] = (rnd(H) - 1.0).to(bf), lin(W, H * dv)
            w[q + "right.in"] = lin(2 * inner + 2 * Gs * N + Hs, W, 2.0)
            w[q + "right.conv"] = (rnd(C_, taps) / math.sqrt(taps) + torch.eye(taps, device=device)[-1]).to(bf)
            w[q + "right.conv.b"] = (0.2 * rnd(C_)).to(bf)
            w[q + "right.dt_bias"] = (rnd(Hs) - 1.0).to(bf)
            w[q + "right.A_log"] = torch.log(0.5 + 4 * torch.rand(Hs, generator=g, device=device)).to(bf)
            w[q + "right.D"] = (1 + 0.5 * rnd(Hs)).to(bf)
            w[q + "right.norm"], w[q + "right.o"] = (1 + 0.2 * rnd(inner)).to(bf), lin(W, inner)
        mlp = cfg.get("mlp")
        if not mlp:
            continue
        q = p + "mlp."
        if mlp["kind"] == "dense":
            w[q + "up"], w[q + "down"], w[q + "act"] = lin(mlp["ff"], W, 2.0), lin(W, mlp["ff"]), rnd(2).to(bf)
        else:
            E = mlp["router"]["experts"]
            w[q + "router"] = lin(E, W, 3.0)
            sizes = [(f"e{e}.", mlp["expert"]["ff"]) for e in range(E)]
            if mlp.get("shared"):
                sizes.append(("shared.", mlp["shared"]["ff"]))
            for name, ff in sizes:
                w[q + name + "gate"], w[q + name + "up"], w[q + name + "down"] = lin(ff, W, 2.0), lin(ff, W, 2.0), lin(W, ff)
    return w
