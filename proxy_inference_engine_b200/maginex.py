"""Maginex: a decoder-only model of PARALLEL blocks -- one RMS norm per layer feeds both the mixer and the feed-forward,
and both outputs join the residual together -- whose sublayers read their input through a short causal convolution over
time.  A layer's mixer is one of: sliding-window attention (grouped heads, partial rotation, learned softmax sinks, values
blended with the first such layer's values, one output gate per head), latent attention (queries and keys / values
through low-rank latents, only the latent is cached, learned sinks, element-wise output gate) or a minGRU recurrence; the
feed-forward is a mixture of squared-relu experts (largest logits, softmax over the chosen ones) plus a shared expert.
Served through the ragged step of libpie_b200_hybrid.so like ``golitar.GolitarModel`` and ``babodra.BabodraModel``: same
``BatchDetails``, same ``cache.HybridCache`` (pages and state slots), same ``engine.HybridEngine``.

config.json: ``architecture`` "Maginex"; ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``, ``canon.taps`` and
``layers``, a list of ``{"type": "attention" | "latent_attention" | "mingru", "mixer": {...}, "mlp": {...} | null}`` with
    attention:         heads, kv_heads, dim, vdim, scale, mask.size (absent: all earlier tokens), rot {base, dims}, v_mix
    latent_attention:  heads, dim, vdim, q_rank, kv_rank, scale
    mingru:            width
    mlp:               kind "moe", expert.ff, router {experts, top}, shared {ff} | null
Tensors: ``embed``, ``head``, ``final.norm``, per layer i ``l<i>.norm1``, ``l<i>.canon1|canon2`` [width, taps],
``l<i>.mix.*`` (attention: q k v g o sink vmix; latent: dq dq.norm uq dkv dkv.norm uk uv g o sink; mingru: z z.b x x.b g
o) and ``l<i>.mlp.router`` (+ ``.b``), ``l<i>.mlp.e<j>.up|down``, ``l<i>.mlp.shared.up|down``.

One step over a ``ragged.BatchDetails`` (x: fp32 residual [T, W]; h: fp32 normed rows; u1 / u2: act dtype):

    x        = embed_scaled(tokens);  h = residual_norm(x; norm1 of layer 0)
    per layer:
      u1, u2 = canon_conv(h)                 h + conv_k(h) for the mixer and the feed-forward; history in the state slot
      attention:  p = linear(u1; [q | k | v | gate])  ->  bias_attn_prepare (rotation, value blend, append to pages)
                  -> bias_attn_run (window, learned sink, per-head gate)
      latent:     p = linear(u1; [dq | dkv | gate])   ->  latent_prepare (two norms; latent -> pages)
                  -> q = linear(cq; uq)  ->  q~ = linear_batched(q; uk^T per head)       keys are never expanded:
                     (kv_rank <= dim: uk^T uq is one matrix, formed at load)
                  -> bias_attn_run over the latent pages (one shared "head" of kv_rank)   (uk^T q) . c = q . (uk c)
                  -> linear_batched(.; uv per head, x sigmoid(gate))                      and uv (sum p c) = sum p (uv c)
      mingru:     p = linear(u1; [z | x | gate], biases)  ->  mingru_scan (state in the slot)
      x += linear(mixed; o)                                                   in place (STREAMS epilogue, one stream)
      moe:        z = linear(u2; router)  ->  moe_route (softmax over the chosen logits)  ->  two grouped products
                  (squared relu between them);  x += shared.down(relu^2(shared.up u2))  in place
      x, h   = residual_norm(x; + sum_k w_k ys[slot_k]; norm1 of the NEXT layer)
    logits   = linear(stream_norm(x[wanted rows]; final norm); head)          fp32

dtype "bfloat16": matrix-product inputs and the pages are bf16; accumulation, residual, norms, convolution, rotation
angles, softmax, routing and the recurrence are fp32.  dtype "float32": weights are widened once and every product is a
plain fp32 multiply-add.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass, field

import torch

from . import _lib
from ._lib import (DTYPE_BF16, DTYPE_F32, EPI_NONE, EPI_RELU2, EPI_SIGMUL, EPI_STREAMS, HybBiasAttn, HybCanon, HybMixSum,
                   HybMoePlan)
from .cache import HybridCache
from .golitar import _Linear, _p, _stream
from .ragged import BatchDetails

MIXERS = ("attention", "latent_attention", "mingru")


@dataclass
class MaginexArgs:
    vocab: int
    width: int
    layers: list
    norm_eps: float = 1e-6
    embed_scale: float = 1.0
    taps: int = 1
    architecture: str = "Maginex"
    raw: dict = field(default_factory=dict)

    @classmethod
    def from_dict(cls, cfg: dict) -> "MaginexArgs":
        for key in ("vocab", "width", "layers"):
            if key not in cfg:
                raise ValueError(f"Maginex config: '{key}' is missing")
        need = {"attention": ("heads", "kv_heads", "dim", "vdim", "scale"),
                "latent_attention": ("heads", "dim", "vdim", "q_rank", "kv_rank", "scale"), "mingru": ("width",)}
        vshape = None
        for i, ly in enumerate(cfg["layers"]):
            if ly.get("type") not in MIXERS:
                raise ValueError(f"Maginex config: layer {i} has unknown type {ly.get('type')!r}")
            m = ly.get("mixer") or {}
            for key in need[ly["type"]]:
                if key not in m:
                    raise ValueError(f"Maginex config: layer {i} mixer lacks '{key}'")
            if ly["type"] == "attention":
                if int(m["heads"]) % int(m["kv_heads"]):
                    raise ValueError(f"Maginex config: layer {i}: heads is not a multiple of kv_heads")
                rot = m.get("rot")
                if rot and (int(rot["dims"]) % 2 or int(rot["dims"]) > int(m["dim"])):
                    raise ValueError(f"Maginex config: layer {i}: rot.dims must be even and at most dim")
                if m.get("v_mix"):
                    shape = (int(m["kv_heads"]), int(m["vdim"]))
                    if vshape is not None and shape != vshape:
                        raise ValueError(f"Maginex config: layer {i}: value-mixing layers must share kv_heads and vdim")
                    vshape = shape
            mlp = ly.get("mlp")
            if mlp:
                if mlp.get("kind", "moe") != "moe":
                    raise ValueError(f"Maginex config: layer {i} has unknown feed-forward kind {mlp.get('kind')!r}")
                if int(mlp["router"]["top"]) > int(mlp["router"]["experts"]):
                    raise ValueError(f"Maginex config: layer {i}: 'top' exceeds the number of experts")
        taps = int((cfg.get("canon") or {}).get("taps") or 1)
        if not 1 <= taps <= 8:
            raise ValueError("Maginex config: canon.taps must be between 1 and 8")
        return cls(vocab=int(cfg["vocab"]), width=int(cfg["width"]), layers=list(cfg["layers"]),
                   norm_eps=float((cfg.get("norm") or {}).get("eps", 1e-6)),
                   embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)), taps=taps,
                   architecture=cfg.get("architecture", "Maginex"), raw=cfg)

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embed_scale}, "canon": {"taps": self.taps},
                "layers": self.layers}


def rotary_frequencies(rot: dict) -> list:
    """Angle per position of rotated pair i: base^(-2 i / dims)."""
    dims = int(rot["dims"])
    return [float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)]


class MaginexModel:
    def __init__(self, args: MaginexArgs, weights: dict, device="cuda", dtype: str = "bfloat16"):
        if dtype not in ("bfloat16", "float32"):
            raise ValueError("dtype must be 'bfloat16' or 'float32'")
        self.args, self.device, self.dtype = args, device, dtype
        self.exact = dtype == "float32"
        self.act_torch = torch.float32 if self.exact else torch.bfloat16
        self.act = DTYPE_F32 if self.exact else DTYPE_BF16
        self.L = _lib.load_hybrid(build_if_missing=True)
        self.W, W, self.S = args.width, args.width, 1        # one residual stream
        taps = args.taps
        f32 = lambda t: t.to(device=device, dtype=torch.float32).contiguous()
        get = lambda name: weights[name]
        lin = lambda w, b=None: _Linear(w, b, self.exact, device)
        wdt = torch.float32 if self.exact else torch.bfloat16
        self.embed = get("embed").to(device=device, dtype=self.act_torch).contiguous()
        self.head = lin(get("head"))
        self.final_norm = f32(get("final.norm"))
        one = torch.ones((1,), dtype=torch.float32, device=device)
        self.unit = {"mix": one.view(1, 1), "out": one}       # one residual stream, taken as it is
        self.layers, self.cache_specs, self.rot_tables = [], [], {}
        first_vmix = True
        for i, cfg in enumerate(args.layers):
            p, m, kind = f"l{i}.", cfg["mixer"], cfg["type"]
            mw = lambda n: get(p + "mix." + n)
            ly = {"type": kind, "norm1": f32(get(p + "norm1")), "canon1": f32(get(p + "canon1")), "mlp": None}
            if tuple(ly["canon1"].shape) != (W, taps):
                raise ValueError(f"{p}canon1 has shape {tuple(ly['canon1'].shape)}, expected {(W, taps)}")
            slots = {"canon": (taps - 1, W)} if taps > 1 else {}
            if kind == "attention":
                H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
                ly["dims"] = (H, G, d, dv)
                ly["proj"] = lin(torch.cat([mw("q"), mw("k"), mw("v"), mw("g")], 0))
                ly["out"] = lin(mw("o"))
                ly["sink"], ly["scale"] = f32(mw("sink")), float(m["scale"])
                ly["window"] = int((m.get("mask") or {}).get("size") or 0)
                rot = m.get("rot") or None
                ly["rot"] = None
                if rot and int(rot["dims"]) > 0:
                    key = (int(rot["dims"]), float(rot["base"]))
                    if key not in self.rot_tables:
                        self.rot_tables[key] = torch.tensor(rotary_frequencies(rot), dtype=torch.float64).to(device)
                    ly["rot"] = key
                ly["vmix"] = None                      # None: no blending; "first": keeps its values; tensor: lambda
                if m.get("v_mix"):
                    ly["vmix"] = "first" if first_vmix else f32(mw("vmix")).reshape(1)
                    first_vmix = False
                self.cache_specs.append({"pages": {"k": (G, d), "v": (G, dv)}, "slots": slots})
            elif kind == "latent_attention":
                H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
                rq, rkv = int(m["q_rank"]), int(m["kv_rank"])
                if rkv > 512:
                    raise ValueError(f"layer {i}: kv_rank {rkv} is beyond the 512 features the latent attention kernel holds")
                ly["dims"] = (H, d, dv, rq, rkv)
                ly["proj"] = lin(torch.cat([mw("dq"), mw("dkv"), mw("g")], 0))
                ly["dq_norm"], ly["dkv_norm"] = f32(mw("dq.norm")), f32(mw("dkv.norm"))
                # queries go INTO the latent space: per head q~ = uk^T q with uk^T [kv_rank, dim].  Where the latent is no
                # wider than a head, uk^T uq is formed once here (one matrix of no more rows than uq: same product count,
                # one launch fewer per step); otherwise q is formed first and the heads' uk^T follow as one batched product
                ukT = mw("uk").reshape(H, d, rkv).transpose(1, 2)
                if rkv <= d:
                    fold = torch.bmm(ukT.double(), mw("uq").reshape(H, d, rq).double()).reshape(H * rkv, rq)
                    ly["uq"], ly["ukT"] = lin(fold.float()), None
                else:
                    ly["uq"], ly["ukT"] = lin(mw("uq")), ukT.to(device=device, dtype=wdt).contiguous()
                ly["uv"] = mw("uv").reshape(H, dv, rkv).to(device=device, dtype=wdt).contiguous()
                ly["out"] = lin(mw("o"))
                ly["sink"], ly["scale"] = f32(mw("sink")), float(m["scale"])
                self.cache_specs.append({"pages": {"c": (1, rkv)}, "slots": slots})
            else:
                n = int(m["width"])
                ly["dims"] = (n,)
                bias = torch.cat([mw("z.b").float(), mw("x.b").float(), torch.zeros(n, device=mw("z.b").device)])
                ly["proj"] = lin(torch.cat([mw("z"), mw("x"), mw("g")], 0), bias)
                ly["out"] = lin(mw("o"))
                self.cache_specs.append({"slots": dict(slots, state=(n,))})
            mlp = cfg.get("mlp")
            if mlp:
                q = p + "mlp."
                E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
                stack = lambda ts: torch.stack(ts, 0).to(device=device, dtype=wdt).contiguous()
                ly["canon2"] = f32(get(p + "canon2"))
                ly["mlp"] = {"E": E, "top": top, "router": lin(get(q + "router"), weights.get(q + "router.b")),
                             "up": stack([get(f"{q}e{e}.up") for e in range(E)]),
                             "down": stack([get(f"{q}e{e}.down") for e in range(E)]),
                             "counters": torch.zeros(2 * E + 2, dtype=torch.int32, device=device), "shared": None}
                if mlp.get("shared"):
                    ly["mlp"]["shared"] = {"up": lin(get(q + "shared.up")), "down": lin(get(q + "shared.down"))}
            self.layers.append(ly)

    # ------------------------------------------------------------------------------------------------
    def make_cache(self, max_tokens: int, max_seqs: int = 4) -> HybridCache:
        return HybridCache(self.cache_specs, max_tokens, max_seqs, self.device, self.act_torch, lib=self.L)

    def _empty(self, shape, dtype=None):
        return torch.empty(shape, dtype=dtype or torch.float32, device=self.device)

    def _linear(self, lin: _Linear, x, M, out_dtype=None, epi=EPI_NONE, into=None):
        """into: the fp32 residual -- the product is ADDED to it in place."""
        out_dtype = DTYPE_F32 if out_dtype is None else out_dtype
        if into is not None:
            out, epi, ld = into, EPI_STREAMS, 0
        else:
            out = self._empty((M, lin.N), torch.float32 if out_dtype == DTYPE_F32 else torch.bfloat16)
            ld = out.stride(0)
        _lib.check_hybrid(self.L.pieh_linear(_p(out), out_dtype, ld, _p(x), self.act, x.stride(0), _p(lin.w), lin.w_dtype,
                                             _p(lin.bias), M, lin.N, lin.K, epi, 0.0,
                                             _p(self.unit["mix"]) if into is not None else None,
                                             _p(self.unit["out"]) if into is not None else None,
                                             1 if into is not None else 0, _stream()), "linear")
        return out

    def _heads(self, out, out_dtype, x, w, M, nb, N, K, epi=EPI_NONE, gate=None, gate_ld=0):
        """nb per-head products in one launch: x [M, nb * K] (head-major columns), w [nb, N, K] -> out [M, nb * N]."""
        wd = DTYPE_F32 if self.exact else DTYPE_BF16
        _lib.check_hybrid(self.L.pieh_linear_batched(_p(out), out_dtype, out.stride(0), N, _p(x), self.act, x.stride(0), K,
                                                     _p(w), wd, N * K, nb, M, N, K, epi, gate, gate_ld, N, _stream()),
                          "linear_batched")
        return out

    def _residual_norm(self, x, mix, h, w, T):
        _lib.check_hybrid(self.L.pieh_residual_norm(_p(x), None, C.byref(mix) if mix else None, _p(h) if w is not None else None,
                                                    _p(w), float(self.args.norm_eps), T, self.W, _stream()), "residual_norm")

    def _rot(self, key, batch, T, cache):
        """(cos, sin) table of this step for one (dims, base), formed once and shared by the layers that use it."""
        if key not in cache:
            cs = self._empty((T, key[0] // 2, 2))
            _lib.check_hybrid(self.L.pieh_rot_table(_p(cs), _p(batch.positions), _p(self.rot_tables[key]), T, key[0] // 2,
                                                    _stream()), "rot_table")
            cache[key] = cs
        return cache[key]

    def _moe(self, ml, u2, x, T):
        """Routes, runs the chosen experts, adds the shared expert into x; returns the mixture for residual_norm."""
        L, E, top, W = self.L, ml["E"], ml["top"], self.W
        P = T * top
        z = self._linear(ml["router"], u2, T)                      # [T, E] fp32 logits
        i32 = lambda n: self._empty((n,), torch.int32)
        bufs = [i32(P), i32(P), i32(P), self._empty((P,)), i32(1 + 3 * (P // 64 + E)), i32(1 + 3 * (P // 128 + E))]
        plan = HybMoePlan(E, top, 1, 1, 1.0, *[b.data_ptr() for b in bufs], ml["counters"].data_ptr(), 1)
        _lib.check_hybrid(L.pieh_moe_route(_p(z), z.stride(0), C.byref(plan), T, _stream()), "moe_route")
        wdt = DTYPE_F32 if self.exact else DTYPE_BF16
        ff = ml["up"].shape[1]
        hid = self._empty((P, ff), self.act_torch)
        _lib.check_hybrid(L.pieh_moe_linear(_p(hid), self.act, ff, _p(u2), self.act, u2.stride(0), _p(ml["up"]), wdt, ff * W,
                                            P, ff, W, 1, 2, 1.0, 0.0, 0.0, C.byref(plan), _stream()), "moe_up")
        ys = self._empty((P, W))
        _lib.check_hybrid(L.pieh_moe_linear(_p(ys), DTYPE_F32, W, _p(hid), self.act, ff, _p(ml["down"]), wdt, W * ff, P, W,
                                            ff, 0, 0, 1.0, 0.0, 0.0, C.byref(plan), _stream()), "moe_down")
        if ml["shared"] is not None:
            sh = self._linear(ml["shared"]["up"], u2, T, out_dtype=self.act, epi=EPI_RELU2)
            self._linear(ml["shared"]["down"], sh, T, into=x)
        mix = HybMixSum(ys.data_ptr(), bufs[2].data_ptr(), bufs[3].data_ptr(), top, None, None, 0)
        return mix, (z, bufs, hid, ys)

    def step(self, batch: BatchDetails, cache: HybridCache, rows: torch.Tensor | None = None, trace: list | None = None):
        """One forward step over ``batch``; pages and state slots come from ``cache`` through the batch's block table and
        ``state_slots``.  rows: int32 device tensor of the token rows whose logits are wanted (None: each sequence's last
        row).  Returns fp32 logits [len(rows), vocab].  trace: if a list, the residual after every layer is appended."""
        batch.validate()
        L, T, W, a = self.L, batch.total_tokens_in_step, self.W, self.args
        desc, keep = batch.hybrid_descriptor()
        bref = C.byref(desc)
        eps = float(a.norm_eps)
        x, h = self._empty((T, W)), self._empty((T, W))
        _lib.check_hybrid(L.pieh_embed_scaled(_p(x), _p(self.embed), self.act, _p(batch.token_ids), float(a.embed_scale), T,
                                              W, a.vocab, _stream()), "embed_scaled")
        self._residual_norm(x, None, h, self.layers[0]["norm1"], T)
        rot_cache, v_keep = {}, None
        for li, (ly, st) in enumerate(zip(self.layers, cache.layers)):
            ml = ly["mlp"]
            u1 = self._empty((T, W), self.act_torch)
            u2 = self._empty((T, W), self.act_torch) if ml else None
            cn = HybCanon(a.taps, 2 if ml else 1, (C.c_void_p * 4)(ly["canon1"].data_ptr(), ly["canon2"].data_ptr() if ml else None),
                          (C.c_void_p * 4)(u1.data_ptr(), u2.data_ptr() if ml else None),
                          st["canon"].data_ptr() if a.taps > 1 else None)
            _lib.check_hybrid(L.pieh_canon_conv(C.byref(cn), self.act, _p(h), W, bref, _stream()), "canon_conv")
            proj = self._linear(ly["proj"], u1, T)
            ld = proj.stride(0)
            if ly["type"] == "attention":
                H, G, d, dv = ly["dims"]
                cs = self._rot(ly["rot"], batch, T, rot_cache) if ly["rot"] else None
                lam = None
                if ly["vmix"] == "first":
                    v_keep = self._empty((T, G * dv))
                elif ly["vmix"] is not None:
                    lam = ly["vmix"]
                at = HybBiasAttn(H, G, d, dv, H * d, H * d + G * d, H * d + G * d + G * dv, None, None, eps, ly["scale"], 0.0,
                                 0.0, None, 0, ly["window"], _p(st["k"]), _p(st["v"]), self.act, _p(ly["sink"]), 1,
                                 ly["rot"][0] if ly["rot"] else 0, _p(cs), _p(lam),
                                 _p(v_keep) if ly["vmix"] is not None else None)
                q = self._empty((T, H * d))
                _lib.check_hybrid(L.pieh_bias_attn_prepare(_p(q), _p(proj), ld, C.byref(at), bref, _stream()), "attn_prepare")
                mixed = self._empty((T, H * dv), self.act_torch)
                _lib.check_hybrid(L.pieh_bias_attn_run(_p(mixed), self.act, _p(q), _p(proj), ld, C.byref(at), bref, _stream()),
                                  "attn_run")
            elif ly["type"] == "latent_attention":
                H, d, dv, rq, rkv = ly["dims"]
                cq = self._empty((T, rq), self.act_torch)
                _lib.check_hybrid(L.pieh_latent_prepare(_p(cq), self.act, _p(proj), ld, rq, rq, rkv, _p(ly["dq_norm"]),
                                                        _p(ly["dkv_norm"]), eps, _p(st["c"]), self.act, bref, _stream()),
                                  "latent_prepare")
                if ly["ukT"] is None:
                    ql = self._linear(ly["uq"], cq, T)                                       # [T, H kv_rank] at once
                else:
                    qh = self._linear(ly["uq"], cq, T, out_dtype=self.act)                   # [T, H d]
                    ql = self._heads(self._empty((T, H * rkv)), DTYPE_F32, qh, ly["ukT"], T, H, rkv, d)
                at = HybBiasAttn(H, 1, rkv, rkv, 0, 0, -1, None, None, eps, ly["scale"], 0.0, 0.0, None, 0, 0, _p(st["c"]),
                                 _p(st["c"]), self.act, _p(ly["sink"]), 0, 0, None, None, None)
                ol = self._empty((T, H * rkv), self.act_torch)
                _lib.check_hybrid(L.pieh_bias_attn_run(_p(ol), self.act, _p(ql), None, 0, C.byref(at), bref, _stream()),
                                  "latent_attn_run")
                mixed = self._heads(self._empty((T, H * dv), self.act_torch), self.act, ol, ly["uv"], T, H, dv, rkv,
                                    epi=EPI_SIGMUL, gate=C.c_void_p(proj.data_ptr() + 4 * (rq + rkv)), gate_ld=ld)
            else:
                (n,) = ly["dims"]
                mixed = self._empty((T, n), self.act_torch)
                scratch = self._empty((3, desc.n_tiles, n)) if desc.n_tiles > desc.n_seq else None
                _lib.check_hybrid(L.pieh_mingru_scan(_p(mixed), self.act, _p(proj), ld, n, _p(st["state"]), _p(scratch), bref,
                                                     _stream()), "mingru_scan")
            self._linear(ly["out"], mixed, T, into=x)
            mix = alive = None
            if ml:
                mix, alive = self._moe(ml, u2, x, T)
            nxt = self.layers[li + 1]["norm1"] if li + 1 < len(self.layers) else None
            if mix is not None or nxt is not None:
                self._residual_norm(x, mix, h, nxt, T)
            del alive
            if trace is not None:
                trace.append(x.clone())
        if rows is None:
            rows = batch.last_token_rows().to(torch.int32)
        R = int(rows.numel())
        xn = self._empty((R, W), self.act_torch)
        _lib.check_hybrid(L.pieh_stream_norm(_p(xn), self.act, _p(x), _p(rows), None, _p(self.final_norm), 0.0, eps, R, 1, W,
                                             _stream()), "final_norm")
        logits = self._linear(self.head, xn, R)
        del keep
        return logits


def random_weights(args: MaginexArgs, seed: int = 0, device="cpu") -> dict:
    """A synthetic checkpoint of this design (bf16 tensors): matrices U(-1, 1) scaled by 1 / sqrt(in), norm weights around
    1, convolution taps and biases small, sinks and blend weights of order one, router rows large enough that choices are
    rarely near ties."""
    g = torch.Generator(device=device).manual_seed(seed)
    bf = torch.bfloat16
    rnd = lambda *s: torch.rand(s, generator=g, device=device) * 2 - 1
    lin = lambda o, i, gain=1.0: (gain * rnd(o, i) / math.sqrt(i)).to(bf)
    W = args.width
    w = {"embed": (torch.randn((args.vocab, W), generator=g, device=device) / args.embed_scale).to(bf),
         "head": lin(args.vocab, W), "final.norm": (1 + 0.1 * rnd(W)).to(bf)}
    for i, cfg in enumerate(args.layers):
        p, m = f"l{i}.", cfg["mixer"]
        q = p + "mix."
        w[p + "norm1"] = (1 + 0.1 * rnd(W)).to(bf)
        w[p + "canon1"] = (0.3 * rnd(W, args.taps)).to(bf)
        if cfg["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            w[q + "q"], w[q + "k"], w[q + "v"] = lin(H * d, W, 2.0), lin(G * d, W, 2.0), lin(G * dv, W)
            w[q + "g"], w[q + "o"] = lin(H, W, 2.0), lin(W, H * dv)
            w[q + "sink"] = rnd(H).to(bf)
            w[q + "vmix"] = (0.5 + 0.3 * rnd(1)).reshape(()).to(bf)
        elif cfg["type"] == "latent_attention":
            H, d, dv, rq, rkv = m["heads"], m["dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            w[q + "dq"], w[q + "dkv"] = lin(rq, W), lin(rkv, W)
            w[q + "dq.norm"], w[q + "dkv.norm"] = (1 + 0.2 * rnd(rq)).to(bf), (1 + 0.2 * rnd(rkv)).to(bf)
            w[q + "uq"], w[q + "uk"], w[q + "uv"] = lin(H * d, rq, 2.0), lin(H * d, rkv, 2.0), lin(H * dv, rkv)
            w[q + "g"], w[q + "o"] = lin(H * dv, W, 2.0), lin(W, H * dv)
            w[q + "sink"] = rnd(H).to(bf)
        else:
            n = m["width"]
            w[q + "z"], w[q + "x"], w[q + "g"], w[q + "o"] = lin(n, W, 2.0), lin(n, W, 2.0), lin(n, W, 2.0), lin(W, n)
            w[q + "z.b"], w[q + "x.b"] = (0.5 * rnd(n)).to(bf), (0.2 * rnd(n)).to(bf)
        mlp = cfg.get("mlp")
        if not mlp:
            continue
        q = p + "mlp."
        w[p + "canon2"] = (0.3 * rnd(W, args.taps)).to(bf)
        E = mlp["router"]["experts"]
        w[q + "router"], w[q + "router.b"] = lin(E, W, 3.0), (0.2 * rnd(E)).to(bf)
        sizes = [(f"e{e}.", mlp["expert"]["ff"]) for e in range(E)]
        if mlp.get("shared"):
            sizes.append(("shared.", mlp["shared"]["ff"]))
        for name, ff in sizes:
            w[q + name + "up"], w[q + name + "down"] = lin(ff, W, 2.0), lin(W, ff)
    return w
