"""Continuous-batching engine for models that step over ``ragged.BatchDetails`` with a ``cache.HybridCache``
(``golitar.GolitarModel``, ``babodra.BabodraModel``, ``maginex.MaginexModel``, ``zelinex.ZelinexModel``): the generate loop of PIE (PIE/engine/inference_engine.py:228-297) lifted from one sequence to
a changing set of them.

    eng = HybridEngine(model, max_tokens=4096, max_seqs=4)
    outs = eng.generate([prompt_a, prompt_b, ...], max_new_tokens=32)           # greedy; sampler=make_sampler(...)

Scheduling policy of ``generate``: every step carries one token of each sequence that is decoding plus portions of
waiting prompts up to ``step_tokens`` rows; a prompt is admitted when a state slot and the pages of its whole length
(prompt + new tokens) are free, and hands both back when it ends, so later prompts re-use them.  ``forward`` is the
step underneath, also usable on its own: the caller names which sequences advance by which tokens (replay of a recorded
schedule, speculative verification, scoring)."""
from __future__ import annotations

import gc
import os

import torch

from .ragged import BatchDetails


class _DecodeGraph:
    """One captured decode step for n sequences of one token each (the launch-bound case): tokens, positions, the
    per-sequence descriptor and the block table live in ONE device buffer that a single copy from pinned host memory
    refills before every replay; the model step underneath is the same ``model.step``."""

    def __init__(self, engine, n: int):
        from ._lib import HybBatch
        self.n, self.W = n, engine.cache.n_pages
        W, dev = self.W, engine.device
        self.host = torch.zeros(9 * n + n * W, dtype=torch.int32).pin_memory()
        self.dev = torch.zeros_like(self.host, device=dev)
        self.copied = torch.cuda.Event()
        d = self.dev
        table = d[9 * n:].view(n, W)
        ptr = lambda off: d.data_ptr() + 4 * off
        # layout: tokens | positions | row->sequence | first row | rows | context | slot | tile sequence | tile row | table
        self.batch = BatchDetails(d[0:n], d[n:2 * n], list(range(n)), [1] * n, [0] * n, table, 0, n, n, [0] * n)
        desc = HybBatch(n, n, ptr(2 * n), ptr(n), ptr(3 * n), ptr(4 * n), ptr(5 * n), ptr(6 * n), table.data_ptr(), W, n,
                        ptr(7 * n), ptr(8 * n))
        self.batch._static_descriptor = (desc, (d,))
        self.rows = torch.arange(n, dtype=torch.int32, device=dev)
        h = self.host
        h[2 * n:3 * n] = torch.arange(n)
        h[3 * n:4 * n] = torch.arange(n)
        h[4 * n:5 * n] = 1
        h[7 * n:8 * n] = torch.arange(n)
        h[8 * n:9 * n] = torch.arange(n)
        self.graph = None
        self.model, self.cache, self.use_pdl = engine.model, engine.cache, engine.use_pdl   # no reference back to the engine

    def run(self, seqs):
        """seqs: [(tokens [1], context, pages, slot)] in batch order -> logits [n, vocab] (a static tensor)."""
        n, W, h = self.n, self.W, self.host
        self.copied.synchronize()
        for i, (tok, ctx, pages, slot) in enumerate(seqs):
            h[i], h[n + i], h[5 * n + i], h[6 * n + i] = tok[0], ctx, ctx, slot
            row = 9 * n + i * W
            h[row: row + len(pages)] = torch.tensor(pages, dtype=torch.int32)
        self.dev.copy_(h, non_blocking=True)
        self.copied.record()
        model, cache = self.model, self.cache
        if self.graph is None:
            # PIE_HYBRID_PDL=1: the captured launches become programmatic dependents of one another (a kernel's blocks
            # are resident while the kernel before it drains and wait at their top, pieh_set_pdl).  Measured on B200 at
            # the 1b layer sizes, batch 4: 1.70 ms per step against 1.67 ms without -- the step is bound by the kernels'
            # own dependent latencies, not by the gaps between them -- so it is off unless asked for
            pdl = getattr(model.L, "pieh_set_pdl", None) if self.use_pdl else None
            try:
                if pdl:
                    pdl(1)
                model.step(self.batch, cache, rows=self.rows)     # first use: opts kernels into their shared memory; the
                torch.cuda.synchronize()                           # state it advanced is put back before the capture
                self._rewind(seqs)
                # nothing may be destroyed while the stream captures (an older engine's graph freed by the cycle collector
                # in the middle of it invalidates the capture): collect now, and keep the collector off until the end
                gc.collect()
                gc.disable()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    self.logits = model.step(self.batch, cache, rows=self.rows)
            finally:
                gc.enable()
                if pdl:
                    pdl(0)
            self.graph = g
            self._rewind(seqs)
        self.graph.replay()
        return self.logits

    def _rewind(self, seqs):
        """Undo the recurrent-state advance of a warm-up / capture pass (the pages are simply overwritten again)."""
        for saved, layer in zip(self._saved, self.cache.layers):
            for k, v in saved.items():
                layer[k].copy_(v)

    def snapshot(self):
        self._saved = [{k: v.clone() for k, v in layer.items() if k in self.cache.slot_keys} for layer in self.cache.layers]


class HybridEngine:
    def __init__(self, model, max_tokens: int, max_seqs: int = 4, use_graph: bool = True):
        """use_graph: steps that are one token for every sequence replay a captured CUDA graph (one per batch size);
        anything else -- prompt portions, mixed steps -- launches the operators directly."""
        self.model = model
        self.cache = model.make_cache(max_tokens, max_seqs)
        self.device = model.device
        self.use_graph = use_graph and str(self.device).startswith("cuda")
        self.use_pdl = os.environ.get("PIE_HYBRID_PDL", "0") == "1"
        self._graphs = {}

    # ---- one step ----------------------------------------------------------------------------------
    def forward(self, entries, trace=None) -> torch.Tensor:
        """entries: [(seq_id, new_token_ids, wanted)] with ``wanted`` the indices into new_token_ids whose logits are
        asked for (None: the last one).  Unknown ids are admitted.  Returns fp32 logits [total wanted, vocab] in entry
        order (an empty tensor if nothing is wanted; the step still runs and advances every sequence)."""
        seqs, rows, row0 = [], [], 0
        for sid, toks, want in entries:
            toks = [int(t) for t in toks]
            if not toks:
                raise ValueError(f"sequence {sid}: no tokens in this step")
            if sid not in self.cache.seqs:
                self.cache.admit(sid)
            s = self.cache.reserve(sid, self.cache.seqs[sid]["length"] + len(toks))
            seqs.append((sid, toks, s["length"], list(s["pages"]), s["slot"]))
            want = [len(toks) - 1] if want is None else [int(w) for w in want]
            for w in want:
                if not 0 <= w < len(toks):
                    raise ValueError(f"sequence {sid}: wanted row {w} outside its {len(toks)} tokens")
            rows += [row0 + w for w in want]
            row0 += len(toks)
        if self.use_graph and all(len(toks) == 1 for _, toks, *_ in seqs) and hasattr(self.model, "layers"):
            n = len(seqs)
            dg = self._graphs.get(n)
            if dg is None:
                dg = self._graphs[n] = _DecodeGraph(self, n)
            if dg.graph is None:
                dg.snapshot()
            logits = dg.run([(toks, ctx, pages, slot) for _, toks, ctx, pages, slot in seqs])
            for sid, toks, *_ in seqs:
                self.cache.seqs[sid]["length"] += 1
            if not rows:
                return logits[:0]
            # the graph writes its logits into one fixed tensor: hand out a copy
            return logits.clone() if rows == list(range(n)) else logits[torch.tensor(rows, device=self.device)]
        batch = BatchDetails.build(seqs, device=self.device)
        # with nothing wanted the head still needs a row: take the last and drop the result
        idx = torch.tensor(rows if rows else [row0 - 1], dtype=torch.int32).to(self.device)
        logits = self.model.step(batch, self.cache, rows=idx, trace=trace)
        for sid, toks, *_ in seqs:
            self.cache.seqs[sid]["length"] += len(toks)
        return logits if rows else logits[:0]

    def finish(self, seq_id) -> None:
        self.cache.release(seq_id)

    # ---- scheduler ---------------------------------------------------------------------------------
    def generate(self, prompts, max_new_tokens: int, sampler=None, step_tokens: int = 512, eos: int | None = None):
        """Greedy (sampler None) or sampled continuation of every prompt; returns the new tokens per prompt.
        sampler: ``samplers.make_sampler(...)`` -- bf16 logits [rows, vocab] -> int32 [rows] on the device."""
        if sampler is None:
            from .samplers import make_sampler
            sampler = make_sampler(0.0)
        waiting = list(range(len(prompts)))          # prompt indices not admitted yet, in order
        live = {}                                    # index -> {"fed": prompt tokens already in the cache, "next": token}
        out = [[] for _ in prompts]
        while waiting or live:
            while waiting and self.cache.free_slots:
                i = waiting[0]
                if not self._room_for(live, prompts, max_new_tokens, i):
                    break
                waiting.pop(0)
                self.cache.admit(("gen", i))
                live[i] = {"fed": 0, "next": None}
            if not live:
                raise MemoryError("a prompt does not fit the engine's page pool")
            entries, takers, budget = [], [], step_tokens
            for i, s in live.items():                # decoding sequences first: one row each
                if s["next"] is not None:
                    entries.append((("gen", i), [s["next"]], None))
                    takers.append(i)
                    budget -= 1
            for i, s in live.items():                # then prompt portions while rows are left
                if s["next"] is None and budget > 0:
                    n = min(budget, len(prompts[i]) - s["fed"])
                    part = prompts[i][s["fed"]: s["fed"] + n]
                    s["fed"] += n
                    budget -= n
                    done = s["fed"] == len(prompts[i])
                    entries.append((("gen", i), part, None if done else []))
                    if done:
                        takers.append(i)
            logits = self.forward(entries)
            if takers:
                toks = sampler(logits.to(torch.bfloat16)).tolist()
                for i, tok in zip(takers, toks):
                    out[i].append(int(tok))
                    live[i]["next"] = int(tok)
                    if len(out[i]) >= max_new_tokens or (eos is not None and tok == eos):
                        self.finish(("gen", i))
                        del live[i]
        return out

    def _room_for(self, live, prompts, max_new_tokens, i) -> bool:
        """Pages for the whole life of prompt i beside what the live sequences may still claim."""
        ps = self.cache.page_size
        pages = lambda n: (n + ps - 1) // ps
        claimed = sum(pages(len(prompts[j]) + max_new_tokens) - len(self.cache.seqs[("gen", j)]["pages"]) for j in live)
        return pages(len(prompts[i]) + max_new_tokens) + claimed <= self.cache.allocator.get_num_free_pages()
