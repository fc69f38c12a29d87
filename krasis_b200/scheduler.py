"""Step scheduler for several live requests: continuous batching of prompt portions and decoded tokens.

A model takes part by offering
    make_caches(max_tokens, max_requests) -> (paged cache, state pool)
    forward_step(tables: seqops.StepTables, want_rows) -> fp32 logits [len(want_rows), vocab]
`Scheduler.step` runs one explicit step (entries given by the caller: a trace replay, a server loop); `Scheduler.generate`
is the generation entry point that plans the steps itself: requests are admitted while state slots and pages are free, prompts
are cut into portions under a per-step token budget, and every running request adds one decoded token to each step.
Pages (`SequenceKVState` over the model's paged cache) and state slots (`RecurrentStatePool`) go back at `finish` and are reused.
"""
from collections import deque
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import seqops as ops
from .attention import SequenceKVState
from .sampling import Sampler, SamplingParams


class Request:
    def __init__(self, rid, kv: SequenceKVState, slot: int):
        self.id, self.kv, self.slot = rid, kv, slot
        self.prompt: List[int] = []
        self.fed = 0                     # prompt tokens already run
        self.output: List[int] = []
        self.pending: Optional[int] = None   # sampled token that has not been run yet

    @property
    def num_tokens(self) -> int:
        return self.kv.seq_len


class Scheduler:
    def __init__(self, model, max_tokens: int, max_requests: int = 4, cuda_graphs: bool = False):
        """cuda_graphs: steps in which every entry brings one token (decoding) are captured once per (entries, page-list width) and
        replayed — same kernels, the Python launch path off the critical path.  The tables of a replayed step are copied into the
        fixed device buffer the graph reads; a capture that fails leaves the eager path in charge."""
        self.model, self.max_requests = model, max_requests
        self.cuda_graphs = bool(cuda_graphs) and torch.cuda.is_available()
        self._graphs = {}
        self.kv_cache, self.state_pool = model.make_caches(max_tokens, max_requests)
        self.live: Dict[object, Request] = {}
        self.steps_run = 0
        self.h2d_bytes = 0

    # ------------------------------------------------------------------------------------------- explicit steps
    def admit(self, rid) -> Request:
        if rid in self.live:
            return self.live[rid]
        if len(self.live) >= self.max_requests:
            raise RuntimeError(f"more than {self.max_requests} live requests")
        req = Request(rid, SequenceKVState(self.kv_cache, seq_id=len(self.live)), self.state_pool.alloc())
        self.live[rid] = req
        return req

    def can_admit(self, num_tokens: int) -> bool:
        ps = self.kv_cache.page_size
        return len(self.live) < self.max_requests and self.kv_cache.free_page_count >= (num_tokens + ps - 1) // ps

    def finish(self, rid) -> None:
        req = self.live.pop(rid)
        req.kv.free()
        self.state_pool.free(req.slot)

    def step(self, entries: Sequence[Tuple[object, Sequence[int], Sequence[int]]]) -> Optional[torch.Tensor]:
        """entries: (request id, next tokens, indices among these tokens whose logits are wanted).  All entries run as one batch.
        Returns the wanted logits in entry order (None if nothing is wanted)."""
        if not entries:
            return None
        rows, packed, cu = [], [], 0
        for rid, tokens, want in entries:
            if len(tokens) == 0:
                raise ValueError("an entry needs at least one token")
            req = self.admit(rid)
            req.kv.ensure_capacity(len(tokens))
            packed.append((tokens, req.kv.seq_len, req.slot, req.kv.pages))
            rows += [cu + int(w) for w in want]
            cu += len(tokens)
        ran, logits = False, None
        if self.cuda_graphs and cu == len(entries):
            ran, logits = self._decode_step_graphed(packed, rows)
        if not ran:
            tb = ops.StepTables(packed, self.model.device)
            self.h2d_bytes += tb.h2d_bytes
            want_rows = torch.tensor(rows, dtype=torch.int64, device=self.model.device) if rows else None
            logits = self.model.forward_step(tb, want_rows)
        for rid, tokens, _ in entries:
            self.live[rid].kv.advance(len(tokens))
        self.steps_run += 1
        return logits

    def _decode_step_graphed(self, packed, rows):
        """One decoded token per entry, replayed from a CUDA graph.  Returns (ran, logits); ran is False where the eager path has to run."""
        dev, S = self.model.device, len(packed)
        maxp = (max(1, max(len(e[3]) for e in packed)) + 7) // 8 * 8
        key = (S, maxp)
        ent = self._graphs.get(key)
        if ent is False:
            return False, None
        if ent is None:
            try:
                n = 3 * S + (S + 1) + S + S * maxp
                buf = torch.zeros(n, dtype=torch.int32, device=dev)
                all_rows = torch.arange(S, dtype=torch.int64, device=dev)
                tb = ops.StepTables(packed, dev, pad_pages_to=8, device_buf=buf)
                # snapshot of every recurrent state: warm-up and capture run the step for real, the replay must start from here
                saved = [t.clone() for t in self.state_pool.tensors]
                side = torch.cuda.Stream(dev)
                side.wait_stream(torch.cuda.current_stream(dev))
                with torch.cuda.stream(side):
                    self.model.forward_step(tb, all_rows)
                torch.cuda.current_stream(dev).wait_stream(side)
                torch.cuda.synchronize(dev)
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    out = self.model.forward_step(tb, all_rows)
                for t, sv in zip(self.state_pool.tensors, saved):
                    t.copy_(sv)
                ent = (graph, buf, out, all_rows)          # everything the captured launches read stays alive with the graph
                self._graphs[key] = ent
            except Exception as exc:            # noqa: BLE001 — never a wrong result: fall back to eager launches
                import warnings
                warnings.warn(f"CUDA graph capture of a decode step failed ({exc}); using eager launches")
                self._graphs[key] = False
                try:
                    torch.cuda.synchronize(dev)
                except Exception:               # noqa: BLE001
                    pass
                return False, None
        graph, buf, out, _ = ent
        tb = ops.StepTables(packed, dev, pad_pages_to=8, device_buf=buf)
        self.h2d_bytes += tb.h2d_bytes
        graph.replay()
        if not rows:
            return True, None
        if rows == list(range(S)):
            return True, out.clone()            # the graph's own output buffer is overwritten by the next replay
        return True, out.index_select(0, torch.tensor(rows, dtype=torch.int64, device=dev))

    # ------------------------------------------------------------------------------------------- generation
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int, sampling: Optional[SamplingParams] = None,
                 step_tokens: int = 512, eos: Optional[int] = None) -> List[List[int]]:
        """Greedy (or sampled) continuation of every prompt; returns the generated ids per prompt, in order."""
        sampler = Sampler(sampling, self.model.device)
        waiting = deque(enumerate(prompts))
        running: List[Request] = []
        results: List[Optional[List[int]]] = [None] * len(prompts)
        while waiting or running:
            while waiting and self.can_admit(len(waiting[0][1]) + max_new_tokens):
                idx, prompt = waiting.popleft()
                if len(prompt) == 0:
                    raise ValueError("empty prompt")
                req = self.admit(("gen", idx))
                req.prompt, req.index = list(prompt), idx
                running.append(req)
            if not running:
                raise RuntimeError("a prompt does not fit the cache pool")
            budget, entries, sampled_from = step_tokens, [], []
            for req in running:                                   # decoded tokens first: they always fit
                if req.pending is not None:
                    entries.append((req.id, [req.pending], [0]))
                    sampled_from.append(req)
                    budget -= 1
            for req in running:
                if req.pending is None and budget > 0:
                    n = min(budget, len(req.prompt) - req.fed)
                    last = req.fed + n == len(req.prompt)
                    entries.append((req.id, req.prompt[req.fed:req.fed + n], [n - 1] if last else []))
                    req.fed += n
                    budget -= n
                    if last:
                        sampled_from.append(req)
            logits = self.step(entries)
            if sampled_from:
                toks = sampler(logits).tolist()
                for req, tok in zip(sampled_from, toks):
                    req.output.append(tok)
                    req.pending = tok
                    if len(req.output) >= max_new_tokens or (eos is not None and tok == eos):
                        results[req.index] = req.output
                        running.remove(req)
                        self.finish(req.id)
        return results
