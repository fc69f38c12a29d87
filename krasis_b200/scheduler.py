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
    def __init__(self, model, max_tokens: int, max_requests: int = 4):
        self.model, self.max_requests = model, max_requests
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
        tb = ops.StepTables(packed, self.model.device)
        self.h2d_bytes += tb.h2d_bytes
        want_rows = torch.tensor(rows, dtype=torch.int64, device=self.model.device) if rows else None
        logits = self.model.forward_step(tb, want_rows)
        for rid, tokens, _ in entries:
            self.live[rid].kv.advance(len(tokens))
        self.steps_run += 1
        return logits

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
