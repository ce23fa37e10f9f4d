"""Continuous-batching scheduler over one ModelRunner (the reference's Scheduler event loop,
python/sglang/srt/managers/scheduler.py: get_next_batch_to_run / run_batch / process_batch_result,
and its PrefillAdder with chunked prefill and mixed batches).

Policy of one step:
  1. every running request that has finished its prompt contributes one decode token;
  2. prompts in progress, then waiting requests (first come, first served, admitted while a request
     slot and enough pages for the WHOLE request — prompt plus max_new_tokens — are free), fill the
     rest of the step's token budget with a portion of their prompt (chunked prefill).
All of it runs as ONE batch through ModelRunner.forward; the last token of a finished prompt and every
decode token are sampled.  `run_step` is that batch execution on its own, for callers that dictate
the portions themselves (trace replay)."""
from __future__ import annotations

from collections import deque
from typing import Deque, Dict, List, Optional

import torch

from ..layers.sampler import Sampler
from ..model_executor.model_runner import ModelRunner
from .schedule_batch import Req, SamplingParams, StepItem


class Scheduler:
    def __init__(self, runner: ModelRunner, chunked_prefill_size: int = 512):
        self.runner = runner
        self.chunk = max(1, int(chunked_prefill_size))
        self.waiting: Deque[Req] = deque()
        self.running: List[Req] = []
        self.sampler = Sampler(runner.device)
        self.reserved_pages: Dict[str, int] = {}
        self.steps = 0

    # ---- request life cycle --------------------------------------------------------------------
    def add_request(self, req: Req) -> None:
        total = len(req.input_ids) + req.sampling_params.max_new_tokens
        if total > self.runner.context_length or total > self.runner.max_total_tokens:
            raise ValueError(f"request {req.rid}: {total} tokens exceed the engine's capacity")
        if not req.input_ids:
            raise ValueError(f"request {req.rid}: empty prompt")
        self.waiting.append(req)

    def _pages(self, tokens: int) -> int:
        p = self.runner.page_size
        return (tokens + p - 1) // p

    def _try_admit(self, req: Req) -> bool:
        need = self._pages(len(req.input_ids) + req.sampling_params.max_new_tokens)
        free = self.runner.free_token_slots() // self.runner.page_size - sum(
            self.reserved_pages[r.rid] - self._pages(r.cached_len) for r in self.running)
        if need > free or not self.runner.admit(req):
            return False
        self.reserved_pages[req.rid] = need
        self.running.append(req)
        return True

    def finish(self, req: Req) -> None:
        req.finished = True
        self.runner.release(req)
        self.reserved_pages.pop(req.rid, None)
        self.sampler.forget(req.rid)
        if req in self.running:
            self.running.remove(req)

    # ---- one batch -----------------------------------------------------------------------------
    def run_step(self, items: List[StepItem], layer_hook=None) -> Optional[torch.Tensor]:
        self.steps += 1
        return self.runner.forward(items, layer_hook=layer_hook)

    def _next_items(self) -> List[StepItem]:
        items, budget = [], self.chunk
        for r in self.running:                       # 1. decodes
            if r.cached_len >= len(r.input_ids):
                items.append(StepItem(r, [r.all_ids[r.cached_len]], want=[0]))
        for r in self.running:                       # 2a. prompts in progress
            left = len(r.input_ids) - r.cached_len
            if left > 0 and budget > 0:
                n = min(left, budget)
                items.append(StepItem(r, r.input_ids[r.cached_len:r.cached_len + n],
                                      want=[n - 1] if n == left else []))
                budget -= n
        while self.waiting and budget > 0:           # 2b. new requests
            if not self._try_admit(self.waiting[0]):
                break
            r = self.waiting.popleft()
            n = min(len(r.input_ids), budget)
            items.append(StepItem(r, r.input_ids[:n], want=[n - 1] if n == len(r.input_ids) else []))
            budget -= n
        return items

    def step(self) -> List[Req]:
        """Runs one scheduling step; -> the requests that finished in it."""
        items = self._next_items()
        if not items:
            if self.waiting and not self.running:
                raise RuntimeError("a waiting request cannot be admitted into an idle engine")
            return []
        logits = self.run_step(items)
        sampled = [it.req for it in items if it.want]
        done = []
        if sampled:
            for r, tok in zip(sampled, self.sampler(logits, sampled)):
                r.output_ids.append(int(tok))
                sp = r.sampling_params
                if len(r.output_ids) >= sp.max_new_tokens or tok in sp.stop_token_ids:
                    done.append(r)
        for r in done:
            self.finish(r)
        return done

    def idle(self) -> bool:
        return not self.waiting and not self.running
