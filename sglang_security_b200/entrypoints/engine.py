"""Offline engine: the call a user makes (the reference's `sglang.Engine.generate`,
python/sglang/srt/entrypoints/engine.py).  Token ids in, token ids out; requests are batched
continuously by managers/scheduler.py."""
from __future__ import annotations

from typing import List, Optional, Sequence, Union

import torch

from ..managers.schedule_batch import Req, SamplingParams
from ..managers.scheduler import Scheduler
from ..model_executor.model_runner import ModelRunner

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, "float16": torch.float16}


class Engine:
    def __init__(self, model_path: str, dtype: Union[str, torch.dtype] = "bfloat16",
                 max_total_tokens: int = 8192, max_running_requests: int = 4,
                 chunked_prefill_size: int = 512, context_length: Optional[int] = None, **runner_kw):
        dt = _DTYPES[dtype] if isinstance(dtype, str) else dtype
        self.runner = ModelRunner(model_path, dt, max_total_tokens, max_running_requests, context_length,
                                  **runner_kw)
        self.scheduler = Scheduler(self.runner, chunked_prefill_size)
        self._n = 0

    def generate(self, input_ids: Sequence[Sequence[int]],
                 sampling_params: Union[SamplingParams, Sequence[SamplingParams], None] = None
                 ) -> List[List[int]]:
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(input_ids)
        reqs = []
        for ids, sp in zip(input_ids, sampling_params):
            self._n += 1
            reqs.append(Req(rid=f"g{self._n}", input_ids=list(ids), sampling_params=sp))
            self.scheduler.add_request(reqs[-1])
        while not self.scheduler.idle():
            self.scheduler.step()
        return [r.output_ids for r in reqs]
