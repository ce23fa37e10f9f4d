"""Requests and the batch of one engine step.

A step is a list of (request, number of new tokens): prompt portions and single decoded tokens side
by side (the reference's ScheduleBatch.prepare_for_extend / mix_with_running,
managers/schedule_batch.py:1117-1291, 1293-1330).  `prepare` allocates page-aligned token slots with
PagedTokenToKVPoolAllocator, writes them into ReqToTokenPool, and builds the ForwardBatch with the
per-token tables the kernels walk."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Sequence

import torch

from ..mem_cache.paged_allocator import (compute_position, get_last_loc,
                                         write_req_to_token_pool)
from ..model_executor.forward_batch_info import ForwardBatch, ForwardMode


@dataclass
class SamplingParams:
    max_new_tokens: int = 16
    temperature: float = 0.0        # 0 = greedy
    top_k: int = 0
    top_p: float = 1.0
    stop_token_ids: Sequence[int] = ()
    seed: Optional[int] = None


@dataclass
class Req:
    rid: str
    input_ids: List[int]
    sampling_params: SamplingParams = field(default_factory=SamplingParams)
    output_ids: List[int] = field(default_factory=list)
    req_pool_idx: Optional[int] = None
    cached_len: int = 0              # tokens whose rows are in the pool
    finished: bool = False

    @property
    def all_ids(self) -> List[int]:
        return self.input_ids + self.output_ids


@dataclass
class StepItem:
    req: Req
    tokens: List[int]                # the new tokens this step feeds
    want: Sequence[int] = ()         # offsets among `tokens` whose logits are asked for


class OutOfCache(RuntimeError):
    pass


def prepare(items: List[StepItem], req_to_token_pool, allocator, token_to_kv_pool, state_pool,
            device) -> ForwardBatch:
    bs = len(items)
    pre = [it.req.cached_len for it in items]
    ext = [len(it.tokens) for it in items]
    seq = [p + e for p, e in zip(pre, ext)]
    total = sum(ext)
    if max(seq) > req_to_token_pool.max_context_len:
        raise OutOfCache(f"a sequence of {max(seq)} tokens exceeds the context length "
                         f"{req_to_token_pool.max_context_len}")
    page = allocator.page_size
    need_pages = sum((q + page - 1) // page - (p + page - 1) // page for p, q in zip(pre, seq))
    if need_pages > len(allocator.free_pages):      # checked here: the device kernel does not
        raise OutOfCache(f"{need_pages} pages needed for {total} new tokens, "
                         f"{len(allocator.free_pages)} free")
    # one staging tensor -> one H2D copy for all the small per-entry tables
    host = torch.tensor([[it.req.req_pool_idx for it in items], pre, ext, seq], dtype=torch.int64)
    ids_host = torch.tensor([t for it in items for t in it.tokens], dtype=torch.int64)
    tok_b_host = torch.repeat_interleave(torch.arange(bs, dtype=torch.int32),
                                         torch.tensor(ext, dtype=torch.int64))
    tables = host.to(device, non_blocking=True)
    input_ids = ids_host.to(device, non_blocking=True)
    tok_b = tok_b_host.to(device, non_blocking=True)
    req_pool_indices, pre_lens, ext_lens, seq_lens = tables[0], tables[1], tables[2], tables[3]
    last_loc = get_last_loc(req_to_token_pool.req_to_token, req_pool_indices, pre_lens)
    out_cache_loc = allocator.alloc_extend(pre_lens, seq_lens, last_loc, total)
    if out_cache_loc is None:
        raise OutOfCache(f"no pages left for {total} new tokens "
                         f"({allocator.available_size()} token slots free)")
    write_req_to_token_pool(req_to_token_pool.req_to_token, req_pool_indices, pre_lens, seq_lens,
                            ext_lens, out_cache_loc)
    ext32, pre32 = ext_lens.to(torch.int32), pre_lens.to(torch.int32)
    positions, ext_start = compute_position(pre32, ext32, total)
    mode = ForwardMode.DECODE if all(e == 1 and p > 0 for e, p in zip(ext, pre)) else (
        ForwardMode.MIXED if any(e == 1 and p > 0 for e, p in zip(ext, pre)) else ForwardMode.EXTEND)
    fb = ForwardBatch(forward_mode=mode, batch_size=bs, req_pool_indices=req_pool_indices,
                      seq_lens=seq_lens, out_cache_loc=out_cache_loc, seq_lens_sum=sum(seq),
                      positions=positions, extend_seq_lens=ext32, extend_prefix_lens=pre32,
                      extend_start_loc=ext_start, extend_seq_lens_cpu=ext, extend_prefix_lens_cpu=pre,
                      extend_num_tokens=total, req_to_token_pool=req_to_token_pool,
                      token_to_kv_pool=token_to_kv_pool)
    fb.tok_pos = positions.to(torch.int32)
    fb.tok_b = tok_b
    fb.ext_start = ext_start
    fb.ext_len = ext32
    fb.max_seq_len = max(seq)
    fb.state_pool = state_pool
    fb.extra["input_ids"] = input_ids
    for it in items:
        it.req.cached_len += len(it.tokens)
    return fb
