"""Trace replay: feeds given token ids through a model step by step and writes the logits at the
places asked for.  It samples nothing and decides nothing: every step of the trace is handed as one
batch to Scheduler.run_step — the same call, model runner, pools and kernels the generation path uses.

    trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Standard input, one JSON object per line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}
For a step with wanted places, DIR/<step>.f32 receives their logits as little-endian fp32
[wanted, vocab] in the order of the entries; after every step a line `done <step>` is printed."""
from __future__ import annotations

import argparse
import json
import os
import sys


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run")
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--max-requests", type=int, default=4)
    ap.add_argument("--layers-out", default=None,
                    help="also write the residual stream after every layer of each step, "
                         "<dir>/<step>.layers.f32 [layers, tokens, width]")
    a = ap.parse_args(argv)

    from .. import build
    build.ensure_built()

    import torch

    from ..managers.schedule_batch import Req, StepItem
    from ..managers.scheduler import Scheduler
    from ..model_executor.model_runner import ModelRunner

    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[a.dtype]
    runner = ModelRunner(a.model, dtype, max_total_tokens=a.max_tokens,
                         max_running_requests=a.max_requests, context_length=a.max_tokens)
    sched = Scheduler(runner)
    os.makedirs(a.out, exist_ok=True)
    live = {}
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        items = []
        for e in step["entries"]:
            req = live.get(e["id"])
            if req is None:
                req = Req(rid=e["id"], input_ids=[])
                if not runner.admit(req):
                    raise RuntimeError(f"no request slot for {e['id']}")
                live[e["id"]] = req
            req.input_ids += list(e["tokens"])
            items.append(StepItem(req, list(e["tokens"]), want=list(e.get("want", []))))
        captured = []
        hook = (lambda lid, x: captured.append(x.detach().float().cpu().clone())) if a.layers_out else None
        logits = sched.run_step(items, layer_hook=hook) if items else None
        if logits is not None:
            data = logits.float().cpu().contiguous().numpy().astype("<f4")
            tmp = os.path.join(a.out, f".{step['step']}.f32.part")
            with open(tmp, "wb") as f:
                f.write(data.tobytes())
            os.replace(tmp, os.path.join(a.out, f"{step['step']}.f32"))
        else:
            torch.cuda.synchronize()
        if captured:
            os.makedirs(a.layers_out, exist_ok=True)
            torch.stack(captured).numpy().astype("<f4").tofile(
                os.path.join(a.layers_out, f"{step['step']}.layers.f32"))
        for rid in step.get("end", []):
            req = live.pop(rid, None)
            if req is not None:
                runner.release(req)
        sys.stdout.write(f"done {step['step']}\n")
        sys.stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
