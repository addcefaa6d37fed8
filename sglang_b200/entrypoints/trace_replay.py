"""Scripted replay: feed given token ids through a model step by step and write the logits of chosen positions.

    python -m sglang_b200.cli trace-run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N   (or ``bin/trace_run``)

Steps arrive on standard input, one JSON object per line::

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

Every entry brings a request's next tokens (a prompt portion of any length, or one decoded token); all entries of a step run as ONE batch
of the engine (``Scheduler.replay_step`` -> ``ModelRunner.forward_batch_generation``: the serving step, KV manager, request slots and
kernels — this file has no forward pass of its own).  ``want`` lists the positions among the entry's tokens whose logits are written to
``<out>/<step>.f32`` (little-endian fp32 [wanted, vocab], in entry order); ``end`` lists requests that are finished after the step and
give their pages and slot back.  After every step the line ``done <step>`` goes to standard output.  Nothing is sampled.

``--max-tokens`` sizes the paged pool (each live request's token count rounded up to the page size of 64); there are four request slots.
``--dtype float32`` runs every product in true fp32 (no TF32).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

PAGE = 64
SLOTS = 4


def main(argv=None) -> int:
    ap = argparse.ArgumentParser("sglang_b200 trace-run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for <step>.f32")
    ap.add_argument("--max-tokens", type=int, required=True, help="tokens the live requests hold at most (page-rounded)")
    ap.add_argument("--device", default="auto", choices=("auto", "cuda", "cpu"))
    ns = ap.parse_args(argv)
    real_stdout = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)                    # anything the libraries print must not mix with the protocol lines
    sys.stdout = sys.stderr

    import numpy as np
    import torch

    from ..server_args import ServerArgs
    from .engine import Engine

    device = ns.device if ns.device != "auto" else ("cuda" if torch.cuda.is_available() else "cpu")
    from .. import build as _build

    if not list(_build.ROOT.glob("sglb_rt*.so")):          # fresh checkout: the C++ host runtime (page allocator, radix tree) first
        _build.build_runtime()
    if device == "cuda":
        from .. import ops

        if not ops.load_native(build_if_missing=True):
            raise RuntimeError("the CUDA extension could not be built or loaded")
    pages = (ns.max_tokens + PAGE - 1) // PAGE
    args = ServerArgs(model_path=ns.model, device=device, skip_tokenizer_init=True, page_size=PAGE, max_total_tokens=pages * PAGE,
                      max_running_requests=SLOTS, context_length=pages * PAGE, disable_radix_cache=True, disable_cuda_graph=True,
                      disable_overlap_schedule=True, chunked_prefill_size=-1, max_prefill_tokens=pages * PAGE, log_level="warning",
                      json_model_override_args=json.dumps({"dtype": ns.dtype}))
    eng = Engine(server_args=args)
    os.makedirs(ns.out, exist_ok=True)
    sched = eng.scheduler
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        msg = json.loads(line)
        entries = [(str(e["id"]), list(e["tokens"]), list(e.get("want") or [])) for e in msg.get("entries", [])]
        logits = sched.replay_step(entries, [str(i) for i in msg.get("end", [])])
        if logits is not None and logits.shape[0]:
            tmp = os.path.join(ns.out, f".{msg['step']}.part")
            np.ascontiguousarray(logits, dtype="<f4").tofile(tmp)
            os.replace(tmp, os.path.join(ns.out, f"{msg['step']}.f32"))
        real_stdout.write(f"done {msg['step']}\n")
        real_stdout.flush()
    return 0


if __name__ == "__main__":
    sys.exit(main())
