"""Trace replay: feed given token ids through the model step by step and write logits.

It samples nothing and has no forward pass, cache or loader of its own: every step goes
through `Engine.step`, the call that generation uses.  The reference's nearest tools
are `trace_dump` (crates/braidinfer-runtime/src/bin/trace_dump.rs:50-123) and the
per-step logit hash of `BRAIDINFER_LOGIT_TRACE`
(crates/braidinfer-runtime/src/generate.rs:383-396); this writes the logits themselves.

Input, one JSON object a line on standard input:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
`entries`: for each request its next tokens and the places among them whose logits are
wanted; a request is opened the first time its id appears.  `end`: requests that are
finished after this step; their slots and pages go back to the cache.
Output: for a step in which something is wanted, <out>/<step>.f32 holds the logits at
the wanted places, in the order of the entries and of `want`, as little-endian
float32 [wanted, vocab].  After every step `done <step>` is printed and flushed.

`--dump-activations DIR` also writes, for every step, DIR/<step>.act.f32: the residual
stream of the step's tokens (in the order of the entries) after the embedding and after
every run of a layer, float32 [1 + runs, tokens, width].  A wrong layer is then found by
comparing these files with a plain implementation's instead of bisecting by hand; the
reference has an in-kernel dump for the same purpose (kernels/dump.h:24-60, sink
crates/braidinfer-runtime/src/tracer.rs:266-306).  Steps that dump are launched kernel
by kernel and complete every deferred sum at once.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, Optional, Sequence

import numpy as np


def replay(engine, lines, out_dir: str, say=None, dump_dir: Optional[str] = None) -> int:
    """Drive `engine` with the steps in `lines` (an iterable of JSON strings)."""
    os.makedirs(out_dir, exist_ok=True)
    if dump_dir:
        os.makedirs(dump_dir, exist_ok=True)
    slots: Dict[str, int] = {}
    n = 0
    for line in lines:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = rec.get("entries", [])
        batch, want = [], []
        for e in entries:
            rid = str(e["id"])
            if rid not in slots:
                slots[rid] = engine.open()
            batch.append((slots[rid], [int(t) for t in e["tokens"]]))
            want.append([int(w) for w in e.get("want", [])])
        if batch:
            taps = []
            if dump_dir:
                logits = engine.step(batch, want=want, tap=lambda i, h: taps.append(h.clone()))
            else:
                logits = engine.step(batch, want=want)
            if dump_dir:
                import torch
                acts = torch.stack(taps).to("cpu").numpy().astype("<f4", copy=False)
                tmp = os.path.join(dump_dir, f".{step}.act.f32.tmp")
                acts.tofile(tmp)
                os.replace(tmp, os.path.join(dump_dir, f"{step}.act.f32"))
            if logits is not None:
                arr = logits.detach().to("cpu").numpy().astype("<f4", copy=False)
                engine.check()
                tmp = os.path.join(out_dir, f".{step}.f32.tmp")
                arr.tofile(tmp)
                os.replace(tmp, os.path.join(out_dir, f"{step}.f32"))
        for rid in rec.get("end", []):
            rid = str(rid)
            if rid not in slots:
                raise KeyError(f"step {step} ends request {rid!r}, which was never started")
            engine.close(slots.pop(rid))
        n += 1
        if say is not None:
            say(f"done {step}")
    return n


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens live requests hold at any time, each rounded up to a multiple of 64")
    ap.add_argument("--dump-activations", metavar="DIR", default=None,
                    help="also write the residual stream after the embedding and after every run of a layer, "
                         "DIR/<step>.act.f32 = float32 [1 + runs, tokens of the step, width]")
    a = ap.parse_args(argv)
    from .engine import Engine
    engine = Engine.from_folder(a.model, dtype=a.dtype, max_tokens=a.max_tokens, verbose=True)

    def say(msg: str) -> None:
        sys.stdout.write(msg + "\n")
        sys.stdout.flush()

    replay(engine, sys.stdin, a.out, say, dump_dir=a.dump_activations)
    engine.check()
    return 0


if __name__ == "__main__":
    sys.exit(main())
