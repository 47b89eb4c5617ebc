"""The `generate` command line, in the reference's manner
(crates/braidinfer-runtime/src/bin/generate.rs:13-60, :234-266): options come from the
environment, the prompt from the arguments.

  MODEL=<folder | random:<preset>>   model folder (config.json + safetensors), or argv[1]
                                     when that is an existing folder (generate.rs:24-34)
  MAX_TOKENS=<n>                     new tokens, default 64 (generate.rs:42-45)
  RAW=1                              prompt as is, no chat template; the only mode here
                                     (generate.rs:47, :235-246)
  MAX_SEQ_LEN=<n>                    cap on context; sizes the cache (generate.rs:56-58)
  prompt                             the remaining arguments joined by spaces, default
                                     "Hello, world!" (generate.rs:36-40)
  BRAIDINFER_LOGIT_TRACE=<file>      append `step= tok= logit_hash=` a chosen token, to find the step where
                                     two runs part (generate.rs:380-396; see engine/generate.py)
This library's own: TEMPERATURE (default 0 = greedy, as the reference's binary is),
TOP_K, TOP_P, MIN_P, REPETITION_PENALTY, SEED, DTYPE=bfloat16|float32, BATCH_FILE=<file
with one prompt a line>.

With a tokenizer.json in the model folder (and the `tokenizers` package) the prompt is
text and so is the output; BOS is prepended unless it is there already or
tokenizer_config.json says add_bos_token false (generate.rs:479-489).  Without one the
prompt is a list of token ids ("1, 5, 17"), or else its UTF-8 bytes, and the output is
token ids.  Prints the reference's two timing lines to stderr.
"""
from __future__ import annotations

import json
import os
import sys
import time
from typing import List, Optional, Sequence, Tuple


class TextCodec:
    """Text <-> token ids for the command line."""

    def __init__(self, folder: Optional[str], vocab_size: int, bos: Optional[int]) -> None:
        self.tok = None
        self.vocab_size = vocab_size
        self.bos = bos
        self.add_bos = None
        if folder:
            tj = os.path.join(folder, "tokenizer.json")
            if os.path.isfile(tj):
                try:
                    from tokenizers import Tokenizer
                    self.tok = Tokenizer.from_file(tj)
                except ImportError:
                    print("[generate] tokenizer.json found but the 'tokenizers' package is missing; "
                          "reading the prompt as token ids", file=sys.stderr)
            tc = os.path.join(folder, "tokenizer_config.json")
            if os.path.isfile(tc):
                try:
                    with open(tc) as f:
                        v = json.load(f).get("add_bos_token")
                    self.add_bos = v if isinstance(v, bool) else None
                except Exception:
                    pass

    def encode(self, prompt: str) -> List[int]:
        if self.tok is not None:
            ids = list(self.tok.encode(prompt, add_special_tokens=False).ids)
            if self.add_bos is not False and self.bos is not None and (not ids or ids[0] != self.bos):
                ids.insert(0, self.bos)
            return ids
        parts = prompt.replace(",", " ").split()
        if parts and all(p.lstrip("-").isdigit() for p in parts):
            return [int(p) for p in parts]
        ids = list(prompt.encode("utf-8"))
        if self.vocab_size < 256:
            ids = [i % self.vocab_size for i in ids]
        return ids

    def decode(self, ids: Sequence[int]) -> str:
        if self.tok is not None:
            return self.tok.decode(list(ids), skip_special_tokens=False)
        return " ".join(str(i) for i in ids)


def _env_float(name: str, default: float) -> float:
    v = os.environ.get(name)
    try:
        return float(v) if v is not None else default
    except ValueError:
        raise SystemExit(f"{name}={v!r} is not a number")


def _env_int(name: str, default: Optional[int]) -> Optional[int]:
    v = os.environ.get(name)
    try:
        return int(v) if v is not None else default
    except ValueError:
        raise SystemExit(f"{name}={v!r} is not an integer")


def main(argv: Optional[Sequence[str]] = None) -> int:
    from ..api import load
    from ..sampling import SamplingParams

    args = list(sys.argv[1:] if argv is None else argv)
    model = os.environ.get("MODEL")
    if model is None and args and (os.path.isdir(args[0]) or args[0].startswith("random:")):
        model = args.pop(0)
    if model is None:
        print("generate: set MODEL=<model folder> (or MODEL=random:<preset>), or give the folder as the "
              "first argument", file=sys.stderr)
        return 2
    prompt = " ".join(args) if args else "Hello, world!"
    max_tokens = _env_int("MAX_TOKENS", 64)
    max_seq_len = _env_int("MAX_SEQ_LEN", None)
    dtype = os.environ.get("DTYPE", "bfloat16")
    temperature = _env_float("TEMPERATURE", 0.0)
    if temperature == 0.0:
        params = SamplingParams.greedy()
    else:
        params = SamplingParams(temperature=temperature, top_k=_env_int("TOP_K", 50), top_p=_env_float("TOP_P", 1.0),
                                min_p=_env_float("MIN_P", 0.0),
                                repetition_penalty=_env_float("REPETITION_PENALTY", 1.0),
                                seed=_env_int("SEED", None))
    prompts_text = [prompt]
    batch_file = os.environ.get("BATCH_FILE")
    if batch_file:
        with open(batch_file) as f:
            prompts_text = [line.rstrip("\n") for line in f if line.strip()]
    t_load = time.perf_counter()
    m = load(model, dtype=dtype, max_seq_len=max_seq_len, max_batch=max(1, min(len(prompts_text), 64)),
             seed=_env_int("WEIGHT_SEED", 0))
    print(f"LOAD PROFILE: load = {(time.perf_counter() - t_load) * 1000:.0f} ms", file=sys.stderr)
    spec = m.spec
    codec = TextCodec(None if model.startswith("random:") else model, spec.vocab_size, spec.bos_token_id)
    stop = list(spec.eos_token_ids)
    print(f"max_seq_len: {m.engine.max_tokens // m.max_batch}", file=sys.stderr)
    print(f"stop tokens: {stop}", file=sys.stderr)
    prompts = [codec.encode(p) for p in prompts_text]
    start = time.perf_counter()
    try:
        outs = m.generate(prompts, params, stop, max_tokens)
    except ValueError as e:                 # an empty prompt, or a request the cache has no room for
        print(f"generate: {e}", file=sys.stderr)
        return 2
    elapsed = time.perf_counter() - start
    n_tokens = 0
    for o in outs:
        print(codec.decode(o.tokens))
        n_tokens += len(o.tokens)
    sys.stdout.flush()
    print(m.last_stats.pptg_line(), file=sys.stderr)
    print(f"{n_tokens} tokens in {elapsed:.3f}s = {n_tokens / elapsed if elapsed > 0 else 0.0:.1f} tok/s",
          file=sys.stderr)
    return 0


if __name__ == "__main__":
    sys.exit(main())
