"""The Python entry point.

The reference is a Rust library with a `generate` binary; its calls are
`Model::load_with_max_seq_len(dir, device, max_seq_len)`, `prefill(tokens)`,
`decode_step(token, position)`, `generate_from_ids(...)`, `greedy_generate(...)` and
`sampling::generate(model, prompt_tokens, params, stop_tokens, max_new_tokens)`
(crates/braidinfer-runtime/src/model/model_load.rs:55, model/state.rs:39,
model/mod.rs:279, generate.rs:314, :468, sampling.rs:181).  This module keeps those
names and meanings and widens them from one sequence to batches.
"""
from __future__ import annotations

import math
import os
from typing import List, Optional, Sequence, Union

from .cache import PAGE_SIZE
from .config import preset, read_config_json
from .engine.engine import Engine
from .models import architecture_for
from .weights import tensor_specs_of
from .engine.generate import Completion, GenerationLoop, GenerationStats
from .sampling import Sampler, SamplingParams

DEFAULT_MAX_SEQ_LEN_CAP = 8192      # the reference's default cap on context (model_load.rs:49, 113-116)
RANDOM_ON_DEVICE_BYTES = 64 << 20   # random models above this many bytes of weights are drawn on the GPU


class Model:
    """A loaded model with its cache, ready to generate."""

    def __init__(self, engine: Engine, max_batch: int) -> None:
        self.engine = engine
        self.config = engine.config           # the architecture's typed configuration, or None for a hand-made ModelSpec
        self.spec = engine.spec
        self.sampler = Sampler(engine.kernels, engine.device)
        self.max_batch = max_batch
        self.last_stats: Optional[GenerationStats] = None

    # -- batched generation
    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]],
                 params: Union[SamplingParams, Sequence[SamplingParams], None] = None,
                 stop_tokens: Optional[Sequence[int]] = None, max_new_tokens: Union[int, Sequence[int]] = 64
                 ) -> Union[List[int], List[Completion]]:
        """Generate after token-id prompts.  One prompt (a list of ints) returns the new
        token ids, as the reference's `sampling::generate` does; a list of prompts
        returns a `Completion` for each.  `stop_tokens` defaults to the model's
        eos_token_id.  A stop token ends a sequence and is not returned."""
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        plist = [list(prompts)] if single else [list(p) for p in prompts]
        if stop_tokens is None:
            stop_tokens = self.spec.eos_token_ids
        loop = GenerationLoop(self.engine, self.sampler, max_batch=self.max_batch)
        out = loop.generate(plist, params, max_new_tokens, stop_tokens)
        self.last_stats = loop.stats
        return out[0].tokens if single else out

    def generate_from_ids(self, prompt_ids: Sequence[int], max_tokens: int = 64) -> List[int]:
        """Greedy generation after one prompt (generate.rs:314-439)."""
        return self.generate(list(prompt_ids), SamplingParams.greedy(), None, max_tokens)

    # -- the step function itself, for callers that schedule their own batches
    def open(self) -> int:
        """Take a slot for a new sequence."""
        return self.engine.open()

    def step(self, entries, want="last"):
        """One step of `entries` = [(slot, tokens), ...] (see `Engine.step`): sequences that start
        together bring their prompts, then one token each; returns float32 logits at the wanted places."""
        return self.engine.step(entries, want=want)

    def close(self, slot: int) -> None:
        """Give a sequence's slot and pages back."""
        self.engine.close(slot)

    def replay(self, lines, out_dir: str, dump_activations: Optional[str] = None) -> int:
        """Feed given token ids step by step and write logits, as `bin/trace_run` does
        (`lines`: JSON step objects, as text lines or dicts; `dump_activations`: a folder for
        the residual stream after every run of a layer, as `--dump-activations` writes it)."""
        import json
        from .engine.trace import replay
        return replay(self.engine, (l if isinstance(l, str) else json.dumps(l) for l in lines), out_dir,
                      dump_dir=dump_activations)

    # -- the step API of the reference, for one sequence at a time
    def prefill(self, tokens: Sequence[int]):
        """Start a sequence with its prompt; returns (slot, float32 logits of the last token)."""
        slot = self.engine.open()
        return slot, self.engine.step([(slot, list(tokens))], want="last")[0]

    def decode_step(self, slot: int, token: int):
        """Append one token to a sequence; returns the logits after it."""
        return self.engine.step([(slot, [int(token)])], want="last")[0]

    def reset_state(self, slot: int) -> None:
        self.engine.close(slot)


def load(model: str, dtype: str = "bfloat16", max_seq_len: Optional[int] = None, max_batch: int = 8,
         seed: int = 0, device: str = "cuda:0", verbose: bool = True, **engine_options) -> Model:
    """Load a model folder (config.json + safetensors), or `random:<preset>` for seeded
    random weights of a named size.  `max_seq_len` caps the context of a sequence
    (default: the config's max_position_embeddings, at most 8192, as in the
    reference); the cache is sized for `max_batch` such sequences."""
    if model.startswith("random:"):
        cfg_dict = preset(model.split(":", 1)[1])
        source = None
    else:
        if not os.path.isdir(model):
            raise FileNotFoundError(f"MODEL={model!r} is not a folder (use a model folder or random:<preset>)")
        cfg_dict = read_config_json(model)
        source = model
    arch = architecture_for(cfg_dict)
    spec = arch.build_spec(arch.config_from_dict(cfg_dict))
    if max_seq_len is None:
        max_seq_len = min(spec.max_position or 2048, DEFAULT_MAX_SEQ_LEN_CAP)
    per_seq = -(-max_seq_len // PAGE_SIZE) * PAGE_SIZE
    opts = dict(dtype=dtype, max_tokens=per_seq * max_batch, max_slots=max_batch, device=device, verbose=verbose)
    opts.update(engine_options)
    if source is None:
        # a large model is drawn on the device: the CPU draw of gigabytes takes minutes
        n_bytes = sum(2 * math.prod(ts.shape) for ts in tensor_specs_of(spec).values())
        engine = Engine.from_random(cfg_dict, seed, on_device=n_bytes > RANDOM_ON_DEVICE_BYTES, **opts)
    else:
        engine = Engine.from_folder(source, **opts)
    return Model(engine, max_batch)
