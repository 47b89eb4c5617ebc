"""The engine: a loaded model, its cache and the step function.

`Engine.open()` takes a slot for a sequence, `Engine.step()` runs the tokens that
sequences bring and returns logits at the wanted places, `Engine.close()` gives the
slot and its pages back.  Generation, the command line and trace replay all drive
this one object.
"""
from __future__ import annotations

import os
from typing import Dict, List, Mapping, Optional, Sequence, Tuple, Union

import torch

from ..cache import CacheError, CacheManager, PAGE_SIZE
from ..config import read_config_json
from ..models import DecoderModel, architecture_for
from ..parts.runtime import Runtime
from ..weights import draw_tensors, load_tensors, tensor_specs_of
from .step import StepContext, StepPacker

# Steps of up to this many tokens in all are given a shape that CUDA graphs can be keyed on (see Engine.step):
# beyond, the device takes longer over a step than the host over its launches.
GRAPH_PROMPT_ROWS = 256
FEW_TOKENS = 8            # up to so many tokens a sequence the attention part slices the context (parts/attention.py)


_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32,
           "f32": torch.float32}


def parse_dtype(name: Union[str, torch.dtype]) -> torch.dtype:
    if isinstance(name, torch.dtype):
        if name not in (torch.bfloat16, torch.float32):
            raise ValueError(f"the engine runs in bfloat16 or float32, not {name}")
        return name
    if name not in _DTYPES:
        raise ValueError(f"unknown dtype {name!r}; choose bfloat16 or float32")
    return _DTYPES[name]


class Engine:
    def __init__(self, config_dict: Optional[Mapping], tensors_or_folder, *, dtype="bfloat16", max_tokens: int = 8192,
                 max_slots: Optional[int] = None, device: str = "cuda:0", gemm_backend: str = "auto",
                 attention_backend: str = "auto", row_multiple: int = 1, use_graphs: bool = True,
                 fuse_reduce: bool = True, scaled_norm: bool = True, verbose: bool = True, spec=None) -> None:
        """`config_dict` (config.json's content) picks the architecture and its description of
        parts; or pass a `ModelSpec` as `spec` directly (then `config_dict` may be None)."""
        from ..csrc.api import get_kernels
        self.dtype = parse_dtype(dtype)
        self.device = torch.device(device)
        torch.cuda.set_device(self.device)
        self.kernels = get_kernels(verbose=verbose)
        if spec is None:
            self.arch = architecture_for(config_dict)
            self.config = self.arch.config_from_dict(config_dict)
            self.spec = self.arch.build_spec(self.config)
        else:
            self.arch, self.config, self.spec = None, None, spec
        self.rt = Runtime(act_dtype=self.dtype, device=self.device, kernels=self.kernels,
                          gemm_backend=gemm_backend, attention_backend=attention_backend, fuse_reduce=fuse_reduce,
                          scaled_norm=scaled_norm)
        self.model = DecoderModel(self.spec, self.rt)
        specs = self.model.tensor_specs()
        if isinstance(tensors_or_folder, (str, os.PathLike)):
            tensors = load_tensors(str(tensors_or_folder), specs, self.dtype, self.device)
        else:
            # tensors handed over directly get the loader's rule for element types: a float32 run
            # widens every floating tensor (exactly), a bfloat16 run keeps what it is given
            tensors = {n: (t.to(self.device).float() if self.dtype == torch.float32 and t.is_floating_point()
                           and t.dtype != torch.float32 else t.to(self.device))
                       for n, t in tensors_or_folder.items()}
        self.weight_bytes = sum(t.numel() * t.element_size() for t in tensors.values())
        self.model.load(tensors)
        del tensors
        self.max_tokens = int(max_tokens)
        n_pages = -(-self.max_tokens // PAGE_SIZE)
        self.max_slots = int(max_slots) if max_slots else max(1, min(n_pages, 1024))
        self.cache = CacheManager(self.model.cache_plan(), self.max_tokens, self.max_slots, self.dtype, self.device)
        self.packer = StepPacker(self.device, row_multiple=row_multiple)
        self.vocab_size = self.spec.vocab_size
        self.steps_run = 0
        # Steps in which every sequence brings one token are launch-bound: the second time
        # a step shape is seen it is captured in a CUDA graph and replayed from then on.
        self.use_graphs = bool(use_graphs) and all(p.graph_safe for p in self.model.all_parts())
        self._graphs: Dict[tuple, object] = {}
        self._graph_seen: Dict[tuple, int] = {}
        self._graph_generation = (self.packer.generation, self.kernels.workspace_generation)
        self._capture_stream: Optional[torch.cuda.Stream] = None
        self._graph_pool = None               # one memory pool for all graphs: they never replay at the same time
        self.graph_replays = 0

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_folder(cls, folder: str, **kw) -> "Engine":
        """A model folder: config.json picks the architecture, safetensors hold the weights."""
        return cls(read_config_json(folder), folder, **kw)

    @classmethod
    def from_spec(cls, spec, seed: int = 0, *, dtype="bfloat16", device: str = "cuda:0", scale=None, **kw) -> "Engine":
        """A model described by a `ModelSpec` (any mix of registered parts) with seeded random
        weights: the tensors its parts ask for are drawn as `write_random_model` draws them.
        `scale` maps a tensor-name suffix to a factor (for tests that want peaked routers or
        attention).  Returns the engine; `engine.drawn` keeps the CPU tensors it was built from."""
        run_dtype = parse_dtype(dtype)
        drawn = draw_tensors(tensor_specs_of(spec), seed, torch.bfloat16)
        for suffix, factor in (scale or {}).items():
            for name in drawn:
                if name.endswith(suffix):
                    drawn[name] = (drawn[name].float() * factor).to(torch.bfloat16)
        dev = torch.device(device)
        tensors = {n: (t.to(dev) if run_dtype == torch.bfloat16 else t.to(dev).float()) for n, t in drawn.items()}
        eng = cls(None, tensors, dtype=dtype, device=device, spec=spec, **kw)
        eng.drawn = drawn
        return eng

    @classmethod
    def from_random(cls, config_dict: Mapping, seed: int = 0, *, dtype="bfloat16", device: str = "cuda:0",
                    on_device: bool = False, **kw) -> "Engine":
        """Random weights without a folder.  By default the tensors are the ones
        `write_random_model` would store (CPU draw, same seed, same values); with
        `on_device` they are drawn on the GPU instead, which large sizes need for speed
        (other values, same distributions)."""
        run_dtype = parse_dtype(dtype)
        arch = architecture_for(config_dict)
        spec = arch.build_spec(arch.config_from_dict(config_dict))
        specs = tensor_specs_of(spec)
        dev = torch.device(device)
        if on_device:
            torch.cuda.set_device(dev)
            g = torch.Generator(device=dev)
            g.manual_seed(int(seed))
            tensors = {}
            for name, ts in specs.items():
                x = torch.empty(ts.shape, dtype=torch.bfloat16, device=dev)
                x.normal_(0.0, ts.std, generator=g)
                if ts.init == "one_plus_normal":
                    x += 1.0
                tensors[name] = x if run_dtype == torch.bfloat16 else x.float()
        else:
            drawn = draw_tensors(specs, seed, torch.bfloat16)
            tensors = {n: (t.to(dev) if run_dtype == torch.bfloat16 else t.to(dev).float()) for n, t in drawn.items()}
        return cls(config_dict, tensors, dtype=dtype, device=device, **kw)

    # ------------------------------------------------------------------ sequences
    def open(self) -> int:
        """Take a slot for a new sequence (its cache is empty, its state zero)."""
        return self.cache.alloc_slot()

    def close(self, slot: int) -> None:
        """Give a sequence's slot and pages back."""
        self.cache.free_slot(slot)

    def length(self, slot: int) -> int:
        return self.cache.length(slot)

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[Tuple[int, Sequence[int]]],
             want: Union[str, Sequence[Sequence[int]], None] = "last",
             device_tokens: Optional[Tuple[torch.Tensor, Sequence[int]]] = None, tap=None) -> Optional[torch.Tensor]:
        """Run `entries` = [(slot, tokens), ...] as one batch.

        `want` says whose logits come back: "last" (each sequence's last token), "all",
        None, or for each sequence a list of places among the tokens it brings.
        Returns float32 logits [wanted, vocab] on the device, in the order of the
        entries and of their wanted places (None if nothing is wanted).

        `device_tokens` = (int32 tensor on the device, rows): in a step of one token a
        sequence, take entry i's token from tensor[rows[i]] instead of from `entries`
        (whose token is then a placeholder), so that a sampler's output can feed the next
        step without a round trip through the host.

        `tap(i, h)`: a function that is shown the residual stream [tokens of the step, width]
        (float32, on the device; padding rows cut off) after the embedding (i = 0) and after
        each schedule entry (i = 1 ...).  A step with a tap is launched kernel by kernel."""
        if not entries:
            return None
        slots = [int(s) for s, _ in entries]
        tokens = [list(t) for _, t in entries]
        for s, t in zip(slots, tokens):
            if len(t) == 0:
                raise ValueError(f"sequence in slot {s} brings no token")
            lo, hi = min(t), max(t)
            if lo < 0 or hi >= self.vocab_size:
                raise ValueError(f"token id {lo if lo < 0 else hi} is outside the vocabulary of {self.vocab_size}")
        if want == "last":
            want_l = [[len(t) - 1] for t in tokens]
        elif want == "all":
            want_l = [list(range(len(t))) for t in tokens]
        elif want is None:
            want_l = [[] for _ in tokens]
        else:
            want_l = [list(w) for w in want]
            if len(want_l) != len(tokens):
                raise ValueError("want must have one list per entry")
        before = [self.cache.length(s) for s in slots]
        n_new = [len(t) for t in tokens]
        tables = self.cache.begin_step(slots, n_new)
        one_each = all(n == 1 for n in n_new)
        # Steps of few tokens are bound by the host when it launches them kernel by kernel (some 330
        # launches take it 6 ms, the device 3): they go through CUDA graphs, which can depend on a
        # step's shape only.  So such a step is given a shape that a few numbers name: its rows are
        # padded to a token tile (short prompts; a one-token step has one row a sequence), its page
        # tables widened, and its launches sized by the bounds that follow from these, not by the
        # lengths themselves.  A step launched kernel by kernel takes the same shape, so that it
        # gives the same bits.
        from ..csrc.api import token_tile
        short_prompt = not one_each and sum(n_new) <= GRAPH_PROMPT_ROWS
        shaped = one_each or short_prompt
        graphable = self.use_graphs and shaped and tap is None
        if device_tokens is not None and not one_each:
            raise ValueError("device_tokens needs a step of one token a sequence")
        ctx = self.packer.pack(slots, tokens, before, want_l, tables, bucket_tables=shaped,
                               token_source_rows=device_tokens[1] if device_tokens is not None else None,
                               pad_rows_to=token_tile(sum(n_new)) if short_prompt else 0)
        ctx.kernels = self.kernels
        if shaped and ctx.page_tables:
            ctx.max_kv_len = max(t.shape[1] for t in ctx.page_tables) * PAGE_SIZE
        if short_prompt:
            # no sequence brings more tokens than the step has rows; steps of a few tokens a sequence keep the
            # attention kernel that slices the context (it is chosen by this bound)
            ctx.max_q_len = FEW_TOKENS if max(n_new) <= FEW_TOKENS else ctx.rows
        if device_tokens is not None:
            self.kernels.gather_i32(device_tokens[0], self.packer.token_source_view, ctx.token_ids)
        try:
            if graphable:
                logits = self._graph_step(ctx)
            elif tap is not None:
                logits = self.model.forward(ctx, self.cache, tap=lambda i, h: tap(i, h[:ctx.n_tokens]))
            else:
                logits = self.model.forward(ctx, self.cache)
        except BaseException:
            # a part gave up in mid-step: a sum it left deferred must not outlive the step, or
            # every later stream-k product would find the workspace taken
            ctx.drop_deferred()
            self.kernels.pending_partial = None
            raise
        self.cache.end_step(slots, n_new)
        self.steps_run += 1
        return logits

    def _graph_step(self, ctx: StepContext) -> Optional[torch.Tensor]:
        """Run a step of few tokens (one a sequence, or short prompts) through a CUDA graph.  The graph holds kernel
        launches only; the step's tables were copied to fixed device addresses before it.
        Launch shapes depend on the step's shape alone (see `step`).  The graph writes its
        logits into its own memory; the caller gets a copy."""
        generation = (self.packer.generation, self.kernels.workspace_generation)
        if generation != self._graph_generation:       # a buffer that graphs point into has moved
            self._graphs.clear()
            self._graph_seen.clear()
            self._graph_generation = generation
        key = (ctx.rows, ctx.n_seqs, ctx.n_want, ctx.max_q_len, tuple(tuple(t.shape) for t in ctx.page_tables))
        entry = self._graphs.get(key)
        if entry is None:
            seen = self._graph_seen.get(key, 0)
            self._graph_seen[key] = seen + 1
            if seen == 0:                    # first sight: run kernel by kernel (also warms every kernel up)
                return self.model.forward(ctx, self.cache)
            if len(self._graphs) >= 64:
                self._graphs.pop(next(iter(self._graphs)))
            before = self.kernels.launches
            graph, static_logits = self._capture(ctx)
            entry = (graph, static_logits, self.kernels.launches - before)
            self.kernels.launches = before
            self._graphs[key] = entry
        graph, static_logits, n_launches = entry
        graph.replay()
        self.kernels.launches += n_launches
        self.graph_replays += 1
        return static_logits.clone() if static_logits is not None else None

    def _capture(self, ctx: StepContext):
        """Record the step's launches into a new graph.  What `torch.cuda.graph` does, without its
        emptying of the device's and the host's memory caches first: after those, every buffer the
        next steps ask for comes from the driver again, and a step with a capture took 10 to 60 ms
        instead of 6.  All graphs share one memory pool."""
        if self._capture_stream is None:
            self._capture_stream = torch.cuda.Stream(device=self.device)
        if not self._graphs:
            # no graph holds the old pool any more (torch has let go of it): a new one
            self._graph_pool = torch.cuda.graph_pool_handle()
        graph = torch.cuda.CUDAGraph()
        stream = self._capture_stream
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            graph.capture_begin(self._graph_pool)
            try:
                static_logits = self.model.forward(ctx, self.cache)
            except BaseException:
                try:
                    graph.capture_end()              # leave capture mode before the error travels on
                except Exception:
                    pass
                raise
            graph.capture_end()
        torch.cuda.current_stream().wait_stream(stream)
        return graph, static_logits

    def logit_hash(self, logits: torch.Tensor) -> List[int]:
        """One 64-bit hash a row of logits, for `BRAIDINFER_LOGIT_TRACE` (see engine/generate.py)."""
        return self.kernels.logit_hash(logits.float().contiguous())

    def check(self) -> None:
        """Raise if a kernel flagged an error since the last check (synchronises)."""
        self.kernels.check_device_errors()
